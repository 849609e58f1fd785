"""The GPUBPETrainer drop-in against the reference's own results (tests/golden/train.json)."""
import json
import random

import numpy as np
import pytest
import torch

from oracle import oracle as O
from supertoken_b200 import GPUBPETrainer, synth
from tests.helpers import corpus_rows, load_golden

pytestmark = pytest.mark.gpu


def make_batch(rows):
    """Padded batch as the reference's batchers build it (pad id -1, prefix-valid)."""
    width = max(1, max((len(r) for r in rows), default=0))
    tokens = torch.full((len(rows), width), -1, dtype=torch.int32)
    valid = torch.zeros((len(rows), width), dtype=torch.uint8)
    lengths = torch.zeros((len(rows),), dtype=torch.int32)
    for i, r in enumerate(rows):
        if len(r):
            tokens[i, :len(r)] = torch.tensor(list(r), dtype=torch.int32)
            valid[i, :len(r)] = 1
            lengths[i] = len(r)
    return tokens, valid, lengths


def test_reference_unit_test_cases():
    t = GPUBPETrainer(base_vocab=16, merges=1, device="cuda", randomize_ties=False)
    t.fit([make_batch([[0, 1, 0, 1], [0, 2, 0, 2]])], log_every=100)
    assert t.merges == [(0, 1)]
    t = GPUBPETrainer(base_vocab=256, merges=1, device="cuda")
    res = t.fit(iter([make_batch([[1, 2, 1, 2, 3], [1, 2, 4, 2]]), make_batch([[1, 2, 1, 2], [1, 2, 1, 2]])]),
                log_every=10)
    assert t.merges[:1] == [(1, 2)] and res["transfer_metrics"]["merge_stats"]
    t = GPUBPETrainer(base_vocab=256, merges=3, device="cuda")
    res = t.fit([make_batch([[1, 2, 3, 1, 2, 4], [1, 2, 3, 1, 2, 3], [1, 2, 4, 2, 4]])], log_every=10)
    assert t.merges == [(1, 2), (256, 3), (256, 4)] and t.vocab_size == 259
    assert set(res) == {"base_vocab", "vocab_size", "merges", "warm_start", "transfer_metrics", "telemetry"}
    assert {"pair_count", "apply_merge", "host_sync"} <= set(res["telemetry"]["timings"])


def test_seeded_tie_randomization():
    batch = make_batch([[0, 1, 0, 1], [0, 2, 0, 2]])
    runs = []
    for seed in (123, 123, 456):
        t = GPUBPETrainer(base_vocab=16, merges=1, device="cuda", randomize_ties=True, tie_seed=seed)
        t.fit([batch], log_every=0)
        runs.append(t.merges)
    assert runs[0] == runs[1] and all(r in ([(0, 1)], [(0, 2)]) for r in runs)
    # the pick is random.Random(seed).randrange(n) over the tied keys in ascending order
    for seed, got in ((123, runs[0]), (456, runs[2])):
        assert got == [[(0, 1), (0, 2)][random.Random(seed).randrange(2)]]


def test_golden_trainer_fixtures_with_padding():
    g = load_golden("train.json")
    for case in g["random"] + g["adversarial"]:
        rows = case["rows"]
        nb = case.get("n_batches", 1)
        per = max(1, (len(rows) + nb - 1) // nb)
        batches = [make_batch(rows[i:i + per]) for i in range(0, len(rows), per)] or [make_batch([[]])]
        t = GPUBPETrainer(base_vocab=case["base_vocab"], merges=case["target"], device="cuda")
        t.fit(batches, log_every=0)
        raw = [tuple(m) for m in case["merges_raw"]]
        ids, off = O.flatten_rows(rows)
        om, _, reason = O.train_flat(ids, off, case["base_vocab"], case["target"], 1)
        assert t.merges[:len(om)] == raw[:len(om)] == om
        assert len(t.merges) == len(raw)            # same stop / padding rule as the reference
        assert t.vocab_size == case["vocab_size"]


def test_padding_draws_follow_the_global_random_module():
    rows = [[1, 2, 1, 2, 3], [7]]
    random.seed(77)
    t = GPUBPETrainer(base_vocab=256, merges=6, device="cuda")
    t.fit([make_batch(rows)], log_every=0)
    random.seed(77)
    expect = [(1, 2)]
    vocab = 257
    while len(expect) < 6:
        expect.append((random.randint(0, vocab - 1), random.randint(0, vocab - 1)))
        vocab += 1
    assert t.merges == expect and t.vocab_size == 262


def test_fit_bytes_and_artifacts(tmp_path):
    c = synth.config1_text(1 << 18, seed=3, file_bytes=1 << 14)
    ids, off = O.flatten_rows(corpus_rows(c))
    om, _, _ = O.train_flat(ids, off, 256, 64, 1)
    t = GPUBPETrainer(merges=64, device="cuda:0")
    res = t.fit_bytes(c.data, c.row_offsets)
    assert res["merges"] == om and t.vocab_size == 320
    paths = t.save_artifacts(tmp_path / "out")
    lines = open(paths["merges"], encoding="utf-8").read().splitlines()
    assert lines[0] == "#version: 0.2" and len(lines) == 65
    vocab = json.load(open(paths["vocab"], encoding="utf-8"))
    assert len(vocab) == 320
    # checkpoint round trip + warm start from the checkpointed merges reproduces the run
    t.save_checkpoint(tmp_path / "ck")
    t2 = GPUBPETrainer(merges=64, device="cuda:0")
    t2.load_state_dict(t2.load_checkpoint(tmp_path / "ck"))
    assert t2.merges == om
    t3 = GPUBPETrainer(merges=64, device="cuda:0", warm_start_merges=om[:20])
    assert t3.fit_bytes(c.data, c.row_offsets)["merges"] == om


def test_fit_bytes_from_pinned_pageable_and_device_memory():
    """The same bytes from pinned host memory, pageable host memory and device memory give the
    oracle's merges (a host buffer is copied in pieces under the pack kernel)."""
    c = synth.config2_mixed(1 << 20, seed=5, lexicon=1200, mean_doc_bytes=900)
    ids, off = O.flatten_rows(corpus_rows(c))
    om, _, _ = O.train_flat(ids, off, 256, 48, 1)
    host = torch.from_numpy(np.ascontiguousarray(c.data))
    pinned = torch.empty(host.numel(), dtype=torch.uint8, pin_memory=True)
    pinned.copy_(host)
    for data in (pinned, host, host.cuda()):
        t = GPUBPETrainer(merges=48, device="cuda:0")
        assert t.fit_bytes(data, c.row_offsets, log_every=0)["merges"] == om


def test_resume_equals_uninterrupted_run_and_warm_start_plan(tmp_path):
    c = synth.config2_mixed(1 << 18, seed=21, lexicon=1500, mean_doc_bytes=600)
    rows = [r.tolist() for r in corpus_rows(c)]
    batches = [make_batch(rows[:len(rows) // 2]), make_batch(rows[len(rows) // 2:])]
    full = GPUBPETrainer(merges=50, device="cuda")
    full.fit(batches, log_every=0)
    half = GPUBPETrainer(merges=20, device="cuda")
    half.fit(batches, log_every=0)
    half.save_checkpoint(tmp_path / "ck")
    resumed = GPUBPETrainer(merges=50, device="cuda")
    state = json.load(open(tmp_path / "ck" / "state.json"))
    assert state["dataset"]["batches"]["sequences"]            # the rewritten rows are in the checkpoint
    state["trainer"]["model"]["target_merges"] = 50
    resumed.fit([], log_every=0, resume_state=state)           # continues from those rows: no batches needed
    assert resumed.merges == full.merges and resumed.vocab_size == full.vocab_size
    assert resumed.merge_counts == full.merge_counts[20:]
    # a checkpoint without rows: the merges are replayed on the batches
    half.save_checkpoint(tmp_path / "ck2", include_batches=False)
    state = half.load_checkpoint(tmp_path / "ck2")
    assert "batches" not in state["payload"]["dataset"] and state["tensors"]["cached_pair_keys"].numel() > 0
    state["payload"]["trainer"]["model"]["target_merges"] = 50
    replayed = GPUBPETrainer(merges=50, device="cuda")
    replayed.fit(batches, log_every=0, resume_state=state)
    assert replayed.merges == full.merges
    # the histogram in tensors.pt is the histogram after the checkpoint's merges
    ids, off = O.flatten_rows(rows)
    for i, (a, b) in enumerate(half.merges):
        O.apply_merge_flat(ids, off, a, b, 256 + i)
    k, cnt = O.count_pairs_flat(ids[:off[-1]].copy(), off, 1)
    assert state["tensors"]["cached_pair_keys"].numpy().astype(np.uint64).tolist() == k.tolist()
    assert state["tensors"]["cached_pair_counts"].tolist() == cnt.tolist()
    # warm-start plan = the top-k bigrams of the initial histogram (ties to the smaller key)
    ids, off = O.flatten_rows(rows)
    k, cnt = O.count_pairs_flat(ids, off, 1)
    order = sorted(range(len(k)), key=lambda i: (-int(cnt[i]), int(k[i])))[:7]
    plan = GPUBPETrainer.precompute_warm_start_plan(batches, 7, device="cuda")
    assert plan["merges"] == [(int(k[i]) >> 32, int(k[i]) & 0xFFFFFFFF) for i in order]
    assert plan["counts"] == [int(cnt[i]) for i in order] and plan["histogram_size"] == len(k)
    assert plan["merges"][0] == full.merges[0]


def test_cli_train_bpe(tmp_path):
    from supertoken_b200 import cli
    c = synth.config1_text(1 << 16, seed=2, file_bytes=1 << 13)
    off = np.asarray(c.row_offsets)
    for i in range(len(off) - 1):
        (tmp_path / f"part{i:02d}.txt").write_bytes(np.asarray(c.data)[off[i]:off[i + 1]].tobytes())
    out = tmp_path / "tok"
    rc = cli.main(["train-bpe", "--data", str(tmp_path / "part*.txt"), "--merges", "30", "--out-dir", str(out),
                   "--log-every", "0", "--io-workers", "4", "--target-util", "0.8"])
    assert rc == 0
    om, _, _ = O.train_flat(*O.flatten_rows(corpus_rows(c)), 256, 30, 1)
    meta = json.load(open(out / "bpe_merges.json"))
    assert [tuple(m) for m in meta["merges"]] == om
    assert open(out / "merges.txt", encoding="utf-8").read().splitlines()[0] == "#version: 0.2"
    assert cli.main(["train-bpe", "--data", str(tmp_path / "nothing*"), "--out-dir", str(out)]) == 2


def test_randomised_ties_follow_the_reference_over_many_tied_merges(tmp_path):
    # tests/golden/extra.json: runs of the reference with randomize_ties=True on rows where every
    # selection is a tie between several pairs, so each merge is the seeded generator's pick
    g = load_golden("extra.json")
    for case in g["ties"]:
        t = GPUBPETrainer(base_vocab=case["base_vocab"], merges=case["target"], device="cuda",
                          randomize_ties=True, tie_seed=case["tie_seed"])
        t.fit([make_batch(case["rows"])], log_every=0)
        assert [list(m) for m in t.merges] == case["merges"]
        plain = GPUBPETrainer(base_vocab=case["base_vocab"], merges=case["target"], device="cuda")
        plain.fit([make_batch(case["rows"])], log_every=0)
        assert [list(m) for m in plain.merges] == case["merges_without_randomisation"]
    # interrupted and resumed: a checkpoint written by the reference after 6 of 12 merges, and one
    # written here, both continue to the merges of the uninterrupted reference run
    case = g["ties"][1]
    t = GPUBPETrainer(base_vocab=256, merges=case["target"], device="cuda")
    payload = json.loads(json.dumps(case["checkpoint_after_6"]))
    payload["trainer"]["model"]["target_merges"] = case["target"]
    t.fit([make_batch(case["rows"])], log_every=0, resume_state={"payload": payload})
    assert [list(m) for m in t.merges] == case["merges"]
    t = GPUBPETrainer(base_vocab=256, merges=case["target"], device="cuda", randomize_ties=True, tie_seed=case["tie_seed"])
    t.fit([make_batch(case["rows"])], log_every=0, checkpoint_interval=5, checkpoint_dir=str(tmp_path / "ck"))
    state = t.load_checkpoint(tmp_path / "ck")               # written after merge 10 of 12
    assert len(state["payload"]["trainer"]["model"]["merges"]) == 10 and "tie_breaker" in state["payload"]["rng"]
    t2 = GPUBPETrainer(base_vocab=256, merges=case["target"], device="cuda")
    t2.fit([], log_every=0, resume_state=state)
    assert [list(m) for m in t2.merges] == case["merges"]


def test_checkpoint_written_by_the_reference_resumes_here():
    ck = load_golden("extra.json")["checkpoint"]
    t = GPUBPETrainer(base_vocab=ck["base_vocab"], merges=ck["target"], device="cuda")
    payload = json.loads(json.dumps(ck["state_json"]))
    payload["trainer"]["model"]["target_merges"] = ck["target"]
    t.fit([], log_every=0, resume_state={"payload": payload, "tensors": {}})
    assert [list(m) for m in t.merges] == ck["merges_final"]
