"""Host-side logic that needs no GPU: generators, artifact formats, batch flattening."""
import json
import os

import numpy as np
import pytest
import torch

from supertoken_b200 import synth
from supertoken_b200.bpe_trainer import GPUBPETrainer, _flatten_batch, hash_merge_pair
from supertoken_b200.export import (build_artifacts, bytes_to_unicode, load_tiktoken_merges,
                                    load_warm_start_merges, write_artifacts)
from tests.helpers import load_golden


def test_generators_numpy_equals_torch():
    for fn, kw in (("config1_text", dict(n_bytes=1 << 16, seed=0, file_bytes=1 << 12)),
                   ("config2_mixed", dict(n_bytes=1 << 16, seed=1, lexicon=3000, mean_doc_bytes=512)),
                   ("config5_adversarial", dict(n_bytes=1 << 18, seed=4))):
        a = getattr(synth, fn)(**kw)
        b = getattr(synth, fn)(device="cpu", **kw)
        assert np.array_equal(a.data, b.data.numpy()), fn
        assert np.array_equal(np.asarray(a.row_offsets), b.row_offsets.numpy()), fn
        assert len(a.data) == kw["n_bytes"]
    ids, off = synth.config3_ids(1 << 16, seed=2)
    idt, oft = synth.config3_ids(1 << 16, seed=2, device="cpu")
    assert np.array_equal(ids, idt.numpy()) and np.array_equal(off, oft.numpy())
    assert ids.min() >= 0 and ids.max() < 65536 and off[0] == 0 and off[-1] == 1 << 16


def test_config2_is_valid_utf8_with_three_scripts():
    c = synth.config2_mixed(1 << 16, seed=1, lexicon=3000, mean_doc_bytes=512)
    text = c.data.tobytes().decode("utf-8", errors="ignore")
    assert any("Ѐ" <= ch <= "ӿ" for ch in text)
    assert any("一" <= ch <= "鿿" for ch in text)
    gaps = np.diff(np.asarray(c.row_offsets))
    assert gaps.min() > 0 and 200 < gaps.mean() < 1200


def test_byte_level_alphabet():
    enc = bytes_to_unicode()
    assert len(enc) == 256 and len(set(enc.values())) == 256
    assert enc[ord("a")] == "a" and enc[ord(" ")] == "Ġ" and enc[10] == "Ċ"


def test_artifact_formats(tmp_path):
    merges = [(104, 101), (256, 108), (32, 257)]
    paths = write_artifacts(str(tmp_path), 256, merges, 259)
    vocab = json.load(open(paths["vocab"], encoding="utf-8"))
    assert vocab["he"] == 256 and vocab["hel"] == 257 and vocab["Ġhel"] == 258 and len(vocab) == 259
    lines = open(paths["merges"], encoding="utf-8").read().splitlines()
    assert lines == ["#version: 0.2", "h e", "he l", "Ġ hel"]
    tok = json.load(open(paths["tokenizer"], encoding="utf-8"))
    assert tok["model"]["type"] == "BPE" and tok["model"]["merges"] == lines[1:]
    tk = open(paths["tiktoken_merges"], "rb").read().splitlines()
    assert len(tk) == 259 and tk[256] == b"aGU= 256"
    meta = json.load(open(paths["metadata"]))
    assert meta["merges"] == [[104, 101], [256, 108], [32, 257]] and meta["vocab_size"] == 259
    with pytest.raises(ValueError):
        build_artifacts(256, [(300, 1)], 257)
    with pytest.raises(ValueError):
        build_artifacts(256, merges, 300)


def test_flatten_batch_and_prefix_rule():
    tokens = torch.tensor([[1, 2, 3, -1], [4, -1, -1, -1], [-1, -1, -1, -1]], dtype=torch.int32)
    valid = torch.tensor([[1, 1, 1, 0], [1, 0, 0, 0], [0, 0, 0, 0]], dtype=torch.uint8)
    ids, off = _flatten_batch((tokens, valid, None))
    assert ids.tolist() == [1, 2, 3, 4] and off.tolist() == [0, 3, 4, 4]
    valid[0, 1] = 0
    with pytest.raises(ValueError):
        _flatten_batch((tokens, valid, None))


def test_privacy_helpers():
    assert hash_merge_pair((1, 2), b"s") != hash_merge_pair((1, 2), b"t")
    t = GPUBPETrainer(merges=2, device="cuda:0", privacy_mode=True, tie_seed=5)
    assert t.randomize_ties and t._privacy_summary()["mode"] == "tie-randomize"
    with pytest.raises(ValueError):
        GPUBPETrainer(device="cuda:0").fit([], checkpoint_interval=5)


def test_cli_parses_the_reference_flags(tmp_path):
    from supertoken_b200 import cli
    (tmp_path / "a.txt").write_bytes(b"hello world")
    args = cli.build_parser().parse_args(
        ["train-bpe", "--data", str(tmp_path / "*.txt"), "--bos", "1", "--eos", "2", "--seed", "3", "--device", "cuda",
         "--merges", "10", "--base-vocab", "256", "--target-util", "0.5", "--min-batch", "1", "--max-batch", "8",
         "--token-bytes", "1024", "--log-every", "5", "--out-dir", str(tmp_path / "o"), "--privacy", "tie-randomize", "--privacy-salt", "s",
         "--tie-seed", "4", "--checkpoint-dir", str(tmp_path / "c"), "--checkpoint-every", "5", "--dry-run",
         "--warm-start", "seeds.json", "--io-workers", "2", "--prefetch-batches", "2", "--prefetch-jitter", "0.1", "--code-mode",
         "--meta-compress", "--aug-strength", "0.2"])
    assert args.merges == 10 and args.privacy == "tie-randomize" and args.dry_run and args.warm_start == "seeds.json"
    assert cli.main(["train-bpe", "--data", str(tmp_path / "*.txt"), "--dry-run"]) == 0
    data, off = cli.load_rows([str(tmp_path / "a.txt")], 300, None)
    assert data.dtype == np.int32 and data[0] == 300 and off.tolist() == [0, 12]


def test_artifact_files_equal_the_reference_writers_byte_for_byte(tmp_path):
    # tests/golden/extra.json holds the five files GPUBPETrainer.save_artifacts of the reference wrote
    for case in load_golden("extra.json")["artifacts"]:
        merges = [tuple(m) for m in case["merges"]]
        t = GPUBPETrainer(base_vocab=case["base_vocab"], merges=len(merges), device="cuda:0")
        t.merges, t.vocab_size = merges, case["base_vocab"] + len(merges)
        paths = t.save_artifacts(tmp_path / f"a{case['base_vocab']}")
        for key, p in paths.items():
            name = p.split("/")[-1]
            got = open(p, "rb").read().decode("utf-8")
            if key == "metadata":
                meta = json.loads(got)
                meta.pop("tiktoken_merges_path")
                got = json.dumps(meta, sort_keys=True)
            assert got == case["files"][name], name
        # and the way back: the merges can be read from the files as the reference's loaders read them
        assert load_tiktoken_merges(paths["tiktoken_merges"], base_vocab=case["base_vocab"]) == merges or case["base_vocab"] != 256
        assert load_warm_start_merges(paths["metadata"]) == merges
    tok = t.export_tokenizer(tmp_path / "tok")
    assert tok.vocab and tok.artifact_path.endswith("tokenizer.json")


def test_checkpoints_written_by_the_reference_load(tmp_path):
    g = load_golden("extra.json")
    ck = g["checkpoint"]
    t = GPUBPETrainer(merges=ck["target"], device="cuda:0")
    rec = t.load_state_dict({"payload": ck["state_json"], "tensors": {}})
    assert [list(m) for m in t.merges] == ck["merges_at_checkpoint"] and t.vocab_size == 256 + len(t.merges)
    assert rec["step"] == len(t.merges) and rec["sequences"] is not None
    # the rows in the checkpoint are the input rows with the checkpoint's merges applied
    from oracle import oracle as O
    ids, off = O.flatten_rows(ck["rows"])
    for i, (a, b) in enumerate(t.merges):
        O.apply_merge_flat(ids, off, a, b, 256 + i)
    assert [r for r in rec["sequences"]] == [ids[off[i]:off[i + 1]].tolist() for i in range(len(off) - 1)]
    # a checkpoint of a run with randomised ties carries the generator's state
    tie = g["ties"][1]
    t = GPUBPETrainer(merges=tie["target"], device="cuda:0")
    rec = t.load_state_dict({"payload": tie["checkpoint_after_6"]})
    assert t.randomize_ties and t._tie_seed_value == 123 and rec["sequences"] is None
    import random
    fresh = random.Random(123)
    assert t._tie_rng.getstate() != fresh.getstate()
    # our own checkpoint files have the reference's layout and round-trip
    t.save_checkpoint(tmp_path / "ck", include_batches=False)
    state = t.load_checkpoint(tmp_path / "ck")
    assert set(state) == {"payload", "tensors"} and set(state["payload"]) >= {"version", "trainer", "dataset", "rng"}
    assert set(state["tensors"]) == {"cached_pair_keys", "cached_pair_counts"}
    t2 = GPUBPETrainer(merges=3, device="cuda:0")
    t2.load_state_dict(state)
    assert t2.merges == t.merges and t2._tie_rng.getstate() == t._tie_rng.getstate()
    assert state["payload"]["trainer"]["model"]["merges"] == tie["checkpoint_after_6"]["trainer"]["model"]["merges"]


# the reference checkout, when there is one beside the build (STBPE_REFERENCE_DIR names another place)
_HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get("STBPE_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


@pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="needs the reference checkout")
def test_drop_in_seam_of_the_reference_command_line(tmp_path, monkeypatch):
    """The swap a maintainer makes: rebind ``GPUBPETrainer`` in the reference's modules, then use the
    reference's own ``train-bpe`` parser and trainer factory (``main.py:21-30``, ``:661-689``, ``:2180-2363``).
    Runs where the reference source tree exists; constructing the trainer needs no GPU."""
    import importlib
    import inspect
    import sys
    monkeypatch.syspath_prepend(REFERENCE)
    monkeypatch.chdir(tmp_path)
    ref_mod = importlib.import_module("gpu_tokenizer.bpe_trainer")
    ref_cls = ref_mod.GPUBPETrainer
    import supertoken_b200.base as base_mod
    importlib.reload(base_mod)   # picks the reference's BaseTrainer now that it is importable
    import supertoken_b200.bpe_trainer as ours_mod
    importlib.reload(ours_mod)
    ours = ours_mod.GPUBPETrainer
    try:
        from gpu_tokenizer.trainers.base import BaseTrainer
        assert issubclass(ours, BaseTrainer)
        for name in ("__init__", "fit"):
            assert list(inspect.signature(getattr(ours, name)).parameters) == \
                list(inspect.signature(getattr(ref_cls, name)).parameters), name
        for name in ("state_dict", "save_checkpoint"):
            assert set(inspect.signature(getattr(ref_cls, name)).parameters) <= \
                set(inspect.signature(getattr(ours, name)).parameters), name
        for attr in ("merges", "vocab_size", "base_vocab", "target_merges", "devices", "device", "autoscaler",
                     "sync_every", "metrics", "throughput_metrics", "handle_chunk_start", "import_merges",
                     "precompute_warm_start_plan", "state_dict", "load_state_dict", "save_checkpoint",
                     "load_checkpoint", "export_tokenizer", "save_artifacts", "save", "_bytes_to_unicode",
                     "_enable_histogram_cache", "_top_pairs_limit", "_cpu_fallback_batches", "_active_batch_size"):
            assert hasattr(ours(merges=1, device="cuda:0"), attr), attr
        main = importlib.import_module("main")
        monkeypatch.setattr(ref_mod, "GPUBPETrainer", ours)
        monkeypatch.setattr(main, "GPUBPETrainer", ours)
        (tmp_path / "a.txt").write_bytes(b"hello hello world")
        args = main._parser().parse_args(
            ["train-bpe", "--data", str(tmp_path / "a.txt"), "--merges", "12", "--base-vocab", "256", "--device", "cuda:0",
             "--out-dir", str(tmp_path / "out"), "--log-every", "0", "--tie-seed", "3", "--checkpoint-every", "4",
             "--checkpoint-dir", str(tmp_path / "ck"), "--io-workers", "1", "--target-util", "0.8"])
        assert args.func is main._cmd_train_bpe
        trainer = main._build_bpe_trainer(args)[0]    # the reference's own factory (main.py:661-689)
        assert isinstance(trainer, ours) and trainer.target_merges == 12 and trainer.base_vocab == 256
    finally:
        for m in [k for k in sys.modules if k == "main" or k.startswith("gpu_tokenizer")]:
            sys.modules.pop(m, None)
        importlib.reload(base_mod)
        importlib.reload(ours_mod)


def test_warm_start_sources_in_every_accepted_form(tmp_path):
    """``train-bpe --warm-start`` takes a JSON manifest (merges at the top level, under ``trainer`` or
    under ``trainer.model``), a bare JSON list, a ``.tiktoken`` rank table or a directory holding one
    of the exported files (``main.py:501-575`` of the reference); anything else ends the command."""
    merges = [(104, 101), (108, 108), (256, 257), (258, 111)]          # h e | l l | he ll | hell o
    as_lists = [list(p) for p in merges]
    forms = {"top.json": {"merges": as_lists}, "trainer.json": {"trainer": {"merges": as_lists}},
             "model.json": {"trainer": {"model": {"merges": as_lists}}}, "bare.json": as_lists}
    for name, payload in forms.items():
        (tmp_path / name).write_text(json.dumps(payload))
        assert load_warm_start_merges(str(tmp_path / name)) == merges, name
    paths = write_artifacts(str(tmp_path / "out"), 256, merges, 260)
    assert load_warm_start_merges(paths["tiktoken_merges"]) == merges
    assert load_warm_start_merges(str(tmp_path / "out")) == merges          # directory: merges.tiktoken first
    os.remove(paths["tiktoken_merges"])
    assert load_warm_start_merges(str(tmp_path / "out")) == merges          # then bpe_merges.json
    assert load_warm_start_merges(None) is None and load_warm_start_merges("") is None
    (tmp_path / "empty").mkdir()
    (tmp_path / "bad.json").write_text(json.dumps({"merges": [[1, 2, 3]]}))
    (tmp_path / "none.json").write_text(json.dumps({"trainer": {}}))
    (tmp_path / "plan.txt").write_text("1 2\n")
    for bad in ("missing.json", "empty", "bad.json", "none.json", "plan.txt"):
        with pytest.raises(SystemExit):
            load_warm_start_merges(str(tmp_path / bad))


def test_round_budget_between_host_checks_is_the_same_on_every_rank():
    """Ranks enqueue rounds without talking to each other, so the number of rounds until the next look
    at the device state may depend only on what all ranks know: merges committed and the target."""
    from supertoken_b200.dist import rounds_until_next_check
    assert rounds_until_next_check(0, 32000, 256) == 32            # early: re-pack and filter decisions
    assert rounds_until_next_check(511, 32000, 256) == 32
    assert rounds_until_next_check(512, 32000, 256) == 256
    assert rounds_until_next_check(0, 20, 256) == 21               # never more than the target needs (+1 applies the last)
    assert rounds_until_next_check(19, 20, 256) == 2
    assert rounds_until_next_check(20, 20, 256) == 1               # always progress
    assert rounds_until_next_check(100, 20, 8) == 1
    for done in range(0, 700, 37):
        for target in (1, 50, 600, 32000):
            n = rounds_until_next_check(done, target, 256)
            assert 1 <= n <= 256 and (done >= target or n <= target - done + 1)
