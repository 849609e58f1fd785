"""Host-side logic that needs no GPU: generators, artifact formats, batch flattening."""
import json

import numpy as np
import pytest
import torch

from supertoken_b200 import synth
from supertoken_b200.bpe_trainer import GPUBPETrainer, _flatten_batch, hash_merge_pair
from supertoken_b200.export import build_artifacts, bytes_to_unicode, write_artifacts


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
         "--token-bytes", "1024", "--log-every", "5", "--out-dir", str(tmp_path / "o"), "--privacy", "--privacy-salt", "s",
         "--tie-seed", "4", "--checkpoint-dir", str(tmp_path / "c"), "--checkpoint-every", "5", "--dry-run",
         "--warm-start", "3", "--io-workers", "2", "--prefetch-batches", "2", "--prefetch-jitter", "0.1", "--code-mode",
         "--meta-compress", "--aug-strength", "0.2"])
    assert args.merges == 10 and args.privacy and args.dry_run
    assert cli.main(["train-bpe", "--data", str(tmp_path / "*.txt"), "--dry-run"]) == 0
    data, off = cli.load_rows([str(tmp_path / "a.txt")], 300, None)
    assert data.dtype == np.int32 and data[0] == 300 and off.tolist() == [0, 12]
