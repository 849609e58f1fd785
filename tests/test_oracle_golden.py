"""Pins the C oracle to the reference: known answers from the reference's own unit
tests and fixtures produced by running the reference itself (tests/golden/)."""
import numpy as np
import pytest

from oracle import oracle as O
from supertoken_b200 import synth
from tests.helpers import corpus_rows, learned_prefix, load_golden


def test_known_answers_from_reference_unit_tests():
    # tests/test_bpe_trainer.py:191-202 (tie -> smallest key)
    m, _, _ = O.train_flat(*O.flatten_rows([[0, 1, 0, 1], [0, 2, 0, 2]]), 16, 1)
    assert m == [(0, 1)]
    # tests/test_bpe_trainer.py:463-477 (first merge over two batches)
    m, _, _ = O.train_flat(*O.flatten_rows([[1, 2, 1, 2, 3], [1, 2, 4, 2], [1, 2, 1, 2], [1, 2, 1, 2]]), 256, 1)
    assert m == [(1, 2)]
    # tests/test_bpe_trainer.py:484-501 (cache-off baseline)
    m, _, _ = O.train_flat(*O.flatten_rows([[1, 2, 3, 1, 2, 4], [1, 2, 3, 1, 2, 3], [1, 2, 4, 2, 4]]), 256, 3)
    assert m == [(1, 2), (256, 3), (256, 4)]
    # tests/test_utils_count_pairs.py:160-167
    k, c = O.count_pairs_rows(np.ones((1, 12), np.int32), np.ones((1, 12), np.uint8))
    assert c.dtype == np.int64 and c.tolist() == [11] and k.tolist() == [(1 << 32) | 1]


def test_count_matches_python_dict_like_reference_test():
    # tests/test_utils_count_pairs.py:68-78: seeded random ids with an arbitrary valid mask
    rng = np.random.default_rng(0)
    seqs = rng.integers(0, 512, (4, 32)).astype(np.int32)
    valid = rng.integers(0, 2, (4, 32)).astype(np.uint8)
    ref = {}
    for r in range(4):
        for i in range(31):
            if valid[r, i] and valid[r, i + 1]:
                key = (int(seqs[r, i]), int(seqs[r, i + 1]))
                ref[key] = ref.get(key, 0) + 1
    k, c = O.count_pairs_rows(seqs, valid)
    got = [((int(x) >> 32, int(x) & 0xFFFFFFFF), int(y)) for x, y in zip(k, c)]
    assert got == sorted(ref.items())


def test_run_collapse_semantics():
    ids, off = O.flatten_rows([[7, 7, 7, 7, 8], [7, 7, 7], [5, 7, 7, 7, 7, 7, 9, 7, 7]])
    O.apply_merge_flat(ids, off, 7, 7, 256)
    assert ids[:off[-1]].tolist() == [256, 8, 256, 5, 256, 9, 256]
    assert off.tolist() == [0, 2, 3, 7]


def test_ops_fixtures():
    g = load_golden("ops.json")
    for case in g["count"]:
        k, c = O.count_pairs_rows(np.array(case["tokens"], np.int32), np.array(case["valid"], np.uint8))
        assert k.tolist() == case["keys"] and c.tolist() == case["counts"]
    for case in g["select"]:
        bk, bc = O.select_best(np.array(case["keys"], np.uint64), np.array(case["counts"], np.int64))
        assert (bk, bc) == (case["best_key"], case["best_count"])
    for case in g["apply"]:
        t = np.array(case["tokens"], np.int32)
        v = np.array(case["valid"], np.uint8)
        lens, spans = O.apply_merge_rows(t, v, case["a"], case["b"], case["new"])
        assert t.tolist() == case["out_tokens"]
        assert v.tolist() == case["out_valid"]
        assert lens.tolist() == case["out_lengths"]
        assert spans.astype(int).tolist() == case["spans"]


@pytest.mark.parametrize("mode", [0, 1])
def test_train_fixtures(mode):
    g = load_golden("train.json")
    for case in g["random"] + g["adversarial"]:
        ids, off = O.flatten_rows(case["rows"])
        m, _, reason = O.train_flat(ids, off, case["base_vocab"], case["target"], mode)
        learned_prefix(case, m, reason)
    for case in g["synthetic"]:
        c = getattr(synth, case["generator"])(**case["kwargs"])
        assert c.sha256() == case["sha256"]
        ids, off = O.flatten_rows(corpus_rows(c))
        m, _, reason = O.train_flat(ids, off, case["base_vocab"], case["target"], mode)
        assert reason == 0
        assert [tuple(x) for x in case["merges_raw"]] == m


def test_literal_and_fast_count_agree():
    rng = np.random.default_rng(5)
    for alphabet, n in ((3, 200000), (70000, 300000)):
        ids = rng.integers(0, alphabet, n).astype(np.int32)
        cuts = np.sort(rng.choice(n, 50, replace=False))
        off = np.concatenate([[0], cuts, [n]]).astype(np.int64)
        k0, c0 = O.count_pairs_flat(ids, off, 0)
        k1, c1 = O.count_pairs_flat(ids, off, 1)
        assert np.array_equal(k0, k1) and np.array_equal(c0, c1)
        assert c0.sum() == sum(max(int(off[i + 1] - off[i]) - 1, 0) for i in range(len(off) - 1))
