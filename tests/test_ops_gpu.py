"""Operator seam (count_pairs / apply_merge_once / select_best_pair on padded CUDA batches)
against fixtures produced by the reference's CPU operators (tests/golden/ops.json)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from supertoken_b200 import ops
from tests.helpers import load_golden

pytestmark = pytest.mark.gpu


def _count(tokens, valid, cap=None):
    B, L = tokens.shape
    cap = cap if cap is not None else max(B * max(L - 1, 0), 1)
    keys = torch.empty((cap, 2), dtype=torch.int32, device="cuda")
    counts = torch.empty((cap,), dtype=torch.int64, device="cuda")
    length = torch.zeros((1,), dtype=torch.int64, device="cuda")
    ops.count_pairs(tokens.cuda(), valid.cuda(), keys, counts, length)
    return keys.cpu(), counts.cpu(), int(length.item())


def test_count_pairs_fixtures():
    for case in load_golden("ops.json")["count"]:
        tokens = torch.tensor(case["tokens"], dtype=torch.int32)
        valid = torch.tensor(case["valid"], dtype=torch.uint8)
        keys, counts, n = _count(tokens, valid)
        assert n == len(case["keys"])
        packed = (keys[:n, 0].to(torch.int64) << 32) | keys[:n, 1].to(torch.int64)
        assert packed.tolist() == case["keys"] and counts[:n].tolist() == case["counts"]
        assert torch.all(keys[n:] == -1) and torch.all(counts[n:] == 0)


def test_count_pairs_reference_unit_cases():
    # tests/test_utils_count_pairs.py:160-167
    keys, counts, n = _count(torch.ones((1, 12), dtype=torch.int32), torch.ones((1, 12), dtype=torch.uint8))
    assert counts.dtype == torch.int64 and n == 1 and counts[:1].tolist() == [11]
    # :68-78 seeded random ids with an arbitrary valid mask against a Python dict
    torch.manual_seed(0)
    seqs = torch.randint(0, 512, (4, 32), dtype=torch.int32)
    valid = torch.randint(0, 2, (4, 32), dtype=torch.uint8)
    ref = {}
    for r in range(4):
        for i in range(31):
            if valid[r, i] and valid[r, i + 1]:
                k = (int(seqs[r, i]), int(seqs[r, i + 1]))
                ref[k] = ref.get(k, 0) + 1
    keys, counts, n = _count(seqs, valid)
    assert [tuple(p) for p in keys[:n].tolist()] == sorted(ref) and counts[:n].tolist() == [ref[k] for k in sorted(ref)]
    with pytest.raises(RuntimeError, match="capacity exceeded"):
        _count(seqs, valid, cap=3)


def test_apply_merge_fixtures():
    for case in load_golden("ops.json")["apply"]:
        tokens = torch.tensor(case["tokens"], dtype=torch.int32).cuda()
        valid = torch.tensor(case["valid"], dtype=torch.uint8).cuda()
        lengths = valid.sum(dim=1).to(torch.int32)
        t, v, l, spans = ops.apply_merge_once(tokens, valid, lengths, case["a"], case["b"], case["new"])
        assert t.cpu().tolist() == case["out_tokens"] and v.cpu().tolist() == case["out_valid"]
        assert l.cpu().tolist() == case["out_lengths"]
        assert spans.cpu().to(torch.int32).tolist() == case["spans"]


def test_apply_merge_long_rows_against_oracle():
    rng = np.random.default_rng(3)
    for B, Lw, alphabet in ((3, 10000, 2), (40, 700, 3), (1, 2048, 1), (2, 2049, 1), (5, 4097, 2)):
        tok = rng.integers(0, alphabet, (B, Lw)).astype(np.int32)
        lens = rng.integers(0, Lw + 1, B)
        val = (np.arange(Lw)[None, :] < lens[:, None]).astype(np.uint8)
        tok[val == 0] = -1
        for a, b in ((0, 0), (0, 1 % alphabet)):
            t_ref, v_ref = tok.copy(), val.copy()
            l_ref, s_ref = O.apply_merge_rows(t_ref, v_ref, a, b, 99)
            t = torch.from_numpy(tok.copy()).cuda()
            v = torch.from_numpy(val.copy()).cuda()
            l = torch.zeros(B, dtype=torch.int32, device="cuda")
            t, v, l, s = ops.apply_merge_once(t, v, l, a, b, 99)
            assert np.array_equal(t.cpu().numpy(), t_ref) and np.array_equal(v.cpu().numpy(), v_ref)
            assert l.cpu().tolist() == l_ref.tolist() and np.array_equal(s.cpu().numpy(), s_ref)


def test_apply_merge_uint16_lengths_and_overflow_guard():
    tokens = torch.tensor([[1, 2, 1, 2, 3]], dtype=torch.int32).cuda()
    valid = torch.ones_like(tokens, dtype=torch.uint8)
    lengths = torch.tensor([5], dtype=torch.uint16).cuda()
    ops.apply_merge_once(tokens, valid, lengths, 1, 2, 256)
    assert lengths.cpu().to(torch.int32).tolist() == [3] and tokens.cpu().tolist() == [[256, 256, 3, 0, 0]]
    with pytest.raises(OverflowError):   # tests/test_utils_apply_merge.py:129-135
        ops.apply_merge_once(tokens, valid, lengths, 0, 1, 1 << 32)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.apply_merge_once(tokens.cpu(), valid.cpu(), lengths.cpu(), 0, 1, 2)


def test_select_best_pair_fixtures():
    for case in load_golden("ops.json")["select"]:
        h = ops.PairHistogramResult(torch.tensor(case["keys"], dtype=torch.int64).cuda(),
                                    torch.tensor(case["counts"], dtype=torch.int64).cuda())
        key, count, idx = ops.select_best_pair(h)
        assert (key, count) == (case["best_key"], case["best_count"]) and case["keys"][idx] == key
    assert ops.select_best_pair(ops.PairHistogramResult(torch.empty(0, dtype=torch.int64),
                                                        torch.empty(0, dtype=torch.int64))) == (None, 0, None)
