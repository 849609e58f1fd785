"""CPU checks of ``bench.py``: the reference arm's JSON contract and the merge-list hash.

The reference arm (``--impl reference``) is the one leg of the benchmark that runs without a GPU:
it times the CPU oracle on the workload.  Here it runs on a 1 MiB slice in a few seconds.
"""
import json
import os
import subprocess
import sys

import numpy as np

from oracle import oracle as O
from supertoken_b200 import synth
from tests.helpers import corpus_rows

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_arm(*extra):
    env = dict(os.environ)
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", *extra],
                         capture_output=True, text=True, cwd=ROOT, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    return json.loads(lines[0])


def test_reference_arm_line_has_the_contract_keys_and_the_oracle_merges():
    line = _reference_arm("--workload", "c1", "--bytes", str(1 << 20), "--steps", "4", "--warmup", "1")
    assert line["impl"] == "reference" and line["metric"] == "bpe_merges_per_sec" and line["unit"] == "merges/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 4 and line["warmup"] == 1
    assert line["value"] > 0 and abs(line["ms_per_step"] * line["value"] - 1000.0) < 1e-3 * 1000.0
    assert line["gpu_launches"] == 0
    cpu = line["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == line["value"] and cpu["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "merges/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert line["config"]["same_workload"] is True and line["config"]["merges_timed"] == 4
    # the hash is that of the oracle's first four merges of the same seeded corpus
    sys.path.insert(0, ROOT)
    import bench
    gen, _, seed, _, _ = bench.WORKLOADS["c1"]
    c = getattr(synth, gen)(n_bytes=1 << 20, seed=seed)
    ids, off = O.flatten_rows(corpus_rows(c))
    merges, counts, _ = O.train_flat(ids, off, 256, 4, 1)
    assert line["config"]["merges_sha256"] == bench.merges_sha256(merges, counts)


def test_merges_sha256_depends_on_order_pairs_and_counts():
    sys.path.insert(0, ROOT)
    import bench
    m, c = [(1, 2), (3, 4)], np.array([7, 5], dtype=np.int64)
    h = bench.merges_sha256(m, c)
    assert len(h) == 64
    assert bench.merges_sha256(m[::-1], c[::-1]) != h
    assert bench.merges_sha256(m, np.array([7, 6])) != h
    assert bench.merges_sha256([(1, 2), (4, 3)], c) != h
    assert bench.merges_sha256(list(m), [7, 5]) == h


def test_reference_arm_under_a_multi_rank_launch_runs_on_rank_0_only_with_all_cores():
    """Launched once per rank: rank 0 prints the line (with the thread count it set itself, whatever
    the launcher exported), the other ranks exit 0 without output."""
    args = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1",
            "--bytes", str(1 << 20), "--steps", "2", "--warmup", "1", "--gpus", "2"]
    env = dict(os.environ, WORLD_SIZE="2", OMP_NUM_THREADS="1")
    other = subprocess.run(args, capture_output=True, text=True, cwd=ROOT, timeout=300,
                           env=dict(env, RANK="1", LOCAL_RANK="1"))
    assert other.returncode == 0 and not [l for l in other.stdout.splitlines() if l.startswith("{")]
    first = subprocess.run(args, capture_output=True, text=True, cwd=ROOT, timeout=300,
                           env=dict(env, RANK="0", LOCAL_RANK="0"))
    assert first.returncode == 0, first.stderr[-2000:]
    line = json.loads([l for l in first.stdout.splitlines() if l.startswith("{")][0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2
    assert line["cpu_baseline"]["cores"] == (os.cpu_count() or 1)
