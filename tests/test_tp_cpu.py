"""Tensor-parallel shard planning and the collective plumbing, on CPU: world-size-2 gloo ranks with the
oracle standing in for the local kernels (no GPU)."""
import os
import socket

import numpy as np
import pytest

import oracle
from ojas_engine_b200 import Q4_K, Q6_K, Q8_0, tp

from conftest import rel_l2
from helpers import synth_weights


def test_shard_plans_cover_exactly():
    for n, world in [(10240, 8), (4096, 3), (7, 8), (28672, 4)]:
        spans = [tp.shard_rows(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and sum(s[1] for s in spans) == n
        assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(world - 1))
    for k, world in [(8192, 8), (28672, 8), (28672, 3), (256, 4)]:
        spans = [tp.shard_k(k, world, r) for r in range(world)]
        assert all(s[0] % 256 == 0 and s[1] % 256 == 0 for s in spans)
        assert sum(s[1] for s in spans) == k
    with pytest.raises(ValueError):
        tp.shard_k(1000, 2, 0)


@pytest.mark.parametrize("t", [Q4_K, Q6_K, Q8_0])
def test_shards_reproduce_the_full_product(t):
    n, k, m, world = 48, 1024, 3, 4
    raw = synth_weights(t, n, k)
    x = np.random.default_rng(0).standard_normal((m, k)).astype(np.float32)
    full = oracle.matmul_kq(raw, t, n, k, x, threads=2)
    cols = []
    for r in range(world):
        sh = tp.ShardedLinear(raw, t, n, k, "col", r, world)
        cols.append(oracle.matmul_kq(sh.raw, t, sh.rows, k, x, threads=2))
    assert np.array_equal(np.concatenate(cols, axis=1), full)          # bit-identical per element
    part = np.zeros_like(full)
    for r in range(world):
        sh = tp.ShardedLinear(raw, t, n, k, "row", r, world)
        part += oracle.matmul_kq(sh.raw, t, n, sh.klen, sh.local_x(x), threads=2)
    assert rel_l2(part, full) < 1e-6                                   # only the fp32 summation order differs


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("mode", ["col", "row"])
def test_two_gloo_ranks(mode, tmp_path):
    import subprocess
    import sys
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_rank_worker.py")
    port = str(_free_port())
    outs = [str(tmp_path / f"rank{r}.npy") for r in range(2)]
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", port, mode, outs[r]]) for r in range(2)]
    for p in procs:
        assert p.wait(timeout=180) == 0
    n, k, m = 50, 768, 2
    raw = synth_weights(Q4_K, n, k)
    x = np.random.default_rng(1).standard_normal((m, k)).astype(np.float32)
    full = oracle.matmul_kq(raw, Q4_K, n, k, x, threads=1)
    for r in range(2):
        got = np.load(outs[r])
        assert got.shape == full.shape
        if mode == "col":
            assert np.array_equal(got, full)
        else:
            assert rel_l2(got, full) < 1e-6


@pytest.mark.parametrize("mode", ["col", "row"])
def test_a_rank_that_never_arrives_is_an_error_not_a_hang(mode, tmp_path):
    """Failure detection on the host: one rank leaves before the collective; the other rank's join raises after the
    group's timeout (5 s here) instead of waiting for ever."""
    import subprocess
    import sys
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_rank_worker.py")
    port = str(_free_port())
    outs = [str(tmp_path / f"rank{r}.txt") for r in range(2)]
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", port, "absent-" + mode, outs[r]]) for r in range(2)]
    for p in procs:
        p.wait(timeout=120)
    with open(outs[0]) as fh:
        outcome = fh.read()
    assert outcome.startswith("error"), outcome
