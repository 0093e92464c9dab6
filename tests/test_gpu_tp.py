"""The tensor-parallel path on GPUs (needs B200s): the peer-store epilogue with its bounded-wait join, checked
against the CPU oracle on the JOINED result.  The multi-rank cases run one process per GPU and are skipped when
fewer than two GPUs are visible; the single-rank cases run the same kernels with a group of one."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

import oracle
import ojas_engine_b200 as ob
from ojas_engine_b200 import Q4_K, Q6_K, tp

from conftest import rel_l2
from helpers import synth_weights

pytestmark = pytest.mark.gpu


def _gpus() -> int:
    import torch
    return torch.cuda.device_count()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_group_of_one_matches_plain_gemv(gpu):
    """world = 1: the epilogue pushes nowhere, raises its own flag, and the join copies / sums one slot."""
    for t, n, k in [(Q4_K, 4096, 4096), (Q6_K, 1000, 2304)]:
        raw = synth_weights(t, n, k)
        w = gpu.load_weight(raw, t, n, k)
        x = np.random.default_rng(3).standard_normal((1, k)).astype(np.float32)
        xb, y1, y2 = gpu.upload(x), gpu.alloc(n), gpu.alloc(n)
        group = tp.TpGroup(gpu, 1, 0, n + (-n) % 4, lambda blob: [blob])
        gpu.gemv(w, xb, y1)
        for mode in (group.COL, group.ROW, group.COL):
            gpu.memset(y2, 0)
            group.gemv(w, xb)
            group.join(mode, y2, n)
            assert np.array_equal(gpu.read(y1, np.uint32, n), gpu.read(y2, np.uint32, n))
        assert rel_l2(gpu.read(y2, np.float32, n), oracle.matvec_kq(raw, t, n, k, x[0])) < 1e-5
        n4 = n - n % 4
        gpu.memset(y2, 0)
        group.allgather(y1, n4, y2)                    # the one-kernel form: push, flag, wait, copy out
        assert np.array_equal(gpu.read(y1, np.uint32, n4), gpu.read(y2, np.uint32, n4))
        group.close()
        for b in (w.buf, xb, y1, y2):
            gpu.free(b)


def test_join_wait_runs_out_and_reports(gpu):
    """A join whose flag nobody raises: the wait ends by itself after its limit, ojas_b200_sync reports a device
    status, and the context and the group stay usable."""
    n, k = 512, 1024
    raw = synth_weights(Q4_K, n, k)
    w = gpu.load_weight(raw, Q4_K, n, k)
    x = np.random.default_rng(4).standard_normal((1, k)).astype(np.float32)
    xb, y = gpu.upload(x), gpu.alloc(n)
    group = tp.TpGroup(gpu, 1, 0, n, lambda blob: [blob])
    group.set_wait_us(2000)
    group.join(group.COL, y, n)                       # no push came before: the flag of this step is never set
    with pytest.raises(ob.OjasB200Error, match="bounded wait"):
        gpu.sync()
    gpu.memset(y, 0)
    group.gemv(w, xb)                                  # the next step works
    group.join(group.COL, y, n)
    assert rel_l2(gpu.read(y, np.float32, n), oracle.matvec_kq(raw, Q4_K, n, k, x[0])) < 1e-5
    group.close()
    for b in (w.buf, xb, y):
        gpu.free(b)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_70b_projections(world):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_gpu_worker.py")
    port = str(_free_port())
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, worker, str(r), str(world), port], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=900)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n(timed out)"
        outs.append(out)
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r}:\n{outs[r][-2000:]}"
