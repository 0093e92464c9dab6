"""The scratch-free GEMM entry point (for callers that may not allocate device memory) against the
regular entry point, through the C ABI.  Collected last on purpose; passes alone and after the other tests."""
import ctypes as C

import numpy as np
import pytest

import ojas_engine_b200 as ob
from ojas_engine_b200 import Q4_K, Q6_K
from ojas_engine_b200 import lib as oblib

from conftest import rel_l2
from helpers import activations, gauss_weights

pytestmark = pytest.mark.gpu


def test_static_scratch_gemm_matches_workspace_gemm(gpu):
    """Two calls in a row (different shapes and formats, so the second must not depend on what the
    first left in the shared array) give the same output as ojas_b200_gemm."""
    for t, m, n, k, seed in [(Q4_K, 300, 640, 2048, 1), (Q6_K, 77, 384, 1024, 2)]:
        raw = gauss_weights(t, n, k, seed)
        x = activations(m, k, seed=seed + 50)
        w = gpu.load_weight(raw, t, n, k)
        xb, y_ref, y_new = gpu.upload(x), gpu.alloc(m * n), gpu.alloc(m * n)
        gpu.gemm(w, xb, y_ref, m)
        gpu.gemm_static(w, xb, y_new, m)
        a, b = gpu.read(y_ref, np.float32, m * n), gpu.read(y_new, np.float32, m * n)
        assert rel_l2(b, a) < 2e-3          # the tolerance the GEMM tests use
        assert rel_l2(b, a) < 1e-5          # same kernels: only the order of split-K atomic adds may differ
        gpu.gemm_static(w, xb, y_new, m, accum=True)
        assert rel_l2(gpu.read(y_new, np.float32, m * n), 2 * a) < 2e-3
        for buf in (w.buf, xb, y_ref, y_new):
            gpu.free(buf)


def _free_bytes():
    import torch
    return torch.cuda.mem_get_info(0)[0]


def test_static_scratch_gemm_allocates_nothing_and_replays_from_a_graph(gpu):
    """After the first call on the device, calls of other shapes and formats leave the device's free memory where it
    was (cudaMemGetInfo), and a call captured into a CUDA graph after that first call replays correctly."""
    cases = [(Q4_K, 64, 256, 1024, 3), (Q6_K, 300, 512, 2048, 4), (ob.Q8_0, 20, 128, 512, 5)]
    bufs = []
    for t, m, n, k, seed in cases:
        raw = gauss_weights(t, n, k, seed)
        x = activations(m, k, seed=seed + 60)
        w = gpu.load_weight(raw, t, n, k)
        bufs.append((w, gpu.upload(x), gpu.alloc(m * n), gpu.alloc(m * n), m, n))
    w, xb, y_ref, y_new, m, n = bufs[0]
    gpu.gemm_static(w, xb, y_new, m)                      # the first call on this device (set-up)
    gpu.sync()
    before = _free_bytes()
    for w, xb, y_ref, y_new, m, n in bufs:                # other tile widths and formats: nothing may be allocated
        gpu.gemm_static(w, xb, y_new, m)
    gpu.sync()
    assert _free_bytes() == before
    w, xb, y_ref, y_new, m, n = bufs[1]
    gpu.gemm(w, xb, y_ref, m)
    want = gpu.read(y_ref, np.float32, m * n)
    gpu.graph_begin()
    gpu.gemm_static(w, xb, y_new, m)
    g = gpu.graph_end()
    for _ in range(3):
        gpu.memset(y_new, 0)
        gpu.graph_launch(g)
        assert rel_l2(gpu.read(y_new, np.float32, m * n), want) < 1e-5
    gpu.graph_destroy(g)
    for w, xb, y_ref, y_new, m, n in bufs:
        for buf in (w.buf, xb, y_ref, y_new):
            gpu.free(buf)


def test_static_scratch_limit_is_enforced(gpu):
    cap = oblib.load().ojas_b200_gemm_static_capacity()
    assert cap == 8 << 20
    w = gpu.load_weight(gauss_weights(Q4_K, 4, 8192), Q4_K, 4, 8192)
    m = cap // 2 // 8192 + 1                 # one row past the capacity
    x, y = gpu.alloc(m * 8192), gpu.alloc(m * 4)
    with pytest.raises(ob.OjasB200Error, match="built-in array"):
        gpu.gemm_static(w, x, y, m)
    gpu.memset(x, 0)
    gpu.gemm_static(w, x, y, m - 1)          # exactly at the capacity is accepted
    assert not gpu.read(y, np.float32, (m - 1) * 4).any()
    for b in (w.buf, x, y):
        gpu.free(b)
