"""The activation producers that end in Q8_K (RMSNorm, SiLU * up) against the CPU oracle (needs a B200)."""
import numpy as np
import pytest

import oracle
import ojas_engine_b200 as ob
from ojas_engine_b200 import Q4_K

from conftest import rel_l2
from helpers import activations, synth_weights

pytestmark = pytest.mark.gpu


def _q8k_bufs(gpu, m, k):
    return gpu.alloc_bytes(m * k), gpu.alloc(m * k // 256), gpu.alloc_bytes(m * k // 32 * 4)


def _read_q8k(gpu, q, s, b, m, k):
    return (gpu.read(q, np.int8, m * k).reshape(m, k), gpu.read(s, np.float32, m * k // 256).reshape(m, -1),
            gpu.read(b, np.int32, m * k // 32).reshape(m, -1))


@pytest.mark.parametrize("m,k", [(1, 4096), (5, 8192), (3, 768), (2, 14336)])
def test_rmsnorm_q8k(gpu, m, k):
    x = activations(m, k, seed=31) * np.float32(3.0)
    w = (1.0 + 0.1 * activations(1, k, seed=32)[0]).astype(np.float32)
    eps = 1e-6
    xb, wb, xn = gpu.upload(x), gpu.upload(w), gpu.alloc(m * k)
    q, s, b = _q8k_bufs(gpu, m, k)
    gpu.rmsnorm_q8k(xb, wb, eps, m, k, q, s, b, xn)
    got_n = gpu.read(xn, np.float32, m * k).reshape(m, k)
    got_q, got_s, got_b = _read_q8k(gpu, q, s, b, m, k)
    for r in range(m):
        want_n = oracle.rmsnorm(x[r], w, eps)
        assert rel_l2(got_n[r], want_n) < 1e-5            # tree sum vs in-order sum: fp32 rounding only
        ws, wq, wb_ = oracle.quant_q8k(got_n[r])            # the quantization step itself: bit for bit
        assert np.array_equal(got_s[r].view(np.uint32), ws.view(np.uint32))
        assert np.array_equal(got_q[r], wq) and np.array_equal(got_b[r], wb_)
        # against the whole CPU composition only a rounding step of a few values may differ
        _, cq, _ = oracle.quant_q8k(want_n)
        assert np.abs(got_q[r].astype(np.int32) - cq.astype(np.int32)).max() <= 1
        assert np.count_nonzero(got_q[r] != cq) <= max(4, k // 256)
    for buf in (xb, wb, xn, q, s, b):
        gpu.free(buf)


def test_rmsnorm_q8k_feeds_the_gemv(gpu):
    """norm -> Q8_K -> gemv_q8k equals norm -> f32 -> gemv (which quantizes in its prologue), bit for bit."""
    n, k = 1024, 4096
    raw = synth_weights(Q4_K, n, k)
    wl = gpu.load_weight(raw, Q4_K, n, k)
    x = activations(1, k, seed=33)
    g = np.ones(k, np.float32)
    xb, gb, xn = gpu.upload(x), gpu.upload(g), gpu.alloc(k)
    q, s, b = _q8k_bufs(gpu, 1, k)
    y1, y2 = gpu.alloc(n), gpu.alloc(n)
    gpu.rmsnorm_q8k(xb, gb, 1e-5, 1, k, q, s, b, xn)
    gpu.gemv_q8k(wl, q, s, b, y1, 1)
    gpu.gemv(wl, xn, y2, 1)
    assert np.array_equal(gpu.read(y1, np.uint32, n), gpu.read(y2, np.uint32, n))
    want = oracle.matvec_kq(raw, Q4_K, n, k, oracle.rmsnorm(x[0], g, 1e-5))
    assert rel_l2(gpu.read(y1, np.float32, n), want) < 2e-3
    for buf in (wl.buf, xb, gb, xn, q, s, b, y1, y2):
        gpu.free(buf)


@pytest.mark.parametrize("m,k", [(1, 14336), (7, 1024)])
def test_silu_mul_q8k_bit_exact(gpu, m, k):
    g, u = activations(m, k, seed=41) * np.float32(2.0), activations(m, k, seed=42)
    gb, ub = gpu.upload(g), gpu.upload(u)
    q, s, b = _q8k_bufs(gpu, m, k)
    gpu.silu_mul_q8k(gb, ub, m, k, q, s, b)
    got_q, got_s, got_b = _read_q8k(gpu, q, s, b, m, k)
    diff = 0
    for r in range(m):
        ws, wq, wb = oracle.quant_q8k(oracle.silu_mul(g[r], u[r]))
        # expf on the device and in libm may differ in the last bit; a handful of values may then round the other way
        assert np.allclose(got_s[r], ws, rtol=1e-6)
        assert np.abs(got_q[r].astype(np.int32) - wq.astype(np.int32)).max() <= 1
        diff += int(np.count_nonzero(got_q[r] != wq))
    assert diff <= max(2, m * k // 2048)
    for buf in (gb, ub, q, s, b):
        gpu.free(buf)


def test_producer_argument_errors(gpu):
    x = gpu.alloc(512)
    q, s, b = _q8k_bufs(gpu, 1, 512)
    with pytest.raises(ob.OjasB200Error, match="multiple of 256"):
        gpu.rmsnorm_q8k(x, x, 1e-5, 1, 300, q, s, b)
    with pytest.raises(ob.OjasB200Error, match="multiple of 256"):
        gpu.silu_mul_q8k(x, x, 1, 100, q, s, b)
    for buf in (x, q, s, b):
        gpu.free(buf)


@pytest.mark.parametrize("t,n,k,m", [(Q4_K, 1024, 4096, 1), (Q4_K, 520, 768, 3), (ob.Q6_K, 512, 2048, 2), (ob.Q8_0, 256, 1024, 1),
                                     (Q4_K, 6144, 4096, 1)])
def test_gemv_with_the_norm_in_its_prologue(gpu, t, n, k, m):
    """ojas_b200_gemv_rmsnorm against the CPU composition (rmsnorm, then matvec_kq) and against the two-launch form
    (producer, then gemv_q8k): the norm's sum of squares is a tree sum in both device forms, so they agree with each
    other and with the CPU to fp32 rounding plus, rarely, a Q8_K rounding step of a value."""
    raw = synth_weights(t, n, k)
    wl = gpu.load_weight(raw, t, n, k)
    x = activations(m, k, seed=41) * np.float32(2.5)
    g = (1.0 + 0.1 * activations(1, k, seed=42)[0]).astype(np.float32)
    eps = 1e-5
    xb, gb = gpu.upload(x), gpu.upload(g)
    y1, y2 = gpu.alloc(m * n), gpu.alloc(m * n)
    gpu.gemv_rmsnorm(wl, xb, gb, eps, y1, m)
    got = gpu.read(y1, np.float32, m * n).reshape(m, n)
    want = np.stack([oracle.matvec_kq(raw, t, n, k, oracle.rmsnorm(x[r], g, eps)) for r in range(m)])
    assert rel_l2(got, want) < 2e-4
    if t != ob.Q8_0:
        q, s, b = _q8k_bufs(gpu, m, k)
        gpu.rmsnorm_q8k(xb, gb, eps, m, k, q, s, b)
        gpu.gemv_q8k(wl, q, s, b, y2, m)
        two = gpu.read(y2, np.float32, m * n).reshape(m, n)
        assert rel_l2(got, two) < 2e-4
        for buf in (q, s, b):
            gpu.free(buf)
    for buf in (wl.buf, xb, gb, y1, y2):
        gpu.free(buf)


@pytest.mark.parametrize("t,n,k,m", [(ob.Q6_K, 512, 14336, 1), (Q4_K, 520, 768, 3), (ob.Q8_0, 256, 1024, 2)])
def test_gemv_with_swiglu_in_its_prologue(gpu, t, n, k, m):
    """ojas_b200_gemv_silu_mul against the two-launch form (producer, then gemv_q8k) bit for bit (the same expression,
    the same quantization), and against the CPU composition."""
    raw = synth_weights(t, n, k)
    wl = gpu.load_weight(raw, t, n, k)
    g, u = activations(m, k, seed=51) * np.float32(2.0), activations(m, k, seed=52)
    gb, ub = gpu.upload(g), gpu.upload(u)
    y1, y2 = gpu.alloc(m * n), gpu.alloc(m * n)
    gpu.gemv_silu_mul(wl, gb, ub, y1, m)
    got = gpu.read(y1, np.float32, m * n).reshape(m, n)
    want = np.stack([oracle.matvec_kq(raw, t, n, k, oracle.silu_mul(g[r], u[r])) for r in range(m)])
    assert rel_l2(got, want) < 2e-4
    if t != ob.Q8_0:
        q, s, b = _q8k_bufs(gpu, m, k)
        gpu.silu_mul_q8k(gb, ub, m, k, q, s, b)
        gpu.gemv_q8k(wl, q, s, b, y2, m)
        assert np.array_equal(gpu.read(y2, np.float32, m * n).view(np.uint32), got.reshape(-1).view(np.uint32))
        for buf in (q, s, b):
            gpu.free(buf)
    for buf in (wl.buf, gb, ub, y1, y2):
        gpu.free(buf)
