"""IQ4_XS (GGUF type 23) and IQ4_NL (type 20) on the repack + GEMV part of the path: layout, outputs against the
oracle's f32 dots, store forms, fused producers, decode-time expert selection by name.  The CPU side of the formats
(decoders pinned by the reference's digests, dot_iq4xs / dot_iq4nl against an independent transcription and the
reference's known answers) is in tests/test_oracle.py."""
import numpy as np
import pytest

import oracle
import ojas_engine_b200 as ob
from ojas_engine_b200 import ACCUM, BIAS, IQ4_NL, IQ4_XS

from conftest import rel_l2
from helpers import activations


BOTH = pytest.mark.parametrize("t", [IQ4_XS, IQ4_NL], ids=["iq4xs", "iq4nl"])
TAG = {IQ4_XS: "iq4xs", IQ4_NL: "iq4nl"}


def _raw(n, k, roll=0, t=IQ4_XS):
    base = oracle.synth_blocks(t, n * k // oracle.block_shape(t)[1]).reshape(n, -1)
    return np.ascontiguousarray(np.roll(base, roll, axis=0))


def test_iq4xs_tile_layout_keeps_every_bit():
    """Host repack: pieces 0-7 of row r of tile (u, s) at byte (p * 8 + r) * 16 = the 128 index bytes; the block's first
    eight bytes (d, scales_h, scales_l) at byte 1024 + 8 r; rows past N are zero blocks."""
    n, k = 21, 768
    raw = _raw(n, k)
    packed = ob.repack_host(IQ4_XS, raw, n, k)
    nsb, units = k // 256, (n + 7) // 8
    assert packed.size >= units * nsb * 1088
    tiles = packed[:units * nsb * 1088].reshape(units, nsb, 1088)
    for r in range(units * 8):
        for s in range(nsb):
            t = tiles[r // 8, s]
            qs = t[:1024].reshape(8, 8, 16)[:, r % 8, :].reshape(-1)
            head = t[1024 + 8 * (r % 8):1024 + 8 * (r % 8) + 8]
            if r >= n:
                assert not qs.any() and not head.any()
                continue
            blk = raw[r, s * 136:(s + 1) * 136]
            assert np.array_equal(qs, blk[8:136]) and np.array_equal(head, blk[0:8])


def test_iq4nl_tile_layout_keeps_every_bit():
    """Host repack: piece b of row r = the sixteen index bytes of the row's block b of the super-block; piece 8 = the
    eight f16 block scales."""
    n, k = 13, 512
    raw = _raw(n, k, t=IQ4_NL)
    packed = ob.repack_host(IQ4_NL, raw, n, k)
    nsb, units = k // 256, (n + 7) // 8
    tiles = packed[:units * nsb * 1152].reshape(units, nsb, 9, 8, 16)
    for r in range(units * 8):
        for s in range(nsb):
            got = tiles[r // 8, s, :, r % 8, :]
            if r >= n:
                assert not got.any()
                continue
            blocks = raw[r, s * 144:(s + 1) * 144].reshape(8, 18)
            assert np.array_equal(got[0:8], blocks[:, 2:]) and np.array_equal(got[8], blocks[:, :2].reshape(-1))


@pytest.mark.gpu
@BOTH
def test_iq4_device_repack_equals_host_repack(gpu, t):
    n, k = 77, 1024
    raw = _raw(n, k, t=t)
    w = gpu.load_weight(raw, t, n, k)
    want = ob.repack_host(t, raw, n, k)
    assert np.array_equal(gpu.read(w.buf, np.uint8, want.size), want)
    gpu.free(w.buf)


@pytest.mark.gpu
@BOTH
@pytest.mark.parametrize("n,k,m", [(512, 4096, 1), (1000, 768, 1), (4096, 4096, 1), (14336, 4096, 1), (330, 1024, 2), (64, 2048, 3),
                                   (520, 512, 5), (256, 4096, 8), (17, 256, 1)])
def test_iq4_gemv_matches_the_oracle(gpu, t, n, k, m):
    raw = _raw(n, k, roll=3, t=t)
    x = activations(m, k, seed=7 + m)
    w = gpu.load_weight(raw, t, n, k)
    guard = 64
    xb = gpu.upload(x)
    y = gpu.upload(np.full(m * n + 2 * guard, 7.25, np.float32))
    yv = ob.Buf(y.ptr + guard * 4, m * n * 4)
    gpu.gemv(w, xb, yv, m)
    full = gpu.read(y, np.float32, m * n + 2 * guard)
    assert np.all(full[:guard] == 7.25) and np.all(full[-guard:] == 7.25)          # nothing written outside [M, N]
    got = full[guard:-guard].reshape(m, n)
    want = oracle.matmul_kq(raw, t, n, k, x)
    assert rel_l2(got, want) < 2e-3          # the bar of the path
    assert rel_l2(got, want) < 1e-5          # three int8 terms per activation: fp32-level
    for b in (w.buf, xb, y):
        gpu.free(b)


@pytest.mark.gpu
@BOTH
def test_iq4_store_forms_fused_producers_and_entry_names(gpu, t):
    n, k = 384, 1024
    raw = _raw(n, k, roll=1, t=t)
    x = activations(1, k, seed=9)
    w = gpu.load_weight(raw, t, n, k)
    want = oracle.matvec_kq(raw, t, n, k, x[0])
    xb = gpu.upload(x)
    y0 = activations(1, n, seed=10)[0]
    bias = activations(1, n, seed=11)[0]
    y, bb = gpu.upload(y0), gpu.upload(bias)
    gpu.gemv(w, xb, y, 1, ACCUM)
    assert rel_l2(gpu.read(y, np.float32, n), want + y0) < 1e-5
    gpu.gemv(w, xb, y, 1, BIAS, bb)
    assert rel_l2(gpu.read(y, np.float32, n), want + bias) < 1e-5
    # RMSNorm in the prologue: the oracle's rmsnorm, then its dot
    nw = activations(1, k, seed=12)[0]
    nb = gpu.upload(nw)
    gpu.gemv_rmsnorm(w, xb, nb, 1e-5, y, 1)
    assert rel_l2(gpu.read(y, np.float32, n), oracle.matvec_kq(raw, t, n, k, oracle.rmsnorm(x[0], nw, 1e-5))) < 1e-5
    tag = TAG[t]
    names = (f"gemv_nat_{tag}", f"gemv_nat_{tag}_accum", f"gemv_nat_{tag}_bias", f"gemv_nat_{tag}_m", f"moe_gu_{tag}", f"moe_down_{tag}")
    assert all(gpu.has_kernel(name) for name in names)
    gpu.memset(y, 0)
    enc = gpu.begin()
    gpu.dispatch(enc, f"gemv_nat_{tag}", [(xb, 0), (w.buf, 0), (y, 0)], [k, n])
    gpu.submit(enc)
    assert rel_l2(gpu.read(y, np.float32, n), want) < 1e-5
    for buf in (w.buf, xb, y, bb, nb):
        gpu.free(buf)


@pytest.mark.gpu
def test_iq4_experts_by_name(gpu):
    """The two IQ expert entries of the engine: moe_gu_iq4xs (x, wg, wu, act, idx)(K, N), grid.y = picks:
    act[j] = silu(gate_e x) * (up_e x) for the picked experts; then moe_down_iq4nl (act, wd, x, idx, wgt)(K, N, KSEL):
    x += sum_j wgt[j] * down_e act[j]."""
    e, n, k = 4, 256, 512
    raw_g, raw_u = _raw(e * n, k, roll=2), _raw(e * n, k, roll=5)
    x = activations(1, k, seed=13)
    wg, wu = gpu.load_weight(raw_g, IQ4_XS, e * n, k), gpu.load_weight(raw_u, IQ4_XS, e * n, k)
    picks = np.array([2, 0], np.uint32)
    xb, ib, act = gpu.upload(x), gpu.upload(picks), gpu.alloc(picks.size * n)
    enc = gpu.begin()
    gpu.dispatch(enc, "moe_gu_iq4xs", [(xb, 0), (wg.buf, 0), (wu.buf, 0), (act, 0), (ib, 0)], [k, n], grid=(1, picks.size, 1))
    gpu.submit(enc)
    got = gpu.read(act, np.float32, picks.size * n).reshape(picks.size, n)
    for j, ex in enumerate(picks):
        g = oracle.matvec_kq(raw_g[ex * n:(ex + 1) * n], IQ4_XS, n, k, x[0])
        u = oracle.matvec_kq(raw_u[ex * n:(ex + 1) * n], IQ4_XS, n, k, x[0])
        assert rel_l2(got[j], oracle.silu_mul(g, u)) < 1e-5
    # down: experts [e, k, n] stored IQ4_NL, rows of width n
    raw_d = _raw(e * k, n, roll=7, t=IQ4_NL)
    wd = gpu.load_weight(raw_d, IQ4_NL, e * k, n)
    wgt = np.array([0.75, 0.25], np.float32)
    h0 = activations(1, k, seed=14)[0]
    hb, wb = gpu.upload(h0), gpu.upload(wgt)
    enc = gpu.begin()
    gpu.dispatch(enc, "moe_down_iq4nl", [(act, 0), (wd.buf, 0), (hb, 0), (ib, 0), (wb, 0)], [n, k, picks.size])
    gpu.submit(enc)
    want = h0.copy()
    for j, ex in enumerate(picks):
        want = want + wgt[j] * oracle.matvec_kq(raw_d[ex * k:(ex + 1) * k], IQ4_NL, k, n, got[j])
    assert rel_l2(gpu.read(hb, np.float32, k), want) < 1e-5
    for buf in (wg.buf, wu.buf, wd.buf, xb, ib, act, hb, wb):
        gpu.free(buf)


@pytest.mark.gpu
@BOTH
@pytest.mark.parametrize("m,n,k,accum,ksplit", [(32, 128, 256, False, 0), (17, 1000, 768, False, 0), (300, 515, 2304, True, 0), (513, 384, 1280, False, 3),
                                                (512, 4096, 4096, False, 0)])
def test_iq4_prefill_gemm_matches_the_oracle(gpu, t, m, n, k, accum, ksplit):
    """The tcgen05 GEMM with IQ4 weights (codebook values looked up and widened to f16, f16(x) activations as for Q8_0) at
    the bar of the path, 2e-3; sampled token rows for the large shape; a sentinel row behind y."""
    raw = _raw(n, k, roll=2, t=t)
    x = activations(m, k, seed=20 + m)
    rows = list(range(m)) if m <= 64 else sorted({0, 1, m // 3, m // 2, m - 2, m - 1})
    want = oracle.matmul_kq(raw, t, n, k, x[rows])
    w = gpu.load_weight(raw, t, n, k)
    y0 = activations(m, n, seed=21) if accum else np.zeros((m, n), np.float32)
    xb, yb = gpu.upload(x), gpu.upload(np.concatenate([y0, np.full((1, n), -77.0, np.float32)]))
    gpu.set_option("gemm_ksplit", ksplit)
    try:
        gpu.gemm(w, xb, yb, m, accum)
        got = gpu.read(yb, np.float32, (m + 1) * n).reshape(m + 1, n)
    finally:
        gpu.set_option("gemm_ksplit", 0)
    assert np.all(got[m] == -77.0), "wrote past row M"
    assert rel_l2(got[rows], want + y0[rows] if accum else want) < 2e-3
    for b in (w.buf, xb, yb):
        gpu.free(b)


@pytest.mark.gpu
@BOTH
def test_iq4_is_refused_where_it_is_not_built(gpu, t):
    n, k = 256, 512
    w = gpu.load_weight(_raw(n, k, t=t), t, n, k)
    x, y = gpu.alloc(16 * k), gpu.alloc(16 * n)
    q, s, b = gpu.alloc_bytes(k), gpu.alloc(k // 256), gpu.alloc_bytes(k // 32 * 4)
    with pytest.raises(ob.OjasB200Error, match="f32 activations"):
        gpu.gemv_q8k(w, q, s, b, y, 1)
    gpu.sync()
    for buf in (w.buf, x, y, q, s, b):
        gpu.free(buf)
