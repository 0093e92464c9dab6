"""IQ4_XS (GGUF type 23) on the repack + GEMV part of the path: layout, outputs against the oracle's f32 dot, store
forms, fused producers, decode-time expert selection by name.  The CPU side of the format (decoder pinned by the
reference's digest, dot_iq4xs against an independent transcription) is in tests/test_oracle.py."""
import numpy as np
import pytest

import oracle
import ojas_engine_b200 as ob
from ojas_engine_b200 import ACCUM, BIAS, IQ4_XS

from conftest import rel_l2
from helpers import activations


def _raw(n, k, roll=0):
    base = oracle.synth_blocks(IQ4_XS, n * k // 256).reshape(n, -1)
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


@pytest.mark.gpu
def test_iq4xs_device_repack_equals_host_repack(gpu):
    n, k = 77, 1024
    raw = _raw(n, k)
    w = gpu.load_weight(raw, IQ4_XS, n, k)
    want = ob.repack_host(IQ4_XS, raw, n, k)
    assert np.array_equal(gpu.read(w.buf, np.uint8, want.size), want)
    gpu.free(w.buf)


@pytest.mark.gpu
@pytest.mark.parametrize("n,k,m", [(512, 4096, 1), (1000, 768, 1), (4096, 4096, 1), (14336, 4096, 1), (330, 1024, 2), (64, 2048, 3),
                                   (520, 512, 5), (256, 4096, 8), (17, 256, 1)])
def test_iq4xs_gemv_matches_the_oracle(gpu, n, k, m):
    raw = _raw(n, k, roll=3)
    x = activations(m, k, seed=7 + m)
    w = gpu.load_weight(raw, IQ4_XS, n, k)
    guard = 64
    xb = gpu.upload(x)
    y = gpu.upload(np.full(m * n + 2 * guard, 7.25, np.float32))
    yv = ob.Buf(y.ptr + guard * 4, m * n * 4)
    gpu.gemv(w, xb, yv, m)
    full = gpu.read(y, np.float32, m * n + 2 * guard)
    assert np.all(full[:guard] == 7.25) and np.all(full[-guard:] == 7.25)          # nothing written outside [M, N]
    got = full[guard:-guard].reshape(m, n)
    want = oracle.matmul_kq(raw, IQ4_XS, n, k, x)
    assert rel_l2(got, want) < 2e-3          # the bar of the path
    assert rel_l2(got, want) < 1e-5          # three int8 terms per activation: fp32-level
    for b in (w.buf, xb, y):
        gpu.free(b)


@pytest.mark.gpu
def test_iq4xs_store_forms_fused_producers_and_entry_names(gpu):
    n, k = 384, 1024
    raw = _raw(n, k, roll=1)
    x = activations(1, k, seed=9)
    w = gpu.load_weight(raw, IQ4_XS, n, k)
    want = oracle.matvec_kq(raw, IQ4_XS, n, k, x[0])
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
    assert rel_l2(gpu.read(y, np.float32, n), oracle.matvec_kq(raw, IQ4_XS, n, k, oracle.rmsnorm(x[0], nw, 1e-5))) < 1e-5
    names = ("gemv_nat_iq4xs", "gemv_nat_iq4xs_accum", "gemv_nat_iq4xs_bias", "gemv_nat_iq4xs_m", "moe_gu_iq4xs")
    assert all(gpu.has_kernel(name) for name in names)
    gpu.memset(y, 0)
    enc = gpu.begin()
    gpu.dispatch(enc, "gemv_nat_iq4xs", [(xb, 0), (w.buf, 0), (y, 0)], [k, n])
    gpu.submit(enc)
    assert rel_l2(gpu.read(y, np.float32, n), want) < 1e-5
    for buf in (w.buf, xb, y, bb, nb):
        gpu.free(buf)


@pytest.mark.gpu
def test_iq4xs_expert_gate_up_by_name(gpu):
    """moe_gu_iq4xs (x, wg, wu, act, idx)(K, N), grid.y = picks: act[j] = silu(gate_e x) * (up_e x) for the picked experts."""
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
    for buf in (wg.buf, wu.buf, xb, ib, act):
        gpu.free(buf)


@pytest.mark.gpu
def test_iq4xs_is_refused_where_it_is_not_built(gpu):
    n, k = 256, 512
    w = gpu.load_weight(_raw(n, k), IQ4_XS, n, k)
    x, y = gpu.alloc(16 * k), gpu.alloc(16 * n)
    with pytest.raises(ob.OjasB200Error):
        gpu.gemm(w, x, y, 16)
    q, s, b = gpu.alloc_bytes(k), gpu.alloc(k // 256), gpu.alloc_bytes(k // 32 * 4)
    with pytest.raises(ob.OjasB200Error, match="f32 activations"):
        gpu.gemv_q8k(w, q, s, b, y, 1)
    gpu.sync()
    for buf in (w.buf, x, y, q, s, b):
        gpu.free(buf)
