"""Q5_K (GGUF type 13): layout, integer block dots, GEMV outputs, entry names, the prefill GEMM (experts: tests/test_gpu_moe.py).  The
CPU side of the format (decoder, dot_q5k against an independent transcription) is in tests/test_oracle.py."""
import numpy as np
import pytest

import oracle
import ojas_engine_b200 as ob
from ojas_engine_b200 import ACCUM, BIAS, PLAIN, Q5_K

from conftest import rel_l2
from helpers import activations


def _raw(n, k, roll=0):
    base = oracle.synth_blocks(Q5_K, n * k // 256).reshape(n, -1)
    return np.ascontiguousarray(np.roll(base, roll, axis=0))


def test_q5k_tile_layout_keeps_every_bit():
    """Host repack: piece p of row r of tile (u, s) at byte (p * 8 + r) * 16; pieces 0-7 = qs, 8 = the first sixteen bytes
    of the block, 9-10 = qh; rows past N are zero blocks."""
    n, k = 21, 768
    raw = _raw(n, k)
    packed = ob.repack_host(Q5_K, raw, n, k)
    nsb, units = k // 256, (n + 7) // 8
    assert packed.size >= units * nsb * 1408
    tiles = packed[:units * nsb * 1408].reshape(units, nsb, 11, 8, 16)
    for r in range(units * 8):
        for s in range(nsb):
            got = tiles[r // 8, s, :, r % 8, :]
            if r >= n:
                assert not got.any()
                continue
            blk = raw[r, s * 176:(s + 1) * 176]
            assert np.array_equal(got[0:8].reshape(-1), blk[48:176])
            assert np.array_equal(got[8], blk[0:16])
            assert np.array_equal(got[9:11].reshape(-1), blk[16:48])


@pytest.mark.gpu
def test_q5k_device_repack_equals_host_repack(gpu):
    n, k = 77, 1024
    raw = _raw(n, k)
    w = gpu.load_weight(raw, Q5_K, n, k)
    want = ob.repack_host(Q5_K, raw, n, k)
    assert np.array_equal(gpu.read(w.buf, np.uint8, want.size), want)
    gpu.free(w.buf)


@pytest.mark.gpu
def test_q5k_integer_block_dots_bit_exact(gpu):
    n, k = 40, 1024
    raw = _raw(n, k)
    x = activations(1, k, seed=5)
    w = gpu.load_weight(raw, Q5_K, n, k)
    xb, out = gpu.upload(x), gpu.alloc_bytes(n * (k // 256) * 8 * 4)
    gpu.gemv_idots(w, xb, out)
    got = gpu.read(out, np.int32, n * (k // 256) * 8).reshape(n, -1)
    act = oracle.quant_q8k(x[0])
    for r in range(n):
        _, want = oracle.dot_q5k(raw[r], act, want_idots=True)
        assert np.array_equal(got[r], want)
    for b in (w.buf, xb, out):
        gpu.free(b)


@pytest.mark.gpu
@pytest.mark.parametrize("n,k,m", [(512, 4096, 1), (1000, 768, 1), (4096, 4096, 1), (330, 1024, 2), (64, 2048, 3), (520, 512, 5), (256, 4096, 8)])
def test_q5k_gemv_matches_the_oracle(gpu, n, k, m):
    raw = _raw(n, k, roll=3)
    x = activations(m, k, seed=7 + m)
    w = gpu.load_weight(raw, Q5_K, n, k)
    guard = 64
    xb = gpu.upload(x)
    y = gpu.upload(np.full(m * n + 2 * guard, 7.25, np.float32))
    yv = ob.Buf(y.ptr + guard * 4, m * n * 4)
    gpu.gemv(w, xb, yv, m)
    full = gpu.read(y, np.float32, m * n + 2 * guard)
    assert np.all(full[:guard] == 7.25) and np.all(full[-guard:] == 7.25)          # nothing written outside [M, N]
    got = full[guard:-guard].reshape(m, n)
    want = oracle.matmul_kq(raw, Q5_K, n, k, x)
    assert rel_l2(got, want) < 1e-5
    for b in (w.buf, xb, y):
        gpu.free(b)


@pytest.mark.gpu
def test_q5k_store_forms_prequantized_rows_and_entry_names(gpu):
    n, k = 384, 1024
    raw = _raw(n, k, roll=1)
    x = activations(1, k, seed=9)
    w = gpu.load_weight(raw, Q5_K, n, k)
    want = oracle.matvec_kq(raw, Q5_K, n, k, x[0])
    xb = gpu.upload(x)
    y0 = activations(1, n, seed=10)[0]
    bias = activations(1, n, seed=11)[0]
    y, bb = gpu.upload(y0), gpu.upload(bias)
    gpu.gemv(w, xb, y, 1, ACCUM)
    assert rel_l2(gpu.read(y, np.float32, n), want + y0) < 1e-5
    gpu.gemv(w, xb, y, 1, BIAS, bb)
    assert rel_l2(gpu.read(y, np.float32, n), want + bias) < 1e-5
    q, s, b = gpu.alloc_bytes(k), gpu.alloc(k // 256), gpu.alloc_bytes(k // 32 * 4)
    gpu.quant_q8k(xb, 1, k, q, s, b)
    gpu.gemv(w, xb, y, 1, PLAIN)
    plain = gpu.read(y, np.float32, n)
    gpu.gemv_q8k(w, q, s, b, y, 1)
    assert np.array_equal(gpu.read(y, np.float32, n), plain)                       # the same kernel minus the prologue
    assert all(gpu.has_kernel(name) for name in ("gemv_nat_q5k", "gemv_nat_q5k_accum", "gemv_nat_q5k_bias", "gemv_nat_q5k_m"))
    gpu.memset(y, 0)
    enc = gpu.begin()
    gpu.dispatch(enc, "gemv_nat_q5k", [(xb, 0), (w.buf, 0), (y, 0)], [k, n])
    gpu.submit(enc)
    assert np.array_equal(gpu.read(y, np.float32, n), plain)
    for buf in (w.buf, xb, y, bb, q, s, b):
        gpu.free(buf)


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,accum,ksplit", [(32, 128, 256, False, 0), (17, 1000, 768, False, 0), (300, 515, 2304, True, 0), (513, 384, 1280, False, 3),
                                                (512, 4096, 4096, False, 0), (2048, 1024, 4096, True, 0)])
def test_q5k_prefill_gemm_matches_the_oracle(gpu, m, n, k, accum, ksplit):
    """The tcgen05 GEMM with Q5_K weights (f16 weight tiles, f16(sx * q) activations) at the bar of the path, 2e-3; sampled
    token rows for the large shapes; a sentinel row behind y."""
    raw = _raw(n, k, roll=2)
    x = activations(m, k, seed=20 + m)
    rows = list(range(m)) if m <= 64 else sorted({0, 1, m // 3, m // 2, m - 2, m - 1})
    want = oracle.matmul_kq(raw, Q5_K, n, k, x[rows])
    w = gpu.load_weight(raw, Q5_K, n, k)
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
@pytest.mark.parametrize("t", [ob.Q4_K, Q5_K, ob.Q6_K, ob.Q8_0, ob.IQ4_XS, ob.IQ4_NL])
def test_token_table_gather_equals_the_cpu_decode(gpu, t):
    """x[m, :] = row ids[m] of a raw GGUF table, bit for bit the oracle's decoder (which the reference's own golden
    digests pin for Q4_K and Q6_K); repeated and out-of-order ids; by name for Q4_K."""
    rows, d = 37, 1024
    raw = oracle.synth_blocks(t, rows * d // oracle.block_shape(t)[1])
    table = oracle.dequant_f32(raw, t, rows * d).reshape(rows, d)
    ids = np.array([5, 0, 36, 5, 17, 1, 36], np.uint32)
    tb, ib, x = gpu.upload(raw), gpu.upload(ids), gpu.alloc(ids.size * d)
    gpu.embed_rows(tb, t, rows, ib, ids.size, d, x)
    got = gpu.read(x, np.float32, ids.size * d).reshape(ids.size, d)
    assert np.array_equal(got.view(np.uint32), table[ids].view(np.uint32))
    if t == ob.Q4_K:
        gpu.memset(x, 0)
        enc = gpu.begin()
        gpu.dispatch(enc, "q35_embed_q4k", [(tb, 0), (ib, 0), (x, 0)], [d, ids.size])
        gpu.submit(enc)
        assert np.array_equal(gpu.read(x, np.float32, ids.size * d).reshape(ids.size, d).view(np.uint32), table[ids].view(np.uint32))
    for b in (tb, ib, x):
        gpu.free(b)
