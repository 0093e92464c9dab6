"""The CPU oracle against the reference's own golden values (no GPU)."""
import json
import os
import sys

import numpy as np
import pytest

import oracle
from oracle import Q4_K, Q6_K, Q8_0

from conftest import rel_l2


GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
with open(os.path.join(GOLDEN, "reference_digests.json")) as _fh:
    REFERENCE_DIGESTS = json.load(_fh)["cases"]


# crates/ojas-formats/tests/quant_formats.rs:33-50: (type, value count, FNV-1a digest)
@pytest.mark.parametrize("case", REFERENCE_DIGESTS, ids=[c["name"] for c in REFERENCE_DIGESTS])
def test_synth_block_digests(case):
    t, n = case["type"], case["values"]
    raw = oracle.synth_blocks(t, 40)
    vals = oracle.dequant_f16(raw, t, n)
    assert vals.size == n
    assert oracle.digest_f16(vals) == int(case["digest"], 16)


def test_oracle_outputs_are_frozen():
    """tests/golden/oracle_vectors.npz (written by tests/golden/make_oracle_vectors.py): the oracle reproduces its own
    committed outputs bit for bit."""
    sys.path.insert(0, GOLDEN)
    import make_oracle_vectors
    want = np.load(os.path.join(GOLDEN, "oracle_vectors.npz"))
    got = make_oracle_vectors.compute()
    assert sorted(got) == sorted(want.files)
    for key in want.files:
        a, b = np.asarray(got[key]), want[key]
        assert a.dtype == b.dtype and a.shape == b.shape, key
        assert a.tobytes() == b.tobytes(), key


def test_q80_rows_fixture():
    # crates/ojas-formats/tests/rows.rs:13-17,57-66: block r has d = 0.25*(r+1), q[j] = j-16+r
    raw = bytearray()
    for r in range(3):
        raw += np.float16(0.25 * (r + 1)).tobytes()
        raw += bytes(((j - 16 + r) & 0xFF) for j in range(32))
    raw = np.frombuffer(bytes(raw), np.uint8)
    got = oracle.dequant_f32(raw, Q8_0, 96).reshape(3, 32)
    for r in range(3):
        want = 0.25 * (r + 1) * (np.arange(32) - 16 + r)
        assert np.array_equal(got[r], want.astype(np.float32))


def test_f16_conversion_matches_numpy():
    bits = np.arange(0, 65536, dtype=np.uint16)
    ours = np.array([oracle.lib().orc_f16_to_f32(int(b)) for b in bits[::7]], np.float32)
    ref = bits[::7].view(np.float16).astype(np.float32)
    ok = (ours == ref) | (np.isnan(ours) & np.isnan(ref))
    assert ok.all()
    rng = np.random.default_rng(3)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 300.0, 7e4)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 2.0 ** -24, 2.0 ** -25, 3 * 2.0 ** -26], np.float32)])
    ours = np.array([oracle.lib().orc_f32_to_f16(float(v)) for v in xs], np.uint16)
    with np.errstate(over="ignore"):
        ref = xs.astype(np.float16).view(np.uint16)
    assert np.array_equal(ours, ref)


def test_quant_q8k_rules():
    # crates/ojas-cpu/src/cpu_math.rs:545-563: scale = amax/127 (1 when all zero), half away from zero
    x = np.zeros(512, np.float32)
    x[:256] = np.linspace(-3, 3, 256, dtype=np.float32)
    scales, q, bsums = oracle.quant_q8k(x)
    assert scales[1] == 1.0 and not q[256:].any() and not bsums[8:].any()
    assert scales[0] == np.float32(3.0) / np.float32(127.0)
    assert q[0] == -127 and q[255] == 127
    assert np.array_equal(bsums[:8], q[:256].astype(np.int32).reshape(8, 32).sum(1))
    # ties: amax = 127 -> scale 1, inv 1: 0.5 -> 1, -0.5 -> -1, 2.5 -> 3 (half away, not half even)
    y = np.zeros(256, np.float32)
    y[0], y[1], y[2], y[3], y[4] = 127.0, 0.5, -0.5, 2.5, -2.5
    _, q2, _ = oracle.quant_q8k(y)
    assert list(q2[:5]) == [127, 1, -1, 3, -3]


@pytest.mark.parametrize("t", [Q4_K, Q6_K])
def test_kquant_dot_identity(t):
    """dot(row, q8k(x)) equals sum dequant(row)[i] * (sx*q[i]) up to f32 rounding, and the dumped
    integer sub-block dots equal a direct integer recomputation."""
    k, n = 1024, 6
    bb, bw = oracle.block_shape(t)
    raw = oracle.synth_blocks(t, n * k // bw).reshape(n, -1)
    x = np.random.default_rng(5).standard_normal(k).astype(np.float32)
    act = oracle.quant_q8k(x)
    scales, q, _ = act
    xhat = (np.repeat(scales, 256) * q.astype(np.float32)).astype(np.float64)
    for r in range(n):
        w = oracle.dequant_f32(raw[r], t, k).astype(np.float64)
        want = float(w @ xhat)
        if t == Q4_K:
            got, idots = oracle.dot_q4k(raw[r], act, want_idots=True)
            blk = raw[r].reshape(-1, 144)[:, 16:].reshape(-1, 4, 32)
            wq = np.stack([blk & 0xF, blk >> 4], axis=2).reshape(-1, 8, 32).astype(np.int64)
            direct = (wq * q.reshape(-1, 8, 32).astype(np.int64)).sum(-1).reshape(-1)
            assert np.array_equal(idots, direct.astype(np.int32))
        else:
            got, idots = oracle.dot_q6k(raw[r], act, want_idots=True)
            # the 6-bit values 0..63 by the GGUF rule (crates/ojas-formats/src/gguf.rs:1086-1108), then per-16 dots
            blk = raw[r].reshape(-1, 210)
            ql, qh = blk[:, :128].reshape(-1, 2, 64).astype(np.int64), blk[:, 128:192].reshape(-1, 2, 32).astype(np.int64)
            w6 = np.empty((blk.shape[0], 2, 4, 32), np.int64)
            w6[:, :, 0] = (ql[:, :, :32] & 0xF) | ((qh & 3) << 4)
            w6[:, :, 1] = (ql[:, :, 32:] & 0xF) | (((qh >> 2) & 3) << 4)
            w6[:, :, 2] = (ql[:, :, :32] >> 4) | (((qh >> 4) & 3) << 4)
            w6[:, :, 3] = (ql[:, :, 32:] >> 4) | (((qh >> 6) & 3) << 4)
            direct = (w6.reshape(-1, 16, 16) * q.reshape(-1, 16, 16).astype(np.int64)).sum(-1).reshape(-1)
            assert np.array_equal(idots, direct.astype(np.int32))
        assert abs(got - want) <= 2e-5 * max(1.0, np.abs(w).dot(np.abs(xhat)))


# ---- the C oracle against an independent transcription of the Rust source (tests/second_entry.py)
def _second_entry_inputs():
    rng = np.random.default_rng(17)
    xs = [rng.standard_normal(768).astype(np.float32), (rng.standard_normal(512) * 1e-3).astype(np.float32), oracle.tvec(512, 3),
          np.zeros(256, np.float32)]
    ties = np.zeros(256, np.float32)
    ties[0] = 127.0
    ties[1:253] = np.arange(-126, 126, dtype=np.float32) + np.float32(0.5)     # exact .5 after scaling by 1
    xs.append(ties)
    return xs


def test_quant_q8k_second_entry():
    import second_entry
    for x in _second_entry_inputs():
        a, b = oracle.quant_q8k(x), second_entry.quant_q8k(x)
        assert np.array_equal(a[0].view(np.uint32), b[0].view(np.uint32))
        assert np.array_equal(a[1], b[1]) and np.array_equal(a[2], b[2])


@pytest.mark.parametrize("t", [Q4_K, Q6_K])
@pytest.mark.parametrize("source", ["synth", "gauss"])
def test_kquant_dots_second_entry(t, source):
    import second_entry
    import ojas_engine_b200 as ob
    k, n = 768, 5
    if source == "synth":
        raw = oracle.synth_blocks(t, n * k // 256).reshape(n, -1)
    else:
        w = (np.random.default_rng(8).standard_normal((n, k)) * 0.02).astype(np.float32)
        raw = ob.encode(t, w).reshape(n, -1)
    x = np.random.default_rng(6).standard_normal(k).astype(np.float32)
    act = oracle.quant_q8k(x)
    for r in range(n):
        if t == Q4_K:
            got, idots = oracle.dot_q4k(raw[r], act, want_idots=True)
            want, widots = second_entry.dot_q4k(raw[r], act)
        else:
            got, idots = oracle.dot_q6k(raw[r], act, want_idots=True)
            want, widots = second_entry.dot_q6k(raw[r], act)
        assert np.array_equal(idots, widots)
        assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32), (got, want)


def test_q80_dot_second_entry():
    import second_entry
    k, n = 512, 6
    raw = oracle.synth_blocks(Q8_0, n * k // 32).reshape(n, -1)
    x = np.random.default_rng(4).standard_normal(k).astype(np.float32)
    for r in range(n):
        assert np.float32(oracle.dot_q80(raw[r], x)).view(np.uint32) == second_entry.dot_q80(raw[r], x).view(np.uint32)


def test_q80_dot_and_matvec():
    k, n = 512, 40
    raw = oracle.synth_blocks(Q8_0, n * k // 32).reshape(n, -1)
    x = oracle.tvec(k, 9)
    w = oracle.dequant_f32(raw.reshape(-1), Q8_0, n * k).reshape(n, k).astype(np.float64)
    y1 = oracle.matvec_kq(raw, Q8_0, n, k, x, threads=1)
    y8 = oracle.matvec_kq(raw, Q8_0, n, k, x, threads=8)
    assert np.array_equal(y1, y8)  # row results do not depend on the thread count
    assert rel_l2(y1, w @ x.astype(np.float64)) < 1e-6
    assert y1[3] == np.float32(oracle.dot_q80(raw[3], x))


def test_matvec_threads_and_batch():
    k, n, m = 768, 37, 3
    raw = oracle.synth_blocks(Q4_K, n * k // 256)
    x = np.random.default_rng(1).standard_normal((m, k)).astype(np.float32)
    ys = oracle.matmul_kq(raw, Q4_K, n, k, x, threads=5)
    for t in range(m):
        assert np.array_equal(ys[t], oracle.matvec_kq(raw, Q4_K, n, k, x[t], threads=1))


def test_moe_topk_semantics():
    # crates/ojas-cuda/src/kernels/moe.rs:45-70: ties go to the lowest index; weights renormalised
    lg = np.array([[0.5, 2.0, 2.0, -1.0]], np.float32)
    idx, wgt = oracle.moe_topk(lg, 2)
    assert list(idx[0]) == [1, 2]
    assert np.allclose(wgt[0], [0.5, 0.5])
    lg = np.random.default_rng(2).standard_normal((16, 8)).astype(np.float32)
    idx, wgt = oracle.moe_topk(lg, 2)
    order = np.argsort(-lg, axis=1, kind="stable")[:, :2]
    assert np.array_equal(idx, order.astype(np.uint32))
    e = np.exp(np.take_along_axis(lg, order, 1).astype(np.float64))
    assert np.allclose(wgt, e / e.sum(1, keepdims=True), atol=1e-6)
    assert np.allclose(wgt.sum(1), 1.0, atol=1e-6)


def test_tvec_generator():
    # crates/ojas-cuda/tests/conformance.rs:223-231
    v = oracle.tvec(4, 7)
    s = (7 * 2654435761 + 1) & 0xFFFFFFFF
    want = []
    for _ in range(4):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        want.append(np.float32(s >> 9) / np.float32(1 << 23) - np.float32(1.0))
    assert np.array_equal(v, np.array(want, np.float32))


def test_matvec_second_entry():
    import second_entry
    rng = np.random.default_rng(11)
    for t, n, k in ((Q4_K, 9, 512), (Q6_K, 7, 768), (Q8_0, 5, 256)):
        raw = oracle.synth_blocks(t, n * k // (32 if t == Q8_0 else 256))
        x = rng.standard_normal(k).astype(np.float32)
        a, b = oracle.matvec_kq(raw, t, n, k, x, threads=1), second_entry.matvec_kq(raw, t, n, k, x)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_producers_second_entry():
    """RMSNorm and SwiGLU of the oracle against the transcription of the Rust source: RMSNorm bit for bit (same order
    of additions), SwiGLU to the last bit of the exponential (libm against numpy: at most one unit in the last place)."""
    import second_entry
    rng = np.random.default_rng(12)
    x = (rng.standard_normal(768) * 3).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(768)).astype(np.float32)
    a, b = oracle.rmsnorm(x, w, 1e-5), second_entry.rmsnorm(x, w, 1e-5)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    g, u = (rng.standard_normal(512) * 2).astype(np.float32), rng.standard_normal(512).astype(np.float32)
    a, b = oracle.silu_mul(g, u), second_entry.silu_mul(g, u)
    assert np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64)).max() <= 2


def test_router_and_expert_ffn_second_entry():
    import second_entry
    rng = np.random.default_rng(13)
    e, ksel, d, ffn, m = 4, 2, 256, 512, 3
    lg = rng.standard_normal((m, e)).astype(np.float32)
    lg[1, 2] = lg[1, 0]                                     # a tie: the lower index wins
    idx, wgt = oracle.moe_topk(lg, ksel)
    for t in range(m):
        i2, w2 = second_entry.moe_topk(lg[t], ksel)
        assert np.array_equal(idx[t], i2) and np.allclose(wgt[t], w2, rtol=2e-6, atol=0)
    wg = oracle.synth_blocks(Q4_K, e * ffn * d // 256)
    wu = np.roll(oracle.synth_blocks(Q4_K, e * ffn * d // 256).reshape(-1, 144), 5, axis=0).reshape(-1).copy()
    wd = oracle.synth_blocks(Q6_K, e * d * ffn // 256)
    h = rng.standard_normal((m, d)).astype(np.float32)
    a = oracle.moe_ffn(wg, wu, wd, Q4_K, Q6_K, h, idx, wgt, d, ffn, threads=1)
    b = second_entry.moe_ffn(wg, wu, wd, Q4_K, Q6_K, h, idx, wgt, d, ffn)
    assert rel_l2(a, b) < 1e-6                              # (the exponential's last bit may flip a Q8_K rounding)


def test_q5k_second_entry_and_identity():
    """Q5_K (type 13) in the oracle: the dot against the transcription of the Rust source bit for bit (integer
    sub-block dots included), matvec_kq likewise, and the identity dot(row, q8k(x)) == sum dequant(row)[i] * (sx * q[i])."""
    import second_entry
    from oracle import Q5_K
    k, n = 768, 6
    raw = oracle.synth_blocks(Q5_K, n * k // 256).reshape(n, -1)
    x = np.random.default_rng(21).standard_normal(k).astype(np.float32)
    act = oracle.quant_q8k(x)
    w = oracle.dequant_f32(raw.reshape(-1), Q5_K, n * k).reshape(n, k).astype(np.float64)
    xd = (np.repeat(act[0], 256).astype(np.float64) * act[1].astype(np.float64))
    for r in range(n):
        got, idots = oracle.dot_q5k(raw[r], act, want_idots=True)
        want, widots = second_entry.dot_q5k(raw[r], act)
        assert np.array_equal(idots, widots)
        assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32)
        assert abs(got - float(w[r] @ xd)) <= 1e-5 * float(np.abs(w[r]) @ np.abs(xd))
    a, b = oracle.matvec_kq(raw, Q5_K, n, k, x, threads=1), second_entry.matvec_kq(raw, Q5_K, n, k, x)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_iq4xs_second_entry_and_identity():
    """IQ4_XS (type 23) in the oracle: the f32 dot against the transcription of the Rust source bit for bit, matvec_kq
    likewise, and the identity dot(row, x) == sum dequant(row)[i] * x[i] (the decode is pinned by the reference's digest)."""
    import second_entry
    from oracle import IQ4_XS
    k, n = 768, 6
    raw = oracle.synth_blocks(IQ4_XS, n * k // 256).reshape(n, -1)
    x = np.random.default_rng(23).standard_normal(k).astype(np.float32)
    w = oracle.dequant_f32(raw.reshape(-1), IQ4_XS, n * k).reshape(n, k).astype(np.float64)
    for r in range(n):
        got, want = oracle.dot_iq4xs(raw[r], x), second_entry.dot_iq4xs(raw[r], x)
        assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32)
        assert abs(got - float(w[r] @ x.astype(np.float64))) <= 1e-5 * float(np.abs(w[r]) @ np.abs(x).astype(np.float64))
    a, b = oracle.matvec_kq(raw, IQ4_XS, n, k, x, threads=1), second_entry.matvec_kq(raw, IQ4_XS, n, k, x)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_iq4nl_known_answers_second_entry_and_identity():
    """IQ4_NL (type 20).  The reference's own unit test (crates/ojas-cpu/src/cpu_math.rs:1203-1223): d = 1.0, qs[0] = 0x93;
    a one-hot x at 0 selects the low nibble (codebook entry 3), at 16 the high nibble (entry 9).  Then the dot against the
    transcription of the Rust source bit for bit, matvec_kq likewise, and dot(row, x) == sum dequant(row)[i] * x[i]."""
    import second_entry
    from oracle import IQ4_NL
    row = np.zeros(18, np.uint8)
    row[0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    row[2] = 0x93
    x = np.zeros(32, np.float32)
    x[0] = 1.0
    assert oracle.dot_iq4nl(row, x) == float(second_entry.KVALUES_IQ4NL[3]) == -65.0
    x[:] = 0
    x[16] = 1.0
    assert oracle.dot_iq4nl(row, x) == float(second_entry.KVALUES_IQ4NL[9]) == 13.0
    k, n = 768, 6
    raw = oracle.synth_blocks(IQ4_NL, n * k // 32).reshape(n, -1)
    x = np.random.default_rng(29).standard_normal(k).astype(np.float32)
    w = oracle.dequant_f32(raw.reshape(-1), IQ4_NL, n * k).reshape(n, k).astype(np.float64)
    for r in range(n):
        got, want = oracle.dot_iq4nl(raw[r], x), second_entry.dot_iq4nl(raw[r], x)
        assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32)
        assert abs(got - float(w[r] @ x.astype(np.float64))) <= 1e-5 * float(np.abs(w[r]) @ np.abs(x).astype(np.float64))
    a, b = oracle.matvec_kq(raw, IQ4_NL, n, k, x, threads=1), second_entry.matvec_kq(raw, IQ4_NL, n, k, x)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
