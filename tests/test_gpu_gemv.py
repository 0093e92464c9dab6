"""Parity of the CUDA GEMV path with the CPU oracle, through the C ABI (needs a B200)."""
import numpy as np
import pytest

import oracle
import ojas_engine_b200 as ob
from ojas_engine_b200 import ACCUM, BIAS, PLAIN, Q4_K, Q6_K, Q8_0

from conftest import rel_l2
from helpers import TYPES, activations, gauss_weights, synth_weights

pytestmark = pytest.mark.gpu

TOL = 2e-3  # relative L2 against the reference CPU path, the bar the path is held to
GUARD, SENTINEL = 256, np.float32(-1234.5)   # floats on either side of every output, and the value they must keep


def _weights(tag, n, k, source, seed=0):
    t = TYPES[tag]
    return synth_weights(t, n, k) if source == "synth" else gauss_weights(t, n, k, seed)


# ---------------------------------------------------------------- quant_q8k: bit exact
def _quant_case(gpu, x):
    m, k = x.shape
    xb = gpu.upload(x)
    q, s, b = gpu.alloc_bytes(m * k), gpu.alloc(m * k // 256), gpu.alloc_bytes(m * k // 32 * 4)
    gpu.quant_q8k(xb, m, k, q, s, b)
    got_q = gpu.read(q, np.int8, m * k).reshape(m, k)
    got_s = gpu.read(s, np.float32, m * k // 256).reshape(m, -1)
    got_b = gpu.read(b, np.int32, m * k // 32).reshape(m, -1)
    for buf in (xb, q, s, b):
        gpu.free(buf)
    for r in range(m):
        ws, wq, wb = oracle.quant_q8k(x[r])
        assert np.array_equal(got_s[r].view(np.uint32), ws.view(np.uint32)), "scales differ"
        assert np.array_equal(got_q[r], wq), f"q differs in row {r}: {np.flatnonzero(got_q[r] != wq)[:8]}"
        assert np.array_equal(got_b[r], wb), "bsums differ"


def test_quant_q8k_bit_exact_random(gpu):
    _quant_case(gpu, activations(64, 4096, seed=11))
    _quant_case(gpu, activations(3, 14336, seed=12) * np.float32(37.5))
    _quant_case(gpu, (oracle.tvec(5 * 768, 3).reshape(5, 768)))


def test_quant_q8k_edges(gpu):
    x = np.zeros((4, 512), np.float32)
    x[0, :5] = [127.0, 0.5, -0.5, 2.5, -2.5]            # scale exactly 1: ties must round away from zero
    x[1, 256:] = np.linspace(-1e-30, 1e-30, 256)         # tiny values
    x[2, :] = np.float32(-3.25)                          # constant block: every q = -127
    x[3, ::2] = 1e30
    # values that land exactly on k + 0.5 after scaling by inv = 1/(amax/127)
    k = np.arange(-126, 126, dtype=np.float32) + np.float32(0.5)
    x[3, 256:256 + k.size] = 0
    y = np.zeros((1, 256), np.float32)
    y[0, 0] = 127.0
    y[0, 1:1 + k.size] = k
    _quant_case(gpu, x)
    _quant_case(gpu, y)


# ---------------------------------------------------------------- integer block dots: bit exact
@pytest.mark.parametrize("tag,per", [("q4k", 32), ("q6k", 16)])
@pytest.mark.parametrize("source", ["synth", "gauss"])
def test_integer_block_dots_bit_exact(gpu, tag, per, source):
    t = TYPES[tag]
    n, k = 300, 2304                                    # ragged: 9 super-blocks, rows not a multiple of the grid
    raw = _weights(tag, n, k, source)
    x = activations(1, k, seed=21)
    w = gpu.load_weight(raw, t, n, k)
    xb = gpu.upload(x)
    out = gpu.alloc_bytes(n * (k // per) * 4)
    gpu.gemv_idots(w, xb, out)
    got = gpu.read(out, np.int32, n * (k // per)).reshape(n, -1)
    act = oracle.quant_q8k(x[0])
    rows = raw.reshape(n, -1)
    for r in range(n):
        _, want = (oracle.dot_q4k if t == Q4_K else oracle.dot_q6k)(rows[r], act, want_idots=True)
        assert np.array_equal(got[r], want), f"row {r}"
    for b in (w.buf, xb, out):
        gpu.free(b)


# ---------------------------------------------------------------- GEMV outputs
def _gemv_case(gpu, tag, n, k, m, source="gauss", form=PLAIN, seed=0):
    t = TYPES[tag]
    raw = _weights(tag, n, k, source, seed)
    x = activations(m, k, seed=seed + 100)
    want = oracle.matmul_kq(raw, t, n, k, x)
    w = gpu.load_weight(raw, t, n, k)
    xb = gpu.upload(x)
    y0 = activations(m, n, seed=seed + 200)
    # y sits between two guard regions of a larger buffer: a store before row 0 or past row m - 1 shows up there
    ybig = gpu.upload(np.concatenate([np.full(GUARD, SENTINEL, np.float32), y0.reshape(-1), np.full(GUARD, SENTINEL, np.float32)]))
    yb = ob.Buf(ybig.ptr + GUARD * 4, m * n * 4)
    bias = None
    if form == BIAS:
        bvec = activations(1, n, seed=seed + 300)[0]
        bias = gpu.upload(bvec)
        want = want + bvec[None, :]
    elif form == ACCUM:
        want = want + y0
    gpu.gemv(w, xb, yb, m, form, bias)
    whole = gpu.read(ybig, np.float32, m * n + 2 * GUARD)
    got = whole[GUARD:GUARD + m * n].reshape(m, n)
    assert np.all(whole[:GUARD] == SENTINEL) and np.all(whole[GUARD + m * n:] == SENTINEL), f"{tag} n={n} k={k} m={m}: store outside y"
    for b in (w.buf, xb, ybig) + ((bias,) if bias else ()):
        gpu.free(b)
    err = rel_l2(got, want)
    assert err < TOL, f"{tag} n={n} k={k} m={m} form={form}: rel L2 {err:.3e}"
    return err


def test_committed_golden_vectors(gpu):
    """tests/golden/oracle_vectors.npz: the committed activation row against the synthetic blocks of every format of the
    path; the GEMV reproduces the committed outputs (fp32 summation order is all that differs), and quant_q8k and the
    router reproduce theirs bit for bit."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_vectors.npz"))
    x = g["x"].reshape(1, -1)
    k, n = x.shape[1], 12
    xb = gpu.upload(x)
    for tag, t in [("q80", Q8_0), ("q4k", Q4_K), ("q5k", ob.Q5_K), ("q6k", Q6_K), ("iq4nl", ob.IQ4_NL), ("iq4xs", ob.IQ4_XS)]:
        raw = oracle.synth_blocks(t, n * k // oracle.block_shape(t)[1])
        w, y = gpu.load_weight(raw, t, n, k), gpu.alloc(n)
        gpu.gemv(w, xb, y, 1)
        assert rel_l2(gpu.read(y, np.float32, n), g[f"y_{tag}"]) < 1e-5, tag
        gpu.free(w.buf)
        gpu.free(y)
    q, s, b = gpu.alloc_bytes(k), gpu.alloc(k // 256), gpu.alloc_bytes(k // 32 * 4)
    gpu.quant_q8k(xb, 1, k, q, s, b)
    assert np.array_equal(gpu.read(q, np.int8, k), g["q8k_q"]) and np.array_equal(gpu.read(b, np.int32, k // 32), g["q8k_bsums"])
    assert np.array_equal(gpu.read(s, np.float32, k // 256).view(np.uint32), g["q8k_scales"].view(np.uint32))
    lg = g["topk_logits"]
    lb, ib, wb = gpu.upload(lg), gpu.alloc_bytes(lg.shape[0] * 2 * 4), gpu.alloc(lg.shape[0] * 2)
    gpu.moe_topk(lb, ib, wb, lg.shape[0], lg.shape[1], 2)
    assert np.array_equal(gpu.read(ib, np.uint32, lg.shape[0] * 2).reshape(-1, 2), g["topk_idx"])
    assert np.allclose(gpu.read(wb, np.float32, lg.shape[0] * 2).reshape(-1, 2), g["topk_wgt"], rtol=1e-5, atol=1e-7)
    for buf in (xb, q, s, b, lb, ib, wb):
        gpu.free(buf)


def test_config1_q4k_gemv(gpu):
    """Q4_K x f32, N = K = 4096, batch 1, seed 0: the operation ojas-cpu runs today."""
    err = _gemv_case(gpu, "q4k", 4096, 4096, 1)
    assert err < 1e-5  # integer dots are exact; only the f32 summation order differs


@pytest.mark.parametrize("tag", ["q80", "q6k"])
@pytest.mark.parametrize("n,k", [(14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("m", [1, 2, 4, 8])
def test_config2_ffn_shapes(gpu, tag, n, k, m):
    _gemv_case(gpu, tag, n, k, m, seed=m)


@pytest.mark.parametrize("tag", ["q4k", "q6k", "q80"])
@pytest.mark.parametrize("source", ["synth", "gauss"])
def test_small_and_ragged_shapes(gpu, tag, source):
    for n, k, m in [(1, 256, 1), (3, 512, 2), (17, 768, 3), (149, 2304, 5), (1000, 4352, 7), (33, 256, 8)]:
        _gemv_case(gpu, tag, n, k, m, source, seed=n)


@pytest.mark.parametrize("tag", ["q4k", "q6k", "q80"])
@pytest.mark.parametrize("form", [ACCUM, BIAS])
def test_store_forms(gpu, tag, form):
    _gemv_case(gpu, tag, 777, 1024, 1, form=form)
    _gemv_case(gpu, tag, 130, 512, 4, form=form)


@pytest.mark.parametrize("tag", ["q4k", "q6k"])
@pytest.mark.parametrize("rows_from", [0, 2, 3, 5])
def test_tensor_core_batch_kernel_from_any_batch_size(gpu, tag, rows_from):
    """Option gemv_mma: 0 = per-lane kernels only, n = the tensor-core batch kernel from n rows (the default takes it from
    five).  Small batches are quantized inside the batch kernel, larger ones (more than 32768 values) by a launch in
    front of it; both against the oracle, ragged shapes and every store form included."""
    gpu.set_option("gemv_mma", rows_from)
    try:
        for n, k, m, form in [(300, 2304, 2, PLAIN), (4096, 4096, 3, PLAIN), (1000, 4352, 4, BIAS), (17, 256, 5, ACCUM), (520, 14336, 3, PLAIN),
                              (14336, 4096, 8, PLAIN), (77, 14336, 8, ACCUM)]:
            err = _gemv_case(gpu, tag, n, k, m, form=form, seed=m + rows_from)
            assert err < 1e-5
    finally:
        gpu.set_option("gemv_mma", 1)


@pytest.mark.parametrize("segments", [0, 2, 4, 7])
def test_q80_batches_over_k_segments(gpu, segments):
    """Q8_0 batches of 3..8 rows walk a long K in equal segments inside one launch (their activations do not fit in
    shared memory whole): automatic on K = 14336, forced on shorter rows; every store form; a segment count that
    does not divide K / 256 falls back to the other path."""
    gpu.set_option("gemv_kseg", segments)
    try:
        for n, k, m, form in [(150, 14336, 8, PLAIN), (1000, 14336, 3, BIAS), (37, 14336, 5, ACCUM), (300, 3584, 8, PLAIN),
                              (4096, 7168, 6, ACCUM), (33, 1024, 4, BIAS)]:
            err = _gemv_case(gpu, "q80", n, k, m, form=form, seed=m + segments)
            assert err < 1e-5
    finally:
        gpu.set_option("gemv_kseg", 0)


@pytest.mark.parametrize("tag", ["q4k", "q6k"])
def test_prequantized_activations_match(gpu, tag):
    """gemv_q8k over quant_q8k's output gives bit-identical results to the fused call."""
    t = TYPES[tag]
    n, k, m = 515, 2048, 3
    raw = _weights(tag, n, k, "gauss")
    x = activations(m, k, seed=5)
    w = gpu.load_weight(raw, t, n, k)
    xb = gpu.upload(x)
    q, s, b = gpu.alloc_bytes(m * k), gpu.alloc(m * k // 256), gpu.alloc_bytes(m * k // 32 * 4)
    y1, y2 = gpu.alloc(m * n), gpu.alloc(m * n)
    gpu.quant_q8k(xb, m, k, q, s, b)
    gpu.gemv_q8k(w, q, s, b, y1, m)
    gpu.gemv(w, xb, y2, m)
    a, c = gpu.read(y1, np.float32, m * n), gpu.read(y2, np.float32, m * n)
    assert np.array_equal(a.view(np.uint32), c.view(np.uint32))
    assert rel_l2(a.reshape(m, n), oracle.matmul_kq(raw, t, n, k, x)) < 1e-5
    for buf in (w.buf, xb, q, s, b, y1, y2):
        gpu.free(buf)


@pytest.mark.parametrize("tag", ["q4k", "q6k", "q80"])
@pytest.mark.parametrize("warps,stages", [(16, 2), (4, 1), (8, 3), (1, 2)])
def test_every_launch_shape(gpu, tag, warps, stages):
    """The host picks the warps per CTA, the ring depth and the team width per shape; force other choices over
    every batch size, small, ragged and large shapes, and check each against the oracle."""
    gpu.set_option("gemv_warps", warps)
    gpu.set_option("gemv_stages", stages)
    try:
        for n, k, m in [(4096, 4096, 1), (300, 2304, 3), (1000, 4352, 8), (17, 256, 5), (14336, 4096, 8), (4096, 14336, 4), (5000, 8192, 1)]:
            for source in ("gauss", "synth"):
                err = _gemv_case(gpu, tag, n, k, m, source, seed=m)
                assert err < 1e-5
        _gemv_case(gpu, tag, 777, 1024, 6, form=ACCUM)
        _gemv_case(gpu, tag, 130, 512, 2, form=BIAS)
    finally:
        gpu.set_option("gemv_warps", 0)
        gpu.set_option("gemv_stages", 0)


def test_prequantized_entry_is_the_same_kernel(gpu):
    """The pre-quantized entry at the headline shape: bit-identical to the fused call."""
    n, k = 4096, 4096
    w = gpu.load_weight(_weights("q4k", n, k, "gauss"), Q4_K, n, k)
    xb = gpu.upload(activations(1, k, seed=9))
    q, sc, b = gpu.alloc_bytes(k), gpu.alloc(k // 256), gpu.alloc_bytes(k // 32 * 4)
    y1, y2 = gpu.alloc(n), gpu.alloc(n)
    gpu.quant_q8k(xb, 1, k, q, sc, b)
    gpu.gemv_q8k(w, q, sc, b, y1, 1)
    gpu.gemv(w, xb, y2, 1)
    assert np.array_equal(gpu.read(y1, np.uint32, n), gpu.read(y2, np.uint32, n))
    for buf in (w.buf, xb, q, sc, b, y1, y2):
        gpu.free(buf)


def test_results_are_deterministic(gpu):
    raw = _weights("q4k", 4096, 4096, "gauss")
    w = gpu.load_weight(raw, Q4_K, 4096, 4096)
    xb = gpu.upload(activations(1, 4096))
    y = gpu.alloc(4096)
    outs = []
    for _ in range(3):
        gpu.gemv(w, xb, y, 1)
        outs.append(gpu.read(y, np.float32, 4096).view(np.uint32).copy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    for b in (w.buf, xb, y):
        gpu.free(b)


def test_linearity_at_full_size(gpu):
    """Size-independent property at a 70B-shaped projection (28672 x 8192 Q4_K): W(2x) = 2 W(x)
    exactly (doubling x doubles every Q8_K scale and leaves q unchanged), and a sampled set of
    rows agrees with the oracle."""
    n, k = 28672, 8192
    raw = synth_weights(Q4_K, n, k)
    w = gpu.load_weight(raw, Q4_K, n, k)
    x = activations(1, k, seed=9)
    xb, x2b = gpu.upload(x), gpu.upload(x * np.float32(2))
    y, y2 = gpu.alloc(n), gpu.alloc(n)
    gpu.gemv(w, xb, y, 1)
    gpu.gemv(w, x2b, y2, 1)
    a, b = gpu.read(y, np.float32, n), gpu.read(y2, np.float32, n)
    assert np.array_equal((a * np.float32(2)).view(np.uint32), b.view(np.uint32))
    rows = np.random.default_rng(0).choice(n, 64, replace=False)
    act = oracle.quant_q8k(x[0])
    want = np.array([oracle.dot_q4k(raw.reshape(n, -1)[r], act) for r in rows], np.float32)
    assert rel_l2(a[rows], want) < 1e-5
    for buf in (w.buf, xb, x2b, y, y2):
        gpu.free(buf)


# ---------------------------------------------------------------- upload layout
@pytest.mark.parametrize("tag", ["q4k", "q6k", "q80"])
def test_device_repack_matches_host(gpu, tag):
    t = TYPES[tag]
    n, k = 37, 1280
    raw = synth_weights(t, n, k)
    w = gpu.load_weight(raw, t, n, k)
    got = gpu.read(w.buf, np.uint8, w.buf.nbytes)
    want = ob.repack_host(t, raw, n, k)
    from helpers import TILE_BYTES
    used = (n + 7) // 8 * (k // 256) * TILE_BYTES[t]          # the tiles, rows past n included (zero blocks)
    assert np.array_equal(got[:used], want[:used])
    gpu.free(w.buf)


# ---------------------------------------------------------------- name-based dispatch and errors
@pytest.mark.parametrize("tag", ["q4k", "q6k", "q80"])
def test_dispatch_by_name(gpu, tag):
    """The engine's calling convention: canonical entry name, positional (buffer, offset) pairs,
    then u32 constants (crates/ojas-core/src/kernel.rs:77-80)."""
    t = TYPES[tag]
    n, k, m = 260, 1024, 11
    raw = _weights(tag, n, k, "gauss")
    x = activations(m, k, seed=2)
    want = oracle.matmul_kq(raw, t, n, k, x)
    w = gpu.load_weight(raw, t, n, k)
    pad = 64  # a byte offset into the activation buffer, as the engine passes sub-ranges
    xb = gpu.alloc_bytes(pad + x.nbytes)
    gpu.write(xb, x, pad)
    y = gpu.upload(np.ones((m, n), np.float32))
    bias = gpu.upload(np.full(n, 0.25, np.float32))
    enc = gpu.begin()
    gpu.dispatch(enc, f"gemv_nat_{tag}", [(xb, pad), (w.buf, 0), (y, 0)], [k, n], grid=(n // 4, 1, 1), block=(64, 1, 1))
    gpu.submit(enc)
    assert rel_l2(gpu.read(y, np.float32, n), want[0]) < TOL
    gpu.dispatch(enc, f"gemv_nat_{tag}_accum", [(xb, pad), (w.buf, 0), (y, 0)], [k, n])
    assert rel_l2(gpu.read(y, np.float32, n), 2 * want[0]) < TOL
    gpu.dispatch(enc, f"gemv_nat_{tag}_bias", [(xb, pad), (w.buf, 0), (y, 0), (bias, 0)], [k, n])
    assert rel_l2(gpu.read(y, np.float32, n), want[0] + 0.25) < TOL
    gpu.dispatch(enc, f"gemv_nat_{tag}_m", [(xb, pad), (w.buf, 0), (y, 0)], [k, n, m, 0])
    assert rel_l2(gpu.read(y, np.float32, m * n).reshape(m, n), want) < TOL
    gpu.dispatch(enc, f"gemv_nat_{tag}_m", [(xb, pad), (w.buf, 0), (y, 0)], [k, n, m, 1])
    assert rel_l2(gpu.read(y, np.float32, m * n).reshape(m, n), 2 * want) < TOL
    for b in (w.buf, xb, y, bias):
        gpu.free(b)


def test_errors_are_reported_not_fatal(gpu):
    w = gpu.load_weight(synth_weights(Q4_K, 4, 256), Q4_K, 4, 256)
    x, y = gpu.upload(np.zeros(256, np.float32)), gpu.alloc(4)
    bad = ob.Lin(w.buf, Q4_K, 4, 300)
    with pytest.raises(ob.OjasB200Error, match="multiple of 256"):
        gpu.gemv(bad, x, y)
    with pytest.raises(ob.OjasB200Error, match="M="):
        gpu.gemv(w, x, y, m=9)
    with pytest.raises(ob.OjasB200Error, match="bias"):
        gpu.gemv(w, x, y, form=BIAS)
    with pytest.raises(ob.OjasB200Error, match="unsupported"):
        gpu.gemv(ob.Lin(w.buf, 10, 4, 256), x, y)                     # Q2_K: not a format of this path
    with pytest.raises(ob.OjasB200Error, match="no kernel named"):
        gpu.dispatch(gpu.begin(), "gemv_nat_q2k", [(x, 0), (w.buf, 0), (y, 0)], [256, 4])
    with pytest.raises(ob.OjasB200Error, match="expected 3 buffers"):
        gpu.dispatch(gpu.begin(), "gemv_nat_q4k", [(x, 0), (w.buf, 0)], [256, 4])
    gpu.gemv(w, x, y)  # the context is still usable after reported errors
    gpu.sync()
    for b in (w.buf, x, y):
        gpu.free(b)


def test_graph_capture_and_replay(gpu):
    """Whole decode steps are captured into CUDA graphs by the engine
    (crates/ojas-cuda/src/device.rs:541-554), so the kernels must be capture-safe."""
    n, k = 1024, 1024
    raw = _weights("q4k", n, k, "gauss")
    w = gpu.load_weight(raw, Q4_K, n, k)
    x = activations(1, k, seed=4)
    xb, y = gpu.upload(x), gpu.alloc(n)
    gpu.gemv(w, xb, y)  # first call outside capture (sets function attributes)
    gpu.sync()
    gpu.memset(y, 0)
    gpu.graph_begin()
    for _ in range(4):
        gpu.gemv(w, xb, y, 1, ACCUM)
    g = gpu.graph_end()
    gpu.graph_launch(g)
    got = gpu.read(y, np.float32, n)
    assert rel_l2(got, 4 * oracle.matvec_kq(raw, Q4_K, n, k, x[0])) < 1e-5
    gpu.graph_destroy(g)
    for b in (w.buf, xb, y):
        gpu.free(b)


def test_profiler_and_environment_options(gpu):
    """The per-launch event profiler (option "profile") names and counts the launches it saw; a second context created
    with OJAS_B200_* variables in the environment starts with those options (an unknown value is ignored)."""
    import os
    n, k = 512, 1024
    w = gpu.load_weight(synth_weights(Q4_K, n, k), Q4_K, n, k)
    x, y = gpu.upload(activations(1, k, seed=3)), gpu.alloc(n)
    gpu.set_option("profile", 1)
    try:
        for _ in range(5):
            gpu.gemv(w, x, y)
        q, s, b = gpu.alloc_bytes(k), gpu.alloc(k // 256), gpu.alloc_bytes(k // 32 * 4)
        gpu.quant_q8k(x, 1, k, q, s, b)
        rows = {name: (launches, ms) for name, launches, ms in gpu.profile_report()}
        assert rows["gemv_q4k"][0] == 5 and rows["quant_q8k"][0] == 1
        assert all(ms >= 0.0 for _, ms in rows.values()) and rows["gemv_q4k"][1] > 0.0
        gpu.profile_reset()
        gpu.gemv(w, x, y)
        assert [(name, launches) for name, launches, _ in gpu.profile_report()] == [("gemv_q4k", 1)]
    finally:
        gpu.set_option("profile", 0)
    assert gpu.profile_report() == []
    want = gpu.read(y, np.float32, n)
    old = {key: os.environ.get(key) for key in ("OJAS_B200_GEMV_WARPS", "OJAS_B200_PROFILE", "OJAS_B200_GEMM_KSPLIT")}
    os.environ.update(OJAS_B200_GEMV_WARPS="4", OJAS_B200_PROFILE="1", OJAS_B200_GEMM_KSPLIT="9999")   # the last one is out of range
    try:
        other = ob.B200Gpu(0)
        w2 = other.load_weight(synth_weights(Q4_K, n, k), Q4_K, n, k)
        x2, y2 = other.upload(activations(1, k, seed=3)), other.alloc(n)
        other.gemv(w2, x2, y2)
        assert np.array_equal(other.read(y2, np.float32, n), want)          # four warps per CTA: same sums in the same order
        assert ("gemv_q4k", 1) in [(name, launches) for name, launches, _ in other.profile_report()]
        other.set_option("profile", 0)
        other.close()
    finally:
        for key, val in old.items():
            if val is None:
                os.environ.pop(key, None)
            else:
                os.environ[key] = val
    for buf in (w.buf, x, y, q, s, b):
        gpu.free(buf)
