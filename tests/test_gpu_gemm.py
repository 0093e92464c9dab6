"""Parity of the tensor-core prefill GEMM with the CPU oracle, through the C ABI (needs a B200)."""
import numpy as np
import pytest

import oracle
import ojas_engine_b200 as ob
from ojas_engine_b200 import Q4_K, Q6_K, Q8_0
from ojas_engine_b200 import lib as oblib

from conftest import rel_l2
from helpers import TYPES, activations, gauss_weights, synth_weights

pytestmark = pytest.mark.gpu

TOL = 2e-3       # relative L2 against the reference CPU path (loop of matvec_kq)
SENT = 12345.5   # guard value past row M, as crates/ojas-cuda/tests/prefill_gemm_q.rs:308-319 does


def _gemm_case(gpu, tag, m, n, k, source="gauss", accum=False, ksplit=0, seed=0, want=None, raw=None, sample=None):
    """`sample`: compare only these token rows with the oracle (every row of a GEMM is computed the same way; the
    oracle takes a matvec per token, which is what bounds the sizes it can check in full)."""
    t = TYPES[tag]
    if raw is None:
        raw = synth_weights(t, n, k) if source == "synth" else gauss_weights(t, n, k, seed)
    x = activations(m, k, seed=seed + 100)
    if want is None:
        want = oracle.matmul_kq(raw, t, n, k, x if sample is None else x[sample])
    w = gpu.load_weight(raw, t, n, k)
    xb = gpu.upload(x)
    y0 = activations(m, n, seed=seed + 200) if accum else np.zeros((m, n), np.float32)
    yinit = np.concatenate([y0, np.full((1, n), SENT, np.float32)])
    yb = gpu.upload(yinit)
    gpu.set_option("gemm_ksplit", ksplit)
    try:
        gpu.gemm(w, xb, yb, m, accum)
        got = gpu.read(yb, np.float32, (m + 1) * n).reshape(m + 1, n)
    finally:
        gpu.set_option("gemm_ksplit", 0)
        for b in (w.buf, xb, yb):
            gpu.free(b)
    assert np.all(got[m] == SENT), "wrote past row M"
    if sample is not None:
        got, y0 = np.concatenate([got[sample], got[m:]]), y0[sample]
        m = len(sample)
    err = rel_l2(got[:m], want + y0 if accum else want)
    assert err < TOL, f"{tag} m={m} n={n} k={k} accum={accum} ksplit={ksplit}: rel L2 {err:.3e}"
    return err


@pytest.mark.parametrize("tag", ["q4k", "q6k", "q80"])
def test_single_tile(gpu, tag):
    _gemm_case(gpu, tag, 32, 128, 256)
    _gemm_case(gpu, tag, 128, 128, 1024, source="synth")


@pytest.mark.parametrize("tag", ["q4k", "q6k", "q80"])
def test_ragged_shapes(gpu, tag):
    for m, n, k in [(9, 130, 256), (17, 1000, 768), (100, 257, 2304), (300, 515, 512), (513, 384, 1280)]:
        _gemm_case(gpu, tag, m, n, k, seed=m)


@pytest.mark.parametrize("tag", ["q4k", "q6k", "q80"])
def test_accumulate_and_split_k(gpu, tag):
    _gemm_case(gpu, tag, 64, 256, 2048, accum=True)
    for ks in (2, 3, 8):
        _gemm_case(gpu, tag, 200, 300, 2048, ksplit=ks)
    _gemm_case(gpu, tag, 40, 256, 4096, accum=True, ksplit=4)


@pytest.mark.parametrize("n,k", [(4096, 4096), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("m", [128, 512])
def test_config3_q4k_prefill(gpu, m, n, k):
    """Q4_K prefill GEMM, the tensor-core configuration: M tokens x K=4096 / 14336, N in {4096, 14336}."""
    _gemm_case(gpu, "q4k", m, n, k, seed=3)


def test_config3_q4k_prefill_m2048(gpu):
    _gemm_case(gpu, "q4k", 2048, 4096, 4096, seed=4)


@pytest.mark.parametrize("n,k", [(14336, 4096), (4096, 14336)])
def test_config3_q4k_prefill_m2048_ffn_shapes(gpu, n, k):
    """The two FFN shapes at M = 2048 (sampled token rows against the oracle; synthetic blocks)."""
    _gemm_case(gpu, "q4k", 2048, n, k, source="synth", sample=[0, 1, 511, 1024, 1500, 2047])


@pytest.mark.parametrize("name,tag,n,k", [("qkv", "q4k", 10240, 8192), ("o", "q4k", 8192, 8192), ("gate_up", "q4k", 28672, 8192),
                                           ("down", "q6k", 8192, 28672)])
def test_config5_70b_projections_unsharded(gpu, name, tag, n, k):
    """The Llama-70B-shaped projections on one GPU: M = 1 through the GEMV (every output against the oracle) and
    M = 512 through the tensor-core GEMM (sampled token rows)."""
    t = TYPES[tag]
    raw = synth_weights(t, n, k)
    w = gpu.load_weight(raw, t, n, k)
    x1 = activations(1, k, seed=7) * np.float32(0.1)
    xb, y = gpu.upload(x1), gpu.alloc(n)
    gpu.gemv(w, xb, y, 1)
    assert rel_l2(gpu.read(y, np.float32, n), oracle.matvec_kq(raw, t, n, k, x1[0])) < 1e-5
    for b in (w.buf, xb, y):
        gpu.free(b)
    _gemm_case(gpu, tag, 512, n, k, raw=raw, sample=[0, 200, 511])


def test_captured_gemm_replays(gpu):
    """A GEMM whose tiles are split across CTAs (16 tiles on 148 SMs), captured once and replayed: every replay must
    give the same, correct result (the marks that order a split tile's pieces take a fresh value on every launch)."""
    m, n, k = 512, 1024, 4096
    raw = gauss_weights(Q4_K, n, k, 5)
    x = activations(m, k, seed=105)
    sample = [0, 100, 255, 256, 511]
    want = oracle.matmul_kq(raw, Q4_K, n, k, x[sample])
    w = gpu.load_weight(raw, Q4_K, n, k)
    xb, yb = gpu.upload(x), gpu.alloc(m * n)
    work = gpu.alloc_bytes(gpu.gemm_workspace_bytes(m, k))
    gpu.gemm(w, xb, yb, m, workspace=work)             # first call outside capture
    gpu.sync()
    gpu.graph_begin()
    gpu.gemm(w, xb, yb, m, workspace=work)
    g = gpu.graph_end()
    first = None
    for _ in range(5):
        gpu.memset(yb, 0xFF)                           # NaNs: a piece that adds before the storing piece would keep them
        gpu.graph_launch(g)
        got = gpu.read(yb, np.float32, m * n).reshape(m, n)
        assert np.isfinite(got).all()
        assert rel_l2(got[sample], want) < TOL
        if first is None:
            first = got
        assert rel_l2(got, first) < 1e-5
    gpu.graph_destroy(g)
    for b in (w.buf, xb, yb, work):
        gpu.free(b)


@pytest.mark.parametrize("name,tag", [("gemm_mm_q4k", "q4k"), ("gemm_mm_q4l", "q4k"), ("gemm_mm_q6k", "q6k"), ("gemm_mm_q8_0", "q80")])
def test_prefill_entries_by_name(gpu, name, tag):
    """The engine's prefill entry names with the engine's own argument lists
    (crates/ojas-cuda/src/kernels/gemm_q.rs:499-556): (x, w, y[, qa, qb]) (K, N, accum, M) and the split-K forms
    (xh f16, w, y[, qa, qb]) (K, N, M, nsplit), which add into a zeroed y."""
    t = TYPES[tag]
    m, n, k = 70, 384, 1024
    raw = gauss_weights(t, n, k, 9)
    x = activations(m, k, seed=19)
    want = oracle.matmul_kq(raw, t, n, k, x)
    w = gpu.load_weight(raw, t, n, k)
    xb, y = gpu.upload(x), gpu.upload(np.ones((m, n), np.float32))
    dummy = gpu.alloc(4)
    extra = [(dummy, 0), (dummy, 0)] if name.endswith("q4l") else []
    enc = gpu.begin()
    gpu.dispatch(enc, name, [(xb, 0), (w.buf, 0), (y, 0)] + extra, [k, n, 0, m])
    assert rel_l2(gpu.read(y, np.float32, m * n).reshape(m, n), want) < TOL
    gpu.dispatch(enc, name, [(xb, 0), (w.buf, 0), (y, 0)] + extra, [k, n, 1, m])             # accum
    assert rel_l2(gpu.read(y, np.float32, m * n).reshape(m, n), 2 * want) < TOL
    xh = gpu.upload(x.astype(np.float16))
    want_h = oracle.matmul_kq(raw, t, n, k, x.astype(np.float16).astype(np.float32))
    gpu.memset(y, 0)
    gpu.dispatch(enc, name + "_sk", [(xh, 0), (w.buf, 0), (y, 0)] + extra, [k, n, m, 4])
    assert rel_l2(gpu.read(y, np.float32, m * n).reshape(m, n), want_h) < TOL
    for b in (w.buf, xb, y, dummy, xh):
        gpu.free(b)


def test_prefill_entries_need_reserved_scratch_beyond_the_builtin_array(gpu):
    m, n, k = 1100, 128, 4096                          # m * k * 2 bytes > 8 MiB
    raw = synth_weights(Q4_K, n, k)
    w = gpu.load_weight(raw, Q4_K, n, k)
    x = activations(m, k, seed=3)
    xb, y = gpu.upload(x), gpu.alloc(m * n)
    have = oblib.load().ojas_b200_reserved_bytes(gpu.ctx)
    if have < gpu.gemm_workspace_bytes(m, k):
        with pytest.raises(ob.OjasB200Error, match="ojas_b200_reserve"):
            gpu.dispatch(gpu.begin(), "gemm_mm_q4k", [(xb, 0), (w.buf, 0), (y, 0)], [k, n, 0, m])
    gpu.reserve(gpu.gemm_workspace_bytes(m, k))
    gpu.dispatch(gpu.begin(), "gemm_mm_q4k", [(xb, 0), (w.buf, 0), (y, 0)], [k, n, 0, m])
    sample = [0, 700, 1099]
    assert rel_l2(gpu.read(y, np.float32, m * n).reshape(m, n)[sample], oracle.matmul_kq(raw, Q4_K, n, k, x[sample])) < TOL
    for b in (w.buf, xb, y):
        gpu.free(b)


def test_random_shapes(gpu):
    """Seeded sweep over ragged shapes, all three formats, accumulate and forced-split forms: the work list of the
    GEMM (shares of (tile, super-block) pairs, split tiles, token-tile widths) takes a different form for almost
    every one of them."""
    rng = np.random.default_rng(2024)
    for _ in range(48):
        tag = ["q4k", "q6k", "q80"][rng.integers(3)]
        k = int(rng.integers(1, 17)) * 256
        n, m = int(rng.integers(1, 2500)), int(rng.integers(9, 600))
        if n * k * m > 2e8:
            m = max(9, int(2e8 // (n * k)))
        _gemm_case(gpu, tag, m, n, k, source="synth" if rng.integers(2) else "gauss", accum=bool(rng.integers(2)),
                   ksplit=int([0, 0, 0, 2, 5][rng.integers(5)]), seed=int(rng.integers(1000)))


def test_repeated_calls_reuse_the_tile_marks(gpu):
    """Tiles whose K range is shared by several CTAs are marked "stored" with a per-launch serial number in
    memory the context owns; launches in a row (same and different shapes) must not see each other's marks."""
    t, n, k = Q4_K, 1024, 4096            # 8 tiles x 16 super-blocks over 128 CTAs: every tile is shared
    raw = gauss_weights(t, n, k, seed=5)
    w = gpu.load_weight(raw, t, n, k)
    for m in (300, 300, 64, 300):
        x = activations(m, k, seed=m)
        xb = gpu.upload(x)
        yb = gpu.upload(np.full((m, n), 7.0, np.float32))      # stale contents must not leak into the result
        gpu.gemm(w, xb, yb, m)
        got = gpu.read(yb, np.float32, m * n).reshape(m, n)
        assert rel_l2(got, oracle.matmul_kq(raw, t, n, k, x)) < TOL
        gpu.free(xb)
        gpu.free(yb)
    gpu.free(w.buf)


def test_gemm_agrees_with_exact_integer_path(gpu):
    """The f16 tensor-core result against the GEMV kernel's exact integer block dots on the same
    inputs (reduced shape): the only differences are the f16 roundings of the two operands."""
    n, k, m = 512, 2048, 8
    for t in (Q4_K, Q6_K):
        raw = gauss_weights(t, n, k, seed=7)
        x = activations(m, k, seed=8)
        w = gpu.load_weight(raw, t, n, k)
        xb, y1, y2 = gpu.upload(x), gpu.alloc(m * n), gpu.alloc(m * n)
        gpu.gemv(w, xb, y1, m)
        gpu.gemm(w, xb, y2, m)
        a, b = gpu.read(y1, np.float32, m * n), gpu.read(y2, np.float32, m * n)
        assert rel_l2(b, a) < 1e-3
        for buf in (w.buf, xb, y1, y2):
            gpu.free(buf)


def test_mm_operator_picks_by_row_count(gpu):
    """CudaSsm::mm (crates/ojas-cuda/src/qwen35.rs:644-702): few rows -> GEMV, many -> tensor-core GEMM."""
    n, k = 384, 1024
    raw = gauss_weights(Q4_K, n, k, seed=1)
    w = gpu.load_weight(raw, Q4_K, n, k)
    for m in (1, 8, 9, 70):
        x = activations(m, k, seed=m)
        xb, y = gpu.upload(x), gpu.upload(np.ones((m, n), np.float32))
        gpu.mm(xb, w, y, m, accum=True)
        got = gpu.read(y, np.float32, m * n).reshape(m, n)
        assert rel_l2(got, oracle.matmul_kq(raw, Q4_K, n, k, x) + 1.0) < TOL
        gpu.free(xb)
        gpu.free(y)
    gpu.free(w.buf)


def test_gemm_argument_errors(gpu):
    w = gpu.load_weight(synth_weights(Q4_K, 4, 256), Q4_K, 4, 256)
    x, y = gpu.upload(np.zeros((16, 256), np.float32)), gpu.alloc(16 * 4)
    small = gpu.alloc_bytes(256)
    with pytest.raises(ob.OjasB200Error, match="workspace"):
        gpu.gemm(w, x, y, 16, workspace=small)
    with pytest.raises(ob.OjasB200Error, match="multiple of 256"):
        gpu.gemm(ob.Lin(w.buf, Q4_K, 4, 100), x, y, 16)
    gpu.gemm(w, x, y, 16)
    gpu.sync()
    for b in (w.buf, x, y, small):
        gpu.free(b)
