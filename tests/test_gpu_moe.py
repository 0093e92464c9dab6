"""MoE router and grouped expert FFN against the CPU oracle, through the C ABI (needs a B200)."""
import numpy as np
import pytest

import oracle
import ojas_engine_b200 as ob
from ojas_engine_b200 import Q4_K, Q6_K

from conftest import rel_l2
from helpers import activations, gauss_weights

pytestmark = pytest.mark.gpu

TOL = 2e-3


def _topk(gpu, logits, ksel):
    m, e = logits.shape
    lb = gpu.upload(logits)
    ib, wb = gpu.alloc_bytes(m * ksel * 4), gpu.alloc(m * ksel)
    gpu.moe_topk(lb, ib, wb, m, e, ksel)
    idx = gpu.read(ib, np.uint32, m * ksel).reshape(m, ksel)
    wgt = gpu.read(wb, np.float32, m * ksel).reshape(m, ksel)
    for b in (lb, ib, wb):
        gpu.free(b)
    return idx, wgt


def test_router_matches_reference_semantics(gpu):
    rng = np.random.default_rng(0)
    for m, e, ksel in [(64, 8, 2), (5, 64, 6), (3, 160, 8), (1, 8, 2), (7, 3, 3)]:
        lg = rng.standard_normal((m, e), dtype=np.float32)
        idx, wgt = _topk(gpu, lg, ksel)
        widx, wwgt = oracle.moe_topk(lg, ksel)
        assert np.array_equal(idx, widx)
        assert np.allclose(wgt, wwgt, rtol=1e-5, atol=1e-7)
        assert np.allclose(wgt.sum(1), 1.0, atol=1e-5)
    ties = np.array([[0.5, 2.0, 2.0, -1.0, 2.0]], np.float32)  # ties resolve to the lowest index
    idx, wgt = _topk(gpu, ties, 2)
    assert list(idx[0]) == [1, 2] and np.allclose(wgt[0], [0.5, 0.5])


def _moe_case(gpu, m, e, ksel, d, ffn, t_gu, t_d, idx=None, accum=False, seed=0, experts=None, tol=TOL):
    rng = np.random.default_rng(seed)
    if experts is None:
        wg = np.concatenate([gauss_weights(t_gu, ffn, d, seed + 10 * i) for i in range(e)])
        wu = np.concatenate([gauss_weights(t_gu, ffn, d, seed + 10 * i + 1) for i in range(e)])
        wd = np.concatenate([gauss_weights(t_d, d, ffn, seed + 10 * i + 2) for i in range(e)])
    else:
        wg, wu, wd = experts
    h = activations(m, d, seed=seed + 5)
    if idx is None:
        lg = rng.standard_normal((m, e), dtype=np.float32)
        idx, wgt = oracle.moe_topk(lg, ksel)
    else:
        idx = np.asarray(idx, np.uint32).reshape(m, ksel)
        wgt = rng.random((m, ksel), dtype=np.float32)
        wgt /= wgt.sum(1, keepdims=True)
    want = oracle.moe_ffn(wg, wu, wd, t_gu, t_d, h, idx, wgt, d, ffn)
    lg_, lu_, ld_ = gpu.load_weight(wg, t_gu, e * ffn, d), gpu.load_weight(wu, t_gu, e * ffn, d), gpu.load_weight(wd, t_d, e * d, ffn)
    hb, ib, wb = gpu.upload(h), gpu.upload(idx), gpu.upload(wgt)
    o0 = activations(m, d, seed=seed + 6) if accum else np.zeros((m, d), np.float32)
    ob_ = gpu.upload(o0)
    gpu.moe_ffn(lg_, lu_, ld_, hb, ib, wb, ob_, m, e, ksel, accum)
    got = gpu.read(ob_, np.float32, m * d).reshape(m, d)
    for b in (lg_.buf, lu_.buf, ld_.buf, hb, ib, wb, ob_):
        gpu.free(b)
    err = rel_l2(got, want + o0)
    assert err < tol, f"moe m={m} e={e} ksel={ksel} d={d} ffn={ffn}: rel L2 {err:.3e}"
    return err


@pytest.mark.parametrize("t_gu,t_d", [(Q4_K, Q4_K), (Q4_K, Q6_K), (Q6_K, Q6_K)])
def test_expert_ffn_small(gpu, t_gu, t_d):
    _moe_case(gpu, 9, 4, 2, 512, 768, t_gu, t_d)
    _moe_case(gpu, 3, 5, 3, 256, 512, t_gu, t_d, accum=True, seed=3)


def test_q5k_experts(gpu):
    """Q5_K experts (synthetic blocks: the library has no Q5_K encoder) on the tensor-core experts kernel, alone and with a
    Q6_K down projection; rows past one pass, the accumulate form; refused when the option turns that kernel off."""
    from ojas_engine_b200 import Q5_K

    def synth(t, n, k, roll, d=None):
        base = oracle.synth_blocks(t, n * k // 256).reshape(n, -1)
        out = np.ascontiguousarray(np.roll(base, roll, axis=0)).reshape(-1, 176 if t == Q5_K else 210)
        if d is not None:                             # smaller super-block scales: the prefill form keeps activations in f16
            out[:, 0:2] = np.frombuffer(np.float16(d).tobytes(), np.uint8)
            out[:, 2:4] = np.frombuffer(np.float16(d / 4).tobytes(), np.uint8)
        return out.reshape(-1)

    for (m, e, ksel, d, ffn, t_d, accum) in [(9, 4, 2, 512, 768, Q5_K, False), (40, 2, 2, 256, 1024, Q6_K, True), (3, 5, 3, 4096, 512, Q5_K, False)]:
        experts = (synth(Q5_K, e * ffn, d, 1), synth(Q5_K, e * ffn, d, 5), synth(t_d, e * d, ffn, 9))
        assert _moe_case(gpu, m, e, ksel, d, ffn, Q5_K, t_d, accum=accum, seed=m, experts=experts) < 3e-4
    gpu.set_option("moe_gemm_rows", 8)                # the prefill form: gate / up stay on the exact kernel, down on the f16 tcgen05 GEMM
    try:
        experts = (synth(Q5_K, 2 * 512, 256, 2, 2e-4), synth(Q5_K, 2 * 512, 256, 3, 2e-4), synth(Q5_K, 2 * 256, 512, 4, 2e-4))
        assert _moe_case(gpu, 64, 2, 2, 256, 512, Q5_K, Q5_K, seed=11, experts=experts) < TOL
    finally:
        gpu.set_option("moe_gemm_rows", 0)
    gpu.set_option("gemv_mma", 0)
    try:
        with pytest.raises(ob.OjasB200Error, match="Q5_K experts"):
            _moe_case(gpu, 2, 2, 1, 256, 256, Q5_K, Q5_K, experts=(synth(Q5_K, 512, 256, 0), synth(Q5_K, 512, 256, 1), synth(Q5_K, 512, 256, 2)))
    finally:
        gpu.set_option("gemv_mma", 1)


def test_uneven_routing(gpu):
    """All tokens on one expert (more rows than one eight-row pass), experts with no tokens at all."""
    m, e, ksel = 21, 6, 2
    idx = np.zeros((m, ksel), np.uint32)
    idx[:, 0], idx[:, 1] = 4, 1                       # experts 0, 2, 3, 5 receive nothing
    idx[::5, 1] = 5
    _moe_case(gpu, m, e, ksel, 512, 512, Q4_K, Q4_K, idx=idx)
    _moe_case(gpu, 1, 8, 2, 256, 256, Q4_K, Q4_K, idx=np.array([[7, 0]]))


def test_int8_tensor_core_experts_passes_and_k_parts(gpu):
    """The int8 tcgen05 form of the Q4_K expert FFN: experts with more rows than one 32-token pass (several passes over
    the weights), a single row, long down rows cut into K parts, the accumulate form; within the bound of the exact
    forms (typically 1e-7)."""
    gpu.set_option("moe_i8", 1)
    try:
        assert _moe_case(gpu, 80, 2, 2, 512, 1024, Q4_K, Q4_K, seed=21) < 3e-4      # 80 rows per expert: three passes
        assert _moe_case(gpu, 1, 4, 2, 256, 2048, Q4_K, Q4_K, seed=22) < 3e-4       # down K = 2048: two K parts
        assert _moe_case(gpu, 33, 3, 1, 768, 4096, Q4_K, Q4_K, accum=True, seed=23) < 3e-4
    finally:
        gpu.set_option("moe_i8", 0)


def test_config4_mixtral_shapes(gpu):
    """8 experts, gate/up 14336 x 4096 and down 4096 x 14336 in Q4_K, 64 tokens, top-2 routing from N(0,1)
    logits, softmax weights over the chosen two.  One expert's N(0, 0.02) weights are generated and
    row-rotated for the other seven to keep set-up short."""
    e, d, ffn, m, ksel = 8, 4096, 14336, 64, 2
    g0 = gauss_weights(Q4_K, ffn, d, 1).reshape(ffn, -1)
    u0 = gauss_weights(Q4_K, ffn, d, 2).reshape(ffn, -1)
    d0 = gauss_weights(Q4_K, d, ffn, 3).reshape(d, -1)
    wg = np.concatenate([np.roll(g0, 31 * i, axis=0).reshape(-1) for i in range(e)])
    wu = np.concatenate([np.roll(u0, 17 * i, axis=0).reshape(-1) for i in range(e)])
    wd = np.concatenate([np.roll(d0, 13 * i, axis=0).reshape(-1) for i in range(e)])
    _moe_case(gpu, m, e, ksel, d, ffn, Q4_K, Q4_K, experts=(wg, wu, wd), seed=0)
    gpu.set_option("moe_i8", 1)                       # the same on the int8 tcgen05 kernel
    try:
        assert _moe_case(gpu, m, e, ksel, d, ffn, Q4_K, Q4_K, experts=(wg, wu, wd), seed=0) < 3e-4
    finally:
        gpu.set_option("moe_i8", 0)


@pytest.mark.parametrize("t_gu,t_d", [(Q4_K, Q4_K), (Q4_K, Q6_K), (Q6_K, Q6_K)])
def test_prefill_sized_batches_on_tensor_cores(gpu, t_gu, t_d):
    """The prefill form (option "moe_gemm_rows"): gate and up with exact integers (Q4_K: on the int8 tcgen05 kernel, several
    32-token passes per expert), the down projection as grouped f16 tcgen05 GEMMs over the Q8_K SwiGLU rows (row counts
    read on the device).  Uneven groups, an empty expert, a group larger than one token tile, accumulate form: within
    the stated 2e-3 of the oracle (what is left is the f16 rounding of the down GEMM's operands, typically 3e-4)."""
    gpu.set_option("moe_gemm_rows", 32)
    try:
        _moe_case(gpu, 192, 4, 2, 512, 768, t_gu, t_d, seed=11, tol=TOL)
        m, e, ksel = 300, 5, 2
        idx = np.zeros((m, ksel), np.uint32)
        idx[:, 0], idx[:, 1] = 3, 1                  # experts 0, 2, 4 get (almost) nothing; expert 3 gets 300 rows
        idx[::7, 1] = 4
        _moe_case(gpu, m, e, ksel, 512, 512, t_gu, t_d, idx=idx, accum=True, seed=12, tol=TOL)
    finally:
        gpu.set_option("moe_gemm_rows", 0)


def test_every_expert_path(gpu):
    """The same small batch through the mma.sync experts kernel (default), the int8 tcgen05 kernel, the per-lane grouped
    kernels and, forced, through the prefill form."""
    # exact integer block dots: typically 1e-7; a 1e-7 difference in a gate / up output (fp32 summation order) can flip
    # the Q8_K rounding of single SwiGLU values, which shows as 1e-4 on the output
    assert _moe_case(gpu, 40, 4, 2, 512, 768, Q4_K, Q4_K, seed=13) < 3e-4
    gpu.set_option("moe_i8", 1)                       # both stages on the int8 tcgen05 kernel
    try:
        assert _moe_case(gpu, 40, 4, 2, 512, 768, Q4_K, Q4_K, seed=13) < 3e-4
    finally:
        gpu.set_option("moe_i8", 0)
    gpu.set_option("gemv_mma", 0)                     # the per-lane grouped kernels
    try:
        assert _moe_case(gpu, 40, 4, 2, 512, 768, Q4_K, Q4_K, seed=13) < 3e-4
    finally:
        gpu.set_option("gemv_mma", 1)
    gpu.set_option("moe_gemm_rows", 1)
    try:
        _moe_case(gpu, 40, 4, 2, 512, 768, Q4_K, Q4_K, seed=13, tol=TOL)
    finally:
        gpu.set_option("moe_gemm_rows", 0)


@pytest.mark.parametrize("tag,t", [("q4k", Q4_K), ("q6k", Q6_K), ("q80", ob.Q8_0)])
def test_decode_expert_entries_by_name(gpu, tag, t):
    """One token through the engine's decode-time expert entries (crates/ojas-cuda/src/kernels/moe.rs:75-178):
    moe_gu_<fmt> (grid.y = picks), moe_down_<fmt>, and their _slots forms with byte-offset tables."""
    e, ksel, d, ffn = 6, 3, 512, 768
    wg = np.concatenate([gauss_weights(t, ffn, d, 40 + i) for i in range(e)])
    wu = np.concatenate([gauss_weights(t, ffn, d, 50 + i) for i in range(e)])
    wd = np.concatenate([gauss_weights(t, d, ffn, 60 + i) for i in range(e)])
    lg_, lu_, ld_ = gpu.load_weight(wg, t, e * ffn, d), gpu.load_weight(wu, t, e * ffn, d), gpu.load_weight(wd, t, e * d, ffn)
    x = activations(1, d, seed=70)[0]
    idx = np.array([4, 0, 5], np.uint32)
    wgt = np.array([0.5, 0.3, 0.2], np.float32)
    rb_gu, rb_d = oracle.row_bytes(t, d), oracle.row_bytes(t, ffn)
    want_act = np.stack([oracle.silu_mul(oracle.matvec_kq(wg[ex * ffn * rb_gu:(ex + 1) * ffn * rb_gu], t, ffn, d, x),
                                         oracle.matvec_kq(wu[ex * ffn * rb_gu:(ex + 1) * ffn * rb_gu], t, ffn, d, x)) for ex in idx])
    x0 = activations(1, d, seed=71)[0]
    want_x = x0.copy()
    for j, ex in enumerate(idx):
        want_x = want_x + wgt[j] * oracle.matvec_kq(wd[ex * d * rb_d:(ex + 1) * d * rb_d], t, d, ffn, want_act[j])
    xb, ib, wb = gpu.upload(x), gpu.upload(idx), gpu.upload(wgt)
    act, xo = gpu.alloc(ksel * ffn), gpu.upload(x0)
    enc = gpu.begin()
    gpu.dispatch(enc, f"moe_gu_{tag}", [(xb, 0), (lg_.buf, 0), (lu_.buf, 0), (act, 0), (ib, 0)], [d, ffn], grid=(ffn // 8, ksel, 1))
    got_act = gpu.read(act, np.float32, ksel * ffn).reshape(ksel, ffn)
    assert rel_l2(got_act, want_act) < 1e-5
    gpu.dispatch(enc, f"moe_down_{tag}", [(act, 0), (ld_.buf, 0), (xo, 0), (ib, 0), (wb, 0)], [ffn, d, ksel])
    assert rel_l2(gpu.read(xo, np.float32, d), want_x) < TOL
    # the same with byte-offset tables (experts "cached" where they already are)
    from helpers import TILE_BYTES
    og = gpu.upload((idx.astype(np.uint64) * (ffn // 8 * (d // 256) * TILE_BYTES[t])).astype(np.uint32))
    od = gpu.upload((idx.astype(np.uint64) * (d // 8 * (ffn // 256) * TILE_BYTES[t])).astype(np.uint32))
    gpu.memset(act, 0)
    gpu.write(xo, x0)
    gpu.dispatch(enc, f"moe_gu_{tag}_slots", [(xb, 0), (lg_.buf, 0), (lu_.buf, 0), (act, 0), (og, 0), (og, 0)], [d, ffn], grid=(ffn // 8, ksel, 1))
    assert np.array_equal(gpu.read(act, np.uint32, ksel * ffn), got_act.view(np.uint32).reshape(-1))
    gpu.dispatch(enc, f"moe_down_{tag}_slots", [(act, 0), (ld_.buf, 0), (xo, 0), (od, 0), (wb, 0)], [ffn, d, ksel])
    assert rel_l2(gpu.read(xo, np.float32, d), want_x) < TOL
    for b in (lg_.buf, lu_.buf, ld_.buf, xb, ib, wb, act, xo, og, od):
        gpu.free(b)


def test_expert_cache_streams_and_serves_offsets(gpu):
    """Experts live on the host; a cache of three slots serves a stream of tokens through the _slots entries.  Results
    equal those of the fully resident tensors, and the cache reports its hits, misses and evictions."""
    t, e, ksel, d, ffn = Q4_K, 6, 2, 512, 768
    wg = [gauss_weights(t, ffn, d, 80 + i) for i in range(e)]
    wu = [gauss_weights(t, ffn, d, 90 + i) for i in range(e)]
    lg_, lu_ = gpu.load_weight(np.concatenate(wg), t, e * ffn, d), gpu.load_weight(np.concatenate(wu), t, e * ffn, d)
    cg = ob.ExpertCache(gpu, t, ffn, d, 3 * ob.repacked_bytes(t, ffn, d))
    cu = ob.ExpertCache(gpu, t, ffn, d, 3 * ob.repacked_bytes(t, ffn, d))
    assert cg.slots == 3
    x = activations(1, d, seed=75)[0]
    xb = gpu.upload(x)
    act, ref = gpu.alloc(ksel * ffn), gpu.alloc(ksel * ffn)
    enc = gpu.begin()
    for picks in ([0, 1], [1, 2], [0, 1], [3, 4], [4, 5], [0, 5]):
        idx = np.array(picks, np.uint32)
        ib = gpu.upload(idx)
        gpu.dispatch(enc, "moe_gu_q4k", [(xb, 0), (lg_.buf, 0), (lu_.buf, 0), (ref, 0), (ib, 0)], [d, ffn], grid=(1, ksel, 1))
        og = gpu.upload(cg.gather(idx, lambda i: wg[i]).astype(np.uint32))
        ou = gpu.upload(cu.gather(idx, lambda i: wu[i]).astype(np.uint32))
        gpu.dispatch(enc, "moe_gu_q4k_slots", [(xb, 0), (cg.arena, 0), (cu.arena, 0), (act, 0), (og, 0), (ou, 0)], [d, ffn], grid=(1, ksel, 1))
        assert np.array_equal(gpu.read(act, np.uint32, ksel * ffn), gpu.read(ref, np.uint32, ksel * ffn))
        for b in (ib, og, ou):
            gpu.free(b)
    st = cg.stats
    assert st["hits"] == 5 and st["misses"] == 7 and st["evictions"] == 4 and st["bytes_streamed"] == 7 * ob.raw_bytes(t, ffn, d)
    with pytest.raises(ob.OjasB200Error, match="more distinct experts"):
        cg.gather(np.array([0, 1, 2, 3], np.uint32), lambda i: wg[i])
    cg.close()
    cu.close()
    for b in (lg_.buf, lu_.buf, xb, act, ref):
        gpu.free(b)


def test_moe_argument_errors(gpu):
    w = gpu.load_weight(gauss_weights(ob.Q8_0, 2 * 256, 256), ob.Q8_0, 2 * 256, 256)
    h, idx, wgt, out = gpu.upload(np.zeros((1, 256), np.float32)), gpu.upload(np.zeros(2, np.uint32)), gpu.upload(np.ones(2, np.float32)), gpu.alloc(256)
    with pytest.raises(ob.OjasB200Error, match="Q4_K, Q5_K or Q6_K"):
        gpu.moe_ffn(w, w, w, h, idx, wgt, out, 1, 2, 2)
    lg = gpu.upload(np.zeros((1, 4), np.float32))
    with pytest.raises(ob.OjasB200Error, match="KSEL"):
        gpu.moe_topk(lg, idx, wgt, 1, 4, 5)
    for b in (w.buf, h, idx, wgt, out, lg):
        gpu.free(b)
