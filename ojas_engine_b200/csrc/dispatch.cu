// Name-based dispatch: the C form of KernelRuntime::dispatch
// (crates/ojas-core/src/kernel.rs:68-83).  The engine's graphs launch kernels by canonical
// entry name with positional buffers (pointer + byte offset) followed by u32 constants
// (crates/ojas-cuda/src/device.rs:391-415); this shim accepts the same call and routes it to
// the typed entry points.  grid and block are accepted and ignored: launch shapes are this
// library's own business.
#include "common.cuh"

struct NameEntry {
    const char *name;
    int nbufs, nconsts;
    int (*fn)(ojas_b200_ctx *, void *const *b, const uint32_t *c, const uint32_t *grid);
};

static uint32_t tag_type(const char *tag) {
    if (!strcmp(tag, "q4k")) return OJAS_B200_Q4_K;
    if (!strcmp(tag, "q5k")) return OJAS_B200_Q5_K;
    if (!strcmp(tag, "q6k")) return OJAS_B200_Q6_K;
    if (!strcmp(tag, "iq4xs")) return OJAS_B200_IQ4_XS;
    if (!strcmp(tag, "iq4nl")) return OJAS_B200_IQ4_NL;
    return OJAS_B200_Q8_0;
}

// gemv_nat_<tag>{,_accum,_bias}: (x, w, y[, bs]) (K, N); _m: (x, w, y) (K, N, M, ACC)
// (crates/ojas-cuda/src/kernels/nat.rs:69-74).
#define GEMV_ENTRIES(tag)                                                                                           \
    static int gemv_##tag##_plain(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) {                          \
        return ojas_b200_gemv(ctx, tag_type(#tag), OJAS_B200_PLAIN, (const float *)b[0], b[1], (float *)b[2],       \
                              nullptr, c[0], c[1], 1);                                                              \
    }                                                                                                               \
    static int gemv_##tag##_accum(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) {                          \
        return ojas_b200_gemv(ctx, tag_type(#tag), OJAS_B200_ACCUM, (const float *)b[0], b[1], (float *)b[2],       \
                              nullptr, c[0], c[1], 1);                                                              \
    }                                                                                                               \
    static int gemv_##tag##_bias(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) {                           \
        return ojas_b200_gemv(ctx, tag_type(#tag), OJAS_B200_BIAS, (const float *)b[0], b[1], (float *)b[2],        \
                              (const float *)b[3], c[0], c[1], 1);                                                  \
    }                                                                                                               \
    static int gemv_##tag##_m(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) {                              \
        const size_t M = c[2];                                                                                      \
        const int form = c[3] ? OJAS_B200_ACCUM : OJAS_B200_PLAIN;                                                  \
        for (size_t m0 = 0; m0 < M; m0 += OJAS_B200_GEMV_MAX_M) {                                                   \
            const size_t mb = M - m0 < OJAS_B200_GEMV_MAX_M ? M - m0 : OJAS_B200_GEMV_MAX_M;                        \
            int rc = ojas_b200_gemv(ctx, tag_type(#tag), form, (const float *)b[0] + m0 * c[0], b[1],               \
                                    (float *)b[2] + m0 * c[1], nullptr, c[0], c[1], mb);                            \
            if (rc) return rc;                                                                                      \
        }                                                                                                           \
        return 0;                                                                                                   \
    }

GEMV_ENTRIES(q4k)
GEMV_ENTRIES(q5k)
GEMV_ENTRIES(q6k)
GEMV_ENTRIES(q80)
GEMV_ENTRIES(iq4xs)   // gemv_nat_iq4xs, gemv_nat_iq4nl: crates/ojas-core/src/quant_src.rs:85-110
GEMV_ENTRIES(iq4nl)

// quant_q8k: (x, q, scales, bsums) (K, M) — the activation step that precedes the K-quant
// dots (crates/ojas-cpu/src/cpu_math.rs:545-563); no CUDA entry of this name exists upstream.
static int d_quant_q8k(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) {
    return ojas_b200_quant_q8k(ctx, (const float *)b[0], c[1], c[0], (int8_t *)b[1], (float *)b[2], (int32_t *)b[3]);
}

// Prefill entries with the engine's own argument lists (crates/ojas-cuda/src/kernels/gemm_q.rs:499-556):
//   gemm_mm_q6k, gemm_mm_q8_0 : (x, w, y) (K, N, accum, M)
//   gemm_mm_q4l               : (x, w4, y, qa, qb) (K, N, accum, M) -- the engine's Q4L relayout of Q4_K is lossy and is
//                               not reproduced here: w4 is this library's repacked Q4_K weight, qa / qb are ignored
//   gemm_mm_q4k               : (x, w, y) (K, N, accum, M), the same without the two unused buffers
//   *_sk                      : (xh, w, y[, qa, qb]) (K, N, M, nsplit): f16 activations, results ADDED into a y the
//                               caller zeroed; nsplit is accepted and ignored (the K split is this library's business)
// The f16 activation tiles go to the context's reserved scratch (ojas_b200_reserve) or, up to 8 MiB, to the array built
// into the library; nothing is allocated here.
static int gemm_named(ojas_b200_ctx *ctx, uint32_t type, const void *x, bool f16, const void *w, float *y, size_t K, size_t N, size_t M, int accum) {
    const size_t need = ojas_b200_gemm_workspace_bytes(M, K);
    void *ws = ojas_scratch_for(ctx, need, "gemm_mm");
    if (!ws) return OJAS_B200_E_LIMIT;
    if (f16) return ojas_b200_gemm_f16(ctx, type, x, w, y, K, N, M, accum, ws, need);
    return ojas_b200_gemm(ctx, type, (const float *)x, w, y, K, N, M, accum, ws, need);
}
#define GEMM_ENTRY(tag, type)                                                                                       \
    static int gemm_##tag(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) {                \
        return gemm_named(ctx, type, b[0], false, b[1], (float *)b[2], c[0], c[1], c[3], (int)c[2]);                \
    }                                                                                                               \
    static int gemm_##tag##_sk(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) {           \
        return gemm_named(ctx, type, b[0], true, b[1], (float *)b[2], c[0], c[1], c[2], 1);                         \
    }
GEMM_ENTRY(q4k, OJAS_B200_Q4_K)
GEMM_ENTRY(q4l, OJAS_B200_Q4_K)
GEMM_ENTRY(q6k, OJAS_B200_Q6_K)
GEMM_ENTRY(q8_0, OJAS_B200_Q8_0)

// Decode-time expert FFN of one token (crates/ojas-cuda/src/kernels/moe.rs:75-178; upstream has the Q8_0 forms on
// CUDA and the K-quant forms on Metal, crates/ojas-metal/src/kernels/moe.rs:513-529):
//   moe_gu_<fmt>         (x, wg, wu, act, idx) (K, N), grid.y = picks: act[j, :] = silu(Wg_e x) * (Wu_e x), e = idx[j]
//   moe_down_<fmt>       (act, wd, x, idx, wgt) (K, N, KSEL): x += sum_j wgt[j] * Wd_e act[j, :]
//   moe_gu_<fmt>_slots   (x, arena_g, arena_u, act, off_g, off_u) (K, N): experts at byte offsets off_g[j], off_u[j]
//   moe_down_<fmt>_slots (act, arena, x, off_d, wgt) (K, N, KSEL)
// wg / wu / wd are this library's repacked stacked experts (expert e starts e * repacked_bytes(N, K) behind the base: N
// must be a multiple of 8); offsets are byte offsets of repacked experts.  The pick is read on the device.  The up
// outputs pass through the context's activation scratch.
static size_t expert_stride(uint32_t type, size_t N, size_t K) { return (N / OJAS_TILE_ROWS) * (K / 256) * (size_t)tile_bytes(type); }

static int moe_gu_named(ojas_b200_ctx *ctx, uint32_t type, void *const *b, const uint32_t *c, const uint32_t *grid, bool slots) {
    const size_t K = c[0], N = c[1], ksel = grid ? grid[1] : 0;
    if (ksel == 0 || ksel > 32) return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_gu: grid.y = %zu picks (1..32)", ksel);
    if (N % OJAS_TILE_ROWS != 0 || N % 4 != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_gu: N=%zu must be a multiple of 8", N);
    if (!ctx->act_scratch || ksel * N * sizeof(float) > OJAS_ACT_SCRATCH_BYTES)
        return ojas_fail(ctx, OJAS_B200_E_LIMIT, "moe_gu: %zu picks x N=%zu exceed the context's activation scratch", ksel, N);
    const float *x = (const float *)b[0];
    float *act = (float *)b[3], *up = (float *)ctx->act_scratch;
    const uint32_t *sg = (const uint32_t *)b[4], *su = slots ? (const uint32_t *)b[5] : (const uint32_t *)b[4];
    const size_t stride = slots ? 0 : expert_stride(type, N, K);
    for (size_t j = 0; j < ksel; j++) {
        int rc = ojas_gemv_selected(ctx, type, OJAS_B200_PLAIN, x, b[1], sg + j, stride, nullptr, act + j * N, K, N);
        if (rc) return rc;
        rc = ojas_gemv_selected(ctx, type, OJAS_B200_PLAIN, x, b[2], su + j, stride, nullptr, up + j * N, K, N);
        if (rc) return rc;
    }
    return ojas_silu_mul_inplace(ctx, act, up, ksel * N);
}

static int moe_down_named(ojas_b200_ctx *ctx, uint32_t type, void *const *b, const uint32_t *c, bool slots) {
    const size_t K = c[0], N = c[1], ksel = c[2];
    if (ksel == 0 || ksel > 32) return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_down: KSEL = %zu (1..32)", ksel);
    if (N % OJAS_TILE_ROWS != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_down: N=%zu must be a multiple of 8", N);
    const float *act = (const float *)b[0], *wgt = (const float *)b[4];
    const uint32_t *sel = (const uint32_t *)b[3];
    const size_t stride = slots ? 0 : expert_stride(type, N, K);
    for (size_t j = 0; j < ksel; j++) {
        const int rc = ojas_gemv_selected(ctx, type, OJAS_B200_ACCUM, act + j * K, b[1], sel + j, stride, wgt + j, (float *)b[2], K, N);
        if (rc) return rc;
    }
    return 0;
}

#define MOE_ENTRIES(tag)                                                                                                               \
    static int moe_gu_##tag(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *g) { return moe_gu_named(ctx, tag_type(#tag), b, c, g, false); }       \
    static int moe_gu_##tag##_slots(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *g) { return moe_gu_named(ctx, tag_type(#tag), b, c, g, true); } \
    static int moe_down_##tag(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) { return moe_down_named(ctx, tag_type(#tag), b, c, false); }       \
    static int moe_down_##tag##_slots(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) { return moe_down_named(ctx, tag_type(#tag), b, c, true); }
MOE_ENTRIES(q4k)
MOE_ENTRIES(q5k)
MOE_ENTRIES(q6k)
MOE_ENTRIES(q80)
MOE_ENTRIES(iq4xs)   // moe_gu_iq4xs: crates/ojas-cuda/src/kernels/moe_iq.rs:64-84 (the other three forms by analogy)
MOE_ENTRIES(iq4nl)   // moe_down_iq4nl: crates/ojas-cuda/src/kernels/moe_iq.rs:87-108 (the other three forms by analogy)

// moe_topk: (lg, idx, wgt) (E, KSEL) — crates/ojas-cuda/src/kernels/moe.rs:45; moe_topk_m adds M.
static int d_moe_topk(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) {
    return ojas_b200_moe_topk(ctx, (const float *)b[0], (uint32_t *)b[1], (float *)b[2], 1, c[0], c[1]);
}
static int d_moe_topk_m(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) {
    return ojas_b200_moe_topk(ctx, (const float *)b[0], (uint32_t *)b[1], (float *)b[2], c[2], c[0], c[1]);
}

// q35_embed_q4k: (emb, ids, x) (d, M) -- crates/ojas-cuda/src/kernels/qwen35.rs:53; the table is raw GGUF Q4_K
static int d_embed_q4k(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c, const uint32_t *) {
    return ojas_b200_embed_rows(ctx, OJAS_B200_Q4_K, b[0], 0xffffffffu, (const uint32_t *)b[1], c[1], c[0], (float *)b[2]);
}

#define GEMV_TABLE(tag)                                      \
    {"gemv_nat_" #tag, 3, 2, gemv_##tag##_plain},            \
    {"gemv_nat_" #tag "_accum", 3, 2, gemv_##tag##_accum},   \
    {"gemv_nat_" #tag "_bias", 4, 2, gemv_##tag##_bias},     \
    {"gemv_nat_" #tag "_m", 3, 4, gemv_##tag##_m}

#define MOE_TABLE(tag)                                                                             \
    {"moe_gu_" #tag, 5, 2, moe_gu_##tag}, {"moe_down_" #tag, 5, 3, moe_down_##tag},                 \
    {"moe_gu_" #tag "_slots", 6, 2, moe_gu_##tag##_slots}, {"moe_down_" #tag "_slots", 5, 3, moe_down_##tag##_slots}

static const NameEntry kTable[] = {
    GEMV_TABLE(q4k), GEMV_TABLE(q5k), GEMV_TABLE(q6k), GEMV_TABLE(q80), GEMV_TABLE(iq4xs), GEMV_TABLE(iq4nl),
    {"quant_q8k", 4, 2, d_quant_q8k},
    {"q35_embed_q4k", 3, 2, d_embed_q4k},
    {"moe_topk", 3, 2, d_moe_topk}, {"moe_topk_m", 3, 3, d_moe_topk_m},
    {"gemm_mm_q4k", 3, 4, gemm_q4k}, {"gemm_mm_q6k", 3, 4, gemm_q6k}, {"gemm_mm_q8_0", 3, 4, gemm_q8_0}, {"gemm_mm_q4l", 5, 4, gemm_q4l},
    {"gemm_mm_q4k_sk", 3, 4, gemm_q4k_sk}, {"gemm_mm_q6k_sk", 3, 4, gemm_q6k_sk}, {"gemm_mm_q8_0_sk", 3, 4, gemm_q8_0_sk},
    {"gemm_mm_q4l_sk", 5, 4, gemm_q4l_sk},
    MOE_TABLE(q4k), MOE_TABLE(q5k), MOE_TABLE(q6k), MOE_TABLE(q80), MOE_TABLE(iq4xs), MOE_TABLE(iq4nl),
};
static const int kTableLen = (int)(sizeof kTable / sizeof kTable[0]);

static const NameEntry *find_entry(const char *name) {
    if (!name) return nullptr;
    for (int i = 0; i < kTableLen; i++)
        if (!strcmp(kTable[i].name, name)) return &kTable[i];
    return nullptr;
}

extern "C" int ojas_b200_has_kernel(const char *name) { return find_entry(name) != nullptr; }
extern "C" int ojas_b200_kernel_count(void) { return kTableLen; }
extern "C" const char *ojas_b200_kernel_name(int i) { return (i >= 0 && i < kTableLen) ? kTable[i].name : nullptr; }

extern "C" int ojas_b200_dispatch(ojas_b200_ctx *ctx, const char *name, void *const *bufs, const uint64_t *offsets,
                                  int nbufs, const uint32_t *consts, int nconsts, const uint32_t grid[3],
                                  const uint32_t block[3]) {
    (void)block;
    if (!ctx) return OJAS_B200_E_ARG;
    const NameEntry *e = find_entry(name);
    if (!e) return ojas_fail(ctx, OJAS_B200_E_NAME, "dispatch: no kernel named '%s'", name ? name : "(null)");
    if (nbufs != e->nbufs || nconsts != e->nconsts)
        return ojas_fail(ctx, OJAS_B200_E_ARG, "dispatch %s: expected %d buffers and %d constants, got %d and %d", name,
                         e->nbufs, e->nconsts, nbufs, nconsts);
    void *ptrs[16];
    for (int i = 0; i < nbufs; i++) {
        if (!bufs || !bufs[i]) return ojas_fail(ctx, OJAS_B200_E_ARG, "dispatch %s: buffer %d is null", name, i);
        ptrs[i] = (uint8_t *)bufs[i] + (offsets ? offsets[i] : 0);
    }
    return e->fn(ctx, ptrs, consts, grid);
}
