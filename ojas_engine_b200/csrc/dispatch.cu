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
    int (*fn)(ojas_b200_ctx *, void *const *b, const uint32_t *c);
};

static uint32_t tag_type(const char *tag) {
    if (!strcmp(tag, "q4k")) return OJAS_B200_Q4_K;
    if (!strcmp(tag, "q6k")) return OJAS_B200_Q6_K;
    return OJAS_B200_Q8_0;
}

// gemv_nat_<tag>{,_accum,_bias}: (x, w, y[, bs]) (K, N); _m: (x, w, y) (K, N, M, ACC)
// (crates/ojas-cuda/src/kernels/nat.rs:69-74).
#define GEMV_ENTRIES(tag)                                                                                           \
    static int gemv_##tag##_plain(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c) {                          \
        return ojas_b200_gemv(ctx, tag_type(#tag), OJAS_B200_PLAIN, (const float *)b[0], b[1], (float *)b[2],       \
                              nullptr, c[0], c[1], 1);                                                              \
    }                                                                                                               \
    static int gemv_##tag##_accum(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c) {                          \
        return ojas_b200_gemv(ctx, tag_type(#tag), OJAS_B200_ACCUM, (const float *)b[0], b[1], (float *)b[2],       \
                              nullptr, c[0], c[1], 1);                                                              \
    }                                                                                                               \
    static int gemv_##tag##_bias(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c) {                           \
        return ojas_b200_gemv(ctx, tag_type(#tag), OJAS_B200_BIAS, (const float *)b[0], b[1], (float *)b[2],        \
                              (const float *)b[3], c[0], c[1], 1);                                                  \
    }                                                                                                               \
    static int gemv_##tag##_m(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c) {                              \
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
GEMV_ENTRIES(q6k)
GEMV_ENTRIES(q80)

// quant_q8k: (x, q, scales, bsums) (K, M) — the activation step that precedes the K-quant
// dots (crates/ojas-cpu/src/cpu_math.rs:545-563); no CUDA entry of this name exists upstream.
static int d_quant_q8k(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c) {
    return ojas_b200_quant_q8k(ctx, (const float *)b[0], c[1], c[0], (int8_t *)b[1], (float *)b[2], (int32_t *)b[3]);
}

// gemm_mm_<q4k|q6k|q8_0>: (x, w, y, workspace) (K, N, accum, M, workspace_bytes) — the prefill entries
// of crates/ojas-cuda/src/kernels/gemm_q.rs:499-531 ((x, w, y, K, N, accum, M)) plus the scratch
// buffer this implementation needs for its f16 activation tiles.
#define GEMM_ENTRY(tag, type)                                                                                     \
    static int gemm_##tag(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c) {                                \
        return ojas_b200_gemm(ctx, type, (const float *)b[0], b[1], (float *)b[2], c[0], c[1], c[3], (int)c[2],   \
                              b[3], (size_t)c[4]);                                                                \
    }
GEMM_ENTRY(q4k, OJAS_B200_Q4_K)
GEMM_ENTRY(q6k, OJAS_B200_Q6_K)
GEMM_ENTRY(q8_0, OJAS_B200_Q8_0)

// moe_topk: (lg, idx, wgt) (E, KSEL) — crates/ojas-cuda/src/kernels/moe.rs:45; moe_topk_m adds M.
static int d_moe_topk(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c) {
    return ojas_b200_moe_topk(ctx, (const float *)b[0], (uint32_t *)b[1], (float *)b[2], 1, c[0], c[1]);
}
static int d_moe_topk_m(ojas_b200_ctx *ctx, void *const *b, const uint32_t *c) {
    return ojas_b200_moe_topk(ctx, (const float *)b[0], (uint32_t *)b[1], (float *)b[2], c[2], c[0], c[1]);
}

#define GEMV_TABLE(tag)                                      \
    {"gemv_nat_" #tag, 3, 2, gemv_##tag##_plain},            \
    {"gemv_nat_" #tag "_accum", 3, 2, gemv_##tag##_accum},   \
    {"gemv_nat_" #tag "_bias", 4, 2, gemv_##tag##_bias},     \
    {"gemv_nat_" #tag "_m", 3, 4, gemv_##tag##_m}

static const NameEntry kTable[] = {
    GEMV_TABLE(q4k), GEMV_TABLE(q6k), GEMV_TABLE(q80),
    {"quant_q8k", 4, 2, d_quant_q8k},
    {"moe_topk", 3, 2, d_moe_topk}, {"moe_topk_m", 3, 3, d_moe_topk_m},
    {"gemm_mm_q4k", 4, 5, gemm_q4k}, {"gemm_mm_q6k", 4, 5, gemm_q6k}, {"gemm_mm_q8_0", 4, 5, gemm_q8_0},
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
    (void)grid; (void)block;
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
    return e->fn(ctx, ptrs, consts);
}
