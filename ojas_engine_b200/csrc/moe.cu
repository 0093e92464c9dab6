// Mixture-of-experts path: router top-k and the expert FFN, grouped by expert.
//
// Semantics follow the engine:
//   router   moe_topk (crates/ojas-cuda/src/kernels/moe.rs:45-70; batched form moe_topk_m,
//            crates/ojas-metal/src/kernels/moe.rs:173-199): softmax over E logits, KSEL arg-max
//            passes (ties -> lowest index), weights renormalised over the picks;
//   experts  act = silu(Wg_e h) * (Wu_e h), out += wgt * (Wd_e act), experts stacked [E*N, K]
//            (moe_gu_* / moe_down_*, crates/ojas-cuda/src/kernels/moe.rs:75-125), with the
//            arithmetic of the CPU path (crates/ojas-cpu/src/cpu_glm.rs:551-582): three matvec_kq
//            per (token, pick), so h AND the SwiGLU output are quantized to Q8_K and every block
//            dot is an exact integer dot.
// Where the engine launches one GEMV per (token, pick) and re-reads an expert once per token routed
// to it, this implementation sorts the assignments by expert and runs one grouped launch per
// expert and projection: each expert's weights stream from HBM once.  Row counts live in device
// memory, so the launch sequence does not depend on the routing (capture-safe).
#include "act_quant.cuh"

// ---------------------------------------------------------------- router
// One warp per token, MOE_ROUTER_WARPS tokens per CTA.  A pick is one warp-wide maximum over 64-bit keys
// (probability bits << 32 | ~expert): probabilities are >= 0, so their bit patterns order like the values, and the
// inverted index in the low half makes the lowest expert win a tie, as the engine's router does
// (crates/ojas-cuda/src/kernels/moe.rs:62-64).  Up to 32 experts a lane keeps its expert's probability in a
// register; beyond that the probabilities of a token sit in this warp's slice of shared memory and every lane
// scans the experts lane, lane + 32, ...  A picked expert is retired by clearing its key.
constexpr int MOE_ROUTER_WARPS = 4;

__device__ __forceinline__ unsigned long long router_key(float p, int e) {
    return ((unsigned long long)__float_as_uint(p) << 32) | (unsigned long long)(0xffffffffu - (unsigned)e);
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long t = __shfl_xor_sync(0xffffffffu, v, o);
        v = t > v ? t : v;
    }
    return v;
}

template <bool SMALL>
__global__ void __launch_bounds__(MOE_ROUTER_WARPS * 32) moe_router_kernel(const float *lg, uint32_t *idx, float *wgt, int M, int E, int ksel) {
    extern __shared__ float router_probs[];                      // !SMALL: [MOE_ROUTER_WARPS][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok = blockIdx.x * MOE_ROUTER_WARPS + warp;
    if (tok >= M) return;
    const float *l = lg + (size_t)tok * E;
    float *probs = SMALL ? nullptr : router_probs + (size_t)warp * E;
    // softmax numerators exp(l - max) and their sum
    float mx = -1e30f;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, __ldg(l + e));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float mine = 0.0f, sum = 0.0f;                               // SMALL: this lane's expert
    for (int e = lane; e < E; e += 32) {
        const float v = expf(__ldg(l + e) - mx);
        if (SMALL) mine = v; else probs[e] = v;
        sum += v;
    }
    sum = warp_sum(sum);
    if (!SMALL) __syncwarp();
    unsigned long long key = (SMALL && lane < E) ? router_key(mine, lane) : 0ull;
    float picked_w = 0.0f, wsum = 0.0f;                          // lane j keeps pick j's weight
    uint32_t picked_e = 0u;
    for (int j = 0; j < ksel; j++) {
        if (!SMALL) {
            key = 0ull;
            for (int e = lane; e < E; e += 32) {
                const float v = probs[e];
                if (v >= 0.0f) { const unsigned long long k2 = router_key(v, e); key = k2 > key ? k2 : key; }
            }
        }
        const unsigned long long best = warp_max_u64(key);
        const uint32_t e = 0xffffffffu - (uint32_t)(best & 0xffffffffull);
        const float w = __uint_as_float((unsigned)(best >> 32)) / sum;
        wsum += w;
        if (lane == j) { picked_e = e; picked_w = w; }
        if (SMALL) { if ((uint32_t)lane == e) key = 0ull; }
        else { if (lane == 0) probs[e] = -1.0f; __syncwarp(); }
    }
    if (lane < ksel) {
        idx[(size_t)tok * ksel + lane] = picked_e;
        wgt[(size_t)tok * ksel + lane] = picked_w / wsum;
    }
}

// ---------------------------------------------------------------- grouping
// Sorts the A = M * KSEL assignments by expert (stable: by assignment id inside an expert).
//   counts[e], offsets[e] : rows of expert e and where they start in the sorted order
//   tok[p]                : token row of sorted position p (the gather index of the gate/up GEMVs)
//   pos[a]                : sorted position of assignment a = t * KSEL + j (for the combine)
// One CTA; warp w handles the experts w, w + 32, ...
__global__ void __launch_bounds__(1024) moe_group_kernel(const uint32_t *idx, int A, int E, int ksel, int *counts, int *offsets,
                                                          int *tok, int *pos) {
    __shared__ int s_off[1025];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = warp; e < E; e += 32) {
        int c = 0;
        for (int a0 = 0; a0 < A; a0 += 32) {
            const int a = a0 + lane;
            const bool hit = a < A && (int)idx[a] == e;
            c += __popc(__ballot_sync(0xffffffffu, hit));
        }
        if (lane == 0) counts[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; e++) { s_off[e] = run; offsets[e] = run; run += counts[e]; }
        s_off[E] = run;
    }
    __syncthreads();
    for (int e = warp; e < E; e += 32) {
        int base = s_off[e];
        for (int a0 = 0; a0 < A; a0 += 32) {
            const int a = a0 + lane;
            const bool hit = a < A && (int)idx[a] == e;
            const unsigned mask = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const int p = base + __popc(mask & ((1u << lane) - 1u));
                tok[p] = a / ksel;
                pos[a] = p;
            }
            base += __popc(mask);
        }
    }
}

// SwiGLU + requantization (act = silu(g) * u, then quant_q8k): producers.cu
int ojas_silu_mul_q8k(ojas_b200_ctx *ctx, const float *g, const float *u, int8_t *q, float *scales, int32_t *bsums, size_t rows, size_t K);

// ---------------------------------------------------------------- SwiGLU on f32 rows (the decode entries by name use it)
// g = silu(g) * u in place, the same expression as silu_mul_q8k_kernel (producers.cu).
__global__ void __launch_bounds__(256) moe_silu_mul_kernel(float4 *g, const float4 *u, long long n4) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    float4 a = g[i];
    const float4 b = __ldg(u + i);
    a.x = __fmul_rn(__fdiv_rn(a.x, 1.0f + expf(-a.x)), b.x);
    a.y = __fmul_rn(__fdiv_rn(a.y, 1.0f + expf(-a.y)), b.y);
    a.z = __fmul_rn(__fdiv_rn(a.z, 1.0f + expf(-a.z)), b.z);
    a.w = __fmul_rn(__fdiv_rn(a.w, 1.0f + expf(-a.w)), b.w);
    g[i] = a;
}

int ojas_silu_mul_inplace(ojas_b200_ctx *ctx, float *g, const float *u, size_t n) {
    if (n % 4 != 0 || ((uintptr_t)g & 15) || ((uintptr_t)u & 15)) return ojas_fail(ctx, OJAS_B200_E_ARG, "silu_mul: rows must be multiples of 4 floats on 16-byte boundaries");
    const long long n4 = (long long)(n / 4);
    if (n4 == 0) return 0;
    moe_silu_mul_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, ctx->stream>>>((float4 *)g, (const float4 *)u, n4);
    OJAS_LAUNCH_CHECK(ctx, "moe_silu_mul");
    return 0;
}

// ---------------------------------------------------------------- combine
// out[t, :] (=, +=) sum_j wgt[t, j] * yd[pos[t*KSEL + j], :], picks added in order j = 0, 1, ... as the
// CPU path does (crates/ojas-cpu/src/cpu_glm.rs:581).
// `parts` > 1: a down output is the sum, in order, of that many planes `part_stride` floats apart (the K parts of the
// int8 tensor-core kernel).
__global__ void __launch_bounds__(256) moe_combine_kernel(const float *yd, const int *pos, const float *wgt, float *out, int ksel, int d,
                                                           int accum, int parts, size_t part_stride) {
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d) return;
    float s = 0.0f;
    for (int j = 0; j < ksel; j++) {
        const float *src = yd + (size_t)pos[t * ksel + j] * d + i;
        float v = src[0];
        for (int p = 1; p < parts; p++) v = __fadd_rn(v, src[(size_t)p * part_stride]);
        s = __fadd_rn(s, __fmul_rn(wgt[t * ksel + j], v));
    }
    float *o = out + (size_t)t * d + i;
    *o = accum ? *o + s : s;
}

// ---------------------------------------------------------------- host side
extern "C" int ojas_b200_moe_topk(ojas_b200_ctx *ctx, const float *logits, uint32_t *idx, float *wgt, size_t M, size_t E, size_t KSEL) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!logits || !idx || !wgt) return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_topk: null pointer");
    if (E == 0 || E > 1024 || KSEL == 0 || KSEL > 32 || KSEL > E)
        return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_topk: E=%zu (1..1024), KSEL=%zu (1..32, <= E)", E, KSEL);
    if (M == 0) return 0;
    if (M > 0x7fffffffu) return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_topk: too many rows");
    const unsigned blocks = (unsigned)((M + MOE_ROUTER_WARPS - 1) / MOE_ROUTER_WARPS);
    if (E <= 32) moe_router_kernel<true><<<blocks, MOE_ROUTER_WARPS * 32, 0, ctx->stream>>>(logits, idx, wgt, (int)M, (int)E, (int)KSEL);
    else moe_router_kernel<false><<<blocks, MOE_ROUTER_WARPS * 32, MOE_ROUTER_WARPS * E * sizeof(float), ctx->stream>>>(logits, idx, wgt, (int)M, (int)E, (int)KSEL);
    OJAS_LAUNCH_CHECK(ctx, "moe_topk");
    return 0;
}

namespace {
constexpr size_t MOE_I8_SPLIT_ROWS = 512, MOE_I8_MAX_PARTS = 8;   // down outputs of up to 512 assignments may be cut into up to 8 K parts
struct MoeWorkspace {
    int8_t *xq; float *xs; int32_t *xb;          // quantized h            [M, d]
    int *counts, *offsets, *tok, *pos;           // grouping
    float *g, *u;                                // gate / up outputs      [A, ffn]
    int8_t *aq; float *as; int32_t *ab;          // quantized SwiGLU       [A, ffn]
    float *yd;                                   // down outputs           [A, d]
    int8_t *qg; void *meta_gu, *meta_d;          // int8 tensor-core form: h's integers in expert order, records of both stages
    float *ydp;                                  // ... and the K-part planes of the down outputs [parts][A, d]
    size_t bytes;
};

MoeWorkspace moe_carve(void *base, size_t M, size_t E, size_t KSEL, size_t d, size_t ffn) {
    const size_t A = M * KSEL;
    uint8_t *p = (uint8_t *)base;
    size_t off = 0;
    auto take = [&](size_t n) { uint8_t *r = p ? p + off : nullptr; off += align256(n); return r; };
    MoeWorkspace w;
    w.xq = (int8_t *)take(M * d); w.xs = (float *)take(M * (d / 256) * 4); w.xb = (int32_t *)take(M * (d / 32) * 4);
    w.counts = (int *)take(E * 4); w.offsets = (int *)take(E * 4); w.tok = (int *)take(A * 4); w.pos = (int *)take(A * 4);
    w.g = (float *)take(A * ffn * 4); w.u = (float *)take(A * ffn * 4);
    w.aq = (int8_t *)take(A * ffn); w.as = (float *)take(A * (ffn / 256) * 4); w.ab = (int32_t *)take(A * (ffn / 32) * 4);
    w.yd = (float *)take(A * d * 4);
    w.qg = (int8_t *)take(A * d); w.meta_gu = take(ojas_experts_i8_meta_bytes(A, d)); w.meta_d = take(ojas_experts_i8_meta_bytes(A, ffn));
    w.ydp = (float *)take(A <= MOE_I8_SPLIT_ROWS ? MOE_I8_MAX_PARTS * A * d * 4 : 0);
    w.bytes = off;
    return w;
}
}  // namespace

extern "C" size_t ojas_b200_moe_workspace_bytes(size_t M, size_t E, size_t KSEL, size_t d, size_t ffn) {
    return moe_carve(nullptr, M, E, KSEL, d, ffn).bytes;
}

extern "C" int ojas_b200_moe_ffn(ojas_b200_ctx *ctx, uint32_t type_gu, uint32_t type_d, const float *h, const void *wg, const void *wu,
                                 const void *wd, const uint32_t *idx, const float *wgt, size_t M, size_t E, size_t KSEL, size_t d,
                                 size_t ffn, float *out, int accum, void *workspace, size_t workspace_bytes) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!h || !wg || !wu || !wd || !idx || !wgt || !out || !workspace) return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_ffn: null pointer");
    if (d == 0 || ffn == 0 || d % 256 != 0 || ffn % 256 != 0)
        return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_ffn: d=%zu and ffn=%zu must be positive multiples of 256", d, ffn);
    if (E == 0 || E > 1024 || KSEL == 0 || KSEL > 32 || KSEL > E) return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_ffn: E=%zu KSEL=%zu out of range", E, KSEL);
    if (M == 0) return 0;
    if (M * KSEL > 0x3fffffffu) return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_ffn: too many assignments");
    auto expert_type = [](uint32_t t) { return t == OJAS_B200_Q4_K || t == OJAS_B200_Q5_K || t == OJAS_B200_Q6_K; };
    if (!expert_type(type_gu) || !expert_type(type_d))
        return ojas_fail(ctx, OJAS_B200_E_UNSUPPORTED, "moe_ffn: expert weights must be Q4_K, Q5_K or Q6_K (got %u / %u)", type_gu, type_d);
    if ((type_gu == OJAS_B200_Q5_K || type_d == OJAS_B200_Q5_K) && ctx->gemv_mma == 0)
        return ojas_fail(ctx, OJAS_B200_E_UNSUPPORTED, "moe_ffn: Q5_K experts run on the tensor-core experts kernel only (option gemv_mma is 0)");
    if (workspace_bytes < ojas_b200_moe_workspace_bytes(M, E, KSEL, d, ffn))
        return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_ffn: workspace of %zu bytes, %zu needed", workspace_bytes,
                         ojas_b200_moe_workspace_bytes(M, E, KSEL, d, ffn));
    if (((uintptr_t)workspace & 255) || ((uintptr_t)wg & 255) || ((uintptr_t)wu & 255) || ((uintptr_t)wd & 255) || ((uintptr_t)h & 15))
        return ojas_fail(ctx, OJAS_B200_E_ARG, "moe_ffn: misaligned pointer");
    const size_t A = M * KSEL;
    const MoeWorkspace w = moe_carve(workspace, M, E, KSEL, d, ffn);

    // Every form quantizes h to Q8_K, sorts the assignments by expert and computes gate and up with EXACT integer block
    // dots (the SwiGLU output is re-quantized, and an inexact gate / up value flips roundings there by whole steps).
    //   decode-sized batches: down is exact too (the default).
    //   prefill-sized batches (option moe_gemm_rows = R, from R rows per expert on average): gate and up on the int8
    //     tcgen05 kernel, down as grouped f16 tensor-core GEMMs over the Q8_K SwiGLU rows (arithmetic of ojas_b200_gemm).
    const bool prefill = ctx->moe_gemm_rows > 0 && A / E >= (size_t)ctx->moe_gemm_rows;
    const bool i8_fits = type_gu == OJAS_B200_Q4_K && E <= 64;
    int rc = ojas_b200_quant_q8k(ctx, h, M, d, w.xq, w.xs, w.xb);
    if (rc) return rc;
    moe_group_kernel<<<1, 1024, 0, ctx->stream>>>(idx, (int)A, (int)E, (int)KSEL, w.counts, w.offsets, w.tok, w.pos);
    OJAS_LAUNCH_CHECK(ctx, "moe_group");

    // ---- gate and up
    bool gu_i8 = false;
    if (i8_fits && (prefill || (ctx->moe_i8 && type_d == OJAS_B200_Q4_K))) {
        rc = ojas_experts_i8_pack(ctx, w.xq, w.xs, w.xb, w.tok, A, d, w.qg, w.meta_gu);
        if (rc) return rc;
        rc = ojas_experts_i8(ctx, (const uint8_t *)wg, (const uint8_t *)wu, w.g, w.u, w.qg, w.meta_gu, A, w.counts, w.offsets, E, d, ffn, 1, 0,
                             prefill ? 64 : 32);          // prefill-sized groups: 64 tokens per pass over an expert's weights
        if (rc < 0) return rc;
        gu_i8 = rc == 0;
    }
    if (!gu_i8) {
        // one launch of the mma.sync experts kernel over every expert and both tensors (Q4_K); otherwise one grouped
        // launch per expert and tensor
        rc = 1;
        if (ctx->gemv_mma != 0) {
            rc = ojas_gemv_experts_kq(ctx, type_gu, (const uint8_t *)wg, (const uint8_t *)wu, w.g, w.u, w.xq, w.xs, w.xb, w.tok, w.counts, w.offsets, E, d,
                                      ffn, (A + E - 1) / E);
            if (rc == 1)
                rc = ojas_gemv_experts_batch(ctx, type_gu, (const uint8_t *)wg, (const uint8_t *)wu, w.g, w.u, w.xq, w.xs, w.xb, w.tok, w.counts,
                                             w.offsets, E, d, ffn, (A + E - 1) / E);
        }
        if (rc < 0) return rc;
        for (size_t e = 0; rc == 1 && e < E; e++) {   // gate and up of expert e over its tokens (gathered rows of h)
            int r2 = ojas_gemv_grouped(ctx, type_gu, weight_rows_at(type_gu, wg, d, e * ffn), w.xq, w.xs, w.xb, w.tok,
                                       w.counts + e, w.offsets + e, w.g, d, ffn);
            if (r2) return r2;
            r2 = ojas_gemv_grouped(ctx, type_gu, weight_rows_at(type_gu, wu, d, e * ffn), w.xq, w.xs, w.xb, w.tok,
                                   w.counts + e, w.offsets + e, w.u, d, ffn);
            if (r2) return r2;
        }
    }
    rc = ojas_silu_mul_q8k(ctx, w.g, w.u, w.aq, w.as, w.ab, A, ffn);
    if (rc) return rc;

    // ---- down
    const dim3 grid((unsigned)((d + 255) / 256), (unsigned)M);
    if (prefill) {
        void *ah = (void *)w.u;                      // the up outputs are consumed: their space takes the f16 SwiGLU rows
        rc = ojas_gemm_prep_q8k(ctx, w.aq, w.as, ah, A, ffn);
        if (rc) return rc;
        OJAS_CUDA(ctx, cudaMemsetAsync(w.yd, 0, A * d * sizeof(float), ctx->stream));    // split tiles are added into zeros
        for (size_t e = 0; e < E; e++) {
            rc = ojas_gemm_grouped(ctx, type_d, ah, A, weight_rows_at(type_d, wd, ffn, e * d), w.yd, ffn, d, A / E, w.counts + e, w.offsets + e);
            if (rc) return rc;
        }
        moe_combine_kernel<<<grid, 256, 0, ctx->stream>>>(w.yd, w.pos, wgt, out, (int)KSEL, (int)d, accum ? 1 : 0, 1, 0);
        OJAS_LAUNCH_CHECK(ctx, "moe_combine");
        return 0;
    }
    if (gu_i8 && type_d == OJAS_B200_Q4_K) {
        rc = ojas_experts_i8_pack(ctx, w.aq, w.as, w.ab, nullptr, A, ffn, nullptr, w.meta_d);
        if (rc) return rc;
        // K parts of the down projection: few 128-row tiles per expert, long rows -> cut K so that every SM gets
        // about six items
        const size_t tiles = (d + 127) / 128, items = (E < A ? E : A) * tiles;
        size_t parts = 1;
        if (A <= MOE_I8_SPLIT_ROWS) {
            parts = (6 * (size_t)ctx->sm_count + items - 1) / items;
            if (parts > MOE_I8_MAX_PARTS) parts = MOE_I8_MAX_PARTS;
            if (parts > ffn / 1024) parts = ffn / 1024 ? ffn / 1024 : 1;
        }
        float *ydst = A <= MOE_I8_SPLIT_ROWS ? w.ydp : w.yd;
        rc = ojas_experts_i8(ctx, (const uint8_t *)wd, nullptr, ydst, nullptr, w.aq, w.meta_d, A, w.counts, w.offsets, E, ffn, d, (int)parts, A * d, 32);
        if (rc) return rc < 0 ? rc : ojas_fail(ctx, OJAS_B200_E_UNSUPPORTED, "moe_ffn: the down projection does not fit the int8 kernel");
        moe_combine_kernel<<<grid, 256, 0, ctx->stream>>>(ydst, w.pos, wgt, out, (int)KSEL, (int)d, accum ? 1 : 0, (int)parts, A * d);
        OJAS_LAUNCH_CHECK(ctx, "moe_combine");
        return 0;
    }
    rc = 1;
    if (ctx->gemv_mma != 0) {
        rc = ojas_gemv_experts_kq(ctx, type_d, (const uint8_t *)wd, nullptr, w.yd, nullptr, w.aq, w.as, w.ab, nullptr, w.counts, w.offsets, E, ffn, d,
                                  (A + E - 1) / E);
        if (rc == 1)
            rc = ojas_gemv_experts_batch(ctx, type_d, (const uint8_t *)wd, nullptr, w.yd, nullptr, w.aq, w.as, w.ab, nullptr, w.counts, w.offsets, E,
                                         ffn, d, (A + E - 1) / E);
    }
    if (rc < 0) return rc;
    for (size_t e = 0; rc == 1 && e < E; e++) {   // down of expert e over its (contiguous, sorted) rows
        const int r2 = ojas_gemv_grouped(ctx, type_d, weight_rows_at(type_d, wd, ffn, e * d), w.aq, w.as, w.ab, nullptr,
                                         w.counts + e, w.offsets + e, w.yd, ffn, d);
        if (r2) return r2;
    }
    moe_combine_kernel<<<grid, 256, 0, ctx->stream>>>(w.yd, w.pos, wgt, out, (int)KSEL, (int)d, accum ? 1 : 0, 1, 0);
    OJAS_LAUNCH_CHECK(ctx, "moe_combine");
    return 0;
}
