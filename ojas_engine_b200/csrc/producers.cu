// Activation producers that end in Q8_K: the K-quant GEMVs take int8 activations, so the operation that makes an
// activation row can quantize it on the way out and the f32 row never travels.  Counterparts of the reference's
// rmsnorm_q8 and silu_mul_q8 (crates/ojas-cuda/src/kernels/ops.rs:27, 352), which end in its q8_1 blocks; here
// they end in the Q8_K form of quant_q8k (crates/ojas-cpu/src/cpu_math.rs:545-563) that the CPU matmul uses, and the
// quantization step is bit-identical to it.
#include "act_quant.cuh"

// RMSNorm (crates/ojas-cpu/src/cpu_math.rs:456-460): inv = 1 / sqrt(mean(x^2) + eps), out = (x * inv) * w.  One CTA
// per row: the sum of squares is a tree sum (the CPU adds in index order: the two agree to fp32 rounding, not bit for
// bit), the normalized row sits in shared memory, then one warp per 256 values quantizes it exactly as quant_q8k.
__global__ void __launch_bounds__(512) rmsnorm_q8k_kernel(const float *x, const float *w, float eps, float *xn, int8_t *q, float *scales,
                                                           int32_t *bsums, int K) {
    extern __shared__ float norm_row[];          // [K]
    __shared__ float warp_part[16];
    __shared__ float inv_s;
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const float *xr = x + (size_t)row * K;
    grid_launch_dependents();                    // the kernel behind this one may start its own set-up (it waits for this grid before it reads q)
    grid_dependency_wait();
    // the row is read once: up to four float4 per thread stay in registers between the sum of squares and the scaling
    constexpr int HOLD = 4;
    float4 held[HOLD];
    const bool fits = K <= (int)blockDim.x * 4 * HOLD;
    float s = 0.0f;
#pragma unroll
    for (int h = 0; h < HOLD; h++) {
        const int i = (h * (int)blockDim.x + (int)threadIdx.x) * 4;
        held[h] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (fits && i < K) {
            held[h] = __ldg(reinterpret_cast<const float4 *>(xr + i));
            s = fmaf(held[h].x, held[h].x, s); s = fmaf(held[h].y, held[h].y, s); s = fmaf(held[h].z, held[h].z, s); s = fmaf(held[h].w, held[h].w, s);
        }
    }
    if (!fits)
        for (int i = threadIdx.x * 4; i < K; i += blockDim.x * 4) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(xr + i));
            s = fmaf(v.x, v.x, s); s = fmaf(v.y, v.y, s); s = fmaf(v.z, v.z, s); s = fmaf(v.w, v.w, s);
        }
    s = warp_sum(s);
    if (lane == 0) warp_part[warp] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.0f;
        for (int j = 0; j < warps; j++) tot += warp_part[j];
        inv_s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), eps)));
    }
    __syncthreads();
    const float inv = inv_s;
    auto emit = [&](int i, const float4 &v) {
        const float4 g = __ldg(reinterpret_cast<const float4 *>(w + i));
        float4 o;
        o.x = __fmul_rn(__fmul_rn(v.x, inv), g.x); o.y = __fmul_rn(__fmul_rn(v.y, inv), g.y);
        o.z = __fmul_rn(__fmul_rn(v.z, inv), g.z); o.w = __fmul_rn(__fmul_rn(v.w, inv), g.w);
        *reinterpret_cast<float4 *>(norm_row + i) = o;
        if (xn) *reinterpret_cast<float4 *>(xn + (size_t)row * K + i) = o;
    };
    if (fits) {
#pragma unroll
        for (int h = 0; h < HOLD; h++) {
            const int i = (h * (int)blockDim.x + (int)threadIdx.x) * 4;
            if (i < K) emit(i, held[h]);
        }
    } else {
        for (int i = threadIdx.x * 4; i < K; i += blockDim.x * 4) emit(i, __ldg(reinterpret_cast<const float4 *>(xr + i)));
    }
    __syncthreads();
    const int nsb = K >> 8;
    for (int sb = warp; sb < nsb; sb += warps) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = norm_row[sb * 256 + lane * 8 + i];
        const Q8kLane ql = quant_q8k_values(v);
        const size_t g = (size_t)row * nsb + sb;
        reinterpret_cast<uint2 *>(q + g * 256)[lane] = ql.packed;
        int t = ql.sum8;
        t += __shfl_xor_sync(0xffffffffu, t, 1);
        t += __shfl_xor_sync(0xffffffffu, t, 2);
        if ((lane & 3) == 0) bsums[g * 8 + (lane >> 2)] = t;
        if (lane == 0) scales[g] = ql.scale;
    }
}

// act = silu(g) * u, then quant_q8k(act): one warp per (row, super-block).  silu(x) = x / (1 + exp(-x))
// (crates/ojas-cpu/src/cpu_math.rs:486).
__global__ void __launch_bounds__(256) silu_mul_q8k_kernel(const float *g, const float *u, int8_t *q, float *scales, int32_t *bsums,
                                                            long long n_sb) {
    const int lane = threadIdx.x & 31;
    const long long sb = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    grid_launch_dependents();
    grid_dependency_wait();                      // g and u come from the kernel before this one
    if (sb >= n_sb) return;
    const float4 g0 = __ldg(reinterpret_cast<const float4 *>(g + sb * 256) + lane * 2), g1 = __ldg(reinterpret_cast<const float4 *>(g + sb * 256) + lane * 2 + 1);
    const float4 u0 = __ldg(reinterpret_cast<const float4 *>(u + sb * 256) + lane * 2), u1 = __ldg(reinterpret_cast<const float4 *>(u + sb * 256) + lane * 2 + 1);
    const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    const float uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __fmul_rn(__fdiv_rn(gv[i], 1.0f + expf(-gv[i])), uv[i]);
    const Q8kLane ql = quant_q8k_values(v);
    reinterpret_cast<uint2 *>(q + sb * 256)[lane] = ql.packed;
    int s = ql.sum8;
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if ((lane & 3) == 0) bsums[sb * 8 + (lane >> 2)] = s;
    if (lane == 0) scales[sb] = ql.scale;
}

int ojas_silu_mul_q8k(ojas_b200_ctx *ctx, const float *g, const float *u, int8_t *q, float *scales, int32_t *bsums, size_t rows, size_t K) {
    const long long n_sb = (long long)rows * (long long)(K / 256);
    if (n_sb <= 0) return 0;
    const long long blocks = (n_sb + 7) / 8;
    if (blocks > 0x7fffffffLL) return ojas_fail(ctx, OJAS_B200_E_ARG, "silu_mul_q8k: too many super-blocks");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, silu_mul_q8k_kernel, g, u, q, scales, bsums, n_sb);
    if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "launch silu_mul_q8k: %s", cudaGetErrorString(e));
    ojas_count_launch(ctx, "silu_mul_q8k");
    return 0;
}

extern "C" int ojas_b200_silu_mul_q8k(ojas_b200_ctx *ctx, const float *g, const float *u, size_t M, size_t K, int8_t *q, float *scales,
                                      int32_t *bsums) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!g || !u || !q || !scales || !bsums) return ojas_fail(ctx, OJAS_B200_E_ARG, "silu_mul_q8k: null pointer");
    if (K == 0 || K % 256 != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "silu_mul_q8k: K=%zu must be a positive multiple of 256", K);
    if (((uintptr_t)g & 15) || ((uintptr_t)u & 15) || ((uintptr_t)q & 7)) return ojas_fail(ctx, OJAS_B200_E_ARG, "silu_mul_q8k: misaligned pointer");
    return ojas_silu_mul_q8k(ctx, g, u, q, scales, bsums, M, K);
}

extern "C" int ojas_b200_rmsnorm_q8k(ojas_b200_ctx *ctx, const float *x, const float *w, float eps, size_t M, size_t K, float *xn,
                                     int8_t *q, float *scales, int32_t *bsums) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!x || !w || !q || !scales || !bsums) return ojas_fail(ctx, OJAS_B200_E_ARG, "rmsnorm_q8k: null pointer");
    if (K == 0 || K % 256 != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "rmsnorm_q8k: K=%zu must be a positive multiple of 256", K);
    if (K * 4 > (size_t)ctx->smem_optin - 1024) return ojas_fail(ctx, OJAS_B200_E_LIMIT, "rmsnorm_q8k: K=%zu does not fit in shared memory", K);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)q & 7) || (xn && ((uintptr_t)xn & 15)))
        return ojas_fail(ctx, OJAS_B200_E_ARG, "rmsnorm_q8k: misaligned pointer");
    if (M == 0) return 0;
    if (M > 0x7fffffffu) return ojas_fail(ctx, OJAS_B200_E_ARG, "rmsnorm_q8k: too many rows");
    const size_t smem = K * 4;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(rmsnorm_q8k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "rmsnorm_q8k: shared memory %zu: %s", smem, cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)M);
    cfg.blockDim = dim3(K >= 4096 ? 512 : 256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, rmsnorm_q8k_kernel, x, w, eps, xn, q, scales, bsums, (int)K);
    if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "launch rmsnorm_q8k: %s", cudaGetErrorString(e));
    ojas_count_launch(ctx, "rmsnorm_q8k");
    return 0;
}
