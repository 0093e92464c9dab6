// Shared declarations of the B200 quantized-matmul library: the context object behind the
// C ABI, status plumbing, the repacked-weight layouts, and small device helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/ojas_b200.h"

// ---------------------------------------------------------------------------- context
struct ojas_b200_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    int smem_optin = 0;          // max dynamic shared memory per block (opt-in)
    uint64_t launches = 0;
    int gemv_mma = 1;            // batch GEMVs on the tensor-core loops: 0 never, 1 from 3 rows (K-quants) / 2 rows (Q8_0), 2 always
    int gemv_slim = 1;           // single-row Q4_K GEMV in the half-size kernel: 0 never, 1 for small matrices, 2 always
    int moe_gemm_rows = 0;       // expert FFN: grouped tensor-core GEMMs from this many rows per expert on average (0: never)
    int gemm_ksplit = 0;         // 0: choose the K split per shape; >0: force it
    int gemv_depth = 4;          // accepted and ignored (the GEMV ring has two stages)
    int pdl = 1;                 // launch GEMVs with programmatic dependent launch (overlap with the kernel before)
    void *act_scratch = nullptr;         // device scratch for a batch's Q8_K activations (values, scales, block sums)
    unsigned int *gemm_flags = nullptr;  // device words, one per GEMM output tile: "the tile has been stored" marks (see gemm_ts.cuh)
    unsigned int gemm_serial = 0;        // value that means "stored" for the GEMM launch in flight; never 0
    unsigned int *host_status = nullptr; // pinned host word written by kernels whose bounded waits ran out
    unsigned int *dev_status = nullptr;  // the same word as the device sees it
    char err[512] = {0};
};

constexpr size_t OJAS_GEMM_FLAG_WORDS = 65536;
// Activation scratch of a context: up to this many int8 values (8 rows of K = 32768), then one f32 scale per 256
// and one i32 sum per 32 of them.
constexpr size_t OJAS_ACT_SCRATCH_VALUES = 262144;
constexpr size_t OJAS_ACT_SCRATCH_BYTES = OJAS_ACT_SCRATCH_VALUES + OJAS_ACT_SCRATCH_VALUES / 256 * 4 + OJAS_ACT_SCRATCH_VALUES / 32 * 4;

int ojas_fail(ojas_b200_ctx *ctx, int code, const char *fmt, ...);

#define OJAS_CUDA(ctx, call)                                                                     \
    do {                                                                                         \
        cudaError_t e__ = (call);                                                                \
        if (e__ != cudaSuccess)                                                                  \
            return ojas_fail((ctx), OJAS_B200_E_CUDA, "%s: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

#define OJAS_LAUNCH_CHECK(ctx, what)                                                                  \
    do {                                                                                              \
        cudaError_t e__ = cudaGetLastError();                                                         \
        if (e__ != cudaSuccess)                                                                       \
            return ojas_fail((ctx), OJAS_B200_E_CUDA, "launch %s: %s", what, cudaGetErrorString(e__)); \
        (ctx)->launches++;                                                                            \
    } while (0)

// ---------------------------------------------------------------------------- layouts
// Repacked weights are a set of planes in one buffer; every plane starts on a 256-byte
// boundary and every row of every plane is a whole number of 16-byte units.
//
// Q4_K  (GGUF: 144 B per 256 weights: f16 d, f16 dmin, u8 sc[12], u8 qs[128])
//   plane qs : [N][K/256][128]  nibbles; within a super-block byte h*64 + c*16 + i holds
//              GGUF qs[c*32 + h*16 + i] (c = 64-weight chunk 0..3, h = 16-byte half), so the
//              four lanes that share a super-block read 64 contiguous bytes per load.
//   plane hdr: [N][K/256][16]   f16 d, f16 dmin, then the sixteen 6-bit scales / mins regrouped
//              per chunk: bytes 4 + 3c .. 6 + 3c hold the little-endian 24-bit group
//              s(2c) | s(2c+1) << 6 | m(2c) << 12 | m(2c+1) << 18  (same 96 bits as GGUF's sc[12]).
// Q6_K  (GGUF: 210 B per 256: u8 ql[128], u8 qh[64], i8 sc[16], f16 d)
//   plane lo : [N][K/256][128]  low nibbles; byte h*64 + c*16 + i: low nibble = weight
//              64c + 16h + i, high nibble = weight 64c + 32 + 16h + i.
//   plane hi : [N][K/256][64]   top two bits; byte c*16 + k*4 + i: bit field t (bits 2t, 2t+1)
//              = weight 64c + 16t + 4k + i.
//   plane sc : [N][K/256][16]   int8 sub-scales, GGUF order.
//   plane d  : [N][K/256]       f16 super-block scale.
// Q8_0  (GGUF: 34 B per 32: f16 d, i8 q[32])
//   plane q  : [N][K]           int8, natural order.
//   plane d  : [N][K/32]        f16.
struct WeightPlanes {
    const uint8_t *p0, *p1, *p2, *p3;
};

static inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

static inline int plane_offsets(uint32_t type, size_t N, size_t K, size_t off[5]) {
    size_t nsb = K / 256;
    off[0] = 0;
    switch (type) {
    case OJAS_B200_Q4_K:
        off[1] = align256(N * nsb * 128);
        off[2] = off[3] = off[4] = off[1] + align256(N * nsb * 16);
        return 0;
    case OJAS_B200_Q6_K:
        off[1] = align256(N * nsb * 128);
        off[2] = off[1] + align256(N * nsb * 64);
        off[3] = off[2] + align256(N * nsb * 16);
        off[4] = off[3] + align256(N * nsb * 2);
        return 0;
    case OJAS_B200_Q8_0:
        off[1] = align256(N * K);
        off[2] = off[3] = off[4] = off[1] + align256(N * (K / 32) * 2);
        return 0;
    default:
        return -1;
    }
}

static inline WeightPlanes weight_planes(uint32_t type, const void *w, size_t N, size_t K) {
    size_t off[5];
    plane_offsets(type, N, K, off);
    const uint8_t *b = (const uint8_t *)w;
    return WeightPlanes{b + off[0], b + off[1], b + off[2], b + off[3]};
}

// Planes of rows [row0, ...) of a stacked tensor (experts stacked along N, as the engine keeps them:
// crates/ojas-cuda/src/kernels/moe.rs:75-125 index `idx[j] * N + row`).
static inline WeightPlanes weight_planes_at(uint32_t type, const void *w, size_t n_total, size_t K, size_t row0) {
    WeightPlanes p = weight_planes(type, w, n_total, K);
    const size_t nsb = K / 256;
    switch (type) {
    case OJAS_B200_Q4_K: p.p0 += row0 * nsb * 128; p.p1 += row0 * nsb * 16; break;
    case OJAS_B200_Q6_K: p.p0 += row0 * nsb * 128; p.p1 += row0 * nsb * 64; p.p2 += row0 * nsb * 16; p.p3 += row0 * nsb * 2; break;
    default: p.p0 += row0 * K; p.p1 += row0 * (K / 32) * 2; break;
    }
    return p;
}

int ojas_gemv_grouped(ojas_b200_ctx *ctx, uint32_t type, const WeightPlanes &planes, const int8_t *q, const float *scales,
                      const int32_t *bsums, const int *row_index, const int *grp_count, const int *grp_offset, float *y,
                      size_t K, size_t N);

// Prefill-sized expert groups: f32 rows -> the GEMM's f16 activation format (Q8_K-quantized when `quant`), and the
// tensor-core GEMM over the rows [*grp_offset, + *grp_count) of xh / y (counts read on the device; y pre-zeroed).
int ojas_gemm_prep(ojas_b200_ctx *ctx, const float *x, void *xh, size_t rows, size_t K, bool quant);
int ojas_gemm_grouped(ojas_b200_ctx *ctx, uint32_t type, const void *xh, size_t x_rows, const WeightPlanes &wp, float *y, size_t K,
                      size_t N, size_t rows_bound, const int *grp_count, const int *grp_offset);

// ---------------------------------------------------------------------------- device helpers
#ifdef __CUDACC__
__device__ __forceinline__ uint4 ldg_stream_u4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Programmatic dependent launch: wait for the kernel before this one in the stream (a no-op
// when the launch did not ask for overlap), and let the kernel after this one start early.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)(h & 0xffffu)));
}

// round half away from zero, exactly (v - trunc(v) is exact in binary32), as Rust's
// f32::round does (crates/ojas-cpu/src/cpu_math.rs:557).
__device__ __forceinline__ float round_half_away(float v) {
    float r = truncf(v);
    float f = v - r;
    if (fabsf(f) >= 0.5f) r += copysignf(1.0f, v);
    return r;
}
#endif
