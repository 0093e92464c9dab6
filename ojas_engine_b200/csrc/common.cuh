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
    struct OjasProfile *prof = nullptr;  // per-launch event profiler (OJAS_B200_PROFILE=1 or option "profile"), null when off
    int gemv_mma = 1;            // Q4_K batches of 3..8 rows and expert groups on the tensor-core batch kernel (0: per-lane kernels only)
    int gemv_warps = 0;          // GEMV: warps per CTA (0: chosen per shape; otherwise 1..16)
    int gemv_kseg = 0;           // Q8_0 batches of 3..8 rows: K segments per launch (0: only when the whole K does not fit; 1: never; n: n when it divides K / 256)
    int gemv_stages = 0;         // GEMV: ring stages per warp (0: chosen per shape; otherwise 1..4)
    int moe_gemm_rows = 0;       // expert FFN: grouped tensor-core GEMMs from this many rows per expert on average (0: never)
    int gemm_ksplit = 0;         // 0: choose the K split per shape; >0: force it
    int pdl = 1;                 // launch GEMVs with programmatic dependent launch (overlap with the kernel before)
    int moe_i8 = 0;                      // 1: decode-sized Q4_K expert FFNs on the int8 tcgen05 kernel too (the prefill form always uses it)
    void *act_scratch = nullptr;         // device scratch for a batch's Q8_K activations (values, scales, block sums)
    void *reserved = nullptr;            // scratch the host reserved with ojas_b200_reserve (never grown inside a compute call)
    size_t reserved_bytes = 0;
    unsigned int *gemm_flags = nullptr;  // device words, one per GEMM output tile: "the tile has been stored" marks (see gemm_ts.cuh),
                                         // then one word: the value that means "stored" for the GEMM launch in flight (never 0)
    unsigned int *host_status = nullptr; // pinned host word written by kernels whose bounded waits ran out
    unsigned int *dev_status = nullptr;  // the same word as the device sees it
    char err[512] = {0};
};

constexpr size_t OJAS_GEMM_FLAG_WORDS = 65536;
// Activation scratch of a context: up to this many int8 values (8 rows of K = 32768), then one f32 scale per 256
// and one i32 sum per 32 of them.
constexpr size_t OJAS_ACT_SCRATCH_VALUES = 262144;
// (Q8_K rows of OJAS_ACT_SCRATCH_VALUES values need 292 KB; the three-term int8 rows of a Q8_0 batch, 3.125 bytes per
// value, up to 8 x 32768 values: 1 MiB covers both)
constexpr size_t OJAS_ACT_SCRATCH_BYTES = (size_t)1 << 20;
static_assert(OJAS_ACT_SCRATCH_VALUES + OJAS_ACT_SCRATCH_VALUES / 256 * 4 + OJAS_ACT_SCRATCH_VALUES / 32 * 4 <= OJAS_ACT_SCRATCH_BYTES, "Q8_K scratch");

int ojas_fail(ojas_b200_ctx *ctx, int code, const char *fmt, ...);

#define OJAS_CUDA(ctx, call)                                                                     \
    do {                                                                                         \
        cudaError_t e__ = (call);                                                                \
        if (e__ != cudaSuccess)                                                                  \
            return ojas_fail((ctx), OJAS_B200_E_CUDA, "%s: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

// Every launch of the library passes here: the launch counter and, when the profiler is on, an event behind the launch.
void ojas_count_launch(ojas_b200_ctx *ctx, const char *name);

#define OJAS_LAUNCH_CHECK(ctx, what)                                                                  \
    do {                                                                                              \
        cudaError_t e__ = cudaGetLastError();                                                         \
        if (e__ != cudaSuccess)                                                                       \
            return ojas_fail((ctx), OJAS_B200_E_CUDA, "launch %s: %s", what, cudaGetErrorString(e__)); \
        ojas_count_launch((ctx), what);                                                               \
    } while (0)

// ---------------------------------------------------------------------------- layouts
// A repacked weight is a grid of TILES: tile (u, s) holds rows 8u .. 8u+7 of super-block s (256 weights) and tiles are
// stored unit-major, [ceil(N/8)][K/256][tile]: everything one 8-row unit needs along K is one contiguous run, and four
// units (32 rows) of one super-block are four runs a row of tiles apart.  Inside a tile the data are 16-byte pieces,
// piece-major and row-minor: piece p of row r sits at byte (p * 8 + r) * 16, so eight lanes that own eight
// consecutive rows read 128 contiguous bytes per piece (coalesced from global memory, conflict-free from shared
// memory, and one bulk copy moves whole tiles).  Rows past N are zero blocks.  Every GGUF bit is kept.
//
// Q4_K  (GGUF: 144 B per 256 weights: f16 d, f16 dmin, u8 sc[12], u8 qs[128])          tile = 1152 B
//   pieces 0..7 : qs[16p .. 16p+15] in GGUF order: low nibbles = weights 64(p/2) + 16(p%2) + i, high nibbles the
//                 same + 32 (crates/ojas-formats/src/gguf.rs:1049-1056)
//   piece  8    : the block's first 16 bytes as they are: d, dmin, sc[12]
// Q5_K  (GGUF: 176 B per 256: f16 d, f16 dmin, u8 sc[12], u8 qh[32], u8 qs[128])      tile = 1408 B
//   pieces 0..8 : as Q4_K (qs, then the first 16 bytes of the block)
//   pieces 9, 10: qh[0..15], qh[16..31]: bit j of qh[l] is the fifth bit of weight l of sub-block j
//                 (crates/ojas-formats/src/gguf.rs:1060-1085)
// Q6_K  (GGUF: 210 B per 256: u8 ql[128], u8 qh[64], i8 sc[16], f16 d)                 tile = 1680 B
//   pieces 0..7 : low nibbles, piece h*4 + c, byte i: low nibble = weight 64c + 16h + i, high nibble = weight
//                 64c + 32 + 16h + i   (c = 64-weight chunk, h = 0, 1)
//   pieces 8..11: top two bits, piece 8 + c, byte b: bit field t (bits 2t, 2t+1) = weight 64c + 16t + b
//   piece  12   : the sixteen int8 sub-block scales, GGUF order
//   then 8 x f16 d, one per row, at byte 13 * 128 + 2r
// Q8_0  (GGUF: 34 B per 32: f16 d, i8 q[32]; eight blocks per 256 weights)             tile = 2176 B
//   pieces 0..15: q[16p .. 16p+15] of the 256 weights, natural order
//   piece  16   : the eight f16 block scales
// IQ4_NL (GGUF: 18 B per 32: f16 d, u8 qs[16]; eight blocks per 256 weights)          tile = 1152 B
//   pieces 0..7 : qs of block p: low nibbles = codebook indices of weights 32p + i, high nibbles of 32p + 16 + i
//                 (crates/ojas-formats/src/gguf.rs:796-812)
//   piece  8    : the eight f16 block scales
// IQ4_XS (GGUF: 136 B per 256: f16 d, u16 scales_h, u8 scales_l[4], u8 qs[128])       tile = 1088 B
//   pieces 0..7 : qs[16p .. 16p+15] = sub-block p: low nibbles = codebook indices of weights 32p + i, high nibbles
//                 of weights 32p + 16 + i (crates/ojas-formats/src/gguf.rs:814-840)
//   then 8 x 8 bytes, one per row, at byte 8 * 128 + 8r: the block's first eight bytes (d, scales_h, scales_l)
constexpr int OJAS_TILE_ROWS = 8;
__host__ __device__ constexpr int tile_bytes(uint32_t type) {
    return type == OJAS_B200_Q4_K ? 1152 : type == OJAS_B200_Q5_K ? 1408 : type == OJAS_B200_Q6_K ? 1680 : type == OJAS_B200_IQ4_XS ? 1088 : type == OJAS_B200_IQ4_NL ? 1152 : 2176;
}
// The formats whose CPU dot takes f32 activations (Q8_0: dot_q80, IQ4_NL: dot_iq4nl, IQ4_XS: dot_iq4xs): the GEMV stages them
// as three int8 terms.
__host__ __device__ constexpr bool f32_act_type(uint32_t type) { return type == OJAS_B200_Q8_0 || type == OJAS_B200_IQ4_XS || type == OJAS_B200_IQ4_NL; }
// Bytes of the leading pieces that hold quants only (what the GEMM stages per tile; scales come after them).
__host__ __device__ constexpr int tile_quant_bytes(uint32_t type) {
    return type == OJAS_B200_Q4_K || type == OJAS_B200_IQ4_XS || type == OJAS_B200_IQ4_NL ? 1024 : type == OJAS_B200_Q5_K ? 1408 : type == OJAS_B200_Q6_K ? 1536 : 2048;   // (Q5_K: the whole tile, its fifth bits lie behind the header)
}

#ifdef __CUDACC__
// Four index bytes of IQ4_NL / IQ4_XS (eight 4-bit indices into the sixteen int8 codebook values) looked up with byte
// permutes: lo = the values of the four low nibbles, hi = of the four high nibbles, as packed int8.
__device__ __forceinline__ void iq4_lookup8(uint32_t q, uint32_t &lo, uint32_t &hi) {
    constexpr uint32_t T0 = 0xBFAD9881u, T1 = 0xF6EADDCFu, T2 = 0x26190D01u, T3 = 0x71594535u;   // the codebook, four values per word
    const uint32_t a0 = __byte_perm(T0, T1, q), b0 = __byte_perm(T2, T3, q);
    const uint32_t v0 = __byte_perm(a0, b0, 0x3210u + ((q & 0x8888u) >> 1));          // values of nibbles 0..3
    const uint32_t qh = q >> 16;
    const uint32_t a1 = __byte_perm(T0, T1, qh), b1 = __byte_perm(T2, T3, qh);
    const uint32_t v1 = __byte_perm(a1, b1, 0x3210u + ((qh & 0x8888u) >> 1));         // values of nibbles 4..7
    lo = __byte_perm(v0, v1, 0x6420u);
    hi = __byte_perm(v0, v1, 0x7531u);
}
#endif

static inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }
static inline bool type_supported(uint32_t type) {
    return type == OJAS_B200_Q4_K || type == OJAS_B200_Q5_K || type == OJAS_B200_Q6_K || type == OJAS_B200_Q8_0 || type == OJAS_B200_IQ4_XS ||
           type == OJAS_B200_IQ4_NL;
}
static inline size_t tile_units(size_t N) { return (N + OJAS_TILE_ROWS - 1) / OJAS_TILE_ROWS; }
static inline size_t repacked_size(uint32_t type, size_t N, size_t K) { return align256(tile_units(N) * (K / 256) * (size_t)tile_bytes(type)); }

// First tile of rows [row0, ...) of a stacked tensor (experts stacked along N, as the engine keeps them:
// crates/ojas-cuda/src/kernels/moe.rs:75-125 index `idx[j] * N + row`).  row0 must be a multiple of 8.
static inline const uint8_t *weight_rows_at(uint32_t type, const void *w, size_t K, size_t row0) {
    return (const uint8_t *)w + (row0 / OJAS_TILE_ROWS) * (K / 256) * (size_t)tile_bytes(type);
}

// ---------------------------------------------------------------------------- tensor-parallel epilogue
// What a kernel needs to hand its results to the other ranks of a tensor-parallel group (tp.cu).  A receive window
// holds STAMPED values: each float travels as an 8-byte pair (its bits, the number of the step it belongs to),
// written with one 8-byte store, so a reader that sees the stamp of the step in flight has the value too: no flag,
// no fence, no grid-wide rendezvous, one NVLink crossing.  step == null everywhere outside a group.
constexpr int OJAS_TP_MAX_RANKS = 8;
struct TpPush {
    uint2 *dst[OJAS_TP_MAX_RANKS];         // this rank's place in every rank's window (the local one included), half 0
    const unsigned *step;                  // local word: the number of the step in flight (the stamp); its low bit
                                           // picks the half of the windows the step uses
    size_t half_pairs;                     // distance of half 1 from half 0 in a window, in pairs
    int n;                                 // destinations
};

// Scratch for a call that needs `bytes`: the reserved buffer when it is large enough, else the array built into the
// library when that is (gemm_tc.cu), else null with the error set.
void *ojas_scratch_for(ojas_b200_ctx *ctx, size_t bytes, const char *who);
int ojas_gemv_selected(ojas_b200_ctx *ctx, uint32_t type, int form, const float *x, const void *w, const uint32_t *sel, size_t sel_stride,
                       const float *alpha, float *y, size_t K, size_t N);
int ojas_silu_mul_inplace(ojas_b200_ctx *ctx, float *g, const float *u, size_t n);
int ojas_gemm_prep_q8k(ojas_b200_ctx *ctx, const int8_t *q, const float *scales, void *xh, size_t rows, size_t K);
size_t ojas_experts_i8_meta_bytes(size_t positions, size_t K);
int ojas_experts_i8_pack(ojas_b200_ctx *ctx, const int8_t *q, const float *scales, const int32_t *bsums, const int *row_index, size_t positions,
                         size_t K, int8_t *q_out, void *meta);
int ojas_experts_i8(ojas_b200_ctx *ctx, const uint8_t *w0, const uint8_t *w1, float *y0, float *y1, const int8_t *q, const void *meta,
                    size_t positions, const int *counts, const int *offsets, size_t E, size_t K, size_t N, int kparts, size_t part_stride, int tok);
int ojas_gemv_experts_batch(ojas_b200_ctx *ctx, uint32_t type, const uint8_t *w0, const uint8_t *w1, float *y0, float *y1, const int8_t *q,
                            const float *scales, const int32_t *bsums, const int *row_index, const int *counts, const int *offsets, size_t E,
                            size_t K, size_t N, size_t rows_hint);
int ojas_gemv_experts_kq(ojas_b200_ctx *ctx, uint32_t type, const uint8_t *w0, const uint8_t *w1, float *y0, float *y1, const int8_t *q,
                         const float *scales, const int32_t *bsums, const int *row_index, const int *counts, const int *offsets, size_t E, size_t K,
                         size_t N, size_t rows_hint);
int ojas_gemv_grouped(ojas_b200_ctx *ctx, uint32_t type, const uint8_t *w, const int8_t *q, const float *scales,
                      const int32_t *bsums, const int *row_index, const int *grp_count, const int *grp_offset, float *y,
                      size_t K, size_t N);

// Prefill-sized expert groups: f32 rows -> the GEMM's f16 activation format (Q8_K-quantized when `quant`), and the
// tensor-core GEMM over the rows [*grp_offset, + *grp_count) of xh / y (counts read on the device; y pre-zeroed).
int ojas_gemm_prep(ojas_b200_ctx *ctx, const float *x, void *xh, size_t rows, size_t K, bool quant);
int ojas_gemm_grouped(ojas_b200_ctx *ctx, uint32_t type, const void *xh, size_t x_rows, const uint8_t *w, float *y, size_t K,
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
