// Prefill GEMM on the 5th-generation tensor cores: y[M,N] (+)= x[M,K] * W[N,K]^T over repacked
// GGUF weights.  Replaces gemm_mm_{q4l,q6k,q8_0} and their split-K forms
// (crates/ojas-cuda/src/kernels/gemm_q.rs:291-590), with the arithmetic contract of the CPU
// path: for Q4_K / Q6_K the activations are first quantized to Q8_K (quant_q8k,
// crates/ojas-cpu/src/cpu_math.rs:545-563) and enter the MMA as f16(sx * q); for Q8_0 they
// enter as f16(x) (dot_q80 keeps f32 activations, :971-981).  Weights are dequantized tile by
// tile to f16 (the reference GEMM does the same in shared memory for mma.sync, gemm_q.rs:6-12)
// and accumulated in fp32 in tensor memory.
//
// One CTA computes 128 weight rows x BN tokens:
//   UMMA M = 128 weight rows  (A operand: dequantized W tile, written to TMEM by the dequantizing warps)
//   UMMA N = BN tokens        (B operand: f16 activation tile in shared memory, loaded by TMA,
//                              K-major with the 128-byte swizzle)
//   accumulator D[128 x BN] fp32 in TMEM; TMEM lane = weight row, column = token, so the
//   epilogue's 32 lanes store 32 consecutive outputs of one token: coalesced without a
//   shared-memory transpose.
// The kernel (gemm_ts.cuh) is persistent: one CTA per SM walks its share of the work list.
// Every wait on an mbarrier is bounded: a wait that runs out sets the context's status word,
// raises the CTA's abort flag, and every role falls through to the common teardown (TMEM is
// always released).
#include <cuda.h>

#include "act_quant.cuh"
#include "tc_util.cuh"

namespace {

constexpr int BM = 128;            // weight rows per CTA
constexpr int BK = 64;             // k per stage = one 64-weight chunk = 128 bytes of f16
constexpr int WQ_BUFS_MAX = 3;
// One staged raw tile = one super-block x 128 rows = the quant pieces of sixteen 8-row tiles of the weight layout
// (common.cuh): Q4_K 16 KB, Q6_K 24 KB, Q8_0 32 KB.  Row r of 8-row tile t keeps its 16-byte piece p at
// t * tile_quant_bytes + (p * 8 + r) * 16, so a warp's 32 consecutive rows read a piece without bank conflicts.
__host__ __device__ constexpr int wq_bytes(int type) { return (BM / OJAS_TILE_ROWS) * tile_quant_bytes((uint32_t)type); }
// raw tiles in flight: three, or two of the large Q8_0 tiles (so that four activation stages still fit)
__host__ __device__ constexpr int wq_bufs(int type) { return type == OJAS_B200_Q8_0 || type == OJAS_B200_Q5_K ? 2 : 3; }

struct GemmArgs {
    const uint8_t *w;    // first tile of the weight rows (layout: common.cuh)
    float *y;
    int M, N, K;
    int accum;           // 1: y += result
    int ksplit;          // 0: K ranges balanced across the CTAs; S > 0: every tile's K range cut into S pieces
    int e2;              // balanced split: cost of a tile's end in half super-blocks (see ts_share_begin)
    const int *grp_count;    // grouped form (experts): the row count and the first row of the group are read on the
    const int *grp_offset;   // device; M is then only an upper bound used to choose the tile width
    unsigned *flags;     // per-tile "stored" marks (null: split tiles are added into a zeroed y instead)
    const unsigned *serial_word;   // device word holding the value that marks a tile as stored in this launch
    int y_tma;           // 1: the epilogue writes y through bulk tensor stores (needs N % 4 == 0 and y on 16 bytes)
    unsigned *status;    // device-visible status word of the context
};

// kind::f16, A and B f16 K-major, D f32, M = 128, N = bn.
__host__ __device__ constexpr uint32_t umma_idesc(int bn) {
    return (1u << 4) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// Zero 32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_zero32(uint32_t taddr) {
    const uint32_t z = 0u;
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, "
                 "%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
                 ::"r"(taddr), "r"(z) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- dequantizers (one row, 32 weights)
// A stage is 64 weights per weight row; two threads share a row: `half` 0 produces weights 0..31 of the
// 64-chunk, half 1 weights 32..63, each as sixteen f16 pairs o[0..15] in k order (o[i] = k 2i, 2i + 1 of
// the half).  For the K-quants the k order inside every group of four is (0, 2, 1, 3): that is the order
// the nibble pairs fall out of a 32-bit word, and the activation tile is written in the same order (see
// gemm_prep_kernel), so the dot is unchanged.
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

// Q4_K: A, B = the chunk's two 16-byte nibble pieces (low nibbles = weights 0..31, high = 32..63),
// H = the block's GGUF header (d, dmin, sc[12]), c = chunk index inside the super-block.  The integer -> f16
// step (OR the value into the mantissa of 1024.0, subtract 1024, one fused multiply-add with the scale and the
// min term) is the one the reference's loaders use (crates/ojas-cuda/src/kernels/gemm_q.rs:104-119).
__device__ __forceinline__ void dequant_q4k_half(const uint4 &A, const uint4 &B, const uint4 &H, int c, int half, uint32_t (&o)[16]) {
    // 6-bit scale and min of sub-block j = 2c + half (get_scale_min_k4, crates/ojas-formats/src/gguf.rs:1132-1140)
    const int j = 2 * c + half;
    uint32_t sv, mv;
    if (j < 4) {
        sv = (H.y >> (8 * j)) & 63u;
        mv = (H.z >> (8 * j)) & 63u;
    } else {
        const uint32_t t = H.w >> (8 * (j - 4));
        sv = (t & 0xFu) | (((H.y >> (8 * (j - 4) + 6)) & 3u) << 4);
        mv = ((t >> 4) & 0xFu) | (((H.z >> (8 * (j - 4) + 6)) & 3u) << 4);
    }
    const float d = f16_bits_to_f32(H.x), dmin = f16_bits_to_f32(H.x >> 16);
    const __half2 ds = __float2half2_rn(d * (float)sv);
    const __half2 nm = __float2half2_rn(-(dmin * (float)mv));
    const __half2 k1024 = u32_as_h2(0x64006400u);
    const int nsh = 4 * half;
    const uint32_t w[8] = {A.x >> nsh, A.y >> nsh, A.z >> nsh, A.w >> nsh, B.x >> nsh, B.y >> nsh, B.z >> nsh, B.w >> nsh};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const __half2 t0 = u32_as_h2((w[i] & 0x000f000fu) | 0x64006400u);          // weights (4i, 4i+2)
        const __half2 t1 = u32_as_h2(((w[i] >> 8) & 0x000f000fu) | 0x64006400u);   // weights (4i+1, 4i+3)
        o[2 * i] = h2_as_u32(__hfma2(__hsub2(t0, k1024), ds, nm));
        o[2 * i + 1] = h2_as_u32(__hfma2(__hsub2(t1, k1024), ds, nm));
    }
}

// Q5_K (crates/ojas-formats/src/gguf.rs:1060-1085): Q4_K with a fifth bit per weight, bit j = 2c + half of qh[l] for weight l
// of the sub-block; Qa, Qb = qh[0..15], qh[16..31].  The bit lands on value 16 of the mantissa before the subtraction.
__device__ __forceinline__ void dequant_q5k_half(const uint4 &A, const uint4 &B, const uint4 &Qa, const uint4 &Qb, const uint4 &H, int c, int half,
                                                 uint32_t (&o)[16]) {
    const int j = 2 * c + half;
    uint32_t sv, mv;
    if (j < 4) {
        sv = (H.y >> (8 * j)) & 63u;
        mv = (H.z >> (8 * j)) & 63u;
    } else {
        const uint32_t t = H.w >> (8 * (j - 4));
        sv = (t & 0xFu) | (((H.y >> (8 * (j - 4) + 6)) & 3u) << 4);
        mv = ((t >> 4) & 0xFu) | (((H.z >> (8 * (j - 4) + 6)) & 3u) << 4);
    }
    const float d = f16_bits_to_f32(H.x), dmin = f16_bits_to_f32(H.x >> 16);
    const __half2 ds = __float2half2_rn(d * (float)sv);
    const __half2 nm = __float2half2_rn(-(dmin * (float)mv));
    const __half2 k1024 = u32_as_h2(0x64006400u);
    const int nsh = 4 * half;
    const uint32_t w[8] = {A.x >> nsh, A.y >> nsh, A.z >> nsh, A.w >> nsh, B.x >> nsh, B.y >> nsh, B.z >> nsh, B.w >> nsh};
    const uint32_t qh[8] = {Qa.x >> j, Qa.y >> j, Qa.z >> j, Qa.w >> j, Qb.x >> j, Qb.y >> j, Qb.z >> j, Qb.w >> j};   // bit 0 of every byte = this sub-block's
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const __half2 t0 = u32_as_h2((w[i] & 0x000f000fu) | ((qh[i] & 0x00010001u) << 4) | 0x64006400u);                 // weights (4i, 4i+2)
        const __half2 t1 = u32_as_h2(((w[i] >> 8) & 0x000f000fu) | (((qh[i] >> 8) & 0x00010001u) << 4) | 0x64006400u);    // weights (4i+1, 4i+3)
        o[2 * i] = h2_as_u32(__hfma2(__hsub2(t0, k1024), ds, nm));
        o[2 * i + 1] = h2_as_u32(__hfma2(__hsub2(t1, k1024), ds, nm));
    }
}

// Q6_K: A, B = low nibbles (same arrangement as Q4_K), Hh = the chunk's 16 bytes of top bits,
// sc4 = the chunk's four int8 sub-scales, dbits = f16 d.  Value = d * sc * (q - 32).  half 0
// handles the groups t = 0, 1 (low nibbles of A, B), half 1 the groups 2, 3 (high nibbles).
__device__ __forceinline__ void dequant_q6k_half(const uint4 &A, const uint4 &B, const uint4 &Hh, uint32_t sc4, uint32_t dbits,
                                                 int half, uint32_t (&o)[16]) {
    const float d = f16_bits_to_f32(dbits);
    const int t0i = 2 * half;
    const __half2 dscA = __float2half2_rn(d * (float)(int)(signed char)((sc4 >> (8 * t0i)) & 0xffu));
    const __half2 dscB = __float2half2_rn(d * (float)(int)(signed char)((sc4 >> (8 * t0i + 8)) & 0xffu));
    const __half2 k1056 = u32_as_h2(0x64206420u);   // 1024 + 32
    const int nsh = 4 * half;
    const uint32_t Aw[4] = {A.x >> nsh, A.y >> nsh, A.z >> nsh, A.w >> nsh};
    const uint32_t Bw[4] = {B.x >> nsh, B.y >> nsh, B.z >> nsh, B.w >> nsh};
    // top-bit fields: group t uses bits (2t, 2t+1) of every byte; bring them to bits 4, 5 of each 16-bit lane
    const uint32_t Hw[4] = {Hh.x >> nsh, Hh.y >> nsh, Hh.z >> nsh, Hh.w >> nsh};   // half 1: fields 2, 3 move to 0, 1
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t h = Hw[k];
        const uint32_t a0 = (Aw[k] & 0x000f000fu) | ((h << 4) & 0x00300030u), a1 = ((Aw[k] >> 8) & 0x000f000fu) | ((h >> 4) & 0x00300030u);
        const uint32_t b0 = (Bw[k] & 0x000f000fu) | ((h << 2) & 0x00300030u), b1 = ((Bw[k] >> 8) & 0x000f000fu) | ((h >> 6) & 0x00300030u);
        o[2 * k] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(a0 | 0x64006400u), k1056), dscA));
        o[2 * k + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(a1 | 0x64006400u), k1056), dscA));
        o[8 + 2 * k] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(b0 | 0x64006400u), k1056), dscB));
        o[8 + 2 * k + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(b1 | 0x64006400u), k1056), dscB));
    }
}

// Q8_0: one 32-weight block (two 16-byte pieces of int8, one f16 scale).  Natural k order.
__device__ __forceinline__ void dequant_q80_half(const uint4 &q0, const uint4 &q1, uint32_t dbits, uint32_t (&o)[16]) {
    const __half2 k1152 = u32_as_h2(0x64806480u);   // 1024 + 128
    const __half2 dd = __half2half2(__ushort_as_half((unsigned short)(dbits & 0xffffu)));
#pragma unroll
    for (int p = 0; p < 2; p++) {
        const uint4 q = p == 0 ? q0 : q1;
        const uint32_t w[4] = {q.x ^ 0x80808080u, q.y ^ 0x80808080u, q.z ^ 0x80808080u, q.w ^ 0x80808080u};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            o[8 * p + 2 * i] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(w[i], 0x64646464u, 0x4140)), k1152), dd));
            o[8 * p + 2 * i + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(w[i], 0x64646464u, 0x4342)), k1152), dd));
        }
    }
}

// IQ4_XS / IQ4_NL: one 32-weight group (sixteen index bytes: low nibbles = weights 0..15, high nibbles = 16..31), scale dl
// (IQ4_XS: d * (ls - 32) rounded to f16; IQ4_NL: the block's f16 d).  The codebook values come out of the lookup as int8
// and take the Q8_0 route into f16.  Natural k order.
__device__ __forceinline__ void dequant_iq4_half(const uint4 &Q, __half dl, uint32_t (&o)[16]) {
    const __half2 k1152 = u32_as_h2(0x64806480u);   // 1024 + 128
    const __half2 dd = __half2half2(dl);
    const uint32_t q[4] = {Q.x, Q.y, Q.z, Q.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t lo, hi;
        iq4_lookup8(q[i], lo, hi);
        lo ^= 0x80808080u;
        hi ^= 0x80808080u;
        o[2 * i] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(lo, 0x64646464u, 0x4140)), k1152), dd));
        o[2 * i + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(lo, 0x64646464u, 0x4342)), k1152), dd));
        o[8 + 2 * i] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(hi, 0x64646464u, 0x4140)), k1152), dd));
        o[8 + 2 * i + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(hi, 0x64646464u, 0x4342)), k1152), dd));
    }
}

#include "gemm_ts.cuh"

// ---------------------------------------------------------------- activation preparation
// x f32 [M, K] -> xh f16 [M, K].  QUANT: xh = f16(sx * q) with (sx, q) = quant_q8k(x), written
// in the k order the K-quant dequantizers produce ((0, 2, 1, 3) inside every group of four).
// Otherwise xh = f16(x) in natural order (Q8_0).  One warp per 256 values.
// XIN = float or __half: the split-K entries of the engine hand over activations that are f16 already
// (crates/ojas-cuda/src/kernels/gemm_q.rs:537-556).
template <bool QUANT, typename XIN>
__global__ void __launch_bounds__(256) gemm_prep_kernel(const XIN *x, __half *xh, long long n_sb, unsigned *serial_word) {
    const int lane = threadIdx.x & 31;
    if (serial_word && blockIdx.x == 0 && threadIdx.x == 0) {     // a fresh tile-mark value for the GEMM behind this kernel, never 0
        const unsigned v = *serial_word + 1u;
        *serial_word = v ? v : 1u;
    }
    const long long sb = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    grid_launch_dependents();   // the GEMM behind this kernel may begin its set-up; it waits for this grid before it reads xh
    if (sb >= n_sb) return;
    float v[8];
    if (sizeof(XIN) == 2) {                 // f16 in: widen (exact), then the same steps as for f32
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(x + sb * 256) + lane);
        const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) { const float2 f = __half22float2(h2[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
        if (QUANT) {
            const Q8kLane ql = quant_q8k_values(v);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t word = i < 4 ? ql.packed.x : ql.packed.y;
                v[i] = __fmul_rn(ql.scale, (float)(int)(signed char)((word >> (8 * (i & 3))) & 0xffu));
            }
        }
    } else if (QUANT) {
        const Q8kLane ql = quant_q8k_warp(reinterpret_cast<const float *>(x) + sb * 256, lane);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t word = i < 4 ? ql.packed.x : ql.packed.y;
            v[i] = __fmul_rn(ql.scale, (float)(int)(signed char)((word >> (8 * (i & 3))) & 0xffu));
        }
    } else {
        const float4 p = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + sb * 256) + lane * 2);
        const float4 q = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + sb * 256) + lane * 2 + 1);
        v[0] = p.x; v[1] = p.y; v[2] = p.z; v[3] = p.w; v[4] = q.x; v[5] = q.y; v[6] = q.z; v[7] = q.w;
    }
    uint4 out;
    if (QUANT) {
        out.x = h2_as_u32(__floats2half2_rn(v[0], v[2])); out.y = h2_as_u32(__floats2half2_rn(v[1], v[3]));
        out.z = h2_as_u32(__floats2half2_rn(v[4], v[6])); out.w = h2_as_u32(__floats2half2_rn(v[5], v[7]));
    } else {
        out.x = h2_as_u32(__floats2half2_rn(v[0], v[1])); out.y = h2_as_u32(__floats2half2_rn(v[2], v[3]));
        out.z = h2_as_u32(__floats2half2_rn(v[4], v[5])); out.w = h2_as_u32(__floats2half2_rn(v[6], v[7]));
    }
    reinterpret_cast<uint4 *>(xh + sb * 256)[lane] = out;
}

// The same tile source from activations that are Q8_K already (q int8 [rows, K], scales f32 per 256): f16(scale * q) in
// the K-quant k order.  One warp per 256 values.
__global__ void __launch_bounds__(256) gemm_prep_q8k_kernel(const int8_t *q, const float *scales, __half *xh, long long n_sb) {
    const int lane = threadIdx.x & 31;
    const long long sb = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    grid_launch_dependents();
    grid_dependency_wait();
    if (sb >= n_sb) return;
    const uint2 w = __ldg(reinterpret_cast<const uint2 *>(q + sb * 256) + lane);
    const float sx = __ldg(scales + sb);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __fmul_rn(sx, (float)(int)(signed char)(((i < 4 ? w.x : w.y) >> (8 * (i & 3))) & 0xffu));
    uint4 out;
    out.x = h2_as_u32(__floats2half2_rn(v[0], v[2])); out.y = h2_as_u32(__floats2half2_rn(v[1], v[3]));
    out.z = h2_as_u32(__floats2half2_rn(v[4], v[6])); out.w = h2_as_u32(__floats2half2_rn(v[5], v[7]));
    reinterpret_cast<uint4 *>(xh + sb * 256)[lane] = out;
}

// ---------------------------------------------------------------- host side
size_t gemm_ts_smem_bytes(int bn, int type) {
    return 1024 + (size_t)ts_b_stages(bn, type) * bn * BK * 2 + (size_t)wq_bufs(type) * wq_bytes(type) +
           TS_EPI_WARPS * TS_EPI_TILE_BYTES + TS_BAR_BYTES;
}

template <int BN, int TYPE>
int launch_gemm_ts_bn(ojas_b200_ctx *ctx, const CUtensorMap &tmap, const CUtensorMap &tmap_w, const CUtensorMap &tmap_y, const GemmArgs &args, dim3 grid) {
    auto kernel = gemm_ts_kernel<BN, TYPE>;
    const size_t smem = gemm_ts_smem_bytes(BN, TYPE);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: shared memory %zu: %s", smem, cudaGetErrorString(e));
    // programmatic dependent launch: the kernel's set-up, weight loads and dequantization overlap the tail of the
    // activation-preparation kernel; only the thread that loads the prepared activations waits for it
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(TS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, kernel, tmap, tmap_w, tmap_y, args);
    if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "launch gemm_ts: %s", cudaGetErrorString(e));
    OJAS_LAUNCH_CHECK(ctx, "gemm_ts");
    return 0;
}

template <int TYPE>
int launch_gemm_ts_type(ojas_b200_ctx *ctx, int bn, const CUtensorMap &tmap, const CUtensorMap &tmap_w, const CUtensorMap &tmap_y, const GemmArgs &args, dim3 grid) {
    switch (bn) {
    case 32: return launch_gemm_ts_bn<32, TYPE>(ctx, tmap, tmap_w, tmap_y, args, grid);
    case 64: return launch_gemm_ts_bn<64, TYPE>(ctx, tmap, tmap_w, tmap_y, args, grid);
    case 128: return launch_gemm_ts_bn<128, TYPE>(ctx, tmap, tmap_w, tmap_y, args, grid);
    default: return launch_gemm_ts_bn<256, TYPE>(ctx, tmap, tmap_w, tmap_y, args, grid);
    }
}

}  // namespace

extern "C" size_t ojas_b200_gemm_workspace_bytes(size_t M, size_t K) { return align256(M * K * 2); }

// Token-tile width for a shape (the widest tile the token count fills) and the K split: 0 = balanced
// (every CTA gets the same number of super-blocks), or the forced number of K ranges per tile.
static void gemm_plan(ojas_b200_ctx *ctx, size_t M, size_t K, int &bn, int &ksplit) {
    bn = M > 128 ? 256 : M > 64 ? 128 : M > 32 ? 64 : 32;
    ksplit = ctx->gemm_ksplit > 0 ? ctx->gemm_ksplit : 0;
    if ((size_t)ksplit > K / 256) ksplit = (int)(K / 256);   // K ranges are whole super-blocks
}

static int gemm_launch(ojas_b200_ctx *ctx, uint32_t type, const __half *xh, size_t x_rows, const uint8_t *w, float *y,
                       size_t K, size_t N, size_t M, int accum, const int *grp_count, const int *grp_offset);

static int gemm_entry(ojas_b200_ctx *ctx, uint32_t type, const void *x, bool x_is_f16, const void *w, float *y, size_t K, size_t N, size_t M,
                      int accum, void *workspace, size_t workspace_bytes);

extern "C" int ojas_b200_gemm(ojas_b200_ctx *ctx, uint32_t type, const float *x, const void *w, float *y, size_t K, size_t N,
                              size_t M, int accum, void *workspace, size_t workspace_bytes) {
    return gemm_entry(ctx, type, x, false, w, y, K, N, M, accum, workspace, workspace_bytes);
}

// The same with f16 activations [M, K] (the engine's split-K entries take them that way): widened exactly, then the
// same arithmetic as ojas_b200_gemm.
extern "C" int ojas_b200_gemm_f16(ojas_b200_ctx *ctx, uint32_t type, const void *xh, const void *w, float *y, size_t K, size_t N,
                                  size_t M, int accum, void *workspace, size_t workspace_bytes) {
    return gemm_entry(ctx, type, xh, true, w, y, K, N, M, accum, workspace, workspace_bytes);
}

static int gemm_entry(ojas_b200_ctx *ctx, uint32_t type, const void *x, bool x_is_f16, const void *w, float *y, size_t K, size_t N, size_t M,
                      int accum, void *workspace, size_t workspace_bytes) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!type_supported(type))
        return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: unsupported GGUF type %u", type);
    if (!x || !w || !y || !workspace) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: null pointer");
    if (K == 0 || K % 256 != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: K=%zu must be a positive multiple of 256", K);
    if (N == 0 || M == 0 || N > 0x7fffffffu || M > 0x7fffffffu) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: M=%zu N=%zu out of range", M, N);
    if (workspace_bytes < ojas_b200_gemm_workspace_bytes(M, K))
        return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: workspace of %zu bytes, %zu needed", workspace_bytes, ojas_b200_gemm_workspace_bytes(M, K));
    if (((uintptr_t)w & 127) || ((uintptr_t)workspace & 255) || ((uintptr_t)x & 15))
        return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: misaligned pointer (weights 128 bytes, workspace 256 bytes, x 16 bytes)");
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: cuTensorMapEncodeTiled is not available from the driver");

    // 1. activations -> f16 tile source
    __half *xh = (__half *)workspace;
    const long long n_sb = (long long)M * (long long)(K / 256);
    const long long blocks = (n_sb + 7) / 8;
    if (blocks > 0x7fffffffLL) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: activation matrix too large");
    unsigned *serial = ctx->gemm_flags + OJAS_GEMM_FLAG_WORDS;
    if (x_is_f16) {
        if (f32_act_type(type)) gemm_prep_kernel<false, __half><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const __half *)x, xh, n_sb, serial);
        else gemm_prep_kernel<true, __half><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const __half *)x, xh, n_sb, serial);
    } else {
        if (f32_act_type(type)) gemm_prep_kernel<false, float><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const float *)x, xh, n_sb, serial);
        else gemm_prep_kernel<true, float><<<(unsigned)blocks, 256, 0, ctx->stream>>>((const float *)x, xh, n_sb, serial);
    }
    OJAS_LAUNCH_CHECK(ctx, "gemm_prep");

    return gemm_launch(ctx, type, xh, M, (const uint8_t *)w, y, K, N, M, accum, nullptr, nullptr);
}

// Tensor maps, plan and launch over prepared f16 activations xh [x_rows][K].  Grouped form (grp_count != null):
// the rows of the group are xh[*grp_offset .. + *grp_count) and go to y[*grp_offset ..); M is an upper bound
// of the count; y must be zero where tiles can be split (the caller clears it) and is written with per-lane
// stores, which can stop at the group's last row.
static int gemm_launch(ojas_b200_ctx *ctx, uint32_t type, const __half *xh, size_t x_rows, const uint8_t *w, float *y,
                       size_t K, size_t N, size_t M, int accum, const int *grp_count, const int *grp_offset) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: cuTensorMapEncodeTiled is not available from the driver");
    const bool grouped = grp_count != nullptr;
    // plan + tensor map over xh [x_rows][K halves], box = 64 halves x bn rows, 128-byte swizzle
    int bn, ksplit;
    gemm_plan(ctx, M, K, bn, ksplit);
    if (grouped) ksplit = 0;
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)x_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)bn};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)xh, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: cuTensorMapEncodeTiled failed (%d)", (int)cr);

    // the weight's quant pieces as a 4-D byte tensor: 128 bytes (one piece of the 8 rows of a tile) x pieces x
    // super-blocks x 8-row units; box = every quant piece of one super-block of sixteen units = 128 rows
    CUtensorMap tmap_w = tmap;
    {
        const size_t tb = (size_t)tile_bytes(type), pieces = (size_t)tile_quant_bytes(type) / 128;
        const cuuint64_t wdims[4] = {128, (cuuint64_t)pieces, (cuuint64_t)(K / 256), (cuuint64_t)tile_units(N)};
        const cuuint64_t wstrides[3] = {128, (cuuint64_t)tb, (cuuint64_t)((K / 256) * tb)};
        const cuuint32_t wbox[4] = {128, (cuuint32_t)pieces, 1, (cuuint32_t)(BM / OJAS_TILE_ROWS)};
        const cuuint32_t westr[4] = {1, 1, 1, 1};
        cr = encode(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void *)w, wdims, wstrides, wbox, westr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: cuTensorMapEncodeTiled (weights) failed (%d)", (int)cr);
    }

    // y as a tensor [M rows][N floats], box = 32 floats x 16 rows (one epilogue warp's staging tile)
    CUtensorMap tmap_y = tmap;
    const bool y_tma = !grouped && (N % 4 == 0) && (((uintptr_t)y & 15) == 0);
    if (y_tma) {
        const cuuint64_t ydims[2] = {(cuuint64_t)N, (cuuint64_t)M};
        const cuuint64_t ystrides[1] = {(cuuint64_t)N * 4};
        const cuuint32_t ybox[2] = {32, 16};
        cr = encode(&tmap_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)y, ydims, ystrides, ybox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: cuTensorMapEncodeTiled (output) failed (%d)", (int)cr);
    }

    GemmArgs args{};
    args.y_tma = y_tma ? 1 : 0;
    args.w = w;
    args.grp_count = grp_count;
    args.grp_offset = grp_offset;
    args.y = y;
    args.M = (int)M; args.N = (int)N; args.K = (int)K;
    args.accum = accum ? 1 : 0;
    args.ksplit = ksplit;
    args.status = ctx->dev_status;
    {
        const size_t tiles = ((N + BM - 1) / BM) * ((M + bn - 1) / bn), nsb = K / 256;
        const size_t units = args.ksplit ? tiles * (size_t)args.ksplit : tiles * nsb;
        const size_t ctas = (units < (size_t)ctx->sm_count && !grouped) ? units : (size_t)ctx->sm_count;
        args.e2 = bn > 128 ? 6 : 0;      // one accumulator: the drain is exposed; two: it overlaps the next tile
        bool partial = args.ksplit > 1;
        if (!args.ksplit)
            for (size_t b = 1; b < ctas && !partial; b++)
                partial = (ts_share_begin((long long)tiles, (int)nsb, args.e2, (long long)b, (long long)ctas) % (long long)nsb) != 0;
        if (grouped) {
            // (the tile count is only known on the device: every SM gets a CTA)
        } else if (partial && !accum) {
            // A tile whose K range is split over CTAs: either the piece with the tile's last super-block stores
            // and marks the tile and the others add after the mark (no zeroing of y), or y is zeroed and every
            // piece adds.
            if (y_tma && !args.ksplit && tiles <= OJAS_GEMM_FLAG_WORDS) {
                args.flags = ctx->gemm_flags;
                args.serial_word = ctx->gemm_flags + OJAS_GEMM_FLAG_WORDS;   // advanced by the preparation kernel of this call
            } else {
                OJAS_CUDA(ctx, cudaMemsetAsync(y, 0, M * N * sizeof(float), ctx->stream));
            }
        }
        const dim3 grid_ts((unsigned)ctas);
        if (type == OJAS_B200_Q4_K) return launch_gemm_ts_type<OJAS_B200_Q4_K>(ctx, bn, tmap, tmap_w, tmap_y, args, grid_ts);
        if (type == OJAS_B200_Q6_K) return launch_gemm_ts_type<OJAS_B200_Q6_K>(ctx, bn, tmap, tmap_w, tmap_y, args, grid_ts);
        if (type == OJAS_B200_Q5_K) return launch_gemm_ts_type<OJAS_B200_Q5_K>(ctx, bn, tmap, tmap_w, tmap_y, args, grid_ts);
        if (type == OJAS_B200_IQ4_XS) return launch_gemm_ts_type<OJAS_B200_IQ4_XS>(ctx, bn, tmap, tmap_w, tmap_y, args, grid_ts);
        if (type == OJAS_B200_IQ4_NL) return launch_gemm_ts_type<OJAS_B200_IQ4_NL>(ctx, bn, tmap, tmap_w, tmap_y, args, grid_ts);
        return launch_gemm_ts_type<OJAS_B200_Q8_0>(ctx, bn, tmap, tmap_w, tmap_y, args, grid_ts);
    }
}

// ---------------------------------------------------------------- pieces the expert FFN uses
int ojas_gemm_prep(ojas_b200_ctx *ctx, const float *x, void *xh, size_t rows, size_t K, bool quant) {
    const long long n_sb = (long long)rows * (long long)(K / 256);
    const long long blocks = (n_sb + 7) / 8;
    if (blocks <= 0) return 0;
    if (blocks > 0x7fffffffLL) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: activation matrix too large");
    if (quant) gemm_prep_kernel<true, float><<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, (__half *)xh, n_sb, nullptr);
    else gemm_prep_kernel<false, float><<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, (__half *)xh, n_sb, nullptr);
    OJAS_LAUNCH_CHECK(ctx, "gemm_prep");
    return 0;
}

int ojas_gemm_prep_q8k(ojas_b200_ctx *ctx, const int8_t *q, const float *scales, void *xh, size_t rows, size_t K) {
    const long long n_sb = (long long)rows * (long long)(K / 256);
    const long long blocks = (n_sb + 7) / 8;
    if (blocks <= 0) return 0;
    if (blocks > 0x7fffffffLL) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: activation matrix too large");
    gemm_prep_q8k_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(q, scales, (__half *)xh, n_sb);
    OJAS_LAUNCH_CHECK(ctx, "gemm_prep_q8k");
    return 0;
}

int ojas_gemm_grouped(ojas_b200_ctx *ctx, uint32_t type, const void *xh, size_t x_rows, const uint8_t *w, float *y, size_t K,
                      size_t N, size_t rows_bound, const int *grp_count, const int *grp_offset) {
    return gemm_launch(ctx, type, (const __half *)xh, x_rows, w, y, K, N, rows_bound, 0, grp_count, grp_offset);
}

// ---------------------------------------------------------------- GEMM without a caller workspace
// Some hosts of this library cannot hand over scratch memory: a plugin loaded into an engine whose
// allocator is closed to it, or a caller inside a region where cudaMalloc is not allowed (a
// latency-critical serving loop that has frozen its memory map).  For them the f16 activation tiles
// of the GEMM live in a fixed array inside the library image.  Every device that loads the library
// carries the array until the process exits, so it is kept modest: 8 MiB, i.e. M * K <= 4 194 304.
#define OJAS_B200_GEMM_STATIC_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_gemm_static_scratch[OJAS_B200_GEMM_STATIC_BYTES];

// In host code the array's name is only a handle; the device address comes from the runtime, once per
// device, with that device current.  (The first call on a device is not thread-safe against another first call on
// the same device: make it from one thread, at set-up.)
static void *gemm_static_scratch_ptr(ojas_b200_ctx *ctx, int *rc_out) {
    static void *ptrs[64] = {nullptr};
    *rc_out = 0;
    if (ctx->device < 0 || ctx->device >= 64) { *rc_out = ojas_fail(ctx, OJAS_B200_E_LIMIT, "gemm_static: device index %d out of range", ctx->device); return nullptr; }
    if (!ptrs[ctx->device]) {
        int cur = -1;
        cudaError_t e = cudaGetDevice(&cur);
        if (e == cudaSuccess && cur != ctx->device) e = cudaSetDevice(ctx->device);
        void *p = nullptr;
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&p, g_gemm_static_scratch);
        if (e == cudaSuccess && cur >= 0 && cur != ctx->device) e = cudaSetDevice(cur);
        if (e != cudaSuccess || !p) {
            *rc_out = ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return nullptr;
        }
        // Load every kernel this entry can launch now (the runtime loads a kernel's code at its first use, which may
        // allocate device memory): after this first call on a device no later call allocates, whatever its shape or type.
        cudaFuncAttributes fa;
#define OJAS_TOUCH(K) cudaFuncGetAttributes(&fa, K)
#define OJAS_TOUCH_TYPE(T) OJAS_TOUCH((gemm_ts_kernel<32, T>)); OJAS_TOUCH((gemm_ts_kernel<64, T>)); OJAS_TOUCH((gemm_ts_kernel<128, T>)); OJAS_TOUCH((gemm_ts_kernel<256, T>))
        OJAS_TOUCH_TYPE(OJAS_B200_Q4_K); OJAS_TOUCH_TYPE(OJAS_B200_Q5_K); OJAS_TOUCH_TYPE(OJAS_B200_Q6_K); OJAS_TOUCH_TYPE(OJAS_B200_Q8_0);
        OJAS_TOUCH_TYPE(OJAS_B200_IQ4_XS); OJAS_TOUCH_TYPE(OJAS_B200_IQ4_NL);
        OJAS_TOUCH((gemm_prep_kernel<true, float>)); OJAS_TOUCH((gemm_prep_kernel<false, float>));
        OJAS_TOUCH((gemm_prep_kernel<true, __half>)); OJAS_TOUCH((gemm_prep_kernel<false, __half>));
#undef OJAS_TOUCH_TYPE
#undef OJAS_TOUCH
        cudaGetLastError();
        ptrs[ctx->device] = p;
    }
    return ptrs[ctx->device];
}

extern "C" size_t ojas_b200_gemm_static_capacity(void) { return OJAS_B200_GEMM_STATIC_BYTES; }

void *ojas_scratch_for(ojas_b200_ctx *ctx, size_t bytes, const char *who) {
    if (ctx->reserved && ctx->reserved_bytes >= bytes) return ctx->reserved;
    if (bytes <= OJAS_B200_GEMM_STATIC_BYTES) {
        int rc = 0;
        void *p = gemm_static_scratch_ptr(ctx, &rc);
        if (p) return p;
        return nullptr;
    }
    ojas_fail(ctx, OJAS_B200_E_LIMIT, "%s: %zu bytes of scratch needed, %zu reserved: call ojas_b200_reserve at set-up", who, bytes, ctx->reserved_bytes);
    return nullptr;
}

extern "C" int ojas_b200_gemm_static(ojas_b200_ctx *ctx, uint32_t type, const float *x, const void *w, float *y, size_t K, size_t N,
                                     size_t M, int accum) {
    if (!ctx) return OJAS_B200_E_ARG;
    const size_t need = ojas_b200_gemm_workspace_bytes(M, K);
    if (M == 0 || K == 0 || need > OJAS_B200_GEMM_STATIC_BYTES || need / 2 < M * K)
        return ojas_fail(ctx, OJAS_B200_E_LIMIT, "gemm_static: M=%zu x K=%zu needs %zu bytes of scratch, the built-in array holds %u (M*K <= %u)",
                         M, K, need, OJAS_B200_GEMM_STATIC_BYTES, OJAS_B200_GEMM_STATIC_BYTES / 2);
    int rc = 0;
    void *scratch = gemm_static_scratch_ptr(ctx, &rc);
    if (!scratch) return rc;
    return ojas_b200_gemm(ctx, type, x, w, y, K, N, M, accum, scratch, OJAS_B200_GEMM_STATIC_BYTES);
}

