// Prefill GEMM on the 5th-generation tensor cores: y[M,N] (+)= x[M,K] * W[N,K]^T over repacked
// GGUF weights.  Replaces gemm_mm_{q4l,q6k,q8_0} and their split-K forms
// (crates/ojas-cuda/src/kernels/gemm_q.rs:291-590), with the arithmetic contract of the CPU
// path: for Q4_K / Q6_K the activations are first quantized to Q8_K (quant_q8k,
// crates/ojas-cpu/src/cpu_math.rs:545-563) and enter the MMA as f16(sx * q); for Q8_0 they
// enter as f16(x) (dot_q80 keeps f32 activations, :971-981).  Weights are dequantized tile by
// tile into shared memory as f16 (the reference GEMM does the same with mma.sync,
// gemm_q.rs:6-12) and accumulated in fp32 in tensor memory.
//
// One CTA computes 128 weight rows x BN tokens:
//   UMMA M = 128 weight rows  (A operand: dequantized W tile, K-major, 128-byte swizzle)
//   UMMA N = BN tokens        (B operand: f16 activation tile, loaded by TMA, same swizzle)
//   accumulator D[128 x BN] fp32 in TMEM; TMEM lane = weight row, column = token, so the
//   epilogue's 32 lanes store 32 consecutive outputs of one token: coalesced without a
//   shared-memory transpose.
// Warps 0-3 dequantize (one thread per weight row, one 64-weight chunk per stage) and later
// drain TMEM; warp 4 issues the TMA loads; warp 5 owns TMEM and issues tcgen05.mma.
// Every wait on an mbarrier is bounded: a wait that runs out sets the context's status word,
// raises the CTA's abort flag, and every role falls through to the common teardown (TMEM is
// always released).
#include <cuda.h>

#include "act_quant.cuh"

namespace {

constexpr int BM = 128;            // weight rows per CTA
constexpr int BK = 64;             // k per stage = one 64-weight chunk = 128 bytes of f16
constexpr int GEMM_STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int GEMM_THREADS = 192;
constexpr long long WAIT_CYCLES = 4000000000LL;   // about two seconds

struct GemmArgs {
    WeightPlanes w;
    float *y;
    int M, N, K;
    int accum;           // 1: y += result
    int ksplit;          // grid.z: K is cut into this many ranges; >1 => atomic adds into y
    unsigned *status;    // device-visible status word of the context
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false if the CTA is aborting (this wait or another one ran out).
__device__ __noinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned *status, unsigned code) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CYCLES) {
            *abort_flag = 1;
            atomicOr(status, code);
            __threadfence_system();
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *tmap, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"((uint64_t)tmap), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// K-major operand tile with the 128-byte swizzle: rows of 128 bytes, groups of eight rows 1024
// bytes apart (stride byte offset), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused with a swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset
    d |= (uint64_t)1 << 46;                              // descriptor version
    d |= (uint64_t)2 << 61;                              // 128-byte swizzle
    return d;
}

// kind::f16, A and B f16 K-major, D f32, M = 128, N = bn.
__host__ __device__ constexpr uint32_t umma_idesc(int bn) {
    return (1u << 4) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

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

// ---------------------------------------------------------------- dequantizers (one row, 64 weights)
// All three write eight 16-byte chunks (8 halves each) of one 128-byte smem row; chunk j goes to
// position j ^ (row & 7) (the 128-byte swizzle).  For the K-quants the k order inside every group
// of four is (0, 2, 1, 3): that is the order the nibble pairs fall out of a 32-bit word, and the
// activation tile is written in the same order (see gemm_prep_kernel), so the dot is unchanged.
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

__device__ __forceinline__ void store_chunk(unsigned char *row_base, int row, int j, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    *reinterpret_cast<uint4 *>(row_base + ((j ^ (row & 7)) << 4)) = make_uint4(a, b, c, d);
}

struct RowRegs { uint4 A, B, H; uint32_t e0, e1; };

// Q4_K: A, B = the chunk's two 16-byte nibble pieces, H = header (d, dmin, 24-bit scale groups).
__device__ __forceinline__ void dequant_q4k(const RowRegs &r, int c, unsigned char *row_base, int row) {
    const int sh = (c * 24) & 31;
    const uint32_t lo_w = (c < 2) ? r.H.y : (c == 2 ? r.H.z : r.H.w);
    const uint32_t hi_w = (c < 2) ? r.H.z : r.H.w;
    const uint32_t sg = __funnelshift_r(lo_w, hi_w, sh);
    const float d = f16_bits_to_f32(r.H.x), dmin = f16_bits_to_f32(r.H.x >> 16);
    const __half2 ds1 = __float2half2_rn(d * (float)(sg & 63u)), ds2 = __float2half2_rn(d * (float)((sg >> 6) & 63u));
    const __half2 nm1 = __float2half2_rn(-(dmin * (float)((sg >> 12) & 63u))), nm2 = __float2half2_rn(-(dmin * (float)((sg >> 18) & 63u)));
    const __half2 k1024 = u32_as_h2(0x64006400u);
    const uint32_t w[8] = {r.A.x, r.A.y, r.A.z, r.A.w, r.B.x, r.B.y, r.B.z, r.B.w};
    uint32_t lo[16], hi[16];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const __half2 t0 = u32_as_h2((w[i] & 0x000f000fu) | 0x64006400u);          // weights (4i, 4i+2) of the low half
        const __half2 t1 = u32_as_h2(((w[i] >> 8) & 0x000f000fu) | 0x64006400u);   // (4i+1, 4i+3)
        const __half2 t2 = u32_as_h2(((w[i] >> 4) & 0x000f000fu) | 0x64006400u);   // high half: (4i, 4i+2)
        const __half2 t3 = u32_as_h2(((w[i] >> 12) & 0x000f000fu) | 0x64006400u);  // (4i+1, 4i+3)
        lo[2 * i] = h2_as_u32(__hfma2(__hsub2(t0, k1024), ds1, nm1));
        lo[2 * i + 1] = h2_as_u32(__hfma2(__hsub2(t1, k1024), ds1, nm1));
        hi[2 * i] = h2_as_u32(__hfma2(__hsub2(t2, k1024), ds2, nm2));
        hi[2 * i + 1] = h2_as_u32(__hfma2(__hsub2(t3, k1024), ds2, nm2));
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
        store_chunk(row_base, row, j, lo[4 * j], lo[4 * j + 1], lo[4 * j + 2], lo[4 * j + 3]);
        store_chunk(row_base, row, 4 + j, hi[4 * j], hi[4 * j + 1], hi[4 * j + 2], hi[4 * j + 3]);
    }
}

// Q6_K: A, B = low nibbles (same arrangement as Q4_K), H = the chunk's 16 bytes of top bits,
// e0 = four int8 sub-scales of the chunk, e1 = f16 d.  Value = d * sc * (q - 32).
__device__ __forceinline__ void dequant_q6k(const RowRegs &r, unsigned char *row_base, int row) {
    const float d = f16_bits_to_f32(r.e1);
    __half2 dsc[4];
#pragma unroll
    for (int t = 0; t < 4; t++) dsc[t] = __float2half2_rn(d * (float)(int)(signed char)((r.e0 >> (8 * t)) & 0xffu));
    const __half2 k1056 = u32_as_h2(0x64206420u);   // 1024 + 32
    const uint32_t Aw[4] = {r.A.x, r.A.y, r.A.z, r.A.w}, Bw[4] = {r.B.x, r.B.y, r.B.z, r.B.w};
    const uint32_t Hw[4] = {r.H.x, r.H.y, r.H.z, r.H.w};
    uint32_t g[4][8];   // g[t] = the 16 weights of group t as eight half2 words
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t h = Hw[k];
        // group 0: A low nibbles, top bits field 0; group 1: B low, field 1; group 2: A high, field 2; group 3: B high, field 3
        const uint32_t n00 = (Aw[k] & 0x000f000fu) | ((h << 4) & 0x00300030u), n01 = ((Aw[k] >> 8) & 0x000f000fu) | ((h >> 4) & 0x00300030u);
        const uint32_t n10 = (Bw[k] & 0x000f000fu) | ((h << 2) & 0x00300030u), n11 = ((Bw[k] >> 8) & 0x000f000fu) | ((h >> 6) & 0x00300030u);
        const uint32_t n20 = ((Aw[k] >> 4) & 0x000f000fu) | (h & 0x00300030u), n21 = ((Aw[k] >> 12) & 0x000f000fu) | ((h >> 8) & 0x00300030u);
        const uint32_t n30 = ((Bw[k] >> 4) & 0x000f000fu) | ((h >> 2) & 0x00300030u), n31 = ((Bw[k] >> 12) & 0x000f000fu) | ((h >> 10) & 0x00300030u);
        g[0][2 * k] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(n00 | 0x64006400u), k1056), dsc[0]));
        g[0][2 * k + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(n01 | 0x64006400u), k1056), dsc[0]));
        g[1][2 * k] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(n10 | 0x64006400u), k1056), dsc[1]));
        g[1][2 * k + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(n11 | 0x64006400u), k1056), dsc[1]));
        g[2][2 * k] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(n20 | 0x64006400u), k1056), dsc[2]));
        g[2][2 * k + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(n21 | 0x64006400u), k1056), dsc[2]));
        g[3][2 * k] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(n30 | 0x64006400u), k1056), dsc[3]));
        g[3][2 * k + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(n31 | 0x64006400u), k1056), dsc[3]));
    }
#pragma unroll
    for (int t = 0; t < 4; t++) {
        store_chunk(row_base, row, 2 * t, g[t][0], g[t][1], g[t][2], g[t][3]);
        store_chunk(row_base, row, 2 * t + 1, g[t][4], g[t][5], g[t][6], g[t][7]);
    }
}

// Q8_0: 64 int8 weights (four 16-byte pieces in A, B, H and the e-registers are not used: the
// caller passes the pieces in q[]), two f16 block scales.  Natural k order.
__device__ __forceinline__ void dequant_q80(const uint4 (&q)[4], uint32_t dpair, unsigned char *row_base, int row) {
    const __half2 k1152 = u32_as_h2(0x64806480u);   // 1024 + 128
    const __half2 d0 = __half2half2(__ushort_as_half((unsigned short)(dpair & 0xffffu)));
    const __half2 d1 = __half2half2(__ushort_as_half((unsigned short)(dpair >> 16)));
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const __half2 dd = p < 2 ? d0 : d1;
        const uint32_t w[4] = {q[p].x ^ 0x80808080u, q[p].y ^ 0x80808080u, q[p].z ^ 0x80808080u, q[p].w ^ 0x80808080u};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            o[2 * i] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(w[i], 0x64646464u, 0x4140)), k1152), dd));
            o[2 * i + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(w[i], 0x64646464u, 0x4342)), k1152), dd));
        }
        store_chunk(row_base, row, 2 * p, o[0], o[1], o[2], o[3]);
        store_chunk(row_base, row, 2 * p + 1, o[4], o[5], o[6], o[7]);
    }
}

// ---------------------------------------------------------------- the GEMM kernel
template <int BN, int TYPE>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmArgs a) {
    extern __shared__ unsigned char gemm_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)gemm_smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int B_STAGE_BYTES = BN * BK * 2;
    unsigned char *smem_a = smem;
    unsigned char *smem_b = smem + GEMM_STAGES * A_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_b + GEMM_STAGES * B_STAGE_BYTES);
    uint64_t *full_a = bars, *full_b = bars + GEMM_STAGES, *empty = bars + 2 * GEMM_STAGES, *accum_bar = bars + 3 * GEMM_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * GEMM_STAGES + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BM, m0 = blockIdx.y * BN;
    const int nsb = a.K >> 8;
    const int kb_total = a.K / BK;
    const int kb_begin = (int)((long long)kb_total * blockIdx.z / a.ksplit);
    const int kb_end = (int)((long long)kb_total * (blockIdx.z + 1) / a.ksplit);
    const int n_kb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_STAGES; s++) {
            mbar_init(&full_a[s], BM);
            mbar_init(&full_b[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {   // TMEM allocation: BN columns (a power of two >= 32)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        // ---------------- producers: thread t dequantizes weight row n0 + t, one 64-weight chunk per stage
        const int t = threadIdx.x;
        const int row = n0 + t;
        const bool live = row < a.N;
        const size_t rowblk = (size_t)(live ? row : 0) * nsb;
        RowRegs cur, nxt;
        uint4 q8[4], q8n[4];
        auto fetch = [&](int kb, RowRegs &r, uint4 (&q)[4]) {
            if (TYPE == OJAS_B200_Q8_0) {
                const uint4 *src = reinterpret_cast<const uint4 *>(a.w.p0) + ((size_t)(live ? row : 0) * a.K + (size_t)kb * BK) / 16;
                q[0] = __ldg(src); q[1] = __ldg(src + 1); q[2] = __ldg(src + 2); q[3] = __ldg(src + 3);
                r.e0 = __ldg(reinterpret_cast<const uint32_t *>(a.w.p1) + ((size_t)(live ? row : 0) * (a.K / 32) + (size_t)kb * 2) / 2);
            } else {
                const int sb = kb >> 2, c = kb & 3;
                const size_t blk = rowblk + sb;
                r.A = __ldg(reinterpret_cast<const uint4 *>(a.w.p0) + blk * 8 + c);
                r.B = __ldg(reinterpret_cast<const uint4 *>(a.w.p0) + blk * 8 + 4 + c);
                if (TYPE == OJAS_B200_Q4_K) {
                    r.H = __ldg(reinterpret_cast<const uint4 *>(a.w.p1) + blk);
                } else {
                    r.H = __ldg(reinterpret_cast<const uint4 *>(a.w.p1) + blk * 4 + c);
                    r.e0 = __ldg(reinterpret_cast<const uint32_t *>(a.w.p2) + blk * 4 + c);
                    r.e1 = __ldg(reinterpret_cast<const unsigned short *>(a.w.p3) + blk);
                }
            }
        };
        if (n_kb > 0) fetch(kb_begin, cur, q8);
        for (int i = 0; i < n_kb; i++) {
            const int kb = kb_begin + i, s = i % GEMM_STAGES;
            const uint32_t ph = (uint32_t)(i / GEMM_STAGES) & 1u;
            if (i + 1 < n_kb) fetch(kb + 1, nxt, q8n);
            if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, a.status, 0x100u)) break;
            unsigned char *row_base = smem_a + s * A_STAGE_BYTES + t * 128;
            if (!live) {
#pragma unroll
                for (int j = 0; j < 8; j++) store_chunk(row_base, t, j, 0u, 0u, 0u, 0u);
            } else if (TYPE == OJAS_B200_Q4_K) {
                dequant_q4k(cur, kb & 3, row_base, t);
            } else if (TYPE == OJAS_B200_Q6_K) {
                dequant_q6k(cur, row_base, t);
            } else {
                dequant_q80(q8, cur.e0, row_base, t);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA
            mbar_arrive(&full_a[s]);
            cur = nxt;
#pragma unroll
            for (int j = 0; j < 4; j++) q8[j] = q8n[j];
        }
        // ---------------- epilogue: warp w drains TMEM lanes 32w .. 32w+31 (weight rows n0 + 32w + lane)
        if (n_kb > 0 && mbar_wait(accum_bar, 0u, abort_flag, a.status, 0x400u)) {
            tc_fence_after();
            const int n = n0 + warp * 32 + lane;
#pragma unroll 1
            for (int col = 0; col < BN; col += 32) {
                if (m0 + col >= a.M) break;            // uniform: the whole CTA shares m0
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)col, v);
                if (n < a.N) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int m = m0 + col + j;
                        if (m < a.M) {
                            float *yp = a.y + (size_t)m * a.N + n;
                            const float val = __uint_as_float(v[j]);
                            if (a.ksplit > 1) atomicAdd(yp, val);
                            else *yp = a.accum ? *yp + val : val;
                        }
                    }
                }
            }
        }
    } else if (warp == 4) {
        // ---------------- TMA: activation tile [BN tokens x 64 k] per stage
        if (lane == 0) {
            for (int i = 0; i < n_kb; i++) {
                const int s = i % GEMM_STAGES;
                const uint32_t ph = (uint32_t)(i / GEMM_STAGES) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, a.status, 0x200u)) break;
                mbar_arrive_expect_tx(&full_b[s], (uint32_t)B_STAGE_BYTES);
                tma_load_2d(smem_b + s * B_STAGE_BYTES, &tmap_x, (kb_begin + i) * BK, m0, &full_b[s]);
            }
        }
    } else {
        // ---------------- MMA issue: one thread
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BN);
            for (int i = 0; i < n_kb; i++) {
                const int s = i % GEMM_STAGES;
                const uint32_t ph = (uint32_t)(i / GEMM_STAGES) & 1u;
                if (!mbar_wait(&full_a[s], ph, abort_flag, a.status, 0x800u)) break;
                if (!mbar_wait(&full_b[s], ph, abort_flag, a.status, 0x1000u)) break;
                tc_fence_after();
                const uint64_t adesc = umma_desc(smem_u32(smem_a + s * A_STAGE_BYTES));
                const uint64_t bdesc = umma_desc(smem_u32(smem_b + s * B_STAGE_BYTES));
#pragma unroll
                for (int k = 0; k < BK / 16; k++)       // 32 bytes further along K per MMA (descriptor units of 16 bytes)
                    umma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty[s]);                 // frees the stage once these MMAs have read it
                if (i == n_kb - 1) umma_commit(accum_bar);
            }
        }
    }

    // ---------------- teardown (every role arrives here, also after an abort)
    if (*abort_flag && warp == 4 && lane == 0) {
        // give copies that are still in flight a bounded time to land before the CTA releases shared memory
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BN) : "memory");
    }
}

// ---------------------------------------------------------------- activation preparation
// x f32 [M, K] -> xh f16 [M, K].  QUANT: xh = f16(sx * q) with (sx, q) = quant_q8k(x), written
// in the k order the K-quant dequantizers produce ((0, 2, 1, 3) inside every group of four).
// Otherwise xh = f16(x) in natural order (Q8_0).  One warp per 256 values.
template <bool QUANT>
__global__ void __launch_bounds__(256) gemm_prep_kernel(const float *x, __half *xh, long long n_sb) {
    const int lane = threadIdx.x & 31;
    const long long sb = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (sb >= n_sb) return;
    float v[8];
    if (QUANT) {
        const Q8kLane ql = quant_q8k_warp(x + sb * 256, lane);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t word = i < 4 ? ql.packed.x : ql.packed.y;
            v[i] = __fmul_rn(ql.scale, (float)(int)(signed char)((word >> (8 * (i & 3))) & 0xffu));
        }
    } else {
        const float4 p = __ldg(reinterpret_cast<const float4 *>(x + sb * 256) + lane * 2);
        const float4 q = __ldg(reinterpret_cast<const float4 *>(x + sb * 256) + lane * 2 + 1);
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

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

size_t gemm_smem_bytes(int bn) { return 1024 + (size_t)GEMM_STAGES * (A_STAGE_BYTES + bn * BK * 2) + 256; }

template <int BN, int TYPE>
int launch_gemm_bn(ojas_b200_ctx *ctx, const CUtensorMap &tmap, const GemmArgs &args, dim3 grid) {
    auto kernel = gemm_tc_kernel<BN, TYPE>;
    const size_t smem = gemm_smem_bytes(BN);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: shared memory %zu: %s", smem, cudaGetErrorString(e));
    kernel<<<grid, GEMM_THREADS, smem, ctx->stream>>>(tmap, args);
    OJAS_LAUNCH_CHECK(ctx, "gemm_tc");
    return 0;
}

template <int TYPE>
int launch_gemm_type(ojas_b200_ctx *ctx, int bn, const CUtensorMap &tmap, const GemmArgs &args, dim3 grid) {
    switch (bn) {
    case 32: return launch_gemm_bn<32, TYPE>(ctx, tmap, args, grid);
    case 64: return launch_gemm_bn<64, TYPE>(ctx, tmap, args, grid);
    case 128: return launch_gemm_bn<128, TYPE>(ctx, tmap, args, grid);
    default: return launch_gemm_bn<256, TYPE>(ctx, tmap, args, grid);
    }
}

}  // namespace

extern "C" size_t ojas_b200_gemm_workspace_bytes(size_t M, size_t K) { return align256(M * K * 2); }

// Token-tile width and K split for a shape: the widest tile the token count fills, then enough
// K ranges to give every SM a CTA (never fewer than four stages of K per range).
static void gemm_plan(ojas_b200_ctx *ctx, size_t M, size_t N, size_t K, int &bn, int &ksplit) {
    bn = M > 128 ? 256 : M > 64 ? 128 : M > 32 ? 64 : 32;
    const size_t tiles = ((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    ksplit = 1;
    if (ctx->gemm_ksplit > 0) {
        ksplit = ctx->gemm_ksplit;
    } else {
        while (tiles * ksplit * 2 <= (size_t)ctx->sm_count && (K / BK) / (ksplit * 2) >= 8) ksplit *= 2;
    }
    if ((size_t)ksplit > K / BK) ksplit = (int)(K / BK);
    if (ksplit < 1) ksplit = 1;
}

extern "C" int ojas_b200_gemm(ojas_b200_ctx *ctx, uint32_t type, const float *x, const void *w, float *y, size_t K, size_t N,
                              size_t M, int accum, void *workspace, size_t workspace_bytes) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (type != OJAS_B200_Q4_K && type != OJAS_B200_Q6_K && type != OJAS_B200_Q8_0)
        return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: unsupported GGUF type %u", type);
    if (!x || !w || !y || !workspace) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: null pointer");
    if (K == 0 || K % 256 != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: K=%zu must be a positive multiple of 256", K);
    if (N == 0 || M == 0 || N > 0x7fffffffu || M > 0x7fffffffu) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: M=%zu N=%zu out of range", M, N);
    if (workspace_bytes < ojas_b200_gemm_workspace_bytes(M, K))
        return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: workspace of %zu bytes, %zu needed", workspace_bytes, ojas_b200_gemm_workspace_bytes(M, K));
    if (((uintptr_t)w & 255) || ((uintptr_t)workspace & 255) || ((uintptr_t)x & 15))
        return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: misaligned pointer (weights and workspace 256 bytes, x 16 bytes)");
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: cuTensorMapEncodeTiled is not available from the driver");

    // 1. activations -> f16 tile source
    __half *xh = (__half *)workspace;
    const long long n_sb = (long long)M * (long long)(K / 256);
    const long long blocks = (n_sb + 7) / 8;
    if (blocks > 0x7fffffffLL) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemm: activation matrix too large");
    if (type == OJAS_B200_Q8_0) gemm_prep_kernel<false><<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, xh, n_sb);
    else gemm_prep_kernel<true><<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, xh, n_sb);
    OJAS_LAUNCH_CHECK(ctx, "gemm_prep");

    // 2. plan + tensor map over xh [M rows][K halves], box = 64 halves x bn rows, 128-byte swizzle
    int bn, ksplit;
    gemm_plan(ctx, M, N, K, bn, ksplit);
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)bn};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)xh, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: cuTensorMapEncodeTiled failed (%d)", (int)cr);

    GemmArgs args{};
    args.w = weight_planes(type, w, N, K);
    args.y = y;
    args.M = (int)M; args.N = (int)N; args.K = (int)K;
    args.accum = accum ? 1 : 0;
    args.ksplit = ksplit;
    args.status = ctx->dev_status;
    if (ksplit > 1 && !accum) {   // split-K adds into y: start from zero unless the caller accumulates
        OJAS_CUDA(ctx, cudaMemsetAsync(y, 0, M * N * sizeof(float), ctx->stream));
    }
    const dim3 grid((unsigned)((N + BM - 1) / BM), (unsigned)((M + bn - 1) / bn), (unsigned)ksplit);
    if (type == OJAS_B200_Q4_K) return launch_gemm_type<OJAS_B200_Q4_K>(ctx, bn, tmap, args, grid);
    if (type == OJAS_B200_Q6_K) return launch_gemm_type<OJAS_B200_Q6_K>(ctx, bn, tmap, args, grid);
    return launch_gemm_type<OJAS_B200_Q8_0>(ctx, bn, tmap, args, grid);
}
