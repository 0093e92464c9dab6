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
// The kernel is persistent (one CTA per SM walks a list of tiles) with two TMEM accumulators, so
// the drain of one tile overlaps the main loop of the next; the warp roles are listed above the
// kernel.
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
constexpr int DEQ_WARPS_PER_GROUP = 8;                 // two groups of eight dequantizing warps
constexpr int WARP_TMA_X = 4 + 2 * DEQ_WARPS_PER_GROUP; // warp 20: TMA of the activation tiles
constexpr int WARP_MMA0 = WARP_TMA_X + 1;              // warps 21-24: one MMA-issuing thread per ring slot
constexpr int WARP_TMA_W = WARP_MMA0 + 4;              // warp 25: TMA of raw Q4_K tiles; owns the TMEM allocation
constexpr int GEMM_THREADS = (WARP_TMA_W + 1) * 32;    // 832
constexpr int WQ_BUFS = 2;          // raw Q4_K nibble tiles (one super-block x 128 rows = 16 KB) in flight
constexpr int WQ_BYTES = BM * 128;
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
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {   // non-blocking probe
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false if the CTA is aborting (this wait or another one ran out).
__device__ __noinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned *status, unsigned code) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++)
            if (mbar_test(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CYCLES) {
            *abort_flag = 1;
            atomicOr(status, code);
            __threadfence_system();
            return false;
        }
    }
}

// Up to 64 hardware-suspended waits (mbarrier.try_wait returns as soon as the phase completes, or after
// a time limit of its own), entirely inside one asm block: the common case costs a few instructions.
__device__ __forceinline__ bool mbar_try_loop(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t.reg .u32 n;\n\tmov.u32 n, 0;\n"
                 "WAIT_LOOP:\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t@p bra WAIT_DONE;\n\t"
                 "add.u32 n, n, 1;\n\tsetp.lt.u32 p, n, 64;\n\t@p bra WAIT_LOOP;\n"
                 "WAIT_DONE:\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// Single-thread roles (MMA issue, TMA) and warp leaders: the fast loop first, the clock-bounded slow
// path only when the barrier is very late.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned *status, unsigned code) {
    if (mbar_try_loop(bar, parity)) return true;
    return mbar_wait(bar, parity, abort_flag, status, code);
}

// Warp form: lane 0 waits, the result is broadcast, __syncwarp orders the other lanes behind it.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned *status, unsigned code) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait_spin(bar, parity, abort_flag, status, code) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
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
// A stage row is 64 weights = 128 bytes of f16 = eight 16-byte chunks; chunk j goes to position
// j ^ (row & 7) (the 128-byte swizzle).  Two threads share a row: `half` 0 writes chunks 0-3
// (weights 0..31 of the 64-chunk), half 1 writes chunks 4-7.  For the K-quants the k order inside
// every group of four is (0, 2, 1, 3): that is the order the nibble pairs fall out of a 32-bit
// word, and the activation tile is written in the same order (see gemm_prep_kernel), so the dot
// is unchanged.
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

__device__ __forceinline__ void store_chunk(unsigned char *row_base, int row, int j, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    *reinterpret_cast<uint4 *>(row_base + ((j ^ (row & 7)) << 4)) = make_uint4(a, b, c, d);
}

// Q4_K: A, B = the chunk's two 16-byte nibble pieces (low nibbles = weights 0..31, high = 32..63),
// H = header (d, dmin, 24-bit scale groups), c = chunk index inside the super-block.
__device__ __forceinline__ void dequant_q4k_half(const uint4 &A, const uint4 &B, const uint4 &H, int c, int half,
                                                 unsigned char *row_base, int row) {
    const int sh = (c * 24) & 31;
    const uint32_t lo_w = (c < 2) ? H.y : (c == 2 ? H.z : H.w);
    const uint32_t hi_w = (c < 2) ? H.z : H.w;
    const uint32_t sg = __funnelshift_r(lo_w, hi_w, sh) >> (6 * half);     // s at bits 0..5, m at bits 12..17
    const float d = f16_bits_to_f32(H.x), dmin = f16_bits_to_f32(H.x >> 16);
    const __half2 ds = __float2half2_rn(d * (float)(sg & 63u));
    const __half2 nm = __float2half2_rn(-(dmin * (float)((sg >> 12) & 63u)));
    const __half2 k1024 = u32_as_h2(0x64006400u);
    const int nsh = 4 * half;
    const uint32_t w[8] = {A.x >> nsh, A.y >> nsh, A.z >> nsh, A.w >> nsh, B.x >> nsh, B.y >> nsh, B.z >> nsh, B.w >> nsh};
    uint32_t o[16];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const __half2 t0 = u32_as_h2((w[i] & 0x000f000fu) | 0x64006400u);          // weights (4i, 4i+2)
        const __half2 t1 = u32_as_h2(((w[i] >> 8) & 0x000f000fu) | 0x64006400u);   // weights (4i+1, 4i+3)
        o[2 * i] = h2_as_u32(__hfma2(__hsub2(t0, k1024), ds, nm));
        o[2 * i + 1] = h2_as_u32(__hfma2(__hsub2(t1, k1024), ds, nm));
    }
#pragma unroll
    for (int j = 0; j < 4; j++) store_chunk(row_base, row, 4 * half + j, o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
}

// Q6_K: A, B = low nibbles (same arrangement as Q4_K), Hh = the chunk's 16 bytes of top bits,
// sc4 = the chunk's four int8 sub-scales, dbits = f16 d.  Value = d * sc * (q - 32).  half 0
// handles the groups t = 0, 1 (low nibbles of A, B), half 1 the groups 2, 3 (high nibbles).
__device__ __forceinline__ void dequant_q6k_half(const uint4 &A, const uint4 &B, const uint4 &Hh, uint32_t sc4, uint32_t dbits,
                                                 int half, unsigned char *row_base, int row) {
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
    uint32_t ga[8], gb[8];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t h = Hw[k];
        const uint32_t a0 = (Aw[k] & 0x000f000fu) | ((h << 4) & 0x00300030u), a1 = ((Aw[k] >> 8) & 0x000f000fu) | ((h >> 4) & 0x00300030u);
        const uint32_t b0 = (Bw[k] & 0x000f000fu) | ((h << 2) & 0x00300030u), b1 = ((Bw[k] >> 8) & 0x000f000fu) | ((h >> 6) & 0x00300030u);
        ga[2 * k] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(a0 | 0x64006400u), k1056), dscA));
        ga[2 * k + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(a1 | 0x64006400u), k1056), dscA));
        gb[2 * k] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(b0 | 0x64006400u), k1056), dscB));
        gb[2 * k + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(b1 | 0x64006400u), k1056), dscB));
    }
    store_chunk(row_base, row, 4 * half, ga[0], ga[1], ga[2], ga[3]);
    store_chunk(row_base, row, 4 * half + 1, ga[4], ga[5], ga[6], ga[7]);
    store_chunk(row_base, row, 4 * half + 2, gb[0], gb[1], gb[2], gb[3]);
    store_chunk(row_base, row, 4 * half + 3, gb[4], gb[5], gb[6], gb[7]);
}

// Q8_0: one 32-weight block (two 16-byte pieces of int8, one f16 scale).  Natural k order.
__device__ __forceinline__ void dequant_q80_half(const uint4 &q0, const uint4 &q1, uint32_t dbits, int half, unsigned char *row_base, int row) {
    const __half2 k1152 = u32_as_h2(0x64806480u);   // 1024 + 128
    const __half2 dd = __half2half2(__ushort_as_half((unsigned short)(dbits & 0xffffu)));
#pragma unroll
    for (int p = 0; p < 2; p++) {
        const uint4 q = p == 0 ? q0 : q1;
        const uint32_t w[4] = {q.x ^ 0x80808080u, q.y ^ 0x80808080u, q.z ^ 0x80808080u, q.w ^ 0x80808080u};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            o[2 * i] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(w[i], 0x64646464u, 0x4140)), k1152), dd));
            o[2 * i + 1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(w[i], 0x64646464u, 0x4342)), k1152), dd));
        }
        store_chunk(row_base, row, 4 * half + 2 * p, o[0], o[1], o[2], o[3]);
        store_chunk(row_base, row, 4 * half + 2 * p + 1, o[4], o[5], o[6], o[7]);
    }
}

// ---------------------------------------------------------------- the GEMM kernel
// Persistent: CTA b works through the tiles b, b + grid, b + 2 grid, ...  A tile is 128 weight
// rows x BN tokens x one K range.  A pipeline stage is one 64-weight chunk c of a super-block and
// always lives in ring slot c; every stage barrier's phase is the parity of the super-block count.
// Roles (warp index):
//   0-3    epilogue: drain one of the two TMEM accumulators to y (and zero it) while the next tile runs
//   4-19   dequantize: group 0 (warps 4-11) fills slots 0 and 2, group 1 (12-19) slots 1 and 3; thread
//          (row, half) turns 32 weights of one weight row into f16 per stage
//   20     TMA of the f16 activation tiles
//   21-24  tcgen05.mma issue, one thread per ring slot
//   25     TMA of the raw Q4_K nibble tiles (one super-block x 128 rows per load); owns TMEM
struct TileCoord { int n0, m0, sb_begin, sb_end; };

__device__ __forceinline__ TileCoord tile_coord(int tile, int n_tiles_n, int n_tiles_m, int ksplit, int nsb) {
    const int nx = tile % n_tiles_n;
    const int r = tile / n_tiles_n;
    const int my = r % n_tiles_m, kz = r / n_tiles_m;
    TileCoord t;
    t.n0 = nx * BM;
    t.m0 = my;      // multiplied by BN by the caller
    t.sb_begin = (int)((long long)nsb * kz / ksplit);
    t.sb_end = (int)((long long)nsb * (kz + 1) / ksplit);
    return t;
}

template <int BN, int TYPE>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                   const __grid_constant__ CUtensorMap tmap_w, const GemmArgs a) {
    extern __shared__ unsigned char gemm_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)gemm_smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int B_STAGE_BYTES = BN * BK * 2;
    constexpr bool STAGED_W = (TYPE == OJAS_B200_Q4_K);   // raw nibble tiles arrive by TMA, one super-block at a time
    constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulators
    unsigned char *smem_a = smem;
    unsigned char *smem_b = smem + GEMM_STAGES * A_STAGE_BYTES;
    unsigned char *smem_wq = smem_b + GEMM_STAGES * B_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_wq + (STAGED_W ? WQ_BUFS * WQ_BYTES : 0));
    uint64_t *full = bars, *empty = bars + GEMM_STAGES;
    uint64_t *wq_full = bars + 2 * GEMM_STAGES, *wq_empty = wq_full + WQ_BUFS;
    uint64_t *tmem_full = wq_empty + WQ_BUFS, *tmem_empty = tmem_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = a.K >> 8;
    const int n_tiles_n = (a.N + BM - 1) / BM, n_tiles_m = (a.M + BN - 1) / BN;
    const int n_tiles = n_tiles_n * n_tiles_m * a.ksplit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_STAGES; s++) {
            mbar_init(&full[s], DEQ_WARPS_PER_GROUP + 1);   // the stage's dequantizing warps + the TMA thread (with its byte count)
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < WQ_BUFS; b++) {
            mbar_init(&wq_full[b], 1);
            mbar_init(&wq_empty[b], 2 * DEQ_WARPS_PER_GROUP);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], GEMM_STAGES);           // one commit per MMA-issuing thread
            mbar_init(&tmem_empty[b], 4);                    // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == WARP_TMA_W) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Several threads issue MMAs into one accumulator, so no MMA can be "the first" (overwrite): every MMA
    // accumulates and the accumulators start from zero (here, and again after each drain).
    if (warp < 4) {
        for (int col = 0; col < TMEM_COLS; col += 32) tmem_zero32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)col);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp < 4) {
        // ---------------- epilogue: warp e drains TMEM lanes 32e .. 32e+31 (weight rows n0 + 32e + lane)
        int it = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, it++) {
            const TileCoord tc = tile_coord(tile, n_tiles_n, n_tiles_m, a.ksplit, nsb);
            const int m0 = tc.m0 * BN, acc = it & 1;
            if (tc.sb_end <= tc.sb_begin) continue;                     // empty K range: nothing was accumulated
            if (!mbar_wait_warp(&tmem_full[acc], (uint32_t)(it >> 1) & 1u, abort_flag, a.status, 0x400u)) break;
            tc_fence_after();
            const int n = tc.n0 + warp * 32 + lane;
            float *ycol = a.y + n;
#pragma unroll 1
            for (int col = 0; col < BN; col += 32) {
                const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(acc * BN + col);
                if (m0 + col < a.M) {                                    // uniform: the whole CTA shares m0
                    uint32_t v[32];
                    tmem_ld32(taddr, v);
                    if (n < a.N) {
                        const int rows = a.M - (m0 + col) < 32 ? a.M - (m0 + col) : 32;
                        float *yp = ycol + (size_t)(m0 + col) * a.N;
                        if (a.ksplit > 1) {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (j < rows) atomicAdd(yp + (size_t)j * a.N, __uint_as_float(v[j]));
                        } else if (a.accum) {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (j < rows) yp[(size_t)j * a.N] += __uint_as_float(v[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (j < rows) yp[(size_t)j * a.N] = __uint_as_float(v[j]);
                        }
                    }
                }
                tmem_zero32(taddr);                                      // ready for the next tile's accumulation
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);                // this warp's quarter of the accumulator is free
        }
    } else if (warp < WARP_TMA_X) {
        // ---------------- dequantizers: two groups of eight warps; group g fills the stages c = g and g + 2 of every
        // super-block, thread (row, half) of the group writes 32 weights of weight row n0 + row per stage
        const int g = (warp - 4) / DEQ_WARPS_PER_GROUP;
        const int t = threadIdx.x - 128 - g * (DEQ_WARPS_PER_GROUP * 32);
        const int row = t & 127, half = t >> 7;
        uint32_t wc = 0;      // running super-block counter: raw-tile ring position, and phase of every stage barrier
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
            const TileCoord tc = tile_coord(tile, n_tiles_n, n_tiles_m, a.ksplit, nsb);
            const int grow = tc.n0 + row;
            const bool live = grow < a.N;
            const size_t lrow = (size_t)(live ? grow : 0);
            const size_t rowblk = lrow * nsb;
            const int n_sb = tc.sb_end - tc.sb_begin;
            uint4 hdr_next = make_uint4(0u, 0u, 0u, 0u);
            if (STAGED_W && n_sb > 0) hdr_next = __ldg(reinterpret_cast<const uint4 *>(a.w.p1) + rowblk + tc.sb_begin);
            // weights that come straight from global memory (Q6_K, Q8_0): the next stage's loads are in flight
            // while this one is converted
            uint4 cA = make_uint4(0u, 0u, 0u, 0u), cB = cA, cH = cA, nA = cA, nB = cA, nH = cA;
            uint32_t ce0 = 0, ce1 = 0, ne0 = 0, ne1 = 0;
            auto fetch = [&](int sb, int c, uint4 &A, uint4 &B, uint4 &H, uint32_t &e0, uint32_t &e1) {
                if (TYPE == OJAS_B200_Q8_0) {
                    const size_t k0 = (size_t)sb * 256 + (size_t)c * BK + (size_t)half * 32;
                    const uint4 *src = reinterpret_cast<const uint4 *>(a.w.p0) + (lrow * a.K + k0) / 16;
                    A = __ldg(src); B = __ldg(src + 1);
                    e0 = __ldg(reinterpret_cast<const unsigned short *>(a.w.p1) + lrow * (a.K / 32) + k0 / 32);
                } else if (TYPE == OJAS_B200_Q6_K) {
                    const size_t blk = rowblk + sb;
                    A = __ldg(reinterpret_cast<const uint4 *>(a.w.p0) + blk * 8 + c);
                    B = __ldg(reinterpret_cast<const uint4 *>(a.w.p0) + blk * 8 + 4 + c);
                    H = __ldg(reinterpret_cast<const uint4 *>(a.w.p1) + blk * 4 + c);
                    e0 = __ldg(reinterpret_cast<const uint32_t *>(a.w.p2) + blk * 4 + c);
                    e1 = __ldg(reinterpret_cast<const unsigned short *>(a.w.p3) + blk);
                }
            };
            if (!STAGED_W && n_sb > 0) fetch(tc.sb_begin, g, cA, cB, cH, ce0, ce1);
            for (int j = 0; ok && j < n_sb; j++, wc++) {
                const int wb = wc % WQ_BUFS;
                const uint32_t ph = wc & 1u;
                const uint4 H = hdr_next;
                const unsigned char *wrow = smem_wq + wb * WQ_BYTES + row * 128;
                if (STAGED_W) {
                    if (j + 1 < n_sb) hdr_next = __ldg(reinterpret_cast<const uint4 *>(a.w.p1) + rowblk + tc.sb_begin + j + 1);
                    if (!mbar_wait_warp(&wq_full[wb], (wc / WQ_BUFS) & 1u, abort_flag, a.status, 0x2000u)) { ok = false; break; }
                }
#pragma unroll
                for (int cc = 0; cc < 2; cc++) {
                    const int c = g + 2 * cc;                            // this group's stage (ring slot = chunk index)
                    if (STAGED_W) {
                        cA = *reinterpret_cast<const uint4 *>(wrow + ((c ^ (row & 7)) << 4));
                        cB = *reinterpret_cast<const uint4 *>(wrow + (((4 + c) ^ (row & 7)) << 4));
                    } else {                                             // prefetch this group's next stage
                        const bool last = (cc == 1) && (j + 1 >= n_sb);
                        if (!last) fetch(tc.sb_begin + j + (cc == 1 ? 1 : 0), cc == 1 ? g : g + 2, nA, nB, nH, ne0, ne1);
                    }
                    if (!mbar_wait_warp(&empty[c], ph ^ 1u, abort_flag, a.status, 0x100u)) { ok = false; break; }
                    unsigned char *row_base = smem_a + c * A_STAGE_BYTES + row * 128;
                    if (!live) {
#pragma unroll
                        for (int q = 0; q < 4; q++) store_chunk(row_base, row, 4 * half + q, 0u, 0u, 0u, 0u);
                    } else if (TYPE == OJAS_B200_Q4_K) {
                        dequant_q4k_half(cA, cB, H, c, half, row_base, row);
                    } else if (TYPE == OJAS_B200_Q6_K) {
                        dequant_q6k_half(cA, cB, cH, ce0, ce1, half, row_base, row);
                    } else {
                        dequant_q80_half(cA, cB, ce0, half, row_base, row);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full[c]);
                    if (!STAGED_W) { cA = nA; cB = nB; cH = nH; ce0 = ne0; ce1 = ne1; }
                }
                if (STAGED_W) {
                    __syncwarp();
                    if (ok && lane == 0) mbar_arrive(&wq_empty[wb]);     // this warp is done with the raw tile
                }
            }
        }
    } else if (warp == WARP_TMA_X) {
        // ---------------- TMA: activation tile [BN tokens x 64 k] per stage
        if (lane == 0) {
            uint32_t wc = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const TileCoord tc = tile_coord(tile, n_tiles_n, n_tiles_m, a.ksplit, nsb);
                const int m0 = tc.m0 * BN;
                for (int sb = tc.sb_begin; ok && sb < tc.sb_end; sb++, wc++) {
                    const uint32_t ph = wc & 1u;
#pragma unroll
                    for (int c = 0; c < GEMM_STAGES; c++) {
                        if (!mbar_wait_spin(&empty[c], ph ^ 1u, abort_flag, a.status, 0x200u)) { ok = false; break; }
                        mbar_arrive_expect_tx(&full[c], (uint32_t)B_STAGE_BYTES);
                        tma_load_2d(smem_b + c * B_STAGE_BYTES, &tmap_x, (sb * 4 + c) * BK, m0, &full[c]);
                    }
                }
            }
        }
    } else if (warp < WARP_TMA_W) {
        // ---------------- MMA issue: four threads, thread c owns ring slot c (chunk c of every super-block).  A
        // single issuing thread spends about a thousand cycles per stage on its own barrier probes and issue
        // latency; four of them keep the tensor pipe fed.  Every MMA accumulates (see the zeroing above).
        if (lane == 0) {
            const int c = warp - WARP_MMA0;
            constexpr uint32_t idesc = umma_idesc(BN);
            const uint64_t adesc = umma_desc(smem_u32(smem_a + c * A_STAGE_BYTES));
            const uint64_t bdesc = umma_desc(smem_u32(smem_b + c * B_STAGE_BYTES));
            uint32_t wc = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, it++) {
                const TileCoord tc = tile_coord(tile, n_tiles_n, n_tiles_m, a.ksplit, nsb);
                const int n_sb = tc.sb_end - tc.sb_begin, acc = it & 1;
                if (n_sb <= 0) continue;
                if (!mbar_wait_spin(&tmem_empty[acc], ((uint32_t)(it >> 1) & 1u) ^ 1u, abort_flag, a.status, 0x8000u)) break;
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + (uint32_t)(acc * BN);
                for (int j = 0; j < n_sb; j++, wc++) {
                    if (!mbar_wait_spin(&full[c], wc & 1u, abort_flag, a.status, 0x800u)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; k++)       // 32 bytes further along K per MMA (descriptor units of 16 bytes)
                        umma_f16(tmem_acc, adesc + 2 * k, bdesc + 2 * k, idesc, 1u);
                    umma_commit(&empty[c]);                 // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(&tmem_full[acc]);       // this thread's share of the accumulator is complete
            }
        }
    } else {
        // ---------------- TMA: raw Q4_K nibble tile [128 rows x 128 bytes] per super-block
        if (STAGED_W && lane == 0) {
            uint32_t wc = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const TileCoord tc = tile_coord(tile, n_tiles_n, n_tiles_m, a.ksplit, nsb);
                for (int sb = tc.sb_begin; sb < tc.sb_end; sb++, wc++) {
                    const int wb = wc % WQ_BUFS;
                    if (!mbar_wait_spin(&wq_empty[wb], ((wc / WQ_BUFS) & 1u) ^ 1u, abort_flag, a.status, 0x4000u)) { ok = false; break; }
                    mbar_arrive_expect_tx(&wq_full[wb], (uint32_t)WQ_BYTES);
                    tma_load_2d(smem_wq + wb * WQ_BYTES, &tmap_w, sb * 128, tc.n0, &wq_full[wb]);
                }
            }
        }
    }

    // ---------------- teardown (every role arrives here, also after an abort)
    if (*abort_flag && warp == WARP_TMA_X && lane == 0) {
        // give copies that are still in flight a bounded time to land before the CTA releases shared memory
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == WARP_TMA_W) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
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

size_t gemm_smem_bytes(int bn, bool staged_w) {
    return 1024 + (size_t)GEMM_STAGES * (A_STAGE_BYTES + bn * BK * 2) + (staged_w ? WQ_BUFS * WQ_BYTES : 0) + 256;
}

template <int BN, int TYPE>
int launch_gemm_bn(ojas_b200_ctx *ctx, const CUtensorMap &tmap, const CUtensorMap &tmap_w, const GemmArgs &args, dim3 grid) {
    auto kernel = gemm_tc_kernel<BN, TYPE>;
    const size_t smem = gemm_smem_bytes(BN, TYPE == OJAS_B200_Q4_K);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: shared memory %zu: %s", smem, cudaGetErrorString(e));
    kernel<<<grid, GEMM_THREADS, smem, ctx->stream>>>(tmap, tmap_w, args);
    OJAS_LAUNCH_CHECK(ctx, "gemm_tc");
    return 0;
}

template <int TYPE>
int launch_gemm_type(ojas_b200_ctx *ctx, int bn, const CUtensorMap &tmap, const CUtensorMap &tmap_w, const GemmArgs &args, dim3 grid) {
    switch (bn) {
    case 32: return launch_gemm_bn<32, TYPE>(ctx, tmap, tmap_w, args, grid);
    case 64: return launch_gemm_bn<64, TYPE>(ctx, tmap, tmap_w, args, grid);
    case 128: return launch_gemm_bn<128, TYPE>(ctx, tmap, tmap_w, args, grid);
    default: return launch_gemm_bn<256, TYPE>(ctx, tmap, tmap_w, args, grid);
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
    if ((size_t)ksplit > K / 256) ksplit = (int)(K / 256);   // K ranges are whole super-blocks
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

    // raw nibble plane as bytes [N rows][K/2 bytes], box = one super-block (128 bytes) x 128 rows
    CUtensorMap tmap_w = tmap;
    if (type == OJAS_B200_Q4_K) {
        const cuuint64_t wdims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)N};
        const cuuint64_t wstrides[1] = {(cuuint64_t)(K / 2)};
        const cuuint32_t wbox[2] = {128, (cuuint32_t)BM};
        cr = encode(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)w, wdims, wstrides, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemm: cuTensorMapEncodeTiled (weights) failed (%d)", (int)cr);
    }

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
    const size_t n_tiles = ((N + BM - 1) / BM) * ((M + bn - 1) / bn) * (size_t)ksplit;
    const dim3 grid((unsigned)(n_tiles < (size_t)ctx->sm_count ? n_tiles : (size_t)ctx->sm_count));
    if (type == OJAS_B200_Q4_K) return launch_gemm_type<OJAS_B200_Q4_K>(ctx, bn, tmap, tmap_w, args, grid);
    if (type == OJAS_B200_Q6_K) return launch_gemm_type<OJAS_B200_Q6_K>(ctx, bn, tmap, tmap_w, args, grid);
    return launch_gemm_type<OJAS_B200_Q8_0>(ctx, bn, tmap, tmap_w, args, grid);
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
// device, with that device current.
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
        ptrs[ctx->device] = p;
    }
    return ptrs[ctx->device];
}

extern "C" size_t ojas_b200_gemm_static_capacity(void) { return OJAS_B200_GEMM_STATIC_BYTES; }

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

