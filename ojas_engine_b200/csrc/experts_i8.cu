// The expert FFN's matmuls on the 5th-generation tensor cores with EXACT integers: tcgen05.mma.kind::i8 over Q4_K
// experts and Q8_K activations (crates/ojas-cuda/src/kernels/moe.rs:75-125 and crates/ojas-cpu/src/cpu_glm.rs:551-582
// give the semantics; the arithmetic is dot_q4k's, crates/ojas-cpu/src/cpu_math.rs:609-635).
//
// dot_q4k of one super-block is d * sx * isum - dmin * sx * mins with the integers
//     isum = sum_j sc_j * (sum_i nibble_ji * q_ji)      (8 sub-blocks of 32 weights, 6-bit scales sc_j)
//     mins = sum_j m_j * bsum_j                          (6-bit mins, block sums of the activations)
// Both are formed by int8 MMAs with int32 accumulation, i.e. exactly.  A scale is split as sc = (sc & 7) + 8 * (sc >> 3)
// and folded into the weights: the expander writes the two int8 tiles nibble * (sc & 7) and nibble * (sc >> 3) (both
// at most 105), so ONE accumulator per term runs over the whole super-block and isum = D_lo + 8 * D_hi.  The block sums
// are split as bsum = lo + 64 * hi (lo in 0..63), and mins = M_lo + 64 * M_hi comes from two small MMAs of the mins
// bytes against the lo / hi bytes.  What is left per (weight row, token, super-block) is two integer operations and
// the fp32 combine; everything per weight runs on the tensor core or once per weight in the expander.
//
//   raw weight tiles   TMA (4-D map over the tile layout, 16 units x 9 pieces x 128 B = 18 KB per super-block), asked
//                      into L2 a few steps ahead
//   A operands         expander warps (thread = weight row) write the K-major, 128-byte-swizzled int8 tiles
//                      [128 rows x 256 k] of both scale parts, and the mins bytes as a K = 32 tile without swizzle
//                      whose second K chunk is a block of zeros
//   B operands         the tokens' Q8_K integers [32 tokens x 256 k] (TMA, 128-byte swizzle) straight from the
//                      activation matrix in expert order; 16-byte records [lo bytes | scale | 0] and [hi bytes | 0]
//                      per (super-block, position) land as the K = 32 tiles of the mins MMAs (bytes 8..15 meet zeros
//                      in A, so the activation scale can ride there)
//   accumulators       TMEM, 4 buffers x (D_lo, D_hi, M_lo, M_hi) x 32 columns = all 512 columns
// Work is the list of (expert with rows, tensor, 128-row tile, K part) items, expert-major, shared out by cost; K
// parts of an item write separate output planes that the consumer adds in order (deterministic).
// Every wait is bounded; a wait that runs out sets the status word and all roles fall through to the teardown.
#include "tc_util.cuh"

namespace {

constexpr int XI_ROWS = 128;
constexpr int XI_UNIT_BYTES = 1152;                          // one 8-row Q4_K tile
constexpr int XI_RAW_BYTES = (XI_ROWS / 8) * XI_UNIT_BYTES;  // 18432
constexpr int XI_PREFETCH_STEPS = 8;                         // raw tiles asked into L2 this many steps ahead of their copy
constexpr int XI_A_HALF = XI_ROWS * 128;                     // 128 k of 128 rows
constexpr int XI_A_PART = 2 * XI_A_HALF;                     // one scale part of a super-block: 32 KB
constexpr int XI_AM_BYTES = XI_ROWS * 16;                    // the mins bytes: first K chunk of a K = 32 tile
constexpr int XI_A_BYTES = 2 * XI_A_PART + XI_AM_BYTES;      // 67584
constexpr int XI_A_STAGES = 2;
constexpr int XI_RAW_STAGES = 3;
constexpr int XI_BAR_BYTES = 512;
constexpr int XI_EPI_WARPS = 8, XI_EXP_WARPS = 8;
constexpr int XI_WARP_EXP0 = XI_EPI_WARPS, XI_WARP_TMA_W = XI_WARP_EXP0 + XI_EXP_WARPS, XI_WARP_TMA_B = XI_WARP_TMA_W + 1,
              XI_WARP_MMA = XI_WARP_TMA_B + 1;
constexpr int XI_THREADS = (XI_WARP_MMA + 1) * 32;           // 608
constexpr int XI_MAX_E = 64;

// Sizes that follow from the token tile: TOK = 32 tokens per pass (decode-sized batches: four accumulator buffers, three
// token stages) or 64 (prefill-sized batches: half the passes over an expert's weights; two buffers, two stages).
template <int TOK>
struct XiCfg {
    static constexpr int BQ_HALF = TOK * 128;                // the tokens' integers of 128 k
    static constexpr int BM_BYTES = TOK * 16;                // lo (and scale) records / hi records of TOK positions
    static constexpr int B_BYTES = 2 * BQ_HALF + 2 * BM_BYTES;
    static constexpr int B_STAGES = TOK == 32 ? 3 : 2;
    static constexpr int ACC_COLS = 4 * TOK;                 // D_lo, D_hi, M_lo, M_hi
    static constexpr int ACC_BUFS = 512 / ACC_COLS;
    static constexpr int ZERO_BYTES = XI_AM_BYTES + BM_BYTES; // second K chunks of the mins tiles
    static constexpr int SMEM = 1024 + XI_A_STAGES * XI_A_BYTES + B_STAGES * B_BYTES + XI_RAW_STAGES * XI_RAW_BYTES + ZERO_BYTES + XI_BAR_BYTES;
    // kind::i8: D s32, A and B signed 8-bit, both K-major, M = 128, N = TOK
    static constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TOK >> 3) << 17) | ((uint32_t)(XI_ROWS >> 4) << 24);
    static_assert(B_BYTES % 1024 == 0 && SMEM <= 232448 - 512, "stage alignment and shared memory");
};
static_assert(XI_A_BYTES % 1024 == 0 && XI_RAW_BYTES % 1024 == 0, "stages keep the 1024-byte alignment of swizzled tiles");

struct XiArgs {
    const uint8_t *w[2];         // stacked experts (tile layout), gate and up or down alone
    float *y[2];                 // [positions][N] per tensor; K part p writes plane y + p * part_stride
    size_t part_stride;
    int nw, kparts;
    size_t expert_bytes;
    const int *counts, *offsets;
    unsigned *status;
    int E, K, N, nsb;
};

struct XiPiece { int e, wsel, n0, off, mb, m_here, sb0, sb1, kp; };

// The CTA's items [it, it_end) in expert-major order; every role walks them with its own copy.
struct XiSched {
    unsigned it, it_end;
    int mb, tiles, nw, kparts, nsb, tok;
    const int *act_e, *counts, *offsets;
    __device__ bool next(XiPiece &p) {
        for (;;) {
            if (it >= it_end) return false;
            const unsigned per_e = (unsigned)(nw * tiles * kparts);
            const unsigned ai = it / per_e, r = it - ai * per_e;
            const int e = act_e[ai];
            const int count = __ldg(counts + e);
            if (mb >= count) { mb = 0; it++; continue; }
            p.e = e;
            p.wsel = (int)(r / (unsigned)(tiles * kparts));
            const unsigned r2 = r - (unsigned)p.wsel * (unsigned)(tiles * kparts);
            p.n0 = (int)(r2 / (unsigned)kparts) * XI_ROWS;
            p.kp = (int)(r2 % (unsigned)kparts);
            p.off = __ldg(offsets + e);
            p.mb = mb;
            p.m_here = count - mb < tok ? count - mb : tok;
            p.sb0 = (int)((long long)nsb * p.kp / kparts);
            p.sb1 = (int)((long long)nsb * (p.kp + 1) / kparts);
            mb += tok;
            return true;
        }
    }
};

__device__ __forceinline__ void umma_i8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// K-major operand without a swizzle: core matrices of 8 rows x 16 bytes (128 contiguous bytes); `lbo` = distance between
// the core matrices of consecutive K chunks, `sbo` = distance between consecutive 8-row groups.
__device__ __forceinline__ uint64_t umma_desc_plain(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo & 0x3FFFFu) >> 4) << 16;
    d |= (uint64_t)((sbo & 0x3FFFFu) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *tmap, int c0, int c1, int c2, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"((uint64_t)tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

template <int TOK>
__global__ void __launch_bounds__(XI_THREADS, 1) experts_i8_kernel(const __grid_constant__ CUtensorMap tmap_w0,
                                                                   const __grid_constant__ CUtensorMap tmap_w1,
                                                                   const __grid_constant__ CUtensorMap tmap_q,
                                                                   const __grid_constant__ CUtensorMap tmap_m, const XiArgs a) {
    using C = XiCfg<TOK>;
    extern __shared__ unsigned char xi_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)xi_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *smem_a = smem;
    unsigned char *smem_b = smem_a + XI_A_STAGES * XI_A_BYTES;
    unsigned char *smem_raw = smem_b + C::B_STAGES * C::B_BYTES;
    unsigned char *zero_a = smem_raw + XI_RAW_STAGES * XI_RAW_BYTES, *zero_b = zero_a + XI_AM_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(zero_a + C::ZERO_BYTES);
    uint64_t *raw_full = bars, *raw_empty = bars + 4, *a_full = bars + 8, *a_empty = bars + 12, *b_full = bars + 16, *b_empty = bars + 20;
    uint64_t *acc_full = bars + 24, *acc_empty = bars + 28;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 32);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    unsigned *share = reinterpret_cast<unsigned *>(tmem_slot + 2);          // [2]
    __shared__ int act_e[XI_MAX_E];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = a.nsb, tiles = (a.N + XI_ROWS - 1) / XI_ROWS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 4; s++) {
            mbar_init(&raw_full[s], 1);
            mbar_init(&raw_empty[s], 4);                     // the four expander warps of the group that reads the stage
            mbar_init(&a_full[s], 4);
            mbar_init(&a_empty[s], 1);                       // one epilogue thread, once the step's MMAs are known to be done
            mbar_init(&b_full[s], 1);
            mbar_init(&b_empty[s], XI_EPI_WARPS);            // every epilogue warp (the activation scales are read there)
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], XI_EPI_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < C::ZERO_BYTES / 16; i += blockDim.x) reinterpret_cast<uint4 *>(zero_a)[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == XI_WARP_TMA_W && lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmap_w0) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmap_w1) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmap_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmap_m) : "memory");
    }
    if (warp == XI_WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    grid_dependency_wait();                                  // counts, offsets, activations and their records come from kernels before this one
    if (threadIdx.x == 32) {
        // The CTA's share of the item list is a share of its cost: an item of an expert with more rows does more
        // token groups in the epilogue and more passes.  Cost of an item = sum over passes of (3 + token groups of 8).
        int n = 0;
        unsigned long long total = 0;
        unsigned ecost[XI_MAX_E];
        const unsigned per_e = (unsigned)(a.nw * tiles * a.kparts);
        for (int e = 0; e < a.E; e++) {
            const int cnt = __ldg(a.counts + e);
            if (cnt <= 0) continue;
            const unsigned full = (unsigned)(cnt / TOK), rest = (unsigned)(cnt % TOK);
            ecost[n] = full * (3u + TOK / 8) + (rest ? 3u + ((rest + 7u) >> 3) : 0u);
            total += (unsigned long long)ecost[n] * per_e;
            act_e[n++] = e;
        }
        for (int side = 0; side < 2; side++) {
            unsigned long long pos = total * (blockIdx.x + side) / gridDim.x;
            unsigned item = 0;
            int i = 0;
            for (; i < n; i++) {
                const unsigned long long span = (unsigned long long)ecost[i] * per_e;
                if (pos < span) break;
                pos -= span;
                item += per_e;
            }
            if (i < n) item += (unsigned)(pos / ecost[i]);
            share[side] = item;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    grid_launch_dependents();
    const uint32_t tmem_base = *tmem_slot;

    XiSched sched;
    sched.it = share[0]; sched.it_end = share[1]; sched.mb = 0; sched.tiles = tiles; sched.nw = a.nw; sched.kparts = a.kparts; sched.nsb = nsb; sched.tok = TOK;
    sched.act_e = act_e; sched.counts = a.counts; sched.offsets = a.offsets;
    XiPiece pc;
    uint32_t step = 0;                                       // super-block steps done by this CTA: every role counts the same

    if (warp < XI_EPI_WARPS) {
        // ---------------- epilogue: thread = weight row (TMEM lane); the two warps of a lane quarter take alternate
        // groups of eight tokens
        const int quarter = warp & 3, th = warp >> 2, row = quarter * 32 + lane;
        bool ok = true;
        while (ok && sched.next(pc)) {
            const int n = pc.n0 + row;
            const bool live = n < a.N;
            const int lrow = live ? n : a.N - 1;
            // f16 d and dmin of this row's block: first word of the header piece of its tile
            const uint8_t *hdr = a.w[pc.wsel] + (size_t)pc.e * a.expert_bytes + (size_t)(lrow >> 3) * nsb * XI_UNIT_BYTES + 8 * 128 + (lrow & 7) * 16;
            const int ntg = (pc.m_here + 7) >> 3;
            constexpr int NH = TOK / 16;                 // token groups of eight per epilogue thread
            float yacc[NH][8];
#pragma unroll
            for (int h = 0; h < NH; h++)
#pragma unroll
                for (int i = 0; i < 8; i++) yacc[h][i] = 0.0f;
            uint32_t dn = __ldg(reinterpret_cast<const uint32_t *>(hdr + (size_t)pc.sb0 * XI_UNIT_BYTES));
            for (int sb = pc.sb0; sb < pc.sb1; sb++, step++) {
                const uint32_t dd = dn;
                if (sb + 1 < pc.sb1) dn = __ldg(reinterpret_cast<const uint32_t *>(hdr + (size_t)(sb + 1) * XI_UNIT_BYTES));
                const int ab = (int)(step % C::ACC_BUFS), bs = (int)(step % C::B_STAGES), as = (int)(step % XI_A_STAGES);
                if (!mbar_wait_warp(&acc_full[ab], (step / C::ACC_BUFS) & 1u, abort_flag, a.status, 0x100000u)) { ok = false; break; }
                tc_fence_after();
                if (warp == 0 && lane == 0) mbar_arrive(&a_empty[as]);      // the step's MMAs are done: its weight tiles are free
                const float d = f16_bits_to_f32(dd), dmin = f16_bits_to_f32(dd >> 16);
                const unsigned char *recs = smem_b + bs * C::B_BYTES + 2 * C::BQ_HALF;     // [token][lo bytes | scale | 0]
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ab * C::ACC_COLS);
#pragma unroll
                for (int h = 0; h < NH; h++) {
                    const int tg = th + 2 * h;
                    if (tg < ntg) {
                        int dlo[8], dhi[8], mlo[8], mhi[8];
                        tmem_ld8(taddr + 0 * TOK + tg * 8, dlo);
                        tmem_ld8(taddr + 1 * TOK + tg * 8, dhi);
                        tmem_ld8(taddr + 2 * TOK + tg * 8, mlo);
                        tmem_ld8(taddr + 3 * TOK + tg * 8, mhi);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int t = 0; t < 8; t++) {
                            const float sx = *reinterpret_cast<const float *>(recs + (tg * 8 + t) * 16 + 8);
                            const int isum = dlo[t] + 8 * dhi[t], mins = mlo[t] + 64 * mhi[t];
                            yacc[h][t] += sx * (d * (float)isum - dmin * (float)mins);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&acc_empty[ab]);
                    mbar_arrive(&b_empty[bs]);
                }
            }
            if (!ok) break;
            float *yout = a.y[pc.wsel] + (size_t)pc.kp * a.part_stride + (size_t)(pc.off + pc.mb) * a.N + n;
#pragma unroll
            for (int h = 0; h < NH; h++)
#pragma unroll
                for (int t = 0; t < 8; t++) {
                    const int tok = (th + 2 * h) * 8 + t;
                    if (live && tok < pc.m_here) yout[(size_t)tok * a.N] = yacc[h][t];
                }
        }
    } else if (warp < XI_WARP_TMA_W) {
        // ---------------- expanders: two groups of four warps take alternate steps (group g owns weight stage g); thread =
        // weight row.  A nibble word w gives the int8 words w & 0x0f0f0f0f (sub-block 2c) and (w >> 4) & 0x0f0f0f0f
        // (sub-block 2c + 1); each is multiplied, four bytes at a time, by the low 3 bits and by the high 3 bits of its
        // sub-block's scale (products <= 105: no carry between bytes).  K-major tile: row r at r * 128 bytes inside its
        // 8-row group of 1024, 16-byte chunk index XOR (r & 7).
        const int g = (warp - XI_WARP_EXP0) >> 2, row = ((warp - XI_WARP_EXP0) & 3) * 32 + lane;
        const int roff = (row >> 3) * XI_UNIT_BYTES + (row & 7) * 16;
        const int aoff = (row >> 3) * 1024 + (row & 7) * 128, sw = row & 7;
        unsigned char *stage = smem_a + g * XI_A_BYTES;
        bool ok = true;
        while (ok && sched.next(pc)) {
            for (int sb = pc.sb0; sb < pc.sb1; sb++, step++) {
                if ((int)(step & 1u) != g) continue;
                const int rs = (int)(step % XI_RAW_STAGES);
                if (!mbar_wait_warp(&raw_full[rs], (step / XI_RAW_STAGES) & 1u, abort_flag, a.status, 0x400000u)) { ok = false; break; }
                const unsigned char *src = smem_raw + rs * XI_RAW_BYTES + roff;
                uint4 P[8];
#pragma unroll
                for (int p = 0; p < 8; p++) P[p] = *reinterpret_cast<const uint4 *>(src + p * 128);
                const uint4 H = *reinterpret_cast<const uint4 *>(src + 8 * 128);
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[rs]);
                // six-bit scales and mins, one per byte (get_scale_min_k4, crates/ojas-formats/src/gguf.rs:1132-1140)
                const uint32_t sc[2] = {H.y & 0x3f3f3f3fu, (H.w & 0x0f0f0f0fu) | ((H.y >> 2) & 0x30303030u)};
                const uint32_t mn[2] = {H.z & 0x3f3f3f3fu, ((H.w >> 4) & 0x0f0f0f0fu) | ((H.z >> 2) & 0x30303030u)};
                if (!mbar_wait_warp(&a_empty[g], ((step >> 1) & 1u) ^ 1u, abort_flag, a.status, 0x800000u)) { ok = false; break; }
                unsigned char *dst = stage + aoff;
#pragma unroll
                for (int p = 0; p < 8; p++) {
                    const int c = p >> 1, h = p & 1;
                    const uint32_t sA = (sc[c >> 1] >> (16 * (c & 1))) & 0xffu, sB = (sc[c >> 1] >> (16 * (c & 1) + 8)) & 0xffu;
                    const uint32_t a3 = sA & 7u, a8 = sA >> 3, b3 = sB & 7u, b8 = sB >> 3;
                    const uint32_t n0[4] = {P[p].x & 0x0f0f0f0fu, P[p].y & 0x0f0f0f0fu, P[p].z & 0x0f0f0f0fu, P[p].w & 0x0f0f0f0fu};
                    const uint32_t n1[4] = {(P[p].x >> 4) & 0x0f0f0f0fu, (P[p].y >> 4) & 0x0f0f0f0fu, (P[p].z >> 4) & 0x0f0f0f0fu,
                                            (P[p].w >> 4) & 0x0f0f0f0fu};
                    unsigned char *reg = dst + (c >> 1) * XI_A_HALF;             // sub-blocks 2c, 2c + 1 lie in K half c / 2
                    const int ch_lo = (((2 * c) & 3) * 2 + h) ^ sw, ch_hi = (((2 * c + 1) & 3) * 2 + h) ^ sw;
                    *reinterpret_cast<uint4 *>(reg + (ch_lo << 4)) = make_uint4(n0[0] * a3, n0[1] * a3, n0[2] * a3, n0[3] * a3);
                    *reinterpret_cast<uint4 *>(reg + XI_A_PART + (ch_lo << 4)) = make_uint4(n0[0] * a8, n0[1] * a8, n0[2] * a8, n0[3] * a8);
                    *reinterpret_cast<uint4 *>(reg + (ch_hi << 4)) = make_uint4(n1[0] * b3, n1[1] * b3, n1[2] * b3, n1[3] * b3);
                    *reinterpret_cast<uint4 *>(reg + XI_A_PART + (ch_hi << 4)) = make_uint4(n1[0] * b8, n1[1] * b8, n1[2] * b8, n1[3] * b8);
                }
                // the mins bytes: first K chunk of the K = 32 tile (core matrices of 8 rows x 16 bytes, one after another)
                *reinterpret_cast<uint4 *>(stage + 2 * XI_A_PART + (row >> 3) * 128 + (row & 7) * 16) = make_uint4(mn[0], mn[1], 0u, 0u);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[g]);
            }
        }
    } else if (warp == XI_WARP_TMA_W) {
        // ---------------- raw weight tiles: one tiled copy per step
        if (lane == 0) {
            const int units_pe = a.N / OJAS_TILE_ROWS;
            // a second cursor runs ahead of the copies and asks the tiles into L2: the copies into shared memory then
            // find them there, and the memory latency is covered by L2 capacity instead of by shared-memory stages
            XiSched pf = sched;
            XiPiece pp;
            bool pf_live = pf.next(pp);
            int pf_sb = pf_live ? pp.sb0 : 0, ahead = 0;
            auto prefetch_more = [&]() {
                while (pf_live && ahead < XI_PREFETCH_STEPS) {
                    const CUtensorMap *tm = pp.wsel ? &tmap_w1 : &tmap_w0;
                    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global [%0, {%1, %2, %3, %4}];"
                                 ::"l"((uint64_t)tm), "r"(0), "r"(0), "r"(pf_sb), "r"(pp.e * units_pe + pp.n0 / OJAS_TILE_ROWS) : "memory");
                    ahead++;
                    if (++pf_sb == pp.sb1) {
                        pf_live = pf.next(pp);
                        pf_sb = pf_live ? pp.sb0 : 0;
                    }
                }
            };
            bool ok = true;
            while (ok && sched.next(pc)) {
                const CUtensorMap *tm = pc.wsel ? &tmap_w1 : &tmap_w0;
                for (int sb = pc.sb0; sb < pc.sb1; sb++, step++) {
                    prefetch_more();
                    const int rs = (int)(step % XI_RAW_STAGES);
                    if (!mbar_wait_spin(&raw_empty[rs], ((step / XI_RAW_STAGES) & 1u) ^ 1u, abort_flag, a.status, 0x1000000u)) { ok = false; break; }
                    mbar_arrive_expect_tx(&raw_full[rs], (uint32_t)XI_RAW_BYTES);
                    tma_load_4d(smem_raw + rs * XI_RAW_BYTES, tm, 0, 0, sb, pc.e * units_pe + pc.n0 / OJAS_TILE_ROWS, &raw_full[rs]);
                    ahead--;
                }
            }
        }
    } else if (warp == XI_WARP_TMA_B) {
        // ---------------- the tokens' integers (two 128-k halves) and their lo / hi records
        if (lane == 0) {
            bool ok = true;
            while (ok && sched.next(pc)) {
                for (int sb = pc.sb0; sb < pc.sb1; sb++, step++) {
                    const int bs = (int)(step % C::B_STAGES);
                    if (!mbar_wait_spin(&b_empty[bs], ((step / C::B_STAGES) & 1u) ^ 1u, abort_flag, a.status, 0x2000000u)) { ok = false; break; }
                    unsigned char *dst = smem_b + bs * C::B_BYTES;
                    mbar_arrive_expect_tx(&b_full[bs], (uint32_t)C::B_BYTES);
                    tma_load_2d(dst, &tmap_q, sb * 256, pc.off + pc.mb, &b_full[bs]);
                    tma_load_2d(dst + C::BQ_HALF, &tmap_q, sb * 256 + 128, pc.off + pc.mb, &b_full[bs]);
                    tma_load_3d(dst + 2 * C::BQ_HALF, &tmap_m, 0, pc.off + pc.mb, sb, &b_full[bs]);
                    tma_load_3d(dst + 2 * C::BQ_HALF + C::BM_BYTES, &tmap_m, 0, pc.off + pc.mb, nsb + sb, &b_full[bs]);
                }
            }
        }
    } else {
        // ---------------- MMA issue.  Per step: sub-block j = K half j / 4, 32 bytes (j % 4) of every row; both scale
        // parts against the same tokens, accumulating over the eight sub-blocks; then the two mins MMAs
        if (lane == 0) {
            // descriptors of stage 0; a later stage adds its distance to the address field and, for the tiles without a
            // swizzle, takes it off the offset that points at the block of zeros
            const uint32_t a0 = smem_u32(smem_a), b0 = smem_u32(smem_b);
            const uint64_t ad0 = umma_desc(a0), bd0 = umma_desc(b0);
            const uint64_t am0 = umma_desc_plain(a0 + 2 * XI_A_PART, smem_u32(zero_a) - (a0 + 2 * XI_A_PART), 128u);
            const uint64_t bm0 = umma_desc_plain(b0 + 2 * C::BQ_HALF, smem_u32(zero_b) - (b0 + 2 * C::BQ_HALF), 128u);
            constexpr uint64_t A_STEP = XI_A_BYTES >> 4, B_STEP = C::B_BYTES >> 4, BM_STEP = C::BM_BYTES >> 4;
            bool ok = true;
            while (ok && sched.next(pc)) {
                for (int sb = pc.sb0; sb < pc.sb1; sb++, step++) {
                    const int ab = (int)(step % C::ACC_BUFS), as = (int)(step % XI_A_STAGES), bs = (int)(step % C::B_STAGES);
                    if (!mbar_wait_spin(&acc_empty[ab], ((step / C::ACC_BUFS) & 1u) ^ 1u, abort_flag, a.status, 0x4000000u)) { ok = false; break; }
                    if (!mbar_wait_spin(&a_full[as], (step / XI_A_STAGES) & 1u, abort_flag, a.status, 0x8000000u)) { ok = false; break; }
                    if (!mbar_wait_spin(&b_full[bs], (step / C::B_STAGES) & 1u, abort_flag, a.status, 0x10000000u)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t acc = tmem_base + (uint32_t)(ab * C::ACC_COLS);
                    const uint64_t ad_lo = ad0 + (uint64_t)as * A_STEP, ad_hi = ad_lo + (XI_A_PART >> 4), bd = bd0 + (uint64_t)bs * B_STEP;
                    const uint64_t am = am0 + (uint64_t)as * A_STEP - (((uint64_t)as * A_STEP) << 16);
                    const uint64_t bm_lo = bm0 + (uint64_t)bs * B_STEP - (((uint64_t)bs * B_STEP) << 16), bm_hi = bm_lo + BM_STEP - (BM_STEP << 16);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint64_t koff = (uint64_t)((j >> 2) * (XI_A_HALF >> 4) + (j & 3) * 2), boff = (uint64_t)((j >> 2) * (C::BQ_HALF >> 4) + (j & 3) * 2);
                        umma_i8_ss(acc, ad_lo + koff, bd + boff, C::IDESC, j > 0 ? 1u : 0u);
                        umma_i8_ss(acc + TOK, ad_hi + koff, bd + boff, C::IDESC, j > 0 ? 1u : 0u);
                    }
                    umma_i8_ss(acc + 2 * TOK, am, bm_lo, C::IDESC, 0u);
                    umma_i8_ss(acc + 3 * TOK, am, bm_hi, C::IDESC, 0u);
                    umma_commit(&acc_full[ab]);
                }
            }
        }
    }

    // ---------------- teardown (every role arrives here, also after an abort)
    if (*abort_flag && warp == XI_WARP_TMA_W && lane == 0) {
        const long long t0 = clock64();                      // copies still in flight get a bounded time to land
        while (clock64() - t0 < 2000000LL) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == XI_WARP_MMA) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// Activations into expert order with their records.  One CTA per position: the row's integers (gathered through
// row_index when given) and, per super-block, two 16-byte records: [bsum low bytes 0-7 | activation scale | 0] in plane 0
// and [bsum high bytes 0-7 | 0] in plane 1, with bsum = low + 64 * high, low in 0..63.  recs is [2][nsb][positions][16].
__global__ void __launch_bounds__(256) experts_i8_pack_kernel(const int8_t *q, const float *scales, const int32_t *bsums, const int *row_index,
                                                              int K, int positions, int8_t *q_out, uint4 *recs) {
    grid_dependency_wait();
    const int pos = blockIdx.x, nsb = K >> 8;
    const int srow = row_index ? __ldg(row_index + pos) : pos;
    if (q_out) {
        const uint4 *src = reinterpret_cast<const uint4 *>(q + (size_t)srow * K);
        uint4 *dst = reinterpret_cast<uint4 *>(q_out + (size_t)pos * K);
        for (int i = threadIdx.x; i < K / 16; i += blockDim.x) dst[i] = __ldg(src + i);
    }
    for (int sb = threadIdx.x; sb < nsb; sb += blockDim.x) {
        const int32_t *b = bsums + ((size_t)srow * nsb + sb) * 8;
        uint32_t lo[2] = {0u, 0u}, hi[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int v = __ldg(b + j);
            lo[j >> 2] |= (uint32_t)(v & 63) << (8 * (j & 3));
            hi[j >> 2] |= (uint32_t)((v >> 6) & 0xff) << (8 * (j & 3));
        }
        recs[(size_t)sb * positions + pos] = make_uint4(lo[0], lo[1], __float_as_uint(__ldg(scales + (size_t)srow * nsb + sb)), 0u);
        recs[((size_t)nsb + sb) * positions + pos] = make_uint4(hi[0], hi[1], 0u, 0u);
    }
}

}  // namespace

size_t ojas_experts_i8_meta_bytes(size_t positions, size_t K) { return align256(2 * (K / 256) * positions * 16); }

int ojas_experts_i8_pack(ojas_b200_ctx *ctx, const int8_t *q, const float *scales, const int32_t *bsums, const int *row_index, size_t positions,
                         size_t K, int8_t *q_out, void *meta) {
    if (positions == 0) return 0;
    experts_i8_pack_kernel<<<(unsigned)positions, 256, 0, ctx->stream>>>(q, scales, bsums, row_index, (int)K, (int)positions, q_out, (uint4 *)meta);
    OJAS_LAUNCH_CHECK(ctx, "experts_i8_pack");
    return 0;
}

// gate and up (w1 != null) or down (w1 == null) of every expert over the positions' Q8_K integers q [positions][K]
// (expert order) and their records.  Returns 1 if the shape is not one this kernel takes, < 0 on an error.
int ojas_experts_i8(ojas_b200_ctx *ctx, const uint8_t *w0, const uint8_t *w1, float *y0, float *y1, const int8_t *q, const void *meta,
                    size_t positions, const int *counts, const int *offsets, size_t E, size_t K, size_t N, int kparts, size_t part_stride, int tok) {
    if (N % OJAS_TILE_ROWS != 0 || E > (size_t)XI_MAX_E || K % 256 != 0 || positions == 0) return 1;
    if (((uintptr_t)q & 15) || ((uintptr_t)meta & 15) || ((uintptr_t)w0 & 127) || ((uintptr_t)w1 & 127)) return 1;
    if (tok != 32 && tok != 64) return 1;
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return 1;
    const size_t nsb = K / 256, units = E * (N / OJAS_TILE_ROWS);
    if (kparts < 1) kparts = 1;
    if ((size_t)kparts > nsb) kparts = (int)nsb;
    CUtensorMap tw[2], tq, tm;
    const cuuint32_t estr4[4] = {1, 1, 1, 1};
    for (int i = 0; i < 2; i++) {
        const uint8_t *w = i ? (w1 ? w1 : w0) : w0;
        const cuuint64_t wdims[4] = {128, 9, (cuuint64_t)nsb, (cuuint64_t)units};
        const cuuint64_t wstrides[3] = {128, (cuuint64_t)XI_UNIT_BYTES, (cuuint64_t)(nsb * XI_UNIT_BYTES)};
        const cuuint32_t wbox[4] = {128, 9, 1, (cuuint32_t)(XI_ROWS / OJAS_TILE_ROWS)};
        CUresult cr = encode(&tw[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void *)w, wdims, wstrides, wbox, estr4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return ojas_fail(ctx, OJAS_B200_E_CUDA, "experts_i8: cuTensorMapEncodeTiled (weights) failed (%d)", (int)cr);
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)positions};
        const cuuint64_t strides[1] = {(cuuint64_t)K};
        const cuuint32_t box[2] = {128, (cuuint32_t)tok};
        CUresult cr = encode(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)q, dims, strides, box, estr4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return ojas_fail(ctx, OJAS_B200_E_CUDA, "experts_i8: cuTensorMapEncodeTiled (activations) failed (%d)", (int)cr);
    }
    {   // the records: [2 planes x nsb][positions][16 bytes]; a box = 32 positions of one (plane, super-block)
        const cuuint64_t dims[3] = {16, (cuuint64_t)positions, (cuuint64_t)(2 * nsb)};
        const cuuint64_t strides[2] = {16, (cuuint64_t)positions * 16};
        const cuuint32_t box[3] = {16, (cuuint32_t)tok, 1};
        CUresult cr = encode(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void *)meta, dims, strides, box, estr4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return ojas_fail(ctx, OJAS_B200_E_CUDA, "experts_i8: cuTensorMapEncodeTiled (records) failed (%d)", (int)cr);
    }
    XiArgs a{};
    a.w[0] = w0; a.w[1] = w1; a.y[0] = y0; a.y[1] = y1; a.nw = w1 ? 2 : 1;
    a.kparts = kparts; a.part_stride = part_stride;
    a.expert_bytes = (N / OJAS_TILE_ROWS) * nsb * (size_t)XI_UNIT_BYTES;
    a.counts = counts; a.offsets = offsets; a.status = ctx->dev_status;
    a.E = (int)E; a.K = (int)K; a.N = (int)N; a.nsb = (int)nsb;
    auto go = [&](auto kernel, int smem) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "experts_i8: shared memory %d: %s", smem, cudaGetErrorString(e));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)ctx->sm_count);
        cfg.blockDim = dim3(XI_THREADS);
        cfg.dynamicSmemBytes = (size_t)smem;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ctx->pdl ? 1 : 0;
        e = cudaLaunchKernelEx(&cfg, kernel, tw[0], tw[1], tq, tm, a);
        if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "launch experts_i8: %s", cudaGetErrorString(e));
        return 0;
    };
    const int rc = tok == 64 ? go(experts_i8_kernel<64>, XiCfg<64>::SMEM) : go(experts_i8_kernel<32>, XiCfg<32>::SMEM);
    if (rc) return rc;
    ojas_count_launch(ctx, "experts_i8");
    return 0;
}
