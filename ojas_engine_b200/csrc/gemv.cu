// Decode GEMV over repacked GGUF weights: y[m, n] = sum_k W[n, k] * x[m, k], M <= 8.
//
// Arithmetic follows matvec_kq (crates/ojas-cpu/src/cpu_math.rs:1145-1189):
//   Q4_K, Q6_K : x is quantized to Q8_K int8 (per-256 scale) and every 32- / 16-weight
//                sub-block dot is an exact int32 dot (dot_q4k :609-635, dot_q6k :674-722);
//   Q8_0       : x stays f32 (dot_q80 :971-981).
// The kernels replace gemv_nat_{q4k,q6k,q80}{,_accum,_bias,_m}
// (crates/ojas-cuda/src/kernels/nat.rs:69-91).
//
// Shape of every kernel: a persistent grid (one CTA of 32 warps per SM).  CTA b owns the
// contiguous row range [N*b/G, N*(b+1)/G).  Work is cut into items of one row x eight
// super-blocks (2048 weights): four lanes share a super-block, each lane owns a 64-weight
// chunk, so one warp load instruction reads whole 32-byte sectors of one contiguous
// kilobyte.  Items go round-robin to warps, each warp keeps the next item's loads in
// flight while it computes the current one, item partial sums land in shared memory and
// are added per row in a fixed order (deterministic results).
#include "act_quant.cuh"

constexpr int GEMV_THREADS = 1024;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

struct GemvArgs {
    const float *x;          // [M, K] f32 (unused when activations come pre-quantized)
    const int8_t *q;         // [M, K] pre-quantized activations (PREQ kernels)
    const float *scales;     // [M, K/256]
    const int32_t *bsums;    // [M, K/32]
    WeightPlanes w;
    float *y;                // [M, N]
    const float *bias;       // [N] or null
    int32_t *idots;          // dump of the integer sub-block dots (DUMP kernels)
    // grouped (per-expert) launches: activation row m of the batch is source row row_index[m]
    // (null: row m); the group's row count and first position come from device memory
    const int *row_index;
    const int *grp_count;
    const int *grp_offset;
    int K, N, M, form;
    int S;                   // segments per row (work split); chosen by the host
    int depth;               // stages in each warp's cp.async ring (2..4); chosen by the host
    int rows_base, rows_rem; // CTA b owns rows_base (+1 if b < rows_rem) rows: N = grid*rows_base + rows_rem
};

// First row and row count of this CTA (no 64-bit division on the device).
__device__ __forceinline__ void cta_rows(const GemvArgs &a, int &r_begin, int &R) {
    const int b = (int)blockIdx.x;
    r_begin = b * a.rows_base + (b < a.rows_rem ? b : a.rows_rem);
    R = a.rows_base + (b < a.rows_rem ? 1 : 0);
}

// Floats reserved for the per-super-block activation scales: a multiple of four, so the block
// sums that follow stay 16-byte aligned for any super-block count.
__host__ __device__ __forceinline__ int sx_floats(int mt, int nsb) { return (mt * nsb + 3) & ~3; }

__device__ __forceinline__ void store_form(float *yp, float v, int form, const float *bias, int n) {
    if (form == OJAS_B200_ACCUM) v += *yp;
    else if (form == OJAS_B200_BIAS) v += __ldg(bias + n);
    *yp = v;
}

// ---------------------------------------------------------------------------- work split
// CTA b owns rows [N*b/G, N*(b+1)/G).  A row is cut into S segments of whole groups (a group
// = eight super-blocks = 2048 weights; S = 1 unless the CTA has fewer rows than warps);
// (row, segment) units go round-robin to the warps.  A warp walks the groups of its unit with
// the next group's loads already in flight, reduces once per unit, and the S partial sums of
// a row are added in a fixed order, so results do not depend on timing.
struct WarpCursor {
    int u;          // unit index inside the CTA
    int row;        // global weight row
    int g, g_end;   // current group and end of the unit's group range
};

__device__ __forceinline__ void cursor_set(WarpCursor &cu, int u, int n_units, int S, int G8, int r_begin) {
    cu.u = u;
    cu.row = 0; cu.g = 0; cu.g_end = 0;
    if (u < n_units) {
        const int rr = u / S, seg = u - rr * S;
        cu.row = r_begin + rr;
        cu.g = seg * G8 / S;
        cu.g_end = (seg + 1) * G8 / S;
    }
}

__device__ __forceinline__ void cursor_advance(WarpCursor &cu, int n_units, int S, int G8, int r_begin) {
    if (++cu.g >= cu.g_end) cursor_set(cu, cu.u + GEMV_WARPS, n_units, S, G8, r_begin);
}

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {   // unsigned bytes x signed bytes
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// End of a unit: warp-reduce the accumulators; S == 1 stores y directly, otherwise the partial
// goes to shared memory for finish_rows.
template <int MT>
__device__ __forceinline__ void unit_done(float (&acc)[MT], const WarpCursor &cu, int S, float *part, const GemvArgs &a, int lane) {
#pragma unroll
    for (int m = 0; m < MT; m++) {
        const float s = warp_sum(acc[m]);
        acc[m] = 0.0f;
        if (lane == 0) {
            if (S == 1) {
                if (m < a.M) store_form(a.y + (size_t)m * a.N + cu.row, s, a.form, a.bias, cu.row);
            } else {
                part[cu.u * MT + m] = s;
            }
        }
    }
}

template <int MT>
__device__ __forceinline__ void finish_rows(const float *part, int R, int S, int r_begin, const GemvArgs &a) {
    if (S == 1) return;
    __syncthreads();
    for (int idx = threadIdx.x; idx < R * MT; idx += blockDim.x) {
        const int r = idx / MT, m = idx - r * MT;
        if (m >= a.M) continue;
        float s = 0.0f;
        for (int g = 0; g < S; g++) s += part[(r * S + g) * MT + m];
        const int n = r_begin + r;
        store_form(a.y + (size_t)m * a.N + n, s, a.form, a.bias, n);
    }
}

__device__ __forceinline__ int src_row(const GemvArgs &a, int m) { return a.row_index ? __ldg(a.row_index + m) : m; }

// Quantize (or copy pre-quantized) activations into shared memory.  BS16: keep per-16 sums
// (Q6_K) instead of per-32 sums (Q4_K).
template <int MT, bool PREQ, bool BS16>
__device__ __forceinline__ void stage_q8k(const GemvArgs &a, unsigned char *xq, float *sx, int *bs, int nsb, int Kpad) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int NB = BS16 ? 16 : 8;
    if (!PREQ) {
        // half-warps: task t = (row m, super-block sb); lane l owns the 16-byte unit (l & 15)
        const int half = lane >> 4, un = lane & 15;
        for (int t0 = warp * 2; t0 < MT * nsb; t0 += (int)(blockDim.x >> 5) * 2) {
            const int t = t0 + half;
            const bool live = t < MT * nsb;
            const int tt = live ? t : t0;                 // idle half-warps shadow a live task and store nothing
            const int m = tt / nsb, sb = tt - m * nsb;
            // Both half-warps always run the quantizer (it shuffles with a full mask, so no lane may
            // skip it); a padding row m >= M reads row M-1 and its result is replaced by zeros.
            const int ml = m < a.M ? m : a.M - 1;
            Q8kHalfLane ql = quant_q8k_halfwarp(a.x + (size_t)ml * a.K + (size_t)sb * 256, lane);
            const bool pad = m >= a.M;
            const uint4 packed = pad ? make_uint4(0u, 0u, 0u, 0u) : ql.packed;
            const int s = pad ? 0 : ql.sum16;
            const float scale = pad ? 0.0f : ql.scale;
            const int s32 = s + __shfl_xor_sync(0xffffffffu, s, 1);
            if (live) {
                reinterpret_cast<uint4 *>(xq + (size_t)m * Kpad)[xq_unit(sb, un >> 2, un & 3)] = packed;
                if (BS16) bs[(m * nsb + sb) * 16 + un] = s;
                else if ((un & 1) == 0) bs[(m * nsb + sb) * 8 + (un >> 1)] = s32;
                if (un == 0) sx[m * nsb + sb] = scale;
            }
        }
    } else {
        const int units = nsb * 16;
        for (int idx = threadIdx.x; idx < MT * units; idx += blockDim.x) {
            const int m = idx / units, rem = idx - m * units;
            const int sb = rem >> 4, un = rem & 15;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m < a.M) v = __ldg(reinterpret_cast<const uint4 *>(a.q + (size_t)src_row(a, m) * a.K) + rem);
            reinterpret_cast<uint4 *>(xq + (size_t)m * Kpad)[xq_unit(sb, un >> 2, un & 3)] = v;
            if (BS16) {
                int s = __dp4a((int)v.x, 0x01010101, 0);
                s = __dp4a((int)v.y, 0x01010101, s);
                s = __dp4a((int)v.z, 0x01010101, s);
                s = __dp4a((int)v.w, 0x01010101, s);
                bs[(m * nsb + sb) * 16 + un] = s;
            }
        }
        for (int idx = threadIdx.x; idx < MT * nsb; idx += blockDim.x) {
            const int m = idx / nsb;
            sx[idx] = (m < a.M) ? __ldg(a.scales + (size_t)src_row(a, m) * nsb + (idx - m * nsb)) : 0.0f;
        }
        if (!BS16) {
            for (int idx = threadIdx.x; idx < MT * nsb * NB; idx += blockDim.x) {
                const int m = idx / (nsb * NB);
                bs[idx] = (m < a.M) ? __ldg(a.bsums + (size_t)src_row(a, m) * nsb * NB + (idx - m * nsb * NB)) : 0;
            }
        }
    }
}

// ---------------------------------------------------------------------------- async staging
// Weights travel global -> shared memory with cp.async (16 bytes per lane, no registers held
// while in flight).  Each warp owns a ring of two stages; a stage holds one step of the warp, and one
// step is always in flight while the other is computed.
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
// Same, executed only when `pred` is non-zero (a predicated instruction, not a branch).
__device__ __forceinline__ void cp_async16_if(void *smem_dst, const void *gmem_src, int pred) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p cp.async.cg.shared.global [%0], [%1], 16;\n\t}"
                 ::"r"(d), "l"(gmem_src), "r"(pred) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---------------------------------------------------------------------------- Q4_K
// A Q4_K step is one row x sixteen super-blocks (4096 weights, 2304 bytes): every lane owns
// chunk c of super-blocks sbi and sbi + 8.  Each warp has two stages in shared memory: the
// copies of step t + 1 are in flight while step t is computed.
constexpr int Q4K_STAGE_BYTES = 2304;   // A0 512, B0 512, A1 512, B1 512, sixteen headers 256

// Walks the (row, segment) units of one warp, step by step, without divisions.
struct StepIter {
    int row, seg, gi;      // current unit's row and segment, step inside the unit
    int left;              // steps left for this warp (0 = done)
};

template <int MT, bool PREQ, bool DUMP, int WARPS = GEMV_WARPS>
__device__ __forceinline__ void gemv_q4k_body(const GemvArgs &a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int nsb = a.K >> 8, S = a.S;
    const int G = (nsb + 15) >> 4, GP = G / S;                // steps per row, per unit (host makes S divide G)
    const int Kpad = ((nsb + 1) >> 1) * 512;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sbi = lane >> 2, c = lane & 3;
    unsigned char *ring = smem + (size_t)warp * 2 * Q4K_STAGE_BYTES;          // this warp's two stages
    unsigned char *xq = smem + (size_t)WARPS * 2 * Q4K_STAGE_BYTES;
    float *sx = reinterpret_cast<float *>(xq + (size_t)MT * Kpad);
    int *bs = reinterpret_cast<int *>(sx + sx_floats(MT, nsb));
    float *part = reinterpret_cast<float *>(bs + MT * nsb * 8);

    int r_begin, R;
    cta_rows(a, r_begin, R);
    const int n_units = R * S;
    const uint4 *qs = reinterpret_cast<const uint4 *>(a.w.p0) + c;
    const uint4 *hdr = reinterpret_cast<const uint4 *>(a.w.p1);
    const int sc_shift = (c * 24) & 31;                       // where this lane's 24-bit scale group starts
    // lane-constant parts of the shared-memory addresses (step g adds a multiple of a fixed stride)
    const uint4 *x_lane = reinterpret_cast<const uint4 *>(xq) + ((sbi >> 1) * 32 + (sbi & 1) * 4 + c);
    const int *bs_lane = bs + sbi * 8 + 2 * c;
    const float *sx_lane = sx + sbi;
    unsigned char *st_lane = ring + lane * 16;
    const int dq = WARPS / S, dr = WARPS - dq * S;            // unit index + WARPS in (row, segment) terms

    auto iter_init = [&](StepIter &it) {
        const int my_units = warp < n_units ? (n_units - warp + WARPS - 1) / WARPS : 0;
        it.left = my_units * GP;
        const int rr = warp / S;
        it.row = r_begin + rr;
        it.seg = warp - rr * S;
        it.gi = 0;
    };
    auto iter_next = [&](StepIter &it) {
        it.left--;
        if (++it.gi == GP) {
            it.gi = 0;
            it.seg += dr;
            it.row += dq;
            if (it.seg >= S) { it.seg -= S; it.row++; }
        }
    };

    // issue the copies of one step into a stage (nothing is issued for lanes past the end of K)
    auto issue = [&](const StepIter &it, int stage) {
        const int sb0 = (it.seg * GP + it.gi) * 16 + sbi;
        const unsigned blk = (unsigned)it.row * (unsigned)nsb + (unsigned)sb0;
        unsigned char *st = st_lane + stage * Q4K_STAGE_BYTES;
        const uint4 *src = qs + (size_t)blk * 8;
        const int ok0 = it.left > 0 && sb0 < nsb, ok1 = it.left > 0 && sb0 + 8 < nsb;
        cp_async16_if(st, src, ok0);
        cp_async16_if(st + 512, src + 4, ok0);
        cp_async16_if(st + 1024, src + 64, ok1);
        cp_async16_if(st + 1536, src + 68, ok1);
        // headers: lanes with c == 0 fetch the one of super-block sbi, lanes with c == 1 that of sbi + 8
        cp_async16_if(ring + stage * Q4K_STAGE_BYTES + 2048 + (c * 8 + sbi) * 16, hdr + blk + c * 8, c == 0 ? ok0 : (c == 1 ? ok1 : 0));
        cp_async_commit();
    };

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.0f;

    // one super-block of the step: A, B = the lane's two 16-byte pieces, H = the header
    auto block_dot = [&](const uint4 &A, const uint4 &B, const uint4 &H, int sb, int row) {
        // 24-bit group: s(2c) | s(2c+1) << 6 | m(2c) << 12 | m(2c+1) << 18
        const uint32_t lo_w = (c < 2) ? H.y : (c == 2 ? H.z : H.w);
        const uint32_t hi_w = (c < 2) ? H.z : H.w;
        const uint32_t sg = __funnelshift_r(lo_w, hi_w, sc_shift);
        const int s1 = (int)(sg & 63u), s2 = (int)((sg >> 6) & 63u);
        const int m1 = (int)((sg >> 12) & 63u), m2 = (int)((sg >> 18) & 63u);
        const float d = f16_bits_to_f32(H.x), dmin = f16_bits_to_f32(H.x >> 16);
        const uint32_t a_lo[4] = {A.x & 0x0f0f0f0fu, A.y & 0x0f0f0f0fu, A.z & 0x0f0f0f0fu, A.w & 0x0f0f0f0fu};
        const uint32_t a_hi[4] = {A.x & 0xf0f0f0f0u, A.y & 0xf0f0f0f0u, A.z & 0xf0f0f0f0u, A.w & 0xf0f0f0f0u};
        const uint32_t b_lo[4] = {B.x & 0x0f0f0f0fu, B.y & 0x0f0f0f0fu, B.z & 0x0f0f0f0fu, B.w & 0x0f0f0f0fu};
        const uint32_t b_hi[4] = {B.x & 0xf0f0f0f0u, B.y & 0xf0f0f0f0u, B.z & 0xf0f0f0f0u, B.w & 0xf0f0f0f0u};
        const int sbg = sb - sbi;                              // first super-block of the 8-group (multiple of 8)
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const uint4 *xm = x_lane + m * (Kpad / 16) + sbg * 16;
            const uint4 X0 = xm[0], X1 = xm[8], X2 = xm[16], X3 = xm[24];
            int pA = 0, pB = 0;   // exact int32 dots of sub-blocks 2c and 2c+1 (pB carries a factor 16)
            pA = dp4a_u8s8(a_lo[0], X0.x, pA); pA = dp4a_u8s8(a_lo[1], X0.y, pA);
            pA = dp4a_u8s8(a_lo[2], X0.z, pA); pA = dp4a_u8s8(a_lo[3], X0.w, pA);
            pA = dp4a_u8s8(b_lo[0], X1.x, pA); pA = dp4a_u8s8(b_lo[1], X1.y, pA);
            pA = dp4a_u8s8(b_lo[2], X1.z, pA); pA = dp4a_u8s8(b_lo[3], X1.w, pA);
            pB = dp4a_u8s8(a_hi[0], X2.x, pB); pB = dp4a_u8s8(a_hi[1], X2.y, pB);
            pB = dp4a_u8s8(a_hi[2], X2.z, pB); pB = dp4a_u8s8(a_hi[3], X2.w, pB);
            pB = dp4a_u8s8(b_hi[0], X3.x, pB); pB = dp4a_u8s8(b_hi[1], X3.y, pB);
            pB = dp4a_u8s8(b_hi[2], X3.z, pB); pB = dp4a_u8s8(b_hi[3], X3.w, pB);
            pB >>= 4;             // the high nibbles were left in place: every product carried x16
            if (DUMP && m == 0) {
                int32_t *o = a.idots + (size_t)row * (nsb * 8) + sb * 8 + 2 * c;
                o[0] = pA; o[1] = pB;
            }
            const int2 b2 = *reinterpret_cast<const int2 *>(bs_lane + m * nsb * 8 + sbg * 8);
            const int isum = s1 * pA + s2 * pB;            // sum_j s_j * idot_j  (exact)
            const int msum = m1 * b2.x + m2 * b2.y;        // sum_j m_j * bsum_j  (exact)
            acc[m] += sx_lane[m * nsb + sbg] * (d * (float)isum - dmin * (float)msum);
        }
    };

    StepIter ii, ic;                         // issue runs one step ahead of compute
    iter_init(ii);
    ic = ii;
    issue(ii, 0);                            // weights are in flight while x is staged
    iter_next(ii);
    grid_dependency_wait();                  // x (and y for the accumulate form) come from the kernel before
    stage_q8k<MT, PREQ, false>(a, xq, sx, bs, nsb, Kpad);
    __syncthreads();
    grid_launch_dependents();

    int stage = 0;
    while (ic.left > 0) {
        issue(ii, stage ^ 1);                // the stage consumed one iteration ago
        iter_next(ii);
        cp_async_wait<1>();                  // this thread's copies for `stage` have landed
        __syncwarp();                        // ... and so have the headers copied by other lanes
        const unsigned char *st = st_lane + stage * Q4K_STAGE_BYTES;
        const unsigned char *sh = ring + stage * Q4K_STAGE_BYTES + 2048 + sbi * 16;
        const int sb0 = (ic.seg * GP + ic.gi) * 16 + sbi;
        if (sb0 < nsb)
            block_dot(*reinterpret_cast<const uint4 *>(st), *reinterpret_cast<const uint4 *>(st + 512),
                      *reinterpret_cast<const uint4 *>(sh), sb0, ic.row);
        if (sb0 + 8 < nsb)
            block_dot(*reinterpret_cast<const uint4 *>(st + 1024), *reinterpret_cast<const uint4 *>(st + 1536),
                      *reinterpret_cast<const uint4 *>(sh + 128), sb0 + 8, ic.row);
        __syncwarp();                        // every lane has read this stage's headers before it is refilled
        if (!DUMP && ic.gi + 1 == GP) {
            WarpCursor cu;
            cu.row = ic.row;
            cu.u = (ic.row - r_begin) * S + ic.seg;
            unit_done<MT>(acc, cu, S, part, a, lane);
        }
        iter_next(ic);
        stage ^= 1;
    }
    cp_async_wait<0>();
    if (!DUMP) finish_rows<MT>(part, R, S, r_begin, a);
}

template <int MT, bool PREQ, bool DUMP>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_q4k_kernel(const GemvArgs a) { gemv_q4k_body<MT, PREQ, DUMP>(a); }

// Half-size form for single-row calls on small matrices: 16 warps and about 80 KB of shared memory, so two CTAs
// fit on an SM and, with programmatic dependent launch, the CTAs of the next GEMV in the stream can become
// resident (and start their weight prefetch) while this one still computes.  Measured gain at 4096 x 4096:
// 4.6 -> 4.1 us per launch in a graph of back-to-back GEMVs; releasing the successor before this kernel's own
// wait, or prefetching both ring stages up front, measured slower.
constexpr int GEMV_SLIM_WARPS = 16;
template <bool PREQ>
__global__ void __launch_bounds__(GEMV_SLIM_WARPS * 32, 2) gemv_q4k_slim_kernel(const GemvArgs a) {
    gemv_q4k_body<1, PREQ, false, GEMV_SLIM_WARPS>(a);
}

// Grouped form: the group's rows (count and first position read from device memory, so the launch
// is capture-safe whatever the routing) are processed MT at a time (eight, or fewer when K is long and shared memory is short); passes after the first
// find the group's weights in L2.
template <int MT>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_q4k_grouped_kernel(const GemvArgs a) {
    const int count = __ldg(a.grp_count), off = __ldg(a.grp_offset);
    for (int mb = 0; mb < count; mb += MT) {
        GemvArgs b = a;
        b.M = count - mb < MT ? count - mb : MT;
        if (a.row_index) b.row_index = a.row_index + off + mb;
        else { b.q = a.q + (size_t)(off + mb) * a.K; b.scales = a.scales + (size_t)(off + mb) * (a.K >> 8); b.bsums = a.bsums + (size_t)(off + mb) * (a.K >> 5); }
        b.y = a.y + (size_t)(off + mb) * a.N;
        gemv_q4k_body<MT, true, false>(b);
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------- Q6_K
struct Q6kRegs { uint4 A, B, H; uint32_t sc; uint32_t d; };

template <int MT, bool PREQ, bool DUMP>
__device__ __forceinline__ void gemv_q6k_body(const GemvArgs &a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int nsb = a.K >> 8, G8 = (nsb + 7) >> 3, S = a.S;
    const int Kpad = ((nsb + 1) >> 1) * 512;
    unsigned char *xq = smem;
    float *sx = reinterpret_cast<float *>(smem + (size_t)MT * Kpad);
    int *bs = reinterpret_cast<int *>(sx + sx_floats(MT, nsb)); // per-16 activation sums
    float *part = reinterpret_cast<float *>(bs + MT * nsb * 16);

    int r_begin, R;
    cta_rows(a, r_begin, R);
    const int n_units = R * S;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sbi = lane >> 2, c = lane & 3;
    const uint4 *lo = reinterpret_cast<const uint4 *>(a.w.p0) + c;
    const uint4 *hi = reinterpret_cast<const uint4 *>(a.w.p1) + c;
    const uint32_t *scp = reinterpret_cast<const uint32_t *>(a.w.p2) + c;
    const unsigned short *dp = reinterpret_cast<const unsigned short *>(a.w.p3);

    auto load = [&](const WarpCursor &cu, Q6kRegs &r) {
        const int sb = cu.g * 8 + sbi;
        r.A = r.B = r.H = make_uint4(0u, 0u, 0u, 0u);
        r.sc = 0u; r.d = 0u;
        if (cu.u < n_units && sb < nsb) {
            const size_t blk = (size_t)cu.row * nsb + sb;
            r.A = ldg_stream_u4(lo + blk * 8);
            r.B = ldg_stream_u4(lo + blk * 8 + 4);
            r.H = ldg_stream_u4(hi + blk * 4);
            r.sc = __ldg(scp + blk * 4);
            r.d = __ldg(dp + blk);
        }
    };

    WarpCursor nx;
    cursor_set(nx, warp, n_units, S, G8, r_begin);
    Q6kRegs rn;
    load(nx, rn);
    grid_dependency_wait();
    stage_q8k<MT, PREQ, true>(a, xq, sx, bs, nsb, Kpad);
    __syncthreads();
    grid_launch_dependents();

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.0f;
    while (nx.u < n_units) {
        const WarpCursor cu = nx;
        const Q6kRegs rc = rn;
        cursor_advance(nx, n_units, S, G8, r_begin);
        load(nx, rn);
        const int sb = cu.g * 8 + sbi;
        if (sb < nsb) {
            const float d = f16_bits_to_f32(rc.d);
            const uint32_t Aw[4] = {rc.A.x, rc.A.y, rc.A.z, rc.A.w};
            const uint32_t Bw[4] = {rc.B.x, rc.B.y, rc.B.z, rc.B.w};
            const uint32_t Hw[4] = {rc.H.x, rc.H.y, rc.H.z, rc.H.w};
            // six-bit values 0..63 of the four 16-weight groups t = 0..3 of this chunk
            uint32_t w6[4][4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                w6[0][k] = (Aw[k] & 0x0f0f0f0fu) | ((Hw[k] << 4) & 0x30303030u);
                w6[1][k] = (Bw[k] & 0x0f0f0f0fu) | ((Hw[k] << 2) & 0x30303030u);
                w6[2][k] = ((Aw[k] >> 4) & 0x0f0f0f0fu) | (Hw[k] & 0x30303030u);
                w6[3][k] = ((Bw[k] >> 4) & 0x0f0f0f0fu) | ((Hw[k] >> 2) & 0x30303030u);
            }
            const int s0 = (int)(signed char)(rc.sc & 0xffu), s1 = (int)(signed char)((rc.sc >> 8) & 0xffu);
            const int s2 = (int)(signed char)((rc.sc >> 16) & 0xffu), s3 = (int)(signed char)(rc.sc >> 24);
            const int st[4] = {s0, s1, s2, s3};
            const int u0 = xq_unit(sb, c, 0);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const uint4 *xm = reinterpret_cast<const uint4 *>(xq + (size_t)m * Kpad) + u0;
                const int4 b4 = *reinterpret_cast<const int4 *>(bs + (m * nsb + sb) * 16 + 4 * c);
                const int bsum[4] = {b4.x, b4.y, b4.z, b4.w};
                int isum = 0;
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const uint4 X = xm[t * 8];
                    int it = dp4a_u8s8(w6[t][0], X.x, 0);   // exact int32 dot of 16 weights
                    it = dp4a_u8s8(w6[t][1], X.y, it);
                    it = dp4a_u8s8(w6[t][2], X.z, it);
                    it = dp4a_u8s8(w6[t][3], X.w, it);
                    if (DUMP && m == 0) a.idots[(size_t)cu.row * (nsb * 16) + sb * 16 + 4 * c + t] = it;
                    isum += st[t] * (it - 32 * bsum[t]);    // s*(i) - 32*s*(x sum), exact
                }
                acc[m] += (sx[m * nsb + sb] * d) * (float)isum;
            }
        }
        if (!DUMP && cu.g + 1 == cu.g_end) unit_done<MT>(acc, cu, S, part, a, lane);
    }
    if (!DUMP) finish_rows<MT>(part, R, S, r_begin, a);
}

template <int MT, bool PREQ, bool DUMP>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_q6k_kernel(const GemvArgs a) { gemv_q6k_body<MT, PREQ, DUMP>(a); }

// Grouped form: the group's rows (count and first position read from device memory, so the launch
// is capture-safe whatever the routing) are processed MT at a time (eight, or fewer when K is long and shared memory is short); passes after the first
// find the group's weights in L2.
template <int MT>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_q6k_grouped_kernel(const GemvArgs a) {
    const int count = __ldg(a.grp_count), off = __ldg(a.grp_offset);
    for (int mb = 0; mb < count; mb += MT) {
        GemvArgs b = a;
        b.M = count - mb < MT ? count - mb : MT;
        if (a.row_index) b.row_index = a.row_index + off + mb;
        else { b.q = a.q + (size_t)(off + mb) * a.K; b.scales = a.scales + (size_t)(off + mb) * (a.K >> 8); b.bsums = a.bsums + (size_t)(off + mb) * (a.K >> 5); }
        b.y = a.y + (size_t)(off + mb) * a.N;
        gemv_q6k_body<MT, true, false>(b);
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------- Q8_0
// f32 activations in shared memory.  A group is 2048 weights of one row: lane l owns the four
// 16-weight pieces j*512 + 16l (j = 0..3), so every weight load instruction of the warp
// reads 512 contiguous bytes.  x is stored so that, for a fixed piece and float4 index, the
// 32 lanes read 512 contiguous bytes.
struct Q80Regs { uint4 W[4]; uint32_t d[4]; };

__device__ __forceinline__ float s8_to_f32(uint32_t w_flipped, int i) {
    // w_flipped = word ^ 0x80808080: byte + 128 in 0..255 goes into the mantissa of 2^23
    const uint32_t bits = __byte_perm(w_flipped, 0x4b000000u, 0x7540 | i);
    return __uint_as_float(bits) - 8388736.0f;
}

template <int MT>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_q80_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int K = a.K, G8 = (K + 2047) >> 11, S = a.S;
    const int Kpad = G8 * 2048;
    float4 *xs = reinterpret_cast<float4 *>(smem);                         // [MT][Kpad/4]
    float *part = reinterpret_cast<float *>(smem + (size_t)MT * Kpad * 4);

    int r_begin, R;
    cta_rows(a, r_begin, R);
    const int n_units = R * S;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint4 *qp = reinterpret_cast<const uint4 *>(a.w.p0);
    const unsigned short *dp = reinterpret_cast<const unsigned short *>(a.w.p1);

    auto load = [&](const WarpCursor &cu, Q80Regs &r) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k0 = cu.g * 2048 + j * 512 + lane * 16;
            r.W[j] = make_uint4(0u, 0u, 0u, 0u);
            r.d[j] = 0u;
            if (cu.u < n_units && k0 < K) {
                const size_t row = (size_t)cu.row;
                r.W[j] = ldg_stream_u4(qp + (row * K + k0) / 16);
                r.d[j] = __ldg(dp + row * (K / 32) + (k0 >> 5));
            }
        }
    };

    WarpCursor nx;
    cursor_set(nx, warp, n_units, S, G8, r_begin);
    Q80Regs rn;
    load(nx, rn);
    grid_dependency_wait();
    // stage x: float4 (piece-block pb, lane l, idx p) -> xs[m][pb*128 + p*32 + l]
    for (int idx = threadIdx.x; idx < MT * (Kpad / 4); idx += blockDim.x) {
        const int m = idx / (Kpad / 4), f4 = idx - m * (Kpad / 4);
        const int pb = f4 >> 7, l = (f4 >> 2) & 31, p = f4 & 3;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < a.M && f4 * 4 < K) v = __ldg(reinterpret_cast<const float4 *>(a.x + (size_t)m * K) + f4);
        xs[(size_t)m * (Kpad / 4) + pb * 128 + p * 32 + l] = v;
    }
    __syncthreads();
    grid_launch_dependents();

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.0f;
    while (nx.u < n_units) {
        const WarpCursor cu = nx;
        const Q80Regs rc = rn;
        cursor_advance(nx, n_units, S, G8, r_begin);
        load(nx, rn);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float d = f16_bits_to_f32(rc.d[j]);
            const uint32_t wv[4] = {rc.W[j].x ^ 0x80808080u, rc.W[j].y ^ 0x80808080u, rc.W[j].z ^ 0x80808080u, rc.W[j].w ^ 0x80808080u};
            float wf[16];
#pragma unroll
            for (int p = 0; p < 4; p++)
#pragma unroll
                for (int i = 0; i < 4; i++) wf[p * 4 + i] = s8_to_f32(wv[p], i);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const float4 *xm = xs + (size_t)m * (Kpad / 4) + (cu.g * 4 + j) * 128 + lane;
                float s = 0.0f;
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    const float4 xv = xm[p * 32];
                    s = fmaf(wf[p * 4 + 0], xv.x, s);
                    s = fmaf(wf[p * 4 + 1], xv.y, s);
                    s = fmaf(wf[p * 4 + 2], xv.z, s);
                    s = fmaf(wf[p * 4 + 3], xv.w, s);
                }
                acc[m] = fmaf(d, s, acc[m]);
            }
        }
        if (cu.g + 1 == cu.g_end) unit_done<MT>(acc, cu, S, part, a, lane);
    }
    finish_rows<MT>(part, R, S, r_begin, a);
}

#include "gemv_mma.cuh"

// ---------------------------------------------------------------------------- quant_q8k
__global__ void __launch_bounds__(256) quant_q8k_kernel(const float *x, int8_t *q, float *scales, int32_t *bsums,
                                                         long long n_sb) {
    const int lane = threadIdx.x & 31;
    const long long sb = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (sb >= n_sb) return;
    Q8kLane ql = quant_q8k_warp(x + sb * 256, lane);
    reinterpret_cast<uint2 *>(q + sb * 256)[lane] = ql.packed;
    int s = ql.sum8;
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if ((lane & 3) == 0) bsums[sb * 8 + (lane >> 2)] = s;
    if (lane == 0) scales[sb] = ql.scale;
}

// ---------------------------------------------------------------------------- host side
// Segments per row: 1 when a CTA has at least ~3/4 as many rows as warps, otherwise enough
// segments to give every warp a unit (never more than the row has groups).
static int gemv_segments(size_t rows_max, size_t G8) {
    if (rows_max >= 24) return 1;
    size_t s = (GEMV_WARPS + rows_max - 1) / rows_max;
    if (s > G8) s = G8;
    return s < 1 ? 1 : (int)s;
}

// Q4_K: steps are sixteen super-blocks and the segment count must divide the steps per row.
static int gemv_segments_q4k(size_t rows_max, size_t nsb, size_t warps = GEMV_WARPS) {
    const size_t G = (nsb + 15) / 16;
    if (rows_max >= (warps * 3) / 4) return 1;
    const size_t want = (warps + rows_max - 1) / rows_max;
    size_t best = 1;
    for (size_t s = 1; s <= G && s <= want; s++)
        if (G % s == 0) best = s;
    return (int)best;
}

static size_t gemv_ring_bytes(uint32_t type, int depth) {
    (void)depth;
    return type == OJAS_B200_Q4_K ? (size_t)GEMV_WARPS * 2 * Q4K_STAGE_BYTES : 0;
}

static size_t gemv_smem_bytes(uint32_t type, int MT, size_t K, size_t rows_max, int S, int depth) {
    const size_t nsb = K / 256, G8 = (nsb + 7) / 8;
    const size_t part = (S > 1 ? rows_max * S * MT * 4 : 0) + 16;
    if (type == OJAS_B200_Q8_0) return (size_t)MT * G8 * 2048 * 4 + part;
    const size_t Kpad = ((nsb + 1) / 2) * 512;
    const size_t nb = (type == OJAS_B200_Q6_K) ? 16 : 8;
    return gemv_ring_bytes(type, depth) + (size_t)MT * Kpad + (size_t)sx_floats(MT, (int)nsb) * 4 + (size_t)MT * nsb * nb * 4 + part;
}

// Deepest ring (4, 3 or 2 stages) that leaves room for `mt` rows of activations; 0 if even 2 does not fit.
static int gemv_depth(ojas_b200_ctx *ctx, uint32_t type, int mt, size_t K, size_t rows_max, int S) {
    int want = ctx->gemv_depth >= 2 && ctx->gemv_depth <= 4 ? ctx->gemv_depth : 4;
    for (int d = want; d >= 2; d--)
        if (gemv_smem_bytes(type, mt, K, rows_max, S, d) <= (size_t)ctx->smem_optin) return d;
    return 0;
}

template <typename KernelT>
static int launch_gemv(ojas_b200_ctx *ctx, KernelT kernel, const GemvArgs &args, int grid, size_t smem, const char *name) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "%s: shared memory %zu: %s", name, smem, cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    if (ctx->pdl) {   // let this kernel's weight prefetch overlap the tail of the kernel before it
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args);
    if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "launch %s: %s", name, cudaGetErrorString(e));
    ctx->launches++;
    return 0;
}

// ---- integer tensor-core path (Q4_K, M <= 8): configuration and launch
static int mma_segments(size_t rows_max, size_t nsb, int warps) {
    const size_t tiles = (rows_max + 15) / 16;
    size_t best = 1;
    for (size_t s = 1; s <= nsb; s++) {
        if (nsb % s) continue;
        best = s;
        if (tiles * s >= (size_t)warps) break;
    }
    return (int)best;
}

static size_t mma_smem_bytes(int warps, size_t M, size_t K, size_t rows_max, int S) {
    const size_t nsb = K / 256, tiles = (rows_max + 15) / 16;
    return (size_t)warps * 2 * MMA_STAGE_BYTES + ((M * (K + MMA_XPAD) + 15) & ~(size_t)15) + (size_t)sx_floats((int)M, (int)nsb) * 4 +
           M * nsb * 8 * 4 + (S > 1 ? tiles * S * 128 * ((M + 7) / 8) * 4 : 0) + 16;
}

// Warps per CTA (hi or lo) and segments per tile (a divisor of the super-blocks per row) for the tensor-core GEMVs:
// among the pairs that fit in shared memory, the one whose busiest warp has the fewest super-block steps; ties go to
// more warps, then to more of them busy, then to fewer segments.  Returns the warps, 0 if nothing fits; sets S, smem.
template <typename SmemFn>
static int mma_pick(size_t limit, size_t rows_max, size_t nsb, int warps_hi, int warps_lo, SmemFn smem_of, int &S, size_t &smem) {
    const size_t tiles = (rows_max + 15) / 16;
    int best_warps = 0;
    size_t best_steps = ~(size_t)0, best_busy = 0;
    for (int warps = warps_hi; warps >= warps_lo; warps >>= 1) {
        for (size_t s = 1; s <= nsb; s++) {
            if (nsb % s) continue;
            const size_t bytes = smem_of(warps, (int)s);
            if (bytes > limit) continue;
            const size_t units = tiles * s;
            const size_t steps = ((units + (size_t)warps - 1) / (size_t)warps) * (nsb / s);
            const size_t busy = units < (size_t)warps ? units : (size_t)warps;
            if (steps < best_steps || (steps == best_steps && warps == best_warps && busy > best_busy)) {
                best_steps = steps;
                best_busy = busy;
                best_warps = warps;
                S = (int)s;
                smem = bytes;
            }
        }
    }
    return best_warps;
}

// Fills S / row partition and picks 32 or 16 warps; returns 0 if neither fits.
static int mma_plan(ojas_b200_ctx *ctx, GemvArgs &a, int &grid, size_t &smem) {
    grid = ctx->sm_count < a.N ? ctx->sm_count : a.N;
    const size_t rows_max = ((size_t)a.N + grid - 1) / grid;
    a.rows_base = a.N / grid;
    a.rows_rem = a.N % grid;
    const size_t M = (size_t)a.M, K = (size_t)a.K;
    return mma_pick((size_t)ctx->smem_optin, rows_max, K / 256, 32, 16,
                    [&](int warps, int S) { return mma_smem_bytes(warps, M, K, rows_max, S); }, a.S, smem);
}

template <typename KernelT>
static int launch_gemv_threads(ojas_b200_ctx *ctx, KernelT kernel, const GemvArgs &args, int grid, int threads, size_t smem, const char *name) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "%s: shared memory %zu: %s", name, smem, cudaGetErrorString(e));
        // ask for the largest shared-memory carve-out, so that two half-size CTAs can share an SM
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    if (ctx->pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args);
    if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "launch %s: %s", name, cudaGetErrorString(e));
    ctx->launches++;
    return 0;
}

// Returns 1 if the shape does not fit this path (the caller falls back to the dp4a kernels), else a status.
static int gemv_mma_launch(ojas_b200_ctx *ctx, bool preq, GemvArgs a) {
    int grid;
    size_t smem;
    const int warps = mma_plan(ctx, a, grid, smem);
    if (warps == 0) return 1;
    if (warps == 32) {
        if (preq) return launch_gemv_threads(ctx, gemv_q4k_mma_kernel<32, true>, a, grid, 1024, smem, "gemv_q4k_mma_q8k");
        return launch_gemv_threads(ctx, gemv_q4k_mma_kernel<32, false>, a, grid, 1024, smem, "gemv_q4k_mma");
    }
    if (preq) return launch_gemv_threads(ctx, gemv_q4k_mma_kernel<16, true>, a, grid, 512, smem, "gemv_q4k_mma_q8k");
    return launch_gemv_threads(ctx, gemv_q4k_mma_kernel<16, false>, a, grid, 512, smem, "gemv_q4k_mma");
}

// ---- the same for Q6_K: 16 or 8 warps (a stage is 3840 bytes), per-16 activation sums
static size_t mma6_smem_bytes(int warps, size_t M, size_t K, size_t rows_max, int S) {
    const size_t nsb = K / 256, tiles = (rows_max + 15) / 16;
    return (size_t)warps * 2 * MMA6_STAGE_BYTES + ((M * (K + MMA_XPAD) + 15) & ~(size_t)15) + (size_t)sx_floats((int)M, (int)nsb) * 4 +
           M * nsb * 16 * 4 + (S > 1 ? tiles * S * 128 * 4 : 0) + 16;
}

static int mma6_plan(ojas_b200_ctx *ctx, GemvArgs &a, int &grid, size_t &smem) {
    grid = ctx->sm_count < a.N ? ctx->sm_count : a.N;
    const size_t rows_max = ((size_t)a.N + grid - 1) / grid;
    a.rows_base = a.N / grid;
    a.rows_rem = a.N % grid;
    const size_t M = (size_t)a.M, K = (size_t)a.K;
    return mma_pick((size_t)ctx->smem_optin, rows_max, K / 256, 16, 8,
                    [&](int warps, int S) { return mma6_smem_bytes(warps, M, K, rows_max, S); }, a.S, smem);
}

static int gemv_mma6_launch(ojas_b200_ctx *ctx, bool preq, GemvArgs a) {
    int grid;
    size_t smem;
    const int warps = mma6_plan(ctx, a, grid, smem);
    if (warps == 0) return 1;
    if (warps == 16) {
        if (preq) return launch_gemv_threads(ctx, gemv_q6k_mma_kernel<16, true>, a, grid, 512, smem, "gemv_q6k_mma_q8k");
        return launch_gemv_threads(ctx, gemv_q6k_mma_kernel<16, false>, a, grid, 512, smem, "gemv_q6k_mma");
    }
    if (preq) return launch_gemv_threads(ctx, gemv_q6k_mma_kernel<8, true>, a, grid, 256, smem, "gemv_q6k_mma_q8k");
    return launch_gemv_threads(ctx, gemv_q6k_mma_kernel<8, false>, a, grid, 256, smem, "gemv_q6k_mma");
}

// ---- Q8_0 batches on the f16 tensor-core path: activations as two f16 terms (4 bytes per value, like fp32)
static size_t mma8_smem_bytes(int warps, size_t M, size_t K, size_t rows_max, int S) {
    const size_t nsb = K / 256, tiles = (rows_max + 15) / 16;
    return (size_t)warps * 2 * MMA8_STAGE_BYTES + 2 * M * (K + MMA8_XPAD) * 2 + (size_t)sx_floats((int)M, (int)nsb) * 4 +
           (S > 1 ? tiles * S * 128 * 4 : 0) + 16;
}

static int mma8_plan(ojas_b200_ctx *ctx, GemvArgs &a, int &grid, size_t &smem) {
    grid = ctx->sm_count < a.N ? ctx->sm_count : a.N;
    const size_t rows_max = ((size_t)a.N + grid - 1) / grid;
    a.rows_base = a.N / grid;
    a.rows_rem = a.N % grid;
    const size_t M = (size_t)a.M, K = (size_t)a.K;
    return mma_pick((size_t)ctx->smem_optin, rows_max, K / 256, 16, 8,
                    [&](int warps, int S) { return mma8_smem_bytes(warps, M, K, rows_max, S); }, a.S, smem);
}

// Batches of up to eight rows; a batch whose activations do not fit in shared memory is cut into smaller
// ones.  Returns 1 if not even one row fits (the caller falls back to the per-lane kernel).
static int gemv_mma8_run(ojas_b200_ctx *ctx, GemvArgs args, size_t M) {
    int cap = 0, grid = 0;
    size_t smem = 0;
    for (int m = 8; m >= 1 && !cap; m >>= 1) {
        GemvArgs t = args;
        t.M = m;
        if (mma8_plan(ctx, t, grid, smem)) cap = m;
    }
    if (!cap) return 1;
    // a batch is split into its two f16 terms once per call (context scratch: 4 bytes per value + factors) instead
    // of once per CTA
    const size_t values = M * (size_t)args.K;
    const bool pre = M >= 2 && ctx->act_scratch && values >= 16384 && values * 4 + values / 256 * 4 <= OJAS_ACT_SCRATCH_BYTES;
    __half *shi = (__half *)ctx->act_scratch, *slo = shi + values;
    float *sfx = (float *)(slo + values);
    if (pre) {
        const long long n_sb = (long long)(values / 256);
        q80_split_kernel<<<(unsigned)((n_sb + 7) / 8), 256, 0, ctx->stream>>>(args.x, (uint4 *)shi, (uint4 *)slo, sfx, n_sb);
        OJAS_LAUNCH_CHECK(ctx, "q80_split");
    }
    for (size_t m0 = 0; m0 < M; m0 += (size_t)cap) {
        GemvArgs b = args;
        b.M = (int)((M - m0) < (size_t)cap ? (M - m0) : (size_t)cap);
        b.x = args.x + m0 * args.K;
        b.y = args.y + m0 * args.N;
        if (pre) {
            b.q = (const int8_t *)(shi + m0 * args.K);
            b.bsums = (const int32_t *)(slo + m0 * args.K);
            b.scales = sfx + m0 * ((size_t)args.K / 256);
        }
        const int warps = mma8_plan(ctx, b, grid, smem);
        int rc;
        if (warps == 16) rc = pre ? launch_gemv_threads(ctx, gemv_q80_mma_kernel<16, true>, b, grid, 512, smem, "gemv_q80_mma")
                                  : launch_gemv_threads(ctx, gemv_q80_mma_kernel<16, false>, b, grid, 512, smem, "gemv_q80_mma");
        else rc = pre ? launch_gemv_threads(ctx, gemv_q80_mma_kernel<8, true>, b, grid, 256, smem, "gemv_q80_mma")
                      : launch_gemv_threads(ctx, gemv_q80_mma_kernel<8, false>, b, grid, 256, smem, "gemv_q80_mma");
        if (rc) return rc;
    }
    return 0;
}

static int pick_mt(size_t M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8; }

// One launch over at most 8 activation rows.
static int gemv_launch_batch(ojas_b200_ctx *ctx, uint32_t type, bool preq, bool dump, GemvArgs args) {
    const int grid = ctx->sm_count < args.N ? ctx->sm_count : args.N;
    const size_t rows_max = ((size_t)args.N + grid - 1) / grid;
    const int MT = pick_mt((size_t)args.M);
    const size_t G8 = ((size_t)args.K / 256 + 7) / 8;
    args.S = dump ? 1 : (type == OJAS_B200_Q4_K ? gemv_segments_q4k(rows_max, (size_t)args.K / 256) : gemv_segments(rows_max, G8));
    args.rows_base = args.N / grid;
    args.rows_rem = args.N % grid;
    args.depth = gemv_depth(ctx, type, MT, (size_t)args.K, rows_max, args.S);
    const size_t smem = gemv_smem_bytes(type, MT, (size_t)args.K, rows_max, args.S, args.depth ? args.depth : 2);
    if (args.depth == 0 || smem > (size_t)ctx->smem_optin)
        return ojas_fail(ctx, OJAS_B200_E_LIMIT, "gemv: %zu bytes of shared memory needed, %d available", smem, ctx->smem_optin);
#define GEMV_CASE(KERNEL, NAME)                                                 \
    switch (MT) {                                                               \
    case 1: return launch_gemv(ctx, KERNEL(1), args, grid, smem, NAME);         \
    case 2: return launch_gemv(ctx, KERNEL(2), args, grid, smem, NAME);         \
    case 4: return launch_gemv(ctx, KERNEL(4), args, grid, smem, NAME);         \
    default: return launch_gemv(ctx, KERNEL(8), args, grid, smem, NAME);        \
    }
    if (type == OJAS_B200_Q4_K && MT == 1 && !dump && ctx->gemv_slim != 0) {
        // single-row calls on matrices small enough that one kernel cannot hide its own latency: the half-size
        // kernel, which overlaps with its neighbours in the stream
        const size_t bytes_per_cta = rows_max * ((size_t)args.K / 256) * 144;
        if (ctx->gemv_slim == 2 || bytes_per_cta <= 160 * 1024) {
            GemvArgs b = args;
            b.S = gemv_segments_q4k(rows_max, (size_t)args.K / 256, GEMV_SLIM_WARPS);
            const size_t nsb = (size_t)args.K / 256, Kpad = ((nsb + 1) / 2) * 512;
            const size_t smem2 = (size_t)GEMV_SLIM_WARPS * 2 * Q4K_STAGE_BYTES + Kpad + (size_t)sx_floats(1, (int)nsb) * 4 + nsb * 8 * 4 +
                                 (b.S > 1 ? rows_max * b.S * 4 : 0) + 16;
            if (smem2 <= 100 * 1024) {
                if (preq) return launch_gemv_threads(ctx, gemv_q4k_slim_kernel<true>, b, grid, GEMV_SLIM_WARPS * 32, smem2, "gemv_q4k_slim_q8k");
                return launch_gemv_threads(ctx, gemv_q4k_slim_kernel<false>, b, grid, GEMV_SLIM_WARPS * 32, smem2, "gemv_q4k_slim");
            }
        }
    }
    if (type == OJAS_B200_Q4_K) {
        if (dump) return launch_gemv(ctx, gemv_q4k_kernel<1, false, true>, args, grid, smem, "gemv_q4k_idots");
        if (preq) {
#define K4P(m) gemv_q4k_kernel<m, true, false>
            GEMV_CASE(K4P, "gemv_q4k_q8k")
        }
#define K4(m) gemv_q4k_kernel<m, false, false>
        GEMV_CASE(K4, "gemv_q4k")
    }
    if (type == OJAS_B200_Q6_K) {
        if (dump) return launch_gemv(ctx, gemv_q6k_kernel<1, false, true>, args, grid, smem, "gemv_q6k_idots");
        if (preq) {
#define K6P(m) gemv_q6k_kernel<m, true, false>
            GEMV_CASE(K6P, "gemv_q6k_q8k")
        }
#define K6(m) gemv_q6k_kernel<m, false, false>
        GEMV_CASE(K6, "gemv_q6k")
    }
    if (type == OJAS_B200_Q8_0) {
#define K8(m) gemv_q80_kernel<m>
        GEMV_CASE(K8, "gemv_q80")
    }
    return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: unsupported GGUF type %u", type);
}

// Largest batch tile whose activations fit in shared memory.
static int gemv_max_mt(ojas_b200_ctx *ctx, uint32_t type, size_t K, size_t N) {
    const int grid = ctx->sm_count < (int)N ? ctx->sm_count : (int)N;
    const size_t rows_max = (N + grid - 1) / grid;
    const int S = type == OJAS_B200_Q4_K ? gemv_segments_q4k(rows_max, K / 256) : gemv_segments(rows_max, (K / 256 + 7) / 8);
    for (int mt = 8; mt >= 1; mt >>= 1)
        if (gemv_depth(ctx, type, mt, K, rows_max, S) != 0) return mt;
    return 0;
}

static int gemv_check(ojas_b200_ctx *ctx, uint32_t type, int form, const void *w, const float *y, const float *bias,
                      size_t K, size_t N, size_t M) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (type != OJAS_B200_Q4_K && type != OJAS_B200_Q6_K && type != OJAS_B200_Q8_0)
        return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: unsupported GGUF type %u", type);
    if (!w || !y) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: null pointer");
    if (K == 0 || K % 256 != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: K=%zu must be a positive multiple of 256", K);
    if (N == 0 || N > 0x7fffffffu / 64) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: N=%zu out of range", N);
    if (M == 0 || M > OJAS_B200_GEMV_MAX_M) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: M=%zu must be 1..%d", M, OJAS_B200_GEMV_MAX_M);
    if (form < OJAS_B200_PLAIN || form > OJAS_B200_BIAS) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: unknown store form %d", form);
    if (form == OJAS_B200_BIAS && !bias) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: bias form without a bias pointer");
    if (((uintptr_t)w & 255) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: weight pointer must be 256-byte aligned");
    return 0;
}

// A batch of K-quant rows from fp32 activations: every CTA of the GEMV would quantize the whole batch for
// itself (M * K / 256 warp tasks each).  From a few dozen tasks per warp on that prologue outweighs the
// matrix, so the batch is quantized once into the context's scratch and the GEMV copies the result.
static bool gemv_prequantize(ojas_b200_ctx *ctx, uint32_t type, bool preq, GemvArgs &args, size_t M) {
    if (preq || type == OJAS_B200_Q8_0 || M < 3 || !ctx->act_scratch) return false;
    const size_t values = M * (size_t)args.K;
    if (values > OJAS_ACT_SCRATCH_VALUES || values < 32768) return false;
    int8_t *q = (int8_t *)ctx->act_scratch;
    float *scales = (float *)(q + OJAS_ACT_SCRATCH_VALUES);
    int32_t *bsums = (int32_t *)(scales + OJAS_ACT_SCRATCH_VALUES / 256);
    const long long n_sb = (long long)(values / 256);
    quant_q8k_kernel<<<(unsigned)((n_sb + 7) / 8), 256, 0, ctx->stream>>>(args.x, q, scales, bsums, n_sb);
    if (cudaGetLastError() != cudaSuccess) return false;
    ctx->launches++;
    args.x = nullptr;
    args.q = q;
    args.scales = scales;
    args.bsums = bsums;
    return true;
}

static int gemv_run(ojas_b200_ctx *ctx, uint32_t type, bool preq, GemvArgs args, size_t M) {
    if (ctx->gemv_mma != 0 && gemv_prequantize(ctx, type, preq, args, M)) preq = true;
    // K-quant batches of 3..8 rows and Q8_0 batches of 2..8 rows (or every call when the option says so) take the tensor-core paths
    if (type == OJAS_B200_Q4_K && ctx->gemv_mma != 0 && (M >= 3 || ctx->gemv_mma == 2)) {   // at two rows the per-lane loop is still faster
        GemvArgs b = args;
        b.M = (int)M;
        const int rc = gemv_mma_launch(ctx, preq, b);
        if (rc != 1) return rc;
    }
    if (type == OJAS_B200_Q8_0 && !preq && ctx->gemv_mma != 0 && (M >= 2 || ctx->gemv_mma == 2)) {
        const int rc = gemv_mma8_run(ctx, args, M);
        if (rc != 1) return rc;
    }
    if (type == OJAS_B200_Q6_K && ctx->gemv_mma != 0 && (M >= 3 || ctx->gemv_mma == 2)) {
        GemvArgs b = args;
        b.M = (int)M;
        const int rc = gemv_mma6_launch(ctx, preq, b);
        if (rc != 1) return rc;
    }
    const int cap = gemv_max_mt(ctx, type, (size_t)args.K, (size_t)args.N);
    if (cap == 0) return ojas_fail(ctx, OJAS_B200_E_LIMIT, "gemv: K=%d does not fit in shared memory", args.K);
    const size_t nsb = (size_t)args.K / 256;
    for (size_t m0 = 0; m0 < M; m0 += (size_t)cap) {
        GemvArgs b = args;
        b.M = (int)((M - m0) < (size_t)cap ? (M - m0) : (size_t)cap);
        if (args.x) b.x = args.x + m0 * args.K;
        if (args.q) { b.q = args.q + m0 * args.K; b.scales = args.scales + m0 * nsb; b.bsums = args.bsums + m0 * nsb * 8; }
        b.y = args.y + m0 * args.N;
        int rc = gemv_launch_batch(ctx, type, preq, false, b);
        if (rc) return rc;
    }
    return 0;
}

static int gemv_max_mt(ojas_b200_ctx *ctx, uint32_t type, size_t K, size_t N);

// One grouped launch (see gemv_*_grouped_kernel): weights `planes` [N, K], activations pre-quantized.
int ojas_gemv_grouped(ojas_b200_ctx *ctx, uint32_t type, const WeightPlanes &planes, const int8_t *q, const float *scales,
                      const int32_t *bsums, const int *row_index, const int *grp_count, const int *grp_offset, float *y,
                      size_t K, size_t N) {
    if (type != OJAS_B200_Q4_K && type != OJAS_B200_Q6_K)
        return ojas_fail(ctx, OJAS_B200_E_UNSUPPORTED, "grouped gemv: only Q4_K and Q6_K experts are supported");
    GemvArgs a{};
    a.q = q; a.scales = scales; a.bsums = bsums; a.w = planes; a.y = y;
    a.row_index = row_index; a.grp_count = grp_count; a.grp_offset = grp_offset;
    a.K = (int)K; a.N = (int)N; a.form = OJAS_B200_PLAIN;
    const int grid = ctx->sm_count < a.N ? ctx->sm_count : a.N;
    const size_t rows_max = ((size_t)a.N + grid - 1) / grid;
    const size_t G8 = (K / 256 + 7) / 8;
    a.S = type == OJAS_B200_Q4_K ? gemv_segments_q4k(rows_max, K / 256) : gemv_segments(rows_max, G8);
    a.rows_base = a.N / grid;
    a.rows_rem = a.N % grid;
    if (type == OJAS_B200_Q4_K && ctx->gemv_mma != 0) {
        GemvArgs b = a;
        int g2;
        size_t smem2;
        b.M = 16;                                     // sixteen rows per pass (16 warps) when their activations fit beside the ring
        mma_plan(ctx, b, g2, smem2);                  // sets the grid and the row split
        b.S = mma_segments(rows_max, K / 256, 16);
        smem2 = mma_smem_bytes(16, 16, K, rows_max, b.S);
        if (smem2 <= (size_t)ctx->smem_optin)
            return launch_gemv_threads(ctx, gemv_q4k_mma_grouped_kernel<16, 2>, b, g2, 512, smem2, "gemv_q4k_mma_grouped16");
        b = a;
        b.M = 8;
        const int warps = mma_plan(ctx, b, g2, smem2);
        if (warps == 32) return launch_gemv_threads(ctx, gemv_q4k_mma_grouped_kernel<32>, b, g2, 1024, smem2, "gemv_q4k_mma_grouped");
        if (warps == 16) return launch_gemv_threads(ctx, gemv_q4k_mma_grouped_kernel<16>, b, g2, 512, smem2, "gemv_q4k_mma_grouped");
    }
    if (type == OJAS_B200_Q6_K && ctx->gemv_mma != 0) {
        GemvArgs b = a;
        b.M = 8;
        int g2;
        size_t smem2;
        const int warps = mma6_plan(ctx, b, g2, smem2);
        if (warps == 16) return launch_gemv_threads(ctx, gemv_q6k_mma_grouped_kernel<16>, b, g2, 512, smem2, "gemv_q6k_mma_grouped");
        if (warps == 8) return launch_gemv_threads(ctx, gemv_q6k_mma_grouped_kernel<8>, b, g2, 256, smem2, "gemv_q6k_mma_grouped");
    }
    const int mt = gemv_max_mt(ctx, type, K, N);      // rows per pass: as many as fit beside the weight ring
    if (mt < 2) return ojas_fail(ctx, OJAS_B200_E_LIMIT, "grouped gemv: K=%zu does not fit in shared memory", K);
    a.M = mt;
    a.depth = gemv_depth(ctx, type, mt, K, rows_max, a.S);
    const size_t smem = gemv_smem_bytes(type, mt, K, rows_max, a.S, a.depth);
    if (type == OJAS_B200_Q4_K) {
        if (mt == 8) return launch_gemv(ctx, gemv_q4k_grouped_kernel<8>, a, grid, smem, "gemv_q4k_grouped");
        if (mt == 4) return launch_gemv(ctx, gemv_q4k_grouped_kernel<4>, a, grid, smem, "gemv_q4k_grouped");
        return launch_gemv(ctx, gemv_q4k_grouped_kernel<2>, a, grid, smem, "gemv_q4k_grouped");
    }
    if (mt == 8) return launch_gemv(ctx, gemv_q6k_grouped_kernel<8>, a, grid, smem, "gemv_q6k_grouped");
    if (mt == 4) return launch_gemv(ctx, gemv_q6k_grouped_kernel<4>, a, grid, smem, "gemv_q6k_grouped");
    return launch_gemv(ctx, gemv_q6k_grouped_kernel<2>, a, grid, smem, "gemv_q6k_grouped");
}

extern "C" int ojas_b200_gemv(ojas_b200_ctx *ctx, uint32_t type, int form, const float *x, const void *w, float *y,
                              const float *bias, size_t K, size_t N, size_t M) {
    int rc = gemv_check(ctx, type, form, w, y, bias, K, N, M);
    if (rc) return rc;
    if (!x) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: null activation pointer");
    if (((uintptr_t)x & 15) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: x must be 16-byte aligned");
    GemvArgs a{};
    a.x = x; a.w = weight_planes(type, w, N, K); a.y = y; a.bias = bias;
    a.K = (int)K; a.N = (int)N; a.M = (int)M; a.form = form;
    return gemv_run(ctx, type, false, a, M);
}

extern "C" int ojas_b200_gemv_q8k(ojas_b200_ctx *ctx, uint32_t type, int form, const int8_t *q, const float *scales,
                                  const int32_t *bsums, const void *w, float *y, const float *bias, size_t K, size_t N,
                                  size_t M) {
    int rc = gemv_check(ctx, type, form, w, y, bias, K, N, M);
    if (rc) return rc;
    if (type == OJAS_B200_Q8_0)
        return ojas_fail(ctx, OJAS_B200_E_UNSUPPORTED, "gemv_q8k: Q8_0 rows meet f32 activations, not Q8_K blocks");
    if (!q || !scales || !bsums) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv_q8k: null activation pointer");
    if (((uintptr_t)q & 15) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv_q8k: q must be 16-byte aligned");
    GemvArgs a{};
    a.q = q; a.scales = scales; a.bsums = bsums; a.w = weight_planes(type, w, N, K); a.y = y; a.bias = bias;
    a.K = (int)K; a.N = (int)N; a.M = (int)M; a.form = form;
    return gemv_run(ctx, type, true, a, M);
}

extern "C" int ojas_b200_gemv_idots(ojas_b200_ctx *ctx, uint32_t type, const float *x, const void *w, int32_t *idots,
                                    size_t K, size_t N) {
    float dummy;
    int rc = gemv_check(ctx, type, OJAS_B200_PLAIN, w, &dummy, nullptr, K, N, 1);
    if (rc) return rc;
    if (type == OJAS_B200_Q8_0) return ojas_fail(ctx, OJAS_B200_E_UNSUPPORTED, "gemv_idots: Q8_0 has no integer block dots");
    if (!x || !idots) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv_idots: null pointer");
    GemvArgs a{};
    a.x = x; a.w = weight_planes(type, w, N, K); a.idots = idots;
    a.K = (int)K; a.N = (int)N; a.M = 1; a.form = OJAS_B200_PLAIN;
    return gemv_launch_batch(ctx, type, false, true, a);
}

extern "C" int ojas_b200_quant_q8k(ojas_b200_ctx *ctx, const float *x, size_t M, size_t K, int8_t *q, float *scales,
                                   int32_t *bsums) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!x || !q || !scales || !bsums) return ojas_fail(ctx, OJAS_B200_E_ARG, "quant_q8k: null pointer");
    if (K == 0 || K % 256 != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "quant_q8k: K=%zu must be a positive multiple of 256", K);
    if (M == 0) return 0;
    if (((uintptr_t)x & 15) != 0 || ((uintptr_t)q & 7) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "quant_q8k: misaligned pointer");
    const long long n_sb = (long long)M * (long long)(K / 256);
    const long long blocks = (n_sb + 7) / 8;
    if (blocks > 0x7fffffffLL) return ojas_fail(ctx, OJAS_B200_E_ARG, "quant_q8k: too many super-blocks");
    quant_q8k_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, q, scales, bsums, n_sb);
    OJAS_LAUNCH_CHECK(ctx, "quant_q8k");
    return 0;
}
