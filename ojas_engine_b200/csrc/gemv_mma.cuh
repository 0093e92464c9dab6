// Small batches of activation rows against Q4_K (and, in the batch kernel, Q6_K) weights on the integer tensor-core path
// (included by gemv.cu):
// 3..8 rows of a decode batch, and the expert groups of the mixture-of-experts FFN (up to 32 rows per pass, every
// expert and both of gate / up in ONE launch).  Same tiles, same ring of bulk-copied stages and same work split as
// the single-row kernel; what changes is the inside of a step.
//
// A step is 32 weight rows x one super-block, worked as two tiles of 16 rows with
//   mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32     (A = 16 rows x 32 nibbles as bytes, B = 32 int8 x 8 tokens)
// one MMA per sub-block and token tile, so every accumulator is the exact int32 sub-block dot of dot_q4k
// (crates/ojas-cpu/src/cpu_math.rs:609-635) for 16 rows x 8 tokens at once.  The k order of an MMA is free as long as
// A and B agree: lane (g, q) supplies the eight weights 8q .. 8q+7 of the sub-block, which are the low (or high)
// nibbles of eight CONTIGUOUS bytes of row g's tile (one 8-byte load, no shuffling), against activations
// 8q .. 8q+7 of token g (one 8-byte load from a token-major copy padded so that the loads do not conflict).
// High nibbles stay in place (x16) and the accumulator is shifted down afterwards.  The mins term
// sum_j m_j * bsum_j is two more MMAs per super-block (A = the eight 6-bit mins as bytes, B = the low / high bytes
// of the tokens' block sums).  Scales and mins are decoded to bytes once per row and super-block with word-wide
// operations.
//
// The launch walks JOBS: (expert, pass of up to NT of its rows, weight tensor).  Row counts and offsets are read on
// the device (capture-safe whatever the routing), an expert without rows costs nothing, and the weight prefetch runs
// across job boundaries while the CTA combines the finished job and stages the next activations.
#pragma once

struct BatchArgs {
    const uint8_t *w[2];          // weight tensors (gate, up: they share the activations), experts stacked along N
    float *y[2];                  // outputs [positions, N], one per weight tensor
    int nw;
    size_t expert_bytes;          // distance between consecutive experts in a weight tensor
    const float *x;               // f32 activation rows [rows, K]: quantized by the kernel itself (small batches); null: q / scales / bsums
    const int8_t *q;              // quantized activation rows [rows, K] (ojas_b200_quant_q8k form)
    const float *scales;          // [rows, K/256]
    const int32_t *bsums;         // [rows, K/32]
    const int *row_index;         // source row of sorted position p (null: p itself)
    const int *counts, *offsets;  // per expert, on the device (null: one group of M rows at position 0)
    const float *bias;
    unsigned *status;
    int form;
    int E, M, K, N, nsb;
    int units_base, units_rem;    // CTA b owns units_base (+1 if b < units_rem) 8-row units of every expert
    int nst_log, S_log, T_log, P;
};

__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The same with a zero accumulator input (no registers to clear before the MMA).
__device__ __forceinline__ void mma_u8s8_z(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}

struct BatchJob {
    int e, mb, wsel;              // expert, first row of the pass inside the expert's group, weight tensor
    int count, off;               // rows of the expert and position of its first row
};

template <int NT>
__device__ __forceinline__ bool batch_job_first(const BatchArgs &a, BatchJob &j) {
    j.e = -1; j.mb = 0; j.wsel = 0; j.count = 0; j.off = 0;
    for (int e = 0; e < a.E; e++) {
        const int c = a.counts ? __ldg(a.counts + e) : a.M;
        if (c > 0) { j.e = e; j.count = c; j.off = a.offsets ? __ldg(a.offsets + e) : 0; return true; }
    }
    return false;
}
template <int NT>
__device__ __forceinline__ bool batch_job_next(const BatchArgs &a, BatchJob &j) {
    if (j.wsel + 1 < a.nw) { j.wsel++; return true; }
    j.wsel = 0;
    if (j.mb + NT < j.count) { j.mb += NT; return true; }
    j.mb = 0;
    for (int e = j.e + 1; e < a.E; e++) {
        const int c = a.counts ? __ldg(a.counts + e) : a.M;
        if (c > 0) { j.e = e; j.count = c; j.off = a.offsets ? __ldg(a.offsets + e) : 0; return true; }
    }
    return false;
}

// Shared-memory bytes of the activations of one pass: NT rows of K + pad int8 (the pad spreads the eight tokens of a
// load over the banks: 32 bytes for the 8-byte loads of Q4_K, 16 for the 4-byte loads of Q6_K), then per row and
// super-block the block sums as bytes (Q4_K: eight sums of 32, low bytes then high bytes; Q6_K: sixteen sums of 16,
// low six bits then the rest) and the scale.
__host__ __device__ constexpr int batch_pad(uint32_t type) { return type == OJAS_B200_Q6_K ? 16 : 32; }
__host__ __device__ constexpr int batch_bs_bytes(uint32_t type) { return type == OJAS_B200_Q6_K ? 32 : 16; }
__host__ __device__ inline size_t batch_act_bytes(uint32_t type, int NT, size_t K) {
    return (size_t)NT * (K + batch_pad(type)) + (size_t)NT * (K / 256) * (batch_bs_bytes(type) + 4);
}

// Q6_K step of the batch kernel (dot_q6k, crates/ojas-cpu/src/cpu_math.rs:674-722): a sub-block is 16 weights, so the
// MMA is m16n8k16 (A = 16 rows x 16 six-bit values as bytes, B = 16 int8 x 8 tokens) and every accumulator is the
// exact int32 dot of one sub-block for 16 rows x 8 tokens; its int8 scale is applied by an integer multiply-add.  Lane
// (g, q) supplies weights 4q .. 4q+3 of the sub-block: the low or high nibbles of FOUR CONTIGUOUS bytes of row g's
// chunk piece, OR-ed with two bits of the same four bytes of the chunk's top-bit piece.  The -32 of every weight is
// sum_j sc_j * (-32 * xsum_j): two more MMAs per super-block (A = the sixteen scales, B = the tokens' sums of 16,
// low six bits and the rest).
__device__ __forceinline__ void mma_k16_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %7, %7, %7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b), "r"(0));
}
__device__ __forceinline__ void mma_k16_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %7, %7, %7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b), "r"(0));
}
__device__ __forceinline__ int sext_byte(uint32_t w, int i) {   // byte i (a compile-time constant after unrolling) as a signed int
    return (int)(signed char)(w >> (8 * i));
}

// One 16-row tile (u0 / u1: its two 8-row weight tiles in the stage) x one super-block x up to NTILE token tiles.
template <int NTILE>
__device__ __forceinline__ void q6k_tile_step(const uint8_t *u0, const uint8_t *u1, bool second, const uint8_t *xq, int xstride, const uint8_t *bsb,
                                              const float *sx, int nsbseg, int sbl, int g8, int q4, int ntile, float (&acc)[NTILE][4]) {
    const uint8_t *t0 = u0 + g8 * 16 + 4 * q4, *t1 = u1 + g8 * 16 + 4 * q4;   // this lane's four bytes of every piece
    const uint4 S0 = *reinterpret_cast<const uint4 *>(u0 + 12 * 128 + g8 * 16), S1 = *reinterpret_cast<const uint4 *>(u1 + 12 * 128 + g8 * 16);
    const uint32_t sw0[4] = {S0.x, S0.y, S0.z, S0.w}, sw1[4] = {S1.x, S1.y, S1.z, S1.w};
    int isum[NTILE][4];
#pragma unroll
    for (int t = 0; t < NTILE; t++)
#pragma unroll
        for (int i = 0; i < 4; i++) isum[t][i] = 0;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint32_t la0 = *reinterpret_cast<const uint32_t *>(t0 + c * 128), lb0 = *reinterpret_cast<const uint32_t *>(t0 + (4 + c) * 128);
        const uint32_t h0 = *reinterpret_cast<const uint32_t *>(t0 + (8 + c) * 128);
        uint32_t la1 = *reinterpret_cast<const uint32_t *>(t1 + c * 128), lb1 = *reinterpret_cast<const uint32_t *>(t1 + (4 + c) * 128);
        uint32_t h1 = *reinterpret_cast<const uint32_t *>(t1 + (8 + c) * 128);
        if (!second) { la1 = 0u; lb1 = 0u; h1 = 0u; }
        // sub-block 4c + f: f = 0 low nibbles of piece c, 1 low nibbles of piece 4 + c, 2 / 3 their high nibbles; top bits = field f
        const uint32_t A0[4] = {(la0 & 0x0f0f0f0fu) | ((h0 << 4) & 0x30303030u), (lb0 & 0x0f0f0f0fu) | ((h0 << 2) & 0x30303030u),
                                ((la0 >> 4) & 0x0f0f0f0fu) | (h0 & 0x30303030u), ((lb0 >> 4) & 0x0f0f0f0fu) | ((h0 >> 2) & 0x30303030u)};
        const uint32_t A1[4] = {(la1 & 0x0f0f0f0fu) | ((h1 << 4) & 0x30303030u), (lb1 & 0x0f0f0f0fu) | ((h1 << 2) & 0x30303030u),
                                ((la1 >> 4) & 0x0f0f0f0fu) | (h1 & 0x30303030u), ((lb1 >> 4) & 0x0f0f0f0fu) | ((h1 >> 2) & 0x30303030u)};
#pragma unroll
        for (int f = 0; f < 4; f++) {
            const int s0 = sext_byte(sw0[c], f), s1 = sext_byte(sw1[c], f);
#pragma unroll
            for (int t = 0; t < NTILE; t++) {
                if (t < ntile) {
                    const uint32_t b = *reinterpret_cast<const uint32_t *>(xq + (size_t)(t * 8 + g8) * xstride + sbl * 256 + 64 * c + 16 * f + 4 * q4);
                    int d[4];
                    mma_k16_u8s8(d, A0[f], A1[f], b);
                    isum[t][0] += s0 * d[0];
                    isum[t][1] += s0 * d[1];
                    isum[t][2] += s1 * d[2];
                    isum[t][3] += s1 * d[3];
                }
            }
        }
    }
    // the -32 term: scales of the two rows (lane q holds scales 4q .. 4q+3) against the tokens' sums of 16
    const uint32_t as0 = *reinterpret_cast<const uint32_t *>(u0 + 12 * 128 + g8 * 16 + 4 * q4);
    const uint32_t as1 = second ? *reinterpret_cast<const uint32_t *>(u1 + 12 * 128 + g8 * 16 + 4 * q4) : 0u;
    const float d0 = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(u0 + 13 * 128 + 2 * g8));
    const float d1 = second ? f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(u1 + 13 * 128 + 2 * g8)) : 0.0f;
#pragma unroll
    for (int t = 0; t < NTILE; t++) {
        if (t < ntile) {
            const uint8_t *bp = bsb + ((size_t)(t * 8 + g8) * nsbseg + sbl) * 32 + 4 * q4;
            int ml[4], mh[4];
            mma_k16_s8s8(ml, as0, as1, *reinterpret_cast<const uint32_t *>(bp));
            mma_k16_s8s8(mh, as0, as1, *reinterpret_cast<const uint32_t *>(bp + 16));
            const float sx0 = sx[(t * 8 + 2 * q4) * nsbseg + sbl], sx1 = sx[(t * 8 + 2 * q4 + 1) * nsbseg + sbl];
            acc[t][0] += (sx0 * d0) * (float)(isum[t][0] - 32 * (ml[0] + 64 * mh[0]));
            acc[t][1] += (sx1 * d0) * (float)(isum[t][1] - 32 * (ml[1] + 64 * mh[1]));
            acc[t][2] += (sx0 * d1) * (float)(isum[t][2] - 32 * (ml[2] + 64 * mh[2]));
            acc[t][3] += (sx1 * d1) * (float)(isum[t][3] - 32 * (ml[3] + 64 * mh[3]));
        }
    }
}

// The batch kernel's step: the stage's 32 rows as two 16-row tiles.
template <int NTILE>
__device__ __forceinline__ void batch_step_q6k(const uint8_t *st, int g, int nu, const uint8_t *xq, int Kpad, const uint8_t *bsb, const float *sx,
                                               int nsb, int sb, int g8, int q4, float (&acc)[2][NTILE][4]) {
    constexpr int TB = tile_bytes(OJAS_B200_Q6_K);
#pragma unroll
    for (int rt = 0; rt < 2; rt++) {
        if (4 * g + 2 * rt >= nu) continue;                         // no unit under this row tile
        const bool second = 4 * g + 2 * rt + 1 < nu;                // the tile's rows 8..15 exist
        const uint8_t *u0 = st + (2 * rt) * TB;
        q6k_tile_step<NTILE>(u0, second ? u0 + TB : u0, second, xq, Kpad, bsb, sx, nsb, sb, g8, q4, NTILE, acc[rt]);
    }
}

template <int TYPE, int NTILE>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32, 1) gemv_kq_batch_kernel(const BatchArgs a) {
    constexpr int NT = 8 * NTILE, TB = tile_bytes(TYPE), STEP = 4 * TB, BSB = batch_bs_bytes(TYPE);
    extern __shared__ __align__(128) unsigned char smem[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g8 = lane >> 2, q4 = lane & 3;
    const int nsb = a.nsb, P = a.P, K = a.K, Kpad = K + batch_pad(TYPE);
    const int nst = 1 << a.nst_log, S = 1 << a.S_log, T = 1 << a.T_log;
    uint8_t *ring = smem + (size_t)warp * nst * STEP;
    uint8_t *xq = smem + (size_t)warps * nst * STEP;               // [NT][Kpad]
    uint8_t *bsb = xq + (size_t)NT * Kpad;                         // [NT][nsb][BSB]
    float *sx = reinterpret_cast<float *>(bsb + (size_t)NT * nsb * BSB);  // [NT][nsb]
    uint64_t *bar = reinterpret_cast<uint64_t *>(xq + ((batch_act_bytes(TYPE, NT, (size_t)K) + 15) & ~(size_t)15)) + warp * GEMV_MAX_STAGES;
    float *part = reinterpret_cast<float *>(reinterpret_cast<uint64_t *>(xq + ((batch_act_bytes(TYPE, NT, (size_t)K) + 15) & ~(size_t)15)) +
                                            GEMV_MAX_WARPS * GEMV_MAX_STAGES);

    const int b = blockIdx.x;
    const int ub = b * a.units_base + (b < a.units_rem ? b : a.units_rem);
    const int nu = a.units_base + (b < a.units_rem ? 1 : 0);
    const int ng = (nu + 3) >> 2;
    const int team = warp >> a.S_log, wi = warp & (S - 1);
    const int tg = team < ng ? (ng - team + T - 1) >> a.T_log : 0;
    const int n = tg * nsb;
    const int nsteps = wi < n ? (n - wi + S - 1) >> a.S_log : 0;   // steps of this warp in every job
    int k_first = 0, sb_first = wi;
    while (sb_first >= nsb) { sb_first -= nsb; k_first++; }

    if (lane == 0) {
        for (int i = 0; i < nst; i++) gv_bar_init(bar + i);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    grid_dependency_wait();                                        // counts, offsets and activations come from kernels before this one

    // issue cursor (lane 0 runs ahead of the computation by up to `nst` steps, across job boundaries)
    BatchJob ji;
    bool more_i = batch_job_first<NT>(a, ji) && nsteps > 0;
    int ik = k_first, isb = sb_first, ileft = nsteps;
    unsigned issued = 0;
    auto issue = [&]() -> bool {
        if (!more_i) return false;
        const int g = team + ik * T;
        const int cnt = (nu - 4 * g) < 4 ? (nu - 4 * g) : 4;
        const uint8_t *src = a.w[ji.wsel] + (size_t)ji.e * a.expert_bytes + ((size_t)(ub + 4 * g) * nsb + isb) * TB;
        const unsigned stg = issued & (unsigned)(nst - 1);
        gv_bar_expect(bar + stg, (unsigned)(cnt * TB));
        for (int t = 0; t < cnt; t++) gv_bulk_load(ring + stg * STEP + t * TB, src + (size_t)t * nsb * TB, TB, bar + stg);
        issued++;
        isb += S;
        while (isb >= nsb) { isb -= nsb; ik++; }
        if (--ileft == 0) {
            more_i = batch_job_next<NT>(a, ji);
            ik = k_first; isb = sb_first; ileft = nsteps;
        }
        return true;
    };
    if (lane == 0)
        for (int i = 0; i < nst; i++) issue();
    grid_launch_dependents();

    BatchJob jc;
    bool dead = false;
    bool more = batch_job_first<NT>(a, jc);
    int staged_e = -1, staged_mb = -1;
    unsigned uses = 0;
    while (more) {
        const int m_here = jc.count - jc.mb < NT ? jc.count - jc.mb : NT;
        if (staged_e != jc.e || staged_mb != jc.mb) {
            // ---- the pass's activation rows: values token-major (padded), block sums as bytes, scales
            __syncthreads();
            const int units = K >> 4;
            for (int m = 0; m < NT; m++) {
                uint4 *dst = reinterpret_cast<uint4 *>(xq + (size_t)m * Kpad);
                if (m < m_here && a.x) {
                    // fresh f32 rows: every warp quantizes super-blocks of the row (bit-exact quant_q8k), as the single-row kernel does
                    const int pos = jc.off + jc.mb + m;
                    const int srow = a.row_index ? __ldg(a.row_index + pos) : pos;
                    for (int sb = warp; sb < nsb; sb += warps)
                        stage_quant_sb<TYPE>(a.x + (size_t)srow * K, sb, lane, xq + (size_t)m * Kpad, bsb + (size_t)m * nsb * BSB, sx + m * nsb);
                } else if (m < m_here) {
                    const int pos = jc.off + jc.mb + m;
                    const int srow = a.row_index ? __ldg(a.row_index + pos) : pos;
                    const uint4 *qsrc = reinterpret_cast<const uint4 *>(a.q + (size_t)srow * K);
                    for (int un = threadIdx.x; un < units; un += blockDim.x) {
                        const uint4 v = __ldg(qsrc + un);
                        dst[un] = v;
                        if (TYPE == OJAS_B200_Q6_K) {               // the sum of this unit's sixteen values
                            int t = __dp4a((int)v.x, 0x01010101, 0);
                            t = __dp4a((int)v.y, 0x01010101, t);
                            t = __dp4a((int)v.z, 0x01010101, t);
                            t = __dp4a((int)v.w, 0x01010101, t);
                            uint8_t *o = bsb + ((size_t)m * nsb + (un >> 4)) * 32;
                            o[un & 15] = (uint8_t)(t & 63);
                            o[16 + (un & 15)] = (uint8_t)((t >> 6) & 0xff);
                        }
                    }
                    if (TYPE != OJAS_B200_Q6_K) {
                        for (int i = threadIdx.x; i < nsb * 8; i += blockDim.x) {
                            const int t = __ldg(a.bsums + (size_t)srow * nsb * 8 + i);
                            uint8_t *o = bsb + ((size_t)m * nsb + (i >> 3)) * 16;
                            o[i & 7] = (uint8_t)(t & 63);
                            o[8 + (i & 7)] = (uint8_t)((t >> 6) & 0xff);
                        }
                    }
                    for (int sb = threadIdx.x; sb < nsb; sb += blockDim.x) sx[m * nsb + sb] = __ldg(a.scales + (size_t)srow * nsb + sb);
                } else {
                    for (int un = threadIdx.x; un < units; un += blockDim.x) dst[un] = make_uint4(0u, 0u, 0u, 0u);
                    for (int i = threadIdx.x; i < nsb * (BSB / 4); i += blockDim.x) reinterpret_cast<uint32_t *>(bsb + (size_t)m * nsb * BSB)[i] = 0u;
                    for (int sb = threadIdx.x; sb < nsb; sb += blockDim.x) sx[m * nsb + sb] = 0.0f;
                }
            }
            staged_e = jc.e; staged_mb = jc.mb;
            __syncthreads();
        }

        // ---- this warp's steps of the job
        float acc[2][NTILE][4];
#pragma unroll
        for (int rt = 0; rt < 2; rt++)
#pragma unroll
            for (int t = 0; t < NTILE; t++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[rt][t][i] = 0.0f;
        int k = k_first, sb = sb_first;
        for (int s = 0; s < nsteps; s++, uses++) {
            const unsigned stg = uses & (unsigned)(nst - 1);
            const int g = team + k * T;
            gv_bar_wait(bar + stg, (uses >> a.nst_log) & 1u, a.status, dead);
            const uint8_t *st = ring + stg * STEP;
            if (TYPE == OJAS_B200_Q6_K) batch_step_q6k<NTILE>(st, g, nu, xq, Kpad, bsb, sx, nsb, sb, g8, q4, acc);
            else
#pragma unroll
            for (int rt = 0; rt < 2; rt++) {
                if (4 * g + 2 * rt >= nu) continue;                 // no unit under this row tile (rows past the CTA's range)
                const bool second = 4 * g + 2 * rt + 1 < nu;        // the tile's rows 8..15 exist
                const uint8_t *t0 = st + (2 * rt) * TB + g8 * 16, *t1 = second ? t0 + TB : t0;
                // scales and mins of the two rows as bytes (get_scale_min_k4, crates/ojas-formats/src/gguf.rs:1132-1140)
                const uint4 H0 = *reinterpret_cast<const uint4 *>(t0 + 8 * 128), H1 = *reinterpret_cast<const uint4 *>(t1 + 8 * 128);
                const uint32_t s0[2] = {H0.y & 0x3f3f3f3fu, (H0.w & 0x0f0f0f0fu) | ((H0.y >> 2) & 0x30303030u)};
                const uint32_t s1[2] = {H1.y & 0x3f3f3f3fu, (H1.w & 0x0f0f0f0fu) | ((H1.y >> 2) & 0x30303030u)};
                const uint32_t m0[2] = {H0.z & 0x3f3f3f3fu, ((H0.w >> 4) & 0x0f0f0f0fu) | ((H0.z >> 2) & 0x30303030u)};
                const uint32_t m1[2] = {H1.z & 0x3f3f3f3fu, ((H1.w >> 4) & 0x0f0f0f0fu) | ((H1.z >> 2) & 0x30303030u)};
                int isum[NTILE][4];
#pragma unroll
                for (int t = 0; t < NTILE; t++)
#pragma unroll
                    for (int i = 0; i < 4; i++) isum[t][i] = 0;
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    // eight contiguous bytes of each row: low nibbles = weights 8q .. 8q+7 of sub-block 2c, high = of 2c+1
                    const uint2 w0 = *reinterpret_cast<const uint2 *>(t0 + (2 * c + (q4 >> 1)) * 128 + (q4 & 1) * 8);
                    uint2 w1 = *reinterpret_cast<const uint2 *>(t1 + (2 * c + (q4 >> 1)) * 128 + (q4 & 1) * 8);
                    if (!second) w1 = make_uint2(0u, 0u);
                    const uint32_t alo[4] = {w0.x & 0x0f0f0f0fu, w1.x & 0x0f0f0f0fu, w0.y & 0x0f0f0f0fu, w1.y & 0x0f0f0f0fu};
                    const uint32_t ahi[4] = {w0.x & 0xf0f0f0f0u, w1.x & 0xf0f0f0f0u, w0.y & 0xf0f0f0f0u, w1.y & 0xf0f0f0f0u};
                    const int sA0 = (int)__byte_perm(s0[c >> 1], 0, 0x4440 + 2 * (c & 1)), sB0 = (int)__byte_perm(s0[c >> 1], 0, 0x4441 + 2 * (c & 1));
                    const int sA1 = (int)__byte_perm(s1[c >> 1], 0, 0x4440 + 2 * (c & 1)), sB1 = (int)__byte_perm(s1[c >> 1], 0, 0x4441 + 2 * (c & 1));
#pragma unroll
                    for (int t = 0; t < NTILE; t++) {
                        const uint8_t *xr = xq + (size_t)(t * 8 + g8) * Kpad + sb * 256 + 64 * c + 8 * q4;
                        const uint2 xa = *reinterpret_cast<const uint2 *>(xr), xb = *reinterpret_cast<const uint2 *>(xr + 32);
                        int dlo[4], dhi[4];
                        mma_u8s8_z(dlo, alo, xa.x, xa.y);
                        mma_u8s8_z(dhi, ahi, xb.x, xb.y);
                        isum[t][0] += sA0 * dlo[0] + sB0 * (dhi[0] >> 4);
                        isum[t][1] += sA0 * dlo[1] + sB0 * (dhi[1] >> 4);
                        isum[t][2] += sA1 * dlo[2] + sB1 * (dhi[2] >> 4);
                        isum[t][3] += sA1 * dlo[3] + sB1 * (dhi[3] >> 4);
                    }
                }
                // mins: A = the eight mins of each row as bytes (lane q = 0 holds mins 0..3, q = 1 mins 4..7), B = the
                // tokens' block sums, low bytes and high bytes
                const uint32_t am[4] = {q4 < 2 ? m0[q4] : 0u, (q4 < 2 && second) ? m1[q4] : 0u, 0u, 0u};
                const float d0 = f16_bits_to_f32(H0.x), dm0 = f16_bits_to_f32(H0.x >> 16);
                const float d1 = second ? f16_bits_to_f32(H1.x) : 0.0f, dm1 = second ? f16_bits_to_f32(H1.x >> 16) : 0.0f;
#pragma unroll
                for (int t = 0; t < NTILE; t++) {
                    const uint8_t *bp = bsb + ((size_t)(t * 8 + g8) * nsb + sb) * 16;
                    const uint32_t blo = q4 < 2 ? *reinterpret_cast<const uint32_t *>(bp + 4 * q4) : 0u;
                    const uint32_t bhi = q4 < 2 ? *reinterpret_cast<const uint32_t *>(bp + 8 + 4 * q4) : 0u;
                    int ml[4], mh[4];
                    mma_u8s8_z(ml, am, blo, 0u);
                    mma_u8s8_z(mh, am, bhi, 0u);
                    const float sx0 = sx[(t * 8 + 2 * q4) * nsb + sb], sx1 = sx[(t * 8 + 2 * q4 + 1) * nsb + sb];
                    acc[rt][t][0] += sx0 * (d0 * (float)isum[t][0] - dm0 * (float)(ml[0] + 64 * mh[0]));
                    acc[rt][t][1] += sx1 * (d0 * (float)isum[t][1] - dm0 * (float)(ml[1] + 64 * mh[1]));
                    acc[rt][t][2] += sx0 * (d1 * (float)isum[t][2] - dm1 * (float)(ml[2] + 64 * mh[2]));
                    acc[rt][t][3] += sx1 * (d1 * (float)isum[t][3] - dm1 * (float)(ml[3] + 64 * mh[3]));
                }
            }
            __syncwarp();
            if (lane == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue();
            }
            const int slot = sb & (S - 1), k_now = k;
            sb += S;
            bool flush = s + 1 == nsteps;
            while (sb >= nsb) { sb -= nsb; k++; flush = true; }
            if (flush) {
#pragma unroll
                for (int rt = 0; rt < 2; rt++)
#pragma unroll
                    for (int t = 0; t < NTILE; t++) {
                        float4 *o = reinterpret_cast<float4 *>(part) + ((((size_t)(team + k_now * T) * P + slot) * 2 + rt) * NTILE + t) * 32 + lane;
                        *o = make_float4(acc[rt][t][0], acc[rt][t][1], acc[rt][t][2], acc[rt][t][3]);
                        acc[rt][t][0] = acc[rt][t][1] = acc[rt][t][2] = acc[rt][t][3] = 0.0f;
                    }
            }
        }
        __syncthreads();
        // ---- combine the warps' partial sums of the job and store: item = (group, row tile, token tile, lane)
        float *yout = a.y[jc.wsel];
        for (int item = threadIdx.x; item < ng * 2 * NTILE * 32; item += blockDim.x) {
            const int ln = item & 31, t = (item >> 5) % NTILE, rt = ((item >> 5) / NTILE) & 1, gl = (item >> 5) / (2 * NTILE);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int p = 0; p < P; p++) {
                const float4 u = reinterpret_cast<const float4 *>(part)[((((size_t)gl * P + p) * 2 + rt) * NTILE + t) * 32 + ln];
                v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
            }
            const int lg = ln >> 2, lq = ln & 3;
            const float vals[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int unit = 4 * gl + 2 * rt + (i >> 1), tok = t * 8 + 2 * lq + (i & 1);
                const int row = (ub + unit) * 8 + lg;
                if (unit < nu && row < a.N && tok < m_here)
                    store_form(yout + (size_t)(jc.off + jc.mb + tok) * a.N + row, vals[i], a.form, a.bias, row);
            }
        }
        more = batch_job_next<NT>(a, jc);
        if (more && staged_e == jc.e && staged_mb == jc.mb) __syncthreads();   // (a new pass syncs before it stages)
    }
}


// ---------------------------------------------------------------------------------------------------------------
// The expert FFN's matmuls in one launch.  Work is the list of 16-row tiles of every (expert with rows, weight
// tensor) pair, expert-major; CTA b takes the b-th equal share of that list, so its tiles belong to one expert (two
// at a boundary) and the expert's activation rows are staged once.  A WARP OWNS A TILE for the whole K range: its
// sums stay in registers and go straight to y, so nothing is exchanged between warps and the only CTA-wide
// barriers are those around the staging of activations.  Activations are staged per K segment of up to 4096 values
// (all NT rows of the pass), so long rows (the down projection) fit beside a deep weight ring; a step is one
// super-block of the tile (two 8-row tiles of the weight, 2304 bytes, two bulk copies) and the ring prefetch of a
// warp runs ahead across segments, tiles and experts.
constexpr int EXPERT_KSEG = 4096;
constexpr int EXPERT_MAX_E = 64;

struct ExpertArgs {
    const uint8_t *w[2];
    float *y[2];
    int nw;
    size_t expert_bytes;
    const int8_t *q;
    const float *scales;
    const int32_t *bsums;
    const int *row_index;
    const int *counts, *offsets;
    unsigned *status;
    int E, K, N, nsb, nst;
};

__host__ __device__ inline size_t expert_act_bytes(uint32_t type, int NT, size_t K) {
    return batch_act_bytes(type, NT, K < (size_t)EXPERT_KSEG ? K : (size_t)EXPERT_KSEG);
}

// One 16-row tile x one super-block x up to NTILE token tiles.  t0 / t1: this lane's row (g8) in the tile's two
// 8-row weight tiles; xq, bsb, sx: the staged activations of the segment, `sbl` the super-block inside the segment.
// FIVE: Q5_K (dot_q5k, crates/ojas-cpu/src/cpu_math.rs:637-671).  Weight l of sub-block j has its fifth bit in bit j of qh[l]
// (pieces 9, 10 of the tile); the lane's eight weights 8q .. 8q+7 are the same l in every sub-block, so it loads its eight
// qh bytes once per step.  Five-bit values do not leave room to keep high nibbles in place, so they are shifted down.
template <int NTILE, bool FIVE = false>
__device__ __forceinline__ void mma_tile_step(const uint8_t *t0, const uint8_t *t1, bool second, const uint8_t *xq, int xstride, const uint8_t *bsb,
                                              const float *sx, int nsbseg, int sbl, int g8, int q4, int ntile, float (&acc)[NTILE][4]) {
    const uint4 H0 = *reinterpret_cast<const uint4 *>(t0 + 8 * 128), H1 = *reinterpret_cast<const uint4 *>(t1 + 8 * 128);
    uint2 q50 = make_uint2(0u, 0u), q51 = q50;
    if (FIVE) {
        q50 = *reinterpret_cast<const uint2 *>(t0 + (9 + (q4 >> 1)) * 128 + (q4 & 1) * 8);
        q51 = second ? *reinterpret_cast<const uint2 *>(t1 + (9 + (q4 >> 1)) * 128 + (q4 & 1) * 8) : make_uint2(0u, 0u);
    }
    const uint32_t s0[2] = {H0.y & 0x3f3f3f3fu, (H0.w & 0x0f0f0f0fu) | ((H0.y >> 2) & 0x30303030u)};
    const uint32_t s1[2] = {H1.y & 0x3f3f3f3fu, (H1.w & 0x0f0f0f0fu) | ((H1.y >> 2) & 0x30303030u)};
    const uint32_t m0[2] = {H0.z & 0x3f3f3f3fu, ((H0.w >> 4) & 0x0f0f0f0fu) | ((H0.z >> 2) & 0x30303030u)};
    const uint32_t m1[2] = {H1.z & 0x3f3f3f3fu, ((H1.w >> 4) & 0x0f0f0f0fu) | ((H1.z >> 2) & 0x30303030u)};
    int isum[NTILE][4];
#pragma unroll
    for (int t = 0; t < NTILE; t++)
#pragma unroll
        for (int i = 0; i < 4; i++) isum[t][i] = 0;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint2 w0 = *reinterpret_cast<const uint2 *>(t0 + (2 * c + (q4 >> 1)) * 128 + (q4 & 1) * 8);
        uint2 w1 = *reinterpret_cast<const uint2 *>(t1 + (2 * c + (q4 >> 1)) * 128 + (q4 & 1) * 8);
        if (!second) w1 = make_uint2(0u, 0u);
        uint32_t alo[4] = {w0.x & 0x0f0f0f0fu, w1.x & 0x0f0f0f0fu, w0.y & 0x0f0f0f0fu, w1.y & 0x0f0f0f0fu};
        uint32_t ahi[4] = {w0.x & 0xf0f0f0f0u, w1.x & 0xf0f0f0f0u, w0.y & 0xf0f0f0f0u, w1.y & 0xf0f0f0f0u};
        if (FIVE) {                                                // sub-block 2c takes bit 2c of the qh bytes, 2c + 1 bit 2c + 1
            const uint32_t hb[4] = {q50.x >> (2 * c), q51.x >> (2 * c), q50.y >> (2 * c), q51.y >> (2 * c)};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                alo[k] |= (hb[k] & 0x01010101u) << 4;
                ahi[k] = (ahi[k] >> 4) | ((hb[k] & 0x02020202u) << 3);
            }
        }
        const int sA0 = (int)__byte_perm(s0[c >> 1], 0, 0x4440 + 2 * (c & 1)), sB0 = (int)__byte_perm(s0[c >> 1], 0, 0x4441 + 2 * (c & 1));
        const int sA1 = (int)__byte_perm(s1[c >> 1], 0, 0x4440 + 2 * (c & 1)), sB1 = (int)__byte_perm(s1[c >> 1], 0, 0x4441 + 2 * (c & 1));
#pragma unroll
        for (int t = 0; t < NTILE; t++) {
            if (t < ntile) {
                const uint8_t *xr = xq + (size_t)(t * 8 + g8) * xstride + sbl * 256 + 64 * c + 8 * q4;
                const uint2 xa = *reinterpret_cast<const uint2 *>(xr), xb = *reinterpret_cast<const uint2 *>(xr + 32);
                int dlo[4], dhi[4];
                mma_u8s8_z(dlo, alo, xa.x, xa.y);
                mma_u8s8_z(dhi, ahi, xb.x, xb.y);
                constexpr int HS = FIVE ? 0 : 4;                   // Q4_K keeps its high nibbles in place (x 16)
                isum[t][0] += sA0 * dlo[0] + sB0 * (dhi[0] >> HS);
                isum[t][1] += sA0 * dlo[1] + sB0 * (dhi[1] >> HS);
                isum[t][2] += sA1 * dlo[2] + sB1 * (dhi[2] >> HS);
                isum[t][3] += sA1 * dlo[3] + sB1 * (dhi[3] >> HS);
            }
        }
    }
    const uint32_t am[4] = {q4 < 2 ? m0[q4] : 0u, (q4 < 2 && second) ? m1[q4] : 0u, 0u, 0u};
    const float d0 = f16_bits_to_f32(H0.x), dm0 = f16_bits_to_f32(H0.x >> 16);
    const float d1 = second ? f16_bits_to_f32(H1.x) : 0.0f, dm1 = second ? f16_bits_to_f32(H1.x >> 16) : 0.0f;
#pragma unroll
    for (int t = 0; t < NTILE; t++) {
        if (t < ntile) {
            const uint8_t *bp = bsb + ((size_t)(t * 8 + g8) * nsbseg + sbl) * 16;
            const uint32_t blo = q4 < 2 ? *reinterpret_cast<const uint32_t *>(bp + 4 * q4) : 0u;
            const uint32_t bhi = q4 < 2 ? *reinterpret_cast<const uint32_t *>(bp + 8 + 4 * q4) : 0u;
            int ml[4], mh[4];
            mma_u8s8_z(ml, am, blo, 0u);
            mma_u8s8_z(mh, am, bhi, 0u);
            const float sx0 = sx[(t * 8 + 2 * q4) * nsbseg + sbl], sx1 = sx[(t * 8 + 2 * q4 + 1) * nsbseg + sbl];
            acc[t][0] += sx0 * (d0 * (float)isum[t][0] - dm0 * (float)(ml[0] + 64 * mh[0]));
            acc[t][1] += sx1 * (d0 * (float)isum[t][1] - dm0 * (float)(ml[1] + 64 * mh[1]));
            acc[t][2] += sx0 * (d1 * (float)isum[t][2] - dm1 * (float)(ml[2] + 64 * mh[2]));
            acc[t][3] += sx1 * (d1 * (float)isum[t][3] - dm1 * (float)(ml[3] + 64 * mh[3]));
        }
    }
}

template <int TYPE, int NTILE>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32, 1) moe_kq_experts_kernel(const ExpertArgs a) {
    constexpr int NT = 8 * NTILE, TB = tile_bytes(TYPE), STEP = 2 * TB, BSB = batch_bs_bytes(TYPE);
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int act_e[EXPERT_MAX_E], act_n;                    // experts that have rows, in order
    __shared__ unsigned share[2];                                 // this CTA's range of the tile list
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g8 = lane >> 2, q4 = lane & 3;
    const int nsb = a.nsb, K = a.K, nst = a.nst;
    const int kseg = K < EXPERT_KSEG ? K : EXPERT_KSEG, nsbseg = kseg >> 8, xstride = kseg + batch_pad(TYPE);
    const int nseg = (K + kseg - 1) / kseg;
    uint8_t *ring = smem + (size_t)warp * nst * STEP;
    uint8_t *xq = smem + (size_t)warps * nst * STEP;
    uint8_t *bsb = xq + (size_t)NT * xstride;
    float *sx = reinterpret_cast<float *>(bsb + (size_t)NT * nsbseg * BSB);
    uint64_t *bar = reinterpret_cast<uint64_t *>(xq + ((expert_act_bytes(TYPE, NT, (size_t)K) + 15) & ~(size_t)15)) + warp * GEMV_MAX_STAGES;

    if (lane == 0) {
        for (int i = 0; i < nst; i++) gv_bar_init(bar + i);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    grid_dependency_wait();                                        // counts, offsets and activations come from kernels before this one
    const int tpe = (a.N + 15) >> 4;                               // 16-row tiles per (expert, tensor)
    if (threadIdx.x == 0) {
        // The CTA's share of the work list is a share of its COST, in units of ROUNDS.  A round is the tiles the CTA's
        // warps take together (one each) from one (expert, tensor) pair: a share that ended inside a round would pay a
        // whole round for a few tiles, and a tile of an expert with more rows does more token tiles per step (and more
        // passes), so shares by tile count would leave the CTAs of quiet experts idle.
        // Cost of a round = sum over the expert's passes of (2 + 3 * token tiles of the pass).
        int n = 0;
        unsigned long long total_cost = 0;
        unsigned ecost[EXPERT_MAX_E];
        const unsigned rpe = (unsigned)((tpe + warps - 1) / warps), rounds_e = (unsigned)a.nw * rpe;
        for (int e = 0; e < a.E; e++) {
            const int cnt = __ldg(a.counts + e);
            if (cnt <= 0) continue;
            const unsigned full = (unsigned)(cnt / NT), rest = (unsigned)(cnt % NT);
            ecost[n] = full * (2u + 3u * NTILE) + (rest ? 2u + 3u * ((rest + 7u) >> 3) : 0u);
            total_cost += (unsigned long long)ecost[n] * rounds_e;
            act_e[n++] = e;
        }
        act_n = n;
        for (int side = 0; side < 2; side++) {
            unsigned long long pos = total_cost * (blockIdx.x + side) / gridDim.x;
            unsigned tile = 0;
            int i = 0;
            for (; i < n; i++) {
                const unsigned long long span = (unsigned long long)ecost[i] * rounds_e;
                if (pos < span) break;
                pos -= span;
                tile += (unsigned)(a.nw * tpe);
            }
            if (i < n) {
                const unsigned rnd = (unsigned)(pos / ecost[i]), pl = rnd / rpe, r = rnd - pl * rpe;
                const unsigned in_pair = r * (unsigned)warps < (unsigned)tpe ? r * (unsigned)warps : (unsigned)tpe;
                tile += pl * (unsigned)tpe + in_pair;
            }
            share[side] = tile;
        }
    }
    __syncthreads();
    grid_launch_dependents();
    const unsigned c0 = share[0], c1 = share[1];
    const int units_total = (a.N + 7) >> 3;

    // ---- issue side (lane 0): the warp's steps in order: for every pair segment of the CTA's range, for every pass
    // of the expert's rows, tiles lo + warp, lo + warp + warps, ..., super-blocks 0 .. nsb - 1
    struct Cursor { unsigned seg_lo, seg_hi, tile; int pair, mb, count, sb; bool live; };
    auto seg_open = [&](Cursor &c, unsigned from) {               // the pair segment that starts at global tile index `from`
        c.live = from < c1;
        if (!c.live) return;
        c.pair = (int)(from / (unsigned)tpe);
        const unsigned pair_end = (unsigned)(c.pair + 1) * (unsigned)tpe;
        c.seg_lo = from; c.seg_hi = pair_end < c1 ? pair_end : c1;
        c.count = __ldg(a.counts + act_e[c.pair / a.nw]);
        c.mb = 0;
        c.tile = c.seg_lo + (unsigned)warp;
        c.sb = 0;
    };
    auto cur_fix = [&](Cursor &c) {                               // skip to the next (pass, segment) when this warp has no tile left in this one
        while (c.live && c.tile >= c.seg_hi) {
            if (c.mb + NT < c.count) { c.mb += NT; c.tile = c.seg_lo + (unsigned)warp; c.sb = 0; }
            else seg_open(c, c.seg_hi);
        }
    };
    Cursor ci;
    seg_open(ci, c0);
    cur_fix(ci);
    int istg = 0;
    auto issue = [&]() {
        if (!ci.live) return;
        const int e = act_e[ci.pair / a.nw], wsel = ci.pair % a.nw;
        const int tl = (int)(ci.tile - (unsigned)ci.pair * (unsigned)tpe);          // tile inside the expert
        const int cnt = units_total - 2 * tl < 2 ? units_total - 2 * tl : 2;
        const uint8_t *src = a.w[wsel] + (size_t)e * a.expert_bytes + ((size_t)(2 * tl) * nsb + ci.sb) * TB;
        gv_bar_expect(bar + istg, (unsigned)(cnt * TB));
        for (int t = 0; t < cnt; t++) gv_bulk_load(ring + istg * STEP + t * TB, src + (size_t)t * nsb * TB, TB, bar + istg);
        if (++istg == nst) istg = 0;
        if (++ci.sb == nsb) { ci.sb = 0; ci.tile += (unsigned)warps; cur_fix(ci); }
    };
    if (lane == 0)
        for (int i = 0; i < nst; i++) issue();

    // ---- compute side: all warps walk the CTA's segments and passes together (the staging is CTA-wide)
    int cstg = 0;
    unsigned cphase = 0;
    bool dead = false;
    for (unsigned from = c0; from < c1;) {
        const int pair = (int)(from / (unsigned)tpe);
        const unsigned pair_end = (unsigned)(pair + 1) * (unsigned)tpe, seg_hi = pair_end < c1 ? pair_end : c1;
        const int e = act_e[pair / a.nw], wsel = pair % a.nw;
        const int count = __ldg(a.counts + e), off = __ldg(a.offsets + e);
        const int rounds = (int)((seg_hi - from + (unsigned)warps - 1) / (unsigned)warps);
        for (int mb = 0; mb < count; mb += NT) {
            const int m_here = count - mb < NT ? count - mb : NT, ntile = (m_here + 7) >> 3;
            for (int rd = 0; rd < rounds; rd++) {
                const unsigned tile = from + (unsigned)(rd * warps + warp);
                const bool mine = tile < seg_hi;
                const int tl = (int)(tile - (unsigned)pair * (unsigned)tpe);
                const bool second = 2 * tl + 1 < units_total;
                float acc[NTILE][4];
#pragma unroll
                for (int t = 0; t < NTILE; t++) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
                for (int ks = 0; ks < nseg; ks++) {
                    const int sb0 = ks * nsbseg, nsb_here = nsb - sb0 < nsbseg ? nsb - sb0 : nsbseg;
                    // ---- stage the pass's rows, K segment ks (skipped when it is what is staged already: one segment, same rows)
                    if (nseg > 1 || rd == 0) {
                        __syncthreads();
                        const int units = nsb_here * 16;
                        for (int idx = threadIdx.x; idx < NT * units; idx += blockDim.x) {
                            const int m = idx / units, un = idx - m * units;
                            uint4 v = make_uint4(0u, 0u, 0u, 0u);
                            if (m < m_here) {
                                const int pos = off + mb + m;
                                const int srow = a.row_index ? __ldg(a.row_index + pos) : pos;
                                v = __ldg(reinterpret_cast<const uint4 *>(a.q + (size_t)srow * K + (size_t)sb0 * 256) + un);
                            }
                            reinterpret_cast<uint4 *>(xq + (size_t)m * xstride)[un] = v;
                            if (TYPE == OJAS_B200_Q6_K) {           // the sum of this unit's sixteen values, as two bytes
                                int t = __dp4a((int)v.x, 0x01010101, 0);
                                t = __dp4a((int)v.y, 0x01010101, t);
                                t = __dp4a((int)v.z, 0x01010101, t);
                                t = __dp4a((int)v.w, 0x01010101, t);
                                uint8_t *o = bsb + ((size_t)m * nsbseg + (un >> 4)) * 32;
                                o[un & 15] = (uint8_t)(t & 63);
                                o[16 + (un & 15)] = (uint8_t)((t >> 6) & 0xff);
                            }
                        }
                        for (int idx = threadIdx.x; TYPE != OJAS_B200_Q6_K && idx < NT * nsb_here * 8; idx += blockDim.x) {
                            const int m = idx / (nsb_here * 8), i = idx - m * (nsb_here * 8);
                            int t = 0;
                            if (m < m_here) {
                                const int pos = off + mb + m;
                                const int srow = a.row_index ? __ldg(a.row_index + pos) : pos;
                                t = __ldg(a.bsums + ((size_t)srow * nsb + sb0) * 8 + i);
                            }
                            uint8_t *o = bsb + ((size_t)m * nsbseg + (i >> 3)) * 16;
                            o[i & 7] = (uint8_t)(t & 63);
                            o[8 + (i & 7)] = (uint8_t)((t >> 6) & 0xff);
                        }
                        for (int idx = threadIdx.x; idx < NT * nsb_here; idx += blockDim.x) {
                            const int m = idx / nsb_here, sbl = idx - m * nsb_here;
                            float v = 0.0f;
                            if (m < m_here) {
                                const int pos = off + mb + m;
                                const int srow = a.row_index ? __ldg(a.row_index + pos) : pos;
                                v = __ldg(a.scales + (size_t)srow * nsb + sb0 + sbl);
                            }
                            sx[m * nsbseg + sbl] = v;
                        }
                        __syncthreads();
                    }
                    if (mine) {
                        for (int sbl = 0; sbl < nsb_here; sbl++) {
                            gv_bar_wait(bar + cstg, cphase, a.status, dead);
                            if (TYPE == OJAS_B200_Q6_K) {
                                const uint8_t *u0 = ring + cstg * STEP;
                                q6k_tile_step<NTILE>(u0, second ? u0 + TB : u0, second, xq, xstride, bsb, sx, nsbseg, sbl, g8, q4, ntile, acc);
                            } else {
                                const uint8_t *t0 = ring + cstg * STEP + g8 * 16, *t1 = second ? t0 + TB : t0;
                                mma_tile_step<NTILE, TYPE == OJAS_B200_Q5_K>(t0, t1, second, xq, xstride, bsb, sx, nsbseg, sbl, g8, q4, ntile, acc);
                            }
                            __syncwarp();
                            if (lane == 0) {
                                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                                issue();
                            }
                            if (++cstg == nst) { cstg = 0; cphase ^= 1u; }
                        }
                    }
                }
                if (mine) {
                    float *yout = a.y[wsel];
#pragma unroll
                    for (int t = 0; t < NTILE; t++)
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int tok = t * 8 + 2 * q4 + (i & 1), row = tl * 16 + (i >> 1) * 8 + g8;
                            if (tok < m_here && row < a.N) yout[(size_t)(off + mb + tok) * a.N + row] = acc[t][i];
                        }
                }
            }
        }
        from = seg_hi;
    }
}
