// Small-batch Q4_K GEMV on the integer tensor-core path (mma.sync m16n8k32, u8 x s8 -> s32).
//
// Same arithmetic as the dp4a kernels (matvec_kq, crates/ojas-cpu/src/cpu_math.rs:1145-1189): the
// accumulator of one MMA holds, for 16 weight rows and up to 8 activation rows, the exact int32 dot
// of one 32-weight sub-block (dot_q4k's idot32, :583-593, :619-632); scales, mins and the Q8_K
// activation scale are applied per super-block in the same integer / fp32 combination.  One
// instruction replaces 16 x 8 lane-level dp4a, which is what makes 2..8 activation rows (the `_m`
// GEMV forms and the grouped expert GEMVs) bandwidth-bound instead of ALU-bound.
//
// Work: CTA b owns a contiguous row range; rows are taken 16 at a time (a tile); a step is one
// tile x one super-block: 16 x 128 bytes of nibbles + 16 headers, copied global -> shared with
// cp.async into a two-stage ring per warp (row stride 144 bytes: conflict-free fragment reads).
// (tile, segment-of-super-blocks) units go round-robin to the warps; partial sums of a tile's
// segments are added in a fixed order.
#pragma once

constexpr int MMA_ROW_STRIDE = 144;                       // 128 bytes of nibbles + 16 of padding
constexpr int MMA_STAGE_BYTES = 16 * MMA_ROW_STRIDE + 256; // 16 rows + 16 headers = 2560
constexpr int MMA_XPAD = 16;                              // activation rows are K + 16 bytes apart (bank spread)

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

// Activations into shared memory in natural order: xq [M][K + 16] int8, sx [M][nsb] f32, and the per-32 sums of
// every super-block as two bytes each, sum = 64 * hi + lo with lo in 0..63 and hi in -64..63 (both fit the s8
// operand of the MMA that forms the mins term): bs bytes [M][nsb][32] = lo[8], hi[8], 16 unused.
template <int WARPS, bool PREQ>
__device__ __forceinline__ void stage_q8k_rows(const GemvArgs &a, unsigned char *xq, float *sx, int *bs, int nsb, int xstride) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (!PREQ) {
        for (int u = warp; u < a.M * nsb; u += WARPS) {
            const int m = u / nsb, sb = u - m * nsb;
            const Q8kLane ql = quant_q8k_warp(a.x + (size_t)m * a.K + (size_t)sb * 256, lane);
            *reinterpret_cast<uint2 *>(xq + (size_t)m * xstride + sb * 256 + lane * 8) = ql.packed;
            int s = ql.sum8;
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if ((lane & 3) == 0) {
                unsigned char *bb = reinterpret_cast<unsigned char *>(bs) + (size_t)(m * nsb + sb) * 32 + (lane >> 2);
                bb[0] = (unsigned char)(s & 63);
                bb[8] = (unsigned char)((s >> 6) & 0xff);
            }
            if (lane == 0) sx[m * nsb + sb] = ql.scale;
        }
    } else {
        const int units = nsb * 16;
        for (int idx = threadIdx.x; idx < a.M * units; idx += blockDim.x) {
            const int m = idx / units, rem = idx - m * units;
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(a.q + (size_t)src_row(a, m) * a.K) + rem);
            *reinterpret_cast<uint4 *>(xq + (size_t)m * xstride + rem * 16) = v;
        }
        for (int idx = threadIdx.x; idx < a.M * nsb; idx += blockDim.x) {
            const int m = idx / nsb;
            sx[idx] = __ldg(a.scales + (size_t)src_row(a, m) * nsb + (idx - m * nsb));
        }
        for (int idx = threadIdx.x; idx < a.M * nsb * 8; idx += blockDim.x) {
            const int m = idx / (nsb * 8), rem = idx - m * nsb * 8;
            const int s = __ldg(a.bsums + (size_t)src_row(a, m) * nsb * 8 + rem);
            unsigned char *bb = reinterpret_cast<unsigned char *>(bs) + (size_t)(m * nsb + (rem >> 3)) * 32 + (rem & 7);
            bb[0] = (unsigned char)(s & 63);
            bb[8] = (unsigned char)((s >> 6) & 0xff);
        }
    }
}

// a.S = segments per tile (divides the super-block count); a.M <= 8 * NT.  NT = 2 runs two MMAs per unpacked
// weight fragment (tokens 0..7 and 8..15): the unpacking and the scale extraction are shared by 16 tokens.
template <int WARPS, bool PREQ, int NT = 1>
__device__ __forceinline__ void gemv_q4k_mma_body(const GemvArgs &a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int nsb = a.K >> 8, S = a.S, SP = nsb / S;          // super-blocks per unit
    const int xstride = a.K + MMA_XPAD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;                    // fragment row / token, k quad
    unsigned char *ring = smem + (size_t)warp * 2 * MMA_STAGE_BYTES;
    unsigned char *xq = smem + (size_t)WARPS * 2 * MMA_STAGE_BYTES;
    float *sx = reinterpret_cast<float *>(xq + (((size_t)a.M * xstride + 15) & ~(size_t)15));
    int *bs = reinterpret_cast<int *>(sx + sx_floats(a.M, nsb));
    float *part = reinterpret_cast<float *>(bs + a.M * nsb * 8);

    int r_begin, R;
    cta_rows(a, r_begin, R);
    const int n_tiles = (R + 15) >> 4, n_units = n_tiles * S;
    const uint4 *qs = reinterpret_cast<const uint4 *>(a.w.p0);
    const uint4 *hdr = reinterpret_cast<const uint4 *>(a.w.p1);

    // unit u -> (tile, segment); step = (unit, super-block inside the segment)
    struct It { int u, j; };
    auto issue = [&](const It &it, int stage) {
        if (it.u < n_units) {
            const int tile = it.u / S, seg = it.u - tile * S;
            const int sb = seg * SP + it.j;
            unsigned char *st = ring + stage * MMA_STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int p = lane + 32 * i, row = p >> 3, piece = p & 7;
                int gr = tile * 16 + row;
                gr = gr < R ? gr : R - 1;                      // rows past the range repeat the last one (never stored)
                cp_async16(st + row * MMA_ROW_STRIDE + piece * 16, qs + ((size_t)(r_begin + gr) * nsb + sb) * 8 + piece);
            }
            if (lane < 16) {
                int gr = tile * 16 + lane;
                gr = gr < R ? gr : R - 1;
                cp_async16(st + 16 * MMA_ROW_STRIDE + lane * 16, hdr + (size_t)(r_begin + gr) * nsb + sb);
            }
        }
        cp_async_commit();
    };
    auto next = [&](It &it) {
        if (++it.j == SP) { it.j = 0; it.u += WARPS; }
    };

    It ii{warp, 0}, ic{warp, 0};
    issue(ii, 0);
    next(ii);
    grid_dependency_wait();
    stage_q8k_rows<WARPS, PREQ>(a, xq, sx, bs, nsb, xstride);
    __syncthreads();
    grid_launch_dependents();

    // this lane's accumulators: rows g, g + 8 of the tile x tokens 8h + 2q, 8h + 2q + 1 (h = token half)
    bool tok_b[NT], tok0[NT], tok1[NT];
    const unsigned char *xb[NT];
    const unsigned char *bsb[NT];                            // this lane's bytes of the mins-term B operand (token 8h + g)
    const float *sx0[NT], *sx1[NT];
    float acc[NT][4];
#pragma unroll
    for (int h = 0; h < NT; h++) {
        const int tb = 8 * h + g, t0 = 8 * h + 2 * q, t1 = t0 + 1;
        tok_b[h] = tb < a.M; tok0[h] = t0 < a.M; tok1[h] = t1 < a.M;
        xb[h] = xq + (size_t)(tok_b[h] ? tb : 0) * xstride + 4 * q;
        bsb[h] = reinterpret_cast<const unsigned char *>(bs) + (size_t)(tok_b[h] ? tb : 0) * nsb * 32 + 4 * q;
        sx0[h] = sx + (tok0[h] ? t0 : 0) * nsb; sx1[h] = sx + (tok1[h] ? t1 : 0) * nsb;
        acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
    }
    int stage = 0;
    while (ic.u < n_units) {
        issue(ii, stage ^ 1);
        next(ii);
        cp_async_wait<1>();
        __syncwarp();
        const int tile = ic.u / S, seg = ic.u - tile * S;
        const int sb = seg * SP + ic.j;
        const unsigned char *st = ring + stage * MMA_STAGE_BYTES;
        const unsigned char *ra = st + g * MMA_ROW_STRIDE + 4 * q, *rb = ra + 8 * MMA_ROW_STRIDE;
        const uint4 Ha = *reinterpret_cast<const uint4 *>(st + 16 * MMA_ROW_STRIDE + g * 16);
        const uint4 Hb = *reinterpret_cast<const uint4 *>(st + 16 * MMA_ROW_STRIDE + (g + 8) * 16);
        int isum[NT][4], msum[NT][4];
#pragma unroll
        for (int h = 0; h < NT; h++)
#pragma unroll
            for (int i = 0; i < 4; i++) isum[h][i] = 0;
        {
            // mins term sum_j m_j * bsum_j for 16 rows x 8 tokens with two MMAs: A = the rows' eight 6-bit mins as
            // bytes (k 0..7), B = the low / high bytes of the tokens' eight sub-block sums; sum = lo + 64 * hi
            const uint32_t ga0 = Ha.y, ga1 = __funnelshift_r(Ha.y, Ha.z, 24), ga2 = __funnelshift_r(Ha.z, Ha.w, 16), ga3 = Ha.w >> 8;
            const uint32_t gb0 = Hb.y, gb1 = __funnelshift_r(Hb.y, Hb.z, 24), gb2 = __funnelshift_r(Hb.z, Hb.w, 16), gb3 = Hb.w >> 8;
            auto two_mins = [](uint32_t grp) { return ((grp >> 12) & 0x3fu) | ((grp >> 10) & 0x3f00u); };   // m(2c), m(2c+1) as bytes
            const uint32_t ma = q == 0 ? (two_mins(ga0) | (two_mins(ga1) << 16)) : q == 1 ? (two_mins(ga2) | (two_mins(ga3) << 16)) : 0u;
            const uint32_t mb = q == 0 ? (two_mins(gb0) | (two_mins(gb1) << 16)) : q == 1 ? (two_mins(gb2) | (two_mins(gb3) << 16)) : 0u;
#pragma unroll
            for (int h = 0; h < NT; h++) {
                uint32_t bl = 0u, bh = 0u;
                if (tok_b[h] && q < 2) {
                    bl = *reinterpret_cast<const uint32_t *>(bsb[h] + sb * 32);
                    bh = *reinterpret_cast<const uint32_t *>(bsb[h] + sb * 32 + 8);
                }
                int dl[4], dh[4];
                mma_u8s8(dl, ma, mb, 0u, 0u, bl, 0u);
                mma_u8s8(dh, ma, mb, 0u, 0u, bh, 0u);
#pragma unroll
                for (int i = 0; i < 4; i++) msum[h][i] = dl[i] + 64 * dh[i];
            }
        }
#pragma unroll
        for (int c = 0; c < 4; c++) {
            // chunk c: piece h = 0 at byte c*16 (weights 64c + 0..15 low nibble, 64c + 32.. high), h = 1 at 64 + c*16
            const uint32_t wa0 = *reinterpret_cast<const uint32_t *>(ra + c * 16), wa1 = *reinterpret_cast<const uint32_t *>(ra + 64 + c * 16);
            const uint32_t wb0 = *reinterpret_cast<const uint32_t *>(rb + c * 16), wb1 = *reinterpret_cast<const uint32_t *>(rb + 64 + c * 16);
            // 24-bit scale groups of the two rows (constant shifts: c is unrolled)
            const uint32_t ga = c == 0 ? Ha.y : c == 1 ? __funnelshift_r(Ha.y, Ha.z, 24) : c == 2 ? __funnelshift_r(Ha.z, Ha.w, 16) : (Ha.w >> 8);
            const uint32_t gb = c == 0 ? Hb.y : c == 1 ? __funnelshift_r(Hb.y, Hb.z, 24) : c == 2 ? __funnelshift_r(Hb.z, Hb.w, 16) : (Hb.w >> 8);
#pragma unroll
            for (int nh = 0; nh < 2; nh++) {                   // sub-block j = 2c + nh: low (0) or high (1) nibbles
                const int j = 2 * c + nh;
                const uint32_t a0 = (wa0 >> (4 * nh)) & 0x0f0f0f0fu, a1 = (wb0 >> (4 * nh)) & 0x0f0f0f0fu;
                const uint32_t a2 = (wa1 >> (4 * nh)) & 0x0f0f0f0fu, a3 = (wb1 >> (4 * nh)) & 0x0f0f0f0fu;
                const int sa = (int)((ga >> (6 * nh)) & 63u), sb_ = (int)((gb >> (6 * nh)) & 63u);
#pragma unroll
                for (int h = 0; h < NT; h++) {                 // token half
                    uint32_t b0 = 0u, b1 = 0u;
                    if (tok_b[h]) {
                        b0 = *reinterpret_cast<const uint32_t *>(xb[h] + sb * 256 + j * 32);
                        b1 = *reinterpret_cast<const uint32_t *>(xb[h] + sb * 256 + j * 32 + 16);
                    }
                    int d[4];
                    mma_u8s8(d, a0, a1, a2, a3, b0, b1);       // exact int32 sub-block dots: rows g, g+8 x two tokens
                    isum[h][0] += sa * d[0]; isum[h][1] += sa * d[1]; isum[h][2] += sb_ * d[2]; isum[h][3] += sb_ * d[3];
                }
            }
        }
        const float da = f16_bits_to_f32(Ha.x), na = f16_bits_to_f32(Ha.x >> 16);
        const float db = f16_bits_to_f32(Hb.x), nb = f16_bits_to_f32(Hb.x >> 16);
#pragma unroll
        for (int h = 0; h < NT; h++) {
            const float s0 = tok0[h] ? sx0[h][sb] : 0.f, s1 = tok1[h] ? sx1[h][sb] : 0.f;
            acc[h][0] += s0 * (da * (float)isum[h][0] - na * (float)msum[h][0]);
            acc[h][1] += s1 * (da * (float)isum[h][1] - na * (float)msum[h][1]);
            acc[h][2] += s0 * (db * (float)isum[h][2] - nb * (float)msum[h][2]);
            acc[h][3] += s1 * (db * (float)isum[h][3] - nb * (float)msum[h][3]);
        }
        __syncwarp();                                          // the stage is free for the next copy
        if (ic.j + 1 == SP) {                                  // end of the unit
            const int row_a = tile * 16 + g, row_b = row_a + 8;
#pragma unroll
            for (int h = 0; h < NT; h++) {
                const int t0 = 8 * h + 2 * q, t1 = t0 + 1;
                if (S == 1) {
                    if (tok0[h] && row_a < R) store_form(a.y + (size_t)t0 * a.N + r_begin + row_a, acc[h][0], a.form, a.bias, r_begin + row_a);
                    if (tok1[h] && row_a < R) store_form(a.y + (size_t)t1 * a.N + r_begin + row_a, acc[h][1], a.form, a.bias, r_begin + row_a);
                    if (tok0[h] && row_b < R) store_form(a.y + (size_t)t0 * a.N + r_begin + row_b, acc[h][2], a.form, a.bias, r_begin + row_b);
                    if (tok1[h] && row_b < R) store_form(a.y + (size_t)t1 * a.N + r_begin + row_b, acc[h][3], a.form, a.bias, r_begin + row_b);
                } else {
                    float *pp = part + (size_t)ic.u * (128 * NT);  // [unit][row 16][token 8 NT]
                    pp[g * (8 * NT) + t0] = acc[h][0]; pp[g * (8 * NT) + t1] = acc[h][1];
                    pp[(g + 8) * (8 * NT) + t0] = acc[h][2]; pp[(g + 8) * (8 * NT) + t1] = acc[h][3];
                }
                acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
            }
        }
        next(ic);
        stage ^= 1;
    }
    cp_async_wait<0>();
    if (S > 1) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < n_tiles * 128 * NT; idx += blockDim.x) {
            const int tile = idx / (128 * NT), rem = idx - tile * (128 * NT);
            const int row = rem / (8 * NT), tok = rem - row * (8 * NT);
            const int r = tile * 16 + row;
            if (r >= R || tok >= a.M) continue;
            float s = 0.f;
            for (int seg = 0; seg < S; seg++) s += part[(size_t)(tile * S + seg) * (128 * NT) + row * (8 * NT) + tok];
            store_form(a.y + (size_t)tok * a.N + r_begin + r, s, a.form, a.bias, r_begin + r);
        }
    }
}

template <int WARPS, bool PREQ>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_q4k_mma_kernel(const GemvArgs a) { gemv_q4k_mma_body<WARPS, PREQ>(a); }

// Grouped form (experts): rows of the group, 8 * NT per pass; see gemv_q4k_grouped_kernel.
template <int WARPS, int NT = 1>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_q4k_mma_grouped_kernel(const GemvArgs a) {
    const int count = __ldg(a.grp_count), off = __ldg(a.grp_offset);
    for (int mb = 0; mb < count; mb += 8 * NT) {
        GemvArgs b = a;
        b.M = count - mb < 8 * NT ? count - mb : 8 * NT;
        if (a.row_index) b.row_index = a.row_index + off + mb;
        else { b.q = a.q + (size_t)(off + mb) * a.K; b.scales = a.scales + (size_t)(off + mb) * (a.K >> 8); b.bsums = a.bsums + (size_t)(off + mb) * (a.K >> 5); }
        b.y = a.y + (size_t)(off + mb) * a.N;
        gemv_q4k_mma_body<WARPS, true, NT>(b);
        __syncthreads();
    }
}

// ============================================================================ Q6_K
// The same scheme for Q6_K (dot_q6k, crates/ojas-cpu/src/cpu_math.rs:674-722): a sub-block is 16 weights with
// its own int8 scale, so the MMA is m16n8k16 (u8 x s8): A = the 6-bit values 0..63 of 16 rows x one sub-block,
// B = 16 int8 activations of up to 8 tokens.  The accumulator is the exact sum q*x; the -32 offset of the
// format is applied as -32 * (sum of the 16 activations), an integer too.  Per super-block and (row, token):
// isum = sum_j sc_j * (dot_j - 32 * xsum_j), exactly the integer the dp4a kernel forms.
//
// Stage = 16 rows x one super-block: low nibbles 16 x 128 B (row stride 144), top bits 16 x 64 B (row stride
// 80), sub-scales 16 x 16 B: 3840 bytes, copied by cp.async; the sixteen f16 super-block scales travel in a
// register of lanes 0..15, loaded one step ahead.
constexpr int MMA6_LO_STRIDE = 144, MMA6_HI_STRIDE = 80;
constexpr int MMA6_HI_OFF = 16 * MMA6_LO_STRIDE;                 // 2304
constexpr int MMA6_SC_OFF = MMA6_HI_OFF + 16 * MMA6_HI_STRIDE;   // 3584
constexpr int MMA6_STAGE_BYTES = MMA6_SC_OFF + 256;              // 3840

__device__ __forceinline__ void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %8, %9, %10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0), "r"(0), "r"(0), "r"(0));
}

__device__ __forceinline__ void mma_s8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %8, %9, %10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0), "r"(0), "r"(0), "r"(0));
}

// Activations in natural order with per-16 sums: xq [M][K + 16] int8, sx [M][nsb] f32, and the sixteen per-16 sums
// of every super-block as two bytes each (sum = 64 * hi + lo, lo in 0..63, hi in -32..31): bs bytes [M][nsb][64] =
// lo[16], hi[16], 32 unused.
template <int WARPS, bool PREQ>
__device__ __forceinline__ void stage_q8k_rows16(const GemvArgs &a, unsigned char *xq, float *sx, int *bs, int nsb, int xstride) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (!PREQ) {
        for (int u = warp; u < a.M * nsb; u += WARPS) {
            const int m = u / nsb, sb = u - m * nsb;
            const Q8kLane ql = quant_q8k_warp(a.x + (size_t)m * a.K + (size_t)sb * 256, lane);
            *reinterpret_cast<uint2 *>(xq + (size_t)m * xstride + sb * 256 + lane * 8) = ql.packed;
            const int s = ql.sum8 + __shfl_xor_sync(0xffffffffu, ql.sum8, 1);
            if ((lane & 1) == 0) {
                unsigned char *bb = reinterpret_cast<unsigned char *>(bs) + (size_t)(m * nsb + sb) * 64 + (lane >> 1);
                bb[0] = (unsigned char)(s & 63);
                bb[16] = (unsigned char)((s >> 6) & 0xff);
            }
            if (lane == 0) sx[m * nsb + sb] = ql.scale;
        }
    } else {
        const int units = nsb * 16;
        for (int idx = threadIdx.x; idx < a.M * units; idx += blockDim.x) {
            const int m = idx / units, rem = idx - m * units;
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(a.q + (size_t)src_row(a, m) * a.K) + rem);
            *reinterpret_cast<uint4 *>(xq + (size_t)m * xstride + rem * 16) = v;
            int s = __dp4a((int)v.x, 0x01010101, 0);
            s = __dp4a((int)v.y, 0x01010101, s);
            s = __dp4a((int)v.z, 0x01010101, s);
            s = __dp4a((int)v.w, 0x01010101, s);
            unsigned char *bb = reinterpret_cast<unsigned char *>(bs) + (size_t)(m * nsb + (rem >> 4)) * 64 + (rem & 15);
            bb[0] = (unsigned char)(s & 63);
            bb[16] = (unsigned char)((s >> 6) & 0xff);
        }
        for (int idx = threadIdx.x; idx < a.M * nsb; idx += blockDim.x) {
            const int m = idx / nsb;
            sx[idx] = __ldg(a.scales + (size_t)src_row(a, m) * nsb + (idx - m * nsb));
        }
    }
}

template <int WARPS, bool PREQ>
__device__ __forceinline__ void gemv_q6k_mma_body(const GemvArgs &a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int nsb = a.K >> 8, S = a.S, SP = nsb / S;
    const int xstride = a.K + MMA_XPAD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    unsigned char *ring = smem + (size_t)warp * 2 * MMA6_STAGE_BYTES;
    unsigned char *xq = smem + (size_t)WARPS * 2 * MMA6_STAGE_BYTES;
    float *sx = reinterpret_cast<float *>(xq + (((size_t)a.M * xstride + 15) & ~(size_t)15));
    int *bs = reinterpret_cast<int *>(sx + sx_floats(a.M, nsb));
    float *part = reinterpret_cast<float *>(bs + a.M * nsb * 16);

    int r_begin, R;
    cta_rows(a, r_begin, R);
    const int n_tiles = (R + 15) >> 4, n_units = n_tiles * S;
    const uint4 *lo = reinterpret_cast<const uint4 *>(a.w.p0);
    const uint4 *hi = reinterpret_cast<const uint4 *>(a.w.p1);
    const uint4 *scp = reinterpret_cast<const uint4 *>(a.w.p2);
    const unsigned short *dp = reinterpret_cast<const unsigned short *>(a.w.p3);

    struct It { int u, j; };
    uint32_t d_next = 0u;                                     // lanes 0..15: f16 d of row (lane) of the step in flight
    auto issue = [&](const It &it, int stage) {
        d_next = 0u;
        if (it.u < n_units) {
            const int tile = it.u / S, seg = it.u - tile * S;
            const int sb = seg * SP + it.j;
            unsigned char *st = ring + stage * MMA6_STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < 4; i++) {                     // 16 rows x 8 pieces of low nibbles
                const int p = lane + 32 * i, row = p >> 3, piece = p & 7;
                int gr = tile * 16 + row;
                gr = gr < R ? gr : R - 1;                     // rows past the range repeat the last one (never stored)
                cp_async16(st + row * MMA6_LO_STRIDE + piece * 16, lo + ((size_t)(r_begin + gr) * nsb + sb) * 8 + piece);
            }
#pragma unroll
            for (int i = 0; i < 2; i++) {                     // 16 rows x 4 pieces of top bits
                const int p = lane + 32 * i, row = p >> 2, piece = p & 3;
                int gr = tile * 16 + row;
                gr = gr < R ? gr : R - 1;
                cp_async16(st + MMA6_HI_OFF + row * MMA6_HI_STRIDE + piece * 16, hi + ((size_t)(r_begin + gr) * nsb + sb) * 4 + piece);
            }
            if (lane < 16) {
                int gr = tile * 16 + lane;
                gr = gr < R ? gr : R - 1;
                const size_t blk = (size_t)(r_begin + gr) * nsb + sb;
                cp_async16(st + MMA6_SC_OFF + lane * 16, scp + blk);
                d_next = __ldg(dp + blk);
            }
        }
        cp_async_commit();
    };
    auto next = [&](It &it) {
        if (++it.j == SP) { it.j = 0; it.u += WARPS; }
    };

    It ii{warp, 0}, ic{warp, 0};
    issue(ii, 0);
    next(ii);
    grid_dependency_wait();
    stage_q8k_rows16<WARPS, PREQ>(a, xq, sx, bs, nsb, xstride);
    __syncthreads();
    grid_launch_dependents();

    const int t0 = 2 * q, t1 = 2 * q + 1;
    const bool tok_b = g < a.M, tok0 = t0 < a.M, tok1 = t1 < a.M;
    const unsigned char *xb = xq + (size_t)(tok_b ? g : 0) * xstride + 4 * q;
    const unsigned char *bsb = reinterpret_cast<const unsigned char *>(bs) + (size_t)(tok_b ? g : 0) * nsb * 64 + 4 * q;
    const float *sx0 = sx + (tok0 ? t0 : 0) * nsb, *sx1 = sx + (tok1 ? t1 : 0) * nsb;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int stage = 0;
    while (ic.u < n_units) {
        const uint32_t d_cur = d_next;                        // belongs to the step about to be consumed
        issue(ii, stage ^ 1);
        next(ii);
        cp_async_wait<1>();
        __syncwarp();
        const int tile = ic.u / S, seg = ic.u - tile * S;
        const int sb = seg * SP + ic.j;
        const unsigned char *st = ring + stage * MMA6_STAGE_BYTES;
        const unsigned char *la = st + g * MMA6_LO_STRIDE + 4 * q, *lb = la + 8 * MMA6_LO_STRIDE;
        const unsigned char *ha = st + MMA6_HI_OFF + g * MMA6_HI_STRIDE + 4 * q, *hb = ha + 8 * MMA6_HI_STRIDE;
        const uint4 Sa = *reinterpret_cast<const uint4 *>(st + MMA6_SC_OFF + g * 16);
        const uint4 Sb = *reinterpret_cast<const uint4 *>(st + MMA6_SC_OFF + (g + 8) * 16);
        const uint32_t sca[4] = {Sa.x, Sa.y, Sa.z, Sa.w}, scb[4] = {Sb.x, Sb.y, Sb.z, Sb.w};
        int isum[4] = {0, 0, 0, 0};
#pragma unroll
        for (int c = 0; c < 4; c++) {
            // chunk c: low-nibble pieces h = 0 (weights 64c+0..15 | 64c+32..47) and h = 1 (64c+16..31 | 64c+48..63)
            const uint32_t la0 = *reinterpret_cast<const uint32_t *>(la + c * 16), la1 = *reinterpret_cast<const uint32_t *>(la + 64 + c * 16);
            const uint32_t lb0 = *reinterpret_cast<const uint32_t *>(lb + c * 16), lb1 = *reinterpret_cast<const uint32_t *>(lb + 64 + c * 16);
            const uint32_t hwa = *reinterpret_cast<const uint32_t *>(ha + c * 16), hwb = *reinterpret_cast<const uint32_t *>(hb + c * 16);
#pragma unroll
            for (int t = 0; t < 4; t++) {                     // sub-block j = 4c + t: weights 64c + 16t .. + 15
                const uint32_t na = (t & 1) ? la1 : la0, nb = (t & 1) ? lb1 : lb0;
                const uint32_t a0 = ((na >> (4 * (t >> 1))) & 0x0f0f0f0fu) | (t < 2 ? ((hwa << (4 - 2 * t)) & 0x30303030u) : ((hwa >> (2 * t - 4)) & 0x30303030u));
                const uint32_t a1 = ((nb >> (4 * (t >> 1))) & 0x0f0f0f0fu) | (t < 2 ? ((hwb << (4 - 2 * t)) & 0x30303030u) : ((hwb >> (2 * t - 4)) & 0x30303030u));
                uint32_t b0 = 0u;
                if (tok_b) b0 = *reinterpret_cast<const uint32_t *>(xb + sb * 256 + (4 * c + t) * 16);
                int d[4];
                mma_u8s8_k16(d, a0, a1, b0);                  // exact sums q*x: rows g, g+8 x tokens 2q, 2q+1
                const int s_a = (int)(signed char)((sca[c] >> (8 * t)) & 0xffu), s_b = (int)(signed char)((scb[c] >> (8 * t)) & 0xffu);
                isum[0] += s_a * d[0]; isum[1] += s_a * d[1];
                isum[2] += s_b * d[2]; isum[3] += s_b * d[3];
            }
        }
        {
            // the format's -32: isum -= 32 * sum_j sc_j * xsum_j, the sum over the sixteen sub-blocks by two MMAs
            // (A = the rows' sixteen int8 sub-scales, B = low / high bytes of the tokens' per-16 activation sums)
            uint32_t bl = 0u, bh = 0u;
            if (tok_b) {
                bl = *reinterpret_cast<const uint32_t *>(bsb + sb * 64);
                bh = *reinterpret_cast<const uint32_t *>(bsb + sb * 64 + 16);
            }
            int cl[4], ch[4];
            const uint32_t wa = q == 0 ? Sa.x : q == 1 ? Sa.y : q == 2 ? Sa.z : Sa.w;
            const uint32_t wb = q == 0 ? Sb.x : q == 1 ? Sb.y : q == 2 ? Sb.z : Sb.w;
            mma_s8s8_k16(cl, wa, wb, bl);
            mma_s8s8_k16(ch, wa, wb, bh);
#pragma unroll
            for (int i = 0; i < 4; i++) isum[i] -= 32 * (cl[i] + 64 * ch[i]);
        }
        const float da = f16_bits_to_f32(__shfl_sync(0xffffffffu, d_cur, g)), db = f16_bits_to_f32(__shfl_sync(0xffffffffu, d_cur, g + 8));
        const float s0 = tok0 ? sx0[sb] : 0.f, s1 = tok1 ? sx1[sb] : 0.f;
        acc[0] += (s0 * da) * (float)isum[0];
        acc[1] += (s1 * da) * (float)isum[1];
        acc[2] += (s0 * db) * (float)isum[2];
        acc[3] += (s1 * db) * (float)isum[3];
        __syncwarp();
        if (ic.j + 1 == SP) {
            const int row_a = tile * 16 + g, row_b = row_a + 8;
            if (S == 1) {
                if (tok0 && row_a < R) store_form(a.y + (size_t)t0 * a.N + r_begin + row_a, acc[0], a.form, a.bias, r_begin + row_a);
                if (tok1 && row_a < R) store_form(a.y + (size_t)t1 * a.N + r_begin + row_a, acc[1], a.form, a.bias, r_begin + row_a);
                if (tok0 && row_b < R) store_form(a.y + (size_t)t0 * a.N + r_begin + row_b, acc[2], a.form, a.bias, r_begin + row_b);
                if (tok1 && row_b < R) store_form(a.y + (size_t)t1 * a.N + r_begin + row_b, acc[3], a.form, a.bias, r_begin + row_b);
            } else {
                float *pp = part + (size_t)ic.u * 128;
                pp[g * 8 + t0] = acc[0]; pp[g * 8 + t1] = acc[1];
                pp[(g + 8) * 8 + t0] = acc[2]; pp[(g + 8) * 8 + t1] = acc[3];
            }
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        }
        next(ic);
        stage ^= 1;
    }
    cp_async_wait<0>();
    if (S > 1) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < n_tiles * 128; idx += blockDim.x) {
            const int tile = idx >> 7, row = (idx >> 3) & 15, tok = idx & 7;
            const int r = tile * 16 + row;
            if (r >= R || tok >= a.M) continue;
            float s = 0.f;
            for (int seg = 0; seg < S; seg++) s += part[(size_t)(tile * S + seg) * 128 + row * 8 + tok];
            store_form(a.y + (size_t)tok * a.N + r_begin + r, s, a.form, a.bias, r_begin + r);
        }
    }
}

template <int WARPS, bool PREQ>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_q6k_mma_kernel(const GemvArgs a) { gemv_q6k_mma_body<WARPS, PREQ>(a); }

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_q6k_mma_grouped_kernel(const GemvArgs a) {
    const int count = __ldg(a.grp_count), off = __ldg(a.grp_offset);
    for (int mb = 0; mb < count; mb += 8) {
        GemvArgs b = a;
        b.M = count - mb < 8 ? count - mb : 8;
        if (a.row_index) b.row_index = a.row_index + off + mb;
        else { b.q = a.q + (size_t)(off + mb) * a.K; b.scales = a.scales + (size_t)(off + mb) * (a.K >> 8); b.bsums = a.bsums + (size_t)(off + mb) * (a.K >> 5); }
        b.y = a.y + (size_t)(off + mb) * a.N;
        gemv_q6k_mma_body<WARPS, true>(b);
        __syncthreads();
    }
}

// ============================================================================ Q8_0
// Q8_0 keeps fp32 activations (dot_q80, crates/ojas-cpu/src/cpu_math.rs:971-981): per 32-weight block
// acc = sum q_i * x_i in fp32, then sum += d * acc.  Here the block sum comes from the f16 tensor-core MMA
// (m16n8k16, fp32 accumulate) without giving up fp32 accuracy: the int8 weights are exact in f16, and each
// activation enters as two f16 terms x = hi + lo (hi = f16(x'), lo = f16(x' - hi), x' = x scaled by a power of
// two per 256 values so that neither term overflows or underflows); every product is exact in fp32, so what
// remains is fp32 summation order, as in the per-lane FMA kernel.  Two MMAs (hi, lo) per 16 weights.
//
// Stage = 16 rows x one super-block: 16 x 256 int8 (row stride 288 so that the 8-byte fragment reads of the
// eight rows of a half-warp fall in different banks) + 16 x 8 f16 block scales: 4864 bytes.
// k order inside a 32-block: lane q owns bytes 8q .. 8q+7; the first four are its share of the first MMA
// (logical k 2q, 2q+1, 2q+8, 2q+9), the last four of the second; the activations use the same order.
constexpr int MMA8_ROW_STRIDE = 288;
constexpr int MMA8_D_OFF = 16 * MMA8_ROW_STRIDE;          // 4608
constexpr int MMA8_STAGE_BYTES = MMA8_D_OFF + 256;        // 4864
constexpr int MMA8_XPAD = 32;                             // activation rows are K + 32 halves apart (bank spread)

__device__ __forceinline__ void mma_f16_k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// two int8 (byte pair `sel` of w ^ 0x80808080) -> half2, exactly: 0x6400 | (b + 128) is 1152 + b
__device__ __forceinline__ uint32_t s8x2_to_h2(uint32_t w_biased, int sel) {
    const uint32_t t = sel == 0 ? __byte_perm(w_biased, 0x64646464u, 0x4140) : __byte_perm(w_biased, 0x64646464u, 0x4342);
    const uint32_t k1152 = 0x64806480u;
    const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&t), *reinterpret_cast<const __half2 *>(&k1152));
    return *reinterpret_cast<const uint32_t *>(&r);
}

// One block of 256 activations -> the two f16 terms and the power-of-two factor that scales their sum back.
__device__ __forceinline__ void q80_split_block(const float *seg, int lane, uint4 &hi, uint4 &lo, float &up) {
    const float4 p0 = __ldg(reinterpret_cast<const float4 *>(seg) + lane * 2);
    const float4 p1 = __ldg(reinterpret_cast<const float4 *>(seg) + lane * 2 + 1);
    const float v[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    // bring the largest magnitude into [2^13, 2^14): hi never overflows f16 and lo stays normal for all
    // but terms 2^-24 below it; mx == 0, infinities and NaNs keep a factor of 1
    int e = 0;
    if (mx > 0.0f && mx < 3.0e38f) e = ilogbf(mx) - 13;
    e = e < -100 ? -100 : e;                                  // keep 2^-e finite for vanishing blocks
    const float down = ldexpf(1.0f, -e);
    up = ldexpf(1.0f, e);
    uint32_t hw[4], lw[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float s0 = v[2 * i] * down, s1 = v[2 * i + 1] * down;
        const __half h0 = __float2half_rn(s0), h1 = __float2half_rn(s1);
        const __half l0 = __float2half_rn(s0 - __half2float(h0)), l1 = __float2half_rn(s1 - __half2float(h1));
        hw[i] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
        lw[i] = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
    }
    hi = make_uint4(hw[0], hw[1], hw[2], hw[3]);
    lo = make_uint4(lw[0], lw[1], lw[2], lw[3]);
}

// The split of a whole batch, once per call: hi, lo [rows][K] f16 in natural order, fx [rows][K / 256].
__global__ void __launch_bounds__(256) q80_split_kernel(const float *x, uint4 *hi, uint4 *lo, float *fx, long long n_sb) {
    const int lane = threadIdx.x & 31;
    const long long sb = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (sb >= n_sb) return;
    uint4 h, l;
    float up;
    q80_split_block(x + sb * 256, lane, h, l, up);
    hi[sb * 32 + lane] = h;
    lo[sb * 32 + lane] = l;
    if (lane == 0) fx[sb] = up;
}

template <int WARPS, bool PRE>
__device__ __forceinline__ void gemv_q80_mma_body(const GemvArgs &a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int nsb = a.K >> 8, S = a.S, SP = nsb / S;
    const int xstride = a.K + MMA8_XPAD;                      // halves
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    unsigned char *ring = smem + (size_t)warp * 2 * MMA8_STAGE_BYTES;
    __half *xh = reinterpret_cast<__half *>(smem + (size_t)WARPS * 2 * MMA8_STAGE_BYTES);   // [M][K + 32]
    __half *xl = xh + (size_t)a.M * xstride;
    float *fx = reinterpret_cast<float *>(xl + (size_t)a.M * xstride);                      // [M][nsb] power-of-two factors
    float *part = fx + sx_floats(a.M, nsb);

    int r_begin, R;
    cta_rows(a, r_begin, R);
    const int n_tiles = (R + 15) >> 4, n_units = n_tiles * S;
    const uint4 *qp = reinterpret_cast<const uint4 *>(a.w.p0);
    const uint4 *dp = reinterpret_cast<const uint4 *>(a.w.p1);                              // 8 f16 per (row, super-block)

    struct It { int u, j; };
    auto issue = [&](const It &it, int stage) {
        if (it.u < n_units) {
            const int tile = it.u / S, seg = it.u - tile * S;
            const int sb = seg * SP + it.j;
            unsigned char *st = ring + stage * MMA8_STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < 8; i++) {                     // 16 rows x 16 pieces of 16 int8
                const int p = lane + 32 * i, row = p >> 4, piece = p & 15;
                int gr = tile * 16 + row;
                gr = gr < R ? gr : R - 1;                     // rows past the range repeat the last one (never stored)
                cp_async16(st + row * MMA8_ROW_STRIDE + piece * 16, qp + ((size_t)(r_begin + gr) * nsb + sb) * 16 + piece);
            }
            if (lane < 16) {
                int gr = tile * 16 + lane;
                gr = gr < R ? gr : R - 1;
                cp_async16(st + MMA8_D_OFF + lane * 16, dp + (size_t)(r_begin + gr) * nsb + sb);
            }
        }
        cp_async_commit();
    };
    auto next = [&](It &it) {
        if (++it.j == SP) { it.j = 0; it.u += WARPS; }
    };

    It ii{warp, 0}, ic{warp, 0};
    issue(ii, 0);
    next(ii);
    grid_dependency_wait();
    if (!PRE) {
        // activations: one warp per (row, 256 values); lane l owns values 8l .. 8l+7
        for (int u = warp; u < a.M * nsb; u += WARPS) {
            const int m = u / nsb, sb = u - m * nsb;
            uint4 hi, lo;
            float up;
            q80_split_block(a.x + (size_t)m * a.K + (size_t)sb * 256, lane, hi, lo, up);
            *reinterpret_cast<uint4 *>(xh + (size_t)m * xstride + sb * 256 + lane * 8) = hi;
            *reinterpret_cast<uint4 *>(xl + (size_t)m * xstride + sb * 256 + lane * 8) = lo;
            if (lane == 0) fx[m * nsb + sb] = up;
        }
    } else {
        // split once per call by q80_split_kernel: a.q = hi terms, a.bsums = lo terms (both [M][K] f16), a.scales = factors
        const int units = a.K >> 3;
        const uint4 *shi = reinterpret_cast<const uint4 *>(a.q), *slo = reinterpret_cast<const uint4 *>(a.bsums);
        for (int idx = threadIdx.x; idx < a.M * units; idx += blockDim.x) {
            const int m = idx / units, un = idx - m * units;
            *reinterpret_cast<uint4 *>(xh + (size_t)m * xstride + un * 8) = __ldg(shi + idx);
            *reinterpret_cast<uint4 *>(xl + (size_t)m * xstride + un * 8) = __ldg(slo + idx);
        }
        for (int idx = threadIdx.x; idx < a.M * nsb; idx += blockDim.x) fx[idx] = __ldg(a.scales + idx);
    }
    __syncthreads();
    grid_launch_dependents();

    const int t0 = 2 * q, t1 = 2 * q + 1;
    const bool tok_b = g < a.M, tok0 = t0 < a.M, tok1 = t1 < a.M;
    const __half *xhb = xh + (size_t)(tok_b ? g : 0) * xstride + 8 * q;
    const __half *xlb = xl + (size_t)(tok_b ? g : 0) * xstride + 8 * q;
    const float *f0 = fx + (tok0 ? t0 : 0) * nsb, *f1 = fx + (tok1 ? t1 : 0) * nsb;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int stage = 0;
    while (ic.u < n_units) {
        issue(ii, stage ^ 1);
        next(ii);
        cp_async_wait<1>();
        __syncwarp();
        const int tile = ic.u / S, seg = ic.u - tile * S;
        const int sb = seg * SP + ic.j;
        const unsigned char *st = ring + stage * MMA8_STAGE_BYTES;
        const unsigned char *wa = st + g * MMA8_ROW_STRIDE + 8 * q, *wb = wa + 8 * MMA8_ROW_STRIDE;
        const uint4 Da = *reinterpret_cast<const uint4 *>(st + MMA8_D_OFF + g * 16);
        const uint4 Db = *reinterpret_cast<const uint4 *>(st + MMA8_D_OFF + (g + 8) * 16);
        const uint32_t dwa[4] = {Da.x, Da.y, Da.z, Da.w}, dwb[4] = {Db.x, Db.y, Db.z, Db.w};
        float sbsum[4] = {0.f, 0.f, 0.f, 0.f};                // sum over the super-block's blocks of d * acc
#pragma unroll
        for (int b = 0; b < 8; b++) {
            const uint2 A2 = *reinterpret_cast<const uint2 *>(wa + b * 32), B2 = *reinterpret_cast<const uint2 *>(wb + b * 32);
            uint4 XH = make_uint4(0u, 0u, 0u, 0u), XL = XH;
            if (tok_b) {
                XH = *reinterpret_cast<const uint4 *>(xhb + sb * 256 + b * 32);
                XL = *reinterpret_cast<const uint4 *>(xlb + sb * 256 + b * 32);
            }
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            {
                const uint32_t wa_ = A2.x ^ 0x80808080u, wb_ = B2.x ^ 0x80808080u;
                const uint32_t a0 = s8x2_to_h2(wa_, 0), a2 = s8x2_to_h2(wa_, 1), a1 = s8x2_to_h2(wb_, 0), a3 = s8x2_to_h2(wb_, 1);
                mma_f16_k16(c, a0, a1, a2, a3, XH.x, XH.y);
                mma_f16_k16(c, a0, a1, a2, a3, XL.x, XL.y);
            }
            {
                const uint32_t wa_ = A2.y ^ 0x80808080u, wb_ = B2.y ^ 0x80808080u;
                const uint32_t a0 = s8x2_to_h2(wa_, 0), a2 = s8x2_to_h2(wa_, 1), a1 = s8x2_to_h2(wb_, 0), a3 = s8x2_to_h2(wb_, 1);
                mma_f16_k16(c, a0, a1, a2, a3, XH.z, XH.w);
                mma_f16_k16(c, a0, a1, a2, a3, XL.z, XL.w);
            }
            const float da = f16_bits_to_f32(dwa[b >> 1] >> (16 * (b & 1))), db = f16_bits_to_f32(dwb[b >> 1] >> (16 * (b & 1)));
            sbsum[0] = fmaf(da, c[0], sbsum[0]); sbsum[1] = fmaf(da, c[1], sbsum[1]);
            sbsum[2] = fmaf(db, c[2], sbsum[2]); sbsum[3] = fmaf(db, c[3], sbsum[3]);
        }
        const float s0 = tok0 ? f0[sb] : 0.f, s1 = tok1 ? f1[sb] : 0.f;
        acc[0] = fmaf(s0, sbsum[0], acc[0]); acc[1] = fmaf(s1, sbsum[1], acc[1]);
        acc[2] = fmaf(s0, sbsum[2], acc[2]); acc[3] = fmaf(s1, sbsum[3], acc[3]);
        __syncwarp();
        if (ic.j + 1 == SP) {
            const int row_a = tile * 16 + g, row_b = row_a + 8;
            if (S == 1) {
                if (tok0 && row_a < R) store_form(a.y + (size_t)t0 * a.N + r_begin + row_a, acc[0], a.form, a.bias, r_begin + row_a);
                if (tok1 && row_a < R) store_form(a.y + (size_t)t1 * a.N + r_begin + row_a, acc[1], a.form, a.bias, r_begin + row_a);
                if (tok0 && row_b < R) store_form(a.y + (size_t)t0 * a.N + r_begin + row_b, acc[2], a.form, a.bias, r_begin + row_b);
                if (tok1 && row_b < R) store_form(a.y + (size_t)t1 * a.N + r_begin + row_b, acc[3], a.form, a.bias, r_begin + row_b);
            } else {
                float *pp = part + (size_t)ic.u * 128;
                pp[g * 8 + t0] = acc[0]; pp[g * 8 + t1] = acc[1];
                pp[(g + 8) * 8 + t0] = acc[2]; pp[(g + 8) * 8 + t1] = acc[3];
            }
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        }
        next(ic);
        stage ^= 1;
    }
    cp_async_wait<0>();
    if (S > 1) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < n_tiles * 128; idx += blockDim.x) {
            const int tile = idx >> 7, row = (idx >> 3) & 15, tok = idx & 7;
            const int r = tile * 16 + row;
            if (r >= R || tok >= a.M) continue;
            float s = 0.f;
            for (int seg = 0; seg < S; seg++) s += part[(size_t)(tile * S + seg) * 128 + row * 8 + tok];
            store_form(a.y + (size_t)tok * a.N + r_begin + r, s, a.form, a.bias, r_begin + r);
        }
    }
}

template <int WARPS, bool PRE>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_q80_mma_kernel(const GemvArgs a) { gemv_q80_mma_body<WARPS, PRE>(a); }
