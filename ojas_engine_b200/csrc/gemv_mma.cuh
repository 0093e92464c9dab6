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

// Activations into shared memory in natural order: xq [M][K + 16] int8, sx [M][nsb] f32, bs [M][nsb * 8] i32.
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
            if ((lane & 3) == 0) bs[(m * nsb + sb) * 8 + (lane >> 2)] = s;
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
            const int m = idx / (nsb * 8);
            bs[idx] = __ldg(a.bsums + (size_t)src_row(a, m) * nsb * 8 + (idx - m * nsb * 8));
        }
    }
}

// a.S = segments per tile (divides the super-block count); a.M <= 8.
template <int WARPS, bool PREQ>
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

    // this lane's accumulators: rows g, g + 8 of the tile x tokens 2q, 2q + 1
    const int t0 = 2 * q, t1 = 2 * q + 1;
    const bool tok_b = g < a.M, tok0 = t0 < a.M, tok1 = t1 < a.M;
    const unsigned char *xb = xq + (size_t)(tok_b ? g : 0) * xstride + 4 * q;
    const int *bs0 = bs + (tok0 ? t0 : 0) * nsb * 8, *bs1 = bs + (tok1 ? t1 : 0) * nsb * 8;
    const float *sx0 = sx + (tok0 ? t0 : 0) * nsb, *sx1 = sx + (tok1 ? t1 : 0) * nsb;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
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
        int isum[4] = {0, 0, 0, 0}, msum[4] = {0, 0, 0, 0};
#pragma unroll
        for (int c = 0; c < 4; c++) {
            // chunk c: piece h = 0 at byte c*16 (weights 64c + 0..15 low nibble, 64c + 32.. high), h = 1 at 64 + c*16
            const uint32_t wa0 = *reinterpret_cast<const uint32_t *>(ra + c * 16), wa1 = *reinterpret_cast<const uint32_t *>(ra + 64 + c * 16);
            const uint32_t wb0 = *reinterpret_cast<const uint32_t *>(rb + c * 16), wb1 = *reinterpret_cast<const uint32_t *>(rb + 64 + c * 16);
            // 24-bit scale groups of the two rows (constant shifts: c is unrolled)
            const uint32_t ga = c == 0 ? Ha.y : c == 1 ? __funnelshift_r(Ha.y, Ha.z, 24) : c == 2 ? __funnelshift_r(Ha.z, Ha.w, 16) : (Ha.w >> 8);
            const uint32_t gb = c == 0 ? Hb.y : c == 1 ? __funnelshift_r(Hb.y, Hb.z, 24) : c == 2 ? __funnelshift_r(Hb.z, Hb.w, 16) : (Hb.w >> 8);
#pragma unroll
            for (int h = 0; h < 2; h++) {                      // sub-block j = 2c + h: low (h = 0) or high nibbles
                const int j = 2 * c + h;
                const uint32_t a0 = (wa0 >> (4 * h)) & 0x0f0f0f0fu, a1 = (wb0 >> (4 * h)) & 0x0f0f0f0fu;
                const uint32_t a2 = (wa1 >> (4 * h)) & 0x0f0f0f0fu, a3 = (wb1 >> (4 * h)) & 0x0f0f0f0fu;
                uint32_t b0 = 0u, b1 = 0u;
                if (tok_b) {
                    b0 = *reinterpret_cast<const uint32_t *>(xb + sb * 256 + j * 32);
                    b1 = *reinterpret_cast<const uint32_t *>(xb + sb * 256 + j * 32 + 16);
                }
                int d[4];
                mma_u8s8(d, a0, a1, a2, a3, b0, b1);           // exact int32 sub-block dots: rows g, g+8 x tokens 2q, 2q+1
                const int sa = (int)((ga >> (6 * h)) & 63u), sb_ = (int)((gb >> (6 * h)) & 63u);
                const int ma = (int)((ga >> (12 + 6 * h)) & 63u), mb = (int)((gb >> (12 + 6 * h)) & 63u);
                const int u0 = tok0 ? bs0[sb * 8 + j] : 0, u1 = tok1 ? bs1[sb * 8 + j] : 0;
                isum[0] += sa * d[0]; isum[1] += sa * d[1]; isum[2] += sb_ * d[2]; isum[3] += sb_ * d[3];
                msum[0] += ma * u0;   msum[1] += ma * u1;   msum[2] += mb * u0;    msum[3] += mb * u1;
            }
        }
        const float da = f16_bits_to_f32(Ha.x), na = f16_bits_to_f32(Ha.x >> 16);
        const float db = f16_bits_to_f32(Hb.x), nb = f16_bits_to_f32(Hb.x >> 16);
        const float s0 = tok0 ? sx0[sb] : 0.f, s1 = tok1 ? sx1[sb] : 0.f;
        acc[0] += s0 * (da * (float)isum[0] - na * (float)msum[0]);
        acc[1] += s1 * (da * (float)isum[1] - na * (float)msum[1]);
        acc[2] += s0 * (db * (float)isum[2] - nb * (float)msum[2]);
        acc[3] += s1 * (db * (float)isum[3] - nb * (float)msum[3]);
        __syncwarp();                                          // the stage is free for the next copy
        if (ic.j + 1 == SP) {                                  // end of the unit: rows g, g+8 x tokens t0, t1
            const int row_a = tile * 16 + g, row_b = row_a + 8;
            if (S == 1) {
                if (tok0 && row_a < R) store_form(a.y + (size_t)t0 * a.N + r_begin + row_a, acc[0], a.form, a.bias, r_begin + row_a);
                if (tok1 && row_a < R) store_form(a.y + (size_t)t1 * a.N + r_begin + row_a, acc[1], a.form, a.bias, r_begin + row_a);
                if (tok0 && row_b < R) store_form(a.y + (size_t)t0 * a.N + r_begin + row_b, acc[2], a.form, a.bias, r_begin + row_b);
                if (tok1 && row_b < R) store_form(a.y + (size_t)t1 * a.N + r_begin + row_b, acc[3], a.form, a.bias, r_begin + row_b);
            } else {
                float *pp = part + (size_t)ic.u * 128;         // [unit][row 16][token 8]
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
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_q4k_mma_kernel(const GemvArgs a) { gemv_q4k_mma_body<WARPS, PREQ>(a); }

// Grouped form (experts): rows of the group, eight per pass; see gemv_q4k_grouped_kernel.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_q4k_mma_grouped_kernel(const GemvArgs a) {
    const int count = __ldg(a.grp_count), off = __ldg(a.grp_offset);
    for (int mb = 0; mb < count; mb += 8) {
        GemvArgs b = a;
        b.M = count - mb < 8 ? count - mb : 8;
        if (a.row_index) b.row_index = a.row_index + off + mb;
        else { b.q = a.q + (size_t)(off + mb) * a.K; b.scales = a.scales + (size_t)(off + mb) * (a.K >> 8); b.bsums = a.bsums + (size_t)(off + mb) * (a.K >> 5); }
        b.y = a.y + (size_t)(off + mb) * a.N;
        gemv_q4k_mma_body<WARPS, true>(b);
        __syncthreads();
    }
}
