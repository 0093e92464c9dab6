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
    int K, N, M, form;
};

__device__ __forceinline__ void store_form(float *yp, float v, int form, const float *bias, int n) {
    if (form == OJAS_B200_ACCUM) v += *yp;
    else if (form == OJAS_B200_BIAS) v += __ldg(bias + n);
    *yp = v;
}

// Fixed-order sum of the item partials of every row of this CTA, then the store.
template <int MT>
__device__ __forceinline__ void finish_rows(const float *part, int R, int G8, int r_begin, const GemvArgs &a) {
    for (int idx = threadIdx.x; idx < R * MT; idx += blockDim.x) {
        const int r = idx / MT, m = idx - r * MT;
        if (m >= a.M) continue;
        float s = 0.0f;
        for (int g = 0; g < G8; g++) s += part[(r * G8 + g) * MT + m];
        const int n = r_begin + r;
        store_form(a.y + (size_t)m * a.N + n, s, a.form, a.bias, n);
    }
}

// Quantize (or copy pre-quantized) activations into shared memory.  BS16: keep per-16 sums
// (Q6_K) instead of per-32 sums (Q4_K).
template <int MT, bool PREQ, bool BS16>
__device__ __forceinline__ void stage_q8k(const GemvArgs &a, unsigned char *xq, float *sx, int *bs, int nsb, int Kpad) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int NB = BS16 ? 16 : 8;
    if (!PREQ) {
        for (int u = warp; u < MT * nsb; u += GEMV_WARPS) {
            const int m = u / nsb, sb = u - m * nsb;
            uint2 packed = make_uint2(0u, 0u);
            int s = 0;
            float scale = 0.0f;
            if (m < a.M) {
                Q8kLane ql = quant_q8k_warp(a.x + (size_t)m * a.K + (size_t)sb * 256, lane);
                packed = ql.packed; s = ql.sum8; scale = ql.scale;
            }
            const int un = lane >> 1;
            *reinterpret_cast<uint2 *>(xq + (size_t)m * Kpad + xq_unit(sb, un >> 2, un & 3) * 16 + (lane & 1) * 8) = packed;
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            if (BS16) {
                if ((lane & 1) == 0) bs[(m * nsb + sb) * 16 + (lane >> 1)] = s;
            } else {
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if ((lane & 3) == 0) bs[(m * nsb + sb) * 8 + (lane >> 2)] = s;
            }
            if (lane == 0) sx[m * nsb + sb] = scale;
        }
    } else {
        const int units = nsb * 16;
        for (int idx = threadIdx.x; idx < MT * units; idx += blockDim.x) {
            const int m = idx / units, rem = idx - m * units;
            const int sb = rem >> 4, un = rem & 15;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m < a.M) v = __ldg(reinterpret_cast<const uint4 *>(a.q + (size_t)m * a.K) + rem);
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
            sx[idx] = (m < a.M) ? __ldg(a.scales + (size_t)m * nsb + (idx - m * nsb)) : 0.0f;
        }
        if (!BS16) {
            for (int idx = threadIdx.x; idx < MT * nsb * NB; idx += blockDim.x) {
                const int m = idx / (nsb * NB);
                bs[idx] = (m < a.M) ? __ldg(a.bsums + (size_t)m * nsb * NB + (idx - m * nsb * NB)) : 0;
            }
        }
    }
}

// ---------------------------------------------------------------------------- Q4_K
struct Q4kRegs { uint4 A, B, H; };

// The two 6-bit sub-block scales and mins of chunk c, packed as bytes (lo = sub-block 2c,
// hi = 2c + 1).  Same bit rules as scale_min_k4 (crates/ojas-cpu/src/cpu_math.rs:566-574).
__device__ __forceinline__ void q4k_scales(const uint4 &H, int c, int &s1, int &s2, int &m1, int &m2) {
    const int sh = (c & 1) * 16;
    const uint32_t a = (H.y >> sh) & 0xffffu, b = (H.z >> sh) & 0xffffu, e = (H.w >> sh) & 0xffffu;
    const uint32_t S_lo = a & 0x3f3fu, M_lo = b & 0x3f3fu;
    const uint32_t S_hi = (e & 0x0f0fu) | ((a >> 2) & 0x3030u);
    const uint32_t M_hi = ((e >> 4) & 0x0f0fu) | ((b >> 2) & 0x3030u);
    const uint32_t S = (c < 2) ? S_lo : S_hi, Mn = (c < 2) ? M_lo : M_hi;
    s1 = (int)(S & 0xffu); s2 = (int)(S >> 8);
    m1 = (int)(Mn & 0xffu); m2 = (int)(Mn >> 8);
}

template <int MT, bool PREQ, bool DUMP>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_q4k_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int nsb = a.K >> 8, G8 = (nsb + 7) >> 3;
    const int Kpad = ((nsb + 1) >> 1) * 512;
    unsigned char *xq = smem;
    float *sx = reinterpret_cast<float *>(smem + (size_t)MT * Kpad);
    int *bs = reinterpret_cast<int *>(sx + MT * nsb);
    float *part = reinterpret_cast<float *>(bs + MT * nsb * 8);

    const int r_begin = (int)((long long)a.N * blockIdx.x / gridDim.x);
    const int r_end = (int)((long long)a.N * (blockIdx.x + 1) / gridDim.x);
    const int R = r_end - r_begin, n_items = R * G8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sbi = lane >> 2, c = lane & 3;
    const uint4 *qs = reinterpret_cast<const uint4 *>(a.w.p0);
    const uint4 *hdr = reinterpret_cast<const uint4 *>(a.w.p1);

    auto load = [&](int item, Q4kRegs &r) {
        const int rr = item / G8, sb = (item - rr * G8) * 8 + sbi;
        r.A = r.B = r.H = make_uint4(0u, 0u, 0u, 0u);
        if (item < n_items && sb < nsb) {
            const size_t blk = (size_t)(r_begin + rr) * nsb + sb;
            r.A = ldg_stream_u4(qs + blk * 8 + c);
            r.B = ldg_stream_u4(qs + blk * 8 + 4 + c);
            r.H = __ldg(hdr + blk);
        }
    };

    Q4kRegs cur;
    load(warp, cur);                      // weights are in flight while x is quantized
    stage_q8k<MT, PREQ, false>(a, xq, sx, bs, nsb, Kpad);
    __syncthreads();

    for (int item = warp; item < n_items; item += GEMV_WARPS) {
        Q4kRegs nxt;
        load(item + GEMV_WARPS, nxt);
        const int rr = item / G8, sb = (item - rr * G8) * 8 + sbi;
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0.0f;
        if (sb < nsb) {
            int s1, s2, m1, m2;
            q4k_scales(cur.H, c, s1, s2, m1, m2);
            const float d = f16_bits_to_f32(cur.H.x), dmin = f16_bits_to_f32(cur.H.x >> 16);
            const uint32_t a_lo[4] = {cur.A.x & 0x0f0f0f0fu, cur.A.y & 0x0f0f0f0fu, cur.A.z & 0x0f0f0f0fu, cur.A.w & 0x0f0f0f0fu};
            const uint32_t a_hi[4] = {(cur.A.x >> 4) & 0x0f0f0f0fu, (cur.A.y >> 4) & 0x0f0f0f0fu, (cur.A.z >> 4) & 0x0f0f0f0fu, (cur.A.w >> 4) & 0x0f0f0f0fu};
            const uint32_t b_lo[4] = {cur.B.x & 0x0f0f0f0fu, cur.B.y & 0x0f0f0f0fu, cur.B.z & 0x0f0f0f0fu, cur.B.w & 0x0f0f0f0fu};
            const uint32_t b_hi[4] = {(cur.B.x >> 4) & 0x0f0f0f0fu, (cur.B.y >> 4) & 0x0f0f0f0fu, (cur.B.z >> 4) & 0x0f0f0f0fu, (cur.B.w >> 4) & 0x0f0f0f0fu};
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const uint4 *xm = reinterpret_cast<const uint4 *>(xq + (size_t)m * Kpad);
                const uint4 X0 = xm[xq_unit(sb, c, 0)], X1 = xm[xq_unit(sb, c, 1)];
                const uint4 X2 = xm[xq_unit(sb, c, 2)], X3 = xm[xq_unit(sb, c, 3)];
                int pA = 0, pB = 0;   // exact int32 dots of sub-blocks 2c and 2c+1
                pA = __dp4a((int)a_lo[0], (int)X0.x, pA); pA = __dp4a((int)a_lo[1], (int)X0.y, pA);
                pA = __dp4a((int)a_lo[2], (int)X0.z, pA); pA = __dp4a((int)a_lo[3], (int)X0.w, pA);
                pA = __dp4a((int)b_lo[0], (int)X1.x, pA); pA = __dp4a((int)b_lo[1], (int)X1.y, pA);
                pA = __dp4a((int)b_lo[2], (int)X1.z, pA); pA = __dp4a((int)b_lo[3], (int)X1.w, pA);
                pB = __dp4a((int)a_hi[0], (int)X2.x, pB); pB = __dp4a((int)a_hi[1], (int)X2.y, pB);
                pB = __dp4a((int)a_hi[2], (int)X2.z, pB); pB = __dp4a((int)a_hi[3], (int)X2.w, pB);
                pB = __dp4a((int)b_hi[0], (int)X3.x, pB); pB = __dp4a((int)b_hi[1], (int)X3.y, pB);
                pB = __dp4a((int)b_hi[2], (int)X3.z, pB); pB = __dp4a((int)b_hi[3], (int)X3.w, pB);
                if (DUMP && m == 0) {
                    int32_t *o = a.idots + (size_t)(r_begin + rr) * (nsb * 8) + sb * 8 + 2 * c;
                    o[0] = pA; o[1] = pB;
                }
                const int2 b2 = *reinterpret_cast<const int2 *>(bs + (m * nsb + sb) * 8 + 2 * c);
                const int isum = s1 * pA + s2 * pB;            // sum_j s_j * idot_j  (exact)
                const int msum = m1 * b2.x + m2 * b2.y;        // sum_j m_j * bsum_j  (exact)
                acc[m] = sx[m * nsb + sb] * (d * (float)isum - dmin * (float)msum);
            }
        }
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const float s = warp_sum(acc[m]);
            if (lane == 0) part[item * MT + m] = s;
        }
        cur = nxt;
    }
    __syncthreads();
    if (!DUMP) finish_rows<MT>(part, R, G8, r_begin, a);
}

// ---------------------------------------------------------------------------- Q6_K
struct Q6kRegs { uint4 A, B, H; uint32_t sc; uint32_t d; };

template <int MT, bool PREQ, bool DUMP>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_q6k_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int nsb = a.K >> 8, G8 = (nsb + 7) >> 3;
    const int Kpad = ((nsb + 1) >> 1) * 512;
    unsigned char *xq = smem;
    float *sx = reinterpret_cast<float *>(smem + (size_t)MT * Kpad);
    int *bs = reinterpret_cast<int *>(sx + MT * nsb);          // per-16 activation sums
    float *part = reinterpret_cast<float *>(bs + MT * nsb * 16);

    const int r_begin = (int)((long long)a.N * blockIdx.x / gridDim.x);
    const int r_end = (int)((long long)a.N * (blockIdx.x + 1) / gridDim.x);
    const int R = r_end - r_begin, n_items = R * G8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sbi = lane >> 2, c = lane & 3;
    const uint4 *lo = reinterpret_cast<const uint4 *>(a.w.p0);
    const uint4 *hi = reinterpret_cast<const uint4 *>(a.w.p1);
    const uint32_t *scp = reinterpret_cast<const uint32_t *>(a.w.p2);
    const unsigned short *dp = reinterpret_cast<const unsigned short *>(a.w.p3);

    auto load = [&](int item, Q6kRegs &r) {
        const int rr = item / G8, sb = (item - rr * G8) * 8 + sbi;
        r.A = r.B = r.H = make_uint4(0u, 0u, 0u, 0u);
        r.sc = 0u; r.d = 0u;
        if (item < n_items && sb < nsb) {
            const size_t blk = (size_t)(r_begin + rr) * nsb + sb;
            r.A = ldg_stream_u4(lo + blk * 8 + c);
            r.B = ldg_stream_u4(lo + blk * 8 + 4 + c);
            r.H = ldg_stream_u4(hi + blk * 4 + c);
            r.sc = __ldg(scp + blk * 4 + c);
            r.d = __ldg(dp + blk);
        }
    };

    Q6kRegs cur;
    load(warp, cur);
    stage_q8k<MT, PREQ, true>(a, xq, sx, bs, nsb, Kpad);
    __syncthreads();

    for (int item = warp; item < n_items; item += GEMV_WARPS) {
        Q6kRegs nxt;
        load(item + GEMV_WARPS, nxt);
        const int rr = item / G8, sb = (item - rr * G8) * 8 + sbi;
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0.0f;
        if (sb < nsb) {
            const float d = f16_bits_to_f32(cur.d);
            const uint32_t Aw[4] = {cur.A.x, cur.A.y, cur.A.z, cur.A.w};
            const uint32_t Bw[4] = {cur.B.x, cur.B.y, cur.B.z, cur.B.w};
            const uint32_t Hw[4] = {cur.H.x, cur.H.y, cur.H.z, cur.H.w};
            // six-bit values 0..63 of the four 16-weight groups t = 0..3 of this chunk
            uint32_t w6[4][4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                w6[0][k] = (Aw[k] & 0x0f0f0f0fu) | ((Hw[k] << 4) & 0x30303030u);
                w6[1][k] = (Bw[k] & 0x0f0f0f0fu) | ((Hw[k] << 2) & 0x30303030u);
                w6[2][k] = ((Aw[k] >> 4) & 0x0f0f0f0fu) | (Hw[k] & 0x30303030u);
                w6[3][k] = ((Bw[k] >> 4) & 0x0f0f0f0fu) | ((Hw[k] >> 2) & 0x30303030u);
            }
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const uint4 *xm = reinterpret_cast<const uint4 *>(xq + (size_t)m * Kpad);
                const int4 b4 = *reinterpret_cast<const int4 *>(bs + (m * nsb + sb) * 16 + 4 * c);
                const int bsum[4] = {b4.x, b4.y, b4.z, b4.w};
                int isum = 0;
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const uint4 X = xm[xq_unit(sb, c, t)];
                    int it = __dp4a((int)w6[t][0], (int)X.x, 0);   // exact int32 dot of 16 weights
                    it = __dp4a((int)w6[t][1], (int)X.y, it);
                    it = __dp4a((int)w6[t][2], (int)X.z, it);
                    it = __dp4a((int)w6[t][3], (int)X.w, it);
                    if (DUMP && m == 0) a.idots[(size_t)(r_begin + rr) * (nsb * 16) + sb * 16 + 4 * c + t] = it;
                    const int st = (int)(signed char)((cur.sc >> (8 * t)) & 0xffu);
                    isum += st * (it - 32 * bsum[t]);              // s*(i) - 32*s*(x sum), exact
                }
                acc[m] = (sx[m * nsb + sb] * d) * (float)isum;
            }
        }
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const float s = warp_sum(acc[m]);
            if (lane == 0) part[item * MT + m] = s;
        }
        cur = nxt;
    }
    __syncthreads();
    if (!DUMP) finish_rows<MT>(part, R, G8, r_begin, a);
}

// ---------------------------------------------------------------------------- Q8_0
// f32 activations in shared memory.  An item is one row x 2048 weights: lane l owns the four
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
    const int K = a.K, G8 = (K + 2047) >> 11;
    const int Kpad = G8 * 2048;
    float4 *xs = reinterpret_cast<float4 *>(smem);                         // [MT][Kpad/4]
    float *part = reinterpret_cast<float *>(smem + (size_t)MT * Kpad * 4);

    const int r_begin = (int)((long long)a.N * blockIdx.x / gridDim.x);
    const int r_end = (int)((long long)a.N * (blockIdx.x + 1) / gridDim.x);
    const int R = r_end - r_begin, n_items = R * G8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint4 *qp = reinterpret_cast<const uint4 *>(a.w.p0);
    const unsigned short *dp = reinterpret_cast<const unsigned short *>(a.w.p1);

    auto load = [&](int item, Q80Regs &r) {
        const int rr = item / G8, g = item - rr * G8;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k0 = g * 2048 + j * 512 + lane * 16;
            r.W[j] = make_uint4(0u, 0u, 0u, 0u);
            r.d[j] = 0u;
            if (item < n_items && k0 < K) {
                const size_t row = (size_t)(r_begin + rr);
                r.W[j] = ldg_stream_u4(qp + (row * K + k0) / 16);
                r.d[j] = __ldg(dp + row * (K / 32) + (k0 >> 5));
            }
        }
    };

    Q80Regs cur;
    load(warp, cur);
    // stage x: float4 (piece-block pb, lane l, idx p) -> xs[m][pb*128 + p*32 + l]
    for (int idx = threadIdx.x; idx < MT * (Kpad / 4); idx += blockDim.x) {
        const int m = idx / (Kpad / 4), f4 = idx - m * (Kpad / 4);
        const int pb = f4 >> 7, l = (f4 >> 2) & 31, p = f4 & 3;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < a.M && f4 * 4 < K) v = __ldg(reinterpret_cast<const float4 *>(a.x + (size_t)m * K) + f4);
        xs[(size_t)m * (Kpad / 4) + pb * 128 + p * 32 + l] = v;
    }
    __syncthreads();

    for (int item = warp; item < n_items; item += GEMV_WARPS) {
        Q80Regs nxt;
        load(item + GEMV_WARPS, nxt);
        const int rr = item / G8, g = item - rr * G8;
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float d = f16_bits_to_f32(cur.d[j]);
            const uint32_t wv[4] = {cur.W[j].x ^ 0x80808080u, cur.W[j].y ^ 0x80808080u, cur.W[j].z ^ 0x80808080u, cur.W[j].w ^ 0x80808080u};
            float wf[16];
#pragma unroll
            for (int p = 0; p < 4; p++)
#pragma unroll
                for (int i = 0; i < 4; i++) wf[p * 4 + i] = s8_to_f32(wv[p], i);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const float4 *xm = xs + (size_t)m * (Kpad / 4) + (g * 4 + j) * 128 + lane;
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
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const float s = warp_sum(acc[m]);
            if (lane == 0) part[item * MT + m] = s;
        }
        cur = nxt;
    }
    __syncthreads();
    finish_rows<MT>(part, R, G8, r_begin, a);
}

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
static size_t gemv_smem_bytes(uint32_t type, int MT, size_t K, size_t rows_max) {
    const size_t nsb = K / 256, G8 = (nsb + 7) / 8;
    const size_t part = rows_max * G8 * MT * 4;
    if (type == OJAS_B200_Q8_0) return (size_t)MT * G8 * 2048 * 4 + part;
    const size_t Kpad = ((nsb + 1) / 2) * 512;
    const size_t nb = (type == OJAS_B200_Q6_K) ? 16 : 8;
    return (size_t)MT * Kpad + (size_t)MT * nsb * 4 + (size_t)MT * nsb * nb * 4 + part;
}

template <typename KernelT>
static int launch_gemv(ojas_b200_ctx *ctx, KernelT kernel, const GemvArgs &args, int grid, size_t smem, const char *name) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "%s: shared memory %zu: %s", name, smem, cudaGetErrorString(e));
    }
    kernel<<<grid, GEMV_THREADS, smem, ctx->stream>>>(args);
    OJAS_LAUNCH_CHECK(ctx, name);
    return 0;
}

static int pick_mt(size_t M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8; }

// One launch over at most 8 activation rows.
static int gemv_launch_batch(ojas_b200_ctx *ctx, uint32_t type, bool preq, bool dump, GemvArgs args) {
    const int grid = ctx->sm_count < args.N ? ctx->sm_count : args.N;
    const size_t rows_max = ((size_t)args.N + grid - 1) / grid;
    const int MT = pick_mt((size_t)args.M);
    const size_t smem = gemv_smem_bytes(type, MT, (size_t)args.K, rows_max);
    if (smem > (size_t)ctx->smem_optin)
        return ojas_fail(ctx, OJAS_B200_E_LIMIT, "gemv: %zu bytes of shared memory needed, %d available", smem, ctx->smem_optin);
#define GEMV_CASE(KERNEL, NAME)                                                 \
    switch (MT) {                                                               \
    case 1: return launch_gemv(ctx, KERNEL(1), args, grid, smem, NAME);         \
    case 2: return launch_gemv(ctx, KERNEL(2), args, grid, smem, NAME);         \
    case 4: return launch_gemv(ctx, KERNEL(4), args, grid, smem, NAME);         \
    default: return launch_gemv(ctx, KERNEL(8), args, grid, smem, NAME);        \
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
    for (int mt = 8; mt >= 1; mt >>= 1)
        if (gemv_smem_bytes(type, mt, K, rows_max) <= (size_t)ctx->smem_optin) return mt;
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

static int gemv_run(ojas_b200_ctx *ctx, uint32_t type, bool preq, GemvArgs args, size_t M) {
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
