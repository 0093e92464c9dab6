// Decode GEMV over repacked GGUF weights: y[m, n] = sum_k W[n, k] * x[m, k], M <= 8.
//
// Arithmetic follows matvec_kq (crates/ojas-cpu/src/cpu_math.rs:1145-1189):
//   Q4_K, Q6_K : x is quantized to Q8_K int8 (per-256 scale) and every 32- / 16-weight
//                sub-block dot is an exact int32 dot (dot_q4k :609-635, dot_q6k :674-722);
//   Q8_0       : x stays f32 (dot_q80 :971-981).
// The kernels replace gemv_nat_{q4k,q6k,q80}{,_accum,_bias,_m}
// (crates/ojas-cuda/src/kernels/nat.rs:69-91).
//
// Shape of the kernel.  The weight is a grid of tiles of 8 rows x 256 weights (common.cuh).  A STEP is one
// super-block of 32 consecutive rows: four tiles, fetched by four bulk copies (cp.async.bulk, completion on an
// mbarrier) into a stage of the warp's own ring in shared memory.  In a step LANE = WEIGHT ROW: the 32 lanes read
// their rows' pieces from the stage without bank conflicts, every lane reads the SAME activations (one broadcast
// per load), the lane's sum never has to cross lanes, and a row's scales are decoded once per 256 weights.
// CTA b owns a contiguous range of 8-row units; its 32-row groups times the super-blocks along K are its steps.
// The warps of a team share a group round-robin along K (a team is all the warps of the CTA unless the host
// narrows it); each warp adds the steps it did for a group in registers, leaves one partial sum per row in shared
// memory, and the partial sums of a row are added in a fixed order (deterministic results).
// Everything up to the first weight copies runs before the kernel waits for its predecessor in the stream
// (programmatic dependent launch); activations and y are only touched after that wait.
#include "act_quant.cuh"

constexpr int GEMV_MAX_WARPS = 16;
constexpr int GEMV_MAX_STAGES = 4;
constexpr unsigned GEMV_WAIT_PROBES = 1u << 18;     // bounded mbarrier wait: a fraction of a second at most, then the status word is set

struct GemvArgs {
    const float *x;          // [M, K] f32 (null when activations come pre-quantized)
    const int8_t *q;         // [M, K] pre-quantized activations (PREQ kernels)
    const float *scales;     // [M, K/256]
    const int32_t *bsums;    // [M, K/32]
    const uint8_t *w;        // first tile of the weight rows of this call
    float *y;                // [M, N]
    const float *bias;       // [N] or null
    int32_t *idots;          // dump of the integer sub-block dots (DUMP kernels)
    // grouped (per-expert) launches: activation row m of the batch is source row row_index[m]
    // (null: row m); the group's row count and first position come from device memory
    const int *row_index;
    const int *grp_count;
    const int *grp_offset;
    unsigned *status;        // device-visible status word of the context
    int K, N, M, form;
    int nsb;                 // super-blocks per row
    int units_base, units_rem;   // CTA b owns units_base (+1 if b < units_rem) 8-row units
    int nst_log;             // ring stages per warp = 1 << nst_log
    int S_log;               // warps per team = 1 << S_log
    int T_log;               // teams per CTA = 1 << T_log (warps per CTA = teams * warps per team)
    int P;                   // partial sums per row and group = min(warps per team, nsb)
    int own_x;               // 1: warp w consumes exactly super-block w, so it quantizes that one for itself
    // K walked in segments (gemv_q80_kseg_kernel): a pass sees K = the segment's length, while activation rows are
    // x_stride values apart and the tiles of consecutive 8-row units w_nsb super-blocks apart (0 = K and nsb)
    int x_stride, w_nsb;
    // Q8_0 batches converted to their three int8 terms once per call (quant_q80_terms_kernel): rows in the layout stage_q80
    // keeps in shared memory, q80_act_row_bytes(x_stride ? x_stride : K) apart; null: every CTA converts x for itself
    const uint8_t *q80;
    // decode-time expert selection (the engine's moe_gu_* / moe_down_* and their _slots forms,
    // crates/ojas-cuda/src/kernels/moe.rs:75-178): the weight rows start `*sel * sel_stride` bytes (sel_stride != 0)
    // or `*sel` bytes (an offset table entry) behind w, read on the device; alpha (may be null): the result is
    // multiplied by *alpha before it is stored (the router weight of the pick).
    const uint32_t *sel;
    size_t sel_stride;
    const float *alpha;
    // fused RMSNorm (crates/ojas-cpu/src/cpu_math.rs:456-460): with norm_w given, row m of x enters as
    // (x * inv_m) * norm_w with inv_m = 1 / sqrt(mean(x_m^2) + norm_eps), formed in the prologue
    const float *norm_w;
    float norm_eps;
    // fused SwiGLU (crates/ojas-cpu/src/cpu_math.rs:486): with x2 given (and no norm_w), row m enters as silu(x) * x2
    const float *x2;
    // tensor-parallel epilogue (tp.cu): instead of y, every result goes, stamped with the step's number, to this
    // rank's place in the receive window of every rank (plain 8-byte stores through peer-mapped pointers).
    TpPush tp;
};

__device__ __forceinline__ void store_form(float *yp, float v, int form, const float *bias, int n) {
    if (form == OJAS_B200_ACCUM) v += *yp;
    else if (form == OJAS_B200_BIAS) v += __ldg(bias + n);
    *yp = v;
}

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {   // unsigned bytes x signed bytes
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_s8s8(uint32_t a, uint32_t b, int c) {   // signed bytes x signed bytes
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ int src_row(const GemvArgs &a, int m) { return a.row_index ? __ldg(a.row_index + m) : m; }

// ---------------------------------------------------------------------------- bulk copies and their barriers
__device__ __forceinline__ uint32_t gv_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gv_bar_init(uint64_t *bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gv_smem(bar)) : "memory");
}
__device__ __forceinline__ void gv_bar_expect(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(gv_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gv_bulk_load(void *dst, const void *src, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(gv_smem(dst)), "l"(src), "r"(bytes), "r"(gv_smem(bar)) : "memory");
}
__device__ __forceinline__ bool gv_bar_try(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(gv_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded: after GEMV_WAIT_PROBES failed probes the status word is set and the warp goes on (its results are then
// wrong, the kernel still ends, ojas_b200_sync reports OJAS_B200_E_DEVICE).
// `dead` stays set once a wait of this warp has run out: its later waits are single probes, so a kernel that has lost a
// copy ends quickly however many steps it has left.
__device__ __forceinline__ void gv_bar_wait(uint64_t *bar, unsigned parity, unsigned *status, bool &dead) {
    const unsigned limit = dead ? 1u : GEMV_WAIT_PROBES;
    for (unsigned i = 0; i < limit; i++)
        if (gv_bar_try(bar, parity)) return;
    if (!dead) {
        dead = true;
        atomicOr(status, 0x40u);
        __threadfence_system();
    }
}

// ---------------------------------------------------------------------------- activations in shared memory
// K-quants: per activation row, nsb super-blocks of { 256 int8 values in natural order }, then per super-block the
// block sums as bytes (so that sum_j m_j * bsum_j and sum_j sc_j * bsum_j are dp4a's): a sum s is kept as
// lo = s & 63 (0..63) and hi = s >> 6 (a signed byte), s = lo + 64 * hi.  Q4_K: eight sums per 32 values -> 16 bytes
// (lo[8], hi[8]); Q6_K: sixteen sums per 16 values -> 32 bytes (lo[16], hi[16]).  Then the f32 scales.
template <int TYPE> struct ActLayout {
    static constexpr int BS_BYTES = TYPE == OJAS_B200_Q6_K ? 32 : 16;       // (Q5_K shares Q4_K's sub-blocks of 32)
    // bytes of one activation row, a multiple of 16 so that every row's values stay 16-byte aligned
    __host__ __device__ static size_t row_bytes(int nsb) { return ((size_t)nsb * (256 + BS_BYTES + 4) + 15) & ~(size_t)15; }
};

// One warp quantizes super-block `sb` of one row into shared memory: bit-exact quant_q8k
// (crates/ojas-cpu/src/cpu_math.rs:545-563).  lane l owns values 8l .. 8l+7.
template <int TYPE>
__device__ __forceinline__ void stage_quant_vals(const Q8kLane &ql, int sb, int lane, uint8_t *xq, uint8_t *bs, float *sx);

template <int TYPE>
__device__ __forceinline__ void stage_quant_sb(const float *xrow, int sb, int lane, uint8_t *xq, uint8_t *bs, float *sx) {
    stage_quant_vals<TYPE>(quant_q8k_warp(xrow + sb * 256, lane), sb, lane, xq, bs, sx);
}

// The lane's eight values of super-block sb of a row, normalized: (x * inv) * w.
__device__ __forceinline__ void load_normed(const float *xrow, const float *nw, float inv, int sb, int lane, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(xrow + sb * 256) + lane * 2), b = __ldg(reinterpret_cast<const float4 *>(xrow + sb * 256) + lane * 2 + 1);
    const float4 g = __ldg(reinterpret_cast<const float4 *>(nw + sb * 256) + lane * 2), h = __ldg(reinterpret_cast<const float4 *>(nw + sb * 256) + lane * 2 + 1);
    v[0] = __fmul_rn(__fmul_rn(a.x, inv), g.x); v[1] = __fmul_rn(__fmul_rn(a.y, inv), g.y);
    v[2] = __fmul_rn(__fmul_rn(a.z, inv), g.z); v[3] = __fmul_rn(__fmul_rn(a.w, inv), g.w);
    v[4] = __fmul_rn(__fmul_rn(b.x, inv), h.x); v[5] = __fmul_rn(__fmul_rn(b.y, inv), h.y);
    v[6] = __fmul_rn(__fmul_rn(b.z, inv), h.z); v[7] = __fmul_rn(__fmul_rn(b.w, inv), h.w);
}

// The lane's eight values of super-block sb of silu(g) * u, the expression of silu_mul_q8k_kernel (producers.cu).
__device__ __forceinline__ void load_silu_mul(const float *grow, const float *urow, int sb, int lane, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(grow + sb * 256) + lane * 2), b = __ldg(reinterpret_cast<const float4 *>(grow + sb * 256) + lane * 2 + 1);
    const float4 g = __ldg(reinterpret_cast<const float4 *>(urow + sb * 256) + lane * 2), h = __ldg(reinterpret_cast<const float4 *>(urow + sb * 256) + lane * 2 + 1);
    const float gv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w}, uv[8] = {g.x, g.y, g.z, g.w, h.x, h.y, h.z, h.w};
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __fmul_rn(__fdiv_rn(gv[i], 1.0f + expf(-gv[i])), uv[i]);
}

// 1 / sqrt(mean(x^2) + eps) of each of the M rows, the same value in every thread: per-thread sums over a strided
// walk of the row, a butterfly per warp, then the warps' sums added in warp order (every thread adds them itself).
template <int MT>
__device__ __forceinline__ void row_inv_norms(const GemvArgs &a, int warps, float (&inv)[MT]) {
    __shared__ float norm_part[MT * GEMV_MAX_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int m = 0; m < MT; m++) {
        float s = 0.0f;
        if (m < a.M) {
            const float *xr = a.x + (size_t)m * a.K;
            for (int i = threadIdx.x * 4; i < a.K; i += blockDim.x * 4) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(xr + i));
                s = fmaf(v.x, v.x, s); s = fmaf(v.y, v.y, s); s = fmaf(v.z, v.z, s); s = fmaf(v.w, v.w, s);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) norm_part[m * GEMV_MAX_WARPS + warp] = s;
    }
    __syncthreads();
#pragma unroll
    for (int m = 0; m < MT; m++) {
        float tot = 0.0f;
        for (int j = 0; j < warps; j++) tot += norm_part[m * GEMV_MAX_WARPS + j];
        inv[m] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)a.K), a.norm_eps)));
    }
}

template <int TYPE>
__device__ __forceinline__ void stage_quant_vals(const Q8kLane &ql, int sb, int lane, uint8_t *xq, uint8_t *bs, float *sx) {
    reinterpret_cast<uint2 *>(xq + sb * 256)[lane] = ql.packed;
    int s = ql.sum8;
    s += __shfl_xor_sync(0xffffffffu, s, 1);                       // sum of 16 values (lanes 2j, 2j+1)
    if (TYPE != OJAS_B200_Q6_K) {
        s += __shfl_xor_sync(0xffffffffu, s, 2);                   // sum of 32 values (lanes 4j .. 4j+3)
        if ((lane & 3) == 0) {
            bs[sb * 16 + (lane >> 2)] = (uint8_t)(s & 63);
            bs[sb * 16 + 8 + (lane >> 2)] = (uint8_t)((s >> 6) & 0xff);
        }
    } else {
        if ((lane & 1) == 0) {
            bs[sb * 32 + (lane >> 1)] = (uint8_t)(s & 63);
            bs[sb * 32 + 16 + (lane >> 1)] = (uint8_t)((s >> 6) & 0xff);
        }
    }
    if (lane == 0) sx[sb] = ql.scale;
}

// Activations of the K-quants.  MT rows (rows >= M are zeros).  !PREQ: quantize f32 rows; PREQ: copy rows that
// ojas_b200_quant_q8k (or the expert FFN) quantized before, gathered through row_index when given.
template <int TYPE, int MT, bool PREQ, int PRO>
__device__ __forceinline__ void stage_kquant(const GemvArgs &a, uint8_t *act, int nsb, int warps) {
    using L = ActLayout<TYPE>;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t rb = L::row_bytes(nsb);
    if (!PREQ) {
        float inv[MT];
        if (PRO == 1) row_inv_norms<MT>(a, warps, inv);
        auto quant_sb = [&](int m, int sb) {
            uint8_t *xq = act + m * rb, *bs = xq + nsb * 256;
            float *sx = reinterpret_cast<float *>(bs + nsb * L::BS_BYTES);
            if (PRO == 1) {
                float v[8];
                load_normed(a.x + (size_t)m * a.K, a.norm_w, inv[m], sb, lane, v);
                stage_quant_vals<TYPE>(quant_q8k_values(v), sb, lane, xq, bs, sx);
            } else if (PRO == 2) {
                float v[8];
                load_silu_mul(a.x + (size_t)m * a.K, a.x2 + (size_t)m * a.K, sb, lane, v);
                stage_quant_vals<TYPE>(quant_q8k_values(v), sb, lane, xq, bs, sx);
            } else {
                stage_quant_sb<TYPE>(a.x + (size_t)m * a.K, sb, lane, xq, bs, sx);
            }
        };
        if (a.own_x) {
#pragma unroll
            for (int m = 0; m < MT; m++)
                if (m < a.M) quant_sb(m, warp);
            __syncwarp();
            return;
        }
#pragma unroll
        for (int m = 0; m < MT; m++)
            if (m < a.M)
                for (int sb = warp; sb < nsb; sb += warps) quant_sb(m, sb);
    } else {
        const int units = nsb * 16;                               // 16-byte units per row
        for (int m = 0; m < a.M; m++) {
            uint8_t *xq = act + m * rb, *bs = xq + nsb * 256;
            float *sx = reinterpret_cast<float *>(bs + nsb * L::BS_BYTES);
            const int srow = src_row(a, m);
            const uint4 *qsrc = reinterpret_cast<const uint4 *>(a.q + (size_t)srow * a.K);
            for (int un = threadIdx.x; un < units; un += blockDim.x) {
                const uint4 v = __ldg(qsrc + un);
                reinterpret_cast<uint4 *>(xq)[un] = v;
                if (TYPE == OJAS_B200_Q6_K) {                     // the sum of this unit's sixteen values
                    int t = __dp4a((int)v.x, 0x01010101, 0);
                    t = __dp4a((int)v.y, 0x01010101, t);
                    t = __dp4a((int)v.z, 0x01010101, t);
                    t = __dp4a((int)v.w, 0x01010101, t);
                    const int sb = un >> 4, j = un & 15;
                    bs[sb * 32 + j] = (uint8_t)(t & 63);
                    bs[sb * 32 + 16 + j] = (uint8_t)((t >> 6) & 0xff);
                }
            }
            for (int sb = threadIdx.x; sb < nsb; sb += blockDim.x) sx[sb] = __ldg(a.scales + (size_t)srow * nsb + sb);
            if (TYPE != OJAS_B200_Q6_K) {
                for (int i = threadIdx.x; i < nsb * 8; i += blockDim.x) {
                    const int t = __ldg(a.bsums + (size_t)srow * nsb * 8 + i);
                    bs[(i >> 3) * 16 + (i & 7)] = (uint8_t)(t & 63);
                    bs[(i >> 3) * 16 + 8 + (i & 7)] = (uint8_t)((t >> 6) & 0xff);
                }
            }
        }
    }
    // rows past M: zeros (their sums are never stored, but the loads must be defined)
    for (int idx = threadIdx.x; idx < (MT - a.M) * (int)(rb / 4); idx += blockDim.x)
        reinterpret_cast<uint32_t *>(act + a.M * rb)[idx] = 0u;
    __syncthreads();
}

// Q8_0 keeps f32 activations on the CPU (dot_q80, crates/ojas-cpu/src/cpu_math.rs:971-981).  Here a value enters as
// three int8 terms per block of 32: x = s * (q1 + q2 / 254 + q3 / 254^2) with s = max|x| / 127 of the block,
// q1 = round(x / s), q2 = round(254 * remainder), q3 = round(254 * remainder of that): the representation error is
// below s * 0.5 / 254^2, i.e. 6e-8 of the block's largest value -- fp32 level -- and the dot of a block becomes three
// exact integer dots (dp4a) instead of 32 conversions and 32 fp32 multiply-adds.
// Per activation row in shared memory: q1 [K], q2 [K], q3 [K] int8, then s [K / 32] f32.
// (16 bytes of padding: eight rows then start in eight different 16-byte bank groups, which the tensor-core form of
// the batch reads at once)
__host__ __device__ inline size_t q80_act_row_bytes(size_t K) { return 3 * K + K / 8 + 16; }

// One warp converts super-block `sb` of a row (this lane's eight values v) into the three int8 planes and the eight
// block scales of `row` (planes K bytes apart, scales behind them).
__device__ __forceinline__ void q80_terms_sb(const float (&v)[8], int lane, uint8_t *row, size_t K, int sb) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));      // a block of 32 = four lanes
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float s = __fdiv_rn(amax, 127.0f), is = amax > 0.0f ? __fdiv_rn(1.0f, s) : 0.0f;
    uint32_t w1[2] = {0u, 0u}, w2[2] = {0u, 0u}, w3[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float t = __fmul_rn(v[i], is);
        const float q1 = fminf(fmaxf(rintf(t), -127.0f), 127.0f);
        const float t2 = __fmul_rn(__fsub_rn(t, q1), 254.0f);
        const float q2 = fminf(fmaxf(rintf(t2), -127.0f), 127.0f);
        const float q3 = fminf(fmaxf(rintf(__fmul_rn(__fsub_rn(t2, q2), 254.0f)), -127.0f), 127.0f);
        w1[i >> 2] |= ((uint32_t)(int)q1 & 0xffu) << (8 * (i & 3));
        w2[i >> 2] |= ((uint32_t)(int)q2 & 0xffu) << (8 * (i & 3));
        w3[i >> 2] |= ((uint32_t)(int)q3 & 0xffu) << (8 * (i & 3));
    }
    const size_t at = (size_t)sb * 256 + lane * 8;
    *reinterpret_cast<uint2 *>(row + at) = make_uint2(w1[0], w1[1]);
    *reinterpret_cast<uint2 *>(row + K + at) = make_uint2(w2[0], w2[1]);
    *reinterpret_cast<uint2 *>(row + 2 * K + at) = make_uint2(w3[0], w3[1]);
    if ((lane & 3) == 0) reinterpret_cast<float *>(row + 3 * K)[sb * 8 + (lane >> 2)] = s;
}

// The conversion once per call, for batches whose every CTA would otherwise repeat it: one warp per (row, super-block),
// rows q80_act_row_bytes(K) apart.
__global__ void __launch_bounds__(256) quant_q80_terms_kernel(const float *x, uint8_t *out, int K, long long n_sb) {
    const int lane = threadIdx.x & 31;
    const long long task = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    grid_launch_dependents();
    if (task >= n_sb) return;
    const int nsb = K >> 8;
    const long long m = task / nsb;
    const int sb = (int)(task - m * nsb);
    const float *seg = x + (size_t)m * K + (size_t)sb * 256;
    const float4 p = __ldg(reinterpret_cast<const float4 *>(seg) + lane * 2), q = __ldg(reinterpret_cast<const float4 *>(seg) + lane * 2 + 1);
    const float v[8] = {p.x, p.y, p.z, p.w, q.x, q.y, q.z, q.w};
    q80_terms_sb(v, lane, out + (size_t)m * q80_act_row_bytes((size_t)K), (size_t)K, sb);
}

template <int MT, int PRO>
__device__ __forceinline__ void stage_q80(const GemvArgs &a, uint8_t *act, int nsb, int warps, int sb0 = 0) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t rb = q80_act_row_bytes((size_t)a.K);
    float inv[MT];
    if (PRO == 1) row_inv_norms<MT>(a, warps, inv);
#pragma unroll
    for (int m = 0; m < MT; m++) {
        uint8_t *row = act + m * rb;
        if (PRO == 0 && m < a.M && a.q80) {
            // converted once per call: copy this pass's segment of the three planes and its block scales
            const size_t Kt = a.x_stride ? (size_t)a.x_stride : (size_t)a.K;
            const uint8_t *src = a.q80 + (size_t)m * q80_act_row_bytes(Kt);
            const int pu = a.K >> 4;                              // 16-byte units per plane of the segment
            for (int u = threadIdx.x; u < 3 * pu; u += blockDim.x) {
                const int t = u / pu, i = u - t * pu;
                reinterpret_cast<uint4 *>(row + (size_t)t * a.K)[i] = __ldg(reinterpret_cast<const uint4 *>(src + (size_t)t * Kt + (size_t)sb0 * 256) + i);
            }
            for (int u = threadIdx.x; u < nsb * 2; u += blockDim.x)   // eight f32 scales per super-block = two units
                reinterpret_cast<uint4 *>(row + 3 * (size_t)a.K)[u] = __ldg(reinterpret_cast<const uint4 *>(src + 3 * Kt + (size_t)sb0 * 32) + u);
        } else if (m < a.M) {
            const float *xr = a.x + (size_t)src_row(a, m) * (PRO == 0 && a.x_stride ? a.x_stride : a.K) + (size_t)sb0 * 256;
            for (int sb = warp; sb < nsb; sb += warps) {
                float v[8];
                if (PRO == 1) {
                    load_normed(xr, a.norm_w, inv[m], sb, lane, v);
                } else if (PRO == 2) {
                    load_silu_mul(xr, a.x2 + (size_t)m * a.K, sb, lane, v);
                } else {
                    const float4 p = __ldg(reinterpret_cast<const float4 *>(xr + sb * 256) + lane * 2), q = __ldg(reinterpret_cast<const float4 *>(xr + sb * 256) + lane * 2 + 1);
                    v[0] = p.x; v[1] = p.y; v[2] = p.z; v[3] = p.w; v[4] = q.x; v[5] = q.y; v[6] = q.z; v[7] = q.w;
                }
                q80_terms_sb(v, lane, row, (size_t)a.K, sb);
            }
        } else {
            for (size_t i = threadIdx.x; i < rb / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(row)[i] = 0u;
        }
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------- one step of one lane (= one row)
// `wl` = this lane's first piece in the stage (tile of its unit + 16 * row-in-unit); piece p is at wl + 128 p.
// `act` = the activations, `sb` = the super-block of the step.

// Q4_K (dot_q4k, crates/ojas-cpu/src/cpu_math.rs:609-635): eight exact int32 sub-block dots, integer
// sum_j s_j * idot_j and sum_j m_j * bsum_j, then sx * (d * isum - dmin * msum).
// FIVE: Q5_K (dot_q5k, :637-671): the same with a fifth bit per weight, bit j of qh[l] for weight l of sub-block j.
template <int MT, bool DUMP, bool FIVE = false>
__device__ __forceinline__ void step_q4k(const uint8_t *wl, const uint8_t *act, int nsb, int sb, float (&acc)[MT], int32_t *dump) {
    using L = ActLayout<OJAS_B200_Q4_K>;
    const size_t rb = L::row_bytes(nsb);
    const uint4 H = *reinterpret_cast<const uint4 *>(wl + 8 * 128);
    uint32_t qh[2][4] = {{0u, 0u, 0u, 0u}, {0u, 0u, 0u, 0u}};
    if (FIVE) {
        const uint4 Q0 = *reinterpret_cast<const uint4 *>(wl + 9 * 128), Q1 = *reinterpret_cast<const uint4 *>(wl + 10 * 128);
        qh[0][0] = Q0.x; qh[0][1] = Q0.y; qh[0][2] = Q0.z; qh[0][3] = Q0.w;
        qh[1][0] = Q1.x; qh[1][1] = Q1.y; qh[1][2] = Q1.z; qh[1][3] = Q1.w;
    }
    // the sixteen 6-bit scales / mins as bytes (get_scale_min_k4, crates/ojas-formats/src/gguf.rs:1132-1140)
    const uint32_t s_lo = H.y & 0x3f3f3f3fu, m_lo = H.z & 0x3f3f3f3fu;
    const uint32_t s_hi = (H.w & 0x0f0f0f0fu) | ((H.y >> 2) & 0x30303030u);
    const uint32_t m_hi = ((H.w >> 4) & 0x0f0f0f0fu) | ((H.z >> 2) & 0x30303030u);
    int isum[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) isum[m] = 0;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        int pA[MT], pB[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) pA[m] = pB[m] = 0;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint4 W = *reinterpret_cast<const uint4 *>(wl + (2 * c + h) * 128);
            uint32_t lo[4] = {W.x & 0x0f0f0f0fu, W.y & 0x0f0f0f0fu, W.z & 0x0f0f0f0fu, W.w & 0x0f0f0f0fu};
            uint32_t hi[4] = {W.x & 0xf0f0f0f0u, W.y & 0xf0f0f0f0u, W.z & 0xf0f0f0f0u, W.w & 0xf0f0f0f0u};
            if (FIVE) {                                   // five-bit values 0..31; the high nibbles come down (no room for x16)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    lo[i] |= ((qh[h][i] >> (2 * c)) & 0x01010101u) << 4;
                    hi[i] = (hi[i] >> 4) | (((qh[h][i] >> (2 * c + 1)) & 0x01010101u) << 4);
                }
            }
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const uint4 *xs = reinterpret_cast<const uint4 *>(act + m * rb + sb * 256);
                const uint4 Xa = xs[4 * c + h], Xb = xs[4 * c + 2 + h];
                pA[m] = dp4a_u8s8(lo[0], Xa.x, pA[m]); pA[m] = dp4a_u8s8(lo[1], Xa.y, pA[m]);
                pA[m] = dp4a_u8s8(lo[2], Xa.z, pA[m]); pA[m] = dp4a_u8s8(lo[3], Xa.w, pA[m]);
                pB[m] = dp4a_u8s8(hi[0], Xb.x, pB[m]); pB[m] = dp4a_u8s8(hi[1], Xb.y, pB[m]);
                pB[m] = dp4a_u8s8(hi[2], Xb.z, pB[m]); pB[m] = dp4a_u8s8(hi[3], Xb.w, pB[m]);
            }
        }
        const uint32_t sw = (c < 2) ? s_lo : s_hi;
        const int sA = (int)__byte_perm(sw, 0, 0x4440 + 2 * (c & 1)), sB = (int)__byte_perm(sw, 0, 0x4441 + 2 * (c & 1));
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const int b = FIVE ? pB[m] : pB[m] >> 4;   // (Q4_K: the high nibbles were left in place: every product carried x16)
            if (DUMP && m == 0) { dump[2 * c] = pA[0]; dump[2 * c + 1] = b; }
            isum[m] += sA * pA[m] + sB * b;
        }
    }
    const float d = f16_bits_to_f32(H.x), dmin = f16_bits_to_f32(H.x >> 16);
#pragma unroll
    for (int m = 0; m < MT; m++) {
        const uint8_t *bsb = act + m * rb + nsb * 256;
        const uint4 bs = *reinterpret_cast<const uint4 *>(bsb + sb * 16);
        int ml = dp4a_u8s8(m_lo, bs.x, 0);
        ml = dp4a_u8s8(m_hi, bs.y, ml);
        int mh = dp4a_u8s8(m_lo, bs.z, 0);
        mh = dp4a_u8s8(m_hi, bs.w, mh);
        const int msum = ml + 64 * mh;
        const float sx = reinterpret_cast<const float *>(bsb + nsb * 16)[sb];
        acc[m] += sx * (d * (float)isum[m] - dmin * (float)msum);
    }
}

// Q6_K (dot_q6k, crates/ojas-cpu/src/cpu_math.rs:674-722): sixteen exact int32 dots of 16 weights on the
// six-bit values 0..63, the format's -32 applied as -32 * sum_j sc_j * (sum of sub-block j's activations).
template <int MT, bool DUMP>
__device__ __forceinline__ void step_q6k(const uint8_t *wl, int r, const uint8_t *act, int nsb, int sb, float (&acc)[MT], int32_t *dump) {
    using L = ActLayout<OJAS_B200_Q6_K>;
    const size_t rb = L::row_bytes(nsb);
    const uint4 SC = *reinterpret_cast<const uint4 *>(wl + 12 * 128);
    const uint32_t scw[4] = {SC.x, SC.y, SC.z, SC.w};
    const float d = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(wl - r * 16 + 13 * 128 + r * 2));
    int isum[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) isum[m] = 0;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint4 Hh = *reinterpret_cast<const uint4 *>(wl + (8 + c) * 128);
        const uint32_t hw[4] = {Hh.x, Hh.y, Hh.z, Hh.w};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint4 Lo = *reinterpret_cast<const uint4 *>(wl + (h * 4 + c) * 128);
            const uint32_t lw[4] = {Lo.x, Lo.y, Lo.z, Lo.w};
            uint32_t v0[4], v1[4];        // sub-blocks 4c + h (low nibbles, field h) and 4c + 2 + h (high nibbles, field 2 + h)
#pragma unroll
            for (int k = 0; k < 4; k++) {
                v0[k] = (lw[k] & 0x0f0f0f0fu) | ((hw[k] << (4 - 2 * h)) & 0x30303030u);
                v1[k] = ((lw[k] >> 4) & 0x0f0f0f0fu) | ((hw[k] >> (2 * h)) & 0x30303030u);
            }
            const int j0 = 4 * c + h, j1 = 4 * c + 2 + h;
            const int s0 = (int)(signed char)(scw[j0 >> 2] >> (8 * (j0 & 3))), s1 = (int)(signed char)(scw[j1 >> 2] >> (8 * (j1 & 3)));
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const uint4 *xs = reinterpret_cast<const uint4 *>(act + m * rb + sb * 256);
                const uint4 X0 = xs[j0], X1 = xs[j1];
                int i0 = dp4a_u8s8(v0[0], X0.x, 0);
                i0 = dp4a_u8s8(v0[1], X0.y, i0); i0 = dp4a_u8s8(v0[2], X0.z, i0); i0 = dp4a_u8s8(v0[3], X0.w, i0);
                int i1 = dp4a_u8s8(v1[0], X1.x, 0);
                i1 = dp4a_u8s8(v1[1], X1.y, i1); i1 = dp4a_u8s8(v1[2], X1.z, i1); i1 = dp4a_u8s8(v1[3], X1.w, i1);
                if (DUMP && m == 0) { dump[j0] = i0; dump[j1] = i1; }
                isum[m] += s0 * i0 + s1 * i1;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
        const uint8_t *bsb = act + m * rb + nsb * 256;
        const uint4 lo = *reinterpret_cast<const uint4 *>(bsb + sb * 32), hi = *reinterpret_cast<const uint4 *>(bsb + sb * 32 + 16);
        int ml = dp4a_s8s8(scw[0], lo.x, 0);
        ml = dp4a_s8s8(scw[1], lo.y, ml); ml = dp4a_s8s8(scw[2], lo.z, ml); ml = dp4a_s8s8(scw[3], lo.w, ml);
        int mh = dp4a_s8s8(scw[0], hi.x, 0);
        mh = dp4a_s8s8(scw[1], hi.y, mh); mh = dp4a_s8s8(scw[2], hi.z, mh); mh = dp4a_s8s8(scw[3], hi.w, mh);
        const int total = isum[m] - 32 * (ml + 64 * mh);       // sum_j sc_j * (idot_j - 32 * xsum_j), exact
        const float sx = reinterpret_cast<const float *>(bsb + nsb * 32)[sb];
        acc[m] += (sx * d) * (float)total;
    }
}

// Q8_0 (dot_q80, crates/ojas-cpu/src/cpu_math.rs:971-981): per block of 32 weights three exact integer dots against the
// activation's three int8 terms, then d * s * (D1 + D2 / 254 + D3 / 254^2).
template <int MT>
__device__ __forceinline__ void step_q80(const uint8_t *wl, const uint8_t *act, int K, int sb, float (&acc)[MT]) {
    const uint4 D = *reinterpret_cast<const uint4 *>(wl + 16 * 128);
    const uint32_t dw[4] = {D.x, D.y, D.z, D.w};
    const size_t rb = q80_act_row_bytes((size_t)K);
    constexpr float C1 = 1.0f / 254.0f;
#pragma unroll
    for (int b = 0; b < 8; b++) {
        const uint4 W0 = *reinterpret_cast<const uint4 *>(wl + (2 * b) * 128), W1 = *reinterpret_cast<const uint4 *>(wl + (2 * b + 1) * 128);
        const int wv[8] = {(int)W0.x, (int)W0.y, (int)W0.z, (int)W0.w, (int)W1.x, (int)W1.y, (int)W1.z, (int)W1.w};
        const float d = f16_bits_to_f32(dw[b >> 1] >> (16 * (b & 1)));
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const uint8_t *row = act + m * rb + (size_t)sb * 256 + b * 32;
            int dot[3];
#pragma unroll
            for (int t = 0; t < 3; t++) {
                const uint4 x0 = *reinterpret_cast<const uint4 *>(row + (size_t)t * K), x1 = *reinterpret_cast<const uint4 *>(row + (size_t)t * K + 16);
                int v = __dp4a(wv[0], (int)x0.x, 0);
                v = __dp4a(wv[1], (int)x0.y, v); v = __dp4a(wv[2], (int)x0.z, v); v = __dp4a(wv[3], (int)x0.w, v);
                v = __dp4a(wv[4], (int)x1.x, v); v = __dp4a(wv[5], (int)x1.y, v); v = __dp4a(wv[6], (int)x1.z, v); v = __dp4a(wv[7], (int)x1.w, v);
                dot[t] = v;
            }
            const float s = reinterpret_cast<const float *>(act + m * rb + 3 * (size_t)K)[sb * 8 + b];
            const float f = fmaf(fmaf((float)dot[2], C1, (float)dot[1]), C1, (float)dot[0]);
            acc[m] = fmaf(__fmul_rn(d, s), f, acc[m]);
        }
    }
}

// IQ4_XS (dot_iq4xs, crates/ojas-cpu/src/cpu_math.rs:943-967): the CPU takes f32 activations, so they enter as three int8
// terms like Q8_0's; a weight is a 4-bit index into the sixteen int8 codebook values.  Four index bytes (eight weights)
// are looked up with byte permutes: the two halves of the codebook are selected by the low three bits of every nibble
// (__byte_perm ignores the fourth), a third permute picks between them by that fourth bit, and two more separate the
// low nibbles (weights j .. j+3 of the group) from the high ones (weights j+16 .. j+19).  Per group of 32: three exact
// integer dots, then d * (ls - 32) * s * (D1 + D2 / 254 + D3 / 254^2).

// NL: IQ4_NL (dot_iq4nl, :993-1010): the same codebook in plain blocks of 32, each with its own f16 scale and no sub-scale.
template <int MT, bool NL>
__device__ __forceinline__ void step_iq4xs(const uint8_t *wl, int r, const uint8_t *act, int K, int sb, float (&acc)[MT]) {
    const uint2 H = NL ? make_uint2(0u, 0u) : *reinterpret_cast<const uint2 *>(wl - r * 16 + 8 * 128 + r * 8);   // d, scales_h | scales_l
    const uint4 D = NL ? *reinterpret_cast<const uint4 *>(wl + 8 * 128) : make_uint4(0u, 0u, 0u, 0u);            // eight block scales
    const uint32_t dw[4] = {D.x, D.y, D.z, D.w};
    const float d = f16_bits_to_f32(H.x);
    const uint32_t sh = H.x >> 16, sl = H.y;
    const size_t rb = q80_act_row_bytes((size_t)K);
    constexpr float C1 = 1.0f / 254.0f;
#pragma unroll
    for (int g = 0; g < 8; g++) {
        const uint4 Q = *reinterpret_cast<const uint4 *>(wl + g * 128);
        uint32_t wv[8];                                          // weights 0..15 of the group, then 16..31
        iq4_lookup8(Q.x, wv[0], wv[4]);
        iq4_lookup8(Q.y, wv[1], wv[5]);
        iq4_lookup8(Q.z, wv[2], wv[6]);
        iq4_lookup8(Q.w, wv[3], wv[7]);
        const int ls = (int)(((sl >> (4 * g)) & 0xFu) | (((sh >> (2 * g)) & 3u) << 4)) - 32;
        const float dl = NL ? f16_bits_to_f32(dw[g >> 1] >> (16 * (g & 1))) : __fmul_rn(d, (float)ls);
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const uint8_t *row = act + m * rb + (size_t)sb * 256 + g * 32;
            int dot[3];
#pragma unroll
            for (int t = 0; t < 3; t++) {
                const uint4 x0 = *reinterpret_cast<const uint4 *>(row + (size_t)t * K), x1 = *reinterpret_cast<const uint4 *>(row + (size_t)t * K + 16);
                int v = __dp4a((int)wv[0], (int)x0.x, 0);
                v = __dp4a((int)wv[1], (int)x0.y, v); v = __dp4a((int)wv[2], (int)x0.z, v); v = __dp4a((int)wv[3], (int)x0.w, v);
                v = __dp4a((int)wv[4], (int)x1.x, v); v = __dp4a((int)wv[5], (int)x1.y, v); v = __dp4a((int)wv[6], (int)x1.z, v); v = __dp4a((int)wv[7], (int)x1.w, v);
                dot[t] = v;
            }
            const float s = reinterpret_cast<const float *>(act + m * rb + 3 * (size_t)K)[sb * 8 + g];
            const float f = fmaf(fmaf((float)dot[2], C1, (float)dot[1]), C1, (float)dot[0]);
            acc[m] = fmaf(__fmul_rn(dl, s), f, acc[m]);
        }
    }
}

// Q8_0, eight activation rows: the same three integer dots per block on the tensor cores.  One warp step = 32 weight
// rows = two 16-row MMA tiles; per block of 32 weights A = 16 rows x 32 int8 (rows g, g + 8 = row g of two 8-row
// units), B = 8 activation rows x 32 int8 of one term: mma.sync.m16n8k32.s8.s8, exact int32.  acc[4 t + i] belongs to
// weight row 16 t + g + 8 (i / 2) of the step and activation row 2 q + (i % 2)  (g = lane / 4, q = lane % 4).
__device__ __forceinline__ void mma_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void step_q80_mma(const uint8_t *stage, const uint8_t *act, int K, int sb, int lane, float (&acc)[8]) {
    constexpr int TB = tile_bytes(OJAS_B200_Q8_0);
    const int g8 = lane >> 2, q4 = lane & 3;
    const size_t rb = q80_act_row_bytes((size_t)K);
    constexpr float C1 = 1.0f / 254.0f;
    const uint8_t *xb = act + g8 * rb + (size_t)sb * 256 + 4 * q4;                 // B fragments: activation row g8
    const float *s0p = reinterpret_cast<const float *>(act + (2 * q4) * rb + 3 * (size_t)K) + sb * 8;
    const float *s1p = reinterpret_cast<const float *>(act + (2 * q4 + 1) * rb + 3 * (size_t)K) + sb * 8;
#pragma unroll
    for (int t = 0; t < 2; t++) {
        const uint8_t *ra = stage + (2 * t) * TB + g8 * 16, *rbw = ra + TB;          // row g8 of the tile's two units
        const uint4 DA = *reinterpret_cast<const uint4 *>(ra + 16 * 128), DB = *reinterpret_cast<const uint4 *>(rbw + 16 * 128);
        const uint32_t da[4] = {DA.x, DA.y, DA.z, DA.w}, db[4] = {DB.x, DB.y, DB.z, DB.w};
#pragma unroll
        for (int b = 0; b < 8; b++) {
            const uint32_t a0 = *reinterpret_cast<const uint32_t *>(ra + (2 * b) * 128 + 4 * q4), a2 = *reinterpret_cast<const uint32_t *>(ra + (2 * b + 1) * 128 + 4 * q4);
            const uint32_t a1 = *reinterpret_cast<const uint32_t *>(rbw + (2 * b) * 128 + 4 * q4), a3 = *reinterpret_cast<const uint32_t *>(rbw + (2 * b + 1) * 128 + 4 * q4);
            float f[4];
#pragma unroll
            for (int term = 2; term >= 0; term--) {
                const uint8_t *xp = xb + (size_t)term * K + b * 32;
                int d[4] = {0, 0, 0, 0};
                mma_s8s8(d, a0, a1, a2, a3, *reinterpret_cast<const uint32_t *>(xp), *reinterpret_cast<const uint32_t *>(xp + 16));
#pragma unroll
                for (int i = 0; i < 4; i++) f[i] = term == 2 ? (float)d[i] : fmaf(f[i], C1, (float)d[i]);
            }
            const float wa = f16_bits_to_f32(da[b >> 1] >> (16 * (b & 1))), wb = f16_bits_to_f32(db[b >> 1] >> (16 * (b & 1)));
            const float s0 = s0p[b], s1 = s1p[b];
            acc[4 * t + 0] = fmaf(__fmul_rn(wa, s0), f[0], acc[4 * t + 0]);
            acc[4 * t + 1] = fmaf(__fmul_rn(wa, s1), f[1], acc[4 * t + 1]);
            acc[4 * t + 2] = fmaf(__fmul_rn(wb, s0), f[2], acc[4 * t + 2]);
            acc[4 * t + 3] = fmaf(__fmul_rn(wb, s1), f[3], acc[4 * t + 3]);
        }
    }
}

// ---------------------------------------------------------------------------- the kernel body
// `ring_uses` counts the steps this warp has put through its ring since the kernel began (the grouped kernel calls
// the body once per pass and the barriers' phases carry over).
template <int TYPE, int MT, bool PREQ, bool DUMP, int PRO = 0>
__device__ __forceinline__ void gemv_body(const GemvArgs &a, unsigned char *smem, unsigned &ring_uses, bool first_pass, int sb0 = 0) {
    constexpr int TB = tile_bytes(TYPE), STEP = 4 * TB;
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = a.nsb, P = a.P;
    const int nst = 1 << a.nst_log, S = 1 << a.S_log, T = 1 << a.T_log;   // powers of two: no divisions below
    uint8_t *ring = smem + (size_t)warp * nst * STEP;
    uint8_t *act = smem + (size_t)warps * nst * STEP;
    const size_t act_bytes = f32_act_type(TYPE) ? (size_t)MT * q80_act_row_bytes((size_t)a.K) : (size_t)MT * ActLayout<f32_act_type(TYPE) ? OJAS_B200_Q4_K : TYPE>::row_bytes(nsb);
    uint64_t *bar = reinterpret_cast<uint64_t *>(act + ((act_bytes + 15) & ~(size_t)15)) + warp * GEMV_MAX_STAGES;
    float *part = reinterpret_cast<float *>(reinterpret_cast<uint64_t *>(act + ((act_bytes + 15) & ~(size_t)15)) + GEMV_MAX_WARPS * GEMV_MAX_STAGES);

    const int b = blockIdx.x;
    const int ub = b * a.units_base + (b < a.units_rem ? b : a.units_rem);
    const int nu = a.units_base + (b < a.units_rem ? 1 : 0);
    const int ng = (nu + 3) >> 2;                                  // 32-row groups of this CTA
    const int team = warp >> a.S_log, wi = warp & (S - 1);
    const int tg = team < ng ? (ng - team + T - 1) >> a.T_log : 0; // groups of this team: team, team + T, ...
    const int n = tg * nsb;                                        // steps of this team
    const int nsteps = wi < n ? (n - wi + S - 1) >> a.S_log : 0;   // this warp takes the team's steps wi, wi + S, ...

    if (first_pass) {
        if (lane == 0) {
            for (int i = 0; i < nst; i++) gv_bar_init(bar + i);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
    }
    const uint8_t *wbase = a.w + (TYPE == OJAS_B200_Q8_0 ? (size_t)sb0 * TB : (size_t)0);   // sb0: first super-block of a K segment (Q8_0 only)
    const int wnsb = (TYPE == OJAS_B200_Q8_0 && a.w_nsb) ? a.w_nsb : nsb;   // super-blocks between the tiles of consecutive units
    if (a.sel) {                                                  // the pick comes from the router kernel before this one
        grid_dependency_wait();
        const size_t s = (size_t)__ldg(a.sel);
        wbase += a.sel_stride ? s * a.sel_stride : s;
    }
    // issue cursor (used by lane 0): k-th group of the team and super-block inside it
    int ik = 0, isb = wi;
    while (isb >= nsb) { isb -= nsb; ik++; }
    const int k_first = ik, sb_first = isb;
    unsigned issued = ring_uses;
    auto issue = [&]() {
        const int g = team + ik * T;
        const int cnt = (nu - 4 * g) < 4 ? (nu - 4 * g) : 4;
        const uint8_t *src = wbase + ((size_t)(ub + 4 * g) * wnsb + isb) * TB;
        const unsigned stg = issued & (unsigned)(nst - 1);
        gv_bar_expect(bar + stg, (unsigned)(cnt * TB));
        for (int t = 0; t < cnt; t++) gv_bulk_load(ring + stg * STEP + t * TB, src + (size_t)t * wnsb * TB, TB, bar + stg);
        issued++;
        isb += S;
        while (isb >= nsb) { isb -= nsb; ik++; }
    };
    if (lane == 0) {
        if (!first_pass) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int i = 0; i < nst && i < nsteps; i++) issue();
    }
    if (first_pass) grid_dependency_wait();                       // activations (and y for the accumulate form) come from the kernel before
    if (f32_act_type(TYPE)) stage_q80<MT, PRO>(a, act, nsb, warps, TYPE == OJAS_B200_Q8_0 ? sb0 : 0);
    else stage_kquant<f32_act_type(TYPE) ? OJAS_B200_Q4_K : TYPE, MT, PREQ, PRO>(a, act, nsb, warps);
    if (first_pass) grid_launch_dependents();
    const float alpha = a.alpha ? __ldg(a.alpha) : 1.0f;
    // tensor-parallel launches: the step in flight is the stamp and picks the half of the windows
    const unsigned tp_stamp = a.tp.step ? *reinterpret_cast<const volatile unsigned *>(a.tp.step) : 0u;
    const size_t tp_half = (size_t)(tp_stamp & 1u) * a.tp.half_pairs;

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.0f;
    int k = k_first, sb = sb_first;
    bool dead = false;
    const int unit = lane >> 3, r = lane & 7;
    const uint8_t *wl = ring + unit * TB + r * 16;
    for (int q = 0; q < nsteps; q++) {
        const unsigned use = ring_uses + (unsigned)q;
        const unsigned stg = use & (unsigned)(nst - 1);
        const int g = team + k * T;
        gv_bar_wait(bar + stg, (use >> a.nst_log) & 1u, a.status, dead);
        if (TYPE == OJAS_B200_Q8_0 && MT == 8) {
            // the whole warp, whatever the number of live units: rows past the CTA's last unit read stale bytes of the
            // ring and are never stored
            step_q80_mma(ring + stg * STEP, act, a.K, sb, lane, reinterpret_cast<float (&)[8]>(acc));
        } else if (4 * g + unit < nu) {
            const int row = (ub + 4 * g + unit) * 8 + r;
            if (TYPE == OJAS_B200_Q4_K) step_q4k<MT, DUMP>(wl + stg * STEP, act, nsb, sb, acc, DUMP ? a.idots + ((size_t)row * nsb + sb) * 8 : nullptr);
            else if (TYPE == OJAS_B200_Q5_K) step_q4k<MT, DUMP, true>(wl + stg * STEP, act, nsb, sb, acc, DUMP ? a.idots + ((size_t)row * nsb + sb) * 8 : nullptr);
            else if (TYPE == OJAS_B200_Q6_K) step_q6k<MT, DUMP>(wl + stg * STEP, r, act, nsb, sb, acc, DUMP ? a.idots + ((size_t)row * nsb + sb) * 16 : nullptr);
            else if (TYPE == OJAS_B200_IQ4_XS) step_iq4xs<MT, false>(wl + stg * STEP, r, act, a.K, sb, acc);
            else if (TYPE == OJAS_B200_IQ4_NL) step_iq4xs<MT, true>(wl + stg * STEP, r, act, a.K, sb, acc);
            else step_q80<MT>(wl + stg * STEP, act, a.K, sb, acc);
        }
        __syncwarp();                                             // every lane has read the stage
        if (q + nst < nsteps && lane == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue();
        }
        const int slot = sb & (S - 1), k_now = k;
        sb += S;
        bool flush = q + 1 == nsteps;
        while (sb >= nsb) { sb -= nsb; k++; flush = true; }
        if (flush && !DUMP) {
            if (TYPE == OJAS_B200_Q8_0 && MT == 8) {              // tensor-core form: see step_q80_mma for who holds what
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int rr = 16 * (i >> 2) + (lane >> 2) + 8 * ((i >> 1) & 1), m = 2 * (lane & 3) + (i & 1);
                    part[(((team + k_now * T) * P + slot) * MT + m) * 32 + rr] = acc[i];
                    acc[i] = 0.0f;
                }
            } else {
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    part[(((team + k_now * T) * P + slot) * MT + m) * 32 + lane] = acc[m];
                    acc[m] = 0.0f;
                }
            }
        }
    }
    ring_uses += (unsigned)nsteps;
    if (DUMP) return;
    __syncthreads();
    // combine: four threads per (group, activation row, weight row), each adds every fourth partial sum
    for (int idx = threadIdx.x; idx < ng * MT * 32 * 4; idx += blockDim.x) {
        const int item = idx >> 2, pq = idx & 3;
        const int g = item / (MT * 32), rem = item & (MT * 32 - 1);      // MT is a power of two
        const int m = rem >> 5, rr = rem & 31;
        float v = 0.0f;
        for (int p = pq; p < P; p += 4) v += part[((g * P + p) * MT + m) * 32 + rr];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v *= alpha;
        const int row = (ub + 4 * g) * 8 + rr;
        if (pq == 0 && m < a.M && 4 * g + (rr >> 3) < nu && row < a.N) {
            if (a.tp.step) {
                const uint2 pair = make_uint2(__float_as_uint(v), tp_stamp);
                for (int i = 0; i < a.tp.n; i++) a.tp.dst[i][tp_half + (size_t)m * a.N + row] = pair;     // every rank's receive window
            } else {
                store_form(a.y + (size_t)m * a.N + row, v, (TYPE == OJAS_B200_Q8_0 && sb0) ? (int)OJAS_B200_ACCUM : a.form, a.bias, row);
            }
        }
    }
}

// MINB = 2: at most 64 registers per thread, so that two CTAs of 16 warps fit on an SM: the CTA of the next GEMV in
// the stream becomes resident (and starts its weight copies) while this one still computes.  Used when the shape
// needs less than half of an SM's shared memory; larger shapes take the 128-register form.
template <int TYPE, int MT, bool PREQ, bool DUMP, int MINB>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32, MINB) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) unsigned char gemv_smem[];
    unsigned ring_uses = 0;
    gemv_body<TYPE, MT, PREQ, DUMP>(a, gemv_smem, ring_uses, true);
}

// The same with a producer in the prologue (f32 activations only): PRO = 1 RMSNorm of the rows, 2 silu(x) * x2.
template <int TYPE, int MT, int PRO>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32, 1) gemv_pro_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) unsigned char gemv_smem[];
    unsigned ring_uses = 0;
    gemv_body<TYPE, MT, false, false, PRO>(a, gemv_smem, ring_uses, true);
}

// Grouped form: the group's rows (count and first position read from device memory, so the launch is capture-safe
// whatever the routing) are processed MT at a time; passes after the first find the group's weights in L2.
template <int TYPE, int MT>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32, 1) gemv_grouped_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) unsigned char gemv_smem[];
    grid_dependency_wait();                                        // the counts come from a kernel before this one
    const int count = __ldg(a.grp_count), off = __ldg(a.grp_offset);
    unsigned ring_uses = 0;
    if (count <= 0) { grid_launch_dependents(); return; }
    for (int mb = 0; mb < count; mb += MT) {
        GemvArgs b = a;
        b.M = count - mb < MT ? count - mb : MT;
        if (a.row_index) b.row_index = a.row_index + off + mb;
        else { b.q = a.q + (size_t)(off + mb) * a.K; b.scales = a.scales + (size_t)(off + mb) * (a.K >> 8); b.bsums = a.bsums + (size_t)(off + mb) * (a.K >> 5); }
        b.y = a.y + (size_t)(off + mb) * a.N;
        gemv_body<TYPE, MT, true, false>(b, gemv_smem, ring_uses, mb == 0);
        __syncthreads();
    }
}

// Q8_0 batches whose activations (3.1 bytes per value and row) do not fit in shared memory for the whole K: the same
// body over equal K segments, every pass staging its segment of the rows and adding onto what the passes before stored
// (the same thread stores the same y element in every pass, so program order is enough).
template <int MT>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32, 1) gemv_q80_kseg_kernel(const GemvArgs a, const int seg_nsb) {
    extern __shared__ __align__(128) unsigned char gemv_smem[];
    unsigned ring_uses = 0;
    for (int sb0 = 0; sb0 < a.w_nsb; sb0 += seg_nsb) {
        gemv_body<OJAS_B200_Q8_0, MT, false, false>(a, gemv_smem, ring_uses, sb0 == 0, sb0);
        __syncthreads();
    }
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
struct GemvPlan {
    int grid, warps, nst_log, S_log, T_log, P, own_x;
    size_t smem;
};

static size_t gemv_act_bytes(uint32_t type, int MT, size_t K) {
    const size_t nsb = K / 256;
    if (f32_act_type(type)) return (size_t)MT * q80_act_row_bytes(K);
    return (size_t)MT * (type == OJAS_B200_Q6_K ? ActLayout<OJAS_B200_Q6_K>::row_bytes((int)nsb) : ActLayout<OJAS_B200_Q4_K>::row_bytes((int)nsb));
}

static int ilog2(size_t v) { int l = 0; while (((size_t)1 << (l + 1)) <= v) l++; return l; }

// Picks the grid, the warps per CTA (a power of two), the ring depth (1, 2 or 4 stages) and the team width for a
// shape: among the choices that fit in shared memory, the one that keeps the most weight bytes in flight.
// Returns false if not even the smallest configuration fits.
static bool gemv_plan(ojas_b200_ctx *ctx, uint32_t type, int MT, size_t K, size_t N, GemvPlan &p) {
    const size_t nsb = K / 256, units = tile_units(N), groups = (units + 3) / 4;
    const size_t step = 4 * (size_t)tile_bytes(type);
    const size_t limit = (size_t)ctx->smem_optin;
    p.grid = (int)(groups < (size_t)ctx->sm_count ? groups : (size_t)ctx->sm_count);
    const size_t units_max = (units + p.grid - 1) / p.grid, ng = (units_max + 3) / 4;
    const size_t steps = ng * nsb;                                 // steps of the busiest CTA
    const size_t fixed = gemv_act_bytes(type, MT, K) + GEMV_MAX_WARPS * GEMV_MAX_STAGES * 8 + 128;
    // the options are upper bounds: a forced choice that does not fit falls back to the next smaller one
    const int w_hi = ctx->gemv_warps ? ctx->gemv_warps : GEMV_MAX_WARPS;
    const int n_hi = ctx->gemv_stages ? ctx->gemv_stages : 2;
    size_t best_bytes = 0;
    bool found = false;
    for (int w = w_hi; w >= 1; w >>= 1) {
        if ((size_t)w > steps && w > 1) continue;                  // more warps than steps: idle warps
        // Teams.  One row (the latency-bound case): all warps share a group, so a CTA's loads in flight are
        // neighbours in memory.  Batches: as many teams as the CTA has groups (each team keeps its partial sums
        // apart, so fewer warps per group means less shared memory for them).
        size_t T = 1;
        if (MT > 1) while (T * 2 <= (size_t)w && T * 2 <= ng) T *= 2;
        size_t S = (size_t)w / T, P = S < nsb ? S : nsb;
        while (S > 1 && ng * P * MT * 128 > 32 * 1024) { S >>= 1; T <<= 1; P = S < nsb ? S : nsb; }
        const size_t part = ng * P * MT * 128;
        const size_t per_warp = (((ng + T - 1) / T) * nsb + S - 1) / S;        // steps of the busiest warp
        for (int n = n_hi; n >= 1; n--) {
            if (n == 3) continue;                                  // depths are powers of two
            const size_t nn = (size_t)n > per_warp ? ((size_t)1 << ilog2(per_warp)) : (size_t)n;
            const size_t bytes = (size_t)w * nn * step, smem = bytes + fixed + part;
            if (smem > limit) continue;
            if (bytes > best_bytes) {
                best_bytes = bytes;
                found = true;
                p.warps = w; p.nst_log = ilog2(nn); p.S_log = ilog2(S); p.T_log = ilog2(T);
                p.P = (int)P;
                p.own_x = (T == 1 && S == nsb) ? 1 : 0;
                p.smem = smem;
            }
        }
    }
    return found;
}

template <typename KernelT>
static int launch_gemv(ojas_b200_ctx *ctx, KernelT kernel, const GemvArgs &args, const GemvPlan &p, const char *name) {
    if (p.smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "%s: shared memory %zu: %s", name, p.smem, cudaGetErrorString(e));
        // the largest carve-out, so that two CTAs (this kernel's and the next one's in the stream) can share an SM
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.grid);
    cfg.blockDim = dim3((unsigned)p.warps * 32);
    cfg.dynamicSmemBytes = p.smem;
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
    ojas_count_launch(ctx, name);
    return 0;
}

static void gemv_fill(GemvArgs &a, ojas_b200_ctx *ctx, const GemvPlan &p) {
    const size_t units = tile_units((size_t)a.N);
    a.nsb = a.K / 256;
    a.units_base = (int)(units / p.grid);
    a.units_rem = (int)(units % p.grid);
    a.nst_log = p.nst_log; a.S_log = p.S_log; a.T_log = p.T_log; a.P = p.P; a.own_x = p.own_x;
    a.status = ctx->dev_status;
}

static int pick_mt(size_t M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8; }
// Q8_0 takes the tensor-core form (eight rows, the absent ones zero) from three rows on
static int pick_mt_for(uint32_t type, size_t M) { return type == OJAS_B200_Q8_0 && M >= 3 ? 8 : pick_mt(M); }

// One launch over at most 8 activation rows.  Returns 1 when the batch does not fit in shared memory at this
// tile height (the caller then cuts the batch).
static int gemv_launch_batch(ojas_b200_ctx *ctx, uint32_t type, bool preq, bool dump, GemvArgs args) {
    const int MT = pick_mt_for(type, (size_t)args.M);
    GemvPlan p;
    if (!gemv_plan(ctx, type, MT, (size_t)args.K, (size_t)args.N, p)) return 1;
    gemv_fill(args, ctx, p);
    if (preq || dump) args.own_x = dump ? args.own_x : 0;
    // two CTAs per SM fit.  (Not for Q8_0 and not for pre-quantized rows: their bodies do not fit in 64 registers, and a
    // spilled value costs a cold round trip to memory in every launch: measured, 12 bytes of spills added 1 us.)
    const bool two = p.smem <= (size_t)ctx->smem_optin / 2 - 1024 && !f32_act_type(type) && !(preq && type == OJAS_B200_Q4_K);
#define GEMV_CASE(T, PQ, NAME)                                                                 \
    switch (MT) {                                                                              \
    case 1: return two ? launch_gemv(ctx, gemv_kernel<T, 1, PQ, false, 2>, args, p, NAME)      \
                       : launch_gemv(ctx, gemv_kernel<T, 1, PQ, false, 1>, args, p, NAME);     \
    case 2: return launch_gemv(ctx, gemv_kernel<T, 2, PQ, false, 1>, args, p, NAME);           \
    case 4: return launch_gemv(ctx, gemv_kernel<T, 4, PQ, false, 1>, args, p, NAME);           \
    default: return launch_gemv(ctx, gemv_kernel<T, 8, PQ, false, 1>, args, p, NAME);          \
    }
    if (args.norm_w || args.x2) {
#define GEMV_PRO_CASE(T, PRO, NAME)                                                    \
    switch (MT) {                                                                      \
    case 1: return launch_gemv(ctx, gemv_pro_kernel<T, 1, PRO>, args, p, NAME);        \
    case 2: return launch_gemv(ctx, gemv_pro_kernel<T, 2, PRO>, args, p, NAME);        \
    case 4: return launch_gemv(ctx, gemv_pro_kernel<T, 4, PRO>, args, p, NAME);        \
    default: return launch_gemv(ctx, gemv_pro_kernel<T, 8, PRO>, args, p, NAME);       \
    }
        if (args.norm_w) {
            if (type == OJAS_B200_Q4_K) { GEMV_PRO_CASE(OJAS_B200_Q4_K, 1, "gemv_q4k_rmsnorm") }
            if (type == OJAS_B200_Q5_K) { GEMV_PRO_CASE(OJAS_B200_Q5_K, 1, "gemv_q5k_rmsnorm") }
            if (type == OJAS_B200_Q6_K) { GEMV_PRO_CASE(OJAS_B200_Q6_K, 1, "gemv_q6k_rmsnorm") }
            if (type == OJAS_B200_IQ4_XS) { GEMV_PRO_CASE(OJAS_B200_IQ4_XS, 1, "gemv_iq4xs_rmsnorm") }
            if (type == OJAS_B200_IQ4_NL) { GEMV_PRO_CASE(OJAS_B200_IQ4_NL, 1, "gemv_iq4nl_rmsnorm") }
            GEMV_PRO_CASE(OJAS_B200_Q8_0, 1, "gemv_q80_rmsnorm")
        }
        if (type == OJAS_B200_Q4_K) { GEMV_PRO_CASE(OJAS_B200_Q4_K, 2, "gemv_q4k_silu_mul") }
        if (type == OJAS_B200_Q5_K) { GEMV_PRO_CASE(OJAS_B200_Q5_K, 2, "gemv_q5k_silu_mul") }
        if (type == OJAS_B200_Q6_K) { GEMV_PRO_CASE(OJAS_B200_Q6_K, 2, "gemv_q6k_silu_mul") }
        if (type == OJAS_B200_IQ4_XS) { GEMV_PRO_CASE(OJAS_B200_IQ4_XS, 2, "gemv_iq4xs_silu_mul") }
        if (type == OJAS_B200_IQ4_NL) { GEMV_PRO_CASE(OJAS_B200_IQ4_NL, 2, "gemv_iq4nl_silu_mul") }
        GEMV_PRO_CASE(OJAS_B200_Q8_0, 2, "gemv_q80_silu_mul")
#undef GEMV_PRO_CASE
    }
    if (type == OJAS_B200_Q4_K) {
        if (dump) return launch_gemv(ctx, gemv_kernel<OJAS_B200_Q4_K, 1, false, true, 1>, args, p, "gemv_q4k_idots");
        if (preq) { GEMV_CASE(OJAS_B200_Q4_K, true, "gemv_q4k_q8k") }
        GEMV_CASE(OJAS_B200_Q4_K, false, "gemv_q4k")
    }
    if (type == OJAS_B200_Q5_K) {
        if (dump) return launch_gemv(ctx, gemv_kernel<OJAS_B200_Q5_K, 1, false, true, 1>, args, p, "gemv_q5k_idots");
        if (preq) { GEMV_CASE(OJAS_B200_Q5_K, true, "gemv_q5k_q8k") }
        GEMV_CASE(OJAS_B200_Q5_K, false, "gemv_q5k")
    }
    if (type == OJAS_B200_Q6_K) {
        if (dump) return launch_gemv(ctx, gemv_kernel<OJAS_B200_Q6_K, 1, false, true, 1>, args, p, "gemv_q6k_idots");
        if (preq) { GEMV_CASE(OJAS_B200_Q6_K, true, "gemv_q6k_q8k") }
        GEMV_CASE(OJAS_B200_Q6_K, false, "gemv_q6k")
    }
    if (type == OJAS_B200_IQ4_XS) { GEMV_CASE(OJAS_B200_IQ4_XS, false, "gemv_iq4xs") }
    if (type == OJAS_B200_IQ4_NL) { GEMV_CASE(OJAS_B200_IQ4_NL, false, "gemv_iq4nl") }
    GEMV_CASE(OJAS_B200_Q8_0, false, "gemv_q80")
#undef GEMV_CASE
}

// ---- the tensor-core batch kernel (gemv_mma.cuh): plan and launch
static bool batch_plan(ojas_b200_ctx *ctx, uint32_t type, int NT, size_t K, size_t N, GemvPlan &p) {
    const size_t nsb = K / 256, units = tile_units(N), groups = (units + 3) / 4;
    const size_t step = 4 * (size_t)tile_bytes(type), limit = (size_t)ctx->smem_optin;
    p.grid = (int)(groups < (size_t)ctx->sm_count ? groups : (size_t)ctx->sm_count);
    const size_t units_max = (units + p.grid - 1) / p.grid, ng = (units_max + 3) / 4;
    const size_t fixed = ((batch_act_bytes(type, NT, K) + 15) & ~(size_t)15) + GEMV_MAX_WARPS * GEMV_MAX_STAGES * 8 + 128;
    const int w_hi = ctx->gemv_warps ? ctx->gemv_warps : GEMV_MAX_WARPS, n_hi = ctx->gemv_stages ? ctx->gemv_stages : 2;
    size_t best_bytes = 0;
    bool found = false;
    for (int w = w_hi; w >= 1; w >>= 1) {
        if ((size_t)w > ng * nsb && w > 1) continue;
        size_t T = 1;
        while (T * 2 <= (size_t)w && T * 2 <= ng) T *= 2;          // as many teams as the CTA has groups
        const size_t S = (size_t)w / T, P = S < nsb ? S : nsb;
        const size_t part = ng * P * (size_t)(NT / 8) * 1024;
        const size_t per_warp = (((ng + T - 1) / T) * nsb + S - 1) / S;
        for (int n = n_hi; n >= 1; n--) {
            if (n == 3) continue;
            const size_t nn = (size_t)n > per_warp ? ((size_t)1 << ilog2(per_warp)) : (size_t)n;
            const size_t bytes = (size_t)w * nn * step, smem = bytes + fixed + part;
            if (smem > limit) continue;
            if (bytes > best_bytes) {
                best_bytes = bytes;
                found = true;
                p.warps = w; p.nst_log = ilog2(nn); p.S_log = ilog2(S); p.T_log = ilog2(T); p.P = (int)P; p.own_x = 0; p.smem = smem;
            }
        }
    }
    return found;
}

// Launches the batch kernel over `E` expert groups (E = 1, counts = null: a plain batch of M rows).  NT (8, 16 or 32)
// is the largest pass that fits; returns 1 when nothing fits.
static int batch_launch(ojas_b200_ctx *ctx, uint32_t type, BatchArgs a, int nt_want) {
    const char *name = type == OJAS_B200_Q6_K ? "gemv_q6k_batch" : "gemv_q4k_batch";
    for (int NT = nt_want; NT >= 8; NT >>= 1) {
        GemvPlan p{};
        if (!batch_plan(ctx, type, NT, (size_t)a.K, (size_t)a.N, p)) continue;
        const size_t units = tile_units((size_t)a.N);
        a.nsb = a.K / 256;
        a.units_base = (int)(units / p.grid);
        a.units_rem = (int)(units % p.grid);
        a.nst_log = p.nst_log; a.S_log = p.S_log; a.T_log = p.T_log; a.P = p.P;
        a.status = ctx->dev_status;
        auto go = [&](auto kernel) -> int {
            if (p.smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
                if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "%s: shared memory %zu: %s", name, p.smem, cudaGetErrorString(e));
            }
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)p.grid);
            cfg.blockDim = dim3((unsigned)p.warps * 32);
            cfg.dynamicSmemBytes = p.smem;
            cfg.stream = ctx->stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = ctx->pdl ? 1 : 0;
            cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, a);
            if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "launch %s: %s", name, cudaGetErrorString(e));
            ojas_count_launch(ctx, name);
            return 0;
        };
        if (type == OJAS_B200_Q6_K) {
            if (NT == 16) return go(gemv_kq_batch_kernel<OJAS_B200_Q6_K, 2>);
            if (NT == 8) return go(gemv_kq_batch_kernel<OJAS_B200_Q6_K, 1>);
            continue;
        }
        if (NT == 32) return go(gemv_kq_batch_kernel<OJAS_B200_Q4_K, 4>);
        if (NT == 16) return go(gemv_kq_batch_kernel<OJAS_B200_Q4_K, 2>);
        return go(gemv_kq_batch_kernel<OJAS_B200_Q4_K, 1>);
    }
    return 1;
}

// The expert FFN's matmuls on the batch kernel, every expert (and both of gate / up) in one launch: each CTA owns the
// same slice of rows of every expert and walks the experts with rows.  Used for Q6_K experts (Q4_K has the experts
// kernel below).  Returns 1 when the shape does not fit.
int ojas_gemv_experts_batch(ojas_b200_ctx *ctx, uint32_t type, const uint8_t *w0, const uint8_t *w1, float *y0, float *y1, const int8_t *q,
                            const float *scales, const int32_t *bsums, const int *row_index, const int *counts, const int *offsets, size_t E,
                            size_t K, size_t N, size_t rows_hint) {
    if ((type != OJAS_B200_Q4_K && type != OJAS_B200_Q6_K) || N % OJAS_TILE_ROWS != 0) return 1;
    BatchArgs b{};
    b.w[0] = w0; b.w[1] = w1; b.y[0] = y0; b.y[1] = y1; b.nw = w1 ? 2 : 1;
    b.expert_bytes = (N / OJAS_TILE_ROWS) * (K / 256) * (size_t)tile_bytes(type);
    b.q = q; b.scales = scales; b.bsums = bsums; b.row_index = row_index; b.counts = counts; b.offsets = offsets;
    b.form = OJAS_B200_PLAIN;
    b.E = (int)E; b.M = 0; b.K = (int)K; b.N = (int)N;
    return batch_launch(ctx, type, b, rows_hint + rows_hint / 2 > 8 ? 16 : 8);
}

// The expert FFN's matmuls on the experts kernel (gemv_mma.cuh): `nw` weight tensors (gate and up share the
// activations) of E stacked experts [E * N, K], rows grouped by expert (counts / offsets on the device).  Returns 1
// when the shape does not fit (the caller falls back to one grouped launch per expert).
int ojas_gemv_experts_kq(ojas_b200_ctx *ctx, uint32_t type, const uint8_t *w0, const uint8_t *w1, float *y0, float *y1, const int8_t *q,
                         const float *scales, const int32_t *bsums, const int *row_index, const int *counts, const int *offsets, size_t E, size_t K,
                         size_t N, size_t rows_hint) {
    if (type != OJAS_B200_Q4_K && type != OJAS_B200_Q5_K && type != OJAS_B200_Q6_K) return 1;
    if (N % OJAS_TILE_ROWS != 0 || E > (size_t)EXPERT_MAX_E) return 1;       // experts must start on a tile boundary
    const char *name = type == OJAS_B200_Q6_K ? "moe_q6k_experts" : type == OJAS_B200_Q5_K ? "moe_q5k_experts" : "moe_q4k_experts";
    ExpertArgs a{};
    a.w[0] = w0; a.w[1] = w1; a.y[0] = y0; a.y[1] = y1; a.nw = w1 ? 2 : 1;
    a.expert_bytes = (N / OJAS_TILE_ROWS) * (K / 256) * (size_t)tile_bytes(type);
    a.q = q; a.scales = scales; a.bsums = bsums; a.row_index = row_index; a.counts = counts; a.offsets = offsets;
    a.E = (int)E; a.K = (int)K; a.N = (int)N; a.nsb = (int)(K / 256);
    a.status = ctx->dev_status;
    // rows per pass: enough for an expert of average load plus half again (a second pass re-reads the weights)
    const size_t want = rows_hint + rows_hint / 2;
    const int ntile = want > 24 ? 4 : want > 16 ? 3 : want > 8 ? 2 : 1;
    const int warps = ctx->gemv_warps ? ctx->gemv_warps : GEMV_MAX_WARPS;
    const size_t step = 2 * (size_t)tile_bytes(type), limit = (size_t)ctx->smem_optin;
    for (int nt = ntile; nt >= 1; nt--) {
        const size_t fixed = ((expert_act_bytes(type, 8 * nt, K) + 15) & ~(size_t)15) + GEMV_MAX_WARPS * GEMV_MAX_STAGES * 8 + 128;
        int nst = ctx->gemv_stages ? ctx->gemv_stages : GEMV_MAX_STAGES;
        while (nst >= 2 && fixed + (size_t)warps * nst * step > limit) nst--;
        if (nst < 2) continue;
        a.nst = nst;
        const size_t smem = fixed + (size_t)warps * nst * step;
        auto go = [&](auto kernel) -> int {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "%s: shared memory %zu: %s", name, smem, cudaGetErrorString(e));
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)ctx->sm_count);
            cfg.blockDim = dim3((unsigned)warps * 32);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = ctx->stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = ctx->pdl ? 1 : 0;
            e = cudaLaunchKernelEx(&cfg, kernel, a);
            if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "launch %s: %s", name, cudaGetErrorString(e));
            ojas_count_launch(ctx, name);
            return 0;
        };
        if (type == OJAS_B200_Q5_K) {
            if (nt == 4) return go(moe_kq_experts_kernel<OJAS_B200_Q5_K, 4>);
            if (nt == 3) return go(moe_kq_experts_kernel<OJAS_B200_Q5_K, 3>);
            if (nt == 2) return go(moe_kq_experts_kernel<OJAS_B200_Q5_K, 2>);
            return go(moe_kq_experts_kernel<OJAS_B200_Q5_K, 1>);
        }
        if (type == OJAS_B200_Q6_K) {
            if (nt == 4) return go(moe_kq_experts_kernel<OJAS_B200_Q6_K, 4>);
            if (nt == 3) return go(moe_kq_experts_kernel<OJAS_B200_Q6_K, 3>);
            if (nt == 2) return go(moe_kq_experts_kernel<OJAS_B200_Q6_K, 2>);
            return go(moe_kq_experts_kernel<OJAS_B200_Q6_K, 1>);
        }
        if (nt == 4) return go(moe_kq_experts_kernel<OJAS_B200_Q4_K, 4>);
        if (nt == 3) return go(moe_kq_experts_kernel<OJAS_B200_Q4_K, 3>);
        if (nt == 2) return go(moe_kq_experts_kernel<OJAS_B200_Q4_K, 2>);
        return go(moe_kq_experts_kernel<OJAS_B200_Q4_K, 1>);
    }
    return 1;
}

static int gemv_check(ojas_b200_ctx *ctx, uint32_t type, int form, const void *w, const float *y, const float *bias,
                      size_t K, size_t N, size_t M) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!type_supported(type)) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: unsupported GGUF type %u", type);
    if (!w || !y) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: null pointer");
    if (K == 0 || K % 256 != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: K=%zu must be a positive multiple of 256", K);
    if (K > (1u << 22)) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: K=%zu out of range", K);
    if (N == 0 || N > 0x7fffffffu / 64) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: N=%zu out of range", N);
    if (M == 0 || M > OJAS_B200_GEMV_MAX_M) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: M=%zu must be 1..%d", M, OJAS_B200_GEMV_MAX_M);
    if (form < OJAS_B200_PLAIN || form > OJAS_B200_BIAS) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: unknown store form %d", form);
    if (form == OJAS_B200_BIAS && !bias) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: bias form without a bias pointer");
    if (((uintptr_t)w & 127) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: weight pointer must be 128-byte aligned");
    return 0;
}

// Up to this many values a batch of f32 rows is quantized by the batch kernel itself (every CTA repeats it: a few warp
// tasks) instead of by a launch in front of it, which costs more than it saves on small matrices.
constexpr size_t GEMV_BATCH_QUANT_INSIDE = 32768;
constexpr size_t GEMV_BATCH_MIN_ROWS = 5;            // the tensor-core batch kernel takes batches from this many rows (measured: up to four the per-lane kernel is faster on every shape)

// A batch of K-quant rows from fp32 activations: every CTA of the GEMV would quantize the whole batch for
// itself (M * K / 256 warp tasks each).  From a few dozen tasks per warp on that prologue outweighs the
// matrix, so the batch is quantized once into the context's scratch and the GEMV copies the result.
static bool gemv_prequantize(ojas_b200_ctx *ctx, uint32_t type, bool preq, GemvArgs &args, size_t M) {
    if (preq || f32_act_type(type) || M < 2 || !ctx->act_scratch || args.norm_w || args.x2) return false;   // (a fused producer runs in the kernel's prologue)
    const size_t values = M * (size_t)args.K;
    if (values > OJAS_ACT_SCRATCH_VALUES) return false;
    if (values <= GEMV_BATCH_QUANT_INSIDE) return false;             // few enough for every CTA to quantize them for itself
    int8_t *q = (int8_t *)ctx->act_scratch;
    float *scales = (float *)(q + OJAS_ACT_SCRATCH_VALUES);
    int32_t *bsums = (int32_t *)(scales + OJAS_ACT_SCRATCH_VALUES / 256);
    const long long n_sb = (long long)(values / 256);
    quant_q8k_kernel<<<(unsigned)((n_sb + 7) / 8), 256, 0, ctx->stream>>>(args.x, q, scales, bsums, n_sb);
    if (cudaGetLastError() != cudaSuccess) return false;
    ojas_count_launch(ctx, "quant_q8k");
    args.x = nullptr;
    args.q = q;
    args.scales = scales;
    args.bsums = bsums;
    return true;
}

// Q8_0 rows 3..8 with a K too long for one pass: the largest equal segmentation of K (a divisor of its super-block
// count) among those that keep the most weight bytes in flight.  Returns 1 when the whole K fits (no segments
// needed) or no segmentation does.
static int gemv_q80_kseg(ojas_b200_ctx *ctx, GemvArgs args, size_t nsb) {
    GemvPlan whole;
    if (ctx->gemv_kseg == 0 && gemv_plan(ctx, OJAS_B200_Q8_0, 8, (size_t)args.K, (size_t)args.N, whole)) return 1;
    GemvPlan best{};
    size_t best_seg = 0, best_bytes = 0;
    for (size_t seg = nsb - 1; seg >= 1; seg--) {
        if (nsb % seg) continue;
        if (ctx->gemv_kseg > 0 && nsb / seg != (size_t)ctx->gemv_kseg) continue;
        GemvPlan p;
        if (!gemv_plan(ctx, OJAS_B200_Q8_0, 8, seg * 256, (size_t)args.N, p)) continue;
        const size_t bytes = (size_t)p.warps * ((size_t)1 << p.nst_log);
        if (bytes > best_bytes) { best_bytes = bytes; best_seg = seg; best = p; }
    }
    if (!best_seg) return 1;
    const int K = args.K;
    args.K = (int)(best_seg * 256);
    gemv_fill(args, ctx, best);
    args.own_x = 0;
    args.x_stride = K;
    args.w_nsb = (int)nsb;
    void (*kernel)(const GemvArgs, const int) = gemv_q80_kseg_kernel<8>;
    if (best.smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)best.smem);
        if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "gemv_q80_kseg: shared memory %zu: %s", best.smem, cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)best.grid);
    cfg.blockDim = dim3((unsigned)best.warps * 32);
    cfg.dynamicSmemBytes = best.smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    if (ctx->pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args, (int)best_seg);
    if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "launch gemv_q80_kseg: %s", cudaGetErrorString(e));
    ojas_count_launch(ctx, "gemv_q80_kseg");
    return 0;
}

static int gemv_run(ojas_b200_ctx *ctx, uint32_t type, bool preq, GemvArgs args, size_t M) {
    const size_t batch_from = ctx->gemv_mma == 1 ? GEMV_BATCH_MIN_ROWS : (size_t)ctx->gemv_mma;      // option gemv_mma: 0 never, 1 default, n: from n rows
    const bool batch_kernel = (type == OJAS_B200_Q4_K || type == OJAS_B200_Q6_K) && ctx->gemv_mma != 0 && M >= batch_from && !args.tp.step && !args.row_index;
    const bool inside = batch_kernel && !preq && args.x && !args.norm_w && !args.x2 && M * (size_t)args.K <= GEMV_BATCH_QUANT_INSIDE;
    if (!inside && gemv_prequantize(ctx, type, preq, args, M)) preq = true;
    if (batch_kernel && (preq || inside)) {                                // tensor-core batch kernel
        BatchArgs b{};
        b.w[0] = args.w; b.y[0] = args.y; b.nw = 1;
        b.x = inside ? args.x : nullptr;
        b.q = args.q; b.scales = args.scales; b.bsums = args.bsums;
        b.bias = args.bias; b.form = args.form;
        b.E = 1; b.M = (int)M; b.K = args.K; b.N = args.N;
        const int rc = batch_launch(ctx, type, b, 8);
        if (rc != 1) return rc;
    }
    const size_t nsb = (size_t)args.K / 256;
    // batches of f32 activations (Q8_0, IQ4_NL, IQ4_XS rows) too large for every CTA to convert for itself: the three int8
    // terms once, into the context's scratch
    if (f32_act_type(type) && M >= 2 && args.x && !args.tp.step && !args.norm_w && !args.x2 && !args.row_index && ctx->act_scratch &&
        M * (size_t)args.K > GEMV_BATCH_QUANT_INSIDE && M * q80_act_row_bytes((size_t)args.K) <= OJAS_ACT_SCRATCH_BYTES) {
        const long long n_sb = (long long)(M * nsb);
        quant_q80_terms_kernel<<<(unsigned)((n_sb + 7) / 8), 256, 0, ctx->stream>>>(args.x, (uint8_t *)ctx->act_scratch, args.K, n_sb);
        if (cudaGetLastError() == cudaSuccess) {
            ojas_count_launch(ctx, "quant_q80_terms");
            args.q80 = (const uint8_t *)ctx->act_scratch;
        }
    }
    if (type == OJAS_B200_Q8_0 && M >= 3 && M <= 8 && !args.tp.step && !args.norm_w && !args.x2 && !args.row_index) {
        const int rc = gemv_q80_kseg(ctx, args, nsb);
        if (rc != 1) return rc;
    }
    // the whole batch in one launch when its activations fit beside the ring, else in halves
    for (size_t cap = M; cap >= 1; cap = cap / 2) {
        GemvPlan p;
        if (!gemv_plan(ctx, type, pick_mt_for(type, cap), (size_t)args.K, (size_t)args.N, p)) {
            if (cap == 1) break;
            continue;
        }
        for (size_t m0 = 0; m0 < M; m0 += cap) {
            GemvArgs b = args;
            b.M = (int)((M - m0) < cap ? (M - m0) : cap);
            if (args.x) b.x = args.x + m0 * args.K;
            if (args.q) { b.q = args.q + m0 * args.K; b.scales = args.scales + m0 * nsb; b.bsums = args.bsums + m0 * nsb * 8; }
            b.y = args.y + m0 * args.N;
            const int rc = gemv_launch_batch(ctx, type, preq, false, b);
            if (rc) return rc == 1 ? ojas_fail(ctx, OJAS_B200_E_LIMIT, "gemv: K=%d does not fit in shared memory", args.K) : rc;
        }
        return 0;
    }
    return ojas_fail(ctx, OJAS_B200_E_LIMIT, "gemv: K=%d does not fit in shared memory", args.K);
}

// One grouped launch (see gemv_grouped_kernel): weight rows `w` [N, K], activations pre-quantized.
int ojas_gemv_grouped(ojas_b200_ctx *ctx, uint32_t type, const uint8_t *w, const int8_t *q, const float *scales,
                      const int32_t *bsums, const int *row_index, const int *grp_count, const int *grp_offset, float *y,
                      size_t K, size_t N) {
    if (type != OJAS_B200_Q4_K && type != OJAS_B200_Q6_K)
        return ojas_fail(ctx, OJAS_B200_E_UNSUPPORTED, "grouped gemv: only Q4_K and Q6_K experts are supported");
    GemvArgs a{};
    a.q = q; a.scales = scales; a.bsums = bsums; a.w = w; a.y = y;
    a.row_index = row_index; a.grp_count = grp_count; a.grp_offset = grp_offset;
    a.K = (int)K; a.N = (int)N; a.form = OJAS_B200_PLAIN;
    for (int mt = 8; mt >= 2; mt >>= 1) {
        GemvPlan p;
        if (!gemv_plan(ctx, type, mt, K, N, p)) continue;
        gemv_fill(a, ctx, p);
        a.own_x = 0;
        a.M = mt;
        if (type == OJAS_B200_Q4_K) {
            if (mt == 8) return launch_gemv(ctx, gemv_grouped_kernel<OJAS_B200_Q4_K, 8>, a, p, "gemv_q4k_grouped");
            if (mt == 4) return launch_gemv(ctx, gemv_grouped_kernel<OJAS_B200_Q4_K, 4>, a, p, "gemv_q4k_grouped");
            return launch_gemv(ctx, gemv_grouped_kernel<OJAS_B200_Q4_K, 2>, a, p, "gemv_q4k_grouped");
        }
        if (mt == 8) return launch_gemv(ctx, gemv_grouped_kernel<OJAS_B200_Q6_K, 8>, a, p, "gemv_q6k_grouped");
        if (mt == 4) return launch_gemv(ctx, gemv_grouped_kernel<OJAS_B200_Q6_K, 4>, a, p, "gemv_q6k_grouped");
        return launch_gemv(ctx, gemv_grouped_kernel<OJAS_B200_Q6_K, 2>, a, p, "gemv_q6k_grouped");
    }
    return ojas_fail(ctx, OJAS_B200_E_LIMIT, "grouped gemv: K=%zu does not fit in shared memory", K);
}

extern "C" int ojas_b200_gemv(ojas_b200_ctx *ctx, uint32_t type, int form, const float *x, const void *w, float *y,
                              const float *bias, size_t K, size_t N, size_t M) {
    int rc = gemv_check(ctx, type, form, w, y, bias, K, N, M);
    if (rc) return rc;
    if (!x) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: null activation pointer");
    if (((uintptr_t)x & 15) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: x must be 16-byte aligned");
    GemvArgs a{};
    a.x = x; a.w = (const uint8_t *)w; a.y = y; a.bias = bias;
    a.K = (int)K; a.N = (int)N; a.M = (int)M; a.form = form;
    return gemv_run(ctx, type, false, a, M);
}

// RMSNorm fused into the GEMV's prologue: y = W ((x * inv) * norm_w), inv = 1 / sqrt(mean(x^2) + eps) per row.  Replaces
// a launch of the producer (ojas_b200_rmsnorm_q8k) in front of a GEMV: every CTA forms the norm of the row(s) itself.
extern "C" int ojas_b200_gemv_rmsnorm(ojas_b200_ctx *ctx, uint32_t type, int form, const float *x, const float *norm_w, float eps, const void *w,
                                      float *y, const float *bias, size_t K, size_t N, size_t M) {
    int rc = gemv_check(ctx, type, form, w, y, bias, K, N, M);
    if (rc) return rc;
    if (!x || !norm_w) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv_rmsnorm: null pointer");
    if (((uintptr_t)x & 15) != 0 || ((uintptr_t)norm_w & 15) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv_rmsnorm: x and norm_w must be 16-byte aligned");
    GemvArgs a{};
    a.x = x; a.w = (const uint8_t *)w; a.y = y; a.bias = bias;
    a.K = (int)K; a.N = (int)N; a.M = (int)M; a.form = form;
    a.norm_w = norm_w; a.norm_eps = eps;
    return gemv_run(ctx, type, false, a, M);
}

// SwiGLU fused into the GEMV's prologue: y = W (silu(g) * u).  Replaces a launch of ojas_b200_silu_mul_q8k in front of the
// down projection.
extern "C" int ojas_b200_gemv_silu_mul(ojas_b200_ctx *ctx, uint32_t type, int form, const float *g, const float *u, const void *w, float *y,
                                       const float *bias, size_t K, size_t N, size_t M) {
    int rc = gemv_check(ctx, type, form, w, y, bias, K, N, M);
    if (rc) return rc;
    if (!g || !u) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv_silu_mul: null pointer");
    if (((uintptr_t)g & 15) != 0 || ((uintptr_t)u & 15) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv_silu_mul: g and u must be 16-byte aligned");
    GemvArgs a{};
    a.x = g; a.x2 = u; a.w = (const uint8_t *)w; a.y = y; a.bias = bias;
    a.K = (int)K; a.N = (int)N; a.M = (int)M; a.form = form;
    return gemv_run(ctx, type, false, a, M);
}

// One activation row against the expert picked on the device: w + *sel * stride (stride != 0) or w + *sel (offset
// table entry); y = (or +=) alpha * W x with alpha read on the device when given.
int ojas_gemv_selected(ojas_b200_ctx *ctx, uint32_t type, int form, const float *x, const void *w, const uint32_t *sel, size_t sel_stride,
                       const float *alpha, float *y, size_t K, size_t N) {
    int rc = gemv_check(ctx, type, form, w, y, nullptr, K, N, 1);
    if (rc) return rc;
    if (!x || !sel) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: null pointer");
    if (((uintptr_t)x & 15) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: x must be 16-byte aligned");
    GemvArgs a{};
    a.x = x; a.w = (const uint8_t *)w; a.y = y;
    a.K = (int)K; a.N = (int)N; a.M = 1; a.form = form;
    a.sel = sel; a.sel_stride = sel_stride; a.alpha = alpha;
    return gemv_run(ctx, type, false, a, 1);
}

// The tensor-parallel form of a single-row GEMV (tp.cu): results also go to the peers' windows.
int ojas_gemv_tp(ojas_b200_ctx *ctx, uint32_t type, const float *x, const void *w, size_t K, size_t N, const TpPush &push) {
    float *y = reinterpret_cast<float *>(push.dst[0]);      // (not written: the results go to the windows)
    int rc = gemv_check(ctx, type, OJAS_B200_PLAIN, w, y, nullptr, K, N, 1);
    if (rc) return rc;
    if (!x) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: null activation pointer");
    if (((uintptr_t)x & 15) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv: x must be 16-byte aligned");
    GemvArgs a{};
    a.x = x; a.w = (const uint8_t *)w; a.y = y;
    a.K = (int)K; a.N = (int)N; a.M = 1; a.form = OJAS_B200_PLAIN;
    a.tp = push;
    return gemv_run(ctx, type, false, a, 1);
}

extern "C" int ojas_b200_gemv_q8k(ojas_b200_ctx *ctx, uint32_t type, int form, const int8_t *q, const float *scales,
                                  const int32_t *bsums, const void *w, float *y, const float *bias, size_t K, size_t N,
                                  size_t M) {
    int rc = gemv_check(ctx, type, form, w, y, bias, K, N, M);
    if (rc) return rc;
    if (f32_act_type(type))
        return ojas_fail(ctx, OJAS_B200_E_UNSUPPORTED, "gemv_q8k: Q8_0, IQ4_NL and IQ4_XS rows meet f32 activations, not Q8_K blocks");
    if (!q || !scales || !bsums) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv_q8k: null activation pointer");
    if (((uintptr_t)q & 15) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv_q8k: q must be 16-byte aligned");
    GemvArgs a{};
    a.q = q; a.scales = scales; a.bsums = bsums; a.w = (const uint8_t *)w; a.y = y; a.bias = bias;
    a.K = (int)K; a.N = (int)N; a.M = (int)M; a.form = form;
    return gemv_run(ctx, type, true, a, M);
}

extern "C" int ojas_b200_gemv_idots(ojas_b200_ctx *ctx, uint32_t type, const float *x, const void *w, int32_t *idots,
                                    size_t K, size_t N) {
    float dummy;
    int rc = gemv_check(ctx, type, OJAS_B200_PLAIN, w, &dummy, nullptr, K, N, 1);
    if (rc) return rc;
    if (f32_act_type(type)) return ojas_fail(ctx, OJAS_B200_E_UNSUPPORTED, "gemv_idots: Q8_0, IQ4_NL and IQ4_XS have no integer block dots");
    if (!x || !idots) return ojas_fail(ctx, OJAS_B200_E_ARG, "gemv_idots: null pointer");
    GemvArgs a{};
    a.x = x; a.w = (const uint8_t *)w; a.idots = idots;
    a.K = (int)K; a.N = (int)N; a.M = 1; a.form = OJAS_B200_PLAIN;
    rc = gemv_launch_batch(ctx, type, false, true, a);
    return rc == 1 ? ojas_fail(ctx, OJAS_B200_E_LIMIT, "gemv_idots: K=%zu does not fit in shared memory", K) : rc;
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
