// Token-table gather: x[m, :] = the dequantized row ids[m] of a table kept as raw GGUF blocks (read in place, no
// re-layout: a table row is touched once per token, there is nothing to stream).  Counterpart of q35_embed_q4k
// (crates/ojas-cuda/src/kernels/qwen35.rs:51-69), for the formats of this path; the arithmetic and its order are the
// decoder's (crates/ojas-formats/src/gguf.rs:704-708, 796-840, 1042-1058, 1060-1085, 1086-1108), so the rows equal the CPU decode
// bit for bit.  One warp per (token, 256 values): the lane owns values 8 lane .. 8 lane + 7 and writes 32 contiguous bytes.
#include "common.cuh"

namespace {

__device__ __forceinline__ void scale_min(int j, const uint8_t *sc, float &s, float &m) {   // get_scale_min_k4, gguf.rs:1132-1140
    if (j < 4) {
        s = (float)(sc[j] & 63);
        m = (float)(sc[j + 4] & 63);
    } else {
        s = (float)((sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4));
        m = (float)((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
    }
}

// The codebook of IQ4_NL / IQ4_XS (ggml's kvalues_iq4nl; the decoder reads it as iq_tables::KVALUES_IQ4NL, gguf.rs:832).
__constant__ int8_t kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

template <int TYPE>
__global__ void __launch_bounds__(256) embed_kernel(const uint8_t *table, const uint32_t *ids, float *x, unsigned d, unsigned M, unsigned rows) {
    const unsigned lane = threadIdx.x & 31, nsb = d >> 8;
    const unsigned long long task = (unsigned long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (task >= (unsigned long long)M * nsb) return;
    const unsigned m = (unsigned)(task / nsb), sb = (unsigned)(task % nsb);
    unsigned id = __ldg(ids + m);
    if (id >= rows) id = rows - 1;                               // an id past the table reads its last row, never out of bounds
    float v[8];
    const unsigned e0 = lane * 8;                                // first of this lane's eight values inside the super-block
    if (TYPE == OJAS_B200_Q8_0) {
        const uint8_t *blk = table + ((size_t)id * nsb + sb) * 272 + (e0 >> 5) * 34;
        const float dd = f16_bits_to_f32((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __fmul_rn(dd, (float)(int8_t)blk[2 + (e0 & 31) + i]);
    } else if (TYPE == OJAS_B200_IQ4_XS) {
        const uint8_t *blk = table + ((size_t)id * nsb + sb) * 136;
        const float dd = f16_bits_to_f32((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
        const unsigned sh = (unsigned)blk[2] | ((unsigned)blk[3] << 8), g = e0 >> 5, o = e0 & 31;
        const int ls = (int)(((blk[4 + g / 2] >> (4 * (g % 2))) & 0xF) | (((sh >> (2 * g)) & 3u) << 4)) - 32;
        const float dl = __fmul_rn(dd, (float)ls);
        const uint8_t *q = blk + 8 + g * 16 + (o & 15);           // values 0..15 of the group are low nibbles, 16..31 high
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __fmul_rn(dl, (float)kIq4nl[(o & 16) ? (q[i] >> 4) : (q[i] & 0xF)]);
    } else if (TYPE == OJAS_B200_IQ4_NL) {
        const uint8_t *blk = table + ((size_t)id * nsb + sb) * 144 + (e0 >> 5) * 18;
        const float dd = f16_bits_to_f32((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
        const unsigned o = e0 & 31;
        const uint8_t *q = blk + 2 + (o & 15);
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __fmul_rn(dd, (float)kIq4nl[(o & 16) ? (q[i] >> 4) : (q[i] & 0xF)]);
    } else if (TYPE == OJAS_B200_Q6_K) {
        const uint8_t *blk = table + ((size_t)id * nsb + sb) * 210;
        const float dd = f16_bits_to_f32((uint32_t)blk[208] | ((uint32_t)blk[209] << 8));
        const unsigned half = e0 >> 7, quarter = (e0 >> 5) & 3, l0 = e0 & 31;
        const uint8_t *ql = blk + half * 64, *qh = blk + 128 + half * 32;
        const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192 + half * 8);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const unsigned l = l0 + i;
            const unsigned nib = (quarter & 1) ? ql[l + 32] : ql[l];
            const int q = (int)(((quarter & 2) ? (nib >> 4) : (nib & 0xF)) | (((qh[l] >> (2 * quarter)) & 3) << 4)) - 32;
            v[i] = __fmul_rn(__fmul_rn(dd, (float)sc[l / 16 + 2 * quarter]), (float)q);
        }
    } else {                                                     // Q4_K, Q5_K
        constexpr bool FIVE = TYPE == OJAS_B200_Q5_K;
        const uint8_t *blk = table + ((size_t)id * nsb + sb) * (FIVE ? 176 : 144);
        const float dd = f16_bits_to_f32((uint32_t)blk[0] | ((uint32_t)blk[1] << 8)), dm = f16_bits_to_f32((uint32_t)blk[2] | ((uint32_t)blk[3] << 8));
        const unsigned chunk = e0 >> 6, hi = (e0 >> 5) & 1, l0 = e0 & 31, j = 2 * chunk + hi;
        float s, mn;
        scale_min((int)j, blk + 4, s, mn);
        const float dl = __fmul_rn(dd, s), ml = __fmul_rn(dm, mn);
        const uint8_t *qs = blk + (FIVE ? 48 : 16) + chunk * 32, *qh = blk + 16;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const unsigned by = qs[l0 + i];
            float q = (float)(hi ? (by >> 4) : (by & 15u));
            if (FIVE) q = __fadd_rn(q, ((qh[l0 + i] >> j) & 1) ? 16.0f : 0.0f);
            v[i] = __fsub_rn(__fmul_rn(dl, q), ml);
        }
    }
    float4 *out = reinterpret_cast<float4 *>(x + (size_t)m * d + (size_t)sb * 256 + e0);
    out[0] = make_float4(v[0], v[1], v[2], v[3]);
    out[1] = make_float4(v[4], v[5], v[6], v[7]);
}

}  // namespace

// table: raw GGUF blocks [rows, d] of ggml_type on the device; ids [M] u32; x [M, d] f32 (16-byte aligned).
extern "C" int ojas_b200_embed_rows(ojas_b200_ctx *ctx, uint32_t type, const void *table, size_t rows, const uint32_t *ids, size_t M, size_t d,
                                    float *x) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!table || !ids || !x) return ojas_fail(ctx, OJAS_B200_E_ARG, "embed_rows: null pointer");
    if (!type_supported(type)) return ojas_fail(ctx, OJAS_B200_E_ARG, "embed_rows: unsupported GGUF type %u", type);
    if (d == 0 || d % 256 != 0 || d > 0x7fffff00u) return ojas_fail(ctx, OJAS_B200_E_ARG, "embed_rows: d=%zu must be a positive multiple of 256", d);
    if (rows == 0 || rows > 0xffffffffu) return ojas_fail(ctx, OJAS_B200_E_ARG, "embed_rows: rows=%zu out of range", rows);
    if (((uintptr_t)x & 15) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "embed_rows: x must be 16-byte aligned");
    if (M == 0) return 0;
    const unsigned long long tasks = (unsigned long long)M * (d / 256), blocks = (tasks + 7) / 8;
    if (M > 0x7fffffffu || blocks > 0x7fffffffULL) return ojas_fail(ctx, OJAS_B200_E_ARG, "embed_rows: too many rows");
    const uint8_t *t = (const uint8_t *)table;
    if (type == OJAS_B200_Q4_K) embed_kernel<OJAS_B200_Q4_K><<<(unsigned)blocks, 256, 0, ctx->stream>>>(t, ids, x, (unsigned)d, (unsigned)M, (unsigned)rows);
    else if (type == OJAS_B200_Q5_K) embed_kernel<OJAS_B200_Q5_K><<<(unsigned)blocks, 256, 0, ctx->stream>>>(t, ids, x, (unsigned)d, (unsigned)M, (unsigned)rows);
    else if (type == OJAS_B200_Q6_K) embed_kernel<OJAS_B200_Q6_K><<<(unsigned)blocks, 256, 0, ctx->stream>>>(t, ids, x, (unsigned)d, (unsigned)M, (unsigned)rows);
    else if (type == OJAS_B200_IQ4_NL) embed_kernel<OJAS_B200_IQ4_NL><<<(unsigned)blocks, 256, 0, ctx->stream>>>(t, ids, x, (unsigned)d, (unsigned)M, (unsigned)rows);
    else if (type == OJAS_B200_IQ4_XS) embed_kernel<OJAS_B200_IQ4_XS><<<(unsigned)blocks, 256, 0, ctx->stream>>>(t, ids, x, (unsigned)d, (unsigned)M, (unsigned)rows);
    else embed_kernel<OJAS_B200_Q8_0><<<(unsigned)blocks, 256, 0, ctx->stream>>>(t, ids, x, (unsigned)d, (unsigned)M, (unsigned)rows);
    OJAS_LAUNCH_CHECK(ctx, "embed_rows");
    return 0;
}
