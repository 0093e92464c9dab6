// Host-side f32 -> GGUF block encoders for Q8_0, Q4_K and Q6_K.
//
// The reference engine has no encoder for these formats (it only ever reads them from model
// files; its own GEMM tests use random blocks, crates/ojas-formats/src/synth.rs:29).  These
// are plain min/max encoders written for this library so that tests and benchmarks can turn
// seeded N(0, sigma) matrices into legal blocks.  Parity never depends on how a block was
// encoded, only on how it is decoded and dotted.
#include <math.h>

#include "common.cuh"

static inline uint16_t f32_to_f16_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }
static inline float f16_bits_to_f32_host(uint16_t h) { return __half2float(__ushort_as_half(h)); }
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : v > hi ? hi : v; }

static void encode_q80_block(const float *x, uint8_t *out) {
    float amax = 0.f;
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
    const uint16_t dh = f32_to_f16_bits(amax / 127.f);
    const float d = f16_bits_to_f32_host(dh);
    out[0] = (uint8_t)(dh & 0xff);
    out[1] = (uint8_t)(dh >> 8);
    for (int i = 0; i < 32; i++) out[2 + i] = (uint8_t)(int8_t)clampi(d > 0.f ? (int)lrintf(x[i] / d) : 0, -127, 127);
}

static void encode_q4k_block(const float *x, uint8_t *out) {
    float scale[8], mn[8];
    float smax = 0.f, mmax = 0.f;
    for (int j = 0; j < 8; j++) {
        float lo = 0.f, hi = 0.f;
        for (int i = 0; i < 32; i++) { lo = fminf(lo, x[32 * j + i]); hi = fmaxf(hi, x[32 * j + i]); }
        mn[j] = -lo;                       // >= 0: the sub-block offset
        scale[j] = (hi - lo) / 15.f;
        smax = fmaxf(smax, scale[j]);
        mmax = fmaxf(mmax, mn[j]);
    }
    const uint16_t dh = f32_to_f16_bits(smax / 63.f), dmh = f32_to_f16_bits(mmax / 63.f);
    const float d = f16_bits_to_f32_host(dh), dmin = f16_bits_to_f32_host(dmh);
    int s[8], m[8];
    for (int j = 0; j < 8; j++) {
        s[j] = d > 0.f ? clampi((int)lrintf(scale[j] / d), 0, 63) : 0;
        m[j] = dmin > 0.f ? clampi((int)lrintf(mn[j] / dmin), 0, 63) : 0;
    }
    out[0] = (uint8_t)(dh & 0xff); out[1] = (uint8_t)(dh >> 8);
    out[2] = (uint8_t)(dmh & 0xff); out[3] = (uint8_t)(dmh >> 8);
    uint8_t *sc = out + 4;
    for (int j = 0; j < 4; j++) {
        sc[j] = (uint8_t)(s[j] | ((s[j + 4] >> 4) << 6));
        sc[j + 4] = (uint8_t)(m[j] | ((m[j + 4] >> 4) << 6));
        sc[j + 8] = (uint8_t)((s[j + 4] & 0xF) | ((m[j + 4] & 0xF) << 4));
    }
    uint8_t *qs = out + 16;
    for (int c = 0; c < 4; c++)
        for (int l = 0; l < 32; l++) {
            int q2[2];
            for (int h = 0; h < 2; h++) {
                const int j = 2 * c + h;
                const float dl = d * (float)s[j], ml = dmin * (float)m[j];
                q2[h] = dl > 0.f ? clampi((int)lrintf((x[32 * j + l] + ml) / dl), 0, 15) : 0;
            }
            qs[32 * c + l] = (uint8_t)(q2[0] | (q2[1] << 4));
        }
}

static void encode_q6k_block(const float *x, uint8_t *out) {
    float scale[16];
    float smax = 0.f;
    for (int j = 0; j < 16; j++) {
        float amax = 0.f;
        for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(x[16 * j + i]));
        scale[j] = amax / 31.f;
        smax = fmaxf(smax, scale[j]);
    }
    const uint16_t dh = f32_to_f16_bits(smax / 127.f);
    const float d = f16_bits_to_f32_host(dh);
    int8_t sc[16];
    uint8_t q6[256];
    for (int j = 0; j < 16; j++) {
        sc[j] = (int8_t)(d > 0.f ? clampi((int)lrintf(scale[j] / d), 0, 127) : 0);
        const float dl = d * (float)sc[j];
        for (int i = 0; i < 16; i++)
            q6[16 * j + i] = (uint8_t)(dl > 0.f ? clampi((int)lrintf(x[16 * j + i] / dl) + 32, 0, 63) : 32);
    }
    memset(out, 0, 210);
    for (int w = 0; w < 256; w++) {   // inverse of the decoder's bit layout (crates/ojas-formats/src/gguf.rs:1086-1108)
        const int hh = w >> 7, quarter = (w >> 5) & 3, l = w & 31;
        uint8_t *ql = out + hh * 64 + ((quarter & 1) ? l + 32 : l);
        *ql |= (uint8_t)((q6[w] & 0xF) << ((quarter & 2) ? 4 : 0));
        out[128 + hh * 32 + l] |= (uint8_t)((q6[w] >> 4) << (2 * quarter));
    }
    for (int j = 0; j < 16; j++) out[192 + j] = (uint8_t)sc[j];
    out[208] = (uint8_t)(dh & 0xff);
    out[209] = (uint8_t)(dh >> 8);
}

extern "C" int ojas_b200_encode_host(uint32_t type, const float *w, size_t N, size_t K, void *raw_out) {
    if (!w || !raw_out || K == 0 || K % 256 != 0) return OJAS_B200_E_ARG;
    uint8_t *out = (uint8_t *)raw_out;
    const size_t total = N * K;
    switch (type) {
    case OJAS_B200_Q8_0:
        for (size_t b = 0; b < total / 32; b++) encode_q80_block(w + b * 32, out + b * 34);
        return 0;
    case OJAS_B200_Q4_K:
        for (size_t b = 0; b < total / 256; b++) encode_q4k_block(w + b * 256, out + b * 144);
        return 0;
    case OJAS_B200_Q6_K:
        for (size_t b = 0; b < total / 256; b++) encode_q6k_block(w + b * 256, out + b * 210);
        return 0;
    default:
        return OJAS_B200_E_ARG;
    }
}
