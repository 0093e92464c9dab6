/*
 * CPU oracle for the quantized-matmul path of ojas-engine.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is a plain-C restatement of the reference's
 * own CPU quantized matmul (crate ojas-cpu) and of the block decoders in
 * ojas-formats. Only the tests, the smoke check and the CPU-baseline leg of the
 * benchmark may call it; the product library never links or loads it.
 *
 * Every function names the reference source it follows (path inside the
 * reference project : line).  Float arithmetic keeps the reference's evaluation
 * order; build with -ffp-contract=off so no multiply-add is fused (the Rust
 * original does not fuse).
 *
 * Pins: the decoders + the synthetic block generator reproduce the two FNV
 * digests the reference's own test holds for Q4_K and Q6_K
 * (crates/ojas-formats/tests/quant_formats.rs:33-50) and the exact Q8_0 rows of
 * crates/ojas-formats/tests/rows.rs:13-17,57-66.  quant_q8k / dot_q4k / dot_q6k /
 * dot_q80 / matvec_kq have no golden vector in the reference ("parity unpinned"
 * for that layer): they are pinned only by being a line-by-line restatement plus
 * the algebraic identity  dot(row, q8k(x)) == sum dequant(row)[i] * (sx*q[i])
 * checked in the tests.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- f16 <-> f32
 * IEEE binary16, round-to-nearest-even on narrowing: what the `half` crate does
 * (crates/ojas-formats/src/gguf.rs:602-609 h16 / rdh). */
ORC_API float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

ORC_API uint16_t orc_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? (0x200u | ((absx >> 13) & 0x3ffu)) : 0));
    }
    if (absx >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x38800000u) { /* subnormal half or zero */
        if (absx < 0x33000000u) return sign; /* < 2^-25 -> 0 (2^-25 itself ties to even = 0) */
        uint32_t e = absx >> 23;
        uint32_t man = (absx & 0x7fffffu) | 0x800000u;
        uint32_t shift = 126 - e; /* result = man >> shift, 14..24 */
        uint32_t half_ulp = 1u << (shift - 1);
        uint32_t res = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        if (rem > half_ulp || (rem == half_ulp && (res & 1))) res++;
        return (uint16_t)(sign | res);
    }
    uint32_t e = (absx >> 23) - 127 + 15;
    uint32_t man = absx & 0x7fffffu;
    uint32_t res = (e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (res & 1))) res++;
    return (uint16_t)(sign | res);
}

static inline float rdh(const uint8_t *b, size_t i) {
    return orc_f16_to_f32((uint16_t)(b[i] | (b[i + 1] << 8)));
}

/* ---------------------------------------------------------------- block shapes
 * crates/ojas-formats/src/synth.rs:12-21 (the formats on the path: Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS). */
ORC_API int orc_block_shape(uint32_t type, uint32_t *block_bytes, uint32_t *block_weights) {
    switch (type) {
    case 8:  *block_bytes = 34;  *block_weights = 32;  return 0;
    case 12: *block_bytes = 144; *block_weights = 256; return 0;
    case 13: *block_bytes = 176; *block_weights = 256; return 0;
    case 14: *block_bytes = 210; *block_weights = 256; return 0;
    case 20: *block_bytes = 18;  *block_weights = 32;  return 0;
    case 23: *block_bytes = 136; *block_weights = 256; return 0;
    default: return -1;
    }
}

/* Random but legal blocks, f16 scale fields pinned.
 * crates/ojas-formats/src/synth.rs:29-64. */
ORC_API int orc_synth_blocks(uint32_t type, size_t nb, uint8_t *out) {
    uint32_t bb, bw;
    if (orc_block_shape(type, &bb, &bw)) return -1;
    uint64_t st = 0x2545F4914F6CDD1DULL;
    for (size_t i = 0; i < nb * bb; i++) {
        st ^= st << 13; st ^= st >> 7; st ^= st << 17;
        out[i] = (uint8_t)(st >> 24);
    }
    uint16_t dmin = orc_f32_to_f16(0.01f);
    for (size_t i = 0; i < nb; i++) {
        uint8_t *blk = out + i * bb;
        uint16_t d = orc_f32_to_f16(0.05f + (float)(i % 7) * 0.01f);
        size_t at = (type == 14) ? 208 : 0;
        blk[at] = (uint8_t)(d & 0xff); blk[at + 1] = (uint8_t)(d >> 8);
        if (type == 12 || type == 13) { blk[2] = (uint8_t)(dmin & 0xff); blk[3] = (uint8_t)(dmin >> 8); }
    }
    return 0;
}

/* ---------------------------------------------------------------- decoders */
/* crates/ojas-formats/src/gguf.rs:1132-1140 and crates/ojas-cpu/src/cpu_math.rs:566-574 */
static inline void scale_min_k4(int j, const uint8_t *s, float *sc, float *mn) {
    if (j < 4) {
        *sc = (float)(s[j] & 63);
        *mn = (float)(s[j + 4] & 63);
    } else {
        uint8_t d = (uint8_t)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
        uint8_t m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
        *sc = (float)d;
        *mn = (float)m;
    }
}

/* The 16-entry non-linear codebook of IQ4_NL / IQ4_XS.  The reference reads it as crate::iq_tables::KVALUES_IQ4NL
 * (crates/ojas-formats/src/gguf.rs:832, crates/ojas-cpu/src/cpu_math.rs:859); the file that defines it is not part of
 * the reference tree, so the values are ggml's published kvalues_iq4nl.  They are pinned by the reference's own decode
 * digest of synthetic IQ4_XS blocks (crates/ojas-formats/tests/quant_formats.rs:48): a wrong entry changes the digest. */
static const int8_t orc_kvalues_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* Decode `n` weights of GGUF `type` to f32 (before the f16 rounding of
 * dequant_to_f16).  Same arithmetic order as crates/ojas-formats/src/gguf.rs:
 * Q8_0 :704-708, Q4_K :1042-1058, Q6_K :1086-1108. */
ORC_API int orc_dequant_f32(const uint8_t *b, uint32_t type, size_t n, float *out) {
    size_t o = 0;
    if (type == 8) {
        for (size_t blk = 0; blk < n / 32; blk++) {
            const uint8_t *p = b + blk * 34;
            float d = rdh(p, 0);
            for (int j = 0; j < 32; j++) out[o++] = d * (float)(int8_t)p[2 + j];
        }
    } else if (type == 12) {
        for (size_t blk = 0; blk < n / 256; blk++) {
            const uint8_t *p = b + blk * 144;
            float d = rdh(p, 0), dmin = rdh(p, 2);
            const uint8_t *sc = p + 4, *qs = p + 16;
            for (int chunk = 0; chunk < 4; chunk++) {
                float d1, m1, d2, m2;
                scale_min_k4(chunk * 2, sc, &d1, &m1);
                scale_min_k4(chunk * 2 + 1, sc, &d2, &m2);
                float dl1 = d * d1, ml1 = dmin * m1, dl2 = d * d2, ml2 = dmin * m2;
                const uint8_t *q = qs + chunk * 32;
                for (int l = 0; l < 32; l++) out[o++] = dl1 * (float)(q[l] & 0xF) - ml1;
                for (int l = 0; l < 32; l++) out[o++] = dl2 * (float)(q[l] >> 4) - ml2;
            }
        }
    } else if (type == 13) {   /* Q5_K, crates/ojas-formats/src/gguf.rs:1060-1085 */
        for (size_t blk = 0; blk < n / 256; blk++) {
            const uint8_t *p = b + blk * 176;
            float d = rdh(p, 0), dmin = rdh(p, 2);
            const uint8_t *sc = p + 4, *qh = p + 16, *qs = p + 48;
            uint8_t u1 = 1, u2 = 2;
            for (int chunk = 0; chunk < 4; chunk++) {
                float d1, m1, d2, m2;
                scale_min_k4(chunk * 2, sc, &d1, &m1);
                scale_min_k4(chunk * 2 + 1, sc, &d2, &m2);
                float dl1 = d * d1, ml1 = dmin * m1, dl2 = d * d2, ml2 = dmin * m2;
                const uint8_t *q = qs + chunk * 32;
                for (int l = 0; l < 32; l++) out[o++] = dl1 * ((float)(q[l] & 0xF) + ((qh[l] & u1) ? 16.0f : 0.0f)) - ml1;
                for (int l = 0; l < 32; l++) out[o++] = dl2 * ((float)(q[l] >> 4) + ((qh[l] & u2) ? 16.0f : 0.0f)) - ml2;
                u1 = (uint8_t)(u1 << 2); u2 = (uint8_t)(u2 << 2);
            }
        }
    } else if (type == 14) {
        float y[128];
        for (size_t blk = 0; blk < n / 256; blk++) {
            const uint8_t *p = b + blk * 210;
            float d = rdh(p, 208);
            for (int h = 0; h < 2; h++) {
                const uint8_t *ql = p + h * 64, *qh = p + 128 + h * 32;
                const int8_t *sc = (const int8_t *)(p + 192 + h * 8);
                for (int l = 0; l < 32; l++) {
                    int is = l / 16;
                    int q1 = ((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                    int q2 = ((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    int q3 = ((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                    int q4 = ((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                    y[l]      = d * (float)sc[is]     * (float)q1;
                    y[l + 32] = d * (float)sc[is + 2] * (float)q2;
                    y[l + 64] = d * (float)sc[is + 4] * (float)q3;
                    y[l + 96] = d * (float)sc[is + 6] * (float)q4;
                }
                for (int i = 0; i < 128; i++) out[o++] = y[i];
            }
        }
    } else if (type == 20) {   /* IQ4_NL, crates/ojas-formats/src/gguf.rs:796-812 */
        for (size_t blk = 0; blk < n / 32; blk++) {
            const uint8_t *p = b + blk * 18;
            float d = rdh(p, 0);
            for (int j = 0; j < 16; j++) out[o++] = d * (float)orc_kvalues_iq4nl[p[2 + j] & 0xF];
            for (int j = 0; j < 16; j++) out[o++] = d * (float)orc_kvalues_iq4nl[p[2 + j] >> 4];
        }
    } else if (type == 23) {   /* IQ4_XS, crates/ojas-formats/src/gguf.rs:814-840 */
        for (size_t blk = 0; blk < n / 256; blk++) {
            const uint8_t *p = b + blk * 136;
            float d = rdh(p, 0);
            unsigned sh = (unsigned)(p[2] | (p[3] << 8));
            const uint8_t *sl = p + 4, *qs = p + 8;
            for (int ib = 0; ib < 8; ib++) {
                int ls = (int)(((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3u) << 4));
                float dl = d * (float)(ls - 32);
                const uint8_t *q = qs + ib * 16;
                for (int j = 0; j < 16; j++) out[o++] = dl * (float)orc_kvalues_iq4nl[q[j] & 0xF];
                for (int j = 0; j < 16; j++) out[o++] = dl * (float)orc_kvalues_iq4nl[q[j] >> 4];
            }
        }
    } else {
        return -1;
    }
    return 0;
}

/* dequant_to_f16 (crates/ojas-formats/src/gguf.rs:612): the f32 value rounded to f16 bits. */
ORC_API int orc_dequant_f16(const uint8_t *b, uint32_t type, size_t n, uint16_t *out) {
    float *tmp = (float *)malloc(n * sizeof(float));
    if (!tmp) return -2;
    int rc = orc_dequant_f32(b, type, n, tmp);
    if (!rc) for (size_t i = 0; i < n; i++) out[i] = orc_f32_to_f16(tmp[i]);
    free(tmp);
    return rc;
}

/* FNV-1a-64 over the "{:.6}" text of every f16 value.
 * crates/ojas-formats/tests/quant_formats.rs:20-31.  glibc "%.6f" prints the
 * exact decimal expansion rounded half-to-even on the exact value, as Rust does. */
ORC_API uint64_t orc_digest_f16(const uint16_t *vals, size_t n) {
    uint64_t h = 0xcbf29ce484222325ULL;
    char buf[64];
    for (size_t i = 0; i < n; i++) {
        float v = orc_f16_to_f32(vals[i]);
        int len = snprintf(buf, sizeof buf, "%.6f", (double)v);
        for (int c = 0; c < len; c++) {
            h ^= (uint8_t)buf[c];
            h *= 0x00000100000001B3ULL;
        }
    }
    return h;
}

/* ---------------------------------------------------------------- activations
 * quant_q8k, crates/ojas-cpu/src/cpu_math.rs:545-563.  k must be a multiple of
 * 256 here (matvec_kq's row_bytes table assumes it, :1148).  Rust's f32::round
 * is half-away-from-zero == roundf; NaN casts to 0. */
ORC_API void orc_quant_q8k(const float *x, size_t k, float *scales, int8_t *q, int32_t *bsums) {
    size_t nsb = k / 256;
    memset(bsums, 0, nsb * 8 * sizeof(int32_t));
    for (size_t sb = 0; sb < nsb; sb++) {
        const float *seg = x + sb * 256;
        float m = 0.0f;
        for (int i = 0; i < 256; i++) {
            float a = fabsf(seg[i]);
            /* f32::max ignores a NaN operand */
            if (a > m) m = a;
        }
        float scale = (m > 0.0f) ? m / 127.0f : 1.0f;
        float inv = 1.0f / scale;
        scales[sb] = scale;
        for (int i = 0; i < 256; i++) {
            float r = roundf(seg[i] * inv);
            if (r < -127.0f) r = -127.0f;
            if (r > 127.0f) r = 127.0f;
            int8_t qi = (r != r) ? 0 : (int8_t)r;
            q[sb * 256 + i] = qi;
            bsums[sb * 8 + i / 32] += qi;
        }
    }
}

/* ---------------------------------------------------------------- block dots */
static inline int32_t idot32(const uint8_t *w, const int8_t *x) { /* cpu_math.rs:583-593 (scalar arm) */
    int32_t s = 0;
    for (int i = 0; i < 32; i++) s += (int32_t)w[i] * (int32_t)x[i];
    return s;
}

/* dot_q4k, crates/ojas-cpu/src/cpu_math.rs:609-635.  If idots != NULL the eight
 * int32 sub-block dots of every super-block are written there (8 per block). */
ORC_API float orc_dot_q4k(const uint8_t *row, size_t nsb, const float *scales, const int8_t *q,
                          const int32_t *bsums, int32_t *idots) {
    float total = 0.0f;
    uint8_t lo[32], hi[32];
    for (size_t sb = 0; sb < nsb; sb++) {
        const uint8_t *blk = row + sb * 144;
        float d = rdh(blk, 0), dmin = rdh(blk, 2);
        const uint8_t *sc = blk + 4, *qs = blk + 16;
        float sx = scales[sb];
        const int8_t *xq = q + sb * 256;
        const int32_t *bs = bsums + sb * 8;
        float sumd = 0.0f, summ = 0.0f;
        for (int c = 0; c < 4; c++) {
            const uint8_t *qq = qs + c * 32;
            for (int l = 0; l < 32; l++) { lo[l] = qq[l] & 0xF; hi[l] = qq[l] >> 4; }
            float s1, m1, s2, m2;
            scale_min_k4(c * 2, sc, &s1, &m1);
            scale_min_k4(c * 2 + 1, sc, &s2, &m2);
            int32_t i1 = idot32(lo, xq + c * 64);
            int32_t i2 = idot32(hi, xq + c * 64 + 32);
            if (idots) { idots[sb * 8 + c * 2] = i1; idots[sb * 8 + c * 2 + 1] = i2; }
            sumd += s1 * (float)i1;
            sumd += s2 * (float)i2;
            summ += m1 * (float)bs[c * 2] + m2 * (float)bs[c * 2 + 1];
        }
        total += sx * (d * sumd - dmin * summ);
    }
    return total;
}

/* dot_q5k, crates/ojas-cpu/src/cpu_math.rs:637-671: Q4_K's arithmetic on five-bit values (the fifth bit of weight l
 * of sub-block j is bit j of qh[l]).  idots as for Q4_K. */
ORC_API float orc_dot_q5k(const uint8_t *row, size_t nsb, const float *scales, const int8_t *q,
                          const int32_t *bsums, int32_t *idots) {
    float total = 0.0f;
    uint8_t lo[32], hi[32];
    for (size_t sb = 0; sb < nsb; sb++) {
        const uint8_t *blk = row + sb * 176;
        float d = rdh(blk, 0), dmin = rdh(blk, 2);
        const uint8_t *sc = blk + 4, *qh = blk + 16, *qs = blk + 48;
        float sx = scales[sb];
        const int8_t *xq = q + sb * 256;
        const int32_t *bs = bsums + sb * 8;
        float sumd = 0.0f, summ = 0.0f;
        uint8_t u1 = 1, u2 = 2;
        for (int c = 0; c < 4; c++) {
            const uint8_t *qq = qs + c * 32;
            for (int l = 0; l < 32; l++) {
                lo[l] = (uint8_t)((qq[l] & 0xF) | ((qh[l] & u1) ? 16 : 0));
                hi[l] = (uint8_t)((qq[l] >> 4) | ((qh[l] & u2) ? 16 : 0));
            }
            float s1, m1, s2, m2;
            scale_min_k4(c * 2, sc, &s1, &m1);
            scale_min_k4(c * 2 + 1, sc, &s2, &m2);
            int32_t i1 = idot32(lo, xq + c * 64);
            int32_t i2 = idot32(hi, xq + c * 64 + 32);
            if (idots) { idots[sb * 8 + c * 2] = i1; idots[sb * 8 + c * 2 + 1] = i2; }
            sumd += s1 * (float)i1;
            sumd += s2 * (float)i2;
            summ += m1 * (float)bs[c * 2] + m2 * (float)bs[c * 2 + 1];
            u1 = (uint8_t)(u1 << 2); u2 = (uint8_t)(u2 << 2);
        }
        total += sx * (d * sumd - dmin * summ);
    }
    return total;
}

/* dot_q6k, crates/ojas-cpu/src/cpu_math.rs:674-722.  idots (optional): 16 int32
 * per super-block, the per-16 dots of the unsigned 0..63 values in weight order. */
ORC_API float orc_dot_q6k(const uint8_t *row, size_t nsb, const float *scales, const int8_t *q,
                          int32_t *idots) {
    float total = 0.0f;
    uint8_t w[32];
    for (size_t sb = 0; sb < nsb; sb++) {
        const uint8_t *blk = row + sb * 210;
        float d = rdh(blk, 208);
        float sx = scales[sb];
        const int8_t *xq = q + sb * 256;
        float sum = 0.0f, sub = 0.0f;
        for (int h = 0; h < 2; h++) {
            const uint8_t *ql = blk + h * 64, *qh = blk + 128 + h * 32;
            const int8_t *sc = (const int8_t *)(blk + 192 + h * 8);
            const int8_t *xh = xq + h * 128;
            for (int quarter = 0; quarter < 4; quarter++) {
                for (int l = 0; l < 32; l++) {
                    switch (quarter) {
                    case 0: w[l] = (uint8_t)((ql[l] & 0xF) | ((qh[l] & 3) << 4)); break;
                    case 1: w[l] = (uint8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)); break;
                    case 2: w[l] = (uint8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)); break;
                    default: w[l] = (uint8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)); break;
                    }
                }
                const int8_t *x32 = xh + quarter * 32;
                float s0 = (float)sc[quarter * 2], s1 = (float)sc[quarter * 2 + 1];
                int32_t i0 = 0, i1 = 0, x0 = 0, x1 = 0;
                for (int l = 0; l < 16; l++) {
                    i0 += (int32_t)w[l] * (int32_t)x32[l];
                    x0 += (int32_t)x32[l];
                    i1 += (int32_t)w[l + 16] * (int32_t)x32[l + 16];
                    x1 += (int32_t)x32[l + 16];
                }
                if (idots) {
                    idots[sb * 16 + h * 8 + quarter * 2] = i0;
                    idots[sb * 16 + h * 8 + quarter * 2 + 1] = i1;
                }
                sum += s0 * (float)i0 + s1 * (float)i1;
                sub += s0 * (float)x0 + s1 * (float)x1;
            }
        }
        total += sx * d * (sum - 32.0f * sub);
    }
    return total;
}

/* dot_q80, crates/ojas-cpu/src/cpu_math.rs:971-981: f32 activations, no quantization. */
ORC_API float orc_dot_q80(const uint8_t *row, const float *x, size_t k) {
    float sum = 0.0f;
    for (size_t b = 0; b < k / 32; b++) {
        const uint8_t *blk = row + b * 34;
        const float *xb = x + b * 32;
        float d = rdh(blk, 0);
        float acc = 0.0f;
        for (int j = 0; j < 32; j++) acc += (float)(int8_t)blk[2 + j] * xb[j];
        sum += d * acc;
    }
    return sum;
}

/* dot_iq4xs, crates/ojas-cpu/src/cpu_math.rs:943-967: f32 activations; per group of 32 the codebook values times x
 * (low nibble j, then high nibble j + 16, alternating), the group's sum times (ls - 32), the block's sum times d. */
ORC_API float orc_dot_iq4xs(const uint8_t *row, const float *x, size_t k) {
    float sum = 0.0f;
    for (size_t b = 0; b < k / 256; b++) {
        const uint8_t *blk = row + b * 136;
        const float *xb = x + b * 256;
        float d = rdh(blk, 0);
        unsigned sh = (unsigned)(blk[2] | (blk[3] << 8));
        const uint8_t *sl = blk + 4, *qs = blk + 8;
        float bsum = 0.0f;
        for (int g = 0; g < 8; g++) {
            int ls = (int)(((sl[g / 2] >> (4 * (g % 2))) & 0xF) | (((sh >> (2 * g)) & 3u) << 4));
            const float *xg = xb + g * 32;
            float gsum = 0.0f;
            for (int j = 0; j < 16; j++) {
                uint8_t q = qs[16 * g + j];
                gsum += (float)orc_kvalues_iq4nl[q & 0xF] * xg[j];
                gsum += (float)orc_kvalues_iq4nl[q >> 4] * xg[j + 16];
            }
            bsum += (float)(ls - 32) * gsum;
        }
        sum += d * bsum;
    }
    return sum;
}

/* dot_iq4nl, crates/ojas-cpu/src/cpu_math.rs:993-1010: blocks of 32 (f16 d, sixteen index bytes), f32 activations. */
ORC_API float orc_dot_iq4nl(const uint8_t *row, const float *x, size_t k) {
    float sum = 0.0f;
    for (size_t b = 0; b < k / 32; b++) {
        const uint8_t *blk = row + b * 18;
        const float *xb = x + b * 32;
        float d = rdh(blk, 0);
        float bsum = 0.0f;
        for (int j = 0; j < 16; j++) {
            uint8_t q = blk[2 + j];
            bsum += (float)orc_kvalues_iq4nl[q & 0xF] * xb[j];
            bsum += (float)orc_kvalues_iq4nl[q >> 4] * xb[j + 16];
        }
        sum += d * bsum;
    }
    return sum;
}

/* ---------------------------------------------------------------- matvec_kq
 * crates/ojas-cpu/src/cpu_math.rs:1145-1189: quantize x once, then `threads`
 * workers steal 8-row chunks from a shared counter.  Row stride follows the
 * reference's table (:1148-1160): k/256 * {144, 176, 210, 272, 144, 136}. */
ORC_API size_t orc_row_bytes(uint32_t type, size_t k) {
    switch (type) {
    case 12: return k / 256 * 144;
    case 13: return k / 256 * 176;
    case 14: return k / 256 * 210;
    case 8:  return k / 256 * 272;
    case 20: return k / 256 * 144;
    case 23: return k / 256 * 136;
    default: return 0;
    }
}

typedef struct {
    const uint8_t *raw; uint32_t type; size_t n, k, row_bytes;
    const float *x; const float *scales; const int8_t *q; const int32_t *bsums;
    float *out; size_t *next;
} mv_job;

static void *mv_worker(void *arg) {
    mv_job *j = (mv_job *)arg;
    for (;;) {
        size_t r0 = __atomic_fetch_add(j->next, 8, __ATOMIC_RELAXED);
        if (r0 >= j->n) break;
        size_t r1 = r0 + 8 < j->n ? r0 + 8 : j->n;
        for (size_t row = r0; row < r1; row++) {
            const uint8_t *rb = j->raw + row * j->row_bytes;
            float v;
            if (j->type == 12) v = orc_dot_q4k(rb, j->k / 256, j->scales, j->q, j->bsums, NULL);
            else if (j->type == 13) v = orc_dot_q5k(rb, j->k / 256, j->scales, j->q, j->bsums, NULL);
            else if (j->type == 8) v = orc_dot_q80(rb, j->x, j->k);
            else if (j->type == 20) v = orc_dot_iq4nl(rb, j->x, j->k);
            else if (j->type == 23) v = orc_dot_iq4xs(rb, j->x, j->k);
            else v = orc_dot_q6k(rb, j->k / 256, j->scales, j->q, NULL);
            j->out[row] = v;
        }
    }
    return NULL;
}

ORC_API int orc_matvec_kq(const uint8_t *raw, uint32_t type, size_t n, size_t k, const float *x,
                          int threads, float *out) {
    if (k == 0 || k % 256 != 0) return -1;
    size_t rb = orc_row_bytes(type, k);
    if (!rb) return -1;
    size_t nsb = k / 256;
    float *scales = (float *)malloc(nsb * sizeof(float));
    int8_t *q = (int8_t *)malloc(k);
    int32_t *bsums = (int32_t *)malloc(nsb * 8 * sizeof(int32_t));
    if (!scales || !q || !bsums) { free(scales); free(q); free(bsums); return -2; }
    orc_quant_q8k(x, k, scales, q, bsums);
    size_t next = 0;
    mv_job job = { raw, type, n, k, rb, x, scales, q, bsums, out, &next };
    int nt = threads < 1 ? 1 : threads;
    if ((size_t)nt > (n ? n : 1)) nt = (int)(n ? n : 1);
    if (nt == 1) {
        mv_worker(&job);
    } else {
        pthread_t *th = (pthread_t *)malloc((size_t)nt * sizeof(pthread_t));
        int started = 0;
        for (int t = 0; t < nt; t++) if (pthread_create(&th[started], NULL, mv_worker, &job) == 0) started++;
        if (!started) mv_worker(&job);
        for (int t = 0; t < started; t++) pthread_join(th[t], NULL);
        free(th);
    }
    free(scales); free(q); free(bsums);
    return 0;
}

/* A batch of m rows the way the reference CPU path runs it: one matvec_kq per token. */
ORC_API int orc_matmul_kq(const uint8_t *raw, uint32_t type, size_t n, size_t k, const float *x,
                          size_t m, int threads, float *out) {
    for (size_t t = 0; t < m; t++) {
        int rc = orc_matvec_kq(raw, type, n, k, x + t * k, threads, out + t * n);
        if (rc) return rc;
    }
    return 0;
}

/* ---------------------------------------------------------------- MoE
 * Router: crates/ojas-cuda/src/kernels/moe.rs:45-70 — softmax over E logits, KSEL
 * arg-max passes (ties -> lowest index), weights renormalised over the picks. */
ORC_API void orc_moe_topk(const float *lg, int E, int ksel, uint32_t *idx, float *wgt) {
    float *pr = (float *)malloc((size_t)E * sizeof(float));
    float mx = -1e30f;
    for (int e = 0; e < E; e++) mx = fmaxf(mx, lg[e]);
    float sum = 0.0f;
    for (int e = 0; e < E; e++) { pr[e] = expf(lg[e] - mx); sum += pr[e]; }
    float wsum = 0.0f;
    for (int j = 0; j < ksel; j++) {
        float bv = -1.0f; int bi = 0;
        for (int e = 0; e < E; e++) if (pr[e] > bv) { bv = pr[e]; bi = e; }
        idx[j] = (uint32_t)bi;
        wgt[j] = bv / sum;
        wsum += bv / sum;
        pr[bi] = -1.0f;
    }
    for (int j = 0; j < ksel; j++) wgt[j] = wgt[j] / wsum;
    free(pr);
}

static inline float silu(float x) { return x / (1.0f + expf(-x)); } /* cpu_math.rs:486 */

/* rmsnorm (crates/ojas-cpu/src/cpu_math.rs:456-460): ss = (sum of v*v in index order) / n, inv = 1 / sqrt(ss + eps),
 * out = (a * inv) * b. */
ORC_API void orc_rmsnorm(const float *x, const float *w, size_t n, float eps, float *out) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; i++) ss += x[i] * x[i];
    ss = ss / (float)n;
    const float inv = 1.0f / sqrtf(ss + eps);
    for (size_t i = 0; i < n; i++) out[i] = x[i] * inv * w[i];
}

/* act = silu(g) * u, the SwiGLU step between the expert matmuls (crates/ojas-cpu/src/cpu_glm.rs:575). */
ORC_API void orc_silu_mul(const float *g, const float *u, size_t n, float *out) {
    for (size_t i = 0; i < n; i++) out[i] = silu(g[i]) * u[i];
}

/* Expert FFN for m tokens the way the CPU path runs it
 * (crates/ojas-cpu/src/cpu_glm.rs:551-582): per token, per pick j: three
 * matvec_kq (gate, up over h; down over act) and out += wgt * down.  Experts are
 * stacked: gate/up [E*ffn, d], down [E*d, ffn].  out is overwritten. */
ORC_API int orc_moe_ffn(const uint8_t *wg, const uint8_t *wu, const uint8_t *wd,
                        uint32_t type_gu, uint32_t type_d, const float *h, const uint32_t *idx,
                        const float *wgt, size_t m, int ksel, size_t d, size_t ffn, int threads,
                        float *out) {
    size_t rb_gu = orc_row_bytes(type_gu, d), rb_d = orc_row_bytes(type_d, ffn);
    if (!rb_gu || !rb_d) return -1;
    float *gv = (float *)malloc(ffn * sizeof(float));
    float *uv = (float *)malloc(ffn * sizeof(float));
    float *dv = (float *)malloc(d * sizeof(float));
    if (!gv || !uv || !dv) { free(gv); free(uv); free(dv); return -2; }
    int rc = 0;
    for (size_t t = 0; t < m && !rc; t++) {
        float *o = out + t * d;
        for (size_t i = 0; i < d; i++) o[i] = 0.0f;
        for (int j = 0; j < ksel && !rc; j++) {
            size_t e = idx[t * (size_t)ksel + j];
            float w = wgt[t * (size_t)ksel + j];
            rc |= orc_matvec_kq(wg + e * ffn * rb_gu, type_gu, ffn, d, h + t * d, threads, gv);
            rc |= orc_matvec_kq(wu + e * ffn * rb_gu, type_gu, ffn, d, h + t * d, threads, uv);
            for (size_t i = 0; i < ffn; i++) gv[i] = silu(gv[i]) * uv[i];
            rc |= orc_matvec_kq(wd + e * d * rb_d, type_d, d, ffn, gv, threads, dv);
            for (size_t i = 0; i < d; i++) o[i] += w * dv[i];
        }
    }
    free(gv); free(uv); free(dv);
    return rc;
}

/* Test vector generator of the reference's GPU conformance tests
 * (crates/ojas-cuda/tests/conformance.rs:223-231). */
ORC_API void orc_tvec(size_t n, uint32_t seed, float *out) {
    uint32_t s = seed * 2654435761u + 1u;
    for (size_t i = 0; i < n; i++) {
        s = s * 1664525u + 1013904223u;
        out[i] = (float)(s >> 9) / (float)(1 << 23) - 1.0f;
    }
}
