// Load-time re-layout of GGUF blocks into the aligned planes the kernels read (layouts are
// described beside WeightPlanes).  Replaces the upload decisions of Repr / Lin::load_as
// (crates/ojas-cuda/src/qwen35.rs:146-226); unlike relayout_q4k_q4l
// (crates/ojas-formats/src/quant.rs:192-222) nothing is rounded: every GGUF bit survives.
// The same per-block routine runs on the device (one thread per block) and on the host.
#include "common.cuh"

struct PlanePtrs { uint8_t *p0, *p1, *p2, *p3; };

// Q4_K block `blk` (row-major block index): GGUF 144 bytes -> 128 nibble bytes + 16 header bytes.
__host__ __device__ static inline void repack_q4k_block(const uint8_t *raw, size_t blk, PlanePtrs o) {
    const uint8_t *src = raw + blk * 144;
    uint8_t *qs = o.p0 + blk * 128, *hdr = o.p1 + blk * 16;
    for (int i = 0; i < 4; i++) hdr[i] = src[i];
    const uint8_t *sc = src + 4;
    for (int c = 0; c < 4; c++) {
        unsigned v[4];   // s(2c), s(2c+1), m(2c), m(2c+1) by the GGUF rule (crates/ojas-formats/src/gguf.rs:1132-1140)
        for (int h = 0; h < 2; h++) {
            const int j = 2 * c + h;
            if (j < 4) { v[h] = sc[j] & 63u; v[2 + h] = sc[j + 4] & 63u; }
            else { v[h] = (sc[j + 4] & 0xFu) | ((unsigned)(sc[j - 4] >> 6) << 4); v[2 + h] = (unsigned)(sc[j + 4] >> 4) | ((unsigned)(sc[j] >> 6) << 4); }
        }
        const unsigned g = v[0] | (v[1] << 6) | (v[2] << 12) | (v[3] << 18);
        hdr[4 + 3 * c] = (uint8_t)(g & 0xff);
        hdr[5 + 3 * c] = (uint8_t)((g >> 8) & 0xff);
        hdr[6 + 3 * c] = (uint8_t)((g >> 16) & 0xff);
    }
    for (int c = 0; c < 4; c++)
        for (int h = 0; h < 2; h++)
            for (int i = 0; i < 16; i++) qs[h * 64 + c * 16 + i] = src[16 + c * 32 + h * 16 + i];
}

// Q6_K block: GGUF 210 bytes (ql[128], qh[64], sc[16], d) -> lo[128], hi[64], sc[16], d[2].
// Six-bit value of weight w (0..255), as the reference decodes it
// (crates/ojas-formats/src/gguf.rs:1086-1108): half = w/128, quarter = (w%128)/32, l = w%32.
__host__ __device__ static inline unsigned q6k_value(const uint8_t *src, int w) {
    const int hh = w >> 7, quarter = (w >> 5) & 3, l = w & 31;
    const uint8_t *ql = src + hh * 64, *qh = src + 128 + hh * 32;
    const unsigned nib = (quarter & 1) ? ql[l + 32] : ql[l];
    const unsigned lo4 = (quarter & 2) ? (nib >> 4) : (nib & 0xFu);
    const unsigned hi2 = (qh[l] >> (2 * quarter)) & 3u;
    return lo4 | (hi2 << 4);
}

__host__ __device__ static inline void repack_q6k_block(const uint8_t *raw, size_t blk, PlanePtrs o) {
    const uint8_t *src = raw + blk * 210;
    uint8_t *lo = o.p0 + blk * 128, *hi = o.p1 + blk * 64, *sc = o.p2 + blk * 16, *d = o.p3 + blk * 2;
    for (int c = 0; c < 4; c++) {
        for (int h = 0; h < 2; h++)
            for (int i = 0; i < 16; i++) {
                const unsigned a = q6k_value(src, 64 * c + 16 * h + i) & 0xFu;
                const unsigned b = q6k_value(src, 64 * c + 32 + 16 * h + i) & 0xFu;
                lo[h * 64 + c * 16 + i] = (uint8_t)(a | (b << 4));
            }
        for (int k = 0; k < 4; k++)
            for (int i = 0; i < 4; i++) {
                unsigned v = 0;
                for (int t = 0; t < 4; t++) v |= (q6k_value(src, 64 * c + 16 * t + 4 * k + i) >> 4) << (2 * t);
                hi[c * 16 + k * 4 + i] = (uint8_t)v;
            }
    }
    for (int i = 0; i < 16; i++) sc[i] = src[192 + i];
    d[0] = src[208];
    d[1] = src[209];
}

// Q8_0 block of 32 weights: GGUF 34 bytes (d, q[32]) -> q[32], d[2].
__host__ __device__ static inline void repack_q80_block(const uint8_t *raw, size_t blk, PlanePtrs o) {
    const uint8_t *src = raw + blk * 34;
    uint8_t *q = o.p0 + blk * 32, *d = o.p1 + blk * 2;
    d[0] = src[0];
    d[1] = src[1];
    for (int i = 0; i < 32; i++) q[i] = src[2 + i];
}

__global__ void repack_kernel(uint32_t type, const uint8_t *raw, size_t nblocks, PlanePtrs o) {
    const size_t blk = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (blk >= nblocks) return;
    if (type == OJAS_B200_Q4_K) repack_q4k_block(raw, blk, o);
    else if (type == OJAS_B200_Q6_K) repack_q6k_block(raw, blk, o);
    else repack_q80_block(raw, blk, o);
}

static size_t block_count(uint32_t type, size_t N, size_t K) { return type == OJAS_B200_Q8_0 ? N * (K / 32) : N * (K / 256); }

extern "C" size_t ojas_b200_raw_bytes(uint32_t type, size_t N, size_t K) {
    switch (type) {
    case OJAS_B200_Q4_K: return N * (K / 256) * 144;
    case OJAS_B200_Q6_K: return N * (K / 256) * 210;
    case OJAS_B200_Q8_0: return N * (K / 256) * 272;
    default: return 0;
    }
}

extern "C" size_t ojas_b200_repacked_bytes(uint32_t type, size_t N, size_t K) {
    size_t off[5];
    if (K % 256 != 0 || plane_offsets(type, N, K, off)) return 0;
    return off[4];
}

static PlanePtrs plane_ptrs(uint32_t type, void *out, size_t N, size_t K) {
    size_t off[5];
    plane_offsets(type, N, K, off);
    uint8_t *b = (uint8_t *)out;
    return PlanePtrs{b + off[0], b + off[1], b + off[2], b + off[3]};
}

extern "C" int ojas_b200_repack(ojas_b200_ctx *ctx, uint32_t type, const void *raw_dev, size_t N, size_t K, void *out_dev) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!raw_dev || !out_dev) return ojas_fail(ctx, OJAS_B200_E_ARG, "repack: null pointer");
    if (K == 0 || K % 256 != 0 || N == 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "repack: N=%zu K=%zu (K must be a positive multiple of 256)", N, K);
    if (!ojas_b200_repacked_bytes(type, N, K)) return ojas_fail(ctx, OJAS_B200_E_ARG, "repack: unsupported GGUF type %u", type);
    if (((uintptr_t)out_dev & 255) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "repack: output must be 256-byte aligned");
    const size_t nb = block_count(type, N, K);
    const size_t grid = (nb + 127) / 128;
    if (grid > 0x7fffffffu) return ojas_fail(ctx, OJAS_B200_E_ARG, "repack: tensor too large for one launch");
    repack_kernel<<<(unsigned)grid, 128, 0, ctx->stream>>>(type, (const uint8_t *)raw_dev, nb, plane_ptrs(type, out_dev, N, K));
    OJAS_LAUNCH_CHECK(ctx, "repack");
    return 0;
}

extern "C" int ojas_b200_repack_host(uint32_t type, const void *raw_host, size_t N, size_t K, void *out_host) {
    if (!raw_host || !out_host || K == 0 || K % 256 != 0 || !ojas_b200_repacked_bytes(type, N, K)) return OJAS_B200_E_ARG;
    memset(out_host, 0, ojas_b200_repacked_bytes(type, N, K));
    const size_t nb = block_count(type, N, K);
    PlanePtrs o = plane_ptrs(type, out_host, N, K);
    const uint8_t *raw = (const uint8_t *)raw_host;
    for (size_t b = 0; b < nb; b++) {
        if (type == OJAS_B200_Q4_K) repack_q4k_block(raw, b, o);
        else if (type == OJAS_B200_Q6_K) repack_q6k_block(raw, b, o);
        else repack_q80_block(raw, b, o);
    }
    return 0;
}
