// Load-time re-layout of GGUF blocks into the row-interleaved tiles the kernels read (the layout is
// described in common.cuh).  Replaces the upload decisions of Repr / Lin::load_as
// (crates/ojas-cuda/src/qwen35.rs:146-226); unlike relayout_q4k_q4l
// (crates/ojas-formats/src/quant.rs:192-222) nothing is rounded: every GGUF bit survives.
// The same per-block routine runs on the device (one thread per 256 weights of one row) and on the host.
#include "common.cuh"

// Destination of 16-byte piece p of row r inside a tile.
__host__ __device__ static inline uint8_t *tile_piece(uint8_t *tile, int p, int r) { return tile + (p * OJAS_TILE_ROWS + r) * 16; }

// Q4_K: the 128 nibble bytes keep their GGUF order (eight pieces), the 16-byte block header is piece 8.
__host__ __device__ static inline void repack_q4k_block(const uint8_t *src, uint8_t *tile, int r) {
    for (int p = 0; p < 8; p++)
        for (int i = 0; i < 16; i++) tile_piece(tile, p, r)[i] = src[16 + p * 16 + i];
    for (int i = 0; i < 16; i++) tile_piece(tile, 8, r)[i] = src[i];
}

// Q5_K: Q4_K's pieces (the nibbles start 48 bytes into the block), then the 32 bytes of fifth bits as two pieces.
__host__ __device__ static inline void repack_q5k_block(const uint8_t *src, uint8_t *tile, int r) {
    for (int p = 0; p < 8; p++)
        for (int i = 0; i < 16; i++) tile_piece(tile, p, r)[i] = src[48 + p * 16 + i];
    for (int i = 0; i < 16; i++) tile_piece(tile, 8, r)[i] = src[i];
    for (int p = 0; p < 2; p++)
        for (int i = 0; i < 16; i++) tile_piece(tile, 9 + p, r)[i] = src[16 + p * 16 + i];
}

// Six-bit value of weight w (0..255) of a Q6_K block, as the reference decodes it
// (crates/ojas-formats/src/gguf.rs:1086-1108): half = w/128, quarter = (w%128)/32, l = w%32.
__host__ __device__ static inline unsigned q6k_value(const uint8_t *src, int w) {
    const int hh = w >> 7, quarter = (w >> 5) & 3, l = w & 31;
    const uint8_t *ql = src + hh * 64, *qh = src + 128 + hh * 32;
    const unsigned nib = (quarter & 1) ? ql[l + 32] : ql[l];
    const unsigned lo4 = (quarter & 2) ? (nib >> 4) : (nib & 0xFu);
    const unsigned hi2 = (qh[l] >> (2 * quarter)) & 3u;
    return lo4 | (hi2 << 4);
}

// Q6_K: low nibbles regrouped per 64-weight chunk c (piece h*4 + c), top bits per chunk (piece 8 + c, field t =
// sub-block 4c + t), the sixteen int8 scales (piece 12), then d.
__host__ __device__ static inline void repack_q6k_block(const uint8_t *src, uint8_t *tile, int r) {
    for (int c = 0; c < 4; c++) {
        for (int h = 0; h < 2; h++)
            for (int i = 0; i < 16; i++) {
                const unsigned a = q6k_value(src, 64 * c + 16 * h + i) & 0xFu;
                const unsigned b = q6k_value(src, 64 * c + 32 + 16 * h + i) & 0xFu;
                tile_piece(tile, h * 4 + c, r)[i] = (uint8_t)(a | (b << 4));
            }
        for (int b = 0; b < 16; b++) {
            unsigned v = 0;
            for (int t = 0; t < 4; t++) v |= (q6k_value(src, 64 * c + 16 * t + b) >> 4) << (2 * t);
            tile_piece(tile, 8 + c, r)[b] = (uint8_t)v;
        }
    }
    for (int i = 0; i < 16; i++) tile_piece(tile, 12, r)[i] = src[192 + i];
    tile[13 * 128 + 2 * r] = src[208];
    tile[13 * 128 + 2 * r + 1] = src[209];
}

// Q8_0: eight GGUF blocks (34 bytes each) = 256 weights: int8 values in natural order, then the eight scales.
__host__ __device__ static inline void repack_q80_block(const uint8_t *src, uint8_t *tile, int r) {
    for (int b = 0; b < 8; b++) {
        const uint8_t *blk = src + b * 34;
        for (int i = 0; i < 32; i++) tile_piece(tile, 2 * b + (i >> 4), r)[i & 15] = blk[2 + i];
        tile_piece(tile, 16, r)[2 * b] = blk[0];
        tile_piece(tile, 16, r)[2 * b + 1] = blk[1];
    }
}

// IQ4_XS: the 128 index bytes as eight pieces (piece g = sub-block g), then the block's eight header bytes per row.
__host__ __device__ static inline void repack_iq4xs_block(const uint8_t *src, uint8_t *tile, int r) {
    for (int p = 0; p < 8; p++)
        for (int i = 0; i < 16; i++) tile_piece(tile, p, r)[i] = src[8 + p * 16 + i];
    for (int i = 0; i < 8; i++) tile[8 * 128 + 8 * r + i] = src[i];
}

// IQ4_NL: eight GGUF blocks (18 bytes each) = 256 weights: the index bytes of block b as piece b, then the eight scales.
__host__ __device__ static inline void repack_iq4nl_block(const uint8_t *src, uint8_t *tile, int r) {
    for (int b = 0; b < 8; b++) {
        const uint8_t *blk = src + b * 18;
        for (int i = 0; i < 16; i++) tile_piece(tile, b, r)[i] = blk[2 + i];
        tile_piece(tile, 8, r)[2 * b] = blk[0];
        tile_piece(tile, 8, r)[2 * b + 1] = blk[1];
    }
}

__host__ __device__ static inline size_t raw_sb_bytes(uint32_t type) {
    return type == OJAS_B200_Q4_K ? 144 : type == OJAS_B200_Q5_K ? 176 : type == OJAS_B200_Q6_K ? 210 : type == OJAS_B200_IQ4_XS ? 136 : type == OJAS_B200_IQ4_NL ? 144 : 272;
}

// Block `blk` = (row n, super-block s) in row-major order of the GGUF tensor.
__host__ __device__ static inline void repack_one(uint32_t type, const uint8_t *raw, size_t blk, size_t nsb, uint8_t *out) {
    const size_t n = blk / nsb, s = blk - n * nsb;
    const uint8_t *src = raw + blk * raw_sb_bytes(type);
    uint8_t *tile = out + ((n / OJAS_TILE_ROWS) * nsb + s) * (size_t)tile_bytes(type);
    const int r = (int)(n % OJAS_TILE_ROWS);
    if (type == OJAS_B200_Q4_K) repack_q4k_block(src, tile, r);
    else if (type == OJAS_B200_Q5_K) repack_q5k_block(src, tile, r);
    else if (type == OJAS_B200_Q6_K) repack_q6k_block(src, tile, r);
    else if (type == OJAS_B200_IQ4_XS) repack_iq4xs_block(src, tile, r);
    else if (type == OJAS_B200_IQ4_NL) repack_iq4nl_block(src, tile, r);
    else repack_q80_block(src, tile, r);
}

__global__ void repack_kernel(uint32_t type, const uint8_t *raw, size_t nblocks, size_t nsb, uint8_t *out) {
    const size_t blk = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (blk < nblocks) repack_one(type, raw, blk, nsb, out);
}

extern "C" size_t ojas_b200_raw_bytes(uint32_t type, size_t N, size_t K) { return type_supported(type) ? N * (K / 256) * raw_sb_bytes(type) : 0; }

extern "C" size_t ojas_b200_repacked_bytes(uint32_t type, size_t N, size_t K) {
    if (K % 256 != 0 || !type_supported(type)) return 0;
    return repacked_size(type, N, K);
}

extern "C" int ojas_b200_repack(ojas_b200_ctx *ctx, uint32_t type, const void *raw_dev, size_t N, size_t K, void *out_dev) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!raw_dev || !out_dev) return ojas_fail(ctx, OJAS_B200_E_ARG, "repack: null pointer");
    if (K == 0 || K % 256 != 0 || N == 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "repack: N=%zu K=%zu (K must be a positive multiple of 256)", N, K);
    if (!ojas_b200_repacked_bytes(type, N, K)) return ojas_fail(ctx, OJAS_B200_E_ARG, "repack: unsupported GGUF type %u", type);
    if (((uintptr_t)out_dev & 255) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "repack: output must be 256-byte aligned");
    const size_t nb = N * (K / 256);
    const size_t grid = (nb + 127) / 128;
    if (grid > 0x7fffffffu) return ojas_fail(ctx, OJAS_B200_E_ARG, "repack: tensor too large for one launch");
    if (N % OJAS_TILE_ROWS != 0)   // the rows that pad the last unit must read as zero blocks
        OJAS_CUDA(ctx, cudaMemsetAsync((uint8_t *)out_dev + (N / OJAS_TILE_ROWS) * (K / 256) * (size_t)tile_bytes(type), 0,
                                       (K / 256) * (size_t)tile_bytes(type), ctx->stream));
    repack_kernel<<<(unsigned)grid, 128, 0, ctx->stream>>>(type, (const uint8_t *)raw_dev, nb, K / 256, (uint8_t *)out_dev);
    OJAS_LAUNCH_CHECK(ctx, "repack");
    return 0;
}

extern "C" int ojas_b200_repack_host(uint32_t type, const void *raw_host, size_t N, size_t K, void *out_host) {
    if (!raw_host || !out_host || K == 0 || K % 256 != 0 || !ojas_b200_repacked_bytes(type, N, K)) return OJAS_B200_E_ARG;
    memset(out_host, 0, ojas_b200_repacked_bytes(type, N, K));
    const size_t nb = N * (K / 256);
    for (size_t b = 0; b < nb; b++) repack_one(type, (const uint8_t *)raw_host, b, K / 256, (uint8_t *)out_host);
    return 0;
}
