// Tensor-parallel shard planning for the quantized matmul (host side only).
//
// The engine has no multi-GPU path; these helpers define one for its [N, K] weights:
//   column-parallel: rank r owns weight rows [row0, row0 + rows) -> it produces y[:, row0 .. row0+rows);
//                    shards are joined by an all-gather.  Every output element is computed exactly as
//                    on one GPU.
//   row-parallel:    rank r owns the K range [k0, k0 + klen), a whole number of 256-weight super-blocks
//                    (Q8_K activation scales are per super-block, so each rank quantizes its own slice
//                    of x and every integer block dot is the one a single GPU would form); partial
//                    results are joined by an all-reduce (sum), which changes only the fp32 summation
//                    order across ranks.
#include "common.cuh"

extern "C" int ojas_b200_tp_shard_rows(size_t N, int world, int rank, size_t *row0, size_t *rows) {
    if (!row0 || !rows || world < 1 || rank < 0 || rank >= world) return OJAS_B200_E_ARG;
    const size_t base = N / (size_t)world, rem = N % (size_t)world;
    *row0 = (size_t)rank * base + ((size_t)rank < rem ? (size_t)rank : rem);
    *rows = base + ((size_t)rank < rem ? 1 : 0);
    return 0;
}

extern "C" int ojas_b200_tp_shard_k(size_t K, int world, int rank, size_t *k0, size_t *klen) {
    if (!k0 || !klen || world < 1 || rank < 0 || rank >= world || K % 256 != 0) return OJAS_B200_E_ARG;
    size_t sb0, nsb;
    int rc = ojas_b200_tp_shard_rows(K / 256, world, rank, &sb0, &nsb);
    if (rc) return rc;
    *k0 = sb0 * 256;
    *klen = nsb * 256;
    return 0;
}

// Copies the K range [k0, k0 + klen) of every row of raw GGUF blocks [N, K] into out [N, klen].
extern "C" int ojas_b200_tp_slice_k_host(uint32_t type, const void *raw, size_t N, size_t K, size_t k0, size_t klen, void *out) {
    if (!raw || !out || K % 256 != 0 || k0 % 256 != 0 || klen % 256 != 0 || k0 + klen > K) return OJAS_B200_E_ARG;
    const size_t per256 = type == OJAS_B200_Q4_K ? 144 : type == OJAS_B200_Q6_K ? 210 : type == OJAS_B200_Q8_0 ? 272 : 0;
    if (!per256) return OJAS_B200_E_ARG;
    const size_t row_in = K / 256 * per256, row_out = klen / 256 * per256, skip = k0 / 256 * per256;
    for (size_t r = 0; r < N; r++) memcpy((uint8_t *)out + r * row_out, (const uint8_t *)raw + r * row_in + skip, row_out);
    return 0;
}
