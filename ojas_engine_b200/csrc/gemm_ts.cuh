// The prefill GEMM with the dequantized weight tiles in tensor memory (included by gemm_tc.cu).
//
// tcgen05.mma takes its A operand either from shared memory or from TMEM.  Here the dequantizing warps
// write the f16 weight tile straight into TMEM (tcgen05.st: lane = weight row, one 32-bit column = two
// consecutive k), so shared memory holds only the activation tiles and the raw weight tiles.  That buys
// ring depth, which is what the pipeline needs: a stage passes through three hand-offs (MMA done ->
// dequantizer, dequantizer -> MMA thread, MMA thread -> tensor pipe), each several hundred cycles, and a
// four-deep ring of 512-cycle stages cannot cover them.
//   TMEM columns   0..255  accumulator(s): one of 256 tokens, or two of <= 128 tokens
//   TMEM columns 256..511  eight A stages of 128 rows x 64 k (32 columns each) = two super-blocks
//   shared memory          4-8 activation stages (BN tokens x 64 k, by TMA) + three raw Q4_K / Q6_K tiles + staging
// Work is cut "stream-K" style: the (tile, super-block) pairs are numbered tile-major and CTA b takes the
// b-th share of equal cost of that list, so every SM gets the same work whatever the tile count.  A tile
// whose K range is split across CTAs is combined without zeroing y: the piece that ends the K range stores
// and marks the tile, the other pieces wait for the mark and add (see the epilogue); without marks (forced
// split, grouped form, y not addressable by TMA) the pieces add into a y the host has zeroed.
// Grouped form (expert FFN): the row count and first row of the group are read from device memory.
#pragma once

constexpr int TS_A_STAGES = 8;
constexpr int TS_A_COL0 = 256;
constexpr int TS_EPI_WARPS = 8;                      // warps 0-7: epilogue (lane quarter = warp % 4)
constexpr int TS_WARP_DEQ0 = TS_EPI_WARPS;                        // warps 8-23: four dequantizing groups
constexpr int TS_WARP_TMA_X = TS_WARP_DEQ0 + 16;
constexpr int TS_WARP_MMA0 = TS_WARP_TMA_X + 1;                   // warps 25-28: MMA issue, thread c owns chunk c
constexpr int TS_WARP_TMA_W = TS_WARP_MMA0 + 4;                   // warp 29: raw-tile TMA, owns the TMEM allocation
constexpr int TS_THREADS = (TS_WARP_TMA_W + 1) * 32;              // 960
constexpr int TS_BAR_BYTES = 512;
constexpr int TS_EPI_TILE_BYTES = 16 * 32 * 4;                    // per epilogue warp: 16 tokens x 32 weight rows, fp32
constexpr int TS_SMEM_BUDGET = 232448 - 1024 - TS_BAR_BYTES - TS_EPI_WARPS * TS_EPI_TILE_BYTES;   // 227 KB minus slack, barriers, staging

__host__ __device__ constexpr int ts_b_stages(int bn, int type) {
    const int s = (TS_SMEM_BUDGET - wq_bufs(type) * wq_bytes(type)) / (bn * BK * 2);
    return s > 8 ? 8 : s;
}

// ---------------------------------------------------------------- work list
struct TsPiece { int tile, n0, m0, sb0, sb1; bool partial; };

// Balanced split.  Every piece of work ends with a drain of the accumulator that the main loop cannot hide when
// there is a single accumulator, so the list is cut at equal *cost*: a super-block costs 2 units, the end of a
// tile e2 units (the drain of a 128 x 256 tile takes about as long as 2.5 super-blocks).  Returns the first
// (tile, super-block) index of share b out of `shares`.
__host__ __device__ inline long long ts_share_begin(long long n_tiles, int nsb, int e2, long long b, long long shares) {
    const long long per_tile = 2LL * nsb + e2;
    const long long t = n_tiles * per_tile * b / shares;
    const long long q = t / per_tile, r = t - q * per_tile;
    return q * nsb + (r < 2LL * nsb ? r / 2 : nsb);
}

struct TsSched {
    long long g, g_end;        // balanced mode: next / one-past-last (tile, super-block) index of this CTA
    int p, p_end, stride;      // forced-split mode: next piece index
    int n_tiles_n, nsb, ksplit, bn, n_tiles;

    __device__ TsSched(const GemmArgs &a, int bn_) {
        bn = bn_;
        nsb = a.K >> 8;
        n_tiles_n = (a.N + BM - 1) / BM;
        n_tiles = n_tiles_n * ((a.M + bn - 1) / bn);
        ksplit = a.ksplit;
        g = ts_share_begin(n_tiles, nsb, a.e2, blockIdx.x, gridDim.x);
        g_end = ts_share_begin(n_tiles, nsb, a.e2, blockIdx.x + 1, gridDim.x);
        p = blockIdx.x;
        p_end = n_tiles * (ksplit > 0 ? ksplit : 1);
        stride = gridDim.x;
    }
    __device__ bool next(TsPiece &pc) {
        int tile;
        if (ksplit == 0) {
            if (g >= g_end) return false;
            tile = (int)(g / nsb);
            pc.sb0 = (int)(g - (long long)tile * nsb);
            const long long left = g_end - g;
            pc.sb1 = left < (long long)(nsb - pc.sb0) ? pc.sb0 + (int)left : nsb;
            g += pc.sb1 - pc.sb0;
            pc.partial = (pc.sb1 - pc.sb0) < nsb;
        } else {
            for (;;) {
                if (p >= p_end) return false;
                tile = p % n_tiles;
                const int kz = p / n_tiles;
                p += stride;
                pc.sb0 = (int)((long long)nsb * kz / ksplit);
                pc.sb1 = (int)((long long)nsb * (kz + 1) / ksplit);
                if (pc.sb1 > pc.sb0) break;
            }
            pc.partial = ksplit > 1;
        }
        pc.tile = tile;
        pc.n0 = (tile % n_tiles_n) * BM;
        pc.m0 = (tile / n_tiles_n) * bn;
        return true;
    }
};

// ---------------------------------------------------------------- tcgen05 forms used only here
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc) : "memory");
}

// Atomic add without a return value: nothing comes back, so the epilogue does not wait a round trip to L2.
__device__ __forceinline__ void red_add_f32(float *p, float v) {
    asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

// Bounded wait for a tile's "stored" mark (written by another CTA that is resident at the same time: the grid
// never exceeds one CTA per SM, and the marking piece is the first thing its CTA does).
__device__ __noinline__ bool flag_wait(const unsigned *flag, unsigned serial, volatile int *abort_flag, unsigned *status) {
    const long long t0 = clock64();
    for (;;) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v == serial) return true;
        __nanosleep(100);
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CYCLES) {
            *abort_flag = 1;
            atomicOr(status, 0x20000u);
            __threadfence_system();
            return false;
        }
    }
}

// Tile [rows of 32 floats] from shared memory into the 2-D tensor behind `tmap` at (x, y): plain store, or add.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *tmap, const void *smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"((uint64_t)tmap), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *tmap, const void *smem_src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"((uint64_t)tmap), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}

// 16 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&o)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]),
                   "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15]) : "memory");
}

// ---------------------------------------------------------------- the kernel
template <int BN, int TYPE>
__global__ void __launch_bounds__(TS_THREADS, 1) gemm_ts_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                 const __grid_constant__ CUtensorMap tmap_w,
                                                                 const __grid_constant__ CUtensorMap tmap_y, const GemmArgs a_in) {
    GemmArgs a = a_in;
    int x_row0 = 0;                                          // first activation row (grouped form: the group's offset)
    if (a_in.grp_count) {
        grid_dependency_wait();                              // the counts come from a kernel before this one
        a.M = __ldg(a_in.grp_count);
        x_row0 = __ldg(a_in.grp_offset);
        a.y = a_in.y + (size_t)x_row0 * a_in.N;
    }
    extern __shared__ unsigned char gemm_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)gemm_smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int B_STAGE_BYTES = BN * BK * 2;
    constexpr int WQ_BYTES = wq_bytes(TYPE), WQ_BUFS = wq_bufs(TYPE);   // raw tiles arrive by TMA, one super-block at a time
    constexpr bool STAGED_W = true;
    constexpr int BS = ts_b_stages(BN, TYPE);
    constexpr int NACC = BN <= 128 ? 2 : 1;
    static_assert(BS >= 4 && BS <= 8, "activation ring depth");
    unsigned char *smem_b = smem;
    unsigned char *smem_wq = smem_b + BS * B_STAGE_BYTES;
    unsigned char *smem_epi = smem_wq + WQ_BUFS * WQ_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_epi + TS_EPI_WARPS * TS_EPI_TILE_BYTES);
    uint64_t *a_full = bars, *a_empty = bars + 8, *b_full = bars + 16, *b_empty = bars + 24;
    uint64_t *wq_full = bars + 32, *wq_empty = wq_full + WQ_BUFS_MAX;
    uint64_t *tmem_full = wq_empty + WQ_BUFS_MAX, *tmem_empty = tmem_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile unsigned *b_seen = reinterpret_cast<volatile unsigned *>(tmem_slot + 2);   // [4], see the MMA threads
    unsigned *epi_done = reinterpret_cast<unsigned *>(tmem_slot + 6);                   // epilogue warps that finished a storing piece

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = a.K >> 8;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TS_A_STAGES; s++) {
            mbar_init(&a_full[s], 4);                         // the four warps of the stage's group
            mbar_init(&a_empty[s], 1);
            mbar_init(&b_full[s], 1);
            mbar_init(&b_empty[s], 1);
        }
        for (int b = 0; b < WQ_BUFS; b++) {
            mbar_init(&wq_full[b], 1);
            mbar_init(&wq_empty[b], 16);                     // every dequantizing warp
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 4);                     // one commit per MMA-issuing thread
            mbar_init(&tmem_empty[b], TS_EPI_WARPS);
        }
        *abort_flag = 0;
        for (int i = 0; i < 4; i++) b_seen[i] = 0u;
        *epi_done = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TS_WARP_TMA_X && lane == 0) {              // the descriptors' first use would otherwise pay their fetch
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmap_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmap_w) : "memory");
        if (a.y_tma) asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmap_y) : "memory");
    }
    if (warp == TS_WARP_TMA_W) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // several threads issue MMAs into one accumulator, so every MMA accumulates and the accumulators start
    // from zero (here, and again after each drain)
    if (warp < 4) {
        for (int col = 0; col < NACC * BN; col += 32) tmem_zero32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)col);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    TsSched sched(a, BN);
    TsPiece pc;

    if (warp < TS_EPI_WARPS) {
        // ---------------- epilogue: warp e drains TMEM lanes 32 (e % 4) .. +31 (weight rows), column half e / 4
        const int quarter = warp & 3, chalf = warp >> 2;
        constexpr bool SPLIT = TS_EPI_WARPS == 8 && BN >= 64;     // two warps per lane quarter share the columns
        constexpr int ECOLS = SPLIT ? BN / 2 : BN;
        const int col_begin = SPLIT ? chalf * ECOLS : 0, col_end = (SPLIT || chalf == 0) ? col_begin + ECOLS : 0;
        float *epi_tile = reinterpret_cast<float *>(smem_epi + warp * TS_EPI_TILE_BYTES);
        // The value that marks a tile as stored in this launch: a device word that the activation-preparation kernel
        // in front of this one advances on every launch (so a replayed CUDA graph gets a fresh value each time).
        unsigned serial = 0u;
        if (a.flags) {
            grid_dependency_wait();
            serial = *reinterpret_cast<volatile const unsigned *>(a.serial_word);
        }
        for (int it = 0; sched.next(pc); it++) {
            const int acc = it % NACC, use = it / NACC;
            if (!mbar_wait_warp_long(&tmem_full[acc], (uint32_t)use & 1u, abort_flag, a.status, 0x400u)) break;
            tc_fence_after();
            const int n = pc.n0 + quarter * 32 + lane;
            float *ycol = a.y + n;
            if (a.y_tma) {
                // 16 tokens at a time through this warp's 2 KB staging tile [16 tokens][32 rows] and one bulk
                // tensor store (or reduce-add) per tile: the copy engine clips the tile at the edges of y and
                // keeps many more bytes in flight than a warp's own stores can
                const int xn = pc.n0 + quarter * 32;
                // split tile with marks: the piece that ends the tile's K range stores, the others add after its mark
                const bool marks = pc.partial && a.flags != nullptr;
                const bool storer = marks && pc.sb1 == nsb;
                const bool add = (pc.partial && !storer) || a.accum;
                if (marks && !storer) {
                    int ok = 1;
                    if (lane == 0) ok = flag_wait(a.flags + pc.tile, serial, abort_flag, a.status) ? 1 : 0;
                    if (!__shfl_sync(0xffffffffu, ok, 0)) break;
                    asm volatile("fence.proxy.async;" ::: "memory");
                }
#pragma unroll 1
                for (int col = col_begin; col < col_end; col += 32) {
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN + col);
                    if (pc.m0 + col < a.M && xn < a.N) {
                        uint32_t v[32];
                        tmem_ld32(taddr, v);
#pragma unroll
                        for (int h = 0; h < 2; h++) {            // two staging rounds of 16 tokens
                            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the tile before has left
                            __syncwarp();
#pragma unroll
                            for (int j = 0; j < 16; j++) epi_tile[j * 32 + lane] = __uint_as_float(v[16 * h + j]);
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            __syncwarp();
                            if (lane == 0 && pc.m0 + col + 16 * h < a.M) {
                                if (add) tma_reduce_add_2d(&tmap_y, epi_tile, xn, pc.m0 + col + 16 * h);
                                else tma_store_2d(&tmap_y, epi_tile, xn, pc.m0 + col + 16 * h);
                                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                            }
                        }
                    }
                }
                // the accumulator is read out: zero this warp's columns in one go
#pragma unroll
                for (int col = 0; col < ECOLS; col += 32)
                    if (col_begin + col < col_end)
                        tmem_zero32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN + col_begin + col));
                if (storer) {
                    // all eight warps' stores have landed -> mark the tile.  Every epilogue warp takes part in every
                    // piece; the warp that finishes last publishes the mark (a count, not a barrier: a warp that left
                    // the loop after an abort cannot leave the others waiting).
                    if (lane == 0) {
                        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                        __threadfence();
                        const unsigned old = atomicAdd(epi_done, 1u);
                        if (old % TS_EPI_WARPS == TS_EPI_WARPS - 1)
                            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.flags + pc.tile), "r"(serial) : "memory");
                    }
                }
            } else {
#pragma unroll 1
                for (int col = col_begin; col < col_end; col += 32) {
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN + col);
                    if (pc.m0 + col < a.M) {
                        uint32_t v[32];
                        tmem_ld32(taddr, v);
                        if (n < a.N) {
                            const int rows = a.M - (pc.m0 + col) < 32 ? a.M - (pc.m0 + col) : 32;
                            float *yp = ycol + (size_t)(pc.m0 + col) * a.N;
                            if (pc.partial) {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    if (j < rows) red_add_f32(yp + (size_t)j * a.N, __uint_as_float(v[j]));
                            } else if (a.accum) {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    if (j < rows) yp[(size_t)j * a.N] += __uint_as_float(v[j]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    if (j < rows) yp[(size_t)j * a.N] = __uint_as_float(v[j]);
                            }
                        }
                    }
                    tmem_zero32(taddr);
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every store has landed before the CTA ends
    } else if (warp < TS_WARP_TMA_X) {
        // ---------------- dequantizers: four groups of four warps; group c owns chunk c of every super-block
        // (A stage (sb & 1) * 4 + c, the stage MMA thread c consumes), thread = weight row: 64 weights -> 32 TMEM
        // columns per stage.  Four stages are in work at once, which is what hides the latency of a stage's
        // own chain (raw tile -> registers -> f16 -> TMEM -> barrier).
        const int c = (warp - TS_WARP_DEQ0) >> 2;
        const int row = ((warp & 3) << 5) + lane;
        const uint32_t tmem_row = tmem_base + ((uint32_t)(row & ~31) << 16) + (uint32_t)TS_A_COL0;
        uint32_t wc = 0;      // running super-block counter
        bool ok = true;
        while (ok && sched.next(pc)) {
            const int grow = pc.n0 + row;
            const bool live = grow < a.N;
            const int lrow = live ? grow : 0;
            constexpr int TB = tile_bytes((uint32_t)TYPE), QB = tile_quant_bytes((uint32_t)TYPE);
            // this row's tile of super-block 0 in global memory, and its place in a staged raw tile
            const uint8_t *grow_tiles = a.w + (size_t)(lrow >> 3) * nsb * TB + (lrow & 7) * 16;
            const int soff = (row >> 3) * QB + (row & 7) * 16;
            const int n_sb = pc.sb1 - pc.sb0;
            // small per-row items come straight from global memory, one super-block ahead: the Q4_K header
            // (d, dmin, scales); the Q6_K chunk's four sub-scales and d; the Q8_0 chunk's two block scales
            uint4 hdr_next = make_uint4(0u, 0u, 0u, 0u);
            auto small_items = [&](int sb) {
                const uint8_t *t = grow_tiles + (size_t)sb * TB;
                if (TYPE == OJAS_B200_Q4_K || TYPE == OJAS_B200_Q5_K) {
                    hdr_next = __ldg(reinterpret_cast<const uint4 *>(t + 8 * 128));
                } else if (TYPE == OJAS_B200_Q6_K) {
                    hdr_next.x = __ldg(reinterpret_cast<const uint32_t *>(t + 12 * 128) + c);
                    hdr_next.y = __ldg(reinterpret_cast<const unsigned short *>(t - (lrow & 7) * 16 + 13 * 128) + (lrow & 7));
                } else if (TYPE == OJAS_B200_IQ4_XS) {    // the block's eight header bytes: d, scales_h | scales_l
                    const uint2 h8 = __ldg(reinterpret_cast<const uint2 *>(t - (lrow & 7) * 16 + 8 * 128 + (lrow & 7) * 8));
                    hdr_next.x = h8.x;
                    hdr_next.y = h8.y;
                } else if (TYPE == OJAS_B200_IQ4_NL) {    // the chunk's two f16 block scales
                    hdr_next.x = __ldg(reinterpret_cast<const uint32_t *>(t + 8 * 128) + c);
                } else {                                  // the chunk's two f16 block scales
                    hdr_next.x = __ldg(reinterpret_cast<const uint32_t *>(t + 16 * 128) + c);
                }
            };
            if (STAGED_W) small_items(pc.sb0);
            uint4 cA = make_uint4(0u, 0u, 0u, 0u), cB = cA, cC = cA, cD = cA;
            uint32_t ce0 = 0, ce1 = 0;
            for (int j = 0; ok && j < n_sb; j++, wc++) {
                const int wb = wc % WQ_BUFS;
                const int aslot = (int)(wc & 1u) * 4 + c;
                const uint4 H = hdr_next;
                if (STAGED_W) {
                    if (j + 1 < n_sb) small_items(pc.sb0 + j + 1);
                    if (!mbar_wait_warp(&wq_full[wb], (wc / WQ_BUFS) & 1u, abort_flag, a.status, 0x2000u)) { ok = false; break; }
                    const unsigned char *wrow = smem_wq + wb * WQ_BYTES + soff;      // piece p of this row: wrow + 128 p
                    if (TYPE == OJAS_B200_Q8_0) {
                        // chunk c = 64 int8: pieces 4c .. 4c + 3
                        cA = *reinterpret_cast<const uint4 *>(wrow + (4 * c + 0) * 128);
                        cB = *reinterpret_cast<const uint4 *>(wrow + (4 * c + 1) * 128);
                        cC = *reinterpret_cast<const uint4 *>(wrow + (4 * c + 2) * 128);
                        cD = *reinterpret_cast<const uint4 *>(wrow + (4 * c + 3) * 128);
                        ce0 = H.x;
                    } else if (TYPE == OJAS_B200_Q4_K || TYPE == OJAS_B200_Q5_K || TYPE == OJAS_B200_IQ4_XS || TYPE == OJAS_B200_IQ4_NL) {
                        cA = *reinterpret_cast<const uint4 *>(wrow + (2 * c) * 128);          // qs[32c .. 32c + 15] (IQ4: the indices of group 2c)
                        cB = *reinterpret_cast<const uint4 *>(wrow + (2 * c + 1) * 128);      // qs[32c + 16 .. 32c + 31]
                        if (TYPE == OJAS_B200_Q5_K) {                                         // the fifth bits of the whole super-block
                            cC = *reinterpret_cast<const uint4 *>(wrow + 9 * 128);
                            cD = *reinterpret_cast<const uint4 *>(wrow + 10 * 128);
                        }
                    } else {
                        cA = *reinterpret_cast<const uint4 *>(wrow + c * 128);                // low nibbles, h = 0
                        cB = *reinterpret_cast<const uint4 *>(wrow + (4 + c) * 128);          // low nibbles, h = 1
                        cC = *reinterpret_cast<const uint4 *>(wrow + (8 + c) * 128);          // top bits
                        ce0 = H.x;
                        ce1 = H.y;
                    }
                }
                uint32_t o[16], o1[16];
                auto convert = [&](int half, uint32_t (&out)[16]) {
                    if (!live) {
#pragma unroll
                        for (int q = 0; q < 16; q++) out[q] = 0u;
                    } else if (TYPE == OJAS_B200_Q4_K) {
                        dequant_q4k_half(cA, cB, H, c, half, out);
                    } else if (TYPE == OJAS_B200_Q5_K) {
                        dequant_q5k_half(cA, cB, cC, cD, H, c, half, out);
                    } else if (TYPE == OJAS_B200_IQ4_XS) {
                        const int g = 2 * c + half;
                        const int ls = (int)(((H.y >> (4 * g)) & 0xFu) | ((((H.x >> 16) >> (2 * g)) & 3u) << 4)) - 32;
                        dequant_iq4_half(half == 0 ? cA : cB, __float2half_rn(f16_bits_to_f32(H.x) * (float)ls), out);
                    } else if (TYPE == OJAS_B200_IQ4_NL) {
                        dequant_iq4_half(half == 0 ? cA : cB, __ushort_as_half((unsigned short)((H.x >> (16 * half)) & 0xffffu)), out);
                    } else if (TYPE == OJAS_B200_Q6_K) {
                        dequant_q6k_half(cA, cB, cC, ce0, ce1, half, out);
                    } else if (half == 0) {
                        dequant_q80_half(cA, cB, ce0, out);
                    } else {
                        dequant_q80_half(cC, cD, ce0 >> 16, out);
                    }
                };
                convert(0, o);
                if (STAGED_W) {                                          // the raw tile is in registers: hand the buffer back
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&wq_empty[wb]);
                }
                if (!mbar_wait_warp(&a_empty[aslot], ((wc >> 1) & 1u) ^ 1u, abort_flag, a.status, 0x100u)) { ok = false; break; }
                tc_fence_after();
                tmem_st16(tmem_row + (uint32_t)(aslot * 32), o);      // (one 32-column store of both halves measured slower)
                convert(1, o1);
                tmem_st16(tmem_row + (uint32_t)(aslot * 32 + 16), o1);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[aslot]);
            }
        }
    } else if (warp == TS_WARP_TMA_X) {
        // ---------------- TMA: activation tile [BN tokens x 64 k] per stage, BS stages in flight
        if (lane == 0) {
            int bslot = 0;
            uint32_t bphase = 0;
            bool ok = true;
            grid_dependency_wait();     // the prepared activations come from the kernel before this one
            while (ok && sched.next(pc)) {
                for (int sb = pc.sb0; ok && sb < pc.sb1; sb++) {
#pragma unroll 1
                    for (int c = 0; c < 4; c++) {
                        if (!mbar_wait_spin(&b_empty[bslot], bphase ^ 1u, abort_flag, a.status, 0x200u)) { ok = false; break; }
                        mbar_arrive_expect_tx(&b_full[bslot], (uint32_t)B_STAGE_BYTES);
                        tma_load_2d(smem_b + bslot * B_STAGE_BYTES, &tmap_x, (sb * 4 + c) * BK, x_row0 + pc.m0, &b_full[bslot]);
                        if (++bslot == BS) { bslot = 0; bphase ^= 1u; }
                    }
                }
            }
        }
    } else if (warp < TS_WARP_TMA_W) {
        // ---------------- MMA issue: thread c owns chunk c of every super-block (A stage (sb & 1) * 4 + c);
        // every MMA accumulates (see the zeroing above)
        if (lane == 0) {
            const int c = warp - TS_WARP_MMA0;
            constexpr uint32_t idesc = umma_idesc(BN);
            uint32_t wc = 0, bphase = 0;
            int bslot = c;
            bool ok = true;
            for (int it = 0; ok && sched.next(pc); it++) {
                const int acc = it % NACC, use = it / NACC;
                if (!mbar_wait_spin(&tmem_empty[acc], ((uint32_t)use & 1u) ^ 1u, abort_flag, a.status, 0x8000u)) break;
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + (uint32_t)(acc * BN);
                for (int sb = pc.sb0; sb < pc.sb1; sb++, wc++) {
                    const int aslot = (int)(wc & 1u) * 4 + c;
                    if (!mbar_wait_spin(&a_full[aslot], (wc >> 1) & 1u, abort_flag, a.status, 0x800u)) { ok = false; break; }
                    // A parity wait tells "this use is filled" from "the use before is not filled yet" only for a
                    // waiter that saw the use before complete.  Use u - 1 of this activation slot (k-block kb - BS)
                    // belongs to another MMA thread unless BS is a multiple of four, so wait until that thread has
                    // seen it land (it publishes the k-blocks it has passed in b_seen).
                    const uint32_t kb = wc * 4u + (uint32_t)c;
                    if ((BS & 3) != 0 && kb >= (uint32_t)BS) {
                        const uint32_t need = kb - (uint32_t)BS;
                        const long long t0 = clock64();
                        while (b_seen[need & 3u] <= need) {
                            __nanosleep(20);                 // (a spinning thread takes issue slots from the warps that work)
                            if (*abort_flag) { ok = false; break; }
                            if (clock64() - t0 > WAIT_CYCLES) { *abort_flag = 1; atomicOr(a.status, 0x10000u); __threadfence_system(); ok = false; break; }
                        }
                        if (!ok) break;
                    }
                    if (!mbar_wait_spin(&b_full[bslot], bphase, abort_flag, a.status, 0x1000u)) { ok = false; break; }
                    b_seen[c] = kb + 1u;
                    tc_fence_after();
                    const uint32_t tmem_a = tmem_base + (uint32_t)(TS_A_COL0 + aslot * 32);
                    const uint64_t bdesc = umma_desc(smem_u32(smem_b + bslot * B_STAGE_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / 16; k++)       // 16 k per MMA: 8 TMEM columns of A, 32 bytes of every B row
                        umma_f16_ts(tmem_acc, tmem_a + 8 * k, bdesc + 2 * k, idesc);
                    umma_commit(&a_empty[aslot]);
                    umma_commit(&b_empty[bslot]);
                    bslot += 4;
                    if (bslot >= BS) { bslot -= BS; bphase ^= 1u; }
                }
                if (ok) umma_commit(&tmem_full[acc]);
            }
        }
    } else {
        // ---------------- raw tile per super-block: the quant pieces of the sixteen 8-row tiles under this CTA's 128
        // rows in one tiled copy (the weight as a 4-D tensor: 128 bytes x pieces x super-blocks x 8-row units; units
        // past the last row read as zeros)
        if (STAGED_W && lane == 0) {
            uint32_t wc = 0;
            bool ok = true;
            while (ok && sched.next(pc)) {
                for (int sb = pc.sb0; sb < pc.sb1; sb++, wc++) {
                    const int wb = wc % WQ_BUFS;
                    if (!mbar_wait_spin(&wq_empty[wb], ((wc / WQ_BUFS) & 1u) ^ 1u, abort_flag, a.status, 0x4000u)) { ok = false; break; }
                    mbar_arrive_expect_tx(&wq_full[wb], (uint32_t)WQ_BYTES);
                    tma_load_4d(smem_wq + wb * WQ_BYTES, &tmap_w, 0, 0, sb, pc.n0 / OJAS_TILE_ROWS, &wq_full[wb]);
                }
            }
        }
    }

    // ---------------- teardown (every role arrives here, also after an abort)
    if (*abort_flag && warp == TS_WARP_TMA_X && lane == 0) {
        // give copies that are still in flight a bounded time to land before the CTA releases shared memory
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TS_WARP_TMA_W) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}
