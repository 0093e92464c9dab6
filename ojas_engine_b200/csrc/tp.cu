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
    const size_t per256 = type == OJAS_B200_Q4_K ? 144 : type == OJAS_B200_Q5_K ? 176 : type == OJAS_B200_Q6_K ? 210 : type == OJAS_B200_Q8_0 ? 272 : type == OJAS_B200_IQ4_XS ? 136 : type == OJAS_B200_IQ4_NL ? 144 : 0;
    if (!per256) return OJAS_B200_E_ARG;
    const size_t row_in = K / 256 * per256, row_out = klen / 256 * per256, skip = k0 / 256 * per256;
    for (size_t r = 0; r < N; r++) memcpy((uint8_t *)out + r * row_out, (const uint8_t *)raw + r * row_in + skip, row_out);
    return 0;
}

// ---------------------------------------------------------------------------- decode join through peer memory
// For one activation row a sharded projection is a few microseconds of GEMV, and a library collective behind it
// costs several times that.  So the GEMV's own epilogue stores its results straight into every rank's RECEIVE
// WINDOW (device memory that the other ranks of the group have mapped through CUDA IPC; plain peer stores, no
// tensor map ever covers peer memory).  Values travel STAMPED: a float is sent as an 8-byte pair (bits, step number)
// in one 8-byte store, so whoever reads the stamp of the step in flight has the value with it.  There is no flag,
// no fence and no rendezvous of the sending grid: the cost of a join is one NVLink crossing.  The join kernel of a
// rank polls the pairs it needs, WITH A LIMIT, and forms the result from its own window: the concatenation of the
// shards (column-parallel) or their sum in rank order (row-parallel; the same order on every rank, so all ranks hold
// the same bits).
//
// Window of a rank:  joined u32, step u32 (256 bytes) | pairs[2][world][slot_floats]
// Two halves, used by alternate steps: a rank can be at most one step ahead of any other (its own join of step s
// needs everybody's values of step s), so while it writes half (s + 1) & 1 nobody can still be reading that half
// from step s - 1.  `step` counts the joins of this rank (starts at 1); the join kernel advances it, so a captured
// graph replays with fresh stamps.
struct ojas_b200_tp {
    ojas_b200_ctx *ctx;
    int world, rank;
    size_t slot_floats;
    uint8_t *window[OJAS_TP_MAX_RANKS];      // [rank] = local allocation, others = IPC mappings
    bool imported[OJAS_TP_MAX_RANKS];
    long long wait_cycles;                   // limit of the join's wait for a value
};

static constexpr size_t TP_WORDS_BYTES = 256;
static inline size_t tp_window_bytes(int world, size_t slot_floats) { return TP_WORDS_BYTES + 2 * (size_t)world * slot_floats * sizeof(uint2); }
static inline unsigned *tp_joined(uint8_t *w) { return (unsigned *)w; }
static inline unsigned *tp_step(uint8_t *w) { return (unsigned *)w + 1; }
static inline uint2 *tp_pairs(uint8_t *w) { return (uint2 *)(w + TP_WORDS_BYTES); }

extern "C" int ojas_b200_tp_create(ojas_b200_ctx *ctx, int world, int rank, size_t slot_floats, ojas_b200_tp **out) {
    if (!ctx || !out) return OJAS_B200_E_ARG;
    *out = nullptr;
    if (world < 1 || world > OJAS_TP_MAX_RANKS || rank < 0 || rank >= world || slot_floats == 0 || slot_floats % 4 != 0)
        return ojas_fail(ctx, OJAS_B200_E_ARG, "tp_create: world=%d (1..%d) rank=%d slot_floats=%zu (a positive multiple of 4)", world,
                         OJAS_TP_MAX_RANKS, rank, slot_floats);
    ojas_b200_tp *tp = new ojas_b200_tp();
    tp->ctx = ctx; tp->world = world; tp->rank = rank; tp->slot_floats = slot_floats;
    tp->wait_cycles = 4000000000LL;          // about two seconds
    for (int i = 0; i < OJAS_TP_MAX_RANKS; i++) { tp->window[i] = nullptr; tp->imported[i] = false; }
    const size_t bytes = tp_window_bytes(world, slot_floats);
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e == cudaSuccess) e = cudaMalloc((void **)&tp->window[rank], bytes);
    if (e == cudaSuccess) e = cudaMemset(tp->window[rank], 0, bytes);      // stamp 0 belongs to no step
    const unsigned one = 1u;
    if (e == cudaSuccess) e = cudaMemcpy(tp_step(tp->window[rank]), &one, sizeof one, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        if (tp->window[rank]) cudaFree(tp->window[rank]);
        delete tp;
        return ojas_fail(ctx, OJAS_B200_E_CUDA, "tp_create: window of %zu bytes: %s", bytes, cudaGetErrorString(e));
    }
    *out = tp;
    return 0;
}

extern "C" void ojas_b200_tp_destroy(ojas_b200_tp *tp) {
    if (!tp) return;
    cudaSetDevice(tp->ctx->device);
    cudaStreamSynchronize(tp->ctx->stream);
    for (int i = 0; i < tp->world; i++)
        if (i != tp->rank && tp->imported[i]) cudaIpcCloseMemHandle(tp->window[i]);
    if (tp->window[tp->rank]) cudaFree(tp->window[tp->rank]);
    delete tp;
}

extern "C" size_t ojas_b200_tp_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

extern "C" int ojas_b200_tp_export(ojas_b200_tp *tp, void *handle_out) {
    if (!tp || !handle_out) return OJAS_B200_E_ARG;
    cudaIpcMemHandle_t h;
    OJAS_CUDA(tp->ctx, cudaIpcGetMemHandle(&h, tp->window[tp->rank]));
    memcpy(handle_out, &h, sizeof h);
    return 0;
}

extern "C" int ojas_b200_tp_import(ojas_b200_tp *tp, int peer, const void *handle) {
    if (!tp || !handle) return OJAS_B200_E_ARG;
    if (peer < 0 || peer >= tp->world || peer == tp->rank) return ojas_fail(tp->ctx, OJAS_B200_E_ARG, "tp_import: peer %d", peer);
    if (tp->imported[peer]) return 0;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void *p = nullptr;
    OJAS_CUDA(tp->ctx, cudaSetDevice(tp->ctx->device));
    OJAS_CUDA(tp->ctx, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    tp->window[peer] = (uint8_t *)p;
    tp->imported[peer] = true;
    return 0;
}

extern "C" int ojas_b200_tp_set_wait_us(ojas_b200_tp *tp, unsigned micros) {
    if (!tp || micros == 0) return OJAS_B200_E_ARG;
    tp->wait_cycles = (long long)micros * 2000LL;       // clock64 ticks at about 2 GHz
    return 0;
}

static int tp_ready(ojas_b200_tp *tp) {
    for (int i = 0; i < tp->world; i++)
        if (!tp->window[i]) return ojas_fail(tp->ctx, OJAS_B200_E_ARG, "tp: the window of rank %d has not been imported", i);
    return 0;
}

// Destinations of a push: float `offset` of this rank's slot in every rank's window (pointers of half 0; the kernel
// adds the half of the step in flight, which it reads from the local step word, so a captured launch stays right on
// replay).
static void tp_fill(ojas_b200_tp *tp, size_t offset, TpPush &p) {
    memset(&p, 0, sizeof p);
    for (int i = 0; i < tp->world; i++) p.dst[p.n++] = tp_pairs(tp->window[i]) + (size_t)tp->rank * tp->slot_floats + offset;
    p.step = tp_step(tp->window[tp->rank]);
    p.half_pairs = (size_t)tp->world * tp->slot_floats;
}

int ojas_gemv_tp(ojas_b200_ctx *ctx, uint32_t type, const float *x, const void *w, size_t K, size_t N, const TpPush &push);

// One activation row through this rank's shard [N, K]; the N results go, stamped, to float `offset` of this rank's
// slot in every rank's window.
extern "C" int ojas_b200_tp_gemv(ojas_b200_tp *tp, uint32_t type, const float *x, const void *w, size_t K, size_t N, size_t offset) {
    if (!tp) return OJAS_B200_E_ARG;
    int rc = tp_ready(tp);
    if (rc) return rc;
    if (offset + N > tp->slot_floats)
        return ojas_fail(tp->ctx, OJAS_B200_E_LIMIT, "tp_gemv: %zu floats at offset %zu exceed the slot of %zu", N, offset, tp->slot_floats);
    TpPush p;
    tp_fill(tp, offset, p);
    return ojas_gemv_tp(tp->ctx, type, x, w, K, N, p);
}

// ---- join
// mode 1: column-parallel, y[off_s + i] = slot s [i] for i < len_s with the shard plan of
// ojas_b200_tp_shard_rows(n_total); 2: row-parallel, y[i] = sum over s in rank order of slot s [i], i < n_total.
// All-gather form (push_src != null): first every thread stamps and stores its share of push_src into this rank's
// slot of every window, then the kernel proceeds as mode 1.
struct TpJoinArgs {
    const uint2 *pairs;         // local window [2][world][slot_floats]
    unsigned *joined, *step;    // local words
    float *y;
    unsigned *status;
    long long wait_cycles;
    size_t slot_floats, n_total;
    int world, mode;
    const float *push_src;
    size_t push_floats;
    TpPush push;
};

// The value stamped `step` at p, or a give-up after the limit (returns false; *v untouched).
__device__ __forceinline__ bool tp_take(const uint2 *p, unsigned step, long long limit, float *v) {
    uint2 t;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(t.x), "=r"(t.y) : "l"(p) : "memory");
    if (t.y != step) {
        const long long t0 = clock64();
        for (;;) {
            __nanosleep(32);
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(t.x), "=r"(t.y) : "l"(p) : "memory");
            if (t.y == step) break;
            if (clock64() - t0 > limit) return false;
        }
    }
    *v = __uint_as_float(t.x);
    return true;
}

__global__ void __launch_bounds__(256) tp_join_kernel(const TpJoinArgs a) {
    grid_dependency_wait();
    const unsigned step = *reinterpret_cast<volatile unsigned *>(a.step);
    const uint2 *pairs = a.pairs + (size_t)(step & 1u) * a.world * a.slot_floats;
    bool ok = true;
    if (a.push_src) {
        const size_t half = (size_t)(step & 1u) * a.push.half_pairs, n2 = a.push_floats >> 1;
        const float2 *src = reinterpret_cast<const float2 *>(a.push_src);
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += (size_t)gridDim.x * blockDim.x) {
            const float2 v = __ldg(src + i);
            const uint4 two = make_uint4(__float_as_uint(v.x), step, __float_as_uint(v.y), step);    // two stamped values per 16-byte store
            for (int p = 0; p < a.push.n; p++) reinterpret_cast<uint4 *>(a.push.dst[p] + half)[i] = two;
        }
    }
    if (a.mode == 1) {
        size_t off = 0;
        const size_t base = a.n_total / (size_t)a.world, rem = a.n_total % (size_t)a.world;
        for (int s = 0; s < a.world; s++) {
            const size_t len = base + ((size_t)s < rem ? 1 : 0);
            for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += (size_t)gridDim.x * blockDim.x) {
                float v;
                if (tp_take(pairs + (size_t)s * a.slot_floats + i, step, ok ? a.wait_cycles : 0, &v)) a.y[off + i] = v;     // after one give-up: single probes
                else ok = false;
            }
            off += len;
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n_total; i += (size_t)gridDim.x * blockDim.x) {
            float sum = 0.0f, v;
            bool all = true;
            for (int s = 0; s < a.world; s++) {
                if (tp_take(pairs + (size_t)s * a.slot_floats + i, step, (ok && all) ? a.wait_cycles : 0, &v)) sum = s == 0 ? v : sum + v;
                else all = false;
            }
            if (all) a.y[i] = sum;
            else ok = false;
        }
    }
    // a rank did not deliver in time: report (y keeps what it had there), and still finish the step so that the context stays usable
    const int bad = __syncthreads_or(ok ? 0 : 1);
    if (threadIdx.x == 0) {
        if (bad) { atomicOr(a.status, 0x80000u); __threadfence_system(); }
        __threadfence();
        const unsigned old = atomicAdd(a.joined, 1u);
        if (old == gridDim.x - 1) {          // the block that finishes last closes the step
            *a.joined = 0u;
            *a.step = step + 1u;
        }
    }
}

static int tp_join_launch(ojas_b200_tp *tp, int mode, float *y, size_t n_total, const float *push_src, size_t push_floats) {
    if (!tp) return OJAS_B200_E_ARG;
    int rc = tp_ready(tp);
    if (rc) return rc;
    if (mode < 1 || mode > 2) return ojas_fail(tp->ctx, OJAS_B200_E_ARG, "tp_join: mode %d (1 = column-parallel, 2 = row-parallel)", mode);
    if (!y || n_total == 0) return ojas_fail(tp->ctx, OJAS_B200_E_ARG, "tp_join: null or empty output");
    const size_t per = mode == 1 ? (n_total + tp->world - 1) / tp->world : n_total;
    if (per > tp->slot_floats) return ojas_fail(tp->ctx, OJAS_B200_E_LIMIT, "tp_join: %zu floats per rank exceed the slot of %zu", per, tp->slot_floats);
    uint8_t *w = tp->window[tp->rank];
    TpJoinArgs a{};
    a.pairs = tp_pairs(w);
    a.joined = tp_joined(w); a.step = tp_step(w);
    a.y = y; a.status = tp->ctx->dev_status; a.wait_cycles = tp->wait_cycles;
    a.slot_floats = tp->slot_floats; a.n_total = n_total; a.world = tp->world; a.mode = mode;
    if (push_src) {
        a.push_src = push_src;
        a.push_floats = push_floats;
        tp_fill(tp, 0, a.push);
    }
    size_t blocks = ((mode == 1 ? per : n_total) + 255) / 256;
    if (blocks > 2 * (size_t)tp->ctx->sm_count) blocks = 2 * (size_t)tp->ctx->sm_count;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = tp->ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tp->ctx->pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, tp_join_kernel, a);
    if (e != cudaSuccess) return ojas_fail(tp->ctx, OJAS_B200_E_CUDA, "launch tp_join: %s", cudaGetErrorString(e));
    ojas_count_launch(tp->ctx, "tp_join");
    return 0;
}

extern "C" int ojas_b200_tp_join(ojas_b200_tp *tp, int mode, float *y, size_t n_total) { return tp_join_launch(tp, mode, y, n_total, nullptr, 0); }

// All-gather of `floats` values per rank in one kernel: every rank stamps and stores src into its slot of every
// window, then polls (bounded) for the others' and copies the slots out: y_all [world][floats].  The step's single
// exchange when a rank produced many results locally (a whole decode step's outputs).
extern "C" int ojas_b200_tp_allgather(ojas_b200_tp *tp, const float *src, size_t floats, float *y_all) {
    if (!tp) return OJAS_B200_E_ARG;
    if (!src || !y_all || floats == 0 || floats % 4 != 0 || ((uintptr_t)src & 15))
        return ojas_fail(tp->ctx, OJAS_B200_E_ARG, "tp_allgather: src must be 16-byte aligned and hold a positive multiple of 4 floats");
    if (floats > tp->slot_floats) return ojas_fail(tp->ctx, OJAS_B200_E_LIMIT, "tp_allgather: %zu floats exceed the slot of %zu", floats, tp->slot_floats);
    return tp_join_launch(tp, 1, y_all, floats * (size_t)tp->world, src, floats);
}
