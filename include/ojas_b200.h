/*
 * ojas_b200.h — C ABI of the B200 (sm_100a) quantized-matmul backend.
 *
 * Every entry point takes plain pointers and sizes.  Device pointers are raw CUDA
 * device addresses (what the engine's CuBuf holds, crates/ojas-cuda/src/device.rs:20-23);
 * nothing here allocates unless its comment says so, and every launch is
 * asynchronous on the context's stream (errors surface at ojas_b200_sync, like the
 * engine's submit(), crates/ojas-cuda/src/device.rs:534-536).
 *
 * All functions return 0 on success or a negative ojas_b200_status; the message of
 * the most recent failure on a context is kept by ojas_b200_last_error().
 *
 * Data contract (crates/ojas-cuda/src/kernels/gemm_q.rs:1-4): x is [M,K] f32
 * row-major, W is [N,K] with one output per row (y = x * W^T), y is [M,N] f32.
 * K must be a multiple of 256 (crates/ojas-cpu/src/cpu_math.rs:1148).
 */
#ifndef OJAS_B200_H
#define OJAS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define OJAS_B200_API __attribute__((visibility("default")))
#else
#define OJAS_B200_API
#endif

typedef struct ojas_b200_ctx ojas_b200_ctx;

/* GGUF tensor type codes on this path (crates/ojas-formats/src/synth.rs:12-21).  Every format has the repack, the GEMV family and the
 * prefill GEMM; the expert FFN (ojas_b200_moe_ffn) takes Q4_K, Q5_K and Q6_K experts.  IQ4_NL and IQ4_XS rows meet f32
 * activations, as Q8_0 rows do (dot_iq4nl / dot_iq4xs, crates/ojas-cpu/src/cpu_math.rs:993-1010, 943-967). */
enum { OJAS_B200_Q8_0 = 8, OJAS_B200_Q4_K = 12, OJAS_B200_Q5_K = 13, OJAS_B200_Q6_K = 14, OJAS_B200_IQ4_NL = 20, OJAS_B200_IQ4_XS = 23 };

/* Store forms of the native GEMV family: y = acc, y += acc, y = acc + bias
 * (crates/ojas-cuda/src/kernels/nat.rs:69-91). */
enum { OJAS_B200_PLAIN = 0, OJAS_B200_ACCUM = 1, OJAS_B200_BIAS = 2 };

typedef enum {
    OJAS_B200_OK = 0,
    OJAS_B200_E_ARG = -1,      /* bad shape, null pointer, unsupported type */
    OJAS_B200_E_CUDA = -2,     /* a CUDA call failed; message holds the CUDA error */
    OJAS_B200_E_UNSUPPORTED = -3,
    OJAS_B200_E_NAME = -4,     /* ojas_b200_dispatch: unknown kernel name */
    OJAS_B200_E_DEVICE = -5,   /* a kernel reported a bounded wait that ran out */
    OJAS_B200_E_LIMIT = -6     /* size beyond a fixed capacity */
} ojas_b200_status;

/* ---- context: replaces CudaGpu (crates/ojas-cuda/src/device.rs:87-146): one device, one
 * stream.  `stream` is a cudaStream_t to adopt, or NULL to create a private non-blocking
 * stream.  Allocates only host memory. */
OJAS_B200_API int ojas_b200_create(int device, void *stream, ojas_b200_ctx **out);
OJAS_B200_API void ojas_b200_destroy(ojas_b200_ctx *ctx);
OJAS_B200_API int ojas_b200_set_stream(ojas_b200_ctx *ctx, void *stream);
OJAS_B200_API void *ojas_b200_stream(ojas_b200_ctx *ctx);
/* Options.  "pdl" (default 1; OJAS_B200_PDL=0 in the environment at creation turns it off, the way the
 * engine reads its OJAS_* switches, crates/ojas-core/src/config.rs:1-22): GEMVs and the GEMM are launched
 * with programmatic dependent launch, so a kernel's weight prefetch and set-up overlap the tail of the
 * kernel before it in the stream (activations and y are only touched after the wait on that kernel).
 * "gemv_mma": Q4_K and Q6_K batches and expert groups on the integer tensor-core kernels: 0 = never, 1 = default (batches
 * from five rows; up to four the per-lane kernel is faster), n = 2..8: batches from n rows.  "gemv_kseg": Q8_0 batches of 3..8 rows walk K in this many equal segments
 * inside one launch (0 = only when the whole K does not fit in shared memory, 1 = never, n = n when it divides K / 256).  "gemv_warps", "gemv_stages" (0 = chosen per shape): upper bounds on the warps per CTA (a power of
 * two, at most 16) and on the depth of a warp's weight ring (1, 2 or 4) of the GEMV kernel; a bound the shape does
 * not fit under falls back to the next smaller choice.  "gemm_ksplit": 0 = K ranges balanced across the SMs,
 * S > 0 = every tile's K range cut into S pieces.  "moe_gemm_rows" (default 0 = off): from this many rows per expert
 * on average the expert FFN takes its prefill form: gate and up on the int8 tensor-core kernel (exact integers), the
 * down projection as grouped f16 tensor-core GEMMs; the FFN output stays within 2e-3 of the CPU path (typically 3e-4
 * instead of 1e-7).  "moe_i8" (default 0): decode-sized Q4_K expert FFNs on the int8 tensor-core kernel too (same
 * results as the default kernel; slower at 64 tokens). */
OJAS_B200_API int ojas_b200_set_option(ojas_b200_ctx *ctx, const char *key, int value);
/* Every option can also be given in the environment, read once at ojas_b200_create: OJAS_B200_<OPTION>=<integer>
 * (OJAS_B200_PDL=0, OJAS_B200_GEMM_KSPLIT=4, ...).
 * "profile" (default 0; OJAS_B200_PROFILE=1): the per-launch event profiler, the counterpart of KernelProfile under
 * OJAS_CUDA_PROFILE (crates/ojas-cuda/src/device.rs:275-318).  One event is recorded behind every launch; a launch is
 * charged the time between the event before it and its own.  profile_report writes "kernel launches total_ms avg_us"
 * lines (largest total first) and returns the length of the full text; it waits for the stream.  Launches made while
 * the stream is being captured are not recorded.  With OJAS_B200_PROFILE set the report is also printed to stderr when
 * the context is destroyed. */
OJAS_B200_API size_t ojas_b200_profile_report(ojas_b200_ctx *ctx, char *buf, size_t len);
OJAS_B200_API int ojas_b200_profile_reset(ojas_b200_ctx *ctx);
OJAS_B200_API const char *ojas_b200_last_error(ojas_b200_ctx *ctx);
OJAS_B200_API int ojas_b200_sm_count(ojas_b200_ctx *ctx);
/* Launches issued by this context since creation (the benchmark's launch counter). */
OJAS_B200_API uint64_t ojas_b200_launch_count(ojas_b200_ctx *ctx);
OJAS_B200_API const char *ojas_b200_version(void);

/* ---- Device trait helpers (crates/ojas-core/src/lib.rs:26-40: alloc / upload / read) and
 * submit (crates/ojas-core/src/kernel.rs:82).  For callers that have no CUDA runtime of
 * their own; a caller that already owns device memory passes its pointers directly. */
OJAS_B200_API int ojas_b200_alloc(ojas_b200_ctx *ctx, size_t bytes, void **dptr);
OJAS_B200_API int ojas_b200_free(ojas_b200_ctx *ctx, void *dptr);
OJAS_B200_API int ojas_b200_upload(ojas_b200_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
OJAS_B200_API int ojas_b200_download(ojas_b200_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes);
OJAS_B200_API int ojas_b200_memset(ojas_b200_ctx *ctx, void *dst_dev, int value, size_t bytes);
OJAS_B200_API int ojas_b200_sync(ojas_b200_ctx *ctx);

/* ---- timing and graphs: the event profiler and capture/replay of the CUDA device
 * (crates/ojas-cuda/src/device.rs:275-318 KernelProfile, :541-554 begin_capture / end_capture /
 * replay).  Every kernel of this library is capture-safe: no allocation, no host
 * synchronisation, no host state that changes launch arguments between replays. */
OJAS_B200_API int ojas_b200_event_create(ojas_b200_ctx *ctx, void **event);
OJAS_B200_API int ojas_b200_event_destroy(ojas_b200_ctx *ctx, void *event);
OJAS_B200_API int ojas_b200_event_record(ojas_b200_ctx *ctx, void *event);
OJAS_B200_API int ojas_b200_event_elapsed_ms(ojas_b200_ctx *ctx, void *start, void *stop, float *ms);
OJAS_B200_API int ojas_b200_graph_begin(ojas_b200_ctx *ctx);
OJAS_B200_API int ojas_b200_graph_end(ojas_b200_ctx *ctx, void **graph_exec);
OJAS_B200_API int ojas_b200_graph_launch(ojas_b200_ctx *ctx, void *graph_exec);
OJAS_B200_API int ojas_b200_graph_destroy(ojas_b200_ctx *ctx, void *graph_exec);
/* Pinned host staging memory (the expert cache stages through pinned memory,
 * crates/ojas-cuda/src/expert_cache.rs:93-150). */
OJAS_B200_API int ojas_b200_host_alloc(ojas_b200_ctx *ctx, size_t bytes, void **hptr);
OJAS_B200_API int ojas_b200_host_free(ojas_b200_ctx *ctx, void *hptr);

/* ---- upload layout: replaces Repr / Lin::load_as (crates/ojas-cuda/src/qwen35.rs:146-226)
 * and relayout_q4k_q4l (crates/ojas-formats/src/quant.rs:192-222).  GGUF blocks are re-laid
 * once at load into 16-byte-aligned planes (lossless: every GGUF bit is kept, no f16
 * rounding of products).  raw_bytes = N * K/256 * {144, 210, 272}. */
OJAS_B200_API size_t ojas_b200_raw_bytes(uint32_t ggml_type, size_t N, size_t K);
OJAS_B200_API size_t ojas_b200_repacked_bytes(uint32_t ggml_type, size_t N, size_t K);
/* raw_dev: GGUF blocks in device memory, rows contiguous.  out_dev: repacked_bytes bytes,
 * 256-byte aligned.  Runs on the stream. */
OJAS_B200_API int ojas_b200_repack(ojas_b200_ctx *ctx, uint32_t ggml_type, const void *raw_dev, size_t N, size_t K,
                     void *out_dev);
/* Host restatement of the same layout (for a loader that repacks before upload, and for
 * checking the device kernel). */
OJAS_B200_API int ojas_b200_repack_host(uint32_t ggml_type, const void *raw_host, size_t N, size_t K, void *out_host);

/* ---- activations: device form of quant_q8k (crates/ojas-cpu/src/cpu_math.rs:545-563).
 * x [M,K] f32 -> q [M,K] i8, scales [M,K/256] f32, bsums [M,K/32] i32; bit-identical to the
 * CPU routine (round half away from zero, scale = amax/127 or 1). */
OJAS_B200_API int ojas_b200_quant_q8k(ojas_b200_ctx *ctx, const float *x, size_t M, size_t K, int8_t *q, float *scales,
                        int32_t *bsums);

/* ---- activation producers that end in Q8_K: counterparts of rmsnorm_q8 and silu_mul_q8
 * (crates/ojas-cuda/src/kernels/ops.rs:27, 352), ending in the Q8_K form the K-quant GEMVs read (ojas_b200_gemv_q8k)
 * instead of the reference's q8_1 blocks, so one quantization feeds every projection of the row (Q, K, V; gate, up)
 * and the f32 row is never re-read.  rmsnorm (crates/ojas-cpu/src/cpu_math.rs:456-460): out = (x / sqrt(mean(x^2) +
 * eps)) * w per row of x [M,K]; the mean is a tree sum (agrees with the CPU's in-order sum to fp32 rounding), the
 * quantization of the normalized row is bit-identical to quant_q8k.  xn (may be null) receives the normalized f32 row.
 * silu_mul: act = silu(g) * u (crates/ojas-cpu/src/cpu_math.rs:486), then quant_q8k(act), bit-identical to the CPU
 * composition. */
OJAS_B200_API int ojas_b200_rmsnorm_q8k(ojas_b200_ctx *ctx, const float *x, const float *w, float eps, size_t M, size_t K, float *xn,
                                        int8_t *q, float *scales, int32_t *bsums);
OJAS_B200_API int ojas_b200_silu_mul_q8k(ojas_b200_ctx *ctx, const float *g, const float *u, size_t M, size_t K, int8_t *q,
                                         float *scales, int32_t *bsums);

/* ---- decode GEMV: replaces gemv_nat_{q4k,q6k,q80}{,_accum,_bias,_m}
 * (crates/ojas-cuda/src/kernels/nat.rs:69-91; bodies crates/ojas-core/src/quant_src.rs:779-867,
 * 1028-1057, 1154-1180) with the arithmetic of matvec_kq (crates/ojas-cpu/src/cpu_math.rs:
 * 1145-1189): Q4_K / Q5_K / Q6_K rows meet int8 Q8_K activations in exact integer block dots, Q8_0,
 * IQ4_NL and IQ4_XS rows meet f32 activations.  w is the repacked weight.  M <= OJAS_B200_GEMV_MAX_M. */
#define OJAS_B200_GEMV_MAX_M 8
OJAS_B200_API int ojas_b200_gemv(ojas_b200_ctx *ctx, uint32_t ggml_type, int form, const float *x, const void *w, float *y,
                   const float *bias, size_t K, size_t N, size_t M);
/* Same with RMSNorm fused into the prologue: y = W ((x * inv) * norm_w), inv = 1 / sqrt(mean(x^2) + eps) per row of x
 * (crates/ojas-cpu/src/cpu_math.rs:456-460; upstream runs rmsnorm_q8 and the GEMV as two launches,
 * crates/ojas-cuda/src/kernels/ops.rs:27).  The sum of squares is a tree sum: equal to the separate producer to fp32
 * rounding, not bit for bit. */
OJAS_B200_API int ojas_b200_gemv_rmsnorm(ojas_b200_ctx *ctx, uint32_t ggml_type, int form, const float *x, const float *norm_w, float eps,
                                         const void *w, float *y, const float *bias, size_t K, size_t N, size_t M);
/* Same with SwiGLU fused into the prologue: y = W (silu(g) * u) (crates/ojas-cpu/src/cpu_math.rs:486; upstream runs
 * silu_mul_q8 and the GEMV as two launches, crates/ojas-cuda/src/kernels/ops.rs:352).  The same expression as
 * ojas_b200_silu_mul_q8k: the two forms agree bit for bit. */
OJAS_B200_API int ojas_b200_gemv_silu_mul(ojas_b200_ctx *ctx, uint32_t ggml_type, int form, const float *g, const float *u, const void *w,
                                          float *y, const float *bias, size_t K, size_t N, size_t M);
/* Same, with activations already quantized by ojas_b200_quant_q8k (Q4_K / Q5_K / Q6_K only):
 * one quantization can feed several projections (gate and up read the same row). */
OJAS_B200_API int ojas_b200_gemv_q8k(ojas_b200_ctx *ctx, uint32_t ggml_type, int form, const int8_t *q, const float *scales,
                       const int32_t *bsums, const void *w, float *y, const float *bias, size_t K, size_t N,
                       size_t M);
/* Checking aid: the integer sub-block dots of row-0 activations against every weight row,
 * exactly as dot_q4k / dot_q6k form them (crates/ojas-cpu/src/cpu_math.rs:619-632, 703-719):
 * Q4_K -> idots [N, K/32], Q6_K -> idots [N, K/16] (int32). */
OJAS_B200_API int ojas_b200_gemv_idots(ojas_b200_ctx *ctx, uint32_t ggml_type, const float *x, const void *w, int32_t *idots,
                         size_t K, size_t N);

/* ---- prefill GEMM on the tensor cores (tcgen05 + TMEM): replaces gemm_mm_{q4l,q6k,q8_0} and
 * their split-K forms (crates/ojas-cuda/src/kernels/gemm_q.rs:499-590; call site CudaSsm::mm,
 * crates/ojas-cuda/src/qwen35.rs:644-702).  y [M,N] = x [M,K] * W^T (accum != 0: y += ...).  Q4_K and
 * Q6_K activations are quantized to Q8_K first, as the CPU path does, and enter the MMA as
 * f16(sx * q); Q8_0 activations enter as f16(x); accumulation is fp32.  `workspace` is
 * caller-owned scratch of at least ojas_b200_gemm_workspace_bytes(M, K) bytes, 256-byte
 * aligned (the f16 activation tiles); nothing is allocated here. */
OJAS_B200_API size_t ojas_b200_gemm_workspace_bytes(size_t M, size_t K);
OJAS_B200_API int ojas_b200_gemm(ojas_b200_ctx *ctx, uint32_t ggml_type, const float *x, const void *w, float *y, size_t K,
                                 size_t N, size_t M, int accum, void *workspace, size_t workspace_bytes);

/* The same with f16 activations xh [M,K] (the engine's split-K prefill entries take them that way,
 * crates/ojas-cuda/src/kernels/gemm_q.rs:537-556): widened exactly, then the arithmetic of ojas_b200_gemm. */
OJAS_B200_API int ojas_b200_gemm_f16(ojas_b200_ctx *ctx, uint32_t ggml_type, const void *xh, const void *w, float *y, size_t K,
                                     size_t N, size_t M, int accum, void *workspace, size_t workspace_bytes);
/* Scratch owned by the context for the entry points that have no workspace argument (the name-based prefill entries
 * gemm_mm_*, whose upstream argument lists carry none).  Grow-only; ALLOCATES: call it at set-up, never on the compute
 * path.  Without it those entries use the array built into the library (up to ojas_b200_gemm_static_capacity() bytes)
 * and refuse larger shapes. */
OJAS_B200_API int ojas_b200_reserve(ojas_b200_ctx *ctx, size_t bytes);
OJAS_B200_API size_t ojas_b200_reserved_bytes(ojas_b200_ctx *ctx);

/* ---- prefill GEMM for callers that cannot provide scratch memory.  No counterpart in the reference.
 * Meant for hosts that may not allocate device memory around the call: a plugin inside an engine
 * whose allocator it cannot reach, or a serving loop that has frozen its memory map.  Same result as
 * ojas_b200_gemm, but the f16 activation tiles go to an 8 MiB array built into the library (each GPU
 * that loads the library holds it until the process exits), so M * K <= 4 194 304
 * (ojas_b200_gemm_static_capacity() bytes / 2); larger shapes are refused with OJAS_B200_E_LIMIT.
 * Calls nothing that allocates.  The first call on a device looks up the array's device address and loads the code of
 * every kernel the entry can launch (all tile widths, every format); make that call at set-up, from one thread,
 * before any stream capture: after it no call on that device allocates, whatever its shape or type.  The array is shared by every call and keeps the last call's
 * contents (each call overwrites the part it uses); two calls whose kernels overlap on the GPU (other
 * streams, other contexts on the same device) race on it. */
OJAS_B200_API size_t ojas_b200_gemm_static_capacity(void);
OJAS_B200_API int ojas_b200_gemm_static(ojas_b200_ctx *ctx, uint32_t ggml_type, const float *x, const void *w, float *y, size_t K,
                                        size_t N, size_t M, int accum);

/* ---- mixture of experts.
 * Router: moe_topk (crates/ojas-cuda/src/kernels/moe.rs:45-70) and its batched form moe_topk_m
 * (crates/ojas-metal/src/kernels/moe.rs:173-199): logits [M,E] -> idx u32 [M,KSEL], wgt f32 [M,KSEL];
 * softmax, KSEL arg-max passes (ties -> lowest index), weights renormalised over the picks. */
OJAS_B200_API int ojas_b200_moe_topk(ojas_b200_ctx *ctx, const float *logits, uint32_t *idx, float *wgt, size_t M, size_t E,
                                     size_t KSEL);
/* Expert FFN: replaces moe_gu_<fmt> / moe_down_<fmt> (crates/ojas-cuda/src/kernels/moe.rs:75-125; the
 * Q4_K / Q6_K forms exist upstream only for Metal, crates/ojas-metal/src/kernels/moe.rs:513-529, 769-815)
 * with the arithmetic of the CPU expert block (crates/ojas-cpu/src/cpu_glm.rs:551-582).
 * h [M,d] f32; wg, wu: repacked stacked experts [E*ffn, d]; wd: [E*d, ffn]; idx, wgt as produced by
 * ojas_b200_moe_topk; out [M,d] f32 = sum_j wgt_j * down_e(silu(gate_e h) * up_e h)  (accum != 0: +=).
 * Assignments are grouped by expert so each expert's weights are read once.  `workspace`: caller-owned
 * scratch of ojas_b200_moe_workspace_bytes(...) bytes, 256-byte aligned.  Expert types: Q4_K, Q5_K, Q6_K. */
OJAS_B200_API size_t ojas_b200_moe_workspace_bytes(size_t M, size_t E, size_t KSEL, size_t d, size_t ffn);
OJAS_B200_API int ojas_b200_moe_ffn(ojas_b200_ctx *ctx, uint32_t type_gu, uint32_t type_d, const float *h, const void *wg,
                                    const void *wu, const void *wd, const uint32_t *idx, const float *wgt, size_t M, size_t E,
                                    size_t KSEL, size_t d, size_t ffn, float *out, int accum, void *workspace,
                                    size_t workspace_bytes);

/* ---- loader side (host code): a GGUF tensor directory (crates/ojas-formats/src/gguf.rs:158-205, 298-455: versions 2
 * and 3, one file) and a cache file of repacked weights keyed to the source file by size and modification time
 * (crates/ojas-models/src/weights.rs:14-32).  err (may be null) receives a message on failure.
 * GGUF stores a matrix as dims[0] = K (contiguous), dims[1] = N.  Rows of several matrices that share K (Q, K, V; gate,
 * up) become ONE matrix by repacking each part into consecutive 8-row units of one buffer: parts whose row counts are
 * multiples of 8 simply follow one another (crates/ojas-cuda/src/qwen35.rs:168-189 concatenates along N the same way). */
typedef struct ojas_b200_gguf ojas_b200_gguf;
typedef struct ojas_b200_weight_cache ojas_b200_weight_cache;
OJAS_B200_API int ojas_b200_gguf_open(const char *path, ojas_b200_gguf **out, char *err, size_t errlen);
OJAS_B200_API void ojas_b200_gguf_close(ojas_b200_gguf *g);
OJAS_B200_API size_t ojas_b200_gguf_tensor_count(const ojas_b200_gguf *g);
OJAS_B200_API int ojas_b200_gguf_tensor_info(const ojas_b200_gguf *g, size_t index, const char **name, uint32_t *ggml_type, uint32_t *ndims,
                                             uint64_t dims[4], uint64_t *file_offset, uint64_t *bytes);
OJAS_B200_API long long ojas_b200_gguf_find(const ojas_b200_gguf *g, const char *name);
OJAS_B200_API int ojas_b200_gguf_read_raw(const ojas_b200_gguf *g, size_t index, void *dst, size_t bytes);
/* build: every matrix of the GGUF in a format of this path re-laid on the host and written to cache_path (atomically).
 * open: maps the file; with gguf_path given it must be the file the cache was built from, else OJAS_B200_E_UNSUPPORTED
 * (rebuild).  entry: name, type, [N, K] and a pointer to the repacked bytes inside the mapping. */
OJAS_B200_API int ojas_b200_weight_cache_build(const char *gguf_path, const char *cache_path, char *err, size_t errlen);
OJAS_B200_API int ojas_b200_weight_cache_open(const char *cache_path, const char *gguf_path, ojas_b200_weight_cache **out, char *err,
                                              size_t errlen);
OJAS_B200_API void ojas_b200_weight_cache_close(ojas_b200_weight_cache *cache);
OJAS_B200_API size_t ojas_b200_weight_cache_count(const ojas_b200_weight_cache *cache);
OJAS_B200_API int ojas_b200_weight_cache_entry(const ojas_b200_weight_cache *cache, size_t index, const char **name, uint32_t *ggml_type,
                                               uint64_t *N, uint64_t *K, const void **data, uint64_t *bytes);

/* ---- token-table gather: x[m, :] = dequantized row ids[m] of a table kept as RAW GGUF blocks [rows, d] on the device
 * (read in place; not the repacked layout).  Replaces q35_embed_q4k (crates/ojas-cuda/src/kernels/qwen35.rs:51-69) for
 * Q4_K, Q5_K, Q6_K, Q8_0, IQ4_NL and IQ4_XS tables; the values equal the CPU decoder's bit for bit.  An id >= rows reads the last row.
 * The entry name "q35_embed_q4k" (emb, ids, x)(d, M) is served by ojas_b200_dispatch. */
OJAS_B200_API int ojas_b200_embed_rows(ojas_b200_ctx *ctx, uint32_t ggml_type, const void *table, size_t rows, const uint32_t *ids, size_t M,
                                       size_t d, float *x);

/* ---- expert residency: replaces ExpertCache (crates/ojas-cuda/src/expert_cache.rs:34-160).  A bounded arena of
 * expert-sized slots in device memory with least-recently-used eviction; misses are streamed from the host through
 * pinned staging memory and re-laid into tiles on the device.  gather() returns byte offsets into the arena: what the
 * moe_gu_<fmt>_slots / moe_down_<fmt>_slots entries take (crates/ojas-cuda/src/kernels/moe.rs:127-178).
 * create / destroy allocate and free; gather allocates nothing.  The expert_lru_* calls are the bookkeeping alone
 * (pure host code): which slot serves which expert, hits, misses, evictions. */
typedef struct ojas_b200_expert_lru ojas_b200_expert_lru;
typedef struct ojas_b200_expert_cache ojas_b200_expert_cache;
OJAS_B200_API int ojas_b200_expert_lru_create(size_t slots, ojas_b200_expert_lru **out);
OJAS_B200_API void ojas_b200_expert_lru_destroy(ojas_b200_expert_lru *lru);
OJAS_B200_API int ojas_b200_expert_lru_plan(ojas_b200_expert_lru *lru, const uint32_t *ids, size_t n, uint32_t *slot_out, uint8_t *miss_out);
OJAS_B200_API void ojas_b200_expert_lru_stats(const ojas_b200_expert_lru *lru, size_t out[3]);
/* One cache holds experts of one tensor: [N, K] of ggml_type each (N a multiple of 8).  budget_bytes / slot bytes
 * slots, at least one. */
OJAS_B200_API int ojas_b200_expert_cache_create(ojas_b200_ctx *ctx, uint32_t ggml_type, size_t N, size_t K, size_t budget_bytes,
                                                ojas_b200_expert_cache **out);
OJAS_B200_API void ojas_b200_expert_cache_destroy(ojas_b200_expert_cache *cache);
OJAS_B200_API size_t ojas_b200_expert_cache_slots(const ojas_b200_expert_cache *cache);
OJAS_B200_API size_t ojas_b200_expert_cache_slot_bytes(const ojas_b200_expert_cache *cache);
OJAS_B200_API void *ojas_b200_expert_cache_arena(const ojas_b200_expert_cache *cache);
OJAS_B200_API void ojas_b200_expert_cache_stats(const ojas_b200_expert_cache *cache, size_t out[4]);
/* ids [n] -> offsets_out [n] (bytes into the arena).  load(user, id, dst, bytes) fills dst with expert id's GGUF blocks
 * (bytes = ojas_b200_raw_bytes(ggml_type, N, K)) and returns 0.  More distinct ids than slots: OJAS_B200_E_LIMIT. */
OJAS_B200_API int ojas_b200_expert_cache_gather(ojas_b200_expert_cache *cache, const uint32_t *ids, size_t n,
                                                int (*load)(void *user, uint32_t id, void *dst, size_t bytes), void *user,
                                                uint64_t *offsets_out);

/* ---- tensor-parallel shard planning (host).  No counterpart in the reference, which is single-GPU
 * (its only distributed code is a TCP pipeline for another backend, crates/ojas-swarm/src/lib.rs:12-40);
 * the shard shapes follow the weight contract of crates/ojas-cuda/src/kernels/gemm_q.rs:1-4.
 * Column-parallel: rank r owns weight rows [row0, row0+rows) and its outputs are all-gathered.
 * Row-parallel: rank r owns K range [k0, k0+klen), whole 256-weight super-blocks, and the partial
 * results are all-reduced.  The collectives themselves run in the caller (NCCL). */
OJAS_B200_API int ojas_b200_tp_shard_rows(size_t N, int world, int rank, size_t *row0, size_t *rows);
OJAS_B200_API int ojas_b200_tp_shard_k(size_t K, int world, int rank, size_t *k0, size_t *klen);
OJAS_B200_API int ojas_b200_tp_slice_k_host(uint32_t ggml_type, const void *raw, size_t N, size_t K, size_t k0, size_t klen,
                                            void *out);

/* ---- decode join through peer memory.  No counterpart in the reference (single-GPU).  For one activation row a
 * sharded projection is a few microseconds of GEMV and a library collective behind it costs several times that, so
 * the GEMV's epilogue stores its results straight into every rank's receive window (device memory the other ranks
 * map through CUDA IPC; plain peer stores, no tensor map covers peer memory).  Values travel stamped (8-byte pairs:
 * the float's bits and the step's number, one store), so there is no flag and no fence: a join costs one NVLink
 * crossing.  Each rank's join kernel polls the pairs it needs WITH A LIMIT (default about 2 s; on expiry the affected
 * outputs are left alone, the step still closes, and ojas_b200_sync returns OJAS_B200_E_DEVICE) and forms the result
 * from its own window.
 * One process per GPU.  Set-up: every rank calls tp_create (allocates its window: 2 * world * slot_floats pairs),
 * tp_export, hands the handle (ojas_b200_tp_handle_bytes() bytes) to the other ranks by any host channel, and
 * tp_import for each peer.  A step: one or more tp_gemv, then tp_join; or local GEMVs, then tp_allgather.  Every rank
 * must run the same sequence of steps.  All launches are capture-safe (the step counter lives in device memory).
 * join modes: 1 column-parallel, y[n_total] = the ranks' shards in rank order (plan of ojas_b200_tp_shard_rows);
 * 2 row-parallel, y[n_total] = sum of the ranks' partial vectors in rank order (the same order on every rank: all
 * ranks end with identical bits). */
typedef struct ojas_b200_tp ojas_b200_tp;
OJAS_B200_API int ojas_b200_tp_create(ojas_b200_ctx *ctx, int world, int rank, size_t slot_floats, ojas_b200_tp **out);
OJAS_B200_API void ojas_b200_tp_destroy(ojas_b200_tp *tp);
OJAS_B200_API size_t ojas_b200_tp_handle_bytes(void);
OJAS_B200_API int ojas_b200_tp_export(ojas_b200_tp *tp, void *handle_out);
OJAS_B200_API int ojas_b200_tp_import(ojas_b200_tp *tp, int peer, const void *handle);
OJAS_B200_API int ojas_b200_tp_set_wait_us(ojas_b200_tp *tp, unsigned micros);
/* x [K] f32 through this rank's repacked shard w [N, K]; the N results go to float `offset` of this rank's slot in
 * every rank's window. */
OJAS_B200_API int ojas_b200_tp_gemv(ojas_b200_tp *tp, uint32_t ggml_type, const float *x, const void *w, size_t K, size_t N,
                                    size_t offset);
OJAS_B200_API int ojas_b200_tp_join(ojas_b200_tp *tp, int mode, float *y, size_t n_total);
/* A whole step's exchange in one kernel: all-gather of `floats` values per rank (src -> every window, bounded wait,
 * copy-out): y_all [world][floats]. */
OJAS_B200_API int ojas_b200_tp_allgather(ojas_b200_tp *tp, const float *src, size_t floats, float *y_all);

/* ---- name-based dispatch: the C form of KernelRuntime::dispatch / has_kernel
 * (crates/ojas-core/src/kernel.rs:68-83; argument marshalling crates/ojas-cuda/src/device.rs:
 * 391-415): buffers are (device pointer, byte offset) pairs in the kernel's positional order,
 * then the u32 constants.  grid and block are accepted for signature compatibility and
 * ignored, except grid[1] of the moe_gu_* entries (the number of picks, as upstream's blockIdx.y).  Names served, with
 * the engine's own argument lists: gemv_nat_{q4k,q6k,q80}{,_accum,_bias,_m} (crates/ojas-cuda/src/kernels/nat.rs:56-64);
 * gemm_mm_{q4l,q6k,q8_0}{,_sk} and gemm_mm_q4k{,_sk} (crates/ojas-cuda/src/kernels/gemm_q.rs:499-556; for q4l the weight
 * buffer is this library's repacked Q4_K and qa / qb are ignored); moe_topk{,_m}; moe_gu_<fmt>, moe_down_<fmt> and their
 * _slots forms for q80, q4k, q6k (crates/ojas-cuda/src/kernels/moe.rs:75-178); quant_q8k.  ojas_b200_kernel_name lists
 * them. */
OJAS_B200_API int ojas_b200_has_kernel(const char *name);
OJAS_B200_API int ojas_b200_kernel_count(void);
OJAS_B200_API const char *ojas_b200_kernel_name(int index);
OJAS_B200_API int ojas_b200_dispatch(ojas_b200_ctx *ctx, const char *name, void *const *bufs, const uint64_t *offsets, int nbufs,
                       const uint32_t *consts, int nconsts, const uint32_t grid[3], const uint32_t block[3]);

/* ---- test-input encoders (host): f32 [N,K] -> GGUF blocks.  The reference has no encoder
 * for these formats (its GEMM tests use random blocks, crates/ojas-formats/src/synth.rs:29);
 * these simple min/max encoders exist so seeded N(0, sigma) matrices can become legal blocks. */
OJAS_B200_API int ojas_b200_encode_host(uint32_t ggml_type, const float *w, size_t N, size_t K, void *raw_out);

#ifdef __cplusplus
}
#endif
#endif /* OJAS_B200_H */
