// Context object and the Device-trait helpers of the C ABI (include/ojas_b200.h).
#include <stdarg.h>
#include <stdlib.h>

#include "common.cuh"

int ojas_fail(ojas_b200_ctx *ctx, int code, const char *fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof ctx->err, fmt, ap);
        va_end(ap);
    }
    return code;
}

extern "C" const char *ojas_b200_version(void) { return "ojas-b200 0.1 (sm_100a)"; }

extern "C" int ojas_b200_create(int device, void *stream, ojas_b200_ctx **out) {
    if (!out) return OJAS_B200_E_ARG;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || device < 0 || device >= count) return e != cudaSuccess ? OJAS_B200_E_CUDA : OJAS_B200_E_ARG;
    ojas_b200_ctx *ctx = new ojas_b200_ctx();
    ctx->device = device;
    cudaDeviceProp prop;
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        delete ctx;
        return OJAS_B200_E_CUDA;
    }
    if (prop.major != 10) {  // the kernels are built for sm_100a only; refuse anything else loudly
        delete ctx;
        return OJAS_B200_E_UNSUPPORTED;
    }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = (int)prop.sharedMemPerBlockOptin;
    if (stream) {
        ctx->stream = (cudaStream_t)stream;
    } else {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete ctx;
            return OJAS_B200_E_CUDA;
        }
        ctx->owns_stream = true;
    }
    // status word in pinned, device-mapped host memory: kernels write it, sync() reads it without a copy
    if (cudaHostAlloc((void **)&ctx->host_status, 64, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void **)&ctx->dev_status, ctx->host_status, 0) != cudaSuccess) {
        if (ctx->host_status) cudaFreeHost(ctx->host_status);
        if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
        delete ctx;
        return OJAS_B200_E_CUDA;
    }
    memset(ctx->host_status, 0, 64);
    if (cudaMalloc((void **)&ctx->gemm_flags, (OJAS_GEMM_FLAG_WORDS + 1) * sizeof(unsigned int)) != cudaSuccess ||
        cudaMemset(ctx->gemm_flags, 0, (OJAS_GEMM_FLAG_WORDS + 1) * sizeof(unsigned int)) != cudaSuccess ||
        cudaMalloc(&ctx->act_scratch, OJAS_ACT_SCRATCH_BYTES) != cudaSuccess) {
        if (ctx->gemm_flags) cudaFree(ctx->gemm_flags);
        cudaFreeHost(ctx->host_status);
        if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
        delete ctx;
        return OJAS_B200_E_CUDA;
    }
    const char *pdl = getenv("OJAS_B200_PDL");   // read once at context creation, like the engine's OJAS_* switches
    ctx->pdl = !(pdl && pdl[0] == '0');          // on unless OJAS_B200_PDL=0
    *out = ctx;
    return 0;
}

extern "C" void ojas_b200_destroy(ojas_b200_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->act_scratch) cudaFree(ctx->act_scratch);
    if (ctx->reserved) cudaFree(ctx->reserved);
    if (ctx->gemm_flags) cudaFree(ctx->gemm_flags);
    if (ctx->host_status) cudaFreeHost(ctx->host_status);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

extern "C" int ojas_b200_set_stream(ojas_b200_ctx *ctx, void *stream) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (ctx->owns_stream) {
        OJAS_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // work queued on the private stream ends before the stream goes
        cudaStreamDestroy(ctx->stream);
        ctx->owns_stream = false;
    }
    ctx->stream = (cudaStream_t)stream;
    return 0;
}

// Grow-only scratch owned by the context, for the entry points that take no workspace argument (the name-based
// prefill entries).  Allocates (and frees the smaller buffer after the stream has drained): call it at set-up, never
// on the compute path.
extern "C" int ojas_b200_reserve(ojas_b200_ctx *ctx, size_t bytes) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (bytes <= ctx->reserved_bytes) return 0;
    OJAS_CUDA(ctx, cudaSetDevice(ctx->device));
    void *p = nullptr;
    OJAS_CUDA(ctx, cudaMalloc(&p, bytes));
    if (ctx->reserved) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(ctx->reserved);
    }
    ctx->reserved = p;
    ctx->reserved_bytes = bytes;
    return 0;
}

extern "C" size_t ojas_b200_reserved_bytes(ojas_b200_ctx *ctx) { return ctx ? ctx->reserved_bytes : 0; }

extern "C" int ojas_b200_set_option(ojas_b200_ctx *ctx, const char *key, int value) {
    if (!ctx || !key) return OJAS_B200_E_ARG;
    if (!strcmp(key, "pdl")) { ctx->pdl = value != 0; return 0; }
    if (!strcmp(key, "gemv_mma")) {
        if (value < 0 || value > 1) return ojas_fail(ctx, OJAS_B200_E_ARG, "set_option: gemv_mma must be 0 or 1");
        ctx->gemv_mma = value;
        return 0;
    }
    if (!strcmp(key, "gemv_warps")) {
        if (value < 0 || value > 16 || (value & (value - 1)) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "set_option: gemv_warps must be 0 (automatic), 1, 2, 4, 8 or 16");
        ctx->gemv_warps = value;
        return 0;
    }
    if (!strcmp(key, "gemv_stages")) {
        if (value < 0 || value > 4) return ojas_fail(ctx, OJAS_B200_E_ARG, "set_option: gemv_stages must be 0 (automatic) or 1..4");
        ctx->gemv_stages = value;
        return 0;
    }
    if (!strcmp(key, "moe_i8")) { ctx->moe_i8 = value != 0; return 0; }
    if (!strcmp(key, "moe_gemm_rows")) {
        if (value < 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "set_option: moe_gemm_rows must be >= 0");
        ctx->moe_gemm_rows = value;
        return 0;
    }
    if (!strcmp(key, "gemm_ksplit")) {
        if (value < 0 || value > 64) return ojas_fail(ctx, OJAS_B200_E_ARG, "set_option: gemm_ksplit must be 0..64");
        ctx->gemm_ksplit = value;
        return 0;
    }
    return ojas_fail(ctx, OJAS_B200_E_ARG, "set_option: unknown key '%s'", key);
}

extern "C" void *ojas_b200_stream(ojas_b200_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }
extern "C" const char *ojas_b200_last_error(ojas_b200_ctx *ctx) { return ctx ? ctx->err : "null context"; }
extern "C" int ojas_b200_sm_count(ojas_b200_ctx *ctx) { return ctx ? ctx->sm_count : 0; }
extern "C" uint64_t ojas_b200_launch_count(ojas_b200_ctx *ctx) { return ctx ? ctx->launches : 0; }

extern "C" int ojas_b200_alloc(ojas_b200_ctx *ctx, size_t bytes, void **dptr) {
    if (!ctx || !dptr) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaSetDevice(ctx->device));
    OJAS_CUDA(ctx, cudaMalloc(dptr, bytes ? bytes : 1));
    return 0;
}

extern "C" int ojas_b200_free(ojas_b200_ctx *ctx, void *dptr) {
    if (!ctx) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaFree(dptr));
    return 0;
}

extern "C" int ojas_b200_upload(ojas_b200_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes) {
    if (!ctx || (bytes && (!dst_dev || !src_host))) return ctx ? ojas_fail(ctx, OJAS_B200_E_ARG, "upload: null pointer") : OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return 0;
}

extern "C" int ojas_b200_download(ojas_b200_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes) {
    if (!ctx || (bytes && (!dst_host || !src_dev))) return ctx ? ojas_fail(ctx, OJAS_B200_E_ARG, "download: null pointer") : OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return 0;
}

extern "C" int ojas_b200_memset(ojas_b200_ctx *ctx, void *dst_dev, int value, size_t bytes) {
    if (!ctx || (bytes && !dst_dev)) return ctx ? ojas_fail(ctx, OJAS_B200_E_ARG, "memset: null pointer") : OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaMemsetAsync(dst_dev, value, bytes, ctx->stream));
    return 0;
}

// submit(): wait for the stream; also surfaces a device status word set by a kernel whose
// bounded wait ran out (no kernel of this library traps or spins without a limit).
extern "C" int ojas_b200_sync(ojas_b200_ctx *ctx) {
    if (!ctx) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const unsigned int st = *(volatile unsigned int *)ctx->host_status;
    if (st != 0) {
        *(volatile unsigned int *)ctx->host_status = 0;
        return ojas_fail(ctx, OJAS_B200_E_DEVICE, "a kernel gave up a bounded wait (status word 0x%x)", st);
    }
    return 0;
}

// ---------------------------------------------------------------------------- events and graphs
extern "C" int ojas_b200_event_create(ojas_b200_ctx *ctx, void **event) {
    if (!ctx || !event) return OJAS_B200_E_ARG;
    cudaEvent_t ev;
    OJAS_CUDA(ctx, cudaEventCreate(&ev));
    *event = (void *)ev;
    return 0;
}

extern "C" int ojas_b200_event_destroy(ojas_b200_ctx *ctx, void *event) {
    if (!ctx) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaEventDestroy((cudaEvent_t)event));
    return 0;
}

extern "C" int ojas_b200_event_record(ojas_b200_ctx *ctx, void *event) {
    if (!ctx || !event) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaEventRecord((cudaEvent_t)event, ctx->stream));
    return 0;
}

extern "C" int ojas_b200_event_elapsed_ms(ojas_b200_ctx *ctx, void *start, void *stop, float *ms) {
    if (!ctx || !start || !stop || !ms) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaEventSynchronize((cudaEvent_t)stop));
    OJAS_CUDA(ctx, cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return 0;
}

extern "C" int ojas_b200_graph_begin(ojas_b200_ctx *ctx) {
    if (!ctx) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    return 0;
}

extern "C" int ojas_b200_graph_end(ojas_b200_ctx *ctx, void **graph_exec) {
    if (!ctx || !graph_exec) return OJAS_B200_E_ARG;
    cudaGraph_t graph = nullptr;
    OJAS_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &graph));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return ojas_fail(ctx, OJAS_B200_E_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    *graph_exec = (void *)exec;
    return 0;
}

extern "C" int ojas_b200_graph_launch(ojas_b200_ctx *ctx, void *graph_exec) {
    if (!ctx || !graph_exec) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaGraphLaunch((cudaGraphExec_t)graph_exec, ctx->stream));
    return 0;
}

extern "C" int ojas_b200_graph_destroy(ojas_b200_ctx *ctx, void *graph_exec) {
    if (!ctx) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
    return 0;
}

// Pinned host memory for the end-to-end path (activations in, results out).
extern "C" int ojas_b200_host_alloc(ojas_b200_ctx *ctx, size_t bytes, void **hptr) {
    if (!ctx || !hptr) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaHostAlloc(hptr, bytes ? bytes : 1, cudaHostAllocDefault));
    return 0;
}

extern "C" int ojas_b200_host_free(ojas_b200_ctx *ctx, void *hptr) {
    if (!ctx) return OJAS_B200_E_ARG;
    OJAS_CUDA(ctx, cudaFreeHost(hptr));
    return 0;
}
