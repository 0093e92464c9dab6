// Context object and the Device-trait helpers of the C ABI (include/ojas_b200.h).
#include <stdarg.h>
#include <stdlib.h>

#include <ctype.h>

#include <string>
#include <vector>

#include "common.cuh"

// ---------------------------------------------------------------------------- per-launch profiler
// The counterpart of KernelProfile (crates/ojas-cuda/src/device.rs:275-318: events around every launch when
// OJAS_CUDA_PROFILE is set, per-kernel milliseconds printed at the end).  Here ONE event is recorded behind every
// launch and a launch is charged the time between the event before it and its own: the stream is in order, so that is
// the time the launch added to the stream (with programmatic dependent launch a kernel's prologue overlaps its
// predecessor and is charged to the predecessor).  Nothing is recorded while the stream is being captured.
struct OjasProfile {
    struct Rec { const char *name; cudaEvent_t ev; };
    struct Sum { std::string name; uint64_t launches; double ms; };
    cudaEvent_t origin = nullptr;
    std::vector<Rec> recs;
    std::vector<cudaEvent_t> spare;
    std::vector<Sum> sums;
};

static void profile_fold(ojas_b200_ctx *ctx) {                   // waits for the stream, turns the records into sums
    OjasProfile *p = ctx->prof;
    if (!p || p->recs.empty()) return;
    cudaEventSynchronize(p->recs.back().ev);
    cudaEvent_t prev = p->origin;
    for (const OjasProfile::Rec &r : p->recs) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, prev, r.ev) != cudaSuccess) ms = 0.0f;
        size_t i = 0;
        while (i < p->sums.size() && p->sums[i].name != r.name) i++;
        if (i == p->sums.size()) p->sums.push_back({r.name, 0, 0.0});
        p->sums[i].launches++;
        p->sums[i].ms += ms;
        if (prev != p->origin) p->spare.push_back(prev);
        prev = r.ev;
    }
    p->spare.push_back(p->origin);                               // the last event becomes the new origin
    p->origin = prev;
    p->recs.clear();
    cudaGetLastError();
}

void ojas_count_launch(ojas_b200_ctx *ctx, const char *name) {
    ctx->launches++;
    OjasProfile *p = ctx->prof;
    if (!p) return;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) { cudaGetLastError(); return; }
    if (p->recs.size() >= 16384) profile_fold(ctx);
    cudaEvent_t ev = nullptr;
    if (!p->spare.empty()) { ev = p->spare.back(); p->spare.pop_back(); }
    else if (cudaEventCreate(&ev) != cudaSuccess) { cudaGetLastError(); return; }
    cudaEventRecord(ev, ctx->stream);
    p->recs.push_back({name, ev});
}

static int profile_set(ojas_b200_ctx *ctx, bool on) {
    if (on == (ctx->prof != nullptr)) return 0;
    if (on) {
        OjasProfile *p = new OjasProfile();
        if (cudaEventCreate(&p->origin) != cudaSuccess) { delete p; return ojas_fail(ctx, OJAS_B200_E_CUDA, "profile: cannot create an event"); }
        cudaEventRecord(p->origin, ctx->stream);
        ctx->prof = p;
        return 0;
    }
    profile_fold(ctx);
    OjasProfile *p = ctx->prof;
    ctx->prof = nullptr;
    for (cudaEvent_t e : p->spare) cudaEventDestroy(e);
    if (p->origin) cudaEventDestroy(p->origin);
    delete p;
    return 0;
}

// "name launches total_ms avg_us" per line, largest total first; returns the length of the full text (which may exceed
// `len`: call again with a larger buffer), 0 when the profiler is off.
extern "C" size_t ojas_b200_profile_report(ojas_b200_ctx *ctx, char *buf, size_t len) {
    if (!ctx || !ctx->prof) return 0;
    profile_fold(ctx);
    std::vector<OjasProfile::Sum> v = ctx->prof->sums;
    for (size_t i = 0; i < v.size(); i++)
        for (size_t j = i + 1; j < v.size(); j++)
            if (v[j].ms > v[i].ms) std::swap(v[i], v[j]);
    std::string text;
    char line[256];
    for (const OjasProfile::Sum &s : v) {
        snprintf(line, sizeof line, "%-28s %10llu %12.3f %10.2f\n", s.name.c_str(), (unsigned long long)s.launches, s.ms,
                 s.launches ? s.ms * 1e3 / (double)s.launches : 0.0);
        text += line;
    }
    if (buf && len) {
        const size_t n = text.size() < len - 1 ? text.size() : len - 1;
        memcpy(buf, text.data(), n);
        buf[n] = 0;
    }
    return text.size();
}

extern "C" int ojas_b200_profile_reset(ojas_b200_ctx *ctx) {
    if (!ctx) return OJAS_B200_E_ARG;
    if (!ctx->prof) return 0;
    profile_fold(ctx);
    ctx->prof->sums.clear();
    return 0;
}

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
    // The option set, read once at context creation the way the engine reads its OJAS_* switches
    // (crates/ojas-core/src/config.rs:1-22, crates/ojas-cuda/src/device.rs:87-118): OJAS_B200_<OPTION>=<integer> for every
    // key of ojas_b200_set_option, e.g. OJAS_B200_PDL=0, OJAS_B200_GEMM_KSPLIT=4, OJAS_B200_PROFILE=1.  A value that the
    // option refuses is ignored.
    static const char *const keys[] = {"pdl", "gemv_mma", "gemv_warps", "gemv_stages", "gemv_kseg", "gemm_ksplit", "moe_gemm_rows", "moe_i8", "profile"};
    for (const char *key : keys) {
        char name[64] = "OJAS_B200_";
        size_t n = strlen(name);
        for (const char *c = key; *c && n + 1 < sizeof name; c++) name[n++] = (char)toupper((unsigned char)*c);
        name[n] = 0;
        const char *v = getenv(name);
        if (v && *v) ojas_b200_set_option(ctx, key, atoi(v));
    }
    ctx->err[0] = 0;
    *out = ctx;
    return 0;
}

extern "C" void ojas_b200_destroy(ojas_b200_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->prof) {
        if (getenv("OJAS_B200_PROFILE")) {                        // switched on from the environment: the report goes to stderr
            const size_t n = ojas_b200_profile_report(ctx, nullptr, 0);
            std::string text(n + 1, '\0');
            ojas_b200_profile_report(ctx, &text[0], n + 1);
            fprintf(stderr, "ojas_b200 profile (kernel, launches, total ms, avg us)\n%s", text.c_str());
        }
        profile_set(ctx, false);
    }
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
    if (!strcmp(key, "profile")) return profile_set(ctx, value != 0);
    if (!strcmp(key, "gemv_mma")) {
        if (value < 0 || value > 8) return ojas_fail(ctx, OJAS_B200_E_ARG, "set_option: gemv_mma must be 0 (never), 1 (default) or the batch size 2..8 from which the tensor-core kernel is used");
        ctx->gemv_mma = value;
        return 0;
    }
    if (!strcmp(key, "gemv_warps")) {
        if (value < 0 || value > 16 || (value & (value - 1)) != 0) return ojas_fail(ctx, OJAS_B200_E_ARG, "set_option: gemv_warps must be 0 (automatic), 1, 2, 4, 8 or 16");
        ctx->gemv_warps = value;
        return 0;
    }
    if (!strcmp(key, "gemv_kseg")) {
        if (value < 0 || value > 64) return ojas_fail(ctx, OJAS_B200_E_ARG, "set_option: gemv_kseg must be 0 (automatic), 1 (never) or a segment count up to 64");
        ctx->gemv_kseg = value;
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
