// Context, error reporting and scratch management behind the C ABI.
#include "mi_internal.cuh"
#include <cstdarg>
#include <new>

namespace mi {

int set_error(mi_ctx* ctx, int status, const char* fmt, ...) {
    if (ctx) {
        char buf[512];
        va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
        ctx->last_error = buf;
    }
    return status;
}

int ensure_scratch(mi_ctx* ctx, size_t part_count, size_t n_counters) {
    if (part_count > ctx->part_count) {
        // the stream may still be using the old buffer
        MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->part) cudaFree(ctx->part);
        ctx->part = nullptr; ctx->part_count = 0;
        size_t want = part_count * 2;
        cudaError_t e = cudaMalloc(&ctx->part, want * sizeof(double));
        if (e != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "scratch: cudaMalloc(%zu) failed: %s", want * sizeof(double), cudaGetErrorString(e));
        ctx->part_count = want;
    }
    if (n_counters > ctx->n_counters) {
        MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->counters) cudaFree(ctx->counters);
        ctx->counters = nullptr; ctx->n_counters = 0;
        size_t want = n_counters * 2;
        cudaError_t e = cudaMalloc(&ctx->counters, want * sizeof(unsigned));
        if (e != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "scratch: cudaMalloc(%zu) failed: %s", want * sizeof(unsigned), cudaGetErrorString(e));
        MI_CUDA(ctx, cudaMemset(ctx->counters, 0, want * sizeof(unsigned)));
        MI_CUDA(ctx, cudaStreamSynchronize(cudaStreamLegacy));          // the context's stream does not wait for the legacy stream
        ctx->n_counters = want;
    }
    return MI_OK;
}

int ensure_staging(mi_ctx* ctx, size_t host_bytes, size_t dev_bytes) {
    if (host_bytes > ctx->h_pinned_bytes) {
        MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->h_pinned) cudaFreeHost(ctx->h_pinned);
        ctx->h_pinned = nullptr; ctx->h_pinned_bytes = 0;
        cudaError_t e = cudaMallocHost(&ctx->h_pinned, host_bytes);
        if (e != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "staging: cudaMallocHost(%zu) failed: %s", host_bytes, cudaGetErrorString(e));
        ctx->h_pinned_bytes = host_bytes;
    }
    if (dev_bytes > ctx->d_stage_bytes) {
        MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->d_stage) cudaFree(ctx->d_stage);
        ctx->d_stage = nullptr; ctx->d_stage_bytes = 0;
        cudaError_t e = cudaMalloc(&ctx->d_stage, dev_bytes);
        if (e != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "staging: cudaMalloc(%zu) failed: %s", dev_bytes, cudaGetErrorString(e));
        ctx->d_stage_bytes = dev_bytes;
    }
    return MI_OK;
}

}  // namespace mi

using namespace mi;

extern "C" const char* mi_version(void) { return "minfer_b200 0.1 (sm_100a)"; }

extern "C" const char* mi_strerror(int status) {
    switch (status) {
        case MI_OK: return "ok";
        case MI_ERR_INVALID: return "invalid argument";
        case MI_ERR_CUDA: return "CUDA runtime error";
        case MI_ERR_NOMEM: return "out of memory";
        case MI_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case MI_ERR_IO: return "I/O error";
        case MI_ERR_FORMAT: return "malformed model file";
        case MI_ERR_UNSUPPORTED: return "unsupported tensor type or shape";
        case MI_ERR_LIMIT: return "request exceeds a fixed capacity";
        default: return "unknown status";
    }
}

extern "C" int mi_ctx_create(int device, mi_ctx** out) {
    if (!out) return MI_ERR_INVALID;
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) return MI_ERR_CUDA;          // no CUDA device: there is no fallback path
    if (device < 0 || device >= n) return MI_ERR_INVALID;
    if (cudaSetDevice(device) != cudaSuccess) return MI_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return MI_ERR_CUDA;
    if (prop.major != 10) return MI_ERR_UNSUPPORTED;             // kernels are built for sm_100a only
    mi_ctx* ctx = new (std::nothrow) mi_ctx();
    if (!ctx) return MI_ERR_NOMEM;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = (int)prop.sharedMemPerBlockOptin;
    if (cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess) { delete ctx; return MI_ERR_CUDA; }
    ctx->stream = ctx->own_stream;
    if (cudaMalloc(&ctx->d_err, sizeof(int)) != cudaSuccess || cudaMemset(ctx->d_err, 0, sizeof(int)) != cudaSuccess) {
        cudaStreamDestroy(ctx->own_stream); delete ctx; return MI_ERR_NOMEM;
    }
    *out = ctx;
    return MI_OK;
}

extern "C" int mi_ctx_destroy(mi_ctx* ctx) {
    if (!ctx) return MI_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->part) cudaFree(ctx->part);
    if (ctx->counters) cudaFree(ctx->counters);
    if (ctx->d_stage) cudaFree(ctx->d_stage);
    if (ctx->h_pinned) cudaFreeHost(ctx->h_pinned);
    if (ctx->d_err) cudaFree(ctx->d_err);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return MI_OK;
}

extern "C" int mi_ctx_set_stream(mi_ctx* ctx, void* cuda_stream) {
    if (!ctx) return MI_ERR_INVALID;
    ctx->stream = cuda_stream ? (cudaStream_t)cuda_stream : ctx->own_stream;   // cudaStreamLegacy is (void*)1
    return MI_OK;
}

extern "C" int mi_ctx_sync(mi_ctx* ctx) {
    if (!ctx) return MI_ERR_INVALID;
    MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    int err = 0;
    MI_CUDA(ctx, cudaMemcpy(&err, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost));
    if (err != 0) {
        // a kernel that gave up may have left the self-resetting arrival counters of the split-K GEMV partly counted
        ctx->errors_reported++;
        MI_CUDA(ctx, cudaMemset(ctx->d_err, 0, sizeof(int)));
        if (ctx->counters) MI_CUDA(ctx, cudaMemset(ctx->counters, 0, ctx->n_counters * sizeof(unsigned)));
        MI_CUDA(ctx, cudaStreamSynchronize(cudaStreamLegacy));
        return set_error(ctx, err, "device reported: %s", mi_strerror(err));
    }
    return MI_OK;
}

extern "C" int mi_ctx_set_wait_budget_ns(mi_ctx* ctx, unsigned long long ns) {
    if (!ctx) return MI_ERR_INVALID;
    if (ns == 0) return set_error(ctx, MI_ERR_INVALID, "wait budget must be positive");
    ctx->wait_ns = ns;
    return MI_OK;
}

extern "C" const char* mi_last_error(const mi_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }
extern "C" int mi_ctx_sm_count(const mi_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

extern "C" int mi_device_malloc(mi_ctx* ctx, size_t bytes, void** out_dev) {
    if (!ctx) return MI_ERR_INVALID;
    if (!out_dev) return set_error(ctx, MI_ERR_INVALID, "device_malloc: null output");
    *out_dev = nullptr;
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaError_t e = cudaMalloc(out_dev, bytes ? bytes : 1);
    if (e != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "device_malloc(%zu): %s", bytes, cudaGetErrorString(e));
    return MI_OK;
}

extern "C" int mi_device_free(mi_ctx* ctx, void* ptr_dev) {
    if (!ctx) return MI_ERR_INVALID;
    if (!ptr_dev) return MI_OK;
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    MI_CUDA(ctx, cudaFree(ptr_dev));
    return MI_OK;
}

extern "C" int mi_memcpy_to_device(mi_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
    if (!ctx) return MI_ERR_INVALID;
    if (bytes == 0) return MI_OK;
    if (!dst_dev || !src_host) return set_error(ctx, MI_ERR_INVALID, "memcpy_to_device: null pointer");
    MI_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MI_OK;
}

extern "C" int mi_memcpy_to_host(mi_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes) {
    if (!ctx) return MI_ERR_INVALID;
    if (bytes == 0) return MI_OK;
    if (!dst_host || !src_dev) return set_error(ctx, MI_ERR_INVALID, "memcpy_to_host: null pointer");
    MI_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MI_OK;
}
