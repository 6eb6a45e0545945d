// Device-side repack of GGUF q4_0 blocks into the tiled streaming layout, and its inverse.
#include "mi_internal.cuh"
#include <cstdarg>

namespace mi {

// One thread per (packed row, block).  raw holds 18-byte blocks (9 halfwords:
// fp16 scale, then 16 nibble bytes), row-major, only 2-byte aligned.
__global__ void repack_q4_0_kernel(const uint16_t* __restrict__ raw, uint8_t* __restrict__ tiled, long long rows,
                                   int nb, int kb, int nt, int groups, long long mat_stride, long long count) {
    const long long per_mat = (long long)groups * 32 * nb;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= per_mat * count) return;
    const long long c = idx / per_mat, rem = idx % per_mat;
    const int b = (int)(rem % nb);
    const long long p = rem / nb;                        // packed row
    const int g = (int)(p / 32), r = (int)(p % 32), t = b / kb, k = b % kb;
    uint16_t d = 0;
    uint32_t q[4] = {0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u};   // nibble 8 = value 0
    if (p < rows) {
        const uint16_t* src = raw + ((c * rows + p) * nb + b) * 9;
        d = src[0];
        #pragma unroll
        for (int i = 0; i < 4; i++) q[i] = (uint32_t)src[1 + 2 * i] | ((uint32_t)src[2 + 2 * i] << 16);
    }
    uint8_t* tile = tiled + c * mat_stride + ((size_t)g * nt + t) * tile_bytes(kb);
    *reinterpret_cast<uint4*>(tile + ((size_t)k * 32 + r) * 16) = make_uint4(q[0], q[1], q[2], q[3]);
    *reinterpret_cast<uint16_t*>(tile + (size_t)kb * 512 + ((size_t)r * kb + k) * 2) = d;
}

// Same scatter with an explicit destination row per source row (dst_row[p], or
// p + row_offset when dst_row is null): used to build fused matrices whose rows
// are permuted or interleaved (Q/K rows pair-adjacent for RoPE, gate/up groups
// alternating).  The destination must have been zero-filled (padding rows keep scale 0).
__global__ void repack_q4_0_map_kernel(const uint16_t* __restrict__ raw, uint8_t* __restrict__ tiled, long long src_rows,
                                       int nb, int kb, int nt, const int* __restrict__ dst_row, int row_offset) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= src_rows * nb) return;
    const int b = (int)(idx % nb);
    const long long p = idx / nb;
    const long long P = dst_row ? dst_row[p] : p + row_offset;
    const int g = (int)(P / 32), r = (int)(P % 32), t = b / kb, k = b % kb;
    const uint16_t* src = raw + (p * nb + b) * 9;
    uint32_t q[4];
    #pragma unroll
    for (int i = 0; i < 4; i++) q[i] = (uint32_t)src[1 + 2 * i] | ((uint32_t)src[2 + 2 * i] << 16);
    uint8_t* tile = tiled + ((size_t)g * nt + t) * tile_bytes(kb);
    *reinterpret_cast<uint4*>(tile + ((size_t)k * 32 + r) * 16) = make_uint4(q[0], q[1], q[2], q[3]);
    *reinterpret_cast<uint16_t*>(tile + (size_t)kb * 512 + ((size_t)r * kb + k) * 2) = src[0];
}

int launch_repack_map(mi_ctx* ctx, const void* raw_dev, long long src_rows, int nb, int kb, uint8_t* tiled,
                      const int* dst_row_dev, int row_offset) {
    const long long n = src_rows * nb;
    if (n == 0) return MI_OK;
    repack_q4_0_map_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(
        reinterpret_cast<const uint16_t*>(raw_dev), tiled, src_rows, nb, kb, nb / kb, dst_row_dev, row_offset);
    MI_CUDA(ctx, cudaGetLastError());
    return MI_OK;
}

__global__ void unpack_q4_0_kernel(const uint8_t* __restrict__ tiled, uint16_t* __restrict__ raw, long long rows,
                                   int nb, int kb, int nt, long long mat_stride, long long count) {
    const long long per_mat = rows * nb;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= per_mat * count) return;
    const long long c = idx / per_mat, rem = idx % per_mat;
    const int b = (int)(rem % nb);
    const long long p = rem / nb;
    const int g = (int)(p / 32), r = (int)(p % 32), t = b / kb, k = b % kb;
    const uint8_t* tile = tiled + c * mat_stride + ((size_t)g * nt + t) * tile_bytes(kb);
    const uint4 q = *reinterpret_cast<const uint4*>(tile + ((size_t)k * 32 + r) * 16);
    const uint16_t d = *reinterpret_cast<const uint16_t*>(tile + (size_t)kb * 512 + ((size_t)r * kb + k) * 2);
    uint16_t* dst = raw + ((c * rows + p) * nb + b) * 9;
    dst[0] = d;
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    #pragma unroll
    for (int i = 0; i < 4; i++) { dst[1 + 2 * i] = (uint16_t)(w[i] & 0xFFFFu); dst[2 + 2 * i] = (uint16_t)(w[i] >> 16); }
}

static int alloc_weight(mi_ctx* ctx, int64_t rows, int64_t cols, int64_t count, mi_weight** out) {
    if (!out) return set_error(ctx, MI_ERR_INVALID, "weight: null output handle");
    *out = nullptr;
    if (rows < 0 || cols < 0 || count < 0) return set_error(ctx, MI_ERR_INVALID, "weight: negative size");
    if (cols % 32 != 0) return set_error(ctx, MI_ERR_INVALID, "weight: cols=%lld is not a multiple of 32", (long long)cols);
    if (cols > 32768) return set_error(ctx, MI_ERR_UNSUPPORTED, "weight: cols=%lld exceeds 32768", (long long)cols);
    mi_weight* w = new (std::nothrow) mi_weight();
    if (!w) return set_error(ctx, MI_ERR_NOMEM, "weight: host allocation failed");
    w->rows = rows; w->cols = cols; w->count = count;
    w->nb = (int)(cols / 32); w->kb = w->nb ? choose_kb(w->nb) : 1; w->nt = w->nb / w->kb;
    w->groups = (int)((rows + 31) / 32);
    w->mat_stride = (size_t)w->groups * w->nt * tile_bytes(w->kb);
    w->bytes = w->mat_stride * (size_t)count;
    if (w->bytes) {
        cudaError_t e = cudaMalloc(&w->dev, w->bytes);
        if (e != cudaSuccess) { delete w; return set_error(ctx, MI_ERR_NOMEM, "weight: cudaMalloc(%zu) failed: %s", w->bytes, cudaGetErrorString(e)); }
    }
    *out = w;
    return MI_OK;
}

}  // namespace mi

using namespace mi;

extern "C" int mi_weight_repack_q4_0_dev(mi_ctx* ctx, const void* raw_dev, int64_t rows, int64_t cols, int64_t count,
                                         mi_weight** out) {
    if (!ctx) return MI_ERR_INVALID;
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    int st = alloc_weight(ctx, rows, cols, count, out);
    if (st != MI_OK) return st;
    mi_weight* w = *out;
    if (w->bytes == 0) return MI_OK;
    if (!raw_dev) { mi_weight_free(ctx, w); *out = nullptr; return set_error(ctx, MI_ERR_INVALID, "weight: null raw pointer"); }
    const long long n = (long long)w->groups * 32 * w->nb * count;
    const int threads = 256;
    repack_q4_0_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, ctx->stream>>>(
        reinterpret_cast<const uint16_t*>(raw_dev), w->dev, rows, w->nb, w->kb, w->nt, w->groups, (long long)w->mat_stride, count);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) { mi_weight_free(ctx, w); *out = nullptr; return set_error(ctx, MI_ERR_CUDA, "weight repack failed: %s", cudaGetErrorString(e)); }
    return MI_OK;
}

extern "C" int mi_weight_upload_q4_0(mi_ctx* ctx, const void* raw_host, int64_t rows, int64_t cols, int64_t count,
                                     mi_weight** out) {
    if (!ctx) return MI_ERR_INVALID;
    if (!out) return set_error(ctx, MI_ERR_INVALID, "weight: null output handle");
    *out = nullptr;
    if (rows < 0 || cols < 0 || count < 0 || cols % 32 != 0)
        return set_error(ctx, MI_ERR_INVALID, "weight: bad shape %lld x %lld x %lld (cols must be a multiple of 32)",
                         (long long)count, (long long)rows, (long long)cols);
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t raw_bytes = (size_t)count * rows * (cols / 32) * 18;
    if (raw_bytes == 0) return mi_weight_repack_q4_0_dev(ctx, nullptr, rows, cols, count, out);
    if (!raw_host) return set_error(ctx, MI_ERR_INVALID, "weight: null raw pointer");
    void* tmp = nullptr;
    cudaError_t e = cudaMalloc(&tmp, raw_bytes);
    if (e != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "weight: cudaMalloc(%zu) for the raw blocks failed: %s", raw_bytes, cudaGetErrorString(e));
    e = cudaMemcpyAsync(tmp, raw_host, raw_bytes, cudaMemcpyHostToDevice, ctx->stream);
    int st = e == cudaSuccess ? mi_weight_repack_q4_0_dev(ctx, tmp, rows, cols, count, out)
                              : set_error(ctx, MI_ERR_CUDA, "weight upload failed: %s", cudaGetErrorString(e));
    cudaStreamSynchronize(ctx->stream);
    cudaFree(tmp);
    return st;
}

extern "C" int mi_weight_download_q4_0(mi_ctx* ctx, const mi_weight* w, void* raw_host) {
    if (!ctx) return MI_ERR_INVALID;
    if (!w || !raw_host) return set_error(ctx, MI_ERR_INVALID, "weight download: null argument");
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t raw_bytes = (size_t)w->count * w->rows * w->nb * 18;
    if (raw_bytes == 0) return MI_OK;
    void* tmp = nullptr;
    cudaError_t e = cudaMalloc(&tmp, raw_bytes);
    if (e != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "weight download: cudaMalloc(%zu) failed", raw_bytes);
    const long long n = (long long)w->rows * w->nb * w->count;
    unpack_q4_0_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(w->dev, reinterpret_cast<uint16_t*>(tmp), w->rows,
                                                                          w->nb, w->kb, w->nt, (long long)w->mat_stride, w->count);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(raw_host, tmp, raw_bytes, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(tmp);
    if (e != cudaSuccess) return set_error(ctx, MI_ERR_CUDA, "weight download failed: %s", cudaGetErrorString(e));
    return MI_OK;
}

extern "C" int mi_weight_free(mi_ctx* ctx, mi_weight* w) {
    (void)ctx;
    if (!w) return MI_OK;
    if (w->dev) cudaFree(w->dev);
    delete w;
    return MI_OK;
}

extern "C" int mi_weight_info(const mi_weight* w, int64_t* rows, int64_t* cols, int64_t* count, int64_t* device_bytes) {
    if (!w) return MI_ERR_INVALID;
    if (rows) *rows = w->rows;
    if (cols) *cols = w->cols;
    if (count) *count = w->count;
    if (device_bytes) *device_bytes = (int64_t)w->bytes;
    return MI_OK;
}
