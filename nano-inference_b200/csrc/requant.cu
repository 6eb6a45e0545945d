// Load-time re-quantizer: weight matrices that a model file stores as Q4_1, Q8_0 or Q6_K blocks become row-major q4_0
// blocks on the device, which the repack kernels then tile like any stored q4_0 tensor.
//
// The arithmetic is the reference loader's, done there on the host one row at a time: dequantize the row
// (src/gguf.h:103-140), then quantize each 32 values symmetrically with d = amax / 7, q = clamp(lrintf(y / d) + 8, 0, 15)
// and d stored as fp16 (src/mega.cu:924-936, 986-993; the same rule as src/cuda_infer.cu:814-842).  Every product of the
// dequantization is exact in fp32 (at most 11 x 7 x 6 significant bits), so the result does not depend on whether a
// compiler contracts it; the device code uses explicitly rounded operations and matches the host code bit for bit.
#include "mi_internal.cuh"

namespace mi {

namespace {

// value of element `lane` of 32-element block `b` of a tensor stored as `type` blocks
template <int TYPE>
__device__ __forceinline__ float block_value(const uint8_t* __restrict__ src, long long b, int lane) {
    if (TYPE == 3) {                                     // Q4_1: fp16 d, fp16 m, 16 nibble bytes; y = q * d + m
        const uint8_t* p = src + b * 20;
        const float d = __half2float(*reinterpret_cast<const __half*>(p)), m = __half2float(*reinterpret_cast<const __half*>(p + 2));
        const uint8_t byte = p[4 + (lane & 15)];
        return __fadd_rn(__fmul_rn(__int2float_rn(lane < 16 ? (byte & 0x0F) : (byte >> 4)), d), m);
    }
    if (TYPE == 8) {                                     // Q8_0: fp16 d, 32 int8; y = q * d
        const uint8_t* p = src + b * 34;
        return __fmul_rn(__int2float_rn((int)(int8_t)p[2 + lane]), __half2float(*reinterpret_cast<const __half*>(p)));
    }
    // Q6_K: 256 elements = ql[128] (low nibbles), qh[64] (high 2 bits), int8 scales[16], fp16 d; y = d * scale * (q - 32).
    // Element e: half n = e / 128, quadrant qd = (e % 128) / 32, l = e % 32.
    const uint8_t* p = src + (b >> 3) * 210;
    const int e = (int)(b & 7) * 32 + lane, n = e >> 7, qd = (e >> 5) & 3, l = e & 31;
    const uint8_t qlb = p[64 * n + l + 32 * (qd & 1)], qhb = p[128 + 32 * n + l];
    const int q = (int)(int8_t)((qd < 2 ? (qlb & 0x0F) : (qlb >> 4)) | (((qhb >> (2 * qd)) & 3) << 4)) - 32;
    const int sc = (int)(int8_t)p[192 + 8 * n + (l >> 4) + 2 * qd];
    const float d = __half2float(*reinterpret_cast<const __half*>(p + 208));
    return __fmul_rn(__fmul_rn(d, __int2float_rn(sc)), __int2float_rn(q));
}

// one warp per 32-element output block
template <int TYPE>
__global__ void __launch_bounds__(256) requant_q4_0_kernel(const uint8_t* __restrict__ src, long long nblk, uint8_t* __restrict__ dst) {
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long b = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < nblk; b += warps) {
        const float y = block_value<TYPE>(src, b, lane);
        float amax = fabsf(y);
        #pragma unroll
        for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float d = __fdiv_rn(amax, 7.f), inv = d > 0.f ? __fdiv_rn(1.f, d) : 0.f;
        int q = __float2int_rn(__fmul_rn(y, inv)) + 8;             // round to nearest even, as lrintf does
        q = min(15, max(0, q));
        const int hi = __shfl_down_sync(0xffffffffu, q, 16);
        uint8_t* o = dst + b * 18;
        if (lane < 16) o[2 + lane] = (uint8_t)(q | (hi << 4));
        if (lane == 0) *reinterpret_cast<__half*>(o) = __float2half_rn(d);
    }
}

}  // namespace

int launch_requant_q4_0(mi_ctx* ctx, int type, const void* src_dev, long long rows, long long cols, void* dst_dev) {
    const int epb = type == 14 ? 256 : 32;
    if (type != 3 && type != 8 && type != 14) return set_error(ctx, MI_ERR_UNSUPPORTED, "requant: ggml type %d is not one of Q4_1 (3), Q8_0 (8), Q6_K (14)", type);
    if (rows < 0 || cols < 0 || cols % epb) return set_error(ctx, MI_ERR_INVALID, "requant: %lld columns are not a multiple of the %d-element block", cols, epb);
    const long long nblk = rows * (cols / 32);
    if (nblk == 0) return MI_OK;
    const unsigned grid = (unsigned)std::min<long long>((nblk + 7) / 8, (long long)ctx->sm_count * 16);
    const uint8_t* s = static_cast<const uint8_t*>(src_dev); uint8_t* d = static_cast<uint8_t*>(dst_dev);
    if (type == 3) requant_q4_0_kernel<3><<<grid, 256, 0, ctx->stream>>>(s, nblk, d);
    else if (type == 8) requant_q4_0_kernel<8><<<grid, 256, 0, ctx->stream>>>(s, nblk, d);
    else requant_q4_0_kernel<14><<<grid, 256, 0, ctx->stream>>>(s, nblk, d);
    MI_CUDA(ctx, cudaGetLastError());
    return MI_OK;
}

}  // namespace mi

// Re-quantizes `rows` x `cols` weights stored as ggml type `type` (device bytes, rows contiguous) into row-major q4_0 blocks
// (18 bytes per 32 columns) at dst_dev.  Asynchronous on the context's stream.
extern "C" int mi_requant_q4_0(mi_ctx* ctx, int type, const void* src_dev, int64_t rows, int64_t cols, void* dst_dev) {
    if (!ctx) return MI_ERR_INVALID;
    if (!src_dev || !dst_dev) return mi::set_error(ctx, MI_ERR_INVALID, "requant: null pointer");
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    return mi::launch_requant_q4_0(ctx, type, src_dev, rows, cols, dst_dev);
}
