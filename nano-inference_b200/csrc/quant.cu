// q8_0 activation quantizer (per 32-element block), one warp per block.
#include "mi_internal.cuh"

namespace mi {

// a = max|x| over the block, inv = a > 0 ? 127/a : 0, xq = rint(x*inv) (round half to even),
// xd = fp16(a/127): the arithmetic of the reference's quant_x_q8 (src/cuda_infer.cu:80-89).
__global__ void quant_q8_kernel(const float* __restrict__ x, long long n_blocks, int8_t* __restrict__ xq,
                                __half* __restrict__ xd) {
    const long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (blk >= n_blocks) return;
    const float v = x[blk * 32 + lane];
    float a = fabsf(v);
    #pragma unroll
    for (int o = 16; o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    const float inv = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
    xq[blk * 32 + lane] = (int8_t)__float2int_rn(__fmul_rn(v, inv));
    if (lane == 0) xd[blk] = __float2half_rn(__fdiv_rn(a, 127.f));
}

int launch_quant_q8(mi_ctx* ctx, const float* x, long long n_blocks, int8_t* xq, __half* xd) {
    if (n_blocks == 0) return MI_OK;
    const int wpb = 8;
    quant_q8_kernel<<<(unsigned)((n_blocks + wpb - 1) / wpb), wpb * 32, 0, ctx->stream>>>(x, n_blocks, xq, xd);
    MI_CUDA(ctx, cudaGetLastError());
    return MI_OK;
}

}  // namespace mi

extern "C" int mi_quant_q8(mi_ctx* ctx, const float* x_dev, int64_t n, int M, int8_t* xq_dev, uint16_t* xd_dev) {
    if (!ctx) return MI_ERR_INVALID;
    if (n < 0 || M < 0 || n % 32 != 0) return mi::set_error(ctx, MI_ERR_INVALID, "quant_q8: n=%lld must be a non-negative multiple of 32", (long long)n);
    if (n == 0 || M == 0) return MI_OK;
    if (!x_dev || !xq_dev || !xd_dev) return mi::set_error(ctx, MI_ERR_INVALID, "quant_q8: null argument");
    return mi::launch_quant_q8(ctx, x_dev, (long long)(n / 32) * M, xq_dev, reinterpret_cast<__half*>(xd_dev));
}
