// q8_0 activation quantizer (per 32-element block): eight lanes per block, four elements per
// lane (one 16-byte load, one 4-byte store), a warp handles four blocks per trip of a
// grid-stride loop sized to the machine.
#include "mi_internal.cuh"

namespace mi {

// a = max|x| over the block, inv = a > 0 ? 127/a : 0, xq = rint(x*inv) (round half to even),
// xd = fp16(a/127): the arithmetic of the reference's quant_x_q8 (src/cuda_infer.cu:80-89).
__global__ void __launch_bounds__(256) quant_q8_kernel(const float* __restrict__ x, long long n_blocks, int8_t* __restrict__ xq,
                                                       __half* __restrict__ xd) {
    const int lane = threadIdx.x & 31, sub = lane >> 3, li = lane & 7;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5), w0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    for (long long b4 = w0 * 4; b4 < n_blocks; b4 += warps * 4) {
        const long long blk = b4 + sub;
        const bool live = blk < n_blocks;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) v = __ldg(reinterpret_cast<const float4*>(x + blk * 32) + li);
        float a = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        #pragma unroll
        for (int o = 4; o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        const float inv = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
        const int q0 = __float2int_rn(__fmul_rn(v.x, inv)), q1 = __float2int_rn(__fmul_rn(v.y, inv));
        const int q2 = __float2int_rn(__fmul_rn(v.z, inv)), q3 = __float2int_rn(__fmul_rn(v.w, inv));
        if (live) {
            reinterpret_cast<unsigned*>(xq + blk * 32)[li] = (unsigned)(q0 & 255) | ((unsigned)(q1 & 255) << 8) | ((unsigned)(q2 & 255) << 16) | ((unsigned)(q3 & 255) << 24);
            if (li == 0) xd[blk] = __float2half_rn(__fdiv_rn(a, 127.f));
        }
    }
}

int launch_quant_q8(mi_ctx* ctx, const float* x, long long n_blocks, int8_t* xq, __half* xd) {
    if (n_blocks == 0) return MI_OK;
    const long long want = (n_blocks + 31) / 32;                       // CTAs if every warp made one trip
    const long long cap = (long long)ctx->sm_count * 8;                 // full occupancy; larger inputs loop
    quant_q8_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, ctx->stream>>>(x, n_blocks, xq, xd);
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
