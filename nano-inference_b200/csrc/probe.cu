// Machine probes: what this GPU gives a read-only streaming kernel and a store-to-load hop between two SMs, measured
// with the library's own access patterns.  The roofline fractions the benchmark reports are quoted against a copy figure
// (read + write); a GEMV only reads, so the read-only ceiling of the very loop shapes used here is reported beside it.
// Method after the reference's bench/roofline.cu:39-116 (16-byte loads, several in flight per thread, a buffer far larger
// than the L2) and :125-149 (its barrier probe; here the hop that replaces the barrier).
#include "mi_internal.cuh"

using namespace mi;

namespace {

// variant 0: grid-stride 16-byte loads, U independent loads in flight per thread, xor-folded so nothing is optimised away
template <int U>
__global__ void __launch_bounds__(256) probe_read_ldg(const uint4* __restrict__ buf, size_t n16, unsigned* sink) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned acc = 0;
    for (; i + (U - 1) * stride < n16; i += U * stride) {
        uint4 v[U];
        #pragma unroll
        for (int u = 0; u < U; u++) v[u] = __ldcs(buf + i + u * stride);
        #pragma unroll
        for (int u = 0; u < U; u++) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
    }
    for (; i < n16; i += stride) { const uint4 v = __ldcs(buf + i); acc ^= v.x ^ v.y ^ v.z ^ v.w; }
    if (acc == 0x9e3779b9u) *sink = acc;
}

// variant 1: the GEMV's own transport - every warp keeps a private ring of S slots of TB bytes full with single-CTA bulk
// copies (completion on an mbarrier per slot, bounded waits) and touches one word per lane of every slot
constexpr int PW = 8, PS = 3, PTB = 4608;
__global__ void __launch_bounds__(PW * 32, 1) probe_read_bulk(const uint8_t* __restrict__ buf, size_t n_tiles, unsigned* sink, int* err) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* ring = smem + (size_t)warp * PS * PTB;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)PW * PS * PTB) + warp * PS;
    if (lane == 0) { for (int s = 0; s < PS; s++) mbar_init(&bars[s], 1); mbar_fence_init(); }
    __syncwarp();
    const uint64_t policy = l2_policy_evict_first();
    const size_t stride = (size_t)gridDim.x * PW;
    size_t pt = (size_t)blockIdx.x * PW + warp, ct = pt;
    int issued = 0, consumed = 0;
    if (lane == 0) for (int s = 0; s < PS && pt < n_tiles; s++, pt += stride, issued++) {
        mbar_expect_tx(&bars[s], PTB); bulk_g2s_hint(ring + (size_t)s * PTB, buf + pt * PTB, PTB, &bars[s], policy);
    }
    unsigned acc = 0; bool ok = true;
    for (; ct < n_tiles && ok; ct += stride) {
        const int slot = consumed % PS;
        if (!mbar_wait_bounded(&bars[slot], (consumed / PS) & 1)) { ok = false; break; }
        acc ^= reinterpret_cast<const unsigned*>(ring + (size_t)slot * PTB)[lane * 36];
        consumed++;
        __syncwarp();
        if (lane == 0 && pt < n_tiles) {
            const int s = issued % PS;
            mbar_expect_tx(&bars[s], PTB); bulk_g2s_hint(ring + (size_t)s * PTB, buf + pt * PTB, PTB, &bars[s], policy);
            issued++; pt += stride;
        }
    }
    if (!ok) {
        if (lane == 0) atomicMax(err, MI_ERR_TIMEOUT);
        for (int i = consumed; i < issued; i++) (void)mbar_wait_bounded(&bars[i % PS], (i / PS) & 1);
    }
    if (acc == 0x9e3779b9u) *sink = acc;
}

// one-way latency of a tagged word from one SM to another: CTA 0 and CTA 1 answer each other's stores `iters` times
__global__ void probe_hop(unsigned long long* word, int iters, long long* cycles, int* err) {
    if (threadIdx.x != 0) return;
    const unsigned me = blockIdx.x;
    const long long t0 = clock64();
    const unsigned long long g0 = gtime_ns();
    for (unsigned i = 1; i <= (unsigned)iters; i++) {
        if ((i & 1u) == me) {
            asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(word), "l"((unsigned long long)i) : "memory");
        } else {
            unsigned long long v;
            for (unsigned it = 1;; it++) {
                asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(word) : "memory");
                if (v == i) break;
                if ((it & 1023u) == 0 && gtime_ns() - g0 > kWaitBudgetNs) { atomicMax(err, MI_ERR_TIMEOUT); return; }
            }
        }
    }
    if (me == 0) *cycles = clock64() - t0;
}

}  // namespace

extern "C" int mi_probe_read_bw(mi_ctx* ctx, size_t bytes, int variant, int repeats, float* gbs_out) {
    if (!ctx) return MI_ERR_INVALID;
    if (!gbs_out || repeats < 1 || bytes < (1u << 20)) return set_error(ctx, MI_ERR_INVALID, "probe_read_bw: bad argument");
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    bytes = bytes / PTB * PTB;
    uint8_t* buf = nullptr; unsigned* sink = nullptr;
    cudaError_t e = cudaMalloc(&buf, bytes);
    if (e != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "probe_read_bw: cudaMalloc(%zu) failed", bytes);
    struct Free { void* a; void* b; ~Free() { cudaFree(a); cudaFree(b); } };
    if (cudaMalloc(&sink, 4) != cudaSuccess) { cudaFree(buf); return set_error(ctx, MI_ERR_NOMEM, "probe_read_bw: cudaMalloc failed"); }
    Free guard{buf, sink};
    MI_CUDA(ctx, cudaMemsetAsync(buf, 0x5a, bytes, ctx->stream));
    cudaEvent_t e0, e1;
    MI_CUDA(ctx, cudaEventCreate(&e0)); MI_CUDA(ctx, cudaEventCreate(&e1));
    const size_t smem = (size_t)PW * PS * PTB + PW * PS * 8;
    if (variant == 1) MI_CUDA(ctx, cudaFuncSetAttribute(probe_read_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    float best_ms = 1e30f;
    for (int r = 0; r < repeats + 1; r++) {                 // first pass untimed; the buffer is larger than the L2, every pass comes from HBM
        MI_CUDA(ctx, cudaEventRecord(e0, ctx->stream));
        if (variant == 0) probe_read_ldg<8><<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(reinterpret_cast<const uint4*>(buf), bytes / 16, sink);
        else if (variant == 1) probe_read_bulk<<<ctx->sm_count, PW * 32, smem, ctx->stream>>>(buf, bytes / PTB, sink, ctx->d_err);
        else { cudaEventDestroy(e0); cudaEventDestroy(e1); return set_error(ctx, MI_ERR_INVALID, "probe_read_bw: variant 0 (16-byte loads) or 1 (bulk-copy ring)"); }
        MI_CUDA(ctx, cudaGetLastError());
        MI_CUDA(ctx, cudaEventRecord(e1, ctx->stream));
        MI_CUDA(ctx, cudaEventSynchronize(e1));
        float ms = 0.f; MI_CUDA(ctx, cudaEventElapsedTime(&ms, e0, e1));
        if (r > 0 && ms < best_ms) best_ms = ms;
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    int st = mi_ctx_sync(ctx);
    if (st != MI_OK) return st;
    *gbs_out = (float)((double)bytes / (best_ms * 1e-3) / 1e9);
    return MI_OK;
}

extern "C" int mi_probe_hop_ns(mi_ctx* ctx, int iters, float* ns_out) {
    if (!ctx) return MI_ERR_INVALID;
    if (!ns_out || iters < 2) return set_error(ctx, MI_ERR_INVALID, "probe_hop_ns: bad argument");
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    unsigned long long* word = nullptr; long long* cyc = nullptr;
    if (cudaMalloc(&word, 8) != cudaSuccess || cudaMalloc(&cyc, 8) != cudaSuccess) { cudaFree(word); return set_error(ctx, MI_ERR_NOMEM, "probe_hop_ns: cudaMalloc failed"); }
    struct Free { void* a; void* b; ~Free() { cudaFree(a); cudaFree(b); } } guard{word, cyc};
    MI_CUDA(ctx, cudaMemsetAsync(word, 0, 8, ctx->stream));
    MI_CUDA(ctx, cudaMemsetAsync(cyc, 0, 8, ctx->stream));
    // the two CTAs wait for each other: a cooperative launch keeps both resident
    void* args[] = {(void*)&word, (void*)&iters, (void*)&cyc, (void*)&ctx->d_err};
    MI_CUDA(ctx, cudaLaunchCooperativeKernel((const void*)probe_hop, dim3(2), dim3(32), args, 0, ctx->stream));
    int st = mi_ctx_sync(ctx);
    if (st != MI_OK) return st;
    long long h = 0;
    MI_CUDA(ctx, cudaMemcpy(&h, cyc, 8, cudaMemcpyDeviceToHost));
    int khz = 0;
    MI_CUDA(ctx, cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device));
    *ns_out = (float)((double)h / iters / ((double)khz * 1e-6));      // cycles per one-way hop / (cycles per ns at the nominal SM clock)
    return MI_OK;
}
