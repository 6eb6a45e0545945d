// Standalone q4_0 x q8_0 GEMV over a stack of equal matrices (one launch), plus
// the integer block-sum dump used for bit-exact parity checks.
#include "gemv_core.cuh"
#include <mutex>

namespace mi {

struct GemvIO {
    const int8_t* xq; const __half* xd;     // activations [nb*32], [nb]
    const float* bias;                      // [rows] or null
    float* y; long long y_stride; int rows; // y[c*y_stride + r]
    int32_t* isum_out;                      // DUMP only
    int* err;
};

template <int KB, int NW, int S, bool DUMP>
__global__ void __launch_bounds__(NW * 32, 1)
gemv_q4_q8_kernel(const __grid_constant__ GemvShape sh, const __grid_constant__ GemvScratch sc,
                  const __grid_constant__ GemvIO io) {
    extern __shared__ __align__(128) uint8_t smem[];
    using SM = GemvSmem<KB, NW, S>;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    GemvWarp<KB, NW, S> gw;
    gw.init(smem, sh, warp, lane);
    gw.prefetch(sh, lane);                   // weights do not depend on any earlier kernel
    pdl_launch_dependents();
    pdl_wait_prior();                        // activations do
    int8_t* xq_s = SM::xq(smem);
    float2* xs_s = SM::xs(smem, sh.nb);
    stage_x_q8(io.xq, io.xd, sh.nb, xq_s, xs_s, tid, NW * 32);
    __syncthreads();
    const bool ok = gw.template run<DUMP>(sh, sc, xq_s, xs_s, lane, io.isum_out,
        [&](int c, int g, int ln, float v) {
            const int r = g * 32 + ln;
            if (r < io.rows) io.y[(long long)c * io.y_stride + r] = v + (io.bias ? io.bias[r] : 0.f);
        });
    if (!ok && lane == 0) atomicMax(io.err, MI_ERR_TIMEOUT);
}

// variant -> {warps per CTA, ring stages per warp}; see launch_kb
constexpr int kNumVariants = 8;

// fixed: scratch supplied by the caller (with its capacity) instead of the context's growable buffers
struct FixedScratch { double* part; unsigned* counters; size_t part_cap, counter_cap; };

template <int KB, int NW, int S, bool DUMP>
static int launch_one(mi_ctx* ctx, const mi_weight* w, const GemvIO& io, int ksplit, const FixedScratch* fixed = nullptr) {
    using SM = GemvSmem<KB, NW, S>;
    const size_t smem = SM::bytes(w->nb);
    if (smem > (size_t)ctx->smem_optin)
        return set_error(ctx, MI_ERR_UNSUPPORTED, "gemv: %zu bytes of shared memory needed, %d available", smem, ctx->smem_optin);
    auto kern = gemv_q4_q8_kernel<KB, NW, S, DUMP>;
    static size_t smem_set[16] = {0};                  // per device: largest size already opted in
    if (smem > smem_set[ctx->device & 15]) {
        MI_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        smem_set[ctx->device & 15] = smem;
    }
    const long long base_units = (long long)w->count * w->groups;
    const long long total_warps = (long long)ctx->sm_count * NW;
    int ks = ksplit;
    if (ks <= 0) {
        ks = 1;
        if (base_units < 2 * total_warps) ks = (int)((2 * total_warps + base_units - 1) / base_units);
        if (ks > 32) ks = 32;
    }
    if (ks > w->nt) ks = w->nt;
    if (DUMP) ks = 1;
    const long long n_units = base_units * ks;
    long long ctas = (n_units + NW - 1) / NW;
    if (ctas > ctx->sm_count) ctas = ctx->sm_count;
    GemvShape sh{w->dev, (long long)w->mat_stride, (int)w->count, w->groups, w->nt, ks, w->nb, (int)w->rows};
    GemvScratch sc{nullptr, nullptr};
    if (ks > 1 && fixed) {
        if ((size_t)base_units * ks * 32 > fixed->part_cap || (size_t)base_units > fixed->counter_cap)
            return set_error(ctx, MI_ERR_LIMIT,
                             "gemv (no-allocation entry point): %lld row groups x %d K-splits need %zu partial sums and %lld counters; "
                             "the built-in scratch holds %zu and %zu", base_units, ks, (size_t)base_units * ks * 32, base_units,
                             fixed->part_cap, fixed->counter_cap);
        sc.part = fixed->part; sc.counters = fixed->counters;
        // the counters this launch uses must read zero when the kernel starts, whatever an earlier call left behind;
        // a call that is refused above, or that needs no K-split, leaves the shared scratch alone
        MI_CUDA(ctx, cudaMemsetAsync(fixed->counters, 0, (size_t)base_units * sizeof(unsigned), ctx->stream));
    } else if (ks > 1) {
        int st = ensure_scratch(ctx, (size_t)base_units * ks * 32, (size_t)base_units);
        if (st != MI_OK) return st;
        sc.part = ctx->part; sc.counters = ctx->counters;
    }
    kern<<<(unsigned)ctas, NW * 32, smem, ctx->stream>>>(sh, sc, io);
    MI_CUDA(ctx, cudaGetLastError());
    return MI_OK;
}

template <int KB, bool DUMP>
static int launch_kb(mi_ctx* ctx, const mi_weight* w, const GemvIO& io, int ksplit, int variant) {
    if (DUMP) return launch_one<KB, 8, 2, true>(ctx, w, io, 1);
    switch (variant) {
        case 0: return launch_one<KB, 8, 3, false>(ctx, w, io, ksplit);
        case 1: return launch_one<KB, 8, 4, false>(ctx, w, io, ksplit);
        case 2: return launch_one<KB, 8, 2, false>(ctx, w, io, ksplit);
        case 3: return launch_one<KB, 16, 2, false>(ctx, w, io, ksplit);
        case 4: return launch_one<KB, 4, 8, false>(ctx, w, io, ksplit);
        case 5: return launch_one<KB, 12, 3, false>(ctx, w, io, ksplit);
        case 6: return launch_one<KB, 6, 4, false>(ctx, w, io, ksplit);
        case 7: return launch_one<KB, 4, 4, false>(ctx, w, io, ksplit);
        default: return set_error(ctx, MI_ERR_INVALID, "gemv: variant %d out of range [0,%d)", variant, kNumVariants);
    }
}

template <bool DUMP>
static int launch_gemv(mi_ctx* ctx, const mi_weight* w, const GemvIO& io, int ksplit, int variant) {
    switch (w->kb) {
        case 8: return launch_kb<8, DUMP>(ctx, w, io, ksplit, variant);
        case 4: return launch_kb<4, DUMP>(ctx, w, io, ksplit, variant);
        case 2: return launch_kb<2, DUMP>(ctx, w, io, ksplit, variant);
        case 1: return launch_kb<1, DUMP>(ctx, w, io, ksplit, variant);
        default: return set_error(ctx, MI_ERR_INVALID, "gemv: bad tile depth %d", w->kb);
    }
}

// ---- scratch that needs no allocation ---------------------------------------------------
// Split-K scratch of the allocation-free entry point: partial sums and arrival counters live
// in the library image itself.  Every GPU that loads the library holds these 528 KB until the
// process exits.  In host code these names are only stand-ins for the symbols; the device
// addresses come from cudaGetSymbolAddress (see noalloc_scratch).
constexpr size_t kNoAllocPartials = 65536;        // doubles: row groups x K-splits x 32 rows
constexpr size_t kNoAllocCounters = 2048;         // one per row group of the stack
static __device__ __align__(256) double g_noalloc_part[kNoAllocPartials];
static __device__ __align__(256) unsigned g_noalloc_counters[kNoAllocCounters];

// Device addresses of the two arrays on the context's device, looked up once per device with
// that device current.  No allocation happens here or later.
static int noalloc_scratch(mi_ctx* ctx, FixedScratch* out) {
    static double* part_addr[16] = {nullptr};
    static unsigned* counter_addr[16] = {nullptr};
    if (ctx->device < 0 || ctx->device >= 16) return set_error(ctx, MI_ERR_UNSUPPORTED, "no-allocation gemv: device index %d beyond 15", ctx->device);
    static std::mutex lock;                             // two host threads may make their first call at once
    std::lock_guard<std::mutex> hold(lock);
    if (!part_addr[ctx->device]) {
        // a symbol's address is looked up on the current device: make the context's device current for the query and
        // put the caller's device back afterwards
        int prev = -1;
        MI_CUDA(ctx, cudaGetDevice(&prev));
        MI_CUDA(ctx, cudaSetDevice(ctx->device));
        double* p = nullptr; unsigned* c = nullptr;
        const cudaError_t e1 = cudaGetSymbolAddress((void**)&p, g_noalloc_part);
        const cudaError_t e2 = cudaGetSymbolAddress((void**)&c, g_noalloc_counters);
        if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
        if (e1 != cudaSuccess || e2 != cudaSuccess)
            return set_error(ctx, MI_ERR_CUDA, "no-allocation gemv: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
        part_addr[ctx->device] = p; counter_addr[ctx->device] = c;
    }
    out->part = part_addr[ctx->device]; out->counters = counter_addr[ctx->device];
    out->part_cap = kNoAllocPartials; out->counter_cap = kNoAllocCounters;
    return MI_OK;
}

}  // namespace mi

using namespace mi;

extern "C" int mi_gemv_q4_q8_noalloc(mi_ctx* ctx, const mi_weight* w, const int8_t* xq_dev, const uint16_t* xd_dev,
                                     const float* bias_dev, float* y_dev) {
    if (!ctx) return MI_ERR_INVALID;
    if (!w || !xq_dev || !xd_dev || !y_dev) return set_error(ctx, MI_ERR_INVALID, "gemv: null argument");
    if (((uintptr_t)xq_dev & 15) != 0) return set_error(ctx, MI_ERR_INVALID, "gemv: xq_dev must be 16-byte aligned");
    if (w->rows == 0 || w->count == 0) return MI_OK;
    FixedScratch fx;
    int st = noalloc_scratch(ctx, &fx);
    if (st != MI_OK) return st;
    GemvIO io{xq_dev, reinterpret_cast<const __half*>(xd_dev), bias_dev, y_dev, (long long)w->rows, (int)w->rows, nullptr, ctx->d_err};
    switch (w->kb) {
        case 8: return launch_one<8, 8, 3, false>(ctx, w, io, 0, &fx);
        case 4: return launch_one<4, 8, 3, false>(ctx, w, io, 0, &fx);
        case 2: return launch_one<2, 8, 3, false>(ctx, w, io, 0, &fx);
        case 1: return launch_one<1, 8, 3, false>(ctx, w, io, 0, &fx);
        default: return set_error(ctx, MI_ERR_INVALID, "gemv: bad tile depth %d", w->kb);
    }
}

extern "C" int mi_gemv_q4_q8_ex(mi_ctx* ctx, const mi_weight* w, const int8_t* xq_dev, const uint16_t* xd_dev,
                                const float* bias_dev, float* y_dev, int ksplit, int variant) {
    if (!ctx) return MI_ERR_INVALID;
    if (!w || !xq_dev || !xd_dev || !y_dev) return set_error(ctx, MI_ERR_INVALID, "gemv: null argument");
    if (((uintptr_t)xq_dev & 15) != 0) return set_error(ctx, MI_ERR_INVALID, "gemv: xq_dev must be 16-byte aligned");
    if (w->rows == 0 || w->count == 0) return MI_OK;
    GemvIO io{xq_dev, reinterpret_cast<const __half*>(xd_dev), bias_dev, y_dev, (long long)w->rows, (int)w->rows, nullptr, ctx->d_err};
    return launch_gemv<false>(ctx, w, io, ksplit, variant);
}

extern "C" int mi_gemv_q4_q8(mi_ctx* ctx, const mi_weight* w, const int8_t* xq_dev, const uint16_t* xd_dev,
                             const float* bias_dev, float* y_dev) {
    return mi_gemv_q4_q8_ex(ctx, w, xq_dev, xd_dev, bias_dev, y_dev, 0, 0);
}

extern "C" int mi_block_isums_q4_q8(mi_ctx* ctx, const mi_weight* w, const int8_t* xq_dev, int32_t* isum_dev) {
    if (!ctx) return MI_ERR_INVALID;
    if (!w || !xq_dev || !isum_dev) return set_error(ctx, MI_ERR_INVALID, "block_isums: null argument");
    if (((uintptr_t)xq_dev & 15) != 0) return set_error(ctx, MI_ERR_INVALID, "block_isums: xq_dev must be 16-byte aligned");
    if (w->rows == 0) return MI_OK;
    // the scales do not enter the integer sums: stage zeros for xd, and a throw-away y
    const size_t xd_bytes = (((size_t)w->nb * 2 + 15) / 16) * 16, total = xd_bytes + (size_t)w->groups * 32 * 4;
    int st = ensure_staging(ctx, 0, total);
    if (st != MI_OK) return st;
    MI_CUDA(ctx, cudaMemsetAsync(ctx->d_stage, 0, total, ctx->stream));
    float* ytmp = reinterpret_cast<float*>((uint8_t*)ctx->d_stage + xd_bytes);
    mi_weight one = *w; one.count = 1;
    GemvIO io{xq_dev, reinterpret_cast<const __half*>(ctx->d_stage), nullptr, ytmp, (long long)w->rows, (int)w->rows, isum_dev, ctx->d_err};
    return launch_gemv<true>(ctx, &one, io, 1, 0);
}

namespace mi { int launch_quant_q8(mi_ctx* ctx, const float* x, long long n_blocks, int8_t* xq, __half* xd); }

extern "C" int mi_gemv_q4_f32_host(mi_ctx* ctx, const mi_weight* w, const float* x_host, const float* bias_dev,
                                   float* y_host) {
    if (!ctx) return MI_ERR_INVALID;
    if (!w || !x_host || !y_host) return set_error(ctx, MI_ERR_INVALID, "gemv_host: null argument");
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t xb = (size_t)w->cols * 4, yb = (size_t)w->count * w->rows * 4;
    const size_t off_xq = (xb + 255) / 256 * 256, off_xd = off_xq + ((size_t)w->cols + 255) / 256 * 256;
    const size_t off_y = off_xd + ((size_t)w->nb * 2 + 255) / 256 * 256;
    int st = ensure_staging(ctx, xb > yb ? xb : yb, off_y + yb);
    if (st != MI_OK) return st;
    uint8_t* d = (uint8_t*)ctx->d_stage;
    memcpy(ctx->h_pinned, x_host, xb);
    MI_CUDA(ctx, cudaMemcpyAsync(d, ctx->h_pinned, xb, cudaMemcpyHostToDevice, ctx->stream));
    st = launch_quant_q8(ctx, (const float*)d, w->nb, (int8_t*)(d + off_xq), (__half*)(d + off_xd));
    if (st != MI_OK) return st;
    st = mi_gemv_q4_q8(ctx, w, (const int8_t*)(d + off_xq), (const uint16_t*)(d + off_xd), bias_dev, (float*)(d + off_y));
    if (st != MI_OK) return st;
    MI_CUDA(ctx, cudaMemcpyAsync(ctx->h_pinned, d + off_y, yb, cudaMemcpyDeviceToHost, ctx->stream));
    MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    memcpy(y_host, ctx->h_pinned, yb);
    return MI_OK;
}
