// Internal declarations shared by the .cu files of libminfer_b200 (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <string>
#include "../../include/minfer_b200.h"

// ---- host-side objects behind the opaque C handles ---------------------------

struct mi_ctx {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    int smem_optin = 0;
    int* d_err = nullptr;            // device error word (0 = none)
    unsigned long long wait_ns = 2000000000ull;   // time budget of the decode kernel's device-side waits (mi_ctx_set_wait_budget_ns)
    unsigned long long errors_reported = 0;       // device errors that mi_ctx_sync has reported so far
    // scratch of the split-K GEMV: partial sums and self-resetting arrival counters
    double* part = nullptr; size_t part_count = 0;
    unsigned* counters = nullptr; size_t n_counters = 0;
    // staging for the host-buffer convenience calls
    bool pdl = false;                // launches may start before their predecessor in the stream has finished (see launch_k)
    void* h_pinned = nullptr; size_t h_pinned_bytes = 0;
    void* d_stage = nullptr; size_t d_stage_bytes = 0;
    std::string last_error;
};

// Tiled q4_0 layout.  A matrix is cut into groups of 32 consecutive rows and
// tiles of kb consecutive 32-element blocks.  Tile (g, t) is one contiguous run
// of kb*576 bytes at ((g*nt + t) * kb*576):
//     bytes [0, kb*512)         : nibbles, 16 bytes per (block k, row r) at (k*32 + r)*16
//                                 (byte j: low nibble = element j, high = element j+16, as in GGUF)
//     bytes [kb*512, kb*576)    : fp16 scales, row-major per row: (r*kb + k)*2
// Rows beyond `rows` in the last group hold zero scales.  A stack holds `count`
// such matrices `mat_stride` bytes apart.
struct mi_weight {
    int64_t rows = 0, cols = 0, count = 1;
    int nb = 0, kb = 0, nt = 0, groups = 0;
    size_t mat_stride = 0, bytes = 0;
    uint8_t* dev = nullptr;
};

namespace mi {

constexpr int kTileRowBytes = 576;                       // bytes per block column of a tile: 32*16 + 32*2
__host__ __device__ constexpr int tile_bytes(int kb) { return kb * kTileRowBytes; }
inline int choose_kb(int nb) { return nb % 8 == 0 ? 8 : nb % 4 == 0 ? 4 : nb % 2 == 0 ? 2 : 1; }

int set_error(mi_ctx* ctx, int status, const char* fmt, ...);
int ensure_scratch(mi_ctx* ctx, size_t part_count, size_t n_counters);
int ensure_staging(mi_ctx* ctx, size_t host_bytes, size_t dev_bytes);
int launch_repack_map(mi_ctx* ctx, const void* raw_dev, long long src_rows, int nb, int kb, uint8_t* tiled,
                      const int* dst_row_dev, int row_offset);
int launch_requant_q4_0(mi_ctx* ctx, int type, const void* src_dev, long long rows, long long cols, void* dst_dev);

// Kernel launch, optionally with programmatic stream serialization: the kernel may become resident while its
// predecessor in the stream still runs; it must execute griddepcontrol.wait (pdl_wait_prior) before it reads what the
// predecessor wrote or writes anything the predecessor may read.  Used for the launch sequence of the M-token pass.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(bool pdl, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

#define MI_CUDA(ctx, call)                                                                    \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess)                                                                \
            return mi::set_error((ctx), MI_ERR_CUDA, "%s failed at %s:%d: %s", #call, __FILE__, __LINE__, \
                                 cudaGetErrorString(e_));                                     \
    } while (0)

// ---- device helpers -----------------------------------------------------------

#ifdef __CUDACC__

// Bounded device waits give up after this many nanoseconds of %globaltimer.
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long gtime_ns() {
    unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Wait for phase `parity` of an mbarrier; false if the time budget ran out.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = gtime_ns();
    for (;;) {
        #pragma unroll 1
        for (int i = 0; i < 256; i++) if (mbar_try_wait(bar, parity)) return true;
        if (gtime_ns() - t0 > kWaitBudgetNs) return false;
    }
}
// Plain (single-CTA destination) bulk copy global -> this CTA's shared memory, completion counted
// in bytes on an mbarrier.  dst, src and bytes must be multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Same copy with an L2 eviction policy: weight tiles are read exactly once per token, so
// they are marked evict-first and do not push the KV cache, norm weights and activations
// (a few MB that every token re-reads) out of the L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
// Programmatic dependent launch: let the next kernel in the stream start its
// independent prologue; wait until the previous kernel's results are visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// One q4_0 block (16 bytes of nibbles) against 32 int8 activations: sum n_k*x_k
// with n the raw nibbles 0..15, low nibbles pairing with elements 0..15 and high
// nibbles with 16..31 (reference src/cuda_infer.cu:110-119, src/mega.cu:157-165).
__device__ __forceinline__ int dot_q4_block(const uint4 w, const int4 xa, const int4 xc) {
    const unsigned M = 0x0F0F0F0Fu;
    int a = __dp4a((int)(w.x & M), xa.x, 0);
    a = __dp4a((int)(w.y & M), xa.y, a);
    a = __dp4a((int)(w.z & M), xa.z, a);
    a = __dp4a((int)(w.w & M), xa.w, a);
    a = __dp4a((int)((w.x >> 4) & M), xc.x, a);
    a = __dp4a((int)((w.y >> 4) & M), xc.y, a);
    a = __dp4a((int)((w.z >> 4) & M), xc.z, a);
    a = __dp4a((int)((w.w >> 4) & M), xc.w, a);
    return a;
}
// Sum of the 32 int8 activations of a block.
__device__ __forceinline__ int sum_x_block(const int4 xa, const int4 xc) {
    int s = __dp4a(0x01010101, xa.x, 0);
    s = __dp4a(0x01010101, xa.y, s); s = __dp4a(0x01010101, xa.z, s); s = __dp4a(0x01010101, xa.w, s);
    s = __dp4a(0x01010101, xc.x, s); s = __dp4a(0x01010101, xc.y, s);
    s = __dp4a(0x01010101, xc.z, s); s = __dp4a(0x01010101, xc.w, s);
    return s;
}
// acc + (dw*dx) * (isum - s8), carried in double.  dw and dx are fp16 values, so
// their fp32 product is exact; isum and s8f = float(8*sum x) are integers far below
// 2^24, so their fp32 difference is exact; the product of the two is exact in
// double.  Only the running sum rounds (to 53 bits), which makes the fp32 value
// of the final sum independent of the order in which blocks are added - K-splits,
// multi-token steps and tensor-parallel shards all give the same bits.  The
// formula is the reference's (src/cuda_infer.cu:122, src/mega.cu:151-155).
__device__ __forceinline__ double blk_acc(double acc, float dw, float dx, int isum, float s8f) {
    return __fma_rn((double)__fmul_rn(dw, dx), (double)__fsub_rn(__int2float_rn(isum), s8f), acc);
}

#endif  // __CUDACC__

}  // namespace mi
