// q4_0 x q8_0 GEMM for the multi-token step (speculative verify / batched rows): the same
// sums as the GEMV for M <= 16 token vectors per weight pass, with the integer block dot
// products on the 5th-generation tensor cores (tcgen05.mma.kind::i8, accumulators in TMEM).
//
// Replaces gemv_dp4a_batch<T> (reference src/cuda_infer.cu:183-222) and mma_s8 / tile_dot
// (reference src/mega.cu:197-244, mma.sync.m16n8k32).
//
// Shape of one MMA: D[128 x N] (int32, TMEM) = A[128 x 32] (unsigned nibbles, smem) x
// B[N x 32]^T (int8 activations, smem), N = 8 or 16 tokens, K = 32 = exactly one q4_0 block,
// because every block has its own fp16 scale: the int32 result of each block is read back
// with tcgen05.ld and scaled on the CUDA cores, acc += (dw*dx) * (isum - 8*sum x) in double -
// the very expression of the GEMV, so a token's result does not depend on how many tokens
// share the pass (nor on the K-split: see blk_acc).
//
// Dataflow of a CTA (128 threads = 128 weight rows = four 32-row groups):
//   raw tiles  : lane 0 bulk-copies the four groups' tiles of K-tile t into a 2-stage ring;
//   unpack     : thread r splits its row's 16 nibble bytes of each block into low / high nibbles
//                (elements 0..15 / 16..31) and writes them as the two 16-byte K-chunks of the
//                canonical K-major core-matrix layout (8 rows x 16 bytes, no swizzle);
//   MMA        : one thread issues one MMA per block of the tile, block k into TMEM columns
//                [k*N, (k+1)*N), then commits to an mbarrier;
//   drain      : thread r = TMEM lane r reads its row's N sums per block and accumulates.
// Activations of the unit's K range wait in shared memory in the same canonical layout.
// Every wait is bounded; TMEM is always released before the kernel returns.
#include "gemv_core.cuh"

namespace mi {

constexpr int TC_THREADS = 128;
constexpr int TC_MAX_TILES = 8;            // K-tiles per unit (bounds the activation staging)

struct GemmParams {
    const uint8_t* base; long long mat_stride;
    int groups, nt, ks, nb, kb, rows;
    int M;                                   // tokens (<= N)
    const int8_t* xq; const __half* xd;      // [M][nb*32], [M][nb]
    const float* bias; float* y;             // y[m*rows + r]
    double* part; unsigned* counters;        // [sgroups][ks][N][128], [sgroups]
    int* err;
};

__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // start address, leading (K-chunk) and stride (8-row core) byte offsets in 16-byte units; version 1; no swizzle
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <int N> __device__ __forceinline__ void tmem_ld_row(uint32_t taddr, int (&v)[N]);
template <> __device__ __forceinline__ void tmem_ld_row<8>(uint32_t taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr));
}
template <> __device__ __forceinline__ void tmem_ld_row<16>(uint32_t taddr, int (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]) : "r"(taddr));
}

template <int KB, int N>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_q4_q8_tc_kernel(const __grid_constant__ GemmParams p) {
    constexpr int TB = KB * kTileRowBytes;            // one raw tile
    constexpr int RAW_STAGE = 4 * TB;                 // four row groups
    constexpr int A_BLOCK = 128 * 32;                 // unpacked bytes of one block for 128 rows
    constexpr int TMEM_COLS = KB * N < 32 ? 32 : KB * N;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* raw = smem;                                             // [2][4][TB]
    uint8_t* a_s = raw + 2 * RAW_STAGE;                              // [KB][2 K-chunks][16 cores][8 rows][16 B]
    uint8_t* b_s = a_s + KB * A_BLOCK;                               // [blocks of the unit][2][N/8][8][16 B]
    float2* xs_s = reinterpret_cast<float2*>(b_s + TC_MAX_TILES * KB * N * 32);   // [blocks][N] {dx, float(8*sum x)}
    uint64_t* bars = reinterpret_cast<uint64_t*>(xs_s + TC_MAX_TILES * KB * N);    // raw[0], raw[1], mma
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
    __shared__ int s_ok;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_init(&bars[2], 1); mbar_fence_init(); s_ok = 1; }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint64_t policy = l2_policy_evict_first();
    // instruction descriptor: D = s32, A = unsigned 8-bit (raw nibbles 0..15), B = signed 8-bit, both K-major, N, M = 128
    constexpr uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

    const int sgroups = (p.groups + 3) / 4;
    const long long n_units = (long long)sgroups * p.ks;
    int raw_issued = 0, raw_consumed = 0, mma_count = 0;
    bool ok = true;

    for (long long u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
        const int sg = (int)(u / p.ks), sp = (int)(u % p.ks);
        const int t0 = sp * p.nt / p.ks, t1 = (sp + 1) * p.nt / p.ks, nblk = (t1 - t0) * KB, b0 = t0 * KB;
        // the tile loader: four groups' tiles of K-tile t into stage s (a missing group re-reads the last one; its rows are never stored)
        auto issue_tile = [&](int t) {
            const int s = raw_issued & 1;
            mbar_expect_tx(&bars[s], RAW_STAGE);
            #pragma unroll
            for (int gi = 0; gi < 4; gi++) {
                const int g = min(sg * 4 + gi, p.groups - 1);
                bulk_g2s_hint(raw + s * RAW_STAGE + gi * TB, p.base + ((size_t)g * p.nt + t) * TB, TB, &bars[s], policy);
            }
            raw_issued++;
        };
        if (tid == 0) { issue_tile(t0); if (t0 + 1 < t1) issue_tile(t0 + 1); }
        // activations of the unit's K range: int8 into the canonical layout (tokens >= M are zero), scales next to them
        for (int i = tid; i < nblk * N * 2; i += TC_THREADS) {
            const int bl = i / (N * 2), rem = i % (N * 2), kc = rem / N, n = rem % N;
            int4 v = make_int4(0, 0, 0, 0);
            if (n < p.M) v = __ldcg(reinterpret_cast<const int4*>(p.xq + ((size_t)n * p.nb + b0 + bl) * 32 + kc * 16));
            *reinterpret_cast<int4*>(b_s + (size_t)bl * (N * 32) + kc * (N * 16) + (n >> 3) * 128 + (n & 7) * 16) = v;
        }
        for (int i = tid; i < nblk * N; i += TC_THREADS) {
            const int bl = i / N, n = i % N;
            float2 v = make_float2(0.f, 0.f);
            if (n < p.M) {
                const int4* xp = reinterpret_cast<const int4*>(p.xq + ((size_t)n * p.nb + b0 + bl) * 32);
                v = make_float2(__half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(p.xd) + (size_t)n * p.nb + b0 + bl))),
                                __int2float_rn(8 * sum_x_block(__ldcg(xp), __ldcg(xp + 1))));
            }
            xs_s[bl * N + n] = v;
        }
        double acc[N];
        #pragma unroll
        for (int n = 0; n < N; n++) acc[n] = 0.0;

        for (int t = t0; t < t1 && ok; t++) {
            const int s = raw_consumed & 1;
            if (!mbar_wait_bounded(&bars[s], (raw_consumed >> 1) & 1)) ok = false;
            // unpack this thread's row: low nibbles = elements 0..15 (K-chunk 0), high nibbles = 16..31 (K-chunk 1)
            const uint8_t* rt = raw + s * RAW_STAGE + warp * TB;
            if (ok) {
                #pragma unroll
                for (int k = 0; k < KB; k++) {
                    const uint4 w = *reinterpret_cast<const uint4*>(rt + (k * 32 + lane) * 16);
                    const unsigned Mk = 0x0F0F0F0Fu;
                    uint8_t* dst = a_s + k * A_BLOCK + (tid >> 3) * 128 + (tid & 7) * 16;
                    *reinterpret_cast<uint4*>(dst) = make_uint4(w.x & Mk, w.y & Mk, w.z & Mk, w.w & Mk);
                    *reinterpret_cast<uint4*>(dst + 2048) = make_uint4((w.x >> 4) & Mk, (w.y >> 4) & Mk, (w.z >> 4) & Mk, (w.w >> 4) & Mk);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy writes -> visible to the tensor core's reads
            tc_fence_before();
            ok = __syncthreads_and(ok ? 1 : 0) != 0;
            if (!ok) break;
            if (tid == 0) {
                tc_fence_after();
                #pragma unroll
                for (int k = 0; k < KB; k++) {
                    const uint64_t da = umma_smem_desc(smem_u32(a_s + k * A_BLOCK), 2048, 128);
                    const uint64_t db = umma_smem_desc(smem_u32(b_s + (size_t)((t - t0) * KB + k) * (N * 32)), N * 16, 128);
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                        ::"r"(tmem_base + (uint32_t)(k * N)), "l"(da), "l"(db), "r"(idesc), "r"(0u), "r"(0u) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars[2])) : "memory");
            }
            if (!mbar_wait_bounded(&bars[2], mma_count & 1)) ok = false;
            mma_count++;
            tc_fence_after();
            if (ok) {
                const uint8_t* sc = rt + KB * 512 + lane * (KB * 2);      // this row's KB fp16 scales
                #pragma unroll
                for (int k = 0; k < KB; k++) {
                    int isum[N];
                    tmem_ld_row<N>(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(k * N), isum);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const float dw = __half2float(*reinterpret_cast<const __half*>(sc + k * 2));
                    const float2* xs = xs_s + ((t - t0) * KB + k) * N;
                    #pragma unroll
                    for (int n = 0; n < N; n++) {
                        const float2 s2 = xs[n];
                        acc[n] = blk_acc(acc[n], dw, s2.x, isum[n], s2.y);
                    }
                }
            }
            raw_consumed++;
            tc_fence_before();
            ok = __syncthreads_and(ok ? 1 : 0) != 0;        // every row is done with the stage, the unpacked blocks and TMEM
            if (ok && tid == 0 && t + 2 < t1) issue_tile(t + 2);
        }
        if (!ok) break;
        // results of the unit: rows sg*128 + tid, tokens 0..M-1
        const int row = sg * 128 + tid;
        if (p.ks == 1) {
            if (row < p.rows)
                for (int n = 0; n < p.M; n++) p.y[(size_t)n * p.rows + row] = __double2float_rn(acc[n]) + (p.bias ? p.bias[row] : 0.f);
        } else {
            double* part = p.part + ((size_t)sg * p.ks + sp) * N * 128;
            #pragma unroll
            for (int n = 0; n < N; n++) __stcg(part + n * 128 + tid, acc[n]);
            __threadfence();
            __syncthreads();
            __shared__ unsigned s_prev;
            if (tid == 0) s_prev = atomicAdd(p.counters + sg, 1u);
            __syncthreads();
            if (s_prev == (unsigned)p.ks - 1) {                 // last split in: fold all of them in split order
                __threadfence();
                const double* p0 = p.part + (size_t)sg * p.ks * N * 128;
                for (int n = 0; n < p.M; n++) {
                    double s = 0.0;
                    for (int q = 0; q < p.ks; q++) s = __dadd_rn(s, __ldcg(p0 + ((size_t)q * N + n) * 128 + tid));
                    if (row < p.rows) p.y[(size_t)n * p.rows + row] = __double2float_rn(s) + (p.bias ? p.bias[row] : 0.f);
                }
                if (tid == 0) p.counters[sg] = 0;
            }
            __syncthreads();
        }
    }
    if (!ok) {
        if (tid == 0) atomicMax(p.err, MI_ERR_TIMEOUT);
        for (int i = raw_consumed; i < raw_issued; i++) (void)mbar_wait_bounded(&bars[i & 1], (i >> 1) & 1);   // copies in flight target this CTA
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
}

template <int KB, int N>
static int launch_gemm(mi_ctx* ctx, const mi_weight* w, GemmParams p) {
    constexpr int TB = KB * kTileRowBytes;
    const size_t smem = 2 * 4 * TB + (size_t)KB * 128 * 32 + (size_t)TC_MAX_TILES * KB * N * 32 + (size_t)TC_MAX_TILES * KB * N * 8 + 64;
    if (smem > (size_t)ctx->smem_optin) return set_error(ctx, MI_ERR_UNSUPPORTED, "gemm: %zu bytes of shared memory needed", smem);
    auto kern = gemm_q4_q8_tc_kernel<KB, N>;
    MI_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int sgroups = (w->groups + 3) / 4;
    int ks = (w->nt + TC_MAX_TILES - 1) / TC_MAX_TILES;                     // a unit stages at most TC_MAX_TILES K-tiles of activations
    while (ks < w->nt && (long long)sgroups * ks < ctx->sm_count) ks++;      // and every SM should get a unit
    p.ks = ks;
    if (ks > 1) {
        int st = ensure_scratch(ctx, (size_t)sgroups * ks * N * 128, (size_t)sgroups);
        if (st != MI_OK) return st;
        p.part = ctx->part; p.counters = ctx->counters;
    }
    long long ctas = (long long)sgroups * ks;
    if (ctas > 2LL * ctx->sm_count) ctas = 2LL * ctx->sm_count;
    kern<<<(unsigned)ctas, TC_THREADS, smem, ctx->stream>>>(p);
    MI_CUDA(ctx, cudaGetLastError());
    return MI_OK;
}

}  // namespace mi

using namespace mi;

extern "C" int mi_gemm_q4_q8(mi_ctx* ctx, const mi_weight* w, const int8_t* xq_dev, const uint16_t* xd_dev, int M,
                             const float* bias_dev, float* y_dev) {
    if (!ctx) return MI_ERR_INVALID;
    if (!w || !xq_dev || !xd_dev || !y_dev) return set_error(ctx, MI_ERR_INVALID, "gemm: null argument");
    if (M < 1 || M > 16) return set_error(ctx, MI_ERR_LIMIT, "gemm: M=%d tokens per pass; this entry point takes 1..16", M);
    if (((uintptr_t)xq_dev & 15) != 0) return set_error(ctx, MI_ERR_INVALID, "gemm: xq_dev must be 16-byte aligned");
    if (w->count != 1) return set_error(ctx, MI_ERR_UNSUPPORTED, "gemm: matrix stacks are not supported");
    if (w->rows == 0) return MI_OK;
    GemmParams p{w->dev, (long long)w->mat_stride, w->groups, w->nt, 1, w->nb, w->kb, (int)w->rows, M, xq_dev,
                 reinterpret_cast<const __half*>(xd_dev), bias_dev, y_dev, nullptr, nullptr, ctx->d_err};
    const bool n8 = M <= 8;
    switch (w->kb) {
        case 8: return n8 ? launch_gemm<8, 8>(ctx, w, p) : launch_gemm<8, 16>(ctx, w, p);
        case 4: return n8 ? launch_gemm<4, 8>(ctx, w, p) : launch_gemm<4, 16>(ctx, w, p);
        case 2: return n8 ? launch_gemm<2, 8>(ctx, w, p) : launch_gemm<2, 16>(ctx, w, p);
        case 1: return n8 ? launch_gemm<1, 8>(ctx, w, p) : launch_gemm<1, 16>(ctx, w, p);
        default: return set_error(ctx, MI_ERR_INVALID, "gemm: bad tile depth %d", w->kb);
    }
}
