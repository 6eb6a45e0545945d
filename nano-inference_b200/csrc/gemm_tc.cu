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
// Dataflow of a CTA (one per SM).  All units of a CTA share one K range, so the activations
// are staged once; the CTA's units are dealt round-robin to three (two when N = 16) independent
// worker groups, each a pipeline of its own (measured: one group alone is bound by the instruction
// issue of its four warps, one per scheduler; three groups give every scheduler three warps to pick from):
//   loader warp : lane g bulk-copies group g's raw tiles (four 32-row groups of one K-tile)
//                 into that group's two-stage ring, as far ahead as the ring allows;
//   group g     : 128 threads, thread r = weight row r of the unit = TMEM lane r.  Unpack:
//                 split the row's 16 nibble bytes of each block into low / high nibbles
//                 (elements 0..15 / 16..31) and write them as the two 16-byte K-chunks of the
//                 canonical K-major core-matrix layout (8 rows x 16 bytes, no swizzle).  Drain:
//                 read the row's N int32 sums per block (tcgen05.ld) and accumulate;
//   MMA warp    : one lane polls the groups' "operand ready" barriers and issues, per tile, one
//                 MMA per block - block k into TMEM columns [k*N, (k+1)*N) of the group's
//                 accumulator - then commits to the group's "MMA done" barrier.
// While a group waits for its MMAs or its next tile, the other two run.  Every wait is bounded;
// a wait that gives up raises an abort flag that ends all roles, the copies in flight are
// waited for, and TMEM is always released before the kernel returns.
#include "gemv_core.cuh"

namespace mi {

constexpr int TC_ROWS = 128;               // weight rows per unit = threads of a worker group
constexpr int TC_RING = 2;                 // raw-tile stages per group
// worker groups, and K-tiles per unit (bounds the activation staging): what 227 KB of shared memory hold
__host__ __device__ constexpr int tc_groups(int N) { return N == 16 ? 2 : 3; }
__host__ __device__ constexpr int tc_max_tiles(int N) { return N == 16 ? 8 : 7; }
__host__ __device__ constexpr int tc_threads(int N) { return tc_groups(N) * TC_ROWS + 64; }    // + the MMA warp + the loader warp

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

// Scale of one activation block as the drain wants it: the fp16 scale as a double and 8 * (sum of the int8s).
// The drain evaluates blk_acc's expression  fma(double(dw*dx), double(float(isum) - float(8 sum x)), acc)  without its
// conversions, which would bound the kernel (two per row, block and token on a pipe that retires 16 per clock and SM):
// dw and dx are fp16 values, so their fp32 product is exact and equals double(dw) * double(dx); the bracket is an
// exact small integer, converted by the 2^52 trick.  Same bits as blk_acc.
struct XScale { double dx; int s8; int pad; };
__device__ __forceinline__ double int_to_double_exact(int v) {      // |v| < 2^31
    return __dsub_rn(__hiloint2double(0x43300000, (int)((unsigned)v ^ 0x80000000u)), 4503601774854144.0);   // 2^52 + 2^31
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
template <int WORKERS> __device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(WORKERS) : "memory"); }   // all worker groups
__device__ __forceinline__ void group_sync(int g) { asm volatile("bar.sync %0, 128;" ::"r"(2 + g) : "memory"); }      // one worker group

template <int KB, int N>
__global__ void __launch_bounds__(tc_threads(N), 1) gemm_q4_q8_tc_kernel(const __grid_constant__ GemmParams p) {
    constexpr int TC_GROUPS = tc_groups(N), TC_WORKERS = TC_GROUPS * TC_ROWS;
    constexpr int TB = KB * kTileRowBytes;            // one raw tile
    constexpr int RAW_STAGE = 4 * TB;                 // four row groups
    constexpr int A_BLOCK = 128 * 32;                 // unpacked bytes of one block for 128 rows
    constexpr int A_BUF = KB * A_BLOCK;
    constexpr int ACC_COLS = KB * N;                  // TMEM columns of one group's accumulator
    constexpr int TMEM_COLS = TC_GROUPS * ACC_COLS <= 32 ? 32 : TC_GROUPS * ACC_COLS <= 64 ? 64 : TC_GROUPS * ACC_COLS <= 128 ? 128
                            : TC_GROUPS * ACC_COLS <= 256 ? 256 : 512;
    constexpr int MAXT = tc_max_tiles(N);
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* raw = smem;                                             // [group][TC_RING][4][TB]
    uint8_t* a_s = raw + TC_GROUPS * TC_RING * RAW_STAGE;            // [group][KB][2 K-chunks][16 cores][8 rows][16 B]
    uint8_t* b_s = a_s + TC_GROUPS * A_BUF;                          // [blocks of the K range][2][N/8][8][16 B]
    XScale* xs_s = reinterpret_cast<XScale*>(b_s + MAXT * KB * N * 32);   // [blocks][N] {dx, 8*sum x}
    uint64_t* bars = reinterpret_cast<uint64_t*>(xs_s + MAXT * KB * N);
    uint64_t* raw_full = bars;                                       // [group][TC_RING]
    uint64_t* raw_empty = raw_full + TC_GROUPS * TC_RING;            // [group][TC_RING]
    uint64_t* a_full = raw_empty + TC_GROUPS * TC_RING;              // [group]
    uint64_t* mma_done = a_full + TC_GROUPS;                         // [group]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_done + TC_GROUPS);
    __shared__ int s_abort;
    __shared__ unsigned s_prev[TC_GROUPS];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < TC_GROUPS * TC_RING; s++) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], TC_ROWS); }
        for (int g = 0; g < TC_GROUPS; g++) { mbar_init(&a_full[g], TC_ROWS); mbar_init(&mma_done[g], 1); }
        mbar_fence_init();
        s_abort = 0;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();          // the next kernel in the stream may become resident; it waits for this grid to finish
    // instruction descriptor: D = s32, A = unsigned 8-bit (raw nibbles 0..15), B = signed 8-bit, both K-major, N, M = 128
    constexpr uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

    // the grid is a multiple of the K-split, so every unit of this CTA has the same K range
    const int sgroups = (p.groups + 3) / 4;
    const long long n_units = (long long)sgroups * p.ks;
    const int sp = (int)(blockIdx.x % p.ks);
    const int t0 = sp * p.nt / p.ks, t1 = (sp + 1) * p.nt / p.ks, ntile = t1 - t0, nblk = ntile * KB, b0 = t0 * KB;
    const int my_units = blockIdx.x < n_units ? (int)((n_units - 1 - blockIdx.x) / gridDim.x) + 1 : 0;
    volatile int* abort_flag = &s_abort;
    int loads_issued = 0;                                 // loader lanes only

    if (warp == TC_WORKERS / 32 + 1) {
        // ---------------- loader: lane g feeds group g
        if (lane < TC_GROUPS) {
            const int g = lane;
            const uint64_t policy = l2_policy_evict_first();
            int it = 0;
            for (int j = g; j < my_units && !*abort_flag; j += TC_GROUPS) {
                const long long u = blockIdx.x + (long long)j * gridDim.x;
                const int sg = (int)(u / p.ks);
                for (int t = t0; t < t1; t++, it++) {
                    const int s = g * TC_RING + it % TC_RING;
                    if (!mbar_wait_bounded(&raw_empty[s], ((it / TC_RING) & 1) ^ 1)) { *abort_flag = 1; break; }   // first round passes at once
                    if (*abort_flag) break;
                    mbar_expect_tx(&raw_full[s], RAW_STAGE);
                    #pragma unroll
                    for (int gi = 0; gi < 4; gi++) {                  // a missing row group re-reads the last one; its rows are never stored
                        const int rg = min(sg * 4 + gi, p.groups - 1);
                        bulk_g2s_hint(raw + s * RAW_STAGE + gi * TB, p.base + ((size_t)rg * p.nt + t) * TB, TB, &raw_full[s], policy);
                    }
                    loads_issued = it + 1;
                }
            }
        }
    } else if (warp == TC_WORKERS / 32) {
        // ---------------- MMA issuer: serves whichever group has its operands ready
        if (lane == 0) {
            int done[TC_GROUPS], total[TC_GROUPS], left = 0;
            #pragma unroll
            for (int g = 0; g < TC_GROUPS; g++) {
                done[g] = 0;
                total[g] = (my_units > g ? (my_units - 1 - g) / TC_GROUPS + 1 : 0) * ntile;
                left += total[g];
            }
            unsigned long long t_idle = gtime_ns();
            while (left > 0 && !*abort_flag) {
                bool progress = false;
                #pragma unroll
                for (int g = 0; g < TC_GROUPS; g++) {
                    if (done[g] < total[g] && mbar_try_wait(&a_full[g], done[g] & 1)) {
                        tc_fence_after();
                        const int ti = done[g] % ntile;
                        #pragma unroll
                        for (int k = 0; k < KB; k++) {
                            const uint64_t da = umma_smem_desc(smem_u32(a_s + g * A_BUF + k * A_BLOCK), 2048, 128);
                            const uint64_t db = umma_smem_desc(smem_u32(b_s + (size_t)(ti * KB + k) * (N * 32)), N * 16, 128);
                            asm volatile(
                                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                                ::"r"(tmem_base + (uint32_t)(g * ACC_COLS + k * N)), "l"(da), "l"(db), "r"(idesc), "r"(0u), "r"(0u) : "memory");
                        }
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&mma_done[g])) : "memory");
                        done[g]++; left--; progress = true;
                    }
                }
                if (progress) t_idle = gtime_ns();
                else if (gtime_ns() - t_idle > kWaitBudgetNs) { *abort_flag = 1; break; }
            }
        }
    } else {
        // ---------------- workers: group g, thread rt = weight row rt of the unit = TMEM lane rt
        const int g = warp >> 2, wq = warp & 3, rt = tid - g * TC_ROWS;
        pdl_wait_prior();             // activations come from the previous kernel; the loader's weight tiles do not
        // activations of the CTA's K range: int8 into the canonical layout (tokens >= M are zero), scales next to them;
        // the loads of a round are all requested before the first store, one trip to L2 per round
        {
            const int items = nblk * N;
            for (int base = 0; base < items; base += 4 * TC_WORKERS) {
                int4 xa[4], xc[4]; unsigned short xdv[4];
                #pragma unroll
                for (int r = 0; r < 4; r++) {
                    const int i = base + r * TC_WORKERS + tid, bl = i / N, n = i % N;
                    xa[r] = make_int4(0, 0, 0, 0); xc[r] = xa[r]; xdv[r] = 0;
                    if (i < items && n < p.M) {
                        const int4* xp = reinterpret_cast<const int4*>(p.xq + ((size_t)n * p.nb + b0 + bl) * 32);
                        xa[r] = __ldcg(xp); xc[r] = __ldcg(xp + 1);
                        xdv[r] = __ldcg(reinterpret_cast<const unsigned short*>(p.xd) + (size_t)n * p.nb + b0 + bl);
                    }
                }
                #pragma unroll
                for (int r = 0; r < 4; r++) {
                    const int i = base + r * TC_WORKERS + tid, bl = i / N, n = i % N;
                    if (i < items) {
                        uint8_t* dst = b_s + (size_t)bl * (N * 32) + (n >> 3) * 128 + (n & 7) * 16;
                        *reinterpret_cast<int4*>(dst) = xa[r];
                        *reinterpret_cast<int4*>(dst + N * 16) = xc[r];
                        xs_s[i] = XScale{(double)__half2float(__ushort_as_half(xdv[r])), 8 * sum_x_block(xa[r], xc[r]), 0};
                    }
                }
            }
            workers_sync<TC_WORKERS>();
        }
        int it = 0;
        bool ok = true;
        for (int j = g; j < my_units && ok; j += TC_GROUPS) {
            const long long u = blockIdx.x + (long long)j * gridDim.x;
            const int sg = (int)(u / p.ks);
            double acc[N];
            #pragma unroll
            for (int n = 0; n < N; n++) acc[n] = 0.0;
            for (int t = t0; t < t1 && ok; t++, it++) {
                const int s = g * TC_RING + it % TC_RING;
                if (*abort_flag || !mbar_wait_bounded(&raw_full[s], (it / TC_RING) & 1)) { ok = false; break; }
                // unpack; the group's operand buffer is free: the MMAs of its previous tile were waited for by that tile's drain
                const uint8_t* rtile = raw + s * RAW_STAGE + wq * TB;
                uint8_t* dst0 = a_s + g * A_BUF + (rt >> 3) * 128 + (rt & 7) * 16;
                #pragma unroll
                for (int k = 0; k < KB; k++) {
                    const uint4 w = *reinterpret_cast<const uint4*>(rtile + (k * 32 + lane) * 16);
                    const unsigned Mk = 0x0F0F0F0Fu;
                    uint8_t* dst = dst0 + k * A_BLOCK;
                    *reinterpret_cast<uint4*>(dst) = make_uint4(w.x & Mk, w.y & Mk, w.z & Mk, w.w & Mk);
                    *reinterpret_cast<uint4*>(dst + 2048) = make_uint4((w.x >> 4) & Mk, (w.y >> 4) & Mk, (w.z >> 4) & Mk, (w.w >> 4) & Mk);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy writes -> visible to the tensor core's reads
                mbar_arrive(&a_full[g]);
                if (!mbar_wait_bounded(&mma_done[g], it & 1)) { ok = false; break; }
                tc_fence_after();
                // drain: four blocks' sums are requested together, then scaled
                const uint8_t* sc = rtile + KB * 512 + lane * (KB * 2);          // this row's KB fp16 scales
                const int ti = t - t0;
                constexpr int KG = KB < 4 ? KB : 4;
                #pragma unroll
                for (int k0 = 0; k0 < KB; k0 += KG) {
                    int isum[KG][N];
                    #pragma unroll
                    for (int k = 0; k < KG; k++)
                        tmem_ld_row<N>(tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(g * ACC_COLS + (k0 + k) * N), isum[k]);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    #pragma unroll
                    for (int k = 0; k < KG; k++) {
                        const double dwd = (double)__half2float(*reinterpret_cast<const __half*>(sc + (k0 + k) * 2));
                        const XScale* xs = xs_s + (ti * KB + k0 + k) * N;
                        #pragma unroll
                        for (int n = 0; n < N; n++) {
                            const XScale s2 = xs[n];
                            acc[n] = __fma_rn(__dmul_rn(dwd, s2.dx), int_to_double_exact(isum[k][n] - s2.s8), acc[n]);
                        }
                    }
                }
                tc_fence_before();
                mbar_arrive(&raw_empty[s]);                   // the ring slot may be overwritten (nibbles unpacked, scales used)
            }
            if (!ok) break;
            // results of the unit: rows sg*128 + rt, tokens 0..M-1
            const int row = sg * 128 + rt;
            if (p.ks == 1) {
                if (row < p.rows)
                    for (int n = 0; n < p.M; n++) p.y[(size_t)n * p.rows + row] = __double2float_rn(acc[n]) + (p.bias ? p.bias[row] : 0.f);
            } else {
                double* part = p.part + ((size_t)sg * p.ks + sp) * N * 128;
                #pragma unroll
                for (int n = 0; n < N; n++) __stcg(part + n * 128 + rt, acc[n]);
                __threadfence();
                group_sync(g);
                if (rt == 0) s_prev[g] = atomicAdd(p.counters + sg, 1u);
                group_sync(g);
                if (s_prev[g] == (unsigned)p.ks - 1) {              // last split in: fold all of them in split order
                    __threadfence();
                    // one split per round, all tokens' partial sums of that split requested together: a round is one trip
                    // to the L2.  (Token by token, each split's load waited for the one before it: ks * M dependent
                    // trips, 15 us of a 16-token pass over a matrix whose bytes take 0.3 us.)  The order of the additions of
                    // a token's sum is the split order either way.
                    const double* p0 = p.part + (size_t)sg * p.ks * N * 128 + rt;
                    double sum[N];
                    #pragma unroll
                    for (int n = 0; n < N; n++) sum[n] = 0.0;
                    for (int q = 0; q < p.ks; q++) {
                        double v[N];
                        #pragma unroll
                        for (int n = 0; n < N; n++) v[n] = n < p.M ? __ldcg(p0 + ((size_t)q * N + n) * 128) : 0.0;
                        #pragma unroll
                        for (int n = 0; n < N; n++) sum[n] = __dadd_rn(sum[n], v[n]);
                    }
                    if (row < p.rows) {
                        const float bv = p.bias ? p.bias[row] : 0.f;
                        #pragma unroll
                        for (int n = 0; n < N; n++)
                            if (n < p.M) p.y[(size_t)n * p.rows + row] = __double2float_rn(sum[n]) + bv;
                    }
                    if (rt == 0) p.counters[sg] = 0;
                }
                group_sync(g);                                // s_prev[g] is rewritten by the group's next unit
            }
        }
        if (!ok) *abort_flag = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0) atomicMax(p.err, MI_ERR_TIMEOUT);
        if (warp == TC_WORKERS / 32 + 1 && lane < TC_GROUPS)   // copies in flight target this CTA: let them land
            for (int j = max(0, loads_issued - TC_RING); j < loads_issued; j++)
                (void)mbar_wait_bounded(&raw_full[lane * TC_RING + j % TC_RING], (j / TC_RING) & 1);
        __syncthreads();
    }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
}

template <int KB, int N>
static int launch_gemm(mi_ctx* ctx, const mi_weight* w, GemmParams p) {
    constexpr int TB = KB * kTileRowBytes;
    constexpr int MAXT = tc_max_tiles(N), TC_GROUPS = tc_groups(N);
    const size_t smem = (size_t)TC_GROUPS * TC_RING * 4 * TB + (size_t)TC_GROUPS * KB * 128 * 32 + (size_t)MAXT * KB * N * 32 +
                        (size_t)MAXT * KB * N * sizeof(XScale) + (2 * TC_GROUPS * TC_RING + 2 * TC_GROUPS) * 8 + 16;
    if (smem > (size_t)ctx->smem_optin) return set_error(ctx, MI_ERR_UNSUPPORTED, "gemm: %zu bytes of shared memory needed", smem);
    auto kern = gemm_q4_q8_tc_kernel<KB, N>;
    MI_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int sgroups = (w->groups + 3) / 4;
    int ks = (w->nt + MAXT - 1) / MAXT;                                      // a CTA stages at most MAXT K-tiles of activations
    while (ks < w->nt && (long long)sgroups * ks < ctx->sm_count) ks++;      // and every SM should get a unit
    p.ks = ks;
    if (ks > 1) {
        int st = ensure_scratch(ctx, (size_t)sgroups * ks * N * 128, (size_t)sgroups);
        if (st != MI_OK) return st;
        p.part = ctx->part; p.counters = ctx->counters;
    }
    // one CTA per SM walks its units; the grid is a multiple of the K-split so that all units of a CTA share a K range
    long long ctas = (long long)sgroups * ks;
    if (ctas > ctx->sm_count) ctas = (long long)(ctx->sm_count / ks) * ks;
    if (ctas < ks) return set_error(ctx, MI_ERR_UNSUPPORTED, "gemm: K-split %d exceeds the SM count", ks);
    MI_CUDA(ctx, launch_k(ctx->pdl, kern, dim3((unsigned)ctas), dim3(tc_threads(N)), smem, ctx->stream, p));
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
