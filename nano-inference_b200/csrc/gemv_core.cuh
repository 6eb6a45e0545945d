// q4_0 x q8_0 GEMV core for sm_100a, shared by the standalone GEMV kernel and the
// fused decode-step kernels.
//
// Work decomposition.  A "unit" is (matrix c, 32-row group g, K-split sp): the
// tiles [sp*nt/ks, (sp+1)*nt/ks) of group g.  Units are dealt round-robin to
// the warps of a persistent grid.  Each warp owns a private ring of S tile
// slots in shared memory; lane 0 keeps the ring full with plain single-CTA
// cp.async.bulk copies (one contiguous tile per copy, completion counted on a
// per-slot mbarrier), running ahead across unit boundaries because the whole
// tile sequence of a warp is known up front.  All 32 lanes then read the tile
// from shared memory, lane = row: one conflict-free 16-byte read per block for
// the nibbles, broadcast reads for the int8 activations.  No cross-lane
// reduction is needed; K-splits meet in global scratch and the last split to
// arrive adds them in split order, so the result does not depend on timing.
// Sums are carried in double (see blk_acc): the fp32 result does not depend on
// the split either.
//
// HBM traffic per weight byte is exactly one read; the tile stream is the only
// traffic that scales with the matrix.
#pragma once
#include "mi_internal.cuh"

namespace mi {

struct GemvShape {
    const uint8_t* base;      // tiled weights of matrix 0
    long long mat_stride;     // bytes between matrices of the stack
    int n_mats, groups, nt, ks, nb;
    int rows;                 // valid rows per matrix (the last group may be padded)
};

struct GemvScratch {
    double* part;             // [n_mats*groups][ks][32] partial sums (ks > 1 only)
    unsigned* counters;       // [n_mats*groups] arrivals, zero between launches
};

// Shared-memory carve-up of a GEMV CTA.
template <int KB, int NW, int S>
struct GemvSmem {
    static constexpr int TB = tile_bytes(KB);
    static constexpr int ring_bytes = NW * S * TB;
    static constexpr int bar_bytes = ((NW * S * 8) + 15) / 16 * 16;
    __host__ __device__ static constexpr size_t bytes(int nb) { return (size_t)ring_bytes + bar_bytes + (size_t)nb * 32 + (size_t)nb * 8; }
    __device__ static uint8_t* ring(uint8_t* s) { return s; }
    __device__ static uint64_t* bars(uint8_t* s) { return reinterpret_cast<uint64_t*>(s + ring_bytes); }
    __device__ static int8_t* xq(uint8_t* s) { return reinterpret_cast<int8_t*>(s + ring_bytes + bar_bytes); }
    __device__ static float2* xs(uint8_t* s, int nb) { return reinterpret_cast<float2*>(s + ring_bytes + bar_bytes + (size_t)nb * 32); }
};

// Position of a warp in its own tile sequence.
struct TileCursor {
    long long u;          // current unit (>= n_units: exhausted)
    int t, t1;            // next tile and end tile within the unit's group
    int c, g, sp;         // matrix, group, split of the unit
    const uint8_t* gbase; // first tile of (c, g)
};

template <int KB>
__device__ __forceinline__ void cursor_set(TileCursor& cu, long long u, long long n_units, const GemvShape& sh) {
    cu.u = u;
    if (u >= n_units) return;
    cu.sp = (int)(u % sh.ks);
    const long long gg = u / sh.ks;
    cu.g = (int)(gg % sh.groups);
    cu.c = (int)(gg / sh.groups);
    cu.t = (int)((long long)cu.sp * sh.nt / sh.ks);
    cu.t1 = (int)((long long)(cu.sp + 1) * sh.nt / sh.ks);
    cu.gbase = sh.base + (size_t)cu.c * sh.mat_stride + (size_t)cu.g * sh.nt * tile_bytes(KB);
}

// The fp16 scales of one tile row (KB of them) as floats.
template <int KB>
__device__ __forceinline__ void load_tile_scales(const uint8_t* tile, int lane, float (&dw)[KB]) {
    const uint8_t* sp = tile + KB * 512 + lane * (KB * 2);
    if constexpr (KB == 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(sp);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
        #pragma unroll
        for (int i = 0; i < 4; i++) { const float2 f = __half22float2(h[i]); dw[2 * i] = f.x; dw[2 * i + 1] = f.y; }
    } else if constexpr (KB == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(sp);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
        #pragma unroll
        for (int i = 0; i < 2; i++) { const float2 f = __half22float2(h[i]); dw[2 * i] = f.x; dw[2 * i + 1] = f.y; }
    } else if constexpr (KB == 2) {
        const __half2 h = *reinterpret_cast<const __half2*>(sp);
        const float2 f = __half22float2(h); dw[0] = f.x; dw[1] = f.y;
    } else {
        dw[0] = __half2float(*reinterpret_cast<const __half*>(sp));
    }
}

// One tile's contribution to the lane's row.  xq_s / xs_s are the staged
// activations of the whole input vector; b0 is the tile's first block.
// DUMP writes the exact integer block values to isum_row[b] instead of relying
// on the float result.
template <int KB, bool DUMP>
__device__ __forceinline__ double tile_dot_row(const uint8_t* tile, int lane, int b0, const int8_t* xq_s,
                                               const float2* xs_s, double acc, int32_t* isum_row) {
    float dw[KB];
    load_tile_scales<KB>(tile, lane, dw);
    const uint4* wq = reinterpret_cast<const uint4*>(tile) + lane;
    #pragma unroll                                      // (four at a time instead of all KB: 6 % slower in the decode kernel)
    for (int k = 0; k < KB; k++) {
        const uint4 w = wq[k * 32];
        const int4 xa = *reinterpret_cast<const int4*>(xq_s + (b0 + k) * 32);
        const int4 xc = *reinterpret_cast<const int4*>(xq_s + (b0 + k) * 32 + 16);
        const float2 s = xs_s[b0 + k];                       // {dx, float(8*sum x)}
        const int isum = dot_q4_block(w, xa, xc);
        if constexpr (DUMP) { if (isum_row) isum_row[b0 + k] = isum - __float2int_rn(s.y); }
        acc = blk_acc(acc, dw[k], s.x, isum, s.y);
    }
    return acc;
}

// Stage a q8_0 activation vector already in global memory: int8 values, and per
// block {fp32 of the fp16 scale, float(8 * sum of the block's int8 values)}.
__device__ __forceinline__ void stage_x_q8(const int8_t* xq, const __half* xd, int nb, int8_t* xq_s, float2* xs_s,
                                           int tid, int nthreads) {
    const int4* src = reinterpret_cast<const int4*>(xq);
    int4* dst = reinterpret_cast<int4*>(xq_s);
    for (int i = tid; i < nb * 2; i += nthreads) dst[i] = src[i];
    for (int b = tid; b < nb; b += nthreads) {
        const int4 xa = src[2 * b], xc = src[2 * b + 1];
        xs_s[b] = make_float2(__half2float(xd[b]), __int2float_rn(8 * sum_x_block(xa, xc)));
    }
}

// The streaming GEMV loop of one warp.  Before calling: barriers initialised
// (gemv_init_barriers), weights prefetch started (gemv_prefetch) and the
// activations staged in shared memory behind a __syncthreads().
//   epi(c, g, lane, value) is called by all 32 lanes once per (matrix, group)
//   with the complete sum of row g*32+lane, rounded to fp32 once.
// Returns false if a bounded wait gave up.
template <int KB, int NW, int S>
struct GemvWarp {
    using SM = GemvSmem<KB, NW, S>;
    static constexpr int TB = SM::TB;
    uint8_t* ring;       // this warp's S slots
    uint64_t* bars;      // this warp's S barriers
    TileCursor pc, cc;   // producer / consumer positions
    int issued, consumed;
    long long n_units;
    int stride;          // total warps in the grid
    uint64_t policy;     // L2 evict-first: a weight byte is read once

    __device__ __forceinline__ void init(uint8_t* smem, const GemvShape& sh, int warp, int lane) {
        ring = SM::ring(smem) + (size_t)warp * S * TB;
        bars = SM::bars(smem) + warp * S;
        n_units = (long long)sh.n_mats * sh.groups * sh.ks;
        stride = gridDim.x * NW;
        issued = consumed = 0; policy = l2_policy_evict_first();
        if (lane == 0) {
            #pragma unroll
            for (int s = 0; s < S; s++) mbar_init(&bars[s], 1);
            mbar_fence_init();
        }
        __syncwarp();
        cursor_set<KB>(pc, (long long)blockIdx.x * NW + warp, n_units, sh);
        cc = pc;
    }
    // lane 0 only: issue the next tile of this warp's sequence, if any
    __device__ __forceinline__ void issue_one(const GemvShape& sh) {
        if (pc.u >= n_units) return;
        const int slot = issued % S;
        mbar_expect_tx(&bars[slot], TB);
        bulk_g2s_hint(ring + (size_t)slot * TB, pc.gbase + (size_t)pc.t * TB, TB, &bars[slot], policy);
        issued++;
        if (++pc.t == pc.t1) cursor_set<KB>(pc, pc.u + stride, n_units, sh);
    }
    __device__ __forceinline__ void prefetch(const GemvShape& sh, int lane) {
        if (lane == 0) {
            #pragma unroll
            for (int s = 0; s < S; s++) issue_one(sh);
        }
    }
    template <bool DUMP, class Epi>
    __device__ __forceinline__ bool run(const GemvShape& sh, const GemvScratch& sc, const int8_t* xq_s,
                                        const float2* xs_s, int lane, int32_t* isum_out, Epi epi) {
        bool ok = true;
        while (cc.u < n_units && ok) {
            double acc = 0.0;
            int32_t* isum_row = (DUMP && cc.g * 32 + lane < sh.rows) ? isum_out + ((size_t)cc.g * 32 + lane) * sh.nb : nullptr;
            for (int t = cc.t; t < cc.t1; t++) {
                const int slot = consumed % S;
                if (!mbar_wait_bounded(&bars[slot], (consumed / S) & 1)) { ok = false; break; }
                acc = tile_dot_row<KB, DUMP>(ring + (size_t)slot * TB, lane, t * KB, xq_s, xs_s, acc, isum_row);
                consumed++;
                __syncwarp();                       // every lane is done with the slot before it is refilled
                if (lane == 0) issue_one(sh);
            }
            if (!ok) break;
            const int cg = cc.c * sh.groups + cc.g;
            if (sh.ks == 1) {
                epi(cc.c, cc.g, lane, __double2float_rn(acc));
            } else {
                double* part = sc.part + ((size_t)cg * sh.ks) * 32;
                __stcg(part + cc.sp * 32 + lane, acc);
                __threadfence();
                __syncwarp();
                unsigned prev = 0;
                if (lane == 0) prev = atomicAdd(sc.counters + cg, 1u);
                prev = __shfl_sync(0xffffffffu, prev, 0);
                if (prev == (unsigned)sh.ks - 1) {          // last split to arrive folds all of them, in split order
                    __threadfence();
                    double sum = __ldcg(part + lane);
                    for (int s = 1; s < sh.ks; s++) sum = __dadd_rn(sum, __ldcg(part + s * 32 + lane));
                    if (lane == 0) sc.counters[cg] = 0;   // ready for the next launch
                    epi(cc.c, cc.g, lane, __double2float_rn(sum));
                }
            }
            cursor_set<KB>(cc, cc.u + stride, n_units, sh);
        }
        if (!ok) {
            // Copies already issued still target this CTA's shared memory: give each a bounded
            // chance to land before the CTA exits.
            for (int i = consumed; i < issued; i++) (void)mbar_wait_bounded(&bars[i % S], (i / S) & 1);
        }
        return ok;
    }
};

}  // namespace mi
