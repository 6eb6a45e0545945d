// The fused decode step for sm_100a: one persistent kernel that runs any range of
// the per-token phases
//     per layer:  QKV  (rmsnorm -> q8 -> GEMV -> +bias, RoPE, q / fp16 KV store)
//                 ATTN (split-KV attention over the fp16 cache, merge, -> q8)
//                 O    (GEMV -> residual add)
//                 GU   (rmsnorm -> q8 -> gate & up GEMV -> SwiGLU -> q8)
//                 DOWN (GEMV -> residual add)
//     finally:    LM   (rmsnorm -> q8 -> lm_head GEMV -> argmax)
// for any range of steps.  Launched with one phase per launch it is a plain
// kernel sequence; launched cooperatively over all phases and steps it is the
// persistent decode loop, phases separated by a bounded-wait grid barrier.
//
// Weight streaming.  Every GEMV phase is a "job": a tiled q4_0 matrix cut into
// units (row group, K-split) dealt to the grid's warps by a fixed rule.  The
// whole tile sequence of a warp - across phases, layers and steps - is therefore
// known up front, and lane 0 of every warp keeps a private shared-memory ring
// full with bulk copies that run ahead of the barriers: weights are immutable,
// so the HBM stream never has to wait for a phase boundary, only for ring space.
//
// Numerics follow the reference (paths relative to its root): quantizer
// src/cuda_infer.cu:80-89; block dot + rounded accumulate src/mega.cu:151-165;
// RMSNorm / RoPE / SwiGLU / argmax src/cpu_infer.cpp:40-61,147,153-154;
// split-KV merge src/cuda_infer.cu:650-702.  Every sum that feeds a stored tensor
// (GEMV rows, RMSNorm sum of squares, attention scores, softmax denominator and
// weighted values) is carried in double and rounded to fp32 once; exp, cos and sin
// come from the double math library.  A q8_0 quantizer is discontinuous, so this
// is what lets two engines (or two split / step / shard configurations of this
// one) agree bit for bit: the fp32 value of a double-carried sum does not depend
// on the order of its terms.  Each token is processed exactly as if it were alone.
#pragma once
#include "gemv_core.cuh"

namespace mi {

constexpr int DNW = 8;            // warps per CTA
constexpr int DNT = DNW * 32;
constexpr int DS = 3;             // ring slots per warp
constexpr int DSLOT = 4608;       // bytes per slot: the largest tile (8 blocks)
constexpr int kAttnChunk = 64;    // smallest KV range worth its own CTA

enum JobKind { JOB_QKV = 0, JOB_O = 1, JOB_GU = 2, JOB_DOWN = 3, JOB_LM = 4 };

struct Job {
    const uint8_t* base;   // tiled weights
    int groups;            // unit groups; one unit group = nacc consecutive 32-row groups
    int nt, ks, nb, kb, nacc, kind;
    int n_units;           // groups * ks
    int rot;               // warp slot that gets unit 0
    int part_off;          // offset (in doubles) of this job's split-K partials
    int cnt_off;           // offset of this job's arrival counters
    int layer;
};

struct LayerPtrs { const float* attn_norm; const float* ffn_norm; const float* bqkv; };

struct DecodeParams {
    int L, E, FF, NH, NKV, HD, KVD, V;
    float eps;
    const Job* jobs;                 // [4L+1] in phase order
    const LayerPtrs* layers;         // [L]
    const float* out_norm;
    const float* rope_freq;          // [HD/2]: base^(-2i/HD), computed on the host with powf
    const uint8_t* emb_base;         // tiled token embedding (may alias the lm_head)
    int emb_nt, emb_kb;
    // state (global, written and read across CTAs: always accessed through L2)
    float* h; float* q; float* att;
    int8_t* att_q; __half* att_d;    // q8_0 of the merged attention output
    int8_t* act_q; __half* act_d;    // q8_0 of SwiGLU(gate, up)
    __half* kc; __half* vc; int max_seq;       // [L][max_seq][KVD]
    double* attn_part; unsigned* attn_cnt; int max_chunks;  // [NH][max_chunks][HD+2], [NKV]
    double* part; unsigned* counters;          // split-K scratch
    float* cand_val; int* cand_idx; unsigned* cand_cnt;     // per-CTA argmax candidates
    const int* in_tokens; int n_forced; int* out_tokens; int* cur_token;
    float* logits; long long logits_stride;    // optional [n_steps][stride]
    int pos0;
    unsigned* bar; int* err;
};

// number of KV chunks for a causal range of Lp positions (host and device agree)
__host__ __device__ inline int attn_chunks(int Lp, int max_chunks) {
    int n = (Lp + kAttnChunk - 1) / kAttnChunk;
    return n < 1 ? 1 : (n > max_chunks ? max_chunks : n);
}

#ifdef __CUDACC__

struct DecodeSmem {
    uint8_t* ring; uint64_t* bars; Job* jobs; float* cs; double* red; uint8_t* stage;
};

__host__ __device__ inline size_t decode_stage_bytes(int E, int FF, int HD, int G) {
    const int maxin = E > FF ? E : FF;
    size_t a = (size_t)E * 4 + maxin + (size_t)(maxin / 32) * 8;
    size_t b = (size_t)DNW * G * (HD + 2) * 8 + (size_t)DNW * 32 * G * 8 + (size_t)G * HD * 4;   // attention: states, weights, q
    return ((a > b ? a : b) + 127) / 128 * 128;
}
__host__ __device__ inline size_t decode_smem_bytes(int njobs, int E, int FF, int HD, int G) {
    return (size_t)DNW * DS * DSLOT + 256 + ((size_t)njobs * sizeof(Job) + 127) / 128 * 128 + 1024 + 256 +
           decode_stage_bytes(E, FF, HD, G);
}

// ---- grid barrier: monotonic arrival counter, bounded wait -----------------------
__device__ __forceinline__ bool grid_barrier(unsigned* bar, unsigned& target, int* ok_s) {
    __syncthreads();
    if (threadIdx.x == 0) {
        target += gridDim.x;
        __threadfence();
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar) : "memory");
        bool ok = true;
        unsigned v;
        unsigned long long t0 = 0;
        for (unsigned it = 0;; it++) {
            asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
            if ((int)(v - target) >= 0) break;
            if ((it & 1023u) == 1023u) {
                const unsigned long long now = gtime_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > kWaitBudgetNs) { ok = false; break; }
            }
        }
        *ok_s = ok ? 1 : 0;
    }
    __syncthreads();
    return *ok_s != 0;
}

// ---- the per-warp weight stream -----------------------------------------------
struct StreamCursor { int step, j, u, a, t, t0, t1; };

struct WarpStream {
    uint8_t* ring; uint64_t* bars; const Job* jobs;
    StreamCursor pc;
    int issued, consumed;
    int step1, j0, j1;      // steps end; job range per step
    int W, sid;             // warp slots in the grid, this warp's slot

    __device__ __forceinline__ int first_unit(const Job& jb) const {
        const int r = jb.rot % W;
        return sid >= r ? sid - r : sid + W - r;
    }
    __device__ __forceinline__ void set_tiles(const Job& jb) {
        const int sp = pc.u % jb.ks;
        pc.t0 = (int)((long long)sp * jb.nt / jb.ks);
        pc.t1 = (int)((long long)(sp + 1) * jb.nt / jb.ks);
        pc.t = pc.t0; pc.a = 0;
    }
    // move the producer to the next (step, job) that has a unit for this warp
    __device__ __forceinline__ void seek() {
        while (pc.step < step1) {
            const Job& jb = jobs[pc.j];
            if (pc.u < jb.n_units) { set_tiles(jb); return; }
            if (++pc.j == j1) { pc.j = j0; pc.step++; }
            if (pc.step < step1) pc.u = first_unit(jobs[pc.j]);
        }
    }
    __device__ __forceinline__ void init(const DecodeSmem& sm, int warp, int lane, int step0, int step1_, int j0_, int j1_) {
        ring = sm.ring + (size_t)warp * DS * DSLOT; bars = sm.bars + warp * DS; jobs = sm.jobs;
        W = gridDim.x * DNW; sid = warp * gridDim.x + blockIdx.x;      // consecutive units land on different SMs
        step1 = step1_; j0 = j0_; j1 = j1_; issued = consumed = 0;
        pc.step = (j0 < j1) ? step0 : step1; pc.j = j0;
        if (pc.step < step1) { pc.u = first_unit(jobs[pc.j]); seek(); }
    }
    __device__ __forceinline__ void issue_one() {       // lane 0 only
        if (pc.step >= step1) return;
        const Job& jb = jobs[pc.j];
        const int g = pc.u / jb.ks, tb = jb.kb * kTileRowBytes, slot = issued % DS;
        const uint8_t* src = jb.base + ((size_t)(g * jb.nacc + pc.a) * jb.nt + pc.t) * tb;
        mbar_expect_tx(&bars[slot], tb);
        bulk_g2s(ring + (size_t)slot * DSLOT, src, tb, &bars[slot]);
        issued++;
        if (++pc.t == pc.t1) {
            if (++pc.a < jb.nacc) pc.t = pc.t0;
            else { pc.u += W; seek(); }
        }
    }
    __device__ __forceinline__ void drain() {
        for (int i = consumed; i < issued; i++) (void)mbar_wait_bounded(&bars[i % DS], (i / DS) & 1);
    }
};

template <int KB>
__device__ __forceinline__ double tiles_dot(WarpStream& ws, int lane, int t0, int t1, const int8_t* xq_s, const float2* xs_s, bool& ok) {
    double acc = 0.0;
    for (int t = t0; t < t1; t++) {
        const int slot = ws.consumed % DS;
        if (!mbar_wait_bounded(&ws.bars[slot], (ws.consumed / DS) & 1)) { ok = false; return acc; }
        acc = tile_dot_row<KB, false>(ws.ring + (size_t)slot * DSLOT, lane, t * KB, xq_s, xs_s, acc, nullptr);
        ws.consumed++;
        __syncwarp();
        if (lane == 0) ws.issue_one();
    }
    return acc;
}

// Consume this warp's units of job j.  epi(g, lane, v0, v1): complete sums (fp32 of the double sum) of rows
// (g*nacc + a)*32 + lane, a = 0 (v0) and 1 (v1, only when nacc == 2).
template <class Epi>
__device__ __forceinline__ bool run_job(WarpStream& ws, const DecodeParams& P, int j, int lane, const int8_t* xq_s,
                                        const float2* xs_s, Epi epi) {
    const Job& jb = ws.jobs[j];
    bool ok = true;
    for (int u = ws.first_unit(jb); u < jb.n_units && ok; u += ws.W) {
        const int g = u / jb.ks, sp = u % jb.ks;
        const int t0 = (int)((long long)sp * jb.nt / jb.ks), t1 = (int)((long long)(sp + 1) * jb.nt / jb.ks);
        double v0 = 0.0, v1 = 0.0;
        switch (jb.kb) {
            case 8: v0 = tiles_dot<8>(ws, lane, t0, t1, xq_s, xs_s, ok); if (jb.nacc == 2 && ok) v1 = tiles_dot<8>(ws, lane, t0, t1, xq_s, xs_s, ok); break;
            case 4: v0 = tiles_dot<4>(ws, lane, t0, t1, xq_s, xs_s, ok); if (jb.nacc == 2 && ok) v1 = tiles_dot<4>(ws, lane, t0, t1, xq_s, xs_s, ok); break;
            case 2: v0 = tiles_dot<2>(ws, lane, t0, t1, xq_s, xs_s, ok); if (jb.nacc == 2 && ok) v1 = tiles_dot<2>(ws, lane, t0, t1, xq_s, xs_s, ok); break;
            default: v0 = tiles_dot<1>(ws, lane, t0, t1, xq_s, xs_s, ok); if (jb.nacc == 2 && ok) v1 = tiles_dot<1>(ws, lane, t0, t1, xq_s, xs_s, ok); break;
        }
        if (!ok) break;
        if (jb.ks == 1) { epi(g, lane, __double2float_rn(v0), __double2float_rn(v1)); continue; }
        double* part = P.part + jb.part_off + (size_t)g * jb.ks * jb.nacc * 32;
        __stcg(part + (sp * jb.nacc) * 32 + lane, v0);
        if (jb.nacc == 2) __stcg(part + (sp * 2 + 1) * 32 + lane, v1);
        __threadfence();
        __syncwarp();
        unsigned prev = 0;
        if (lane == 0) prev = atomicAdd(P.counters + jb.cnt_off + g, 1u);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev == (unsigned)jb.ks - 1) {              // last split in: fold all of them in split order
            __threadfence();
            double s0 = __ldcg(part + lane), s1 = jb.nacc == 2 ? __ldcg(part + 32 + lane) : 0.0;
            for (int s = 1; s < jb.ks; s++) {
                s0 = __dadd_rn(s0, __ldcg(part + (s * jb.nacc) * 32 + lane));
                if (jb.nacc == 2) s1 = __dadd_rn(s1, __ldcg(part + (s * 2 + 1) * 32 + lane));
            }
            if (lane == 0) P.counters[jb.cnt_off + g] = 0;
            epi(g, lane, __double2float_rn(s0), __double2float_rn(s1));
        }
    }
    return ok;
}

// ---- activation staging (whole CTA; ends with __syncthreads) -----------------------

// q8_0 of one 32-element block held one element per lane; returns the int8 value,
// writes {fp32 of fp16(a/127), float(8*sum q)} through lane 0.
__device__ __forceinline__ int quant_block_warp(float v, int lane, float2* xs_out, __half* xd_out) {
    float a = fabsf(v);
    #pragma unroll
    for (int o = 16; o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    const float inv = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
    const int q = __float2int_rn(__fmul_rn(v, inv));
    int s = q;
    #pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
        const __half d = __float2half_rn(__fdiv_rn(a, 127.f));
        if (xs_out) *xs_out = make_float2(__half2float(d), __int2float_rn(8 * s));
        if (xd_out) *xd_out = d;
    }
    return q;
}

// hs[0..E) (shared, fp32) -> rmsnorm * w -> q8_0 in xq_s / xs_s.  Sum of squares in
// double (every x*x is exact there), then the reference's fp32 expression
// x * (1/sqrt(float(ss/n) + eps)) * w (src/cpu_infer.cpp:40-46).
__device__ __forceinline__ void stage_norm_q8(const float* hs, const float* __restrict__ w, int E, float eps, double* red,
                                              int8_t* xq_s, float2* xs_s) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    double ss = 0.0;
    for (int i = tid; i < E; i += DNT) { const double x = hs[i]; ss = __fma_rn(x, x, ss); }
    #pragma unroll
    for (int o = 16; o; o >>= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    double tot = 0.0;
    #pragma unroll
    for (int v = 0; v < DNW; v++) tot = __dadd_rn(tot, red[v]);
    const float mean = __double2float_rn(__ddiv_rn(tot, (double)E));
    const float scale = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(mean, eps)));
    for (int b = warp; b < E / 32; b += DNW) {
        const int e = b * 32 + lane;
        const float v = __fmul_rn(__fmul_rn(hs[e], scale), __ldg(w + e));
        xq_s[e] = (int8_t)quant_block_warp(v, lane, xs_s + b, nullptr);
    }
    __syncthreads();
}

// q8_0 vector already in global memory (written by another CTA): copy through L2.
__device__ __forceinline__ void stage_copy_q8(const int8_t* xq, const __half* xd, int nb, int8_t* xq_s, float2* xs_s) {
    const int tid = threadIdx.x;
    const int4* src = reinterpret_cast<const int4*>(xq);
    int4* dst = reinterpret_cast<int4*>(xq_s);
    for (int b = tid; b < nb; b += DNT) {
        const int4 xa = __ldcg(src + 2 * b), xc = __ldcg(src + 2 * b + 1);
        dst[2 * b] = xa; dst[2 * b + 1] = xc;
        const __half d = __ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(xd) + b));
        xs_s[b] = make_float2(__half2float(d), __int2float_rn(8 * sum_x_block(xa, xc)));
    }
    __syncthreads();
}

// row `token` of the tiled embedding matrix -> hs (fp32), value (nibble - 8) * d
// (reference src/gguf.h:94-102).
__device__ __forceinline__ void embed_row(const DecodeParams& P, int token, float* hs) {
    const int g = token >> 5, r = token & 31, kb = P.emb_kb, tb = kb * kTileRowBytes;
    for (int e = threadIdx.x; e < P.E; e += DNT) {
        const int b = e >> 5, el = e & 31, t = b / kb, k = b % kb;
        const uint8_t* tile = P.emb_base + ((size_t)g * P.emb_nt + t) * tb;
        const uint8_t byte = __ldg(tile + ((size_t)k * 32 + r) * 16 + (el & 15));
        const float d = __half2float(__ldg(reinterpret_cast<const __half*>(tile + (size_t)kb * 512 + ((size_t)r * kb + k) * 2)));
        const int n = el < 16 ? (byte & 0x0F) : (byte >> 4);
        hs[e] = __fmul_rn(__int2float_rn(n - 8), d);
    }
}

// ---- attention --------------------------------------------------------------------
// CTA = (kv head, chunk of the causal range); its warps split the chunk.  A warp
// walks its positions 32 at a time in two passes.  Pass 1, lane = position: the
// full q.k dot of the lane's K row against all G query heads of the kv head (q
// comes from shared memory as broadcast reads, so there is no cross-lane
// reduction and one K read serves the whole GQA group).  Pass 2, lane = dims
// {lane + 32 i}: the 32 positions' softmax weights (parked in shared memory) times
// their V rows.  Running state per head: max m (an fp32 score), denominator l and
// output o[] in double.  States fold warps -> chunk (shared memory, warp order) ->
// head (global scratch, chunk order, by the last CTA of the kv head to arrive);
// then o/l is rounded to fp32, stored, and quantized to q8_0 for the O projection.
__device__ __forceinline__ void softmax_merge(float& m, double& l, float ma, double la, float mb, double lb, double& fa, double& fb) {
    m = fmaxf(ma, mb);
    fa = ma == -INFINITY ? 0.0 : exp((double)ma - (double)m);
    fb = mb == -INFINITY ? 0.0 : exp((double)mb - (double)m);
    l = __fma_rn(la, fa, __dmul_rn(lb, fb));
}

template <int HD, int G>
__device__ __forceinline__ void attention_phase(const DecodeParams& P, int l, int pos, uint8_t* stage) {
    constexpr int DPW = HD / 32;           // dims per lane in pass 2 and while folding (dim = lane + 32*i)
    constexpr int SW = HD + 2;             // doubles per (head) state: o[HD], m, l
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int Lp = pos + 1, nch = attn_chunks(Lp, P.max_chunks);
    if ((int)blockIdx.x >= P.NKV * nch) return;
    const int kvh = blockIdx.x / nch, ch = blockIdx.x % nch;
    const int p0 = (int)((long long)ch * Lp / nch), p1 = (int)((long long)(ch + 1) * Lp / nch);
    double* scr = reinterpret_cast<double*>(stage);                        // [warp][G][SW]
    double* wts = scr + DNW * G * SW;                                       // [warp][32][G]
    float* qs = reinterpret_cast<float*>(wts + DNW * 32 * G);               // [G][HD]
    for (int i = tid; i < G * HD; i += DNT) qs[i] = __ldcg(P.q + (size_t)kvh * G * HD + i);
    __syncthreads();
    const float inv = __fdiv_rn(1.f, __fsqrt_rn((float)HD));
    const int n = p1 - p0, a0 = p0 + (int)((long long)n * warp / DNW), a1 = p0 + (int)((long long)n * (warp + 1) / DNW);
    const __half* kbase = P.kc + ((size_t)l * P.max_seq) * P.KVD + (size_t)kvh * HD;
    const __half* vbase = P.vc + ((size_t)l * P.max_seq) * P.KVD + (size_t)kvh * HD;
    double* wl = wts + (size_t)warp * 32 * G;
    float m[G]; double ls[G], o[G][DPW];
    #pragma unroll
    for (int j = 0; j < G; j++) {
        m[j] = -INFINITY; ls[j] = 0.0;
        #pragma unroll
        for (int i = 0; i < DPW; i++) o[j][i] = 0.0;
    }
    for (int b0 = a0; b0 < a1; b0 += 32) {                                  // warp-uniform trip count
        const int p = b0 + lane;
        const bool valid = p < a1;
        // pass 1: scores of position p for the G heads
        float sc[G];
        {
            double d[G];
            #pragma unroll
            for (int j = 0; j < G; j++) d[j] = 0.0;
            const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)(valid ? p : a1 - 1) * P.KVD);
            #pragma unroll 2
            for (int c = 0; c < HD / 8; c++) {
                const uint4 ku = __ldcg(kp + c);
                const __half2* kh = reinterpret_cast<const __half2*>(&ku);
                float kf[8];
                #pragma unroll
                for (int e = 0; e < 4; e++) { const float2 f = __half22float2(kh[e]); kf[2 * e] = f.x; kf[2 * e + 1] = f.y; }
                #pragma unroll
                for (int j = 0; j < G; j++) {
                    const float4 qa = *reinterpret_cast<const float4*>(qs + j * HD + c * 8);
                    const float4 qb = *reinterpret_cast<const float4*>(qs + j * HD + c * 8 + 4);
                    d[j] = __fma_rn((double)qa.x, (double)kf[0], d[j]); d[j] = __fma_rn((double)qa.y, (double)kf[1], d[j]);
                    d[j] = __fma_rn((double)qa.z, (double)kf[2], d[j]); d[j] = __fma_rn((double)qa.w, (double)kf[3], d[j]);
                    d[j] = __fma_rn((double)qb.x, (double)kf[4], d[j]); d[j] = __fma_rn((double)qb.y, (double)kf[5], d[j]);
                    d[j] = __fma_rn((double)qb.z, (double)kf[6], d[j]); d[j] = __fma_rn((double)qb.w, (double)kf[7], d[j]);
                }
            }
            #pragma unroll
            for (int j = 0; j < G; j++) sc[j] = valid ? __fmul_rn(__double2float_rn(d[j]), inv) : -INFINITY;
        }
        // new running max, rescale, this batch's weights
        #pragma unroll
        for (int j = 0; j < G; j++) {
            float bm = sc[j];
            #pragma unroll
            for (int sft = 16; sft; sft >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, sft));
            const float mn = fmaxf(m[j], bm);                                // finite: the batch holds a valid position
            const double cr = m[j] == -INFINITY ? 0.0 : exp((double)m[j] - (double)mn);
            const double w = valid ? exp((double)sc[j] - (double)mn) : 0.0;
            wl[lane * G + j] = w;
            double wsum = w;
            #pragma unroll
            for (int sft = 16; sft; sft >>= 1) wsum = __dadd_rn(wsum, __shfl_xor_sync(0xffffffffu, wsum, sft));
            ls[j] = __fma_rn(ls[j], cr, wsum);
            #pragma unroll
            for (int i = 0; i < DPW; i++) o[j][i] = __dmul_rn(o[j][i], cr);
            m[j] = mn;
        }
        __syncwarp();
        // pass 2: o += w[p] * V[p]
        const int np = min(32, a1 - b0);
        for (int pp = 0; pp < np; pp++) {
            const __half* vp = vbase + (size_t)(b0 + pp) * P.KVD;
            double vv[DPW];
            #pragma unroll
            for (int i = 0; i < DPW; i++) vv[i] = (double)__half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(vp) + lane + 32 * i)));
            #pragma unroll
            for (int j = 0; j < G; j++) {
                const double w = wl[pp * G + j];
                #pragma unroll
                for (int i = 0; i < DPW; i++) o[j][i] = __fma_rn(w, vv[i], o[j][i]);
            }
        }
        __syncwarp();
    }
    #pragma unroll
    for (int j = 0; j < G; j++) {
        double* sw = scr + (size_t)(warp * G + j) * SW;
        #pragma unroll
        for (int i = 0; i < DPW; i++) sw[lane + 32 * i] = o[j][i];
        if (lane == 0) { sw[HD] = (double)m[j]; sw[HD + 1] = ls[j]; }
    }
    __syncthreads();
    // warp j folds head j's DNW warp states in warp order and publishes the chunk partial
    if (warp < G) {
        const int j = warp, head = kvh * G + j;
        double ob[DPW], ll; float mm;
        {
            const double* s0 = scr + (size_t)j * SW;
            #pragma unroll
            for (int i = 0; i < DPW; i++) ob[i] = s0[lane + 32 * i];
            mm = (float)s0[HD]; ll = s0[HD + 1];
        }
        for (int w = 1; w < DNW; w++) {
            const double* s2 = scr + (size_t)(w * G + j) * SW;
            float mn; double ln, fa, fb;
            softmax_merge(mn, ln, mm, ll, (float)s2[HD], s2[HD + 1], fa, fb);
            #pragma unroll
            for (int i = 0; i < DPW; i++) ob[i] = __fma_rn(ob[i], fa, __dmul_rn(s2[lane + 32 * i], fb));
            mm = mn; ll = ln;
        }
        double* gp = P.attn_part + ((size_t)head * P.max_chunks + ch) * SW;
        #pragma unroll
        for (int i = 0; i < DPW; i++) __stcg(gp + lane + 32 * i, ob[i]);
        if (lane == 0) { __stcg(gp + HD, (double)mm); __stcg(gp + HD + 1, ll); }
    }
    __threadfence();
    __syncthreads();
    __shared__ unsigned s_prev;
    if (tid == 0) s_prev = atomicAdd(P.attn_cnt + kvh, 1u);
    __syncthreads();
    if (s_prev != (unsigned)nch - 1) return;
    // last chunk of this kv head: fold the chunk partials in chunk order, normalise, emit fp32 + q8_0
    __threadfence();
    if (tid == 0) P.attn_cnt[kvh] = 0;
    if (warp < G) {
        const int j = warp, head = kvh * G + j;
        const double* gp = P.attn_part + (size_t)head * P.max_chunks * SW;
        double ob[DPW], ll = __ldcg(gp + HD + 1); float mm = (float)__ldcg(gp + HD);
        #pragma unroll
        for (int i = 0; i < DPW; i++) ob[i] = __ldcg(gp + lane + 32 * i);
        for (int c = 1; c < nch; c++) {
            const double* g2 = gp + (size_t)c * SW;
            float mn; double ln, fa, fb;
            softmax_merge(mn, ln, mm, ll, (float)__ldcg(g2 + HD), __ldcg(g2 + HD + 1), fa, fb);
            #pragma unroll
            for (int i = 0; i < DPW; i++) ob[i] = __fma_rn(ob[i], fa, __dmul_rn(__ldcg(g2 + lane + 32 * i), fb));
            mm = mn; ll = ln;
        }
        #pragma unroll
        for (int i = 0; i < DPW; i++) {
            const float v = __double2float_rn(__ddiv_rn(ob[i], ll));
            const int e = head * HD + 32 * i + lane;
            __stcg(P.att + e, v);
            const int qv = quant_block_warp(v, lane, nullptr, P.att_d + (e >> 5));
            P.att_q[e] = (int8_t)qv;
        }
    }
}

// ---- the kernel ---------------------------------------------------------------------
template <int HD, int G>
__global__ void __launch_bounds__(DNT, 1)
decode_kernel(const __grid_constant__ DecodeParams P, int step0, int step1, int ph0, int ph1) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int njobs = 4 * P.L + 1, nph = 5 * P.L + 1;
    DecodeSmem sm;
    sm.ring = smem;
    sm.bars = reinterpret_cast<uint64_t*>(smem + (size_t)DNW * DS * DSLOT);
    sm.jobs = reinterpret_cast<Job*>(smem + (size_t)DNW * DS * DSLOT + 256);
    uint8_t* after_jobs = reinterpret_cast<uint8_t*>(sm.jobs) + ((size_t)njobs * sizeof(Job) + 127) / 128 * 128;
    sm.cs = reinterpret_cast<float*>(after_jobs);                 // [HD]: cos then sin
    sm.red = reinterpret_cast<double*>(after_jobs + 1024);         // 32 doubles
    sm.stage = after_jobs + 1024 + 256;
    __shared__ int s_ok;

    for (int i = tid; i < njobs * (int)(sizeof(Job) / 4); i += DNT)
        reinterpret_cast<int*>(sm.jobs)[i] = __ldg(reinterpret_cast<const int*>(P.jobs) + i);
    if (lane == 0) {
        #pragma unroll
        for (int s = 0; s < DS; s++) mbar_init(&sm.bars[warp * DS + s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    // jobs covered by the phase range of this launch
    auto job_of_phase = [&](int ph) -> int {          // first job at or after phase ph
        if (ph >= nph - 1) return ph >= nph ? njobs : njobs - 1;
        const int l = ph / 5, k = ph % 5;
        return 4 * l + (k == 0 ? 0 : k <= 2 ? 1 : k == 3 ? 2 : 3);
    };
    WarpStream ws;
    ws.init(sm, warp, lane, step0, step1, job_of_phase(ph0), job_of_phase(ph1));
    if (lane == 0) {
        #pragma unroll
        for (int s = 0; s < DS; s++) ws.issue_one();
    }
    pdl_launch_dependents();
    pdl_wait_prior();

    float* hs = reinterpret_cast<float*>(sm.stage);
    const int maxin = P.E > P.FF ? P.E : P.FF;
    int8_t* xq_s = reinterpret_cast<int8_t*>(sm.stage + (size_t)P.E * 4);
    float2* xs_s = reinterpret_cast<float2*>(sm.stage + (size_t)P.E * 4 + maxin);
    unsigned bar_target = 0;
    bool ok = true;
    const bool single = (step1 - step0 == 1) && (ph1 - ph0 == 1);

    for (int step = step0; step < step1 && ok; step++) {
        const int pos = P.pos0 + step;
        if (tid < HD / 2) {
            const double th = (double)__fmul_rn((float)pos, __ldg(P.rope_freq + tid));    // fp32 angle, as src/cpu_infer.cpp:54
            sm.cs[tid] = __double2float_rn(cos(th)); sm.cs[HD / 2 + tid] = __double2float_rn(sin(th));
        }
        __syncthreads();
        for (int ph = ph0; ph < ph1 && ok; ph++) {
            const int l = ph / 5, k = ph == nph - 1 ? 5 : ph % 5;
            if (k == 0) {
                // ---- QKV
                if (l == 0) {
                    const int tok = step < P.n_forced ? __ldg(P.in_tokens + step) : __ldcg(P.cur_token);
                    embed_row(P, tok, hs);
                    __syncthreads();
                    if (blockIdx.x == 0) for (int i = tid; i < P.E; i += DNT) __stcg(P.h + i, hs[i]);
                } else {
                    for (int i = tid; i < P.E; i += DNT) hs[i] = __ldcg(P.h + i);
                    __syncthreads();
                }
                stage_norm_q8(hs, P.layers[l].attn_norm, P.E, P.eps, sm.red, xq_s, xs_s);
                const float* bias = P.layers[l].bqkv;
                const int nq = P.NH * HD;
                __half* kdst = P.kc + ((size_t)l * P.max_seq + pos) * P.KVD;
                __half* vdst = P.vc + ((size_t)l * P.max_seq + pos) * P.KVD;
                ok = run_job(ws, P, 4 * l + 0, lane, xq_s, xs_s, [&](int g, int ln, float v0, float) {
                    const int p = g * 32 + ln;
                    const float v = __fadd_rn(v0, __ldg(bias + p));
                    const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
                    if (p < nq + P.KVD) {                                  // q or k: rotate the (even, odd) lane pair
                        const int base = p < nq ? p : p - nq, head = base / HD, within = base % HD, i = within >> 1;
                        const double c = sm.cs[i], s = sm.cs[HD / 2 + i];
                        float out; int orig;                               // products are exact in double: one rounding each
                        if ((within & 1) == 0) { out = __double2float_rn(__dsub_rn(__dmul_rn((double)v, c), __dmul_rn((double)partner, s))); orig = head * HD + i; }
                        else { out = __double2float_rn(__dadd_rn(__dmul_rn((double)partner, s), __dmul_rn((double)v, c))); orig = head * HD + i + HD / 2; }
                        if (p < nq) __stcg(P.q + orig, out);
                        else kdst[orig] = __float2half_rn(out);
                    } else {
                        vdst[p - nq - P.KVD] = __float2half_rn(v);
                    }
                });
            } else if (k == 1) {
                attention_phase<HD, G>(P, l, pos, sm.stage);
            } else if (k == 2) {
                stage_copy_q8(P.att_q, P.att_d, P.E / 32, xq_s, xs_s);
                ok = run_job(ws, P, 4 * l + 1, lane, xq_s, xs_s, [&](int g, int ln, float v0, float) {
                    const int r = g * 32 + ln;
                    if (r < P.E) __stcg(P.h + r, __fadd_rn(__ldcg(P.h + r), v0));
                });
            } else if (k == 3) {
                for (int i = tid; i < P.E; i += DNT) hs[i] = __ldcg(P.h + i);
                __syncthreads();
                stage_norm_q8(hs, P.layers[l].ffn_norm, P.E, P.eps, sm.red, xq_s, xs_s);
                ok = run_job(ws, P, 4 * l + 2, lane, xq_s, xs_s, [&](int g, int ln, float gate, float up) {
                    const double gd = (double)gate;
                    const float a = __double2float_rn(__dmul_rn(__ddiv_rn(gd, __dadd_rn(1.0, exp(-gd))), (double)up));
                    const int r = g * 32 + ln;                            // FF is a multiple of 32: whole q8_0 block per warp
                    const int qv = quant_block_warp(a, ln, nullptr, P.act_d + g);
                    P.act_q[r] = (int8_t)qv;
                });
            } else if (k == 4) {
                stage_copy_q8(P.act_q, P.act_d, P.FF / 32, xq_s, xs_s);
                ok = run_job(ws, P, 4 * l + 3, lane, xq_s, xs_s, [&](int g, int ln, float v0, float) {
                    const int r = g * 32 + ln;
                    if (r < P.E) __stcg(P.h + r, __fadd_rn(__ldcg(P.h + r), v0));
                });
            } else {
                // ---- final norm, lm_head, greedy argmax (lowest index wins ties)
                for (int i = tid; i < P.E; i += DNT) hs[i] = __ldcg(P.h + i);
                __syncthreads();
                stage_norm_q8(hs, P.out_norm, P.E, P.eps, sm.red, xq_s, xs_s);
                float best = -INFINITY; int bidx = 0x7fffffff;
                float* lg = P.logits ? P.logits + (long long)(step - step0) * P.logits_stride : nullptr;
                ok = run_job(ws, P, 4 * P.L, lane, xq_s, xs_s, [&](int g, int ln, float v0, float) {
                    const int r = g * 32 + ln;
                    if (r < P.V) {
                        if (lg) lg[r] = v0;
                        if (v0 > best || (v0 == best && r < bidx)) { best = v0; bidx = r; }
                    }
                });
                #pragma unroll
                for (int o = 16; o; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
                    if (ob > best || (ob == best && oi < bidx)) { best = ob; bidx = oi; }
                }
                __syncthreads();                                        // staging region is free again
                float* cv = reinterpret_cast<float*>(sm.red); int* ci = reinterpret_cast<int*>(sm.red) + 16;
                if (lane == 0) { cv[warp] = best; ci[warp] = bidx; }
                __syncthreads();
                if (tid == 0) {
                    for (int w = 1; w < DNW; w++) if (cv[w] > cv[0] || (cv[w] == cv[0] && ci[w] < ci[0])) { cv[0] = cv[w]; ci[0] = ci[w]; }
                    __stcg(P.cand_val + blockIdx.x, cv[0]); __stcg(P.cand_idx + blockIdx.x, ci[0]);
                    __threadfence();
                    const unsigned prev = atomicAdd(P.cand_cnt, 1u);
                    if (prev == gridDim.x - 1) {                        // last CTA: final pick over all CTAs' candidates
                        __threadfence();
                        float b = -INFINITY; int bi = 0x7fffffff;
                        for (unsigned c = 0; c < gridDim.x; c++) {
                            const float v = __ldcg(P.cand_val + c); const int ix = __ldcg(P.cand_idx + c);
                            if (v > b || (v == b && ix < bi)) { b = v; bi = ix; }
                        }
                        *P.cand_cnt = 0;
                        __stcg(P.cur_token, bi);
                        P.out_tokens[step] = bi;
                    }
                }
            }
            ok = __syncthreads_and(ok ? 1 : 0) != 0;          // a wait that gave up in one warp stops the whole CTA
            if (!ok) break;
            const bool last = (step == step1 - 1) && (ph == ph1 - 1);
            if (!single && !last) ok = grid_barrier(P.bar, bar_target, &s_ok);
        }
    }
    if (!ok) {
        if (lane == 0) atomicMax(P.err, MI_ERR_TIMEOUT);
        ws.drain();
    }
}

#endif  // __CUDACC__
}  // namespace mi
