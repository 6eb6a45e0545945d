// The fused decode step for sm_100a: one persistent kernel that runs any range of
// the per-token phases
//     per layer:  QKV  (residual add -> rmsnorm -> q8 -> GEMV -> +bias, RoPE, q / k / v)
//                 ATTN (split-KV attention over the fp16 cache, merge, -> q8)
//                 O    (GEMV)
//                 GU   (residual add -> rmsnorm -> q8 -> gate & up GEMV -> SwiGLU -> q8)
//                 DOWN (GEMV, K-split over CTAs, folded by the split-0 CTA)
//     finally:    LM   (residual add -> rmsnorm -> q8 -> lm_head GEMV -> argmax)
// for any range of steps.  Launched with one phase per launch it is a plain
// kernel sequence; launched cooperatively (all CTAs resident) over all phases and
// steps it is the persistent decode loop.
//
// No grid barrier.  The reference's persistent kernel separates its phases by a
// grid-wide barrier (src/mega.cu:123-134, five per layer).  Here every value that
// one CTA hands to another travels as a TAGGED WORD: 8 bytes = {32-bit payload,
// 32-bit tag}, written and read as one naturally aligned 64-bit access (single-copy
// atomic).  The tag numbers the (step, phase) that produced the value.  A consumer
// simply loads the words it needs and looks at their tags; words that are not there
// yet are polled (bounded by a time budget).  There is no separate flag, hence no
// release fence before it and no second round trip after it: a phase boundary costs
// one store-to-load hop through the L2 instead of arrive + poll + reload, and a CTA
// waits only for the values it actually consumes.  Buffers are reused every layer;
// a word can only be overwritten after every reader has passed on, because the
// writer's own inputs descend from outputs of those readers (each layer has phases
// in which every CTA produces something that every CTA consumes).  A reader that
// nevertheless fell behind would see a wrong tag and time out - never wrong data.
// The same words, stored additionally into the other GPUs' copies of the buffers
// over NVLink (plain 8-byte peer stores), are the whole tensor-parallel exchange.
//
// The residual stream lives in shared memory: every CTA adds the same projection
// outputs to its own copy (the arithmetic is deterministic, all copies hold the
// same bits), so it never travels.  The first GEMV CTA also writes it to global memory
// for launches that start in the middle of a step, and for inspection.
//
// Work split.  Every GEMV phase is a "job" over a tiled q4_0 matrix.  For the
// per-layer matrices a unit is (32-row group [gate/up: a pair of groups], K-split)
// and belongs to a CTA: its eight warps take the unit's tiles round-robin and
// fold their double partial sums through shared memory.  The down projection has
// fewer row groups than the grid has CTAs, so its K dimension is additionally split
// across CTAs; splits 1.. hand their double partial sums (two tagged words each) to
// the CTA of split 0, which adds them in split order and publishes the fp32 row.
// The lm_head has thousands of row groups: there a unit is a row group and belongs
// to one warp.
//
// Weight streaming.  The whole tile sequence of a warp - across phases, layers
// and steps - follows from shapes and indices alone, so lane 0 of every warp
// keeps a private shared-memory ring full with bulk copies that run ahead of
// the phase boundaries: weights are immutable, the HBM stream never waits for a
// phase, only for ring space.
//
// Numerics follow the reference (paths relative to its root): quantizer
// src/cuda_infer.cu:80-89; block dot src/mega.cu:151-165; RMSNorm / RoPE / SwiGLU /
// argmax src/cpu_infer.cpp:40-61,147,153-154; split-KV merge
// src/cuda_infer.cu:650-702.  Every sum that feeds a stored tensor (GEMV rows,
// RMSNorm sum of squares, attention scores, softmax denominator and weighted
// values) is carried in double and rounded to fp32 once; exp, cos and sin come
// from the double math library.  A q8_0 quantizer is discontinuous, so this is
// what lets two engines (or two split / step / shard configurations of this one)
// agree bit for bit: every term of a GEMV sum is a multiple of 2^-48 (fp16 x fp16 x
// integer), so while a sum stays below 2^5 in magnitude the double additions are
// exact and the fp32 value cannot depend on their order; beyond that it has been
// observed, not proved.  Each token is processed exactly as if it were alone.
#pragma once
#include "gemv_core.cuh"
#ifndef MI_ATT_FN
#define MI_ATT_FN static __device__ __noinline__
#endif
// functions that sit out of line to keep the loop body small; the short-context build inlines them instead, because every
// call site inside the step loop, executed or not, makes the compiler keep the loop's values where a call preserves them
#if defined(MI_LEAN) && MI_LEAN
#define MI_COLD_FN static __device__ __forceinline__
#else
#define MI_COLD_FN static __device__ __noinline__
#endif
#ifndef MI_PIECE
#define MI_PIECE __forceinline__
#endif
#ifndef MI_ATTN_HPC_EVEN
#define MI_ATTN_HPC_EVEN(G) 2
#endif

// The kernel exists in four builds.  The default one carries no profiling code and no peer stores.  A translation unit
// that defines MI_PROF 1 before including this file gets the instrumented build (timer marks between the hot instructions
// cost a few percent when merely compiled in); MI_TP 1 gives the tensor-parallel build, whose publishing stores also go to
// the other GPUs; MI_LEAN 2 and 3 are the same idea for 257..kPerHeadAttnMax positions (one query head per CTA and chunk) and
// beyond (a whole GQA group per CTA and chunk): one attention variant each; MI_LEAN 1 gives the short-context build, which holds no attention code but that of the dedicated
// attention CTAs (launched only for step ranges that end within kShortAttnMax positions on a model with such CTAs: without
// the other attention variants in the same function the GEMV CTAs' loop keeps its values in registers).  They live in
// different inline namespaces, so all can be linked into one library and picked at launch time.
#ifndef MI_PROF
#define MI_PROF 0
#endif
#ifndef MI_TP
#define MI_TP 0
#endif
#ifndef MI_LEAN
#define MI_LEAN 0
#endif
#if MI_PROF && MI_TP && MI_LEAN
#define MI_KVARIANT tpxproflean
#elif MI_PROF && MI_LEAN
#define MI_KVARIANT proflean
#elif MI_PROF
#define MI_KVARIANT prof
#elif MI_TP && MI_LEAN
#define MI_KVARIANT tpxlean
#elif MI_TP
#define MI_KVARIANT tpx
#elif MI_LEAN == 2
#define MI_KVARIANT leanmid
#elif MI_LEAN == 3
#define MI_KVARIANT leanlong
#elif MI_LEAN
#define MI_KVARIANT lean
#else
#define MI_KVARIANT fast
#endif

namespace mi {

constexpr int DNW = 8;            // warps per CTA
constexpr int DNT = DNW * 32;
constexpr int DS = 3;             // ring slots per warp
constexpr int DSLOT = 4608;       // bytes per slot: the largest tile (8 blocks)
constexpr int kAttnChunk = 64;    // smallest KV range worth its own CTA
constexpr int kShortAttnMax = 256;      // up to this many cached positions one CTA handles the whole range of a query head (attention_short)
constexpr int kPerHeadAttnMax = 1024;   // up to this many cached positions a CTA handles one query head, beyond it a whole GQA group
constexpr int kMaxKSplit = 4;     // cross-CTA K-splits of the down projection
constexpr int kMaxWorldTP = 8;

// profile slots: 2*k = staging of phase kind k, 2*k+1 = its main work; 12 = time spent waiting for tagged words, 13 = step prologue
enum { kProfWait = 12, kProfStep = 13, kProfSlots = 32 };

enum JobKind { JOB_QKV = 0, JOB_O = 1, JOB_GU = 2, JOB_DOWN = 3, JOB_LM = 4 };

struct Job {
    const uint8_t* base;   // tiled weights
    int groups;            // unit groups; one unit group = nacc consecutive 32-row groups
    int nt, ks, nb, kb, nacc, kind;
    int n_units;           // groups * ks
    int rot;               // CTA (per-layer jobs) or warp slot (lm_head) that gets unit 0
    int wrot;              // warp that gets tile 0 of a CTA unit
    unsigned ks_inv;       // ceil(2^32 / ks): x / ks == __umulhi(x, ks_inv) for the unit and tile counts that occur (set by the host)
    int layer;
    int g_off;             // first unit group this GPU owns (tensor parallelism; base points at it, groups counts the owned ones)
    int pad_;
};

struct LayerPtrs { const float* attn_norm; const float* ffn_norm; const float* bqkv; };

// Tensor parallelism inside the kernel: the other GPUs' exchange blocks (CUDA IPC mappings).  on == 0: single GPU, or
// exchanges done by the host program between launches.
struct TpPeerParams {
    int on, rank, world, pad_;
    unsigned long long* xw_peer[kMaxWorldTP];     // exchange block on every GPU (own entry = local block)
};

// Offsets (in 8-byte words) of the tagged vectors inside the exchange block.  q8_0 vectors are stored as
// [n/4] words of four int8 values followed by [n/32 (+1 if odd)] words of {fp16 scale bits | int16 sum of the block's values << 16}.
struct XwLayout {
    int qkv;        // [qkv rows, padded to 32]   fp32 bits: q | k | v after bias and RoPE, packed (pair-adjacent) order
    int att;        // q8_0 of the merged attention output [NH*HD]
    int o;          // [E] fp32 bits: O projection
    int act;        // q8_0 of SwiGLU(gate, up) [FF]                                     (pushed to the other GPUs)
    int down;       // [E] fp32 bits: down projection                                    (pushed)
    int dpart;      // [E/32][kMaxKSplit-1][32][2]: double partial sums (lo, hi) of the down K-splits 1..
    int cand;       // [kMaxWorldTP][grid][4]: argmax candidates {best value}, {its row}, {second-best value}, -   (pushed)
    int tokw;       // [2]: the token picked by the step that just ended, for the attention CTAs (written only under a stop rule)
    int total;
};

// Host-mapped (pinned, device-visible) memory through which a running generation hands its tokens to the host
// (src/mega.cu:1130-1137): the kernel fills tokens / margins / ns from entry `base` on and raises *count.
struct TokenRing { int* count; int* tokens; float* margins; unsigned long long* ns; int capacity, base; };

struct DecodeParams {
    int L, E, FF, NH, NKV, HD, KVD, V;
    float eps;
    const Job* jobs;                 // [4L+1] in phase order
    const unsigned long long* tile_tab;   // per warp slot: source address | kb code of every tile of one step, in consumption order
    const unsigned* tile_start;      // [grid*DNW][4L+2]: index of each job's first tile in the warp's list (last = count)
    int tile_stride;                 // entries reserved per warp slot in tile_tab
    const LayerPtrs* layers;         // [L]
    const float* out_norm;
    const float* rope_freq;          // [HD/2]: base^(-2i/HD), computed on the host with powf
    const float* rope_cs;            // [rope_rows][HD]: cos then sin of every position's HD/2 angles, made once at load (rope_cs_kernel)
    int rope_rows;                   // = the model's max_seq at load
    const uint8_t* emb_base;         // tiled token embedding (may alias the lm_head)
    int emb_nt, emb_kb;
    const uint8_t* emb_q8;           // or, when set: the embedding as stored Q8_0 rows (34-byte blocks), read instead of emb_base
    // residual stream as committed by CTA 0: read by a launch that starts in the middle of a step, and by tests
    float* h_in;                     // at the input of the current layer
    float* h_mid;                    // after the attention block
    // the exchange block: every vector one CTA hands to another, as tagged words
    unsigned long long* xw; XwLayout xo;
    // Tag of (step s of the launch, phase p) = epoch + s * (5L+1) + p + 1.  The epoch lives in device memory and the kernel
    // advances it itself: a launch whose phase range ends a step leaves it past every tag the launch used (a launch that
    // gave up on a wait: further still).  Replayed launch sequences and calls after a failure therefore never meet a stale
    // word with a matching tag; launches that continue a step (phase range not starting at 0) share its epoch.
    unsigned* epoch_dev;
    unsigned long long wait_ns;      // time budget of every device-side wait
    int drop_phase;                  // test hook: the producers of this phase publish nothing (-1: none), so that its consumers' waits run out
    // plain (untagged) vectors: inputs / outputs of the attention code when it runs as a kernel of its own (M-token step)
    float* qkv_out;
    float* att;                      // merged attention output, fp32 (also written by the decode loop, for inspection)
    int8_t* att_q; __half* att_d;
    __half* kc; __half* vc; int max_seq;       // [L][max_seq][KVD]
    double* attn_part; unsigned* attn_cnt; int max_chunks;  // [NH][max_chunks][HD+2], [NKV]
    float* out_margins;              // optional [n_steps]: top-1 minus top-2 logit of every step
    TokenRing ring;                  // optional: host-mapped ring the first GEMV CTA publishes every step's token into
    float* best_val;                 // value of the best logit (tensor parallelism with host-side exchange: this GPU's rows only)
    const int* in_tokens; int n_forced; int* out_tokens; int* cur_token;
    int stop_token;                  // >= 0: a run over whole steps ends after the step that picks this token as the next input
                                     // (text generation's end-of-sequence rule, src/mega.cu:868-874); -1: off
    float* logits; long long logits_stride;    // optional [n_steps][stride]
    int pos0;
    const int* pos_dev;              // optional: first position read from device memory instead (a captured launch sequence stays position-free)
    int* err;
    unsigned long long* prof;        // optional [32]: nanoseconds per phase part on CTA prof_cta (see kProf*)
    int prof_cta;
    // CTAs [0, attn_ctas) do nothing but attention; the GEMV phases (and the greedy pick) are dealt over the other
    // CTAs [attn_ctas, grid).  At short context one CTA per query head runs attention, and a CTA that also carried GEMV
    // units would walk both phases' code every layer; kept apart, each CTA's instructions stay in its instruction cache.
    // 0: every CTA does everything.  Beyond kShortAttnMax positions the GEMV CTAs take attention chunks as well.
    int attn_ctas;
    TpPeerParams tp;
};

// number of KV chunks for a causal range of Lp positions (host and device agree)
__host__ __device__ inline int attn_chunks(int Lp, int max_chunks, int chunk = kAttnChunk) {
    int n = (Lp + chunk - 1) / chunk;
    return n < 1 ? 1 : (n > max_chunks ? max_chunks : n);
}
__host__ __device__ inline int q8_words(int n) { return n / 4 + (n / 32 + 1) / 2 * 2; }     // tagged words of a q8_0 vector of n values

#ifdef __CUDACC__
inline namespace MI_KVARIANT {

struct DecodeSmem {
    uint8_t* ring; uint64_t* bars; Job* jobs; LayerPtrs* lp; float* cs; double* red; double* fold; float* h; uint8_t* stage;
};

constexpr int kFoldBytes = 2 * DNW * 2 * 32 * 8;      // two buffers of [warp][acc][lane] doubles

__host__ __device__ inline size_t decode_stage_bytes(int E, int FF, int HD, int G) {
    const int maxin = E > FF ? E : FF;
    size_t a = (size_t)maxin + (size_t)(maxin / 32) * 8;               // xq, xs
    size_t b = (size_t)DNW * G * (HD + 2) * 8 + (size_t)DNW * 32 * G * 8 + (size_t)G * (HD + 16) * 8;   // attention: states, weights, q (double, padded)
    return ((a > b ? a : b) + 127) / 128 * 128;
}
__host__ __device__ inline size_t decode_smem_bytes(int njobs, int E, int FF, int HD, int G) {
    return (size_t)DNW * DS * DSLOT + 256 + ((size_t)njobs * sizeof(Job) + 127) / 128 * 128 + 64 * sizeof(LayerPtrs) + 1024 + 256 + kFoldBytes +
           ((size_t)E * 4 + 127) / 128 * 128 + decode_stage_bytes(E, FF, HD, G);
}

// close the current profile interval: charge the time since t to slot k (CTA 0, thread 0 only).
// The sums live in shared memory and are flushed once at kernel exit, so a mark costs a
// timer read and a shared-memory add, not a global round trip on the critical path.
#if MI_PROF
__shared__ unsigned long long s_prof[kProfSlots];
__shared__ unsigned long long s_prof_t;          // start of the open interval (thread 0 of the profiled CTA)
#endif
__device__ __forceinline__ void prof_mark(const DecodeParams& P, int k) {
#if MI_PROF
    if (P.prof && (int)blockIdx.x == P.prof_cta && threadIdx.x == 0) { const unsigned long long n = gtime_ns(); s_prof[k] += n - s_prof_t; s_prof_t = n; }
#endif
}

// A greedy-pick candidate: best value, its row (lowest row wins ties), and the runner-up value.
struct Cand {
    float best; int idx; float second;
    __device__ __forceinline__ void add(float v, int r) {
        if (v > best || (v == best && r < idx)) { second = best; best = v; idx = r; }
        else if (v > second) second = v;
    }
    __device__ __forceinline__ void merge(const Cand& o) {
        if (o.best > best || (o.best == best && o.idx < idx)) { second = fmaxf(best, o.second); best = o.best; idx = o.idx; }
        else second = fmaxf(second, o.best);
    }
    __device__ __forceinline__ void warp_reduce() {
        #pragma unroll
        for (int s = 16; s; s >>= 1) {
            Cand o;
            o.best = __shfl_xor_sync(0xffffffffu, best, s); o.idx = __shfl_xor_sync(0xffffffffu, idx, s); o.second = __shfl_xor_sync(0xffffffffu, second, s);
            merge(o);
        }
    }
};

// ---- tagged words ---------------------------------------------------------------------
// One 64-bit access carries value and tag together, so there is nothing to order between them.
// The accesses are volatile: they are performed at the L2 (the point where all SMs of this GPU,
// and peers storing over NVLink, meet), once each, in program order.
__device__ __forceinline__ unsigned long long tw_ld(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void tw_ld2(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {   // 16-byte aligned pair; each word is checked on its own
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ void tw_st(unsigned long long* p, unsigned tag, unsigned payload) {
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(((unsigned long long)tag << 32) | payload) : "memory");
}
__device__ __forceinline__ bool tw_is(unsigned long long w, unsigned tag) { return (unsigned)(w >> 32) == tag; }

// Where a phase publishes: locally, and (tensor-parallel build, shared vectors) into every other GPU's block.
struct Pub {
    unsigned long long* xw; unsigned tag; bool mute;
#if MI_TP
    const TpPeerParams* tp;
#endif
    __device__ __forceinline__ void local(int off, unsigned payload) const { if (!mute) tw_st(xw + off, tag, payload); }
    __device__ __forceinline__ void shared(int off, unsigned payload) const {
        if (mute) return;
        tw_st(xw + off, tag, payload);
#if MI_TP
        if (tp->on) {
            for (int p = 0; p < tp->world; p++) if (p != tp->rank) tw_st(tp->xw_peer[p] + off, tag, payload);
        }
#endif
    }
};

// Poll one word until it carries `tag`.  Gives up (false) when the time budget has run out or another CTA has reported
// an error; the caller then leaves the kernel through its error path.
MI_COLD_FN bool tw_spin(const unsigned long long* p, unsigned tag, unsigned long long budget_ns, const int* err) {
    unsigned long long t0 = 0;
    for (unsigned it = 1;; it++) {
        if (tw_is(tw_ld(p), tag)) return true;
        if ((it & 31u) == 0) {
            const unsigned long long now = gtime_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > budget_ns || *reinterpret_cast<const volatile int*>(err) != 0) return false;
        }
    }
}

// One warp waits together: the lowest lane that misses a word polls that word, the other lanes sit at the vote, so a
// waiting warp keeps one load in flight, not thirty-two (148 CTAs polling with every thread load the L2 as hard as the
// weight stream does).  Called by all lanes of a warp with the first missing address of each (null: none).  Returns 0 when
// no lane misses anything, 1 after the polled word has arrived (every lane then fetches its missing words again), -1 when
// the wait gave up.
__device__ __forceinline__ int tw_wait_warp(const unsigned long long* miss, unsigned tag, unsigned long long budget_ns, const int* err) {
    const unsigned mm = __ballot_sync(0xffffffffu, miss != nullptr);
    if (!mm) return 0;
    const int leader = __ffs(mm) - 1;
    int r = 1;
    if ((int)(threadIdx.x & 31) == leader) r = tw_spin(miss, tag, budget_ns, err) ? 1 : -1;
    return __shfl_sync(0xffffffffu, r, leader);
}

// Load the N words addr(k) (k with bit k of `valid` set) and return their payloads once all carry `tag`.  All loads are
// issued before any is looked at; if some word is not there yet, the warp polls one such word and then every lane fetches
// its missing words again (they were produced together, most have landed meanwhile).  All 32 lanes of a warp must call.
template <int N, class AddrFn>
__device__ __forceinline__ bool tw_poll(const DecodeParams& P, unsigned tag, unsigned valid, AddrFn addr, unsigned (&out)[N]) {
    unsigned long long w[N];
    #pragma unroll
    for (int k = 0; k < N; k++) w[k] = (valid >> k & 1u) ? tw_ld(addr(k)) : ((unsigned long long)tag << 32);
    for (;;) {
        const unsigned long long* miss = nullptr;
        #pragma unroll
        for (int k = N - 1; k >= 0; k--) if (!tw_is(w[k], tag)) miss = addr(k);
        const int st = tw_wait_warp(miss, tag, P.wait_ns, P.err);
        if (st == 0) break;
        if (st < 0) return false;
        #pragma unroll
        for (int k = 0; k < N; k++) if (!tw_is(w[k], tag)) w[k] = tw_ld(addr(k));
    }
    #pragma unroll
    for (int k = 0; k < N; k++) out[k] = (unsigned)w[k];
    return true;
}

// ---- the per-warp weight stream -----------------------------------------------
// Tiles of a unit are numbered i = a*ntu + (t - t0) (a = accumulator, ntu = tiles of
// the unit's K range).  In a CTA unit warp w owns the tiles with (i + wrot(u)) % 8 == w;
// in a warp unit (lm_head) the owning warp takes all of them.
struct UnitShape { int g, sp, t0, ntu, n, wrot; };

__device__ __forceinline__ UnitShape unit_shape(const Job& jb, int u, int uidx) {
    UnitShape s;
    if (jb.ks == 1) { s.g = u; s.sp = 0; s.t0 = 0; s.ntu = jb.nt; }
    else {
        // divisions by the K-split count through the host's reciprocal: exact for operands below 2^20 with ks <= kMaxKSplit
        s.g = (int)__umulhi((unsigned)u, jb.ks_inv); s.sp = u - s.g * jb.ks;
        s.t0 = (int)__umulhi((unsigned)(s.sp * jb.nt), jb.ks_inv);
        s.ntu = (int)__umulhi((unsigned)((s.sp + 1) * jb.nt), jb.ks_inv) - s.t0;
    }
    s.n = jb.nacc * s.ntu;
    s.wrot = (jb.wrot + uidx * 3) & (DNW - 1);      // uidx: how many units this CTA had before u in the job
    return s;
}

// Producer side of a warp's ring.  The order in which a warp consumes tiles is a pure
// function of shapes and indices, so the host lists it once per model: entry k of a warp's
// list is the global address of its k-th tile of a step (16-byte aligned; the low two bits
// carry log2 of the tile depth).  The producer walks that list, wrapping at the end of the
// launch's job range, with the next entry already loaded so that issuing a copy costs a
// handful of instructions and no division.
struct WarpStream {
    uint8_t* ring; uint64_t* bars; const Job* jobs;
    const unsigned long long* tab;   // this warp's list
    unsigned e0, e1, c;              // entry range of the launch's jobs within a step; cursor
    long long left;                  // tiles still to issue in this launch
    unsigned long long next;         // entry at the cursor (valid while left > 0)
    int issued, consumed;
    int W, sid, warp;                // warp slots in the grid, this warp's slot, warp in CTA
    int gcta, ggrid;                 // this CTA's index among the CTAs that carry GEMV units (negative: attention only), their number
    uint64_t policy;                 // L2 evict-first for the weight stream

    __device__ __forceinline__ void init(const DecodeSmem& sm, const DecodeParams& P, int warp_, int step0, int step1, int j0, int j1) {
        warp = warp_; policy = l2_policy_evict_first();
        ring = sm.ring + (size_t)warp * DS * DSLOT; bars = sm.bars + warp * DS; jobs = sm.jobs;
        gcta = (int)blockIdx.x - P.attn_ctas; ggrid = (int)gridDim.x - P.attn_ctas;
        W = ggrid * DNW; sid = warp * ggrid + gcta;      // consecutive warp units land on different SMs
        if (gcta < 0) { e0 = e1 = c = 0; issued = consumed = 0; left = 0; next = 0ull; tab = nullptr; return; }
        const int slot = gcta * DNW + warp, nj = 4 * P.L + 2;
        tab = P.tile_tab + (size_t)slot * P.tile_stride;
        e0 = __ldg(P.tile_start + (size_t)slot * nj + j0);
        e1 = __ldg(P.tile_start + (size_t)slot * nj + j1);
        c = e0; issued = consumed = 0;
        left = j0 < j1 ? (long long)(step1 - step0) * (e1 - e0) : 0;
        next = left > 0 ? __ldg(tab + c) : 0ull;
    }
    __device__ __forceinline__ void issue_one() {       // lane 0 only
        if (left <= 0) return;
        const unsigned long long e = next;
        const int tb = kTileRowBytes << (int)(e & 3ull), slot = issued % DS;
        mbar_expect_tx(&bars[slot], tb);
        bulk_g2s_hint(ring + (size_t)slot * DSLOT, reinterpret_cast<const void*>(e & ~15ull), tb, &bars[slot], policy);
        issued++;
        if (++c == e1) c = e0;
        if (--left > 0) next = __ldg(tab + c);
    }
    __device__ __forceinline__ void drain() {
        for (int k = consumed; k < issued; k++) (void)mbar_wait_bounded(&bars[k % DS], (k / DS) & 1);
    }
    __device__ __forceinline__ int first_cta_unit(const Job& jb) const {
        const int G = ggrid, r = jb.rot, b = gcta;         // the host keeps rot below the number of GEMV CTAs
        return b >= r ? b - r : b + G - r;
    }
    __device__ __forceinline__ int first_warp_unit(const Job& jb) const {
        const int r = jb.rot % W; return sid >= r ? sid - r : sid + W - r;
    }
};

// The per-token loop body must stay small: it is executed phase after phase by every SM, and measured, the kernel ran
// 15 % faster once the four GEMV phases shared one copy of their code.  So the double-precision exponential has one
// out-of-line copy, and the variants a given model never takes (other tile depths, other norm widths) sit out of line
// instead of between the hot instructions.
MI_COLD_FN double exp_shared(double x) { return exp(x); }
static __device__ __noinline__ double tile_dot_row_rare(int kb, const uint8_t* tile, int lane, int t, const int8_t* xq_s, const float2* xs_s, double acc) {
    switch (kb) {
        case 4: return tile_dot_row<4, false>(tile, lane, t * 4, xq_s, xs_s, acc, nullptr);
        case 2: return tile_dot_row<2, false>(tile, lane, t * 2, xq_s, xs_s, acc, nullptr);
        default: return tile_dot_row<1, false>(tile, lane, t, xq_s, xs_s, acc, nullptr);
    }
}

// consume the next tile of this warp's stream into acc (block index b0 = t * kb)
__device__ __forceinline__ double tile_consume(WarpStream& ws, int lane, int kb, int t, const int8_t* xq_s, const float2* xs_s,
                                               double acc, bool& ok, const DecodeParams* PP = nullptr) {
    if (!ok) return acc;
    const int slot = ws.consumed % DS;
    if (PP) prof_mark(*PP, 18);
    if (!mbar_wait_bounded(&ws.bars[slot], (ws.consumed / DS) & 1)) { ok = false; return acc; }
    if (PP) prof_mark(*PP, 20);
    const uint8_t* tile = ws.ring + (size_t)slot * DSLOT;
#if MI_LEAN
    acc = tile_dot_row<8, false>(tile, lane, t * 8, xq_s, xs_s, acc, nullptr);          // lean_shape_ok(): every tile is 8 blocks deep
#else
    if (kb == 8) acc = tile_dot_row<8, false>(tile, lane, t * 8, xq_s, xs_s, acc, nullptr);
    else acc = tile_dot_row_rare(kb, tile, lane, t, xq_s, xs_s, acc);
#endif
    ws.consumed++;
    __syncwarp();
    if (PP) prof_mark(*PP, 21);
    if (lane == 0) ws.issue_one();
    __syncwarp();
    if (PP) prof_mark(*PP, 22);
    return acc;
}

// q8_0 of one 32-element block held one element per lane; returns the int8 value, and through
// d_out / s_out (all lanes) the fp16 scale and the integer sum of the block's values.
__device__ __forceinline__ int quant_block_warp2(float v, __half& d_out, int& s_out) {
    const float a = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(v))));
    const float inv = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
    const int q = __float2int_rn(__fmul_rn(v, inv));
    s_out = __reduce_add_sync(0xffffffffu, q);
    d_out = __float2half_rn(__fdiv_rn(a, 127.f));
    return q;
}
// Publish one q8_0 block (lane = element) as tagged words: lanes 0, 4, 8, .. store four int8 values each, lane 0
// also the scale word.  qoff / soff: word offsets of the vector's value and scale parts; b: block index.
template <bool SHARED>
__device__ __forceinline__ void publish_q8_block(const Pub& pub, int qoff, int soff, int b, int lane, int q, __half d, int s) {
    unsigned v = (unsigned)q & 0xffu;
    v |= __shfl_down_sync(0xffffffffu, v, 1) << 8;
    v |= __shfl_down_sync(0xffffffffu, v, 2) << 16;
    const unsigned sw = (unsigned)__half_as_ushort(d) | ((unsigned)s << 16);
    if ((lane & 3) == 0) { if (SHARED) pub.shared(qoff + b * 8 + (lane >> 2), v); else pub.local(qoff + b * 8 + (lane >> 2), v); }
    if (lane == 0) { if (SHARED) pub.shared(soff + b, sw); else pub.local(soff + b, sw); }
}

// Per-layer job: this CTA's units, tiles split over its warps, partial sums folded in
// shared memory in warp order by warp 0, which then calls epi(g, lane, v0, v1) with the
// complete sums rounded to fp32.  A job that is K-split across CTAs (ks > 1; down projection)
// adds one hop: the CTAs of splits 1.. publish their double partial sums as tagged word pairs,
// the CTA of split 0 waits for them, adds them to its own in split order and calls epi.
// Every warp passes the same number of __syncthreads, also after a wait gave up.
template <class Epi>
__device__ MI_PIECE bool run_cta_job(WarpStream& ws, const DecodeParams& P, const DecodeSmem& sm, int j, int lane,
                                            const int8_t* xq_s, const float2* xs_s, const Pub& pub, Epi epi) {
    const Job jb = ws.jobs[j];                          // registers: the fields are used many times
    bool ok = true;
    int uidx = 0;
    for (int u = ws.first_cta_unit(jb); u < jb.n_units; u += ws.ggrid, uidx++) {
        const UnitShape s = unit_shape(jb, u, uidx);
        double a0 = 0.0, a1 = 0.0;
        for (int i = (ws.warp - s.wrot) & (DNW - 1); i < s.n; i += DNW) {
            const bool first = i < s.ntu;                       // which of the unit's two accumulators (gate / up) the tile feeds
            const double r = tile_consume(ws, lane, jb.kb, s.t0 + (first ? i : i - s.ntu), xq_s, xs_s, first ? a0 : a1, ok, &P);
            if (first) a0 = r; else a1 = r;
        }
        prof_mark(P, 18);
        double* fb = sm.fold + (size_t)(uidx & 1) * DNW * 2 * 32;
        fb[(ws.warp * 2) * 32 + lane] = a0;
        fb[(ws.warp * 2 + 1) * 32 + lane] = a1;
        __syncthreads();
        if (ws.warp == 0) {
            double v0 = fb[lane], v1 = fb[32 + lane];
            #pragma unroll
            for (int w = 1; w < DNW; w++) { v0 = __dadd_rn(v0, fb[(w * 2) * 32 + lane]); v1 = __dadd_rn(v1, fb[(w * 2 + 1) * 32 + lane]); }
            const int gg = s.g + jb.g_off;
            if (jb.ks > 1) {
                const int slot = P.xo.dpart + ((gg * (kMaxKSplit - 1)) * 32 + lane) * 2;
                if (s.sp != 0) {
                    const unsigned long long bits = (unsigned long long)__double_as_longlong(v0);
                    pub.local(slot + (s.sp - 1) * 64, (unsigned)bits);
                    pub.local(slot + (s.sp - 1) * 64 + 1, (unsigned)(bits >> 32));
                } else {
                    unsigned pw[2 * (kMaxKSplit - 1)];
                    const unsigned long long* base = P.xw + slot;
                    const bool got = tw_poll(P, pub.tag, (1u << (2 * (jb.ks - 1))) - 1u, [&](int k) { return base + (k >> 1) * 64 + (k & 1); }, pw);   // all lanes, always
                    ok = __all_sync(0xffffffffu, (ok && got) ? 1 : 0) != 0;
                    if (ok) {
                        #pragma unroll
                        for (int q = 0; q < kMaxKSplit - 1; q++)
                            if (q < jb.ks - 1) v0 = __dadd_rn(v0, __longlong_as_double((long long)(((unsigned long long)pw[2 * q + 1] << 32) | pw[2 * q])));
                        epi(gg, lane, __double2float_rn(v0), 0.f);
                    }
                }
            } else {
                epi(gg, lane, __double2float_rn(v0), __double2float_rn(v1));
            }
        }
        prof_mark(P, 19);
    }
    return ok;
}

// lm_head: a unit (row group) belongs to one warp; epi(g, lane, v).
template <class Epi>
__device__ MI_PIECE bool run_warp_job(WarpStream& ws, int j, int lane, const int8_t* xq_s, const float2* xs_s, Epi epi) {
    const Job jb = ws.jobs[j];
    bool ok = true;
    for (int u = ws.first_warp_unit(jb); u < jb.n_units && ok; u += ws.W) {
        double acc = 0.0;
        for (int t = 0; t < jb.nt; t++) acc = tile_consume(ws, lane, jb.kb, t, xq_s, xs_s, acc, ok);
        if (ok) epi(u + jb.g_off, lane, __double2float_rn(acc));
    }
    return ok;
}

// ---- activation staging (whole CTA; returns a CTA-uniform ok) -----------------------

// Warp-wide maximum of non-negative floats and warp-wide integer sum as single redux
// instructions (the bit pattern of a non-negative float orders like an unsigned integer);
// a shuffle tree costs five issue slots of a pipe that retires one warp instruction per clock.
__device__ __forceinline__ float warp_max_nonneg(float a) { return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(a))); }
__device__ __forceinline__ int warp_sum_int(int v) { return __reduce_add_sync(0xffffffffu, v); }
// warp-wide maximum of arbitrary finite floats (or -inf): order-preserving key
__device__ __forceinline__ float warp_max_float(float a) {
    const unsigned b = __float_as_uint(a), key = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    const unsigned m = __reduce_max_sync(0xffffffffu, key);
    return __uint_as_float((m & 0x80000000u) ? (m & 0x7fffffffu) : ~m);
}

// q8_0 of one 32-element block held one element per lane; returns the int8 value,
// writes the fp16 scale through lane 0 (plain stores: the attention kernel of the M-token step).
__device__ __forceinline__ int quant_block_warp(float v, int lane, float2* xs_out, __half* xd_out) {
    const float a = warp_max_nonneg(fabsf(v));
    const float inv = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
    const int q = __float2int_rn(__fmul_rn(v, inv));
    const int s = warp_sum_int(q);
    if (lane == 0) {
        const __half d = __float2half_rn(__fdiv_rn(a, 127.f));
        if (xs_out) *xs_out = make_float2(__half2float(d), __int2float_rn(8 * s));
        if (xd_out) *xd_out = d;
    }
    return q;
}

// Residual add + RMSNorm + q8_0 staging:
//   x = h (this CTA's copy of the residual stream in shared memory; or gsrc, the copy the first GEMV CTA committed to
//       global memory, when the launch starts here; or the embedding row of `token`)
//       + the projection output published as tagged fp32 words at addw   [if addw]
//   h = x;  the first GEMV CTA also commits x to global memory;
//   xq_s / xs_s = q8_0( x * (1/sqrt(float(ss/n) + eps)) * w )   (src/cpu_infer.cpp:40-46).
// Two thread mappings.  Gathering (tagged words in, residual add, sum of squares): warp w owns the 32-element blocks
// w, w+8, ...; lane = element, so every warp-wide load of tagged words is one contiguous 256-byte run and all of a
// thread's words are requested before anything waits on them.  Quantizing (after the sum of squares is known): EPL
// consecutive elements per thread, 32/EPL threads per q8_0 block, read back from shared memory; the block maximum and the
// block sum fold over 32/EPL lanes with log2(32/EPL) shuffles.  (One element per thread and warp-wide REDUX reductions,
// twelve per warp at the 1.5B shape, measured 1500 cycles for the quantizer alone: the reduction unit, not the
// arithmetic, set the time.)  Sum of squares in double (every x*x is exact there).
// h_s must hold the residual stream already (residual_init below puts the embedding row, or the copy committed to global
// memory, there with this same thread mapping, so no barrier is needed in between).
template <int NB, int EPL>
__device__ __forceinline__ bool stage_norm_q8_t(const DecodeParams& P, float* h_s,
                                                const unsigned long long* addw, unsigned tag, float* commit, const float* __restrict__ w,
                                                int E, float eps, double* red, int8_t* xq_s, float2* xs_s) {
    constexpr int LPB = 32 / EPL;                        // lanes per block while quantizing
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nb = E / 32;
    // the norm weights of the quantizing pass: requested now, used after the barrier
    const int qt_b = tid / LPB, qt_e0 = tid * EPL;
    const bool qlive = qt_b < nb;
    float wv[EPL];
    #pragma unroll
    for (int i = 0; i < EPL; i++) wv[i] = __ldg(w + (qlive ? qt_e0 : 0) + i);
    float x[NB];
    unsigned valid = 0;
    #pragma unroll
    for (int k = 0; k < NB; k++) {
        const int b = min(warp + k * DNW, nb - 1), e = b * 32 + lane;      // clamped: every address is valid
        if (warp + k * DNW < nb) valid |= 1u << k;
        x[k] = h_s[e];
    }
    bool ok = true;
    if (addw) {
        unsigned aw[NB];
        prof_mark(P, 27);
        ok = tw_poll(P, tag, valid, [&](int k) { return addw + (size_t)(warp + k * DNW) * 32 + lane; }, aw);
        prof_mark(P, kProfWait);
        #pragma unroll
        for (int k = 0; k < NB; k++) if (valid >> k & 1u) x[k] = __fadd_rn(x[k], __uint_as_float(aw[k]));
        prof_mark(P, 28);
    }
    double ss = 0.0;
    #pragma unroll
    for (int k = 0; k < NB; k++) {
        if (valid >> k & 1u) {
            const int e = (warp + k * DNW) * 32 + lane;
            h_s[e] = x[k];
            if (commit && (int)blockIdx.x == P.attn_ctas) __stcg(commit + e, x[k]);
            const double xd = x[k]; ss = __fma_rn(xd, xd, ss);
        }
    }
    #pragma unroll
    for (int o = 16; o; o >>= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    if (lane == 0) red[warp] = ss;
    prof_mark(P, 23);
    if (!__syncthreads_and(ok ? 1 : 0)) return false;
    prof_mark(P, 24);
    double tot = 0.0;
    #pragma unroll
    for (int v = 0; v < DNW; v++) tot = __dadd_rn(tot, red[v]);
    const float mean = __double2float_rn(__ddiv_rn(tot, (double)E));
    const float scale = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(mean, eps)));
    // quantize: this thread's EPL elements of block qt_b (vectors beyond 256 * EPL elements: further rounds)
    for (int t = tid; (t & ~31) / LPB < nb; t += DNT) {              // warp-uniform trip count: the folds below are warp-wide
        const int b = t / LPB;
        const bool live = b < nb;
        const int e0 = live ? t * EPL : 0;                            // a lane past the vector computes on block 0 and stores nothing
        float v[EPL], a = 0.f;
        #pragma unroll
        for (int i = 0; i < EPL; i++) {
            const float wi = t == tid ? wv[i] : __ldg(w + e0 + i);
            v[i] = __fmul_rn(__fmul_rn(h_s[e0 + i], scale), wi); a = fmaxf(a, fabsf(v[i]));
        }
        #pragma unroll
        for (int o = 1; o < LPB; o <<= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        const float inv = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
        int q[EPL], sq = 0;
        #pragma unroll
        for (int i = 0; i < EPL; i++) { q[i] = __float2int_rn(__fmul_rn(v[i], inv)); sq += q[i]; }
        #pragma unroll
        for (int o = 1; o < LPB; o <<= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (live) {
            if constexpr (EPL >= 4) {
                #pragma unroll
                for (int i = 0; i < EPL; i += 4)
                    *reinterpret_cast<unsigned*>(xq_s + e0 + i) = (unsigned)(q[i] & 0xff) | ((unsigned)(q[i + 1] & 0xff) << 8) |
                                                                  ((unsigned)(q[i + 2] & 0xff) << 16) | ((unsigned)(q[i + 3] & 0xff) << 24);
            } else {
                #pragma unroll
                for (int i = 0; i < EPL; i++) xq_s[e0 + i] = (int8_t)q[i];
            }
            if ((t % LPB) == 0) xs_s[b] = make_float2(__half2float(__float2half_rn(__fdiv_rn(a, 127.f))), __int2float_rn(8 * sq));
        }
    }
    prof_mark(P, 25);
    __syncthreads();
    prof_mark(P, 26);
    return true;
}

// The residual stream into this CTA's shared memory, where a step or a launch begins: the embedding row of `token`
// (value (nibble - 8) * d, src/gguf.h:94-102; or a Q8_0 row as stored, int8 * d, src/gguf.h:112-118 and src/mega.cu:639-642),
// or the copy the first GEMV CTA committed to global memory (a launch that starts in mid-step).  Thread mapping of the norm
// prologue's gathering pass: each thread later reads only what it wrote here.
__device__ __forceinline__ void residual_init(const DecodeParams& P, float* h_s, const float* gsrc, int token, int E) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nb = E / 32;
    for (int b = warp; b < nb; b += DNW) {
        const int e = b * 32 + lane;
        float x;
        if (gsrc) x = __ldcg(gsrc + e);
        else if (P.emb_q8) {
            const uint8_t* bp = P.emb_q8 + ((size_t)token * nb + b) * 34;
            x = __fmul_rn(__int2float_rn((int)(int8_t)__ldg(bp + 2 + lane)), __half2float(__ldg(reinterpret_cast<const __half*>(bp))));
        } else {
            const int g = token >> 5, r = token & 31, kb = P.emb_kb, t = b / kb, kk = b % kb;
            const uint8_t* tile = P.emb_base + ((size_t)g * P.emb_nt + t) * (kb * kTileRowBytes);
            const uint8_t byte = __ldg(tile + ((size_t)kk * 32 + r) * 16 + (lane & 15));
            const float d = __half2float(__ldg(reinterpret_cast<const __half*>(tile + (size_t)kb * 512 + ((size_t)r * kb + kk) * 2)));
            x = __fmul_rn(__int2float_rn((lane < 16 ? (byte & 0x0F) : (byte >> 4)) - 8), d);
        }
        h_s[e] = x;
    }
}

#define MI_NORM_ARGS const DecodeParams& P, float* h_s, const unsigned long long* addw, unsigned tag, \
                     float* commit, const float* __restrict__ w, int E, float eps, double* red, int8_t* xq_s, float2* xs_s
#define MI_NORM_PASS P, h_s, addw, tag, commit, w, E, eps, red, xq_s, xs_s
// blocks per warp while gathering (NB) and elements per thread while quantizing (EPL: the largest of 8, 4, 2, 1 with
// which 256 threads cover the vector, 8 in several rounds beyond 2048 elements)
static __device__ __noinline__ bool stage_norm_q8_rare(MI_NORM_ARGS) {
    if (E <= 256) return stage_norm_q8_t<1, 1>(MI_NORM_PASS);
    if (E <= 512) return stage_norm_q8_t<2, 2>(MI_NORM_PASS);
    if (E <= 1024) return stage_norm_q8_t<4, 4>(MI_NORM_PASS);
    if (E <= 4096) return stage_norm_q8_t<16, 8>(MI_NORM_PASS);
    return stage_norm_q8_t<32, 8>(MI_NORM_PASS);
}
__device__ __forceinline__ bool stage_norm_q8u(MI_NORM_ARGS) {
#if MI_LEAN
    return stage_norm_q8_t<8, 8>(MI_NORM_PASS);                                         // lean_shape_ok(): 1024 < E <= 2048
#else
    if (E > 1024 && E <= 2048) return stage_norm_q8_t<8, 8>(MI_NORM_PASS);
    return stage_norm_q8_rare(MI_NORM_PASS);
#endif
}

// A q8_0 vector published as tagged words by other CTAs -> shared memory: int8 values, and per block {fp32 of the fp16
// scale, float(8 * sum of the block's values)}.  Thread t takes the 16-byte word pairs t, t + 256, ...; all of a
// thread's loads are in flight together.
template <int NP>
__device__ MI_PIECE bool stage_poll_q8_t(const DecodeParams& P, const unsigned long long* vw, int n, unsigned tag, int8_t* xq_s, float2* xs_s) {
    const int tid = threadIdx.x, nq2 = n / 8, tot2 = nq2 + (n / 32 + 1) / 2, nbk = n / 32;     // pairs of value words, all pairs, blocks
    unsigned long long w[NP][2];
    #pragma unroll
    for (int k = 0; k < NP; k++) {
        const int pr = tid + k * DNT;
        if (pr < tot2) tw_ld2(vw + 2 * pr, w[k][0], w[k][1]);
        else w[k][0] = w[k][1] = (unsigned long long)tag << 32;
        if (pr == tot2 - 1 && (nbk & 1)) w[k][1] = (unsigned long long)tag << 32;      // odd block count: the pad word is never written
    }
    bool ok = true;
    for (;;) {
        const unsigned long long* miss = nullptr;
        #pragma unroll
        for (int k = NP - 1; k >= 0; k--) {
            if (!tw_is(w[k][1], tag)) miss = vw + 2 * (tid + k * DNT) + 1;
            if (!tw_is(w[k][0], tag)) miss = vw + 2 * (tid + k * DNT);
        }
        const int st = tw_wait_warp(miss, tag, P.wait_ns, P.err);
        if (st == 0) break;
        if (st < 0) { ok = false; break; }
        #pragma unroll
        for (int k = 0; k < NP; k++) {
            if (!tw_is(w[k][0], tag) || !tw_is(w[k][1], tag)) {
                const int pr = tid + k * DNT;
                tw_ld2(vw + 2 * pr, w[k][0], w[k][1]);
                if (pr == tot2 - 1 && (nbk & 1)) w[k][1] = (unsigned long long)tag << 32;
            }
        }
    }
    #pragma unroll
    for (int k = 0; k < NP; k++) {
        const int pr = tid + k * DNT;
        if (pr < nq2) {
            reinterpret_cast<uint2*>(xq_s)[pr] = make_uint2((unsigned)w[k][0], (unsigned)w[k][1]);
        } else if (pr < tot2) {
            #pragma unroll
            for (int h = 0; h < 2; h++) {
                const int b = 2 * (pr - nq2) + h;
                if (b < nbk) {
                    const unsigned sw = (unsigned)w[k][h];
                    xs_s[b] = make_float2(__half2float(__ushort_as_half((unsigned short)(sw & 0xffffu))), __int2float_rn(8 * (int)(short)(sw >> 16)));
                }
            }
        }
    }
    return __syncthreads_and(ok ? 1 : 0) != 0;
}
static __device__ __noinline__ bool stage_poll_q8_rare(const DecodeParams& P, const unsigned long long* vw, int n, unsigned tag, int8_t* xq_s, float2* xs_s) {
    const int np = (q8_words(n) / 2 + DNT - 1) / DNT;
    if (np <= 8) return stage_poll_q8_t<8>(P, vw, n, tag, xq_s, xs_s);
    return stage_poll_q8_t<18>(P, vw, n, tag, xq_s, xs_s);
}
__device__ __forceinline__ bool stage_poll_q8(const DecodeParams& P, const unsigned long long* vw, int n, unsigned tag, int8_t* xq_s, float2* xs_s) {
    const int np = (q8_words(n) / 2 + DNT - 1) / DNT;
    if (np <= 1) return stage_poll_q8_t<1>(P, vw, n, tag, xq_s, xs_s);
    if (np <= 5) return stage_poll_q8_t<5>(P, vw, n, tag, xq_s, xs_s);
#if MI_LEAN
    return stage_poll_q8_t<8>(P, vw, n, tag, xq_s, xs_s);                               // lean_shape_ok(): at most 8 word pairs per thread
#else
    return stage_poll_q8_rare(P, vw, n, tag, xq_s, xs_s);
#endif
}

// Shapes the short-context build takes: it holds one variant of each prologue and of the tile loop and no call to the others.
inline bool lean_shape_ok(int E, int FF, int NQ) {
    auto kb8 = [](int n) { return (n / 32) % 8 == 0; };
    auto np = [](int n) { return (q8_words(n) / 2 + DNT - 1) / DNT; };
    return E > 1024 && E <= 2048 && kb8(E) && kb8(FF) && kb8(NQ) && np(FF) <= 8 && np(NQ) <= 8;
}

// ---- attention --------------------------------------------------------------------
// CTA = (kv head, chunk of the causal range); its warps split the chunk.  A warp
// walks its positions 32 at a time in two passes.  Pass 1, lane = position: the
// full q.k dot of the lane's K row against all G query heads of the kv head (q
// waits in shared memory as doubles, read as broadcasts: no cross-lane reduction,
// and one K read serves the whole GQA group).  Pass 2, lane = dims {lane + 32 i}:
// the 32 positions' softmax weights (parked in shared memory) times their V rows.
// Running state per head: max m (an fp32 score), denominator l and output o[] in
// double.  States fold warps -> chunk (shared memory) -> head (global scratch, by
// the last CTA of the kv head to arrive), each fold against the common maximum so
// that the rescale factors are independent of one another; then o/l is rounded to
// fp32, stored, and quantized to q8_0 for the O projection.
// G = query heads handled by one CTA: all heads of a kv head (one K/V read serves the group: long
// contexts, bandwidth matters) or a single head (short contexts: K/V come from L2 anyway, and six
// times as many CTAs each carry a sixth of the serial work).  GQ = query heads per kv head.
// STORE_KV: the CTA whose range ends at the new position writes that position's K and V from the packed QKV
// vector (the decode loop); callers that stored them beforehand pass false.  QNAT: q is in natural dimension
// order (the stand-alone entry point) instead of the packed pair-adjacent order of the fused QKV projection.
// TG: inputs (q, and k / v of the new position) and the q8_0 output travel as tagged words (the decode loop); otherwise they
// are plain arrays (the attention kernel of the M-token step).  Returns false if a wait gave up (CTA-uniform).
template <int HD, int G, int GQ, bool STORE_KV = true, bool QNAT = false, bool TG = false>
__device__ __forceinline__ bool attention_phase(const DecodeParams& P, int l, int pos, uint8_t* stage,
                                                unsigned tag_in = 0, const Pub pub = Pub()) {
    constexpr int DPW = HD / 32;           // dims per lane in pass 2 and while folding (dim = lane + 32*i)
    constexpr int SW = HD + 2;             // doubles per (head) state: o[HD], m, l
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ngrp = P.NH / G;
    // one head per CTA: 256 positions are one 32-position batch per warp, and a single chunk needs no cross-CTA merge
    const int Lp = pos + 1, nch = attn_chunks(Lp, min(P.max_chunks, (int)gridDim.x / ngrp), G == 1 ? 256 : kAttnChunk);
    if ((int)blockIdx.x >= ngrp * nch) return true;
    const int grp = blockIdx.x / nch, ch = blockIdx.x % nch, h0 = grp * G, kvh = h0 / GQ;
    const int p0 = (int)((long long)ch * Lp / nch), p1 = (int)((long long)(ch + 1) * Lp / nch);
    double* scr = reinterpret_cast<double*>(stage);                        // [warp][G][SW]
    double* wts = scr + DNW * G * SW;                                       // [warp][32][G]
    constexpr int LPP = 8, DPL = HD / LPP, QSTR = DPL + 2;                   // lanes per position in pass 1, dims per lane, padded stride
    double* qs = wts + DNW * 32 * G;                                        // [G][LPP][QSTR]: 16-byte skew per lane, conflict-free
    const bool store_kv = STORE_KV && ch == nch - 1;     // this CTA's range ends at the new position: it stores that position's K and V (fp16); CTAs that share a kv head store the same bits
    if constexpr (TG) {
        // q of this CTA's G query heads, and k / v of the new position, from the tagged QKV vector (packed order: dim d of a
        // head sits at 2d (d < HD/2) or 2(d-HD/2)+1); one poll for all of a thread's words
        constexpr int QN = (G * HD + DNT - 1) / DNT;
        const int nq = P.NH * HD;
        unsigned qw[QN + 2], valid = 0;
        #pragma unroll
        for (int k = 0; k < QN; k++) if (tid + k * DNT < G * HD) valid |= 1u << k;
        if (store_kv && tid < HD) valid |= 3u << QN;
        const unsigned long long* qv = P.xw + P.xo.qkv;
        const int dk = tid < HD / 2 ? 2 * tid : 2 * (tid - HD / 2) + 1;           // packed slot of dim `tid` (threads below HD)
        bool okq = tw_poll(P, tag_in, valid, [&](int k) -> const unsigned long long* {
            if (k < QN) {
                const int i = tid + k * DNT, j = i / HD, d = i % HD, pk = d < HD / 2 ? 2 * d : 2 * (d - HD / 2) + 1;
                return qv + (size_t)(h0 + j) * HD + pk;
            }
            return k == QN ? qv + nq + (size_t)kvh * HD + dk : qv + nq + P.KVD + (size_t)kvh * HD + tid;
        }, qw);
        #pragma unroll
        for (int k = 0; k < QN; k++) {
            const int i = tid + k * DNT;
            if (i < G * HD) { const int j = i / HD, d = i % HD; qs[(j * LPP + d / DPL) * QSTR + d % DPL] = (double)__uint_as_float(qw[k]); }
        }
        if (store_kv && tid < HD) {
            P.kc[((size_t)l * P.max_seq + pos) * P.KVD + (size_t)kvh * HD + tid] = __float2half_rn(__uint_as_float(qw[QN]));
            P.vc[((size_t)l * P.max_seq + pos) * P.KVD + (size_t)kvh * HD + tid] = __float2half_rn(__uint_as_float(qw[QN + 1]));
        }
        if (!__syncthreads_and(okq ? 1 : 0)) return false;
    } else {
        for (int i = tid; i < G * HD; i += DNT) {
            const int j = i / HD, d = i % HD, pk = QNAT ? d : (d < HD / 2 ? 2 * d : 2 * (d - HD / 2) + 1);
            qs[(j * LPP + d / DPL) * QSTR + d % DPL] = (double)__ldcg(P.qkv_out + (size_t)(h0 + j) * HD + pk);
        }
        if (store_kv) {
            const int nq = P.NH * HD;
            for (int d = tid; d < HD; d += DNT) {
                const int pk = d < HD / 2 ? 2 * d : 2 * (d - HD / 2) + 1;
                P.kc[((size_t)l * P.max_seq + pos) * P.KVD + (size_t)kvh * HD + d] = __float2half_rn(__ldcg(P.qkv_out + nq + (size_t)kvh * HD + pk));
                P.vc[((size_t)l * P.max_seq + pos) * P.KVD + (size_t)kvh * HD + d] = __float2half_rn(__ldcg(P.qkv_out + nq + P.KVD + (size_t)kvh * HD + d));
            }
        }
        __syncthreads();
    }
    prof_mark(P, 14);
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
        const int np = min(32, a1 - b0);
        // pass 1: eight lanes share a position (DPL dims each), four positions per sweep; the
        // scores of the batch are parked in the weights buffer, one row per position.  All K rows
        // of the batch are requested before the first one is used.
        {
            const int sub = lane >> 3, li = lane & 7;
            constexpr int KV4 = DPL * 2 / 16 > 0 ? DPL * 2 / 16 : 1;        // 16-byte loads per lane and position
            // two rounds of four sweeps (16 positions): half the unrolled code of one round of eight; a round's K rows
            // are all requested before the first one is used
            #pragma unroll 1
            for (int s0 = 0; s0 < 8 && s0 * 4 < np; s0 += 4) {
                uint4 kraw[4][KV4];
                #pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int sw = s0 + u;
                    if (sw * 4 >= np) continue;                              // warp-uniform
                    const int pi = min(sw * 4 + sub, np - 1);
                    const __half* kr = kbase + (size_t)(b0 + pi) * P.KVD + li * DPL;
                    if constexpr (DPL >= 8) {
                        #pragma unroll
                        for (int c = 0; c < KV4; c++) kraw[u][c] = __ldcg(reinterpret_cast<const uint4*>(kr) + c);
                    } else {
                        const uint2 k2 = __ldcg(reinterpret_cast<const uint2*>(kr));
                        kraw[u][0] = make_uint4(k2.x, k2.y, 0u, 0u);
                    }
                }
                #pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int sw = s0 + u;
                    if (sw * 4 < np) {                                       // warp-uniform
                        const int pi = sw * 4 + sub;
                        double kd[DPL];
                        #pragma unroll
                        for (int c = 0; c < KV4; c++) {
                            const __half2* hh = reinterpret_cast<const __half2*>(&kraw[u][c]);
                            #pragma unroll
                            for (int e = 0; e < 4; e++) {
                                if (c * 8 + 2 * e < DPL) {
                                    const float2 f = __half22float2(hh[e]);
                                    kd[c * 8 + 2 * e] = (double)f.x; kd[c * 8 + 2 * e + 1] = (double)f.y;
                                }
                            }
                        }
                        double d[G];
                        #pragma unroll
                        for (int j = 0; j < G; j++) {
                            const double* qj = qs + (j * LPP + li) * QSTR;
                            double acc = 0.0;
                            #pragma unroll
                            for (int e = 0; e < DPL; e += 2) {
                                const double2 qq = *reinterpret_cast<const double2*>(qj + e);
                                acc = __fma_rn(qq.x, kd[e], acc);
                                acc = __fma_rn(qq.y, kd[e + 1], acc);
                            }
                            d[j] = acc;
                        }
                        #pragma unroll
                        for (int sft = 1; sft <= 4; sft <<= 1)
                            #pragma unroll
                            for (int j = 0; j < G; j++) d[j] = __dadd_rn(d[j], __shfl_xor_sync(0xffffffffu, d[j], sft));
                        if (li == 0 && pi < np) {
                            #pragma unroll
                            for (int j = 0; j < G; j++) wl[pi * G + j] = (double)__fmul_rn(__double2float_rn(d[j]), inv);
                        }
                    }
                }
            }
        }
        __syncwarp();
        const bool valid = lane < np;
        float sc[G];
        #pragma unroll
        for (int j = 0; j < G; j++) sc[j] = valid ? (float)wl[lane * G + j] : -INFINITY;
        __syncwarp();
        // new running max, rescale, this batch's weights
        #pragma unroll
        for (int j = 0; j < G; j++) {
            const float bm = warp_max_float(sc[j]);
            const float mn = fmaxf(m[j], bm);                                // finite: the batch holds a valid position
            // the running maximum is warp-uniform; while it stands the rescale factor is exp(0) = 1 exactly
            const double cr = mn == m[j] ? 1.0 : (m[j] == -INFINITY ? 0.0 : exp_shared((double)m[j] - (double)mn));
            const double w = valid ? exp_shared((double)sc[j] - (double)mn) : 0.0;
            wl[lane * G + j] = w;                                            // the denominator picks the weights up in pass 2
            ls[j] = __dmul_rn(ls[j], cr);
            #pragma unroll
            for (int i = 0; i < DPW; i++) o[j][i] = __dmul_rn(o[j][i], cr);
            m[j] = mn;
        }
        __syncwarp();
        // pass 2: o += w[p] * V[p]
        constexpr int VB = G == 1 ? 16 : 8;                                  // V rows requested together (one head per CTA: registers to spare)
        for (int pp0 = 0; pp0 < np; pp0 += VB) {
            unsigned short vh[VB][DPW];
            #pragma unroll
            for (int u = 0; u < VB; u++) {
                if (u >= 8 && pp0 + u >= np) continue;                       // warp-uniform: the second half of a round may be empty
                const unsigned short* vp = reinterpret_cast<const unsigned short*>(vbase + (size_t)(b0 + min(pp0 + u, np - 1)) * P.KVD);
                #pragma unroll
                for (int i = 0; i < DPW; i++) vh[u][i] = __ldcg(vp + lane + 32 * i);
            }
            #pragma unroll
            for (int u = 0; u < VB; u++) {
                if (pp0 + u < np) {
                    double vd[DPW];
                    #pragma unroll
                    for (int i = 0; i < DPW; i++) vd[i] = (double)__half2float(__ushort_as_half(vh[u][i]));
                    #pragma unroll
                    for (int j = 0; j < G; j++) {
                        const double w = wl[(pp0 + u) * G + j];
                        ls[j] = __dadd_rn(ls[j], w);
                        #pragma unroll
                        for (int i = 0; i < DPW; i++) o[j][i] = __fma_rn(w, vd[i], o[j][i]);
                    }
                }
            }
        }
        __syncwarp();
    }
    prof_mark(P, 15);
    #pragma unroll
    for (int j = 0; j < G; j++) {
        double* sw = scr + (size_t)(warp * G + j) * SW;
        #pragma unroll
        for (int i = 0; i < DPW; i++) sw[lane + 32 * i] = o[j][i];
        if (lane == 0) { sw[HD] = (double)m[j]; sw[HD + 1] = ls[j]; }
    }
    // the new position's K / V rows (plain stores above) are performed before anything this CTA publishes from here on:
    // a CTA that reads them in a later step has consumed words that descend from this CTA's output
    if (TG && store_kv && tid < HD) __threadfence();
    __syncthreads();
    // warp j folds head j's DNW warp states against their common maximum and publishes the chunk partial
    if (warp < G) {
        const int j = warp, head = h0 + j;
        // lane w takes warp w's maximum: one exponential for all eight rescale factors, then broadcast
        const float mw_l = lane < DNW ? (float)scr[(size_t)(lane * G + j) * SW + HD] : -INFINITY;
        const float mm = warp_max_float(mw_l);
        const double f_l = mw_l == -INFINITY ? 0.0 : exp_shared((double)mw_l - (double)mm);
        double f[DNW];
        #pragma unroll
        for (int w = 0; w < DNW; w++) f[w] = __shfl_sync(0xffffffffu, f_l, w);
        double ob[DPW], ll = 0.0;
        #pragma unroll
        for (int i = 0; i < DPW; i++) ob[i] = 0.0;
        #pragma unroll
        for (int w = 0; w < DNW; w++) {
            const double* s2 = scr + (size_t)(w * G + j) * SW;
            ll = __fma_rn(s2[HD + 1], f[w], ll);
            #pragma unroll
            for (int i = 0; i < DPW; i++) ob[i] = __fma_rn(s2[lane + 32 * i], f[w], ob[i]);
        }
        if (nch == 1) {                                                     // the chunk is the whole range: finish here
            #pragma unroll
            for (int i = 0; i < DPW; i++) {
                const float v = __double2float_rn(__ddiv_rn(ob[i], ll));
                const int e = head * HD + 32 * i + lane;
                __stcg(P.att + e, v);
                if constexpr (TG) {
                    __half dq; int sq;
                    const int qv8 = quant_block_warp2(v, dq, sq);
                    publish_q8_block<false>(pub, P.xo.att, P.xo.att + P.NH * HD / 4, e >> 5, lane, qv8, dq, sq);
                } else {
                    P.att_q[e] = (int8_t)quant_block_warp(v, lane, nullptr, P.att_d + (e >> 5));
                }
            }
        } else {
            double* gp = P.attn_part + ((size_t)head * P.max_chunks + ch) * SW;
            #pragma unroll
            for (int i = 0; i < DPW; i++) __stcg(gp + lane + 32 * i, ob[i]);
            if (lane == 0) { __stcg(gp + HD, (double)mm); __stcg(gp + HD + 1, ll); }
        }
    }
    prof_mark(P, 16);
    if (nch == 1) return true;
    __threadfence();
    __syncthreads();
    __shared__ unsigned s_prev;
    if (tid == 0) s_prev = atomicAdd(P.attn_cnt + grp, 1u);
    __syncthreads();
    if (s_prev != (unsigned)nch - 1) return true;
    // last chunk of this kv head: fold the chunk partials against their common maximum, normalise, emit fp32 + q8_0
    __threadfence();
    if (tid == 0) P.attn_cnt[grp] = 0;
    if (warp < G) {
        const int j = warp, head = h0 + j;
        const double* gp = P.attn_part + (size_t)head * P.max_chunks * SW;
        // rescale factors of all chunks first (lane = chunk, so the exponentials run side by side), parked in the
        // warp-state buffer, which nobody reads any more; then the fold in chunk order, eight chunks' loads in flight
        double* fs = scr + (size_t)j * DNW * SW;                            // nch <= grid size / kv heads <= DNW * SW
        float mm = -INFINITY;
        for (int c = lane; c < nch; c += 32) {
            const float mc = (float)__ldcg(gp + (size_t)c * SW + HD);
            fs[c] = (double)mc; mm = fmaxf(mm, mc);
        }
        #pragma unroll
        for (int sft = 16; sft; sft >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, sft));
        for (int c = lane; c < nch; c += 32) {
            const float mc = (float)fs[c];
            fs[c] = mc == -INFINITY ? 0.0 : exp_shared((double)mc - (double)mm);
        }
        __syncwarp();
        double ob[DPW], ll = 0.0;
        #pragma unroll
        for (int i = 0; i < DPW; i++) ob[i] = 0.0;
        for (int c0 = 0; c0 < nch; c0 += 8) {
            double lv[8], ov[8][DPW];
            #pragma unroll
            for (int u = 0; u < 8; u++) {
                const double* g2 = gp + (size_t)min(c0 + u, nch - 1) * SW;
                lv[u] = __ldcg(g2 + HD + 1);
                #pragma unroll
                for (int i = 0; i < DPW; i++) ov[u][i] = __ldcg(g2 + lane + 32 * i);
            }
            #pragma unroll
            for (int u = 0; u < 8; u++) {
                if (c0 + u < nch) {
                    const double f = fs[c0 + u];
                    ll = __fma_rn(lv[u], f, ll);
                    #pragma unroll
                    for (int i = 0; i < DPW; i++) ob[i] = __fma_rn(ov[u][i], f, ob[i]);
                }
            }
        }
        #pragma unroll
        for (int i = 0; i < DPW; i++) {
            const float v = __double2float_rn(__ddiv_rn(ob[i], ll));
            const int e = head * HD + 32 * i + lane;
            __stcg(P.att + e, v);
            if constexpr (TG) {
                __half dq; int sq;
                const int qv8 = quant_block_warp2(v, dq, sq);
                publish_q8_block<false>(pub, P.xo.att, P.xo.att + P.NH * HD / 4, e >> 5, lane, qv8, dq, sq);
            } else {
                P.att_q[e] = (int8_t)quant_block_warp(v, lane, nullptr, P.att_d + (e >> 5));
            }
        }
    }
    return true;
}

// ---- attention over a short causal range (at most 256 positions): one CTA per query head ---------------
// The whole range of a head fits one CTA, so the softmax is computed the way the reference's CPU program writes it
// (src/cpu_infer.cpp:121-140): all scores, their maximum, exp(score - max) once per position, then the weighted sum of the
// V rows and the division - no running maximum, no rescaling, no merge of partial states.
//   pass 1  warp w takes a contiguous eighth of the positions; eight lanes share a position (HD/8 dims each), the dot
//           product is carried in double and folded over the eight lanes; score = fp32(dot) * 1/sqrt(HD) in fp32;
//   max     every warp scans the scores in shared memory; thread t computes the weight of position t (one double exp);
//   pass 2  warp w, same positions: lane = dims {lane + 32 i}; o += w[p] * V[p], l += w[p] in position order;
//   finish  warp i (i < HD/32) adds the eight warps' partial sums in warp order, divides, rounds to fp32, quantizes its
//           32-dim block to q8_0 and publishes it.
// Same interface and template flags as attention_phase.
template <int HD, int GQ, bool STORE_KV = true, bool QNAT = false, bool TG = false>
MI_ATT_FN bool attention_short(const DecodeParams& P, int l, int pos, uint8_t* stage,
                                                unsigned tag_in = 0, const Pub pub = Pub()) {
    constexpr int DPW = HD / 32;
    constexpr int LPP = 8, DPL = HD / LPP, QSTR = DPL + 2;                 // lanes per position in pass 1, dims per lane, padded stride
    constexpr int KV4 = DPL * 2 / 16 > 0 ? DPL * 2 / 16 : 1;              // 16-byte loads per lane and position
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if ((int)blockIdx.x >= P.NH) return true;
    const int head = blockIdx.x, kvh = head / GQ, Lp = pos + 1;
    double* qs = reinterpret_cast<double*>(stage);                         // [LPP][QSTR]
    double* wt = qs + LPP * QSTR;                                          // [256] weights
    double* ow = wt + 256;                                                 // [DNW][HD] partial outputs
    double* lw = ow + DNW * HD;                                            // [DNW] partial denominators
    float* sc = reinterpret_cast<float*>(lw + DNW);                        // [256] scores
    if constexpr (TG) {
        const int nq = P.NH * HD;
        unsigned qw[3], valid = 0;
        if (tid < HD) valid = STORE_KV ? 7u : 1u;
        const unsigned long long* qv = P.xw + P.xo.qkv;
        const int dk = tid < HD / 2 ? 2 * tid : 2 * (tid - HD / 2) + 1;    // packed slot of dim `tid`
        const bool okq = tw_poll(P, tag_in, valid, [&](int k) -> const unsigned long long* {
            return k == 0 ? qv + (size_t)head * HD + dk : k == 1 ? qv + nq + (size_t)kvh * HD + dk : qv + nq + P.KVD + (size_t)kvh * HD + tid;
        }, qw);
        if (tid < HD) {
            qs[(tid / DPL) * QSTR + tid % DPL] = (double)__uint_as_float(qw[0]);
            if (STORE_KV) {                                               // CTAs that share a kv head store the same bits
                P.kc[((size_t)l * P.max_seq + pos) * P.KVD + (size_t)kvh * HD + tid] = __float2half_rn(__uint_as_float(qw[1]));
                P.vc[((size_t)l * P.max_seq + pos) * P.KVD + (size_t)kvh * HD + tid] = __float2half_rn(__uint_as_float(qw[2]));
            }
        }
        if (!__syncthreads_and(okq ? 1 : 0)) return false;
    } else {
        if (tid < HD) {
            const int pk = QNAT ? tid : (tid < HD / 2 ? 2 * tid : 2 * (tid - HD / 2) + 1);
            qs[(tid / DPL) * QSTR + tid % DPL] = (double)__ldcg(P.qkv_out + (size_t)head * HD + pk);
            if (STORE_KV) {
                const int nq = P.NH * HD, pkk = tid < HD / 2 ? 2 * tid : 2 * (tid - HD / 2) + 1;
                P.kc[((size_t)l * P.max_seq + pos) * P.KVD + (size_t)kvh * HD + tid] = __float2half_rn(__ldcg(P.qkv_out + nq + (size_t)kvh * HD + pkk));
                P.vc[((size_t)l * P.max_seq + pos) * P.KVD + (size_t)kvh * HD + tid] = __float2half_rn(__ldcg(P.qkv_out + nq + P.KVD + (size_t)kvh * HD + tid));
            }
        }
        __syncthreads();
    }
    prof_mark(P, 14);
    const float inv = __fdiv_rn(1.f, __fsqrt_rn((float)HD));
    const int a0 = (int)((long long)Lp * warp / DNW), a1 = (int)((long long)Lp * (warp + 1) / DNW);      // at most 32 positions
    const __half* kbase = P.kc + ((size_t)l * P.max_seq) * P.KVD + (size_t)kvh * HD;
    const __half* vbase = P.vc + ((size_t)l * P.max_seq) * P.KVD + (size_t)kvh * HD;
    const int np = a1 - a0;
    // pass 1: four positions per sweep, rounds of four sweeps whose K rows are all requested before the first is used
    {
        const int sub = lane >> 3, li = lane & 7;
        const double* qj = qs + li * QSTR;
        #pragma unroll 1
        for (int s0 = 0; s0 * 4 < np; s0 += 4) {
            uint4 kraw[4][KV4];
            #pragma unroll
            for (int u = 0; u < 4; u++) {
                if ((s0 + u) * 4 >= np) continue;                          // warp-uniform
                const int pi = min((s0 + u) * 4 + sub, np - 1);
                const __half* kr = kbase + (size_t)(a0 + pi) * P.KVD + li * DPL;
                if constexpr (DPL >= 8) {
                    #pragma unroll
                    for (int c = 0; c < KV4; c++) kraw[u][c] = __ldcg(reinterpret_cast<const uint4*>(kr) + c);
                } else {
                    const uint2 k2 = __ldcg(reinterpret_cast<const uint2*>(kr));
                    kraw[u][0] = make_uint4(k2.x, k2.y, 0u, 0u);
                }
            }
            #pragma unroll
            for (int u = 0; u < 4; u++) {
                if ((s0 + u) * 4 < np) {                                   // warp-uniform
                    const int pi = (s0 + u) * 4 + sub;
                    double acc = 0.0;
                    #pragma unroll
                    for (int c = 0; c < KV4; c++) {
                        const __half2* hh = reinterpret_cast<const __half2*>(&kraw[u][c]);
                        #pragma unroll
                        for (int e = 0; e < 4; e++) {
                            if (c * 8 + 2 * e < DPL) {
                                const float2 f = __half22float2(hh[e]);
                                const double2 qq = *reinterpret_cast<const double2*>(qj + c * 8 + 2 * e);
                                acc = __fma_rn(qq.x, (double)f.x, acc);
                                acc = __fma_rn(qq.y, (double)f.y, acc);
                            }
                        }
                    }
                    #pragma unroll
                    for (int sft = 1; sft <= 4; sft <<= 1) acc = __dadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, sft));
                    if (li == 0 && pi < np) sc[a0 + pi] = __fmul_rn(__double2float_rn(acc), inv);
                }
            }
        }
    }
    prof_mark(P, 27);
    // the V rows of this warp's positions: requested now, used after the weights are known
    // (lane = the dim pairs {2 lane, 2 lane + 1} + 64 j: one 4-byte load per pair; head_dim 32: lane = dim)
    // (the first sixteen; a warp has more only beyond 128 positions, and fetches those when it gets there)
    constexpr int VB = 16, VP = DPW >= 2 ? DPW / 2 : 1;
    unsigned vh[VB][VP];
    auto load_v = [&](int r) {
        #pragma unroll
        for (int u = 0; u < VB; u++) {
            const __half* vrow = vbase + (size_t)(a0 + min(r * VB + u, max(np - 1, 0))) * P.KVD;
            if constexpr (DPW >= 2) {
                #pragma unroll
                for (int j = 0; j < VP; j++) vh[u][j] = __ldcg(reinterpret_cast<const unsigned*>(vrow) + lane + 32 * j);
            } else {
                vh[u][0] = __ldcg(reinterpret_cast<const unsigned short*>(vrow) + lane);
            }
        }
    };
    if (np > 0) load_v(0);
    prof_mark(P, 28);
    __syncthreads();
    prof_mark(P, 15);
    // maximum over the whole range (every warp scans all scores), then one weight per thread
    float mx = -INFINITY;
    #pragma unroll
    for (int i = 0; i < 8; i++) if (lane + 32 * i < Lp) mx = fmaxf(mx, sc[lane + 32 * i]);
    mx = warp_max_float(mx);
    if (tid < Lp) wt[tid] = exp_shared((double)sc[tid] - (double)mx);
    prof_mark(P, 29);
    __syncthreads();
    prof_mark(P, 30);
    // pass 2
    double o[DPW], ls = 0.0;
    #pragma unroll
    for (int i = 0; i < DPW; i++) o[i] = 0.0;
    #pragma unroll 1
    for (int r = 0; r * VB < np; r++) {
        if (r > 0) load_v(r);
        #pragma unroll
        for (int u = 0; u < VB; u++) {
            if (r * VB + u < np) {
                const double w = wt[a0 + r * VB + u];
                ls = __dadd_rn(ls, w);
                if constexpr (DPW >= 2) {
                    #pragma unroll
                    for (int j = 0; j < VP; j++) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&vh[u][j]));
                        o[2 * j] = __fma_rn(w, (double)f.x, o[2 * j]);
                        o[2 * j + 1] = __fma_rn(w, (double)f.y, o[2 * j + 1]);
                    }
                } else {
                    o[0] = __fma_rn(w, (double)__half2float(__ushort_as_half((unsigned short)vh[u][0])), o[0]);
                }
            }
        }
    }
    if constexpr (DPW >= 2) {
        #pragma unroll
        for (int j = 0; j < VP; j++) *reinterpret_cast<double2*>(ow + warp * HD + 2 * (lane + 32 * j)) = make_double2(o[2 * j], o[2 * j + 1]);
    } else {
        ow[warp * HD + lane] = o[0];
    }
    if (lane == 0) lw[warp] = ls;
    prof_mark(P, 31);
    // the new position's K / V rows (plain stores above) are performed before anything this CTA publishes
    if (TG && STORE_KV && tid < HD) __threadfence();
    __syncthreads();
    prof_mark(P, 16);
    if (warp < DPW) {
        const int d = warp * 32 + lane;
        double ob = ow[d], ll = lw[0];
        #pragma unroll
        for (int w = 1; w < DNW; w++) { ob = __dadd_rn(ob, ow[w * HD + d]); ll = __dadd_rn(ll, lw[w]); }
        const float v = __double2float_rn(__ddiv_rn(ob, ll));
        const int e = head * HD + d;
        __stcg(P.att + e, v);
        if constexpr (TG) {
            __half dq; int sq;
            const int qv8 = quant_block_warp2(v, dq, sq);
            publish_q8_block<false>(pub, P.xo.att, P.xo.att + P.NH * HD / 4, e >> 5, lane, qv8, dq, sq);
        } else {
            P.att_q[e] = (int8_t)quant_block_warp(v, lane, nullptr, P.att_d + (e >> 5));
        }
    }
    prof_mark(P, 17);
    return true;
}

// ---- short-range attention on the CTAs set aside for it ------------------------------------------------
// A CTA of [0, attn_ctas) handles HPC query heads of one kv head and nothing else, which buys two things.  (1) The K and V
// rows of the cached positions are known long before the layer's q arrives, so the CTA copies them into shared memory
// ahead of time (one bulk copy per row, rows padded by 16 bytes against bank conflicts; the copy for the next layer is
// issued as soon as this layer's arithmetic has left the buffer): between q's arrival and the published output there is
// no global load at all.  (2) One fp16 -> double conversion of a K or V element serves all HPC heads.
// The new position's K and V come with q as tagged words; they go into the shared-memory rows directly and to the global
// cache after the output has been published (fenced before this CTA's next output, which is what later readers wait for).
// Per head the arithmetic is attention_short's, operation for operation: same bits.
constexpr int kAttnRows = kShortAttnMax;
template <int HD> __host__ __device__ constexpr int attn_row_bytes() { return 2 * HD + 16; }
__host__ __device__ inline size_t attn_dedicated_smem(int HD, int HPC) {
    return (size_t)2 * kAttnRows * (2 * HD + 16) + (size_t)HPC * (HD + 16) * 8 + (size_t)HPC * kAttnRows * 8 + (size_t)DNW * HPC * HD * 8 +
           (size_t)DNW * HPC * 8 + (size_t)HPC * kAttnRows * 4 + 64;
}
// query heads per attention CTA: two where the group size is even (1.5B: six CTAs of two heads; three heads per CTA
// measured 4.5 us per layer on the critical path, see the profile table in the repository's design notes), the whole
// group where it is odd, one head for groups of one or two
__host__ __device__ constexpr int attn_heads_per_cta(int G) { return (G % 2 == 0 && G > 2) ? MI_ATTN_HPC_EVEN(G) : (G <= 2 ? 1 : G); }

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

struct AttnPrefetch { uint64_t* bar; unsigned parity; int layer, pos; bool pending; bool ok; };

// Request the K and V rows of positions [0, pos) of `layer` for this CTA's kv head (whole CTA; ends with the copies in flight).
template <int HD>
__device__ __forceinline__ void attn_prefetch_issue(const DecodeParams& P, uint8_t* smem, AttnPrefetch& pf, int layer, int pos, int kvh) {
    constexpr int RSB = attn_row_bytes<HD>();
    const int tid = threadIdx.x;
    pf.layer = layer; pf.pos = pos; pf.pending = pos > 0;
    if (pos <= 0) return;
    if (tid == 0) { fence_proxy_async(); mbar_expect_tx(pf.bar, 2u * (unsigned)pos * (2u * HD)); }
    __syncthreads();
    uint8_t* Kb = smem; uint8_t* Vb = smem + (size_t)kAttnRows * RSB;
    for (int p = tid; p < pos; p += DNT) {
        const size_t row = ((size_t)layer * P.max_seq + p) * P.KVD + (size_t)kvh * HD;
        bulk_g2s(Kb + (size_t)p * RSB, P.kc + row, 2 * HD, pf.bar);
        bulk_g2s(Vb + (size_t)p * RSB, P.vc + row, 2 * HD, pf.bar);
    }
}

template <int HD, int GQ, int HPC>
__device__ __forceinline__ AttnPrefetch attention_dedicated(const DecodeParams& P, int l, int pos, uint8_t* smem, AttnPrefetch pf,
                                                                unsigned tag_in, const Pub pub, int next_layer, int next_pos) {
    constexpr int DPW = HD / 32, RSB = attn_row_bytes<HD>();
    constexpr int LPP = 8, DPL = HD / LPP, QSTR = DPL + 2;
    constexpr int QN = (HPC * HD + DNT - 1) / DNT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h0 = (int)blockIdx.x * HPC, kvh = h0 / GQ, Lp = pos + 1, nq = P.NH * HD;
    uint8_t* Kb = smem; uint8_t* Vb = smem + (size_t)kAttnRows * RSB;
    double* qs = reinterpret_cast<double*>(smem + (size_t)2 * kAttnRows * RSB);   // [HPC][LPP][QSTR]
    double* wt = qs + HPC * LPP * QSTR;                                         // [HPC][rows]
    double* ow = wt + HPC * kAttnRows;                                          // [DNW][HPC][HD]
    double* lw = ow + DNW * HPC * HD;                                           // [DNW][HPC]
    float* sc = reinterpret_cast<float*>(lw + DNW * HPC);                       // [HPC][rows]
    // the rows of this (layer, position) should be on their way already; a launch's first layer requests them here
    if (!(pf.layer == l && pf.pos == pos)) {
        if (pf.pending) { (void)mbar_wait_bounded(pf.bar, pf.parity); pf.parity ^= 1u; }
        attn_prefetch_issue<HD>(P, smem, pf, l, pos, kvh);
    }
    // q of this CTA's heads and k / v of the new position (tagged words, packed order: dim d sits at 2d (d < HD/2) or 2(d-HD/2)+1)
    unsigned qw[QN + 2], valid = 0;
    #pragma unroll
    for (int k = 0; k < QN; k++) if (tid + k * DNT < HPC * HD) valid |= 1u << k;
    if (tid < HD) valid |= 3u << QN;
    const unsigned long long* qv = P.xw + P.xo.qkv;
    const int dk = tid < HD / 2 ? 2 * tid : 2 * (tid - HD / 2) + 1;
    bool ok = tw_poll(P, tag_in, valid, [&](int k) -> const unsigned long long* {
        if (k < QN) {
            const int i = tid + k * DNT, j = i / HD, d = i % HD, pk = d < HD / 2 ? 2 * d : 2 * (d - HD / 2) + 1;
            return qv + (size_t)(h0 + j) * HD + pk;
        }
        return k == QN ? qv + nq + (size_t)kvh * HD + dk : qv + nq + P.KVD + (size_t)kvh * HD + tid;
    }, qw);
    #pragma unroll
    for (int k = 0; k < QN; k++) {
        const int i = tid + k * DNT;
        if (i < HPC * HD) { const int j = i / HD, d = i % HD; qs[(j * LPP + d / DPL) * QSTR + d % DPL] = (double)__uint_as_float(qw[k]); }
    }
    const __half knew = __float2half_rn(__uint_as_float(qw[QN])), vnew = __float2half_rn(__uint_as_float(qw[QN + 1]));
    if (tid < HD) {
        reinterpret_cast<__half*>(Kb + (size_t)pos * RSB)[tid] = knew;
        reinterpret_cast<__half*>(Vb + (size_t)pos * RSB)[tid] = vnew;
    }
    prof_mark(P, 14);
    if (ok && pf.pending) { ok = mbar_wait_bounded(pf.bar, pf.parity); pf.parity ^= 1u; pf.pending = false; }
    if (!__syncthreads_and(ok ? 1 : 0)) { pf.ok = false; return pf; }
    prof_mark(P, 27);
    const float inv = __fdiv_rn(1.f, __fsqrt_rn((float)HD));
    const int a0 = (int)((long long)Lp * warp / DNW), a1 = (int)((long long)Lp * (warp + 1) / DNW), np = a1 - a0;
    // pass 1: thread = position (the range is at most 256 rows).  A thread walks its K row front to back, one fp16 ->
    // double conversion of an element serving all heads, and adds the products in dimension order with one accumulator
    // per head: the order in which the reference's CPU program adds this sum (src/cpu_infer.cpp:127-130).  q comes as
    // 16-byte broadcast loads (every lane reads the same address); rows are 16 bytes longer than their data, so the
    // eight lanes of a quarter warp cover all banks.  (Eight lanes per
    // position with a shuffle tree per sweep measured 1.8 us per layer at a hundred positions: the conversions and the
    // tree of every sweep were serial.)
    if (warp * 32 < Lp) {
        const uint4* kr = reinterpret_cast<const uint4*>(Kb + (size_t)min(tid, Lp - 1) * RSB);
        double acc[HPC];
        #pragma unroll
        for (int j = 0; j < HPC; j++) acc[j] = 0.0;
        #pragma unroll 2
        for (int c = 0; c < HD / 8; c++) {
            const uint4 kk = kr[c];
            const __half2* hh = reinterpret_cast<const __half2*>(&kk);
            double kd[8];
            #pragma unroll
            for (int e = 0; e < 4; e++) { const float2 f = __half22float2(hh[e]); kd[2 * e] = (double)f.x; kd[2 * e + 1] = (double)f.y; }
            #pragma unroll
            for (int j = 0; j < HPC; j++) {
                #pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const int d = c * 8 + e;
                    const double2 qq = *reinterpret_cast<const double2*>(qs + (j * LPP + d / DPL) * QSTR + d % DPL);
                    acc[j] = __fma_rn(qq.x, kd[e], acc[j]);
                    acc[j] = __fma_rn(qq.y, kd[e + 1], acc[j]);
                }
            }
        }
        if (tid < Lp) {
            #pragma unroll
            for (int j = 0; j < HPC; j++) sc[j * kAttnRows + tid] = __fmul_rn(__double2float_rn(acc[j]), inv);
        }
    }
    __syncthreads();
    prof_mark(P, 15);
    // per head: maximum over the whole range, then one weight per (head, position)
    float mx[HPC];
    #pragma unroll
    for (int j = 0; j < HPC; j++) {
        float m = -INFINITY;
        #pragma unroll
        for (int i = 0; i < kAttnRows / 32; i++) if (lane + 32 * i < Lp) m = fmaxf(m, sc[j * kAttnRows + lane + 32 * i]);
        mx[j] = warp_max_float(m);
    }
    for (int idx = tid; idx < HPC * Lp; idx += DNT) {
        const int j = idx / Lp, p = idx - j * Lp;
        float mj = mx[0];
        #pragma unroll
        for (int jj = 1; jj < HPC; jj++) if (j == jj) mj = mx[jj];
        wt[j * kAttnRows + p] = exp_shared((double)sc[j * kAttnRows + p] - (double)mj);
    }
    prof_mark(P, 29);
    __syncthreads();
    prof_mark(P, 30);
    // pass 2: lane = the dim pairs {2 lane, 2 lane + 1} + 64 jj (head_dim 32: lane = dim)
    constexpr int VP = DPW >= 2 ? DPW / 2 : 1;
    double o[HPC][DPW], ls[HPC];
    #pragma unroll
    for (int j = 0; j < HPC; j++) {
        ls[j] = 0.0;
        #pragma unroll
        for (int i = 0; i < DPW; i++) o[j][i] = 0.0;
    }
    #pragma unroll 2
    for (int u = 0; u < np; u++) {
        const uint8_t* vrow = Vb + (size_t)(a0 + u) * RSB;
        double vd[DPW];
        if constexpr (DPW >= 2) {
            #pragma unroll
            for (int jj = 0; jj < VP; jj++) {
                const float2 f = __half22float2(reinterpret_cast<const __half2*>(vrow)[lane + 32 * jj]);
                vd[2 * jj] = (double)f.x; vd[2 * jj + 1] = (double)f.y;
            }
        } else {
            vd[0] = (double)__half2float(reinterpret_cast<const __half*>(vrow)[lane]);
        }
        #pragma unroll
        for (int j = 0; j < HPC; j++) {
            const double w = wt[j * kAttnRows + a0 + u];
            ls[j] = __dadd_rn(ls[j], w);
            #pragma unroll
            for (int i = 0; i < DPW; i++) o[j][i] = __fma_rn(w, vd[i], o[j][i]);
        }
    }
    #pragma unroll
    for (int j = 0; j < HPC; j++) {
        double* od = ow + (size_t)(warp * HPC + j) * HD;
        if constexpr (DPW >= 2) {
            #pragma unroll
            for (int jj = 0; jj < VP; jj++) *reinterpret_cast<double2*>(od + 2 * (lane + 32 * jj)) = make_double2(o[j][2 * jj], o[j][2 * jj + 1]);
        } else {
            od[lane] = o[j][0];
        }
        if (lane == 0) lw[warp * HPC + j] = ls[j];
    }
    prof_mark(P, 31);
    __syncthreads();
    prof_mark(P, 16);
    // finish: one 32-dim block of one head per warp and round
    for (int b = warp; b < HPC * DPW; b += DNW) {
        const int j = b / DPW, d = (b % DPW) * 32 + lane;
        double ob = ow[(size_t)j * HD + d], ll = lw[j];
        #pragma unroll
        for (int w = 1; w < DNW; w++) { ob = __dadd_rn(ob, ow[(size_t)(w * HPC + j) * HD + d]); ll = __dadd_rn(ll, lw[w * HPC + j]); }
        const float v = __double2float_rn(__ddiv_rn(ob, ll));
        const int e = (h0 + j) * HD + d;
        __stcg(P.att + e, v);
        __half dq; int sq;
        const int qv8 = quant_block_warp2(v, dq, sq);
        publish_q8_block<false>(pub, P.xo.att, P.xo.att + P.NH * HD / 4, e >> 5, lane, qv8, dq, sq);
    }
    prof_mark(P, 17);
    // the new position into the global cache (CTAs that share a kv head store the same bits); performed, for the generic and
    // the bulk-copy path alike, before this CTA publishes anything else
    if (tid < HD) {
        P.kc[((size_t)l * P.max_seq + pos) * P.KVD + (size_t)kvh * HD + tid] = knew;
        P.vc[((size_t)l * P.max_seq + pos) * P.KVD + (size_t)kvh * HD + tid] = vnew;
        __threadfence();
        fence_proxy_async();
    }
    __syncthreads();                                  // the buffer is free, the stores are fenced
    if (next_layer >= 0 && next_pos + 1 <= kShortAttnMax) attn_prefetch_issue<HD>(P, smem, pf, next_layer, next_pos, kvh);
    else { pf.layer = -1; pf.pending = false; }
    pf.ok = true;
    return pf;
}

// The whole life of a CTA that does nothing but attention: every step, every layer, wait for q, attend, publish.  One call
// at the top of the kernel, out of line: its registers and instructions are its own, and the CTAs that carry the GEMV phases
// never see any of it (measured: an out-of-line call inside their per-layer loop, or this code inlined into it, costs the
// GEMV phases 10 - 25 %).
// whether this build holds the attention variant a position needs (the host picks the build by the launch's positions)
__device__ __forceinline__ bool lean_regime_ok(int pos, int attn_ctas) {
#if MI_LEAN == 1
    return pos + 1 <= kShortAttnMax && attn_ctas > 0;
#elif MI_LEAN == 2
    return pos + 1 > kShortAttnMax && pos + 1 <= kPerHeadAttnMax;
#elif MI_LEAN == 3
    return pos + 1 > kPerHeadAttnMax;
#else
    return true;
#endif
}

template <int HD, int G>
static __device__ __noinline__ void attn_cta_main(const DecodeParams& P, int step0, int step1, int ph0, int ph1, uint8_t* smem, uint8_t* stage, uint64_t* bar) {
    const int nph = 5 * P.L + 1;
    pdl_launch_dependents();
    pdl_wait_prior();
    AttnPrefetch apf; apf.bar = bar; apf.parity = 0; apf.layer = -1; apf.pos = -1; apf.pending = false; apf.ok = true;
    const unsigned epoch = __ldcg(P.epoch_dev);
    const int pos_base = P.pos_dev ? __ldcg(P.pos_dev) : P.pos0;
    bool ok = true;
    int err_code = MI_ERR_TIMEOUT;
#if MI_PROF
    const long long prof_c0 = clock64(); const unsigned long long prof_t0 = gtime_ns();
    if (threadIdx.x == 0) s_prof_t = prof_t0;
#endif
    for (int step = step0; step < step1 && ok; step++) {
        const int pos = pos_base + step;
        if (pos < 0 || pos >= P.max_seq || !lean_regime_ok(pos, P.attn_ctas)) { ok = false; err_code = MI_ERR_LIMIT; break; }
        const unsigned tag0 = epoch + (unsigned)(step - step0) * (unsigned)nph + 1u;
        if (P.stop_token >= 0 && step > step0 && step >= P.n_forced && ph0 == 0 && ph1 == nph) {
            // the stop rule: learn the token the previous step picked (its lm_head phase carries tag tag0 - 1)
            unsigned tw[1];
            const bool got = tw_poll(P, tag0 - 1u, 1u, [&](int) { return P.xw + P.xo.tokw; }, tw);
            ok = __syncthreads_and(got ? 1 : 0) != 0;
            if (!ok || (int)tw[0] == P.stop_token) break;
        }
        for (int l = max(0, (ph0 + 3) / 5); 5 * l + 1 < ph1 && l < P.L && ok; l++) {
            const int ph = 5 * l + 1;
            Pub pub;
            pub.xw = P.xw; pub.tag = tag0 + (unsigned)ph; pub.mute = ph == P.drop_phase;
#if MI_TP
            pub.tp = &P.tp;
#endif
#if MI_LEAN <= 1
            if (pos + 1 <= kShortAttnMax) {
                // where this CTA's next attention will be: the next layer of this step, or layer 0 of the next step
                int nl = -1, np_ = pos;
                if (ph + 5 < ph1 && l + 1 < P.L) nl = l + 1;
                else if (step + 1 < step1 && ph0 <= 1) { nl = 0; np_ = pos + 1; }
                apf = attention_dedicated<HD, G, attn_heads_per_cta(G)>(P, l, pos, smem, apf, pub.tag - 1u, pub, nl, np_);
                ok = apf.ok;
            }
#endif
#if MI_LEAN == 0
            else {
                if (apf.pending) { (void)mbar_wait_bounded(apf.bar, apf.parity); apf.parity ^= 1u; apf.pending = false; apf.layer = -1; }
                if (pos + 1 <= kPerHeadAttnMax) ok = attention_phase<HD, 1, G, true, false, true>(P, l, pos, stage, pub.tag - 1u, pub);
                else ok = attention_phase<HD, G, G, true, false, true>(P, l, pos, stage, pub.tag - 1u, pub);
            }
#elif MI_LEAN == 2
            ok = attention_phase<HD, 1, G, true, false, true>(P, l, pos, stage, pub.tag - 1u, pub);
#elif MI_LEAN == 3
            ok = attention_phase<HD, G, G, true, false, true>(P, l, pos, stage, pub.tag - 1u, pub);
#endif
            ok = __syncthreads_and(ok ? 1 : 0) != 0;
            prof_mark(P, 3);
        }
    }
#if MI_PROF
    if (P.prof && (int)blockIdx.x == P.prof_cta) {
        if (threadIdx.x == 0) { s_prof[8] = (unsigned long long)(clock64() - prof_c0); s_prof[9] = gtime_ns() - prof_t0; }
        __syncthreads();
        if (threadIdx.x < kProfSlots) P.prof[threadIdx.x] += s_prof[threadIdx.x];
    }
#endif
    if (apf.pending) (void)mbar_wait_bounded(apf.bar, apf.parity);      // copies in flight target this CTA's shared memory
    if (!ok && (threadIdx.x & 31) == 0) atomicMax(P.err, err_code);
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
    sm.lp = reinterpret_cast<LayerPtrs*>(after_jobs);              // [<= 64]
    after_jobs += 64 * sizeof(LayerPtrs);
    sm.cs = reinterpret_cast<float*>(after_jobs);                 // [HD]: cos then sin
    sm.red = reinterpret_cast<double*>(after_jobs + 1024);         // 32 doubles
    sm.fold = reinterpret_cast<double*>(after_jobs + 1024 + 256);
    sm.h = reinterpret_cast<float*>(after_jobs + 1024 + 256 + kFoldBytes);
    sm.stage = after_jobs + 1024 + 256 + kFoldBytes + ((size_t)P.E * 4 + 127) / 128 * 128;
    __shared__ int s_tok;
    __shared__ uint64_t s_attn_bar;
#if MI_PROF
    if (tid < kProfSlots) s_prof[tid] = 0;
#endif

    for (int i = tid; i < njobs * (int)(sizeof(Job) / 4); i += DNT)
        reinterpret_cast<int*>(sm.jobs)[i] = __ldg(reinterpret_cast<const int*>(P.jobs) + i);
    for (int i = tid; i < P.L * (int)(sizeof(LayerPtrs) / 4); i += DNT)
        reinterpret_cast<int*>(sm.lp)[i] = __ldg(reinterpret_cast<const int*>(P.layers) + i);
    const bool attn_only = (int)blockIdx.x < P.attn_ctas;        // this CTA does nothing but attention; it lays the shared memory out its own way
    if (lane == 0) {
        if (!attn_only) {
            #pragma unroll
            for (int s = 0; s < DS; s++) mbar_init(&sm.bars[warp * DS + s], 1);
        }
        if (warp == 0) mbar_init(&s_attn_bar, 1);
        mbar_fence_init();
    }
    __syncthreads();

    if (attn_only) {                                  // CTAs [0, attn_ctas): attention and nothing else
        attn_cta_main<HD, G>(P, step0, step1, ph0, ph1, smem, sm.stage, &s_attn_bar);
        return;
    }

    // jobs covered by the phase range of this launch
    auto job_of_phase = [&](int ph) -> int {          // first job at or after phase ph
        if (ph >= nph - 1) return ph >= nph ? njobs : njobs - 1;
        const int l = ph / 5, k = ph % 5;
        return 4 * l + (k == 0 ? 0 : k <= 2 ? 1 : k == 3 ? 2 : 3);
    };
    WarpStream ws;
    ws.init(sm, P, warp, step0, step1, job_of_phase(ph0), job_of_phase(ph1));
    if (lane == 0) {
        #pragma unroll
        for (int s = 0; s < DS; s++) ws.issue_one();
    }
    pdl_launch_dependents();
    pdl_wait_prior();

    const int maxin = P.E > P.FF ? P.E : P.FF;
    int8_t* xq_s = reinterpret_cast<int8_t*>(sm.stage);
    float2* xs_s = reinterpret_cast<float2*>(sm.stage + maxin);
    bool ok = true, h_valid = false;                   // h_valid: this CTA's shared-memory copy of the residual stream is current
    bool stopped = false;                              // the run ended early on the stop token: tiles of later steps are in flight
    int err_code = MI_ERR_TIMEOUT;
    const unsigned epoch = __ldcg(P.epoch_dev);
    const int pos_base = P.pos_dev ? __ldcg(P.pos_dev) : P.pos0;
    // candidates of the greedy pick: one {value, index} pair of words per CTA (and per GPU when the exchange runs in here)
    const int cand_world = P.tp.on ? P.tp.world : 1, n_cand = cand_world * ws.ggrid;
    const int my_cand = P.xo.cand + ((P.tp.on ? P.tp.rank : 0) * ws.ggrid + ws.gcta) * 4;

    // cos / sin of a position's angles come from the table made at load: the double-precision cosine and sine and their
    // argument reduction stay out of this function (as code, and as calls inside the step loop)
    auto rope_table = [&](int pos) {
        if (tid < HD) sm.cs[tid] = __ldg(P.rope_cs + (size_t)min(max(pos, 0), P.max_seq - 1) * HD + tid);
    };

#if MI_PROF
    const long long prof_c0 = clock64(); const unsigned long long prof_t0 = gtime_ns();
    if (tid == 0) s_prof_t = prof_t0;
#endif
    if (step0 < step1) rope_table(pos_base + step0);
    __syncthreads();
    for (int step = step0; step < step1 && ok; step++) {
        const int pos = pos_base + step;
        if (pos < 0 || pos >= P.max_seq || !lean_regime_ok(pos, P.attn_ctas)) { ok = false; err_code = MI_ERR_LIMIT; break; }   // the same on every CTA: nobody waits for anybody
        const unsigned tag0 = epoch + (unsigned)(step - step0) * (unsigned)nph + 1u;        // tag of (step, phase 0)
        if (step > step0 && ph1 != nph) { rope_table(pos); __syncthreads(); }     // (otherwise the previous step's lm_head phase has made the table)
        prof_mark(P, kProfStep);
        for (int ph = ph0; ph < ph1 && ok; ph++) {
            const int l = ph / 5, k = ph == nph - 1 ? 5 : ph % 5;
            Pub pub;
            pub.xw = P.xw; pub.tag = tag0 + (unsigned)ph; pub.mute = ph == P.drop_phase;
#if MI_TP
            pub.tp = &P.tp;
#endif
            // One call site each for the norm prologue, the q8 prologue and the CTA job: the four per-layer GEMV
            // phases run the same instructions (they stay in the instruction cache from phase to phase) and differ
            // only in pointers and in the few lines of their epilogue.
            if (k == 0 || k == 3 || k == 5) {
                // QKV : h = (l == 0) ? embedding : h + down projection of layer l-1        (committed as h_in)
                // GU  : h = h + O projection                                                 (committed as h_mid)
                // LM  : final norm over h + last down projection
                const float* gsrc = nullptr; const unsigned long long* addw = nullptr; float* commit = nullptr; const float* nw = nullptr;
                if (k == 0 && l == 0) {
                    int tok = step < P.n_forced ? __ldg(P.in_tokens + step) : (step == step0 ? __ldcg(P.cur_token) : s_tok);
                    tok = min(max(tok, 0), P.V - 1);
                    residual_init(P, sm.h, nullptr, tok, P.E);
                    commit = P.h_in; nw = sm.lp[0].attn_norm;
                } else if (k == 0) {
                    gsrc = h_valid ? nullptr : P.h_mid; addw = P.xw + P.xo.down; commit = P.h_in; nw = sm.lp[l].attn_norm;
                } else if (k == 3) {
                    gsrc = h_valid ? nullptr : P.h_in; addw = P.xw + P.xo.o; commit = P.h_mid; nw = sm.lp[l].ffn_norm;
                } else {
                    gsrc = h_valid ? nullptr : P.h_mid; addw = P.xw + P.xo.down; nw = P.out_norm;
                }
                if (gsrc) residual_init(P, sm.h, gsrc, 0, P.E);                 // a launch that starts in mid-step
                // the committed copy serves launches that start in mid-step (and state read-back); a launch over whole steps has no reader for it
                if (MI_LEAN && ph0 == 0 && ph1 == nph) commit = nullptr;
                ok = stage_norm_q8u(P, sm.h, addw, pub.tag - 1u, commit, nw, P.E, P.eps, sm.red, xq_s, xs_s);
                h_valid = true;
                prof_mark(P, 2 * k);
            } else if (k == 2 || k == 4) {
                const Job& jb = sm.jobs[4 * l + (k == 2 ? 1 : 3)];
                if (ws.first_cta_unit(jb) < jb.n_units) {        // only CTAs that have a unit of the job consume its input
                    prof_mark(P, 2 * k);
                    if (k == 2) ok = stage_poll_q8(P, P.xw + P.xo.att, P.NH * HD, pub.tag - 1u, xq_s, xs_s);
                    else ok = stage_poll_q8(P, P.xw + P.xo.act, P.FF, pub.tag - 1u, xq_s, xs_s);
                    prof_mark(P, kProfWait);
                }
            }
            if (!ok) break;
            if (k == 1) {
                if (pos + 1 <= kShortAttnMax && P.attn_ctas > 0) {
                    // the attention CTAs' business
                }
#if MI_LEAN == 0
                else if (pos + 1 <= kShortAttnMax) ok = attention_short<HD, G, true, false, true>(P, l, pos, sm.stage, pub.tag - 1u, pub);
                else if (pos + 1 <= kPerHeadAttnMax) ok = attention_phase<HD, 1, G, true, false, true>(P, l, pos, sm.stage, pub.tag - 1u, pub);
                else ok = attention_phase<HD, G, G, true, false, true>(P, l, pos, sm.stage, pub.tag - 1u, pub);
#elif MI_LEAN == 2
                else ok = attention_phase<HD, 1, G, true, false, true>(P, l, pos, sm.stage, pub.tag - 1u, pub);
#elif MI_LEAN == 3
                else ok = attention_phase<HD, G, G, true, false, true>(P, l, pos, sm.stage, pub.tag - 1u, pub);
#endif
            } else if (k != 5) {
                const int jn = 4 * l + (k == 0 ? 0 : k == 2 ? 1 : k == 3 ? 2 : 3);
                const float* bias = sm.lp[l].bqkv;
                const int nq = P.NH * HD;
                ok = run_cta_job(ws, P, sm, jn, lane, xq_s, xs_s, pub, [&](int g, int ln, float v0, float v1) {
                    if (k == 0) {                                            // + bias, RoPE, packed q / k / v
                        const int p = g * 32 + ln;
                        const float v = __fadd_rn(v0, __ldg(bias + p));
                        const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
                        float out = v;
                        if (p < nq + P.KVD) {                                  // q or k: rotate the (even, odd) lane pair
                            const int within = (p < nq ? p : p - nq) % HD, i = within >> 1;
                            const double c = sm.cs[i], s = sm.cs[HD / 2 + i];    // products are exact in double: one rounding each
                            if ((within & 1) == 0) out = __double2float_rn(__dsub_rn(__dmul_rn((double)v, c), __dmul_rn((double)partner, s)));
                            else out = __double2float_rn(__dadd_rn(__dmul_rn((double)partner, s), __dmul_rn((double)v, c)));
                        }
                        if (p < nq + 2 * P.KVD) pub.local(P.xo.qkv + p, __float_as_uint(out));
                    } else if (k == 3) {                                     // SwiGLU of (gate, up), one q8_0 block per warp
                        const double gd = (double)v0;
                        const float a = __double2float_rn(__dmul_rn(__ddiv_rn(gd, __dadd_rn(1.0, exp_shared(-gd))), (double)v1));
                        __half dq; int sq;
                        const int qv = quant_block_warp2(a, dq, sq);         // FF is a multiple of 32: group g is block g
                        publish_q8_block<true>(pub, P.xo.act, P.xo.act + P.FF / 4, g, ln, qv, dq, sq);
                    } else if (k == 2) {
                        pub.local(P.xo.o + g * 32 + ln, __float_as_uint(v0));
                    } else {
                        pub.shared(P.xo.down + g * 32 + ln, __float_as_uint(v0));
                    }
                });
            } else {
                // ---- lm_head on the staged final norm, greedy argmax (lowest index wins ties)
                // Each candidate is {best value, its row, second-best value}: the runner-up gives the logit margin (top-1 minus
                // top-2) that the reference's engine reports per token (src/mega.cu:523-550, 385-392).
                Cand cd; cd.best = -INFINITY; cd.idx = 0x7fffffff; cd.second = -INFINITY;
                float* lg = P.logits ? P.logits + (long long)(step - step0) * P.logits_stride : nullptr;
                ok = run_warp_job(ws, 4 * P.L, lane, xq_s, xs_s, [&](int g, int ln, float v0) {
                    const int r = g * 32 + ln;
                    if (r < P.V) {
                        if (lg) lg[r] = v0;
                        // the reference's scan starts from logits[0] and moves on strict '>' (src/cpu_infer.cpp:153-154): a NaN
                        // never wins, and a NaN in row 0 is never beaten
                        const float vv = (r == 0 && v0 != v0) ? INFINITY : v0;
                        cd.add(vv, r);
                    }
                });
                cd.warp_reduce();
                __syncthreads();
                float* cv = reinterpret_cast<float*>(sm.red); int* ci = reinterpret_cast<int*>(sm.red) + 16; float* c2 = reinterpret_cast<float*>(sm.red) + 32;
                if (lane == 0) { cv[warp] = cd.best; ci[warp] = cd.idx; c2[warp] = cd.second; }
                __syncthreads();
                if (tid == 0) {
                    Cand t; t.best = cv[0]; t.idx = ci[0]; t.second = c2[0];
                    for (int w = 1; w < DNW; w++) { Cand o; o.best = cv[w]; o.idx = ci[w]; o.second = c2[w]; t.merge(o); }
                    pub.shared(my_cand, __float_as_uint(t.best));
                    pub.shared(my_cand + 1, (unsigned)t.idx);
                    pub.shared(my_cand + 2, __float_as_uint(t.second));
                }
                // the next step's angles while the other CTAs' candidates arrive
                if (step + 1 < step1) rope_table(pos + 1);
                // every CTA makes the pick over all candidates itself (the same bits everywhere); the first GEMV CTA writes it out
                prof_mark(P, 2 * k + 1);
                cd.best = -INFINITY; cd.idx = 0x7fffffff; cd.second = -INFINITY;
                bool okc = ok;
                for (int c0 = 0; c0 < n_cand && okc; c0 += 2 * DNT) {
                    unsigned cw[6], valid = 0;
                    if (c0 + tid < n_cand) valid |= 7u;
                    if (c0 + DNT + tid < n_cand) valid |= 56u;
                    const unsigned long long* cb = P.xw + P.xo.cand + (size_t)(c0 + tid) * 4;
                    okc = tw_poll(P, pub.tag, valid, [&](int q) { return cb + (q / 3) * (4 * DNT) + (q % 3); }, cw);
                    #pragma unroll
                    for (int h = 0; h < 2; h++) {
                        if (okc && (valid >> (3 * h) & 1u)) {
                            Cand o; o.best = __uint_as_float(cw[3 * h]); o.idx = (int)cw[3 * h + 1]; o.second = __uint_as_float(cw[3 * h + 2]);
                            cd.merge(o);
                        }
                    }
                }
                prof_mark(P, kProfWait);
                cd.warp_reduce();
                ok = __syncthreads_and(okc ? 1 : 0) != 0;       // also: cv / ci / c2 are free again
                if (lane == 0) { cv[warp] = cd.best; ci[warp] = cd.idx; c2[warp] = cd.second; }
                __syncthreads();
                if (tid == 0) {
                    Cand t; t.best = cv[0]; t.idx = ci[0]; t.second = c2[0];
                    for (int w = 1; w < DNW; w++) { Cand o; o.best = cv[w]; o.idx = ci[w]; o.second = c2[w]; t.merge(o); }
                    const int tok = t.idx == 0x7fffffff ? 0 : t.idx;
                    s_tok = tok;
                    if (ws.gcta == 0 && ok) {
                        const float margin = __fsub_rn(t.best, t.second);
                        const bool stopping = P.stop_token >= 0 && tok == P.stop_token && step + 1 >= P.n_forced && ph0 == 0;
                        if (P.stop_token >= 0 && P.attn_ctas > 0) pub.local(P.xo.tokw, (unsigned)tok);
                        __stcg(P.cur_token, tok); __stcg(P.best_val, t.best); P.out_tokens[step] = tok;
                        if (P.out_margins) P.out_margins[step] = margin;
                        if (P.ring.count) {
                            // the host reads along: token, margin and time of every step into mapped host memory, the count of
                            // valid entries every fourth step and at the end, after a system-scope fence (src/mega.cu:847-856)
                            const int slot = P.ring.base + (step - step0);
                            if (slot < P.ring.capacity) {
                                P.ring.tokens[slot] = tok; P.ring.margins[slot] = margin; P.ring.ns[slot] = gtime_ns();
                                if (((step - step0) & 3) == 3 || step == step1 - 1 || stopping) { __threadfence_system(); *reinterpret_cast<volatile int*>(P.ring.count) = slot + 1; }
                            }
                        }
                    }
                }
            }
            ok = __syncthreads_and(ok ? 1 : 0) != 0;          // a wait that gave up in one warp stops the whole CTA
            prof_mark(P, 2 * k + 1);
        }
        // the stop rule (every CTA has made the same pick): the step that produced the stop token was the last
        if (P.stop_token >= 0 && ok && ph0 == 0 && ph1 == nph && s_tok == P.stop_token && step + 1 >= P.n_forced && step + 1 < step1) {
            stopped = true;
            break;
        }
    }
#if MI_PROF
    if (P.prof && (int)blockIdx.x == P.prof_cta) {
        if (tid == 0) { s_prof[8] = (unsigned long long)(clock64() - prof_c0); s_prof[9] = gtime_ns() - prof_t0; }     // SM cycles and nanoseconds of the launch (overwrites two phase slots)
        __syncthreads();
        if (tid < kProfSlots) P.prof[tid] += s_prof[tid];
    }
#endif
    // the first GEMV CTA has seen every CTA's last candidates, which descend from every attention CTA's output (or it has given
    // up after a full time budget): all CTAs have read the epoch
    if (ws.gcta == 0 && tid == 0 && (ph1 == nph || !ok))
        *P.epoch_dev = epoch + (unsigned)(step1 - step0) * (unsigned)nph + (ok ? 0u : (unsigned)nph);
    if (!ok) {
        if (lane == 0) atomicMax(P.err, err_code);
        ws.drain();
    } else if (stopped) {
        ws.drain();
    }
}

}  // inline namespace
#endif  // __CUDACC__
}  // namespace mi
