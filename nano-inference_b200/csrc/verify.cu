// The M-token step: M <= 16 tokens at consecutive positions scored in one pass over the
// weights (speculative verify, chunked prompt processing), and the stand-alone split-KV
// attention entry point.
//
// Replaces forward_batch (reference src/cuda_infer.cu:990-1029: quant_x_q8_batch,
// gemv_dp4a_batch<T>, rope / kv_store / attention per token) and the M-token path of the
// persistent kernel (reference src/mega.cu:246-299 gemv_seq, :414-521 attention).
//
// One pass is a sequence of launches per layer
//     norm+q8 (M tokens) -> tcgen05 GEMM QKV -> RoPE + fp16 KV store -> attention (M queries)
//     -> GEMM O -> residual + norm+q8 -> GEMM gate/up -> SwiGLU+q8 -> GEMM down
// and finally norm+q8 -> GEMM lm_head -> argmax per token.  Every token goes through the
// very expressions of the single-token decode kernel (same quantizer, same double-carried
// sums, the same attention code with the token's own causal range and chunking), so its
// logits do not depend on how many tokens share the pass.
#include "model.cuh"

#include <algorithm>
#include <cstdlib>

using namespace mi;

namespace {

constexpr int VMAX = 16;

// x = (embedding row | X) (+ Y), committed to X; q8_0(rmsnorm(x) * w) (src/cpu_infer.cpp:40-46).
// One CTA per token.  Gathering: warp w owns the blocks w, w+8, ... with lane = element, all loads of a round requested
// before any is used (X is read and written here, so the compiler may not move a later load above an earlier store).
// Quantizing: eight consecutive elements per thread, four lanes per q8_0 block, two shuffle folds for the block maximum.
__global__ void __launch_bounds__(DNT) vf_norm_quant(const DecodeParams P, const int* __restrict__ tokens, bool embed, float* X, const float* Y,
                                                      int ystride, const float* __restrict__ w, int8_t* xq, __half* xd) {
    extern __shared__ __align__(16) float xs[];
    __shared__ double red[DNW];
    pdl_launch_dependents(); pdl_wait_prior();
    const int m = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, E = P.E, nb = E / 32;
    const int token = embed ? __ldg(tokens + m) : 0;
    constexpr int RB = 8;                                            // blocks per warp and round
    double ss = 0.0;
    for (int b0 = warp; b0 < nb; b0 += RB * DNW) {
        float x[RB], y[RB];
        #pragma unroll
        for (int k = 0; k < RB; k++) {
            const int b = b0 + k * DNW, e = min(b, nb - 1) * 32 + lane;
            y[k] = Y ? Y[(size_t)m * ystride + e] : 0.f;
            if (embed && P.emb_q8) {                                // a Q8_0 row as stored: int8 * d (src/gguf.h:112-118)
                const uint8_t* bp = P.emb_q8 + ((size_t)token * nb + min(b, nb - 1)) * 34;
                x[k] = __fmul_rn(__int2float_rn((int)(int8_t)__ldg(bp + 2 + lane)), __half2float(__ldg(reinterpret_cast<const __half*>(bp))));
            } else if (embed) {                                     // value (nibble - 8) * d (src/gguf.h:94-102)
                const int bb = min(b, nb - 1), g = token >> 5, r = token & 31, kb = P.emb_kb, t = bb / kb, kk = bb % kb;
                const uint8_t* tile = P.emb_base + ((size_t)g * P.emb_nt + t) * (kb * kTileRowBytes);
                const uint8_t byte = __ldg(tile + ((size_t)kk * 32 + r) * 16 + (lane & 15));
                const float d = __half2float(__ldg(reinterpret_cast<const __half*>(tile + (size_t)kb * 512 + ((size_t)r * kb + kk) * 2)));
                x[k] = __fmul_rn(__int2float_rn((lane < 16 ? (byte & 0x0F) : (byte >> 4)) - 8), d);
            } else {
                x[k] = X[(size_t)m * E + e];
            }
        }
        #pragma unroll
        for (int k = 0; k < RB; k++) {
            const int b = b0 + k * DNW;
            if (b < nb) {
                const int e = b * 32 + lane;
                const float v = Y ? __fadd_rn(x[k], y[k]) : x[k];
                X[(size_t)m * E + e] = v;
                xs[e] = v;
                const double xdv = v; ss = __fma_rn(xdv, xdv, ss);
            }
        }
    }
    #pragma unroll
    for (int o = 16; o; o >>= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    double tot = 0.0;
    #pragma unroll
    for (int v = 0; v < DNW; v++) tot = __dadd_rn(tot, red[v]);
    const float mean = __double2float_rn(__ddiv_rn(tot, (double)E));
    const float scale = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(mean, P.eps)));
    for (int t = tid; (t & ~31) * 8 < E; t += DNT) {                 // warp-uniform trip count: the folds are warp-wide
        const bool live = t * 8 < E;
        const int e0 = live ? t * 8 : 0;
        const float4 h0 = *reinterpret_cast<const float4*>(xs + e0), h1 = *reinterpret_cast<const float4*>(xs + e0 + 4);
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + e0)), w1 = __ldg(reinterpret_cast<const float4*>(w + e0 + 4));
        const float hv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w}, wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        float v[8], a = 0.f;
        #pragma unroll
        for (int i = 0; i < 8; i++) { v[i] = __fmul_rn(__fmul_rn(hv[i], scale), wv[i]); a = fmaxf(a, fabsf(v[i])); }
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
        const float inv = a > 0.f ? __fdiv_rn(127.f, a) : 0.f;
        unsigned lo = 0, hi = 0;
        #pragma unroll
        for (int i = 0; i < 4; i++) {
            lo |= ((unsigned)__float2int_rn(__fmul_rn(v[i], inv)) & 0xffu) << (8 * i);
            hi |= ((unsigned)__float2int_rn(__fmul_rn(v[4 + i], inv)) & 0xffu) << (8 * i);
        }
        if (live) {
            *reinterpret_cast<uint2*>(xq + (size_t)m * E + e0) = make_uint2(lo, hi);
            if ((t & 3) == 0) xd[(size_t)m * nb + (e0 >> 5)] = __float2half_rn(__fdiv_rn(a, 127.f));
        }
    }
}

// RoPE on the packed (pair-adjacent) q and k rows of every token, fp16 K / V into the cache
// (pos_arr / slot_arr, when given: token m sits at position pos_arr[m] of the sequence whose cache is slab slot_arr[m] -
// independent sequences sharing one weight pass; otherwise consecutive positions pos0 + m of one sequence)
__global__ void __launch_bounds__(DNT) vf_rope_kv(const DecodeParams P, int l, const int* pos0_dev, float* qkv, int stride,
                                                  const int* pos_arr, const int* slot_arr, long long slab_stride) {
    pdl_launch_dependents(); pdl_wait_prior();
    const int m = blockIdx.x, pos = pos_arr ? __ldg(pos_arr + m) : __ldg(pos0_dev) + m, HD = P.HD, nq = P.NH * HD;
    const size_t slab = slot_arr ? (size_t)__ldg(slot_arr + m) * (size_t)slab_stride : 0;
    float* v = qkv + (size_t)m * stride;
    for (int pr = threadIdx.x; pr < (nq + P.KVD) / 2; pr += blockDim.x) {
        const int p = 2 * pr, within = (p < nq ? p : p - nq) % HD, i = within >> 1;
        double c, s;
        if (pos < P.rope_rows) {                                      // the table made at load holds these very values
            c = (double)__ldg(P.rope_cs + (size_t)pos * HD + i); s = (double)__ldg(P.rope_cs + (size_t)pos * HD + HD / 2 + i);
        } else {
            const double th = (double)__fmul_rn((float)pos, __ldg(P.rope_freq + i));  // fp32 angle, as src/cpu_infer.cpp:54
            c = (double)__double2float_rn(cos(th)); s = (double)__double2float_rn(sin(th));
        }
        const double x0 = v[p], x1 = v[p + 1];
        v[p] = __double2float_rn(__dsub_rn(__dmul_rn(x0, c), __dmul_rn(x1, s)));
        v[p + 1] = __double2float_rn(__dadd_rn(__dmul_rn(x0, s), __dmul_rn(x1, c)));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < P.KVD; e += blockDim.x) {
        const int kvh = e / HD, d = e % HD, pk = d < HD / 2 ? 2 * d : 2 * (d - HD / 2) + 1;
        P.kc[slab + ((size_t)l * P.max_seq + pos) * P.KVD + e] = __float2half_rn(v[nq + kvh * HD + pk]);
        P.vc[slab + ((size_t)l * P.max_seq + pos) * P.KVD + e] = __float2half_rn(v[nq + P.KVD + e]);
    }
}

// attention of M queries: blockIdx.y = query; every query runs the decode kernel's attention over its own causal range
template <int HD, int G, bool QNAT>
__global__ void __launch_bounds__(DNT, 1) vf_attention(const __grid_constant__ DecodeParams P, int l, const int* pos0_dev, int pos0_val, long long q_stride,
                                                       const int* pos_arr, const int* slot_arr, long long slab_stride) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents(); pdl_wait_prior();
    const int m = blockIdx.y, nq = P.NH * HD;
    DecodeParams Q = P;
    Q.qkv_out = P.qkv_out + (size_t)m * q_stride;
    Q.att = P.att + (size_t)m * nq; Q.att_q = P.att_q + (size_t)m * nq; Q.att_d = P.att_d + (size_t)m * (nq / 32);
    Q.attn_part = P.attn_part + (size_t)m * P.NH * P.max_chunks * (HD + 2);
    Q.attn_cnt = P.attn_cnt + (size_t)m * P.NH;
    Q.prof = nullptr;
    const int pos = pos_arr ? __ldg(pos_arr + m) : (pos0_dev ? __ldg(pos0_dev) : pos0_val) + m;
    if (slot_arr) { const size_t slab = (size_t)__ldg(slot_arr + m) * (size_t)slab_stride; Q.kc = P.kc + slab; Q.vc = P.vc + slab; }
    if (pos + 1 <= kShortAttnMax) attention_short<HD, G, false, QNAT>(Q, l, pos, smem);
    else if (pos + 1 <= kPerHeadAttnMax) attention_phase<HD, 1, G, false, QNAT>(Q, l, pos, smem);
    else attention_phase<HD, G, G, false, QNAT>(Q, l, pos, smem);
}

// SwiGLU of the interleaved gate / up groups -> q8_0; one warp per 32-element block
__global__ void __launch_bounds__(DNT) vf_swiglu_quant(const float* Y, int FF, int8_t* act_q, __half* act_d) {
    pdl_launch_dependents(); pdl_wait_prior();
    const int m = blockIdx.y, g = blockIdx.x * DNW + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (g >= FF / 32) return;
    const float* y = Y + (size_t)m * 2 * FF + (size_t)g * 64;
    const double gd = (double)y[lane];
    const float a = __double2float_rn(__dmul_rn(__ddiv_rn(gd, __dadd_rn(1.0, exp(-gd))), (double)y[32 + lane]));
    act_q[(size_t)m * FF + g * 32 + lane] = (int8_t)quant_block_warp(a, lane, nullptr, act_d + (size_t)m * (FF / 32) + g);
}

// greedy pick per token, lowest index on ties (src/cpu_infer.cpp:153-154).  grid = (slices, tokens): every CTA
// reduces its slice of the row and folds {order-preserving value bits, ~index} into a 64-bit maximum; the last CTA of
// a token to arrive writes the index and clears the scratch for the next pass.
constexpr int kArgmaxSlices = 32;
__global__ void __launch_bounds__(512) vf_argmax(const float* logits, long long stride, int V, int* out, unsigned long long* key, unsigned* cnt) {
    __shared__ float bv[16]; __shared__ int bi[16];
    pdl_launch_dependents(); pdl_wait_prior();
    const int m = blockIdx.y;
    const float* lg = logits + (size_t)m * stride;
    const int per = (V + gridDim.x - 1) / gridDim.x, r0 = blockIdx.x * per, r1 = min(V, r0 + per);
    float best = -INFINITY; int idx = 0x7fffffff;
    for (int r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
        const float v = lg[r];
        if (v > best || (v == best && r < idx)) { best = v; idx = r; }
    }
    #pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++) if (bv[w] > bv[0] || (bv[w] == bv[0] && bi[w] < bi[0])) { bv[0] = bv[w]; bi[0] = bi[w]; }
        if (bi[0] != 0x7fffffff) {
            const unsigned fb = __float_as_uint(bv[0]), ord = (fb & 0x80000000u) ? ~fb : (fb | 0x80000000u);
            atomicMax(key + m, ((unsigned long long)ord << 32) | (unsigned)(0xFFFFFFFFu - (unsigned)bi[0]));
        }
        __threadfence();
        if (atomicAdd(cnt + m, 1u) == gridDim.x - 1) {
            __threadfence();
            const unsigned long long k = atomicExch(key + m, 0ull);
            out[m] = (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull));
            cnt[m] = 0;
        }
    }
}

// logit margin of every token of the pass: its greedy logit minus the largest other logit.  blockIdx.x = slice of the
// vocabulary, blockIdx.y = token; the slices' maxima meet in the token's key (order-preserving integer image of the
// float, as in vf_argmax, whose key and counter - back at zero when it has finished - serve here again), and the last
// slice to arrive writes the margin.  (One CTA per token read 600 KB through a single SM: 74 us of a 2.2 ms pass.)
__global__ void __launch_bounds__(512) vf_margin(const float* logits, long long stride, int V, const int* winner, float* margins,
                                                 unsigned long long* key, unsigned* cnt) {
    __shared__ float red[16];
    pdl_launch_dependents(); pdl_wait_prior();
    const int m = blockIdx.y, win = winner[m];
    const float* lg = logits + (size_t)m * stride;
    const int per = (V + gridDim.x - 1) / gridDim.x, r0 = blockIdx.x * per, r1 = min(V, r0 + per);
    float second = -INFINITY;
    for (int r = r0 + threadIdx.x; r < r1; r += blockDim.x) { const float v = lg[r]; if (r != win && v > second) second = v; }
    #pragma unroll
    for (int o = 16; o; o >>= 1) second = fmaxf(second, __shfl_xor_sync(0xffffffffu, second, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = second;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++) second = fmaxf(second, red[w]);
        const unsigned fb = __float_as_uint(second), ord = (fb & 0x80000000u) ? ~fb : (fb | 0x80000000u);
        atomicMax(key + m, (unsigned long long)ord << 32);
        __threadfence();
        if (atomicAdd(cnt + m, 1u) == gridDim.x - 1) {
            __threadfence();
            const unsigned o2 = (unsigned)(atomicExch(key + m, 0ull) >> 32);
            const float sec = __uint_as_float((o2 & 0x80000000u) ? (o2 & 0x7fffffffu) : ~o2);
            const float best = (win >= 0 && win < V) ? lg[win] : -INFINITY;
            margins[m] = __fsub_rn(best == best ? best : INFINITY, sec);     // (a NaN in row 0 wins like +inf, as in the single-token step)
            cnt[m] = 0;
        }
    }
}

size_t attn_smem_bytes(int HD, int G) {
    return ((size_t)DNW * G * (HD + 2) * 8 + (size_t)DNW * 32 * G * 8 + (size_t)G * (HD + 16) * 8 + 127) / 128 * 128;
}

template <bool QNAT>
int launch_attention(mi_ctx* ctx, const DecodeParams& P, int HD, int G, int grid, int M, int l, const int* pos0_dev, int pos0, long long q_stride,
                     const int* pos_arr = nullptr, const int* slot_arr = nullptr, long long slab_stride = 0) {
    void (*kern)(DecodeParams, int, const int*, int, long long, const int*, const int*, long long) = nullptr;
    #define MI_PICK(hd, g) if (HD == hd && G == g) kern = vf_attention<hd, g, QNAT>;
    MI_PICK(32, 2) MI_PICK(64, 2) MI_PICK(64, 7) MI_PICK(128, 6) MI_PICK(128, 8)
    #undef MI_PICK
    if (!kern) return set_error(ctx, MI_ERR_UNSUPPORTED, "attention: head_dim %d with %d query heads per kv head is not instantiated", HD, G);
    const size_t smem = attn_smem_bytes(HD, G);
    MI_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MI_CUDA(ctx, launch_k(ctx->pdl, kern, dim3(grid, M), dim3(DNT), smem, ctx->stream, P, l, pos0_dev, pos0, q_stride, pos_arr, slot_arr, slab_stride));
    return MI_OK;
}

int ensure_bufs(mi_ctx* ctx, mi_model* m) {
    VerifyBufs& b = m->vb;
    if (b.cap >= VMAX) return MI_OK;
    const int M = VMAX, E = m->E, FF = m->FF, NQ = m->NH * m->HD, qr = (m->qkv_rows + 31) / 32 * 32;
    const size_t ymax = std::max<size_t>({(size_t)qr, (size_t)2 * FF, (size_t)E});
    int st;
    if ((st = dev_alloc(ctx, m, &b.X, (size_t)M * E)) || (st = dev_alloc(ctx, m, &b.Y, (size_t)M * ymax)) ||
        (st = dev_alloc(ctx, m, &b.qkv, (size_t)M * qr)) ||
        (st = dev_alloc(ctx, m, &b.xq, (size_t)M * E)) || (st = dev_alloc(ctx, m, &b.xd, (size_t)M * E / 32)) ||
        (st = dev_alloc(ctx, m, &b.att, (size_t)M * NQ)) || (st = dev_alloc(ctx, m, &b.att_q, (size_t)M * NQ)) ||
        (st = dev_alloc(ctx, m, &b.att_d, (size_t)M * NQ / 32)) ||
        (st = dev_alloc(ctx, m, &b.act_q, (size_t)M * FF)) || (st = dev_alloc(ctx, m, &b.act_d, (size_t)M * FF / 32)) ||
        (st = dev_alloc(ctx, m, &b.logits, (size_t)M * m->V)) ||
        (st = dev_alloc(ctx, m, &b.tokens, (size_t)M + 1)) || (st = dev_alloc(ctx, m, &b.out, (size_t)M)) ||
        (st = dev_alloc(ctx, m, &b.attn_part, (size_t)M * m->NH * m->max_chunks * (m->HD + 2))) ||
        (st = dev_alloc(ctx, m, &b.attn_cnt, (size_t)M * m->NH)) ||
        (st = dev_alloc(ctx, m, &b.amax_key, (size_t)M)) || (st = dev_alloc(ctx, m, &b.amax_cnt, (size_t)M)) ||
        (st = dev_alloc(ctx, m, &b.margins, (size_t)M)))
        return st;
    b.pos0 = b.tokens + M;            // tokens and position travel in one copy
    b.cap = M;
    return MI_OK;
}

}  // namespace

namespace {

// enqueue one pass over the tokens in b.tokens at the position in b.pos0 (both already on the device)
// regime: how many CTAs per query the attention launch needs - 0: every query sees <= 256 positions (one CTA per head),
// 1: <= 1024 (up to four chunks per head), 2: beyond (the whole grid).  Launching the full grid for eight queries of a
// short context means eight waves of CTAs that exit at once; the chunking of a query does not depend on the regime.
// (bv: the tokens are one step each of independent sequences - positions, cache slabs and the cache itself come from it)
struct BatchView { const int* pos; const int* slot; __half* kc; __half* vc; int max_seq; long long slab_stride; };

int enqueue_pass(mi_ctx* ctx, mi_model* m, int M, int regime, const BatchView* bv = nullptr) {
    VerifyBufs& b = m->vb;
    const int E = m->E, FF = m->FF, L = m->L, V = m->V;
    DecodeParams P = m->P;
    if (bv) { P.kc = bv->kc; P.vc = bv->vc; P.max_seq = bv->max_seq; }
    const int* pos_arr = bv ? bv->pos : nullptr; const int* slot_arr = bv ? bv->slot : nullptr;
    const long long slab_stride = bv ? bv->slab_stride : 0;
    P.qkv_out = b.qkv; P.att = b.att; P.att_q = b.att_q; P.att_d = b.att_d; P.attn_part = b.attn_part; P.attn_cnt = b.attn_cnt;
    P.prof = nullptr;
    const std::vector<LayerPtrs>& lp = m->layer_ptrs;
    const size_t nsm = (size_t)E * 4;
    const int attn_grid = regime == 0 ? std::min(m->grid, m->NH) : regime == 1 ? std::min(m->grid, m->NH * (kPerHeadAttnMax / 256)) : m->grid;
    int st;
    // every launch of the pass may overlap its predecessor's tail (each kernel waits before touching shared data);
    // MINFER_VERIFY_PDL=0 restores plain stream order
    static const bool use_pdl = [] { const char* e = getenv("MINFER_VERIFY_PDL"); return !(e && atoi(e) == 0); }();
    const bool pdl = use_pdl;
    struct PdlScope { mi_ctx* c; bool old; ~PdlScope() { c->pdl = old; } } scope{ctx, ctx->pdl};
    ctx->pdl = pdl;
    if (nsm > 48 * 1024) MI_CUDA(ctx, cudaFuncSetAttribute(vf_norm_quant, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)nsm));
    for (int l = 0; l < L; l++) {
        const mi_weight *wqkv = &m->views[4 * l], *wo = &m->views[4 * l + 1], *wgu = &m->views[4 * l + 2], *wdn = &m->views[4 * l + 3];
        MI_CUDA(ctx, launch_k(pdl, vf_norm_quant, dim3(M), dim3(DNT), nsm, ctx->stream, P, (const int*)b.tokens, l == 0, b.X,
                              (const float*)(l == 0 ? nullptr : b.Y), E, lp[l].attn_norm, b.xq, b.xd));
        // the GEMM packs its output at the matrix's own row count: y[m * rows + r]
        if ((st = mi_gemm_q4_q8(ctx, wqkv, b.xq, reinterpret_cast<const uint16_t*>(b.xd), M, lp[l].bqkv, b.qkv))) return st;
        MI_CUDA(ctx, launch_k(pdl, vf_rope_kv, dim3(M), dim3(DNT), 0, ctx->stream, P, l, (const int*)b.pos0, b.qkv, (int)wqkv->rows, pos_arr, slot_arr,
                              slab_stride));
        if ((st = launch_attention<false>(ctx, P, m->HD, m->G, attn_grid, M, l, b.pos0, 0, wqkv->rows, pos_arr, slot_arr, slab_stride))) return st;
        if ((st = mi_gemm_q4_q8(ctx, wo, b.att_q, reinterpret_cast<const uint16_t*>(b.att_d), M, nullptr, b.Y))) return st;
        MI_CUDA(ctx, launch_k(pdl, vf_norm_quant, dim3(M), dim3(DNT), nsm, ctx->stream, P, (const int*)b.tokens, false, b.X, (const float*)b.Y, E,
                              lp[l].ffn_norm, b.xq, b.xd));
        if ((st = mi_gemm_q4_q8(ctx, wgu, b.xq, reinterpret_cast<const uint16_t*>(b.xd), M, nullptr, b.Y))) return st;
        MI_CUDA(ctx, launch_k(pdl, vf_swiglu_quant, dim3((FF / 32 + DNW - 1) / DNW, M), dim3(DNT), 0, ctx->stream, (const float*)b.Y, FF, b.act_q, b.act_d));
        if ((st = mi_gemm_q4_q8(ctx, wdn, b.act_q, reinterpret_cast<const uint16_t*>(b.act_d), M, nullptr, b.Y))) return st;
    }
    MI_CUDA(ctx, launch_k(pdl, vf_norm_quant, dim3(M), dim3(DNT), nsm, ctx->stream, P, (const int*)b.tokens, false, b.X, (const float*)b.Y, E,
                          m->P.out_norm, b.xq, b.xd));
    if ((st = mi_gemm_q4_q8(ctx, &m->views[4 * L], b.xq, reinterpret_cast<const uint16_t*>(b.xd), M, nullptr, b.logits))) return st;
    MI_CUDA(ctx, launch_k(pdl, vf_argmax, dim3(kArgmaxSlices, M), dim3(512), 0, ctx->stream, (const float*)b.logits, (long long)V, V, b.out,
                          b.amax_key, b.amax_cnt));
    MI_CUDA(ctx, launch_k(pdl, vf_margin, dim3(kArgmaxSlices, M), dim3(512), 0, ctx->stream, (const float*)b.logits, (long long)V, V, (const int*)b.out, b.margins,
                          b.amax_key, b.amax_cnt));
    return MI_OK;
}

// The pass as a CUDA graph per M: the launch sequence (about nine kernels per layer) is fixed
// once tokens and position live on the device.  A graph is built on the second call with a
// given M - the first one runs plainly and lets the GEMM grow its scratch - and rebuilt if
// that scratch has moved since.  Streams that cannot capture (the legacy default stream) and
// MINFER_VERIFY_GRAPH=0 run plainly.
int run_pass(mi_ctx* ctx, mi_model* m, int M, int regime) {
    VerifyBufs& b = m->vb;
    static const bool use_graph = [] { const char* e = getenv("MINFER_VERIFY_GRAPH"); return !(e && atoi(e) == 0); }();
    const bool capturable = ctx->stream != nullptr && ctx->stream != cudaStreamLegacy && ctx->stream != cudaStreamPerThread;
    if (!use_graph || !capturable) return enqueue_pass(ctx, m, M, regime);
    const int key = M + 17 * regime;
    if (b.graph[key] && (b.graph_part[key] != (const void*)ctx->part || b.graph_cnt[key] != (const void*)ctx->counters)) {
        cudaGraphExecDestroy((cudaGraphExec_t)b.graph[key]);      // the GEMM scratch it points into has been reallocated since
        b.graph[key] = nullptr;
    }
    if (!b.graph[key]) {
        if (!b.warm[key]) { b.warm[key] = true; return enqueue_pass(ctx, m, M, regime); }
        cudaGraph_t g = nullptr;
        MI_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        const int st = enqueue_pass(ctx, m, M, regime);
        const cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
        if (st != MI_OK) { if (g) cudaGraphDestroy(g); return st; }
        if (e != cudaSuccess) return set_error(ctx, MI_ERR_CUDA, "verify: stream capture failed: %s", cudaGetErrorString(e));
        cudaGraphExec_t ge = nullptr;
        const cudaError_t e2 = cudaGraphInstantiate(&ge, g, 0);
        cudaGraphDestroy(g);
        if (e2 != cudaSuccess) return set_error(ctx, MI_ERR_CUDA, "verify: graph instantiation failed: %s", cudaGetErrorString(e2));
        b.graph[key] = ge; b.graph_part[key] = ctx->part; b.graph_cnt[key] = ctx->counters;
    }
    MI_CUDA(ctx, cudaGraphLaunch((cudaGraphExec_t)b.graph[key], ctx->stream));
    return MI_OK;
}

}  // namespace

extern "C" int mi_verify(mi_ctx* ctx, mi_model* m, const int32_t* tokens_host, int M, int pos0, int32_t* out_tokens_host,
                         float* logits_dev, float* elapsed_ms) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m || !tokens_host) return set_error(ctx, MI_ERR_INVALID, "verify: null argument");
    if (M < 1 || M > VMAX) return set_error(ctx, MI_ERR_LIMIT, "verify: M=%d tokens per pass; this entry point takes 1..%d", M, VMAX);
    if (pos0 < 0 || pos0 + M > m->max_seq)
        return set_error(ctx, MI_ERR_LIMIT, "verify: positions %d..%d exceed the KV cache of %d", pos0, pos0 + M - 1, m->max_seq);
    if (m->tp_world != 1) return set_error(ctx, MI_ERR_UNSUPPORTED, "verify: the M-token step runs on an unsharded model");
    for (int i = 0; i < M; i++)
        if (tokens_host[i] < 0 || tokens_host[i] >= m->V) return set_error(ctx, MI_ERR_INVALID, "verify: token id %d out of range", tokens_host[i]);
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    int st;
    if ((st = ensure_bufs(ctx, m))) return st;
    VerifyBufs& b = m->vb;
    int32_t head[VMAX + 1] = {};
    for (int i = 0; i < M; i++) head[i] = tokens_host[i];
    head[VMAX] = pos0;
    MI_CUDA(ctx, cudaMemcpyAsync(b.tokens, head, sizeof(head), cudaMemcpyHostToDevice, ctx->stream));   // pageable source: staged before the call returns
    MI_CUDA(ctx, cudaEventRecord(m->ev0, ctx->stream));
    const int lp_max = pos0 + M, regime = lp_max <= 256 ? 0 : lp_max <= kPerHeadAttnMax ? 1 : 2;
    if ((st = run_pass(ctx, m, M, regime))) return st;
    MI_CUDA(ctx, cudaEventRecord(m->ev1, ctx->stream));
    if (logits_dev) MI_CUDA(ctx, cudaMemcpyAsync(logits_dev, b.logits, (size_t)M * m->V * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    if (out_tokens_host) MI_CUDA(ctx, cudaMemcpyAsync(out_tokens_host, b.out, (size_t)M * 4, cudaMemcpyDeviceToHost, ctx->stream));
    // the single-token loop continues from the last scored token's pick
    MI_CUDA(ctx, cudaMemcpyAsync(m->P.cur_token, b.out + (M - 1), 4, cudaMemcpyDeviceToDevice, ctx->stream));
    st = mi_ctx_sync(ctx);
    if (st != MI_OK) return st;
    if (elapsed_ms) MI_CUDA(ctx, cudaEventElapsedTime(elapsed_ms, m->ev0, m->ev1));
    return MI_OK;
}

extern "C" int mi_verify_margins(mi_ctx* ctx, mi_model* m, int n, float* margins_host) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m || !margins_host || n < 0 || n > VMAX || !m->vb.margins) return set_error(ctx, MI_ERR_INVALID, "verify_margins: bad argument, or no M-token pass has run");
    if (n == 0) return MI_OK;
    MI_CUDA(ctx, cudaMemcpyAsync(margins_host, m->vb.margins, (size_t)n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MI_OK;
}

extern "C" int mi_attn_splitkv(mi_ctx* ctx, const float* q_dev, const uint16_t* kcache_dev, const uint16_t* vcache_dev, int n_head,
                               int n_head_kv, int head_dim, int pos0, int M, float* out_dev) {
    if (!ctx) return MI_ERR_INVALID;
    if (!q_dev || !kcache_dev || !vcache_dev || !out_dev) return set_error(ctx, MI_ERR_INVALID, "attention: null argument");
    if (M < 1 || M > VMAX) return set_error(ctx, MI_ERR_LIMIT, "attention: M=%d queries per call; this entry point takes 1..%d", M, VMAX);
    if (n_head <= 0 || n_head_kv <= 0 || n_head % n_head_kv || pos0 < 0) return set_error(ctx, MI_ERR_INVALID, "attention: bad head counts or position");
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    const int G = n_head / n_head_kv, grid = ctx->sm_count, max_chunks = std::max(1, grid / n_head_kv), NQ = n_head * head_dim;
    // scratch: chunk partials as doubles, the q8_0 by-products of the decode path (unused here), arrival counters
    const size_t part = (size_t)M * n_head * max_chunks * (head_dim + 2);
    const size_t extra = ((size_t)M * NQ + (size_t)M * NQ / 32 * 2 + 7) / 8 + 1;        // in doubles
    int st = ensure_scratch(ctx, part + extra, (size_t)M * n_head);
    if (st != MI_OK) return st;
    DecodeParams P{};
    P.NH = n_head; P.NKV = n_head_kv; P.HD = head_dim; P.KVD = n_head_kv * head_dim;
    P.qkv_out = const_cast<float*>(q_dev);
    P.kc = reinterpret_cast<__half*>(const_cast<uint16_t*>(kcache_dev)); P.vc = reinterpret_cast<__half*>(const_cast<uint16_t*>(vcache_dev));
    P.max_seq = 0;                        // one layer: the layer index never moves the base
    P.max_chunks = max_chunks;
    P.att = out_dev;
    P.attn_part = ctx->part; P.attn_cnt = ctx->counters;
    P.att_q = reinterpret_cast<int8_t*>(ctx->part + part);
    P.att_d = reinterpret_cast<__half*>(reinterpret_cast<int8_t*>(ctx->part + part) + (size_t)M * NQ);
    P.err = ctx->d_err;
    // CTAs per query that the longest causal range of the call can use (the chunking of a query does not depend on it)
    const int lp_max = pos0 + M;
    const int agrid = lp_max <= 256 ? std::min(grid, n_head) : lp_max <= kPerHeadAttnMax ? std::min(grid, n_head * (kPerHeadAttnMax / 256)) : grid;
    return launch_attention<true>(ctx, P, head_dim, G, agrid, M, 0, nullptr, pos0, NQ);
}


// ---- batched decode of independent sequences -------------------------------------------------------------
// One step of up to B sequences per call: the current token of each goes through ONE pass over the weights as a column
// of the M-token step (sixteen columns per pass; larger batches run several passes), with its own position and its
// own slab of a KV cache that belongs to the batch object.  Every column is processed exactly as if it were alone, so
// a sequence's ids and logits are the bits of its batch-1 run, whatever else shares the pass.  The reference serves one
// sequence at a time (README.md:54); the closest code is gemv_dp4a_batch<T> (src/cuda_infer.cu:183-222).
struct mi_batch {
    mi_model* model = nullptr;
    int n_slots = 0, max_seq = 0;
    __half* kc = nullptr; __half* vc = nullptr;       // [slot][layer][max_seq][KVD]
    int* d_meta = nullptr;                              // [3][16]: tokens, positions, slots of the running pass
    long long slab_stride = 0;
};

extern "C" int mi_batch_create(mi_ctx* ctx, mi_model* m, int n_slots, int max_seq, mi_batch** out) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m || !out || n_slots < 1 || max_seq < 1) return set_error(ctx, MI_ERR_INVALID, "batch_create: bad argument");
    if (m->tp_world != 1) return set_error(ctx, MI_ERR_UNSUPPORTED, "batch_create: the M-token step runs on an unsharded model");
    *out = nullptr;
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    mi_batch* b = new (std::nothrow) mi_batch();
    if (!b) return set_error(ctx, MI_ERR_NOMEM, "batch_create: host allocation failed");
    b->model = m; b->n_slots = n_slots; b->max_seq = max_seq;
    b->slab_stride = (long long)m->L * max_seq * m->KVD;
    const size_t bytes = (size_t)n_slots * (size_t)b->slab_stride * sizeof(__half);
    if (cudaMalloc(&b->kc, bytes) != cudaSuccess || cudaMalloc(&b->vc, bytes) != cudaSuccess || cudaMalloc(&b->d_meta, 3 * 16 * sizeof(int)) != cudaSuccess) {
        cudaFree(b->kc); cudaFree(b->vc); cudaFree(b->d_meta); delete b;
        return set_error(ctx, MI_ERR_NOMEM, "batch_create: %d KV slabs of %zu bytes do not fit", n_slots, bytes / n_slots);
    }
    *out = b;
    return MI_OK;
}

extern "C" int mi_batch_free(mi_ctx* ctx, mi_batch* b) {
    if (!b) return MI_OK;
    if (ctx) { cudaSetDevice(ctx->device); cudaStreamSynchronize(ctx->stream); }
    cudaFree(b->kc); cudaFree(b->vc); cudaFree(b->d_meta);
    delete b;
    return MI_OK;
}

extern "C" int mi_batch_step(mi_ctx* ctx, mi_batch* b, int n, const int32_t* tokens_host, const int32_t* slots_host, const int32_t* positions_host,
                             int32_t* out_tokens_host, float* logits_dev, float* elapsed_ms) {
    if (!ctx) return MI_ERR_INVALID;
    if (!b || !tokens_host || !slots_host || !positions_host || n < 1) return set_error(ctx, MI_ERR_INVALID, "batch_step: bad argument");
    mi_model* m = b->model;
    for (int i = 0; i < n; i++) {
        if (tokens_host[i] < 0 || tokens_host[i] >= m->V) return set_error(ctx, MI_ERR_INVALID, "batch_step: token id %d out of range", tokens_host[i]);
        if (slots_host[i] < 0 || slots_host[i] >= b->n_slots) return set_error(ctx, MI_ERR_INVALID, "batch_step: slot %d of %d", slots_host[i], b->n_slots);
        if (positions_host[i] < 0 || positions_host[i] >= b->max_seq)
            return set_error(ctx, MI_ERR_LIMIT, "batch_step: position %d outside the KV slab of %d", positions_host[i], b->max_seq);
        for (int j = 0; j < i; j++)
            if (slots_host[j] == slots_host[i]) return set_error(ctx, MI_ERR_INVALID, "batch_step: slot %d appears twice in one step", slots_host[i]);
    }
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    int st;
    if ((st = ensure_bufs(ctx, m))) return st;
    VerifyBufs& vb = m->vb;
    MI_CUDA(ctx, cudaEventRecord(m->ev0, ctx->stream));
    for (int i0 = 0; i0 < n; i0 += VMAX) {
        const int M = std::min(VMAX, n - i0);
        int32_t meta[3 * 16] = {};
        int lp_max = 0;
        for (int i = 0; i < M; i++) {
            meta[i] = tokens_host[i0 + i]; meta[16 + i] = positions_host[i0 + i]; meta[32 + i] = slots_host[i0 + i];
            lp_max = std::max(lp_max, positions_host[i0 + i] + 1);
        }
        MI_CUDA(ctx, cudaMemcpyAsync(b->d_meta, meta, sizeof meta, cudaMemcpyHostToDevice, ctx->stream));
        MI_CUDA(ctx, cudaMemcpyAsync(vb.tokens, b->d_meta, (size_t)M * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        const BatchView bv{b->d_meta + 16, b->d_meta + 32, b->kc, b->vc, b->max_seq, b->slab_stride};
        const int regime = lp_max <= 256 ? 0 : lp_max <= kPerHeadAttnMax ? 1 : 2;
        if ((st = enqueue_pass(ctx, m, M, regime, &bv))) return st;
        if (logits_dev) MI_CUDA(ctx, cudaMemcpyAsync(logits_dev + (size_t)i0 * m->V, vb.logits, (size_t)M * m->V * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        if (out_tokens_host) MI_CUDA(ctx, cudaMemcpyAsync(out_tokens_host + i0, vb.out, (size_t)M * 4, cudaMemcpyDeviceToHost, ctx->stream));
        if (i0 + VMAX < n) MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));       // the pageable meta block is reused by the next pass
    }
    MI_CUDA(ctx, cudaEventRecord(m->ev1, ctx->stream));
    st = mi_ctx_sync(ctx);
    if (st != MI_OK) return st;
    if (elapsed_ms) MI_CUDA(ctx, cudaEventElapsedTime(elapsed_ms, m->ev0, m->ev1));
    return MI_OK;
}
