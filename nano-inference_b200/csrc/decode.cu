// Model loading (GGUF -> tiled device layout), job planning and launching of the
// fused decode kernel; the model / decode part of the C ABI.
#include "model.cuh"
#include "gguf_file.hpp"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <vector>

using namespace mi;

namespace mi {
const void* decode_kernel_prof(int HD, int G); const void* decode_kernel_tp(int HD, int G); const void* decode_kernel_lean(int HD, int G);
const void* decode_kernel_prof_lean(int HD, int G);
const void* decode_kernel_tp_lean(int HD, int G);
const void* decode_kernel_tp_prof_lean(int HD, int G);
const void* decode_kernel_lean_mid(int HD, int G);
const void* decode_kernel_lean_long(int HD, int G);
int reset_after_error(mi_ctx* ctx, mi_model* m);
}

namespace {

struct Staging {       // one reusable device buffer for raw GGUF bytes, one for re-quantized q4_0 rows
    void* d = nullptr; size_t cap = 0;
    void* q = nullptr; size_t qcap = 0;
    ~Staging() { if (d) cudaFree(d); if (q) cudaFree(q); }
    int room_q(mi_ctx* ctx, size_t n) {                   // call after put(): the stream has drained, nothing reads q any more
        if (n <= qcap) return MI_OK;
        if (q) { cudaFree(q); q = nullptr; qcap = 0; }
        if (cudaMalloc(&q, n) != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "model: staging cudaMalloc(%zu) failed", n);
        qcap = n;
        return MI_OK;
    }
    int put(mi_ctx* ctx, const void* src, size_t n) {
        if (n > cap) {
            if (d) { cudaStreamSynchronize(ctx->stream); cudaFree(d); d = nullptr; cap = 0; }
            cudaError_t e = cudaMalloc(&d, n);
            if (e != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "model: staging cudaMalloc(%zu) failed", n);
            cap = n;
        }
        // the previous repack (same stream) must be done with the buffer before it is overwritten
        MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        MI_CUDA(ctx, cudaMemcpy(d, src, n, cudaMemcpyHostToDevice));
        MI_CUDA(ctx, cudaStreamSynchronize(cudaStreamLegacy));        // a pageable copy may return before its last DMA has landed
        return MI_OK;
    }
};

// A weight matrix asked for as GGML_Q4_0 may also be stored as Q4_1, Q8_0 or Q6_K: the loader re-quantizes those to q4_0.
const mib200::GgufTensor* need(mi_ctx* ctx, const mib200::GgufFile& g, const std::string& name, uint32_t type,
                               int64_t cols, int64_t rows, int* st) {
    const mib200::GgufTensor* t = g.find(name);
    if (!t) { *st = set_error(ctx, MI_ERR_FORMAT, "model: tensor not found: %s", name.c_str()); return nullptr; }
    const bool requant = type == mib200::GGML_Q4_0 && (t->type == mib200::GGML_Q4_1 || t->type == mib200::GGML_Q8_0 ||
                                                       (t->type == mib200::GGML_Q6_K && cols % 256 == 0));
    if (t->type != type && !requant) {
        *st = set_error(ctx, MI_ERR_UNSUPPORTED, "model: tensor %s has ggml type %u, this path takes %s only", name.c_str(), t->type,
                        type == mib200::GGML_Q4_0 ? "Q4_0, Q4_1, Q8_0 or Q6_K" : "F32");
        return nullptr;
    }
    if (t->cols() != cols || t->rows() != rows) {
        *st = set_error(ctx, MI_ERR_FORMAT, "model: tensor %s is %lld x %lld, expected %lld x %lld", name.c_str(),
                        (long long)t->rows(), (long long)t->cols(), (long long)rows, (long long)cols);
        return nullptr;
    }
    return t;
}

// Tiled buffer for `rows` packed rows of `cols` columns, zero-filled.
int alloc_tiled(mi_ctx* ctx, mi_model* m, int64_t rows, int64_t cols, uint8_t** out, int* kb_out, int* nt_out) {
    const int nb = (int)(cols / 32), kb = choose_kb(nb), nt = nb / kb;
    const size_t groups = (size_t)((rows + 31) / 32);
    *kb_out = kb; *nt_out = nt;
    return dev_alloc(ctx, m, out, groups * nt * tile_bytes(kb), true);
}

// Cross-CTA K-split of a per-layer job.  A job whose result feeds an in-phase epilogue
// (QKV: bias + RoPE; gate/up: SwiGLU + q8_0) is never split across CTAs: its eight warps
// already share every unit, and so is the O projection (measured: 6 tiles per row group, one
// per warp, gains nothing from a split).  The down projection (35 tiles per row group at the
// 1.5B shape, 48 row groups for 148 CTAs) is split until every CTA has a unit; the CTA of
// split 0 collects the other splits' partial sums (see run_cta_job).
int plan_ks(int kind, int groups, int nt, int grid) {
    if (kind != JOB_DOWN) return 1;
    int ks = grid / std::max(groups, 1);
    return std::max(1, std::min(std::min(ks, nt), kMaxKSplit));
}

// cos and sin of the rotary angles of every position: angle = fp32(pos * freq) as src/cpu_infer.cpp:54, then the double
// cosine / sine rounded to fp32 once (the products of the rotation are formed in double by the QKV epilogue)
__global__ void rope_cs_kernel(const float* __restrict__ freq, float* __restrict__ cs, int HD, int max_seq) {
    const int pos = blockIdx.x, i = threadIdx.x;
    if (pos >= max_seq || i >= HD / 2) return;
    const double th = (double)__fmul_rn((float)pos, freq[i]);
    cs[(size_t)pos * HD + i] = __double2float_rn(cos(th));
    cs[(size_t)pos * HD + HD / 2 + i] = __double2float_rn(sin(th));
}

// range_hint 1 / 2 / 3: the caller vouches that every position of the launch lies in that context range (up to kShortAttnMax,
// up to kPerHeadAttnMax, beyond) although the position is device-resident; 0: decided from pos0 and the steps.  (A build
// launched outside its range ends with MI_ERR_LIMIT on every CTA, it computes nothing wrong.)  only_prepare: pick the
// kernel and raise its shared-memory limit, launch nothing (what must not happen inside a stream capture).
int dispatch_launch(mi_ctx* ctx, mi_model* m, const DecodeParams& P, int step0, int step1, int ph0, int ph1, bool coop, int range_hint = 0,
                    bool only_prepare = false) {
    void (*kern)(DecodeParams, int, int, int, int) = nullptr;
    // every step of this launch ends within the range the dedicated attention CTAs handle, on a shape the short-context
    // build takes: that build has no other attention variant in it (decode_lean.cu)
    const bool shape_ok = lean_shape_ok(m->E, m->FF, m->NH * m->HD) && !getenv("MINFER_NO_LEAN");
    const bool by_pos = !P.pos_dev && range_hint == 0;
    const bool lean = m->attn_ctas > 0 && shape_ok && (range_hint == 1 || (by_pos && (long long)P.pos0 + step1 <= kShortAttnMax));
    auto as_kernel = [](const void* p) { return reinterpret_cast<void (*)(DecodeParams, int, int, int, int)>(const_cast<void*>(p)); };
    // the context-range builds are instantiated for the head shapes that occur with the embedding widths they take; a
    // null pointer from their pickers means "not built for this head shape": the general build of the same family runs
    const bool mid = shape_ok && (range_hint == 2 || (by_pos && (long long)P.pos0 + step0 + 1 > kShortAttnMax && (long long)P.pos0 + step1 <= kPerHeadAttnMax));
    const bool far = shape_ok && (range_hint == 3 || (by_pos && (long long)P.pos0 + step0 + 1 > kPerHeadAttnMax));
    const void* pick = nullptr;
    if (P.tp.on) {                                  // the builds with the exchange between GPUs inside (decode_tp.cu, decode_tp_lean.cu)
        if (lean && P.prof) pick = decode_kernel_tp_prof_lean(m->HD, m->G);
        if (lean && !pick) pick = decode_kernel_tp_lean(m->HD, m->G);
        if (!pick) pick = decode_kernel_tp(m->HD, m->G);
    } else if (P.prof) {                            // the instrumented builds (decode_prof.cu, decode_prof_lean.cu)
        if (lean) pick = decode_kernel_prof_lean(m->HD, m->G);
        if (!pick) pick = decode_kernel_prof(m->HD, m->G);
    } else {
        if (lean) pick = decode_kernel_lean(m->HD, m->G);
        else if (mid) pick = decode_kernel_lean_mid(m->HD, m->G);
        else if (far) pick = decode_kernel_lean_long(m->HD, m->G);
    }
    if (pick) kern = as_kernel(pick);
    else {
        #define MI_PICK(hd, g) if (m->HD == hd && m->G == g) kern = decode_kernel<hd, g>;
        MI_PICK(32, 2) MI_PICK(64, 2) MI_PICK(64, 7) MI_PICK(128, 6) MI_PICK(128, 8)
        #undef MI_PICK
    }
    if (!kern) return set_error(ctx, MI_ERR_UNSUPPORTED, "decode: head_dim %d with %d query heads per kv head is not instantiated", m->HD, m->G);
    // the opt-in shared-memory size is a property of (device, kernel): raise it whenever this model needs more than any before
    {
        static std::mutex mu;
        static std::map<std::pair<int, const void*>, size_t> raised;
        std::lock_guard<std::mutex> lock(mu);
        size_t& have = raised[{ctx->device, (const void*)kern}];
        if (have < m->smem) {
            MI_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)m->smem));
            have = m->smem;
        }
    }
    // Always a cooperative launch: CTAs wait for one another's tagged words inside every phase range (the K-split fold
    // of the down projection, the greedy pick over all CTAs' candidates), so all of them must be resident together.
    (void)coop;
    if (only_prepare) return MI_OK;
    void* args[] = {(void*)&P, &step0, &step1, &ph0, &ph1};
    MI_CUDA(ctx, cudaLaunchCooperativeKernel((const void*)kern, dim3(m->grid), dim3(DNT), args, m->smem, ctx->stream));
    return MI_OK;
}

}  // namespace

extern "C" int mi_model_free(mi_ctx* ctx, mi_model* m) {
    (void)ctx;
    if (!m) return MI_OK;
    cudaSetDevice(m->device);
    cudaDeviceSynchronize();
    for (void* p : m->ipc_opened) cudaIpcCloseMemHandle(p);
    for (void* p : m->allocs) cudaFree(p);
    for (void* g : m->vb.graph) if (g) cudaGraphExecDestroy((cudaGraphExec_t)g);
    for (void* g : m->step_graph) if (g) cudaGraphExecDestroy((cudaGraphExec_t)g);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    delete m;
    return MI_OK;
}

extern "C" void mi_tp_partition(int groups, int rank, int world, int* begin, int* end) {
    if (world < 1) world = 1;
    if (begin) *begin = (int)((long long)groups * rank / world);
    if (end) *end = (int)((long long)groups * (rank + 1) / world);
}

extern "C" int mi_model_load_gguf(mi_ctx* ctx, const char* path, int max_seq, mi_model** out) {
    return mi_model_load_gguf_tp(ctx, path, max_seq, 0, 1, out);
}

extern "C" int mi_model_load_gguf_tp(mi_ctx* ctx, const char* path, int max_seq, int tp_rank, int tp_world, mi_model** out) {
    if (!ctx) return MI_ERR_INVALID;
    if (!out || !path) return set_error(ctx, MI_ERR_INVALID, "model: null argument");
    *out = nullptr;
    if (max_seq <= 0) return set_error(ctx, MI_ERR_INVALID, "model: max_seq must be positive");
    if (tp_world < 1 || tp_rank < 0 || tp_rank >= tp_world) return set_error(ctx, MI_ERR_INVALID, "model: bad tensor-parallel rank %d of %d", tp_rank, tp_world);
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    mib200::GgufFile g;
    std::string err = g.open(path);
    if (!err.empty()) {
        const bool io = err.rfind("cannot", 0) == 0 || err.rfind("mmap", 0) == 0;
        return set_error(ctx, io ? MI_ERR_IO : MI_ERR_FORMAT, "model: %s", err.c_str());
    }
    mi_model* m = new (std::nothrow) mi_model();
    if (!m) return set_error(ctx, MI_ERR_NOMEM, "model: host allocation failed");
    struct Guard { mi_ctx* c; mi_model* m; bool keep = false; ~Guard() { if (!keep) mi_model_free(c, m); } } guard{ctx, m};
    m->device = ctx->device; m->tp_rank = tp_rank; m->tp_world = tp_world;
    // hyper-parameters: the keys the reference drivers read (src/cpu_infer.cpp:71-79)
    m->L = (int)g.num("qwen2.block_count", 0);
    m->E = (int)g.num("qwen2.embedding_length", 0);
    m->FF = (int)g.num("qwen2.feed_forward_length", 0);
    m->NH = (int)g.num("qwen2.attention.head_count", 0);
    m->NKV = (int)g.num("qwen2.attention.head_count_kv", 0);
    m->rope_base = (float)g.num("qwen2.rope.freq_base", 1e6);
    m->eps = (float)g.num("qwen2.attention.layer_norm_rms_epsilon", 1e-6);
    m->V = (int)g.n_tokens();
    if (m->L <= 0 || m->E <= 0 || m->FF <= 0 || m->NH <= 0 || m->NKV <= 0 || m->V <= 0)
        return set_error(ctx, MI_ERR_FORMAT, "model: missing qwen2.* metadata or tokenizer.ggml.tokens");
    if (m->E % m->NH || m->NH % m->NKV) return set_error(ctx, MI_ERR_FORMAT, "model: head counts do not divide");
    m->HD = m->E / m->NH; m->KVD = m->NKV * m->HD; m->G = m->NH / m->NKV;
    if (m->E % 32 || m->FF % 32 || m->HD % 32 || m->HD > 128 || m->G > DNW || m->L > 64 || m->E > 8192 || m->FF > 32768)
        return set_error(ctx, MI_ERR_UNSUPPORTED, "model: shape outside this path (E, FF, head_dim multiples of 32; <= 8 query heads per kv head)");
    m->max_seq = max_seq;
    m->grid = ctx->sm_count;
    if (const char* gs = getenv("MINFER_GRID")) { int v = atoi(gs); if (v > 0 && v <= ctx->sm_count) m->grid = v; }
    m->max_chunks = std::max(1, m->grid / m->NKV);
    // CTAs set aside for attention (see DecodeParams::attn_ctas): one per query head, where the grid is large enough to spare them
    {
        const int hpc = attn_heads_per_cta(m->G);
        m->attn_ctas = (m->NH / hpc * 8 <= m->grid && attn_dedicated_smem(m->HD, hpc) + 1024 <= (size_t)ctx->smem_optin) ? m->NH / hpc : 0;
        if (const char* ac = getenv("MINFER_ATTN_CTAS")) { int v = atoi(ac); if (v == 0) m->attn_ctas = 0; }
    }
    const int GG = m->grid - m->attn_ctas;                // CTAs that carry GEMV units

    const int E = m->E, FF = m->FF, HD = m->HD, KVD = m->KVD, L = m->L, V = m->V, NQ = m->NH * m->HD;
    int st = MI_OK;
    Staging stg;
    DecodeParams& P = m->P;
    P.L = L; P.E = E; P.FF = FF; P.NH = m->NH; P.NKV = m->NKV; P.HD = HD; P.KVD = KVD; P.V = V; P.eps = m->eps;

    // ---- row maps (device): q/k rows pair-adjacent for RoPE, gate/up groups interleaved
    auto rope_map = [&](int nheads, int offset) {
        std::vector<int> mp((size_t)nheads * HD);
        for (int h = 0; h < nheads; h++)
            for (int i = 0; i < HD / 2; i++) {
                mp[(size_t)h * HD + i] = offset + h * HD + 2 * i;                 // source row (h, i)        -> even slot
                mp[(size_t)h * HD + i + HD / 2] = offset + h * HD + 2 * i + 1;   // source row (h, i + HD/2) -> odd slot
            }
        return mp;
    };
    std::vector<int> mq = rope_map(m->NH, 0), mk = rope_map(m->NKV, NQ), mg((size_t)FF), mu((size_t)FF);
    for (int r = 0; r < FF; r++) { mg[r] = (r / 32) * 64 + r % 32; mu[r] = (r / 32) * 64 + 32 + r % 32; }
    int *d_mq, *d_mk, *d_mg, *d_mu;
    if ((st = dev_alloc(ctx, m, &d_mq, mq.size())) || (st = dev_alloc(ctx, m, &d_mk, mk.size())) ||
        (st = dev_alloc(ctx, m, &d_mg, mg.size())) || (st = dev_alloc(ctx, m, &d_mu, mu.size()))) return st;
    MI_CUDA(ctx, cudaMemcpy(d_mq, mq.data(), mq.size() * 4, cudaMemcpyHostToDevice));
    MI_CUDA(ctx, cudaMemcpy(d_mk, mk.data(), mk.size() * 4, cudaMemcpyHostToDevice));
    MI_CUDA(ctx, cudaMemcpy(d_mg, mg.data(), mg.size() * 4, cudaMemcpyHostToDevice));
    MI_CUDA(ctx, cudaMemcpy(d_mu, mu.data(), mu.size() * 4, cudaMemcpyHostToDevice));

    auto upload_f32 = [&](const mib200::GgufTensor* t, float** dst, size_t padded) -> int {
        int s = dev_alloc(ctx, m, dst, padded, true);
        if (s) return s;
        MI_CUDA(ctx, cudaMemcpy(*dst, t->data, (size_t)t->cols() * 4, cudaMemcpyHostToDevice));
        return MI_OK;
    };
    auto repack = [&](const mib200::GgufTensor* t, uint8_t* dst, const int* map, int offset) -> int {
        int s = stg.put(ctx, t->data, t->nbytes());
        if (s) return s;
        const void* rows_q4 = stg.d;
        if (t->type != mib200::GGML_Q4_0) {            // stored in another block format: q4_0 rows first (requant.cu)
            if ((s = stg.room_q(ctx, (size_t)t->rows() * (t->cols() / 32) * 18))) return s;
            if ((s = launch_requant_q4_0(ctx, (int)t->type, stg.d, t->rows(), t->cols(), stg.q))) return s;
            rows_q4 = stg.q; m->requantized++;
        }
        return launch_repack_map(ctx, rows_q4, t->rows(), (int)(t->cols() / 32), choose_kb((int)(t->cols() / 32)), dst, map, offset);
    };

    // ---- embedding / lm_head
    const mib200::GgufTensor* te = need(ctx, g, "token_embd.weight", mib200::GGML_Q4_0, E, V, &st); if (!te) return st;
    const mib200::GgufTensor* tl = g.find("output.weight");            // optional: tied to the embedding when absent
    m->tied = !tl || (tl->type == te->type && tl->nbytes() == te->nbytes() && memcmp(tl->data, te->data, te->nbytes()) == 0);
    if (tl && !m->tied) { tl = need(ctx, g, "output.weight", mib200::GGML_Q4_0, E, V, &st); if (!tl) return st; }
    // The lm_head is always a tiled q4_0 matrix.  The embedding shares it when the file ties them, except that a Q8_0
    // embedding is kept as stored and read row by row (the reference's persistent engine does the same, src/mega.cu:1110-1111).
    uint8_t *d_emb = nullptr, *d_lm = nullptr; int ekb, ent;
    if ((st = alloc_tiled(ctx, m, V, E, &d_lm, &ekb, &ent))) return st;
    if ((st = repack(m->tied ? te : tl, d_lm, nullptr, 0))) return st;
    d_emb = d_lm;
    if (te->type == mib200::GGML_Q8_0) {
        uint8_t* d_e8;
        if ((st = dev_alloc(ctx, m, &d_e8, te->nbytes()))) return st;
        MI_CUDA(ctx, cudaMemcpy(d_e8, te->data, te->nbytes(), cudaMemcpyHostToDevice));
        P.emb_q8 = d_e8;
    } else if (!m->tied) {
        if ((st = alloc_tiled(ctx, m, V, E, &d_emb, &ekb, &ent))) return st;
        if ((st = repack(te, d_emb, nullptr, 0))) return st;
    }
    P.emb_base = d_emb; P.emb_kb = ekb; P.emb_nt = ent;
    const mib200::GgufTensor* tn = need(ctx, g, "output_norm.weight", mib200::GGML_F32, E, 1, &st); if (!tn) return st;
    float* d_outnorm; if ((st = upload_f32(tn, &d_outnorm, E))) return st;
    P.out_norm = d_outnorm;

    // ---- layers
    std::vector<LayerPtrs> lp(L);
    const int qkv_rows = NQ + 2 * KVD, W = GG * DNW;
    m->qkv_rows = qkv_rows;
    int rot = 0, wrot = 0;
    auto add_job = [&](const uint8_t* base, int groups, int cols, int nacc, int kind, int layer) {
        Job jb{}; jb.nb = cols / 32; jb.kb = choose_kb(jb.nb); jb.nt = jb.nb / jb.kb;
        jb.nacc = nacc; jb.kind = kind; jb.layer = layer;
        // tensor parallelism: this GPU owns a contiguous range of the job's unit groups (rows); every GPU holds the
        // whole matrix but streams only its rows.  The K-split is planned from the largest share so that all GPUs
        // lay the partial sums out identically.
        // The QKV and O projections (a tenth of a layer's bytes) are the exception: every GPU computes all their rows,
        // so that attention and the O projection need no exchange at all.
        const bool replicated = kind == JOB_QKV || kind == JOB_O;
        int g0 = 0, g1 = groups;
        if (!replicated) mi_tp_partition(groups, tp_rank, tp_world, &g0, &g1);
        jb.g_off = g0; jb.groups = g1 - g0;
        jb.base = base + (size_t)g0 * nacc * jb.nt * tile_bytes(jb.kb);
        jb.ks = plan_ks(kind, replicated ? groups : (groups + tp_world - 1) / tp_world, jb.nt, GG);
        const char* force = kind == JOB_DOWN ? getenv("MINFER_KS_DOWN") : nullptr;   // tuning knob
        if (force) jb.ks = std::max(1, std::min(std::min(atoi(force), jb.nt), kMaxKSplit));
        if (jb.ks >= GG) jb.ks = std::max(1, GG - 1);       // the CTAs of a row group's splits must be distinct
        jb.n_units = jb.groups * jb.ks;
        jb.ks_inv = (unsigned)(((1ull << 32) + (unsigned)jb.ks - 1) / (unsigned)jb.ks);    // ks == 1: 2^32 wraps to 0, and that path does not divide
        if (kind == JOB_LM) { jb.rot = 0; jb.wrot = 0; }
        else {
            // successive jobs start where the previous one stopped, over CTAs and over the warps of a CTA
            jb.rot = rot; jb.wrot = wrot;
            rot = (int)(((long long)rot + jb.n_units) % GG);
            wrot = (wrot + nacc * ((jb.nt + jb.ks - 1) / jb.ks)) & (DNW - 1);
        }
        m->jobs.push_back(jb);
        mi_weight v;                                  // the whole matrix, for the M-token step
        v.rows = (int64_t)groups * nacc * 32; v.cols = cols; v.count = 1; v.nb = jb.nb; v.kb = jb.kb; v.nt = jb.nt;
        v.groups = groups * nacc; v.mat_stride = 0; v.bytes = (size_t)v.groups * jb.nt * tile_bytes(jb.kb);
        v.dev = const_cast<uint8_t*>(base);
        m->views.push_back(v);
    };
    for (int l = 0; l < L; l++) {
        const std::string p = "blk." + std::to_string(l) + ".";
        const mib200::GgufTensor *an, *fn, *wq, *wk, *wv, *wo, *wg, *wu, *wd, *bq, *bk, *bv;
        if (!(an = need(ctx, g, p + "attn_norm.weight", mib200::GGML_F32, E, 1, &st))) return st;
        if (!(fn = need(ctx, g, p + "ffn_norm.weight", mib200::GGML_F32, E, 1, &st))) return st;
        if (!(wq = need(ctx, g, p + "attn_q.weight", mib200::GGML_Q4_0, E, NQ, &st))) return st;
        if (!(wk = need(ctx, g, p + "attn_k.weight", mib200::GGML_Q4_0, E, KVD, &st))) return st;
        if (!(wv = need(ctx, g, p + "attn_v.weight", mib200::GGML_Q4_0, E, KVD, &st))) return st;
        if (!(wo = need(ctx, g, p + "attn_output.weight", mib200::GGML_Q4_0, NQ, E, &st))) return st;
        if (!(wg = need(ctx, g, p + "ffn_gate.weight", mib200::GGML_Q4_0, E, FF, &st))) return st;
        if (!(wu = need(ctx, g, p + "ffn_up.weight", mib200::GGML_Q4_0, E, FF, &st))) return st;
        if (!(wd = need(ctx, g, p + "ffn_down.weight", mib200::GGML_Q4_0, FF, E, &st))) return st;
        if (!(bq = need(ctx, g, p + "attn_q.bias", mib200::GGML_F32, NQ, 1, &st))) return st;
        if (!(bk = need(ctx, g, p + "attn_k.bias", mib200::GGML_F32, KVD, 1, &st))) return st;
        if (!(bv = need(ctx, g, p + "attn_v.bias", mib200::GGML_F32, KVD, 1, &st))) return st;
        float *d_an, *d_fn, *d_b;
        if ((st = upload_f32(an, &d_an, E)) || (st = upload_f32(fn, &d_fn, E))) return st;
        // fused bias in packed row order
        std::vector<float> hb((size_t)(qkv_rows + 31) / 32 * 32, 0.f);
        const float *fq = (const float*)bq->data, *fk = (const float*)bk->data, *fv = (const float*)bv->data;
        for (int r = 0; r < NQ; r++) hb[mq[r]] = fq[r];
        for (int r = 0; r < KVD; r++) hb[mk[r]] = fk[r];
        for (int r = 0; r < KVD; r++) hb[NQ + KVD + r] = fv[r];
        if ((st = dev_alloc(ctx, m, &d_b, hb.size()))) return st;
        MI_CUDA(ctx, cudaMemcpy(d_b, hb.data(), hb.size() * 4, cudaMemcpyHostToDevice));
        lp[l] = LayerPtrs{d_an, d_fn, d_b};
        uint8_t *d_qkv, *d_o, *d_gu, *d_dn; int kb, nt;
        if ((st = alloc_tiled(ctx, m, qkv_rows, E, &d_qkv, &kb, &nt))) return st;
        if ((st = repack(wq, d_qkv, d_mq, 0)) || (st = repack(wk, d_qkv, d_mk, 0)) || (st = repack(wv, d_qkv, nullptr, NQ + KVD))) return st;
        if ((st = alloc_tiled(ctx, m, E, NQ, &d_o, &kb, &nt)) || (st = repack(wo, d_o, nullptr, 0))) return st;
        if ((st = alloc_tiled(ctx, m, 2 * (int64_t)FF, E, &d_gu, &kb, &nt))) return st;
        if ((st = repack(wg, d_gu, d_mg, 0)) || (st = repack(wu, d_gu, d_mu, 0))) return st;
        if ((st = alloc_tiled(ctx, m, E, FF, &d_dn, &kb, &nt)) || (st = repack(wd, d_dn, nullptr, 0))) return st;
        add_job(d_qkv, (qkv_rows + 31) / 32, E, 1, JOB_QKV, l);
        add_job(d_o, (E + 31) / 32, NQ, 1, JOB_O, l);
        add_job(d_gu, FF / 32, E, 2, JOB_GU, l);
        add_job(d_dn, (E + 31) / 32, FF, 1, JOB_DOWN, l);
        m->weight_bytes_q4 += ((int64_t)NQ * E + 2 * (int64_t)KVD * E + (int64_t)E * NQ + 3 * (int64_t)FF * E) / 32 * 18;
    }
    add_job(d_lm, (V + 31) / 32, E, 1, JOB_LM, L);
    m->views.back().rows = V;
    m->weight_bytes_q4 += (int64_t)V * E / 32 * 18;
    MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));

    // ---- per-warp tile lists: the order in which each warp of the grid consumes tiles during one step
    {
        const int nj = (int)m->jobs.size(), G = GG;
        std::vector<std::vector<unsigned long long>> lists((size_t)G * DNW);
        std::vector<unsigned> start((size_t)G * DNW * (nj + 1), 0);
        for (int j = 0; j < nj; j++) {
            const Job& jb = m->jobs[j];
            const size_t tb = (size_t)jb.kb * kTileRowBytes;
            const unsigned long long code = jb.kb == 8 ? 3 : jb.kb == 4 ? 2 : jb.kb == 2 ? 1 : 0;
            for (int slot = 0; slot < G * DNW; slot++) start[(size_t)slot * (nj + 1) + j] = (unsigned)lists[slot].size();
            if (jb.kind == JOB_LM) {
                for (int u = 0; u < jb.n_units; u++) {                  // warp unit u -> slot sid = (u + rot) % W, sid = warp*G + cta
                    const int sid = (int)(((long long)u + jb.rot) % W), cta = sid % G, warp = sid / G;
                    auto& L = lists[(size_t)cta * DNW + warp];
                    for (int t = 0; t < jb.nt; t++) L.push_back((unsigned long long)(uintptr_t)(jb.base + ((size_t)u * jb.nt + t) * tb) | code);
                }
            } else {
                for (int cta = 0; cta < G; cta++) {
                    const int r = jb.rot % G, u0 = cta >= r ? cta - r : cta + G - r;
                    int uidx = 0;
                    for (int u = u0; u < jb.n_units; u += G, uidx++) {
                        const int g = u / jb.ks, sp = u % jb.ks, t0 = sp * jb.nt / jb.ks, ntu = (sp + 1) * jb.nt / jb.ks - t0, n = jb.nacc * ntu;
                        const int wr = (jb.wrot + uidx * 3) & (DNW - 1);
                        for (int warp = 0; warp < DNW; warp++)
                            for (int i = (warp - wr) & (DNW - 1); i < n; i += DNW) {
                                const int a = i / ntu, t = t0 + i % ntu;
                                lists[(size_t)cta * DNW + warp].push_back(
                                    (unsigned long long)(uintptr_t)(jb.base + ((size_t)(g * jb.nacc + a) * jb.nt + t) * tb) | code);
                            }
                    }
                }
            }
        }
        size_t stride = 1;
        for (int slot = 0; slot < G * DNW; slot++) {
            start[(size_t)slot * (nj + 1) + nj] = (unsigned)lists[slot].size();
            stride = std::max(stride, lists[slot].size());
        }
        std::vector<unsigned long long> tab((size_t)G * DNW * stride, 0ull);
        for (int slot = 0; slot < G * DNW; slot++) std::copy(lists[slot].begin(), lists[slot].end(), tab.begin() + (size_t)slot * stride);
        unsigned long long* d_tab; unsigned* d_start;
        if ((st = dev_alloc(ctx, m, &d_tab, tab.size())) || (st = dev_alloc(ctx, m, &d_start, start.size()))) return st;
        MI_CUDA(ctx, cudaMemcpy(d_tab, tab.data(), tab.size() * 8, cudaMemcpyHostToDevice));
        MI_CUDA(ctx, cudaMemcpy(d_start, start.data(), start.size() * 4, cudaMemcpyHostToDevice));
        P.tile_tab = d_tab; P.tile_start = d_start; P.tile_stride = (int)stride;
    }

    LayerPtrs* d_lp; Job* d_jobs;
    if ((st = dev_alloc(ctx, m, &d_lp, lp.size())) || (st = dev_alloc(ctx, m, &d_jobs, m->jobs.size()))) return st;
    MI_CUDA(ctx, cudaMemcpy(d_lp, lp.data(), lp.size() * sizeof(LayerPtrs), cudaMemcpyHostToDevice));
    MI_CUDA(ctx, cudaMemcpy(d_jobs, m->jobs.data(), m->jobs.size() * sizeof(Job), cudaMemcpyHostToDevice));
    P.layers = d_lp; P.jobs = d_jobs;
    m->layer_ptrs = lp;

    // rope frequencies exactly as the reference computes them on the host: powf(base, -2i/hd) (src/cpu_infer.cpp:54)
    std::vector<float> freq(HD / 2);
    for (int i = 0; i < HD / 2; i++) freq[i] = std::pow(m->rope_base, -2.f * i / HD);
    float* d_freq; if ((st = dev_alloc(ctx, m, &d_freq, freq.size()))) return st;
    MI_CUDA(ctx, cudaMemcpy(d_freq, freq.data(), freq.size() * 4, cudaMemcpyHostToDevice));
    P.rope_freq = d_freq;
    float* d_cs; if ((st = dev_alloc(ctx, m, &d_cs, (size_t)max_seq * HD, false))) return st;
    rope_cs_kernel<<<max_seq, HD / 2, 0, ctx->stream>>>(d_freq, d_cs, HD, max_seq);
    MI_CUDA(ctx, cudaGetLastError());
    P.rope_cs = d_cs; P.rope_rows = max_seq;
    P.stop_token = -1;

    // ---- state
    // the exchange block: every vector one CTA hands to another, as tagged 8-byte words (layout: XwLayout)
    {
        XwLayout& x = P.xo;
        int off = 0;
        auto take = [&](int words) { const int o = off; off += (words + 1) / 2 * 2; return o; };     // every vector 16-byte aligned
        x.qkv = take((qkv_rows + 31) / 32 * 32);
        x.att = take(q8_words(NQ));
        x.o = take((E + 31) / 32 * 32);
        x.act = take(q8_words(FF));
        x.down = take((E + 31) / 32 * 32);
        x.dpart = take((E + 31) / 32 * (kMaxKSplit - 1) * 64);
        x.cand = take(kMaxWorldTP * m->grid * 4);
        x.tokw = take(2);
        x.total = off;
    }
    if ((st = dev_alloc(ctx, m, &P.h_in, E)) || (st = dev_alloc(ctx, m, &P.h_mid, E)) || (st = dev_alloc(ctx, m, &P.att, NQ)) ||
        (st = dev_alloc(ctx, m, &P.xw, (size_t)P.xo.total)) ||
        (st = dev_alloc(ctx, m, &P.kc, (size_t)L * max_seq * KVD)) || (st = dev_alloc(ctx, m, &P.vc, (size_t)L * max_seq * KVD)) ||
        (st = dev_alloc(ctx, m, &P.attn_part, (size_t)m->NH * m->max_chunks * (HD + 2))) || (st = dev_alloc(ctx, m, &P.attn_cnt, m->NH)) ||
        (st = dev_alloc(ctx, m, &P.prof, kProfSlots)) || (st = dev_alloc(ctx, m, &m->best_buf, 2)) ||
        (st = dev_alloc(ctx, m, &m->d_pos, 2)))
        return st;
    P.best_val = m->best_buf; P.cur_token = reinterpret_cast<int*>(m->best_buf + 1);                        // {value, token}: exchanged as one piece
    // the tag counter lives on the device and the kernel advances it itself (a launch that completes a step leaves it
    // past every tag it used): replayed launch sequences and calls after a failed one always get fresh tags.
    // Words start as zero, so the counter starts at 1.
    {
        const int init[2] = {0, 1};
        MI_CUDA(ctx, cudaMemcpy(m->d_pos, init, sizeof(init), cudaMemcpyHostToDevice));
    }
    P.epoch_dev = reinterpret_cast<unsigned*>(m->d_pos + 1);
    P.drop_phase = -1; P.attn_ctas = m->attn_ctas; P.prof_cta = m->attn_ctas;
    if (const char* pc = getenv("MINFER_PROFILE_CTA")) P.prof_cta = std::max(0, std::min(atoi(pc), m->grid - 1));
    P.max_seq = max_seq; P.max_chunks = m->max_chunks; P.err = ctx->d_err;
    m->prof_buf = P.prof;
    if (!getenv("MINFER_PROFILE")) P.prof = nullptr;         // the buffer exists either way; kernels only write it when asked
    m->smem = decode_smem_bytes((int)m->jobs.size(), E, FF, HD, m->G);
    if (m->attn_ctas > 0) {
        const int hpc = (m->G % 2 == 0 && m->G > 2) ? m->G / 2 : (m->G <= 2 ? 1 : m->G);
        m->smem = std::max(m->smem, attn_dedicated_smem(HD, hpc));       // the attention CTAs lay the same allocation out their own way
    }
    if (m->smem > (size_t)ctx->smem_optin)
        return set_error(ctx, MI_ERR_UNSUPPORTED, "model: decode kernel needs %zu bytes of shared memory, %d available", m->smem, ctx->smem_optin);
    MI_CUDA(ctx, cudaEventCreate(&m->ev0));
    MI_CUDA(ctx, cudaEventCreate(&m->ev1));
    MI_CUDA(ctx, cudaDeviceSynchronize());           // every upload and fill of the load has landed, whatever stream it used
    guard.keep = true;
    *out = m;
    return MI_OK;
}

extern "C" int mi_model_info(const mi_model* m, mi_model_config* c) {
    if (!m || !c) return MI_ERR_INVALID;
    c->n_layer = m->L; c->n_embd = m->E; c->n_ff = m->FF; c->n_head = m->NH; c->n_head_kv = m->NKV; c->head_dim = m->HD;
    c->n_vocab = m->V; c->max_seq = m->max_seq; c->tied_lm_head = m->tied ? 1 : 0; c->grid_ctas = m->grid;
    c->rope_base = m->rope_base; c->rms_eps = m->eps;
    c->q4_weight_bytes_per_token = m->weight_bytes_q4;
    c->kv_bytes_per_position = (int64_t)2 * m->L * m->KVD * 2;
    return MI_OK;
}

extern "C" int mi_model_state_ptr(const mi_model* m, int which, void** ptr, int64_t* bytes) {
    if (!m || !ptr) return MI_ERR_INVALID;
    const DecodeParams& P = m->P;
    const int NQ = m->NH * m->HD;
    switch (which) {
        case MI_STATE_H: *ptr = P.h_in; if (bytes) *bytes = (int64_t)m->E * 4; break;
        case MI_STATE_H_MID: *ptr = P.h_mid; if (bytes) *bytes = (int64_t)m->E * 4; break;
        case MI_STATE_Q: *ptr = P.xw + P.xo.qkv; if (bytes) *bytes = (int64_t)(NQ + 2 * m->KVD) * 8; break;
        case MI_STATE_ATT: *ptr = P.att; if (bytes) *bytes = (int64_t)NQ * 4; break;
        case MI_STATE_KCACHE: *ptr = P.kc; if (bytes) *bytes = (int64_t)m->L * m->max_seq * m->KVD * 2; break;
        case MI_STATE_VCACHE: *ptr = P.vc; if (bytes) *bytes = (int64_t)m->L * m->max_seq * m->KVD * 2; break;
        case MI_STATE_ACT_Q: *ptr = P.xw + P.xo.act; if (bytes) *bytes = (int64_t)m->FF / 4 * 8; break;
        case MI_STATE_ACT_D: *ptr = P.xw + P.xo.act + m->FF / 4; if (bytes) *bytes = (int64_t)m->FF / 32 * 8; break;
        case MI_STATE_PROFILE: *ptr = m->prof_buf; if (bytes) *bytes = (int64_t)kProfSlots * 8; break;
        default: return MI_ERR_INVALID;
    }
    return MI_OK;
}

struct mi_token_ring {
    int capacity = 0;
    void* host = nullptr;           // one mapped pinned allocation: count | tokens | margins | ns
    int* h_count = nullptr; int32_t* h_tokens = nullptr; float* h_margins = nullptr; unsigned long long* h_ns = nullptr;
    int* d_count = nullptr; int32_t* d_tokens = nullptr; float* d_margins = nullptr; unsigned long long* d_ns = nullptr;
    int used = 0;                   // entries handed to launches so far
};

extern "C" int mi_ring_create(mi_ctx* ctx, int capacity, mi_token_ring** out) {
    if (!ctx) return MI_ERR_INVALID;
    if (!out || capacity < 1) return set_error(ctx, MI_ERR_INVALID, "ring_create: bad argument");
    *out = nullptr;
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    mi_token_ring* r = new (std::nothrow) mi_token_ring();
    if (!r) return set_error(ctx, MI_ERR_NOMEM, "ring_create: host allocation failed");
    const size_t cap = (size_t)capacity, bytes = 64 + cap * 4 + cap * 4 + cap * 8 + 64;
    cudaError_t e = cudaHostAlloc(&r->host, bytes, cudaHostAllocMapped);
    if (e != cudaSuccess) { delete r; return set_error(ctx, MI_ERR_NOMEM, "ring_create: cudaHostAlloc(%zu) failed: %s", bytes, cudaGetErrorString(e)); }
    memset(r->host, 0, bytes);
    void* dev = nullptr;
    e = cudaHostGetDevicePointer(&dev, r->host, 0);
    if (e != cudaSuccess) { cudaFreeHost(r->host); delete r; return set_error(ctx, MI_ERR_CUDA, "ring_create: cudaHostGetDevicePointer failed"); }
    auto carve = [&](uint8_t* base) {
        struct { int* c; int32_t* t; float* g; unsigned long long* n; } v;
        v.c = reinterpret_cast<int*>(base); v.n = reinterpret_cast<unsigned long long*>(base + 64);
        v.t = reinterpret_cast<int32_t*>(base + 64 + cap * 8); v.g = reinterpret_cast<float*>(base + 64 + cap * 8 + cap * 4);
        return v;
    };
    auto h = carve(reinterpret_cast<uint8_t*>(r->host)); auto d = carve(reinterpret_cast<uint8_t*>(dev));
    r->h_count = h.c; r->h_tokens = h.t; r->h_margins = h.g; r->h_ns = h.n;
    r->d_count = d.c; r->d_tokens = d.t; r->d_margins = d.g; r->d_ns = d.n;
    r->capacity = capacity;
    *out = r;
    return MI_OK;
}

extern "C" int mi_ring_destroy(mi_ctx* ctx, mi_token_ring* r) {
    if (!r) return MI_OK;
    if (ctx) { cudaSetDevice(ctx->device); cudaStreamSynchronize(ctx->stream); }
    if (r->host) cudaFreeHost(r->host);
    delete r;
    return MI_OK;
}

extern "C" int mi_ring_reset(mi_ctx* ctx, mi_token_ring* r) {
    if (!r) return MI_ERR_INVALID;
    if (ctx) { cudaSetDevice(ctx->device); cudaStreamSynchronize(ctx->stream); }
    r->used = 0;
    __atomic_store_n(r->h_count, 0, __ATOMIC_RELEASE);
    return MI_OK;
}

extern "C" int mi_ring_peek(const mi_token_ring* r, int* count, const int32_t** tokens, const float** margins, const uint64_t** ns) {
    if (!r) return MI_ERR_INVALID;
    if (count) *count = __atomic_load_n(r->h_count, __ATOMIC_ACQUIRE);
    if (tokens) *tokens = r->h_tokens;
    if (margins) *margins = r->h_margins;
    if (ns) *ns = reinterpret_cast<const uint64_t*>(r->h_ns);
    return MI_OK;
}

// ---- the kernel-sequence engine as a replayed graph -----------------------------------------------------------------
// One step of the kernel-sequence engine is 5L+1 cooperative launches; issued one by one they cost the host about 10 us
// each, more than the kernels take.  So the step is captured once per context range - position and token device-resident,
// which phase a launch runs is its only argument - and replayed per token, as the reference's kernel-sequence driver
// replays its captured step (src/cuda_infer.cu:1089-1109).  The graph's first node puts a forced token in place, its last
// nodes file the step's token and margin under the step's index and advance position and index; the arrays they use are
// named by a control block in device memory that every call refills, so a graph outlives reallocation of those arrays.
struct SeqCtl { const int* in; int* out; float* mg; int n_forced; int step; };
__global__ void seq_set_pos_kernel(int* pos, int value) { *pos = value; }
__global__ void seq_pre_kernel(const SeqCtl* c, int* cur_token) { if (c->step < c->n_forced) *cur_token = c->in[c->step]; }
__global__ void seq_post_kernel(SeqCtl* c, const int* tok, const float* margin, int* pos) {
    c->out[c->step] = *tok; c->mg[c->step] = *margin; c->step += 1; *pos += 1;
}

static int step_graph(mi_ctx* ctx, mi_model* m, int range, cudaGraphExec_t* out) {
    if (m->step_graph[range] && m->step_graph_wait[range] == ctx->wait_ns) { *out = (cudaGraphExec_t)m->step_graph[range]; return MI_OK; }
    if (m->step_graph[range]) { cudaGraphExecDestroy((cudaGraphExec_t)m->step_graph[range]); m->step_graph[range] = nullptr; }
    int st;
    if (!m->d_seq_ctl) {
        SeqCtl* c; if ((st = dev_alloc(ctx, m, &c, 1)) || (st = dev_alloc(ctx, m, &m->d_step_out, 2)) || (st = dev_alloc(ctx, m, &m->d_step_margin, 2))) return st;
        m->d_seq_ctl = c;
    }
    const int nph = 5 * m->L + 1;
    DecodeParams P = m->P;
    P.in_tokens = nullptr; P.n_forced = 0; P.out_tokens = m->d_step_out; P.out_margins = m->d_step_margin; P.pos0 = 0; P.pos_dev = m->d_pos;
    P.logits = nullptr; P.logits_stride = m->V; P.wait_ns = ctx->wait_ns; P.stop_token = -1;
    if ((st = dispatch_launch(ctx, m, P, 0, 1, 0, 1, false, range, true))) return st;      // kernel picked, shared-memory limit raised: not inside the capture
    // captured on a stream of its own: the context's stream may be the legacy default stream, which cannot capture
    MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    cudaStream_t cs = nullptr, user = ctx->stream;
    MI_CUDA(ctx, cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking));
    cudaError_t eb = cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal);
    if (eb != cudaSuccess) { cudaStreamDestroy(cs); return set_error(ctx, MI_ERR_CUDA, "decode: the step cannot be captured: %s", cudaGetErrorString(eb)); }
    ctx->stream = cs;
    seq_pre_kernel<<<1, 1, 0, cs>>>(static_cast<const SeqCtl*>(m->d_seq_ctl), m->P.cur_token);
    st = MI_OK;
    for (int ph = 0; ph < nph && st == MI_OK; ph++) st = dispatch_launch(ctx, m, P, 0, 1, ph, ph + 1, false, range);
    seq_post_kernel<<<1, 1, 0, cs>>>(static_cast<SeqCtl*>(m->d_seq_ctl), m->d_step_out, m->d_step_margin, m->d_pos);
    ctx->stream = user;
    cudaGraph_t g = nullptr;
    const cudaError_t e = cudaStreamEndCapture(cs, &g);
    cudaStreamDestroy(cs);
    if (st != MI_OK) { if (g) cudaGraphDestroy(g); return st; }
    if (e != cudaSuccess) { if (g) cudaGraphDestroy(g); return set_error(ctx, MI_ERR_CUDA, "decode: capturing the step failed: %s", cudaGetErrorString(e)); }
    cudaGraphExec_t x = nullptr;
    const cudaError_t e2 = cudaGraphInstantiate(&x, g, 0);
    cudaGraphDestroy(g);
    if (e2 != cudaSuccess) return set_error(ctx, MI_ERR_CUDA, "decode: instantiating the step graph failed: %s", cudaGetErrorString(e2));
    m->step_graph[range] = x; m->step_graph_wait[range] = ctx->wait_ns;
    *out = x;
    return MI_OK;
}

static int decode_impl(mi_ctx* ctx, mi_model* m, const int32_t* in_tokens_host, int n_forced, int n_steps, int pos0,
                       int32_t* out_tokens_host, float* logits_dev, int mode, int ph0, int ph1, float* elapsed_ms,
                       mi_token_ring* ring = nullptr, bool async = false) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m) return set_error(ctx, MI_ERR_INVALID, "decode: null model");
    if (n_steps < 0 || n_forced < 0 || pos0 < 0) return set_error(ctx, MI_ERR_INVALID, "decode: negative count");
    if (n_steps == 0) { if (elapsed_ms) *elapsed_ms = 0.f; return MI_OK; }
    if (n_forced > n_steps) n_forced = n_steps;
    if (n_forced > 0 && !in_tokens_host) return set_error(ctx, MI_ERR_INVALID, "decode: null input tokens");
    if ((long long)pos0 + n_steps > m->max_seq)
        return set_error(ctx, MI_ERR_LIMIT, "decode: positions %d..%d exceed the KV cache of %d", pos0, pos0 + n_steps - 1, m->max_seq);
    for (int i = 0; i < n_forced; i++)
        if (in_tokens_host[i] < 0 || in_tokens_host[i] >= m->V) return set_error(ctx, MI_ERR_INVALID, "decode: token id %d out of range", in_tokens_host[i]);
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    int st;
    if (n_forced > m->in_capacity) {
        if ((st = dev_alloc(ctx, m, &m->d_in_tokens, (size_t)n_forced * 2))) return st;
        m->in_capacity = n_forced * 2;
    }
    if (n_steps > m->out_capacity) {
        if ((st = dev_alloc(ctx, m, &m->d_out_tokens, (size_t)n_steps * 2)) || (st = dev_alloc(ctx, m, &m->d_margins, (size_t)n_steps * 2))) return st;
        m->out_capacity = n_steps * 2;
    }
    m->last_steps = n_steps; m->last_count = n_steps;
    if (ring && ring->used + n_steps > ring->capacity)
        return set_error(ctx, MI_ERR_LIMIT, "decode: the token ring holds %d entries, %d are used and %d more are asked for", ring->capacity, ring->used, n_steps);
    if (n_forced) MI_CUDA(ctx, cudaMemcpyAsync(m->d_in_tokens, in_tokens_host, (size_t)n_forced * 4, cudaMemcpyHostToDevice, ctx->stream));
    DecodeParams P = m->P;
    if (m->tp_world > 1) {
        // a sharded model decodes through this entry point only with the exchange inside the kernel (peer memory mapped,
        // persistent engine); every GPU must make the same call
        if (!m->tp_peer_on || mode != MI_DECODE_PERSISTENT)
            return set_error(ctx, MI_ERR_UNSUPPORTED, "decode: a sharded model needs mi_tp_ipc_open and the persistent engine here (or mi_decode_launch + exchanges)");
        TpPeerParams& T = P.tp;
        T.on = 1; T.rank = m->tp_rank; T.world = m->tp_world;
        for (int r = 0; r < m->tp_world; r++) T.xw_peer[r] = reinterpret_cast<unsigned long long*>(m->tp_peer[r][0]);
    }
    P.wait_ns = ctx->wait_ns;
    // the stop rule applies to runs over whole steps that feed their own predictions back
    const int stop = (ph0 == 0 && ph1 == 5 * m->L + 1 && n_steps > n_forced - 1) ? m->stop_token : -1;
    P.stop_token = stop;
    if ((st = mi::reset_after_error(ctx, m))) return st;
    P.in_tokens = m->d_in_tokens; P.n_forced = n_forced; P.out_tokens = m->d_out_tokens; P.pos0 = pos0;
    P.out_margins = m->d_margins;
    P.logits = logits_dev; P.logits_stride = m->V;
    if (ring) {
        P.ring.count = ring->d_count; P.ring.tokens = ring->d_tokens; P.ring.margins = ring->d_margins; P.ring.ns = ring->d_ns;
        P.ring.capacity = ring->capacity; P.ring.base = ring->used;
        ring->used += n_steps;
    }
    const int nph = 5 * m->L + 1;
    MI_CUDA(ctx, cudaEventRecord(m->ev0, ctx->stream));
    if (mode == MI_DECODE_PERSISTENT) {
        // One launch, or one per context range the steps pass through (up to kShortAttnMax positions, up to kPerHeadAttnMax,
        // beyond): each range has a build of the kernel with only its attention variant (dispatch_launch picks by the
        // launch's positions), a launch that straddles a boundary would fall back to the general build.  Under the stop
        // rule the host cannot know whether an earlier launch ended the run, so the run stays one launch.
        int cuts[4] = {0, 0, 0, n_steps}, nc = 1;
        if (stop < 0 && !P.tp.on && lean_shape_ok(m->E, m->FF, m->NH * m->HD)) {
            for (int edge : {kShortAttnMax, kPerHeadAttnMax}) {
                const long long s = (long long)edge - pos0;            // first step whose position count exceeds the edge
                if (s > cuts[nc - 1] && s < n_steps) cuts[nc++] = (int)s;
            }
        }
        cuts[nc] = n_steps;
        for (int i = 0; i < nc; i++) {
            DecodeParams Ps = P;
            if (Ps.logits) Ps.logits += (long long)cuts[i] * Ps.logits_stride;   // the kernel indexes logits and ring entries from its first step
            Ps.ring.base += cuts[i];
            if ((st = dispatch_launch(ctx, m, Ps, cuts[i], cuts[i + 1], 0, nph, true))) return st;
        }
    } else if (mode == MI_DECODE_PER_PHASE && !logits_dev && stop < 0 && !ring && ph0 == 0 && ph1 == nph && m->tp_world == 1 && P.drop_phase < 0 && !P.prof &&
               !getenv("MINFER_SEQ_NO_GRAPH")) {
        // whole steps, nothing to look at between them: the captured step, replayed per token
        cudaGraphExec_t gx[4] = {nullptr, nullptr, nullptr, nullptr};
        for (int s = 0; s < n_steps; s++) {             // every graph this run needs exists before the first replay
            const int range = pos0 + s + 1 <= kShortAttnMax ? 1 : pos0 + s + 1 <= kPerHeadAttnMax ? 2 : 3;
            if (!gx[range] && (st = step_graph(ctx, m, range, &gx[range]))) return st;
        }
        const SeqCtl ctl{m->d_in_tokens, m->d_out_tokens, m->d_margins, n_forced, 0};
        MI_CUDA(ctx, cudaMemcpyAsync(m->d_seq_ctl, &ctl, sizeof ctl, cudaMemcpyHostToDevice, ctx->stream));
        seq_set_pos_kernel<<<1, 1, 0, ctx->stream>>>(m->d_pos, pos0);
        MI_CUDA(ctx, cudaGetLastError());
        MI_CUDA(ctx, cudaEventRecord(m->ev0, ctx->stream));         // (the timed region starts after the set-up above)
        for (int s = 0; s < n_steps; s++) {
            const int range = pos0 + s + 1 <= kShortAttnMax ? 1 : pos0 + s + 1 <= kPerHeadAttnMax ? 2 : 3;
            MI_CUDA(ctx, cudaGraphLaunch(gx[range], ctx->stream));
        }
    } else if (mode == MI_DECODE_PER_PHASE) {
        for (int s = 0; s < n_steps; s++) {
            DecodeParams Ps = P;
            if (Ps.logits) Ps.logits += (long long)s * Ps.logits_stride;    // the kernel indexes logits from its first step
            for (int ph = ph0; ph < ph1; ph++)
                if ((st = dispatch_launch(ctx, m, Ps, s, s + 1, ph, ph + 1, false))) return st;
            if (stop >= 0 && s + 1 >= n_forced && s + 1 < n_steps) {
                // under the stop rule this engine looks at every token before it launches the next step, as the reference's
                // kernel-sequence driver does (src/cuda_infer.cu:1186-1193)
                int32_t tok = -1;
                MI_CUDA(ctx, cudaMemcpyAsync(&tok, m->d_out_tokens + s, 4, cudaMemcpyDeviceToHost, ctx->stream));
                if ((st = mi_ctx_sync(ctx))) return st;
                if (tok == stop) { m->last_count = s + 1; break; }
            }
        }
    } else {
        return set_error(ctx, MI_ERR_INVALID, "decode: unknown mode %d", mode);
    }
    MI_CUDA(ctx, cudaEventRecord(m->ev1, ctx->stream));
    if (async) return MI_OK;                          // the caller follows the ring and synchronizes itself
    std::vector<int32_t> scan;
    if (stop >= 0 && !out_tokens_host) { scan.resize((size_t)n_steps); out_tokens_host = scan.data(); }
    if (out_tokens_host)
        MI_CUDA(ctx, cudaMemcpyAsync(out_tokens_host, m->d_out_tokens, (size_t)n_steps * 4, cudaMemcpyDeviceToHost, ctx->stream));
    st = mi_ctx_sync(ctx);
    if (st != MI_OK) return st;
    if (stop >= 0 && mode == MI_DECODE_PERSISTENT)    // the kernel ended the run after the first consumed prediction equal to the stop token
        for (int s = std::max(n_forced - 1, 0); s < n_steps; s++)
            if (out_tokens_host[s] == stop) { m->last_count = s + 1; break; }
    if (elapsed_ms) MI_CUDA(ctx, cudaEventElapsedTime(elapsed_ms, m->ev0, m->ev1));
    return MI_OK;
}

extern "C" int mi_decode(mi_ctx* ctx, mi_model* m, const int32_t* in_tokens_host, int n_forced, int n_steps, int pos0,
                         int32_t* out_tokens_host, float* logits_dev, int mode, float* elapsed_ms) {
    return decode_impl(ctx, m, in_tokens_host, n_forced, n_steps, pos0, out_tokens_host, logits_dev, mode, 0,
                       m ? 5 * m->L + 1 : 0, elapsed_ms);
}

extern "C" int mi_decode_run(mi_ctx* ctx, mi_model* m, const int32_t* in_tokens_host, int n_forced, int n_steps, int pos0, mi_token_ring* ring) {
    if (!ctx) return MI_ERR_INVALID;
    if (!ring) return set_error(ctx, MI_ERR_INVALID, "decode_run: null ring");
    return decode_impl(ctx, m, in_tokens_host, n_forced, n_steps, pos0, nullptr, nullptr, MI_DECODE_PERSISTENT, 0, m ? 5 * m->L + 1 : 0, nullptr, ring, true);
}

extern "C" int mi_model_set_stop_token(mi_model* m, int token) {
    if (!m || token >= m->V) return MI_ERR_INVALID;
    m->stop_token = token < 0 ? -1 : token;
    return MI_OK;
}

extern "C" int mi_model_last_count(const mi_model* m) { return m ? m->last_count : 0; }

extern "C" int mi_decode_margins(mi_ctx* ctx, mi_model* m, int n, float* margins_host) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m || !margins_host || n < 0 || n > m->last_steps) return set_error(ctx, MI_ERR_INVALID, "decode_margins: the last decode call ran %d steps", m ? m->last_steps : 0);
    if (n == 0) return MI_OK;
    MI_CUDA(ctx, cudaMemcpyAsync(margins_host, m->d_margins, (size_t)n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    MI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MI_OK;
}

extern "C" int mi_decode_phases(mi_ctx* ctx, mi_model* m, int32_t token, int pos, int phase_begin, int phase_end) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m) return set_error(ctx, MI_ERR_INVALID, "decode: null model");
    const int nph = 5 * m->L + 1;
    if (phase_begin < 0 || phase_end > nph || phase_begin > phase_end) return set_error(ctx, MI_ERR_INVALID, "decode: bad phase range");
    int32_t out;
    return decode_impl(ctx, m, &token, 1, 1, pos, &out, nullptr, MI_DECODE_PER_PHASE, phase_begin, phase_end, nullptr);
}

// ---- tensor parallelism: asynchronous phase launches and the buffers the GPUs exchange ------------------

namespace {
__global__ void set_token_kernel(int* dst, int tok) { *dst = tok; }
__global__ void add_int_kernel(int* dst, int delta) { *dst += delta; }
__global__ void reset_counters_kernel(unsigned* a, int na, unsigned* b, int nb) {
    for (int i = threadIdx.x; i < na; i += blockDim.x) a[i] = 0;
    for (int i = threadIdx.x; i < nb; i += blockDim.x) b[i] = 0;
}
// gathered: [world] x {float best value, int token}; the largest value wins, the lowest token id on ties
// (the rule of src/cpu_infer.cpp:153-154 applied across the GPUs' row ranges)
__global__ void tp_pick_kernel(const float* gathered, int world, float* best_val, int* cur_token) {
    float b = gathered[0]; int t = reinterpret_cast<const int*>(gathered)[1];
    for (int r = 1; r < world; r++) {
        const float v = gathered[2 * r]; const int ix = reinterpret_cast<const int*>(gathered)[2 * r + 1];
        if (v > b || (v == b && ix < t)) { b = v; t = ix; }
    }
    *best_val = b; *cur_token = t;
}
}  // namespace

extern "C" int mi_model_tp_region(const mi_model* m, int which, int layer, void** ptr, int64_t* bytes) {
    if (!m || !ptr || !bytes) return MI_ERR_INVALID;
    const DecodeParams& P = m->P;
    switch (which) {
        case MI_TP_QKV: *ptr = P.xw + P.xo.qkv; *bytes = (int64_t)(m->qkv_rows + 31) / 32 * 32 * 8; return MI_OK;
        case MI_TP_ACT: *ptr = P.xw + P.xo.act; *bytes = (int64_t)q8_words(m->FF) * 8; return MI_OK;
        case MI_TP_BEST: *ptr = m->best_buf; *bytes = 8; return MI_OK;
        case MI_TP_PART_O: case MI_TP_PART_DOWN:
            if (layer < 0 || layer >= m->L) return MI_ERR_INVALID;
            *ptr = P.xw + (which == MI_TP_PART_O ? P.xo.o : P.xo.down); *bytes = (int64_t)(m->E + 31) / 32 * 32 * 8; return MI_OK;
        default: return MI_ERR_INVALID;
    }
}

extern "C" int mi_model_set_token(mi_ctx* ctx, mi_model* m, int32_t token) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m) return set_error(ctx, MI_ERR_INVALID, "set_token: null model");
    if (token < 0 || token >= m->V) return set_error(ctx, MI_ERR_INVALID, "set_token: token id %d out of range", token);
    set_token_kernel<<<1, 1, 0, ctx->stream>>>(m->P.cur_token, token);
    MI_CUDA(ctx, cudaGetLastError());
    return MI_OK;
}

extern "C" int mi_model_set_pos(mi_ctx* ctx, mi_model* m, int pos) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m) return set_error(ctx, MI_ERR_INVALID, "set_pos: null model");
    if (pos < 0 || pos >= m->max_seq) return set_error(ctx, MI_ERR_LIMIT, "set_pos: position %d outside the KV cache of %d", pos, m->max_seq);
    set_token_kernel<<<1, 1, 0, ctx->stream>>>(m->d_pos, pos);
    MI_CUDA(ctx, cudaGetLastError());
    return MI_OK;
}

extern "C" int mi_model_advance_pos(mi_ctx* ctx, mi_model* m, int delta) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m) return set_error(ctx, MI_ERR_INVALID, "advance_pos: null model");
    add_int_kernel<<<1, 1, 0, ctx->stream>>>(m->d_pos, delta);
    MI_CUDA(ctx, cudaGetLastError());
    return MI_OK;
}

extern "C" int mi_model_get_token(mi_ctx* ctx, mi_model* m, int32_t* token, float* best_val) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m) return set_error(ctx, MI_ERR_INVALID, "get_token: null model");
    float h[2];
    MI_CUDA(ctx, cudaMemcpyAsync(h, m->best_buf, 8, cudaMemcpyDeviceToHost, ctx->stream));
    int st = mi_ctx_sync(ctx);
    if (st != MI_OK) return st;
    if (best_val) *best_val = h[0];
    if (token) memcpy(token, &h[1], 4);
    return MI_OK;
}

extern "C" int mi_tp_pick(mi_ctx* ctx, mi_model* m, const void* gathered_dev, int world) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m || !gathered_dev || world < 1) return set_error(ctx, MI_ERR_INVALID, "tp_pick: bad argument");
    tp_pick_kernel<<<1, 1, 0, ctx->stream>>>(reinterpret_cast<const float*>(gathered_dev), world, m->best_buf, m->P.cur_token);
    MI_CUDA(ctx, cudaGetLastError());
    return MI_OK;
}

static int launch_phases(mi_ctx* ctx, mi_model* m, int pos, int phase_begin, int phase_end, bool fused);

extern "C" int mi_decode_launch(mi_ctx* ctx, mi_model* m, int pos, int phase_begin, int phase_end) {
    return launch_phases(ctx, m, pos, phase_begin, phase_end, false);
}

extern "C" int mi_decode_launch_fused(mi_ctx* ctx, mi_model* m, int pos, int phase_begin, int phase_end) {
    return launch_phases(ctx, m, pos, phase_begin, phase_end, true);
}

static int launch_phases(mi_ctx* ctx, mi_model* m, int pos, int phase_begin, int phase_end, bool fused) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m) return set_error(ctx, MI_ERR_INVALID, "decode_launch: null model");
    const int nph = 5 * m->L + 1;
    if (phase_begin < 0 || phase_end > nph || phase_begin > phase_end) return set_error(ctx, MI_ERR_INVALID, "decode_launch: bad phase range");
    // pos == MI_POS_DEVICE: the position is the model's device-resident one (mi_model_set_pos / mi_model_advance_pos); the
    // caller keeps it inside the KV cache
    const bool dev_pos = pos == MI_POS_DEVICE;
    if (!dev_pos && (pos < 0 || pos >= m->max_seq)) return set_error(ctx, MI_ERR_LIMIT, "decode_launch: position %d outside the KV cache of %d", pos, m->max_seq);
    int st;
    if (m->out_capacity < 1) {
        if ((st = dev_alloc(ctx, m, &m->d_out_tokens, 16)) || (st = dev_alloc(ctx, m, &m->d_margins, 16))) return st;
        m->out_capacity = 16;
    }
    DecodeParams P = m->P;
    P.in_tokens = nullptr; P.n_forced = 0; P.out_tokens = m->d_out_tokens; P.out_margins = m->d_margins; P.pos0 = dev_pos ? 0 : pos; P.logits = nullptr; P.logits_stride = m->V;
    P.pos_dev = dev_pos ? m->d_pos : nullptr;
    P.wait_ns = ctx->wait_ns;
    if ((st = mi::reset_after_error(ctx, m))) return st;
    for (int ph = phase_begin; ph < phase_end; ph++) {
        if (m->tp_world > 1 && ph < nph - 1 && !m->tp_peer_on) {          // (peer exchange: every GPU writes only what it owns, nothing is summed)
            // entries of the exchanged buffer that this GPU does not own must read zero before the all-reduce
            // (no phase of a fused range reads a buffer that a later phase of the range writes)
            const int l = ph / 5, k = ph % 5;
            void* p = nullptr; int64_t nb = 0;
            if (k == 3) mi_model_tp_region(m, MI_TP_ACT, l, &p, &nb);               // QKV and O are computed in full by every GPU
            else if (k == 4) mi_model_tp_region(m, MI_TP_PART_DOWN, l, &p, &nb);
            if (p) MI_CUDA(ctx, cudaMemsetAsync(p, 0, (size_t)nb, ctx->stream));
        }
        if (!fused && (st = dispatch_launch(ctx, m, P, 0, 1, ph, ph + 1, false))) return st;
    }
    if (fused && phase_end > phase_begin) {
        // one cooperative launch for the range, the weight ring running ahead across its phases
        if ((st = dispatch_launch(ctx, m, P, 0, 1, phase_begin, phase_end, true))) return st;
    }
    return MI_OK;
}

// A kernel that gave up on a wait may have left the self-resetting arrival counters of the attention merge (decode loop
// and M-token step) partly counted.  mi_ctx_sync counts the errors it reports; the first launch on a model after a new
// one clears that model's counters.
int mi::reset_after_error(mi_ctx* ctx, mi_model* m) {
    if (m->errors_seen == ctx->errors_reported) return MI_OK;
    m->errors_seen = ctx->errors_reported;
    reset_counters_kernel<<<1, 256, 0, ctx->stream>>>(m->P.attn_cnt, m->NH, m->vb.attn_cnt, m->vb.attn_cnt ? 16 * m->NH : 0);
    MI_CUDA(ctx, cudaGetLastError());
    if (m->vb.amax_cnt) {
        MI_CUDA(ctx, cudaMemsetAsync(m->vb.amax_cnt, 0, 16 * sizeof(unsigned), ctx->stream));
        MI_CUDA(ctx, cudaMemsetAsync(m->vb.amax_key, 0, 16 * sizeof(unsigned long long), ctx->stream));
    }
    return MI_OK;
}

// Test hook: the producers of one phase (index 5 * layer + kind, or the lm_head phase 5 * n_layer) publish nothing from
// now on, so that the waits of its consumers run out; -1 restores normal operation.
extern "C" int mi_model_debug_drop_phase(mi_model* m, int phase) {
    if (!m) return MI_ERR_INVALID;
    m->P.drop_phase = phase;
    return MI_OK;
}
