// Shared body of the two driver programs.  They keep the command line, environment
// knobs and stdout / stderr line shapes of the reference's drivers
//     <exe> <model.gguf> <n_gen> <id0> <id1> ...
// (reference src/cuda_infer.cu:844-1201 and src/mega.cu:1009-1259) and call the CUDA
// path only through the C ABI of minfer_b200.h.  Like the reference's CK()/REQUIRE()
// they print and exit on any error; the library itself never exits.
//
// stdout with RAWIDS=1: the n_gen greedy ids separated by a space, then a newline
// (the first id is the prediction after the last prompt token:
// src/cpu_infer.cpp:161-167).  Without RAWIDS: the text of the generated tokens,
// streamed piece by piece through the byte-level detokenizer (mi_detok_piece), and
// generation ends at the file's tokenizer.ggml.eos_token_id, whose piece is not
// printed (src/cuda_infer.cu:861-873, 1192; src/mega.cu:1017, 1173).
//
// Environment: TEACHER=k (ids are a reference sequence whose first k are the
// prompt; report top-1 agreement at every later position, with this engine's logit
// margin on the misses, as src/cuda_infer.cu:1148-1160 / src/mega.cu:1192-1205),
// MAXSEQ=n (KV cache positions; default prompt + n_gen + 8), WARMUP=n (untimed steps
// before the run), PROFILE=1 (per-phase time on one CTA, persistent engine), GPU=i
// (device index), TCHUNK=m (prompt / teacher-forced tokens per weight pass through
// the M-token step, 1..16, default 16; 1 = one decode step per token;
// src/cuda_infer.cu:1130-1144), SPEC=0|1|2 (lossless n-gram speculation;
// default 1 in mega, 0 in cuda_infer, as in the reference: src/mega.cu:1020,
// src/cuda_infer.cu:1167; 2 = submit every draft in full instead of the length
// the loop's cost model picks), NGMAX / NG (longest n-gram, default 3), DRAFTK (drafted
// tokens per step, default 4), MARGINS=1 (last stderr line "i:tok:margin ..." for
// every generated token, src/mega.cu:1241), SEGMENTS=w (tok/s over windows of w
// tokens, src/mega.cu:1236-1240), ATTN (accepted and ignored: attention is always
// split-KV here).  The mega driver prints ids as they arrive through the host-mapped
// token ring while the kernel is still generating (src/mega.cu:1166-1178).
#pragma once
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "gguf_file.hpp"
#include "minfer_b200.h"

namespace mib200 {

[[noreturn]] inline void die(mi_ctx* ctx, const char* what, int st) {
    fprintf(stderr, "%s failed: %s%s%s\n", what, mi_strerror(st), ctx ? " - " : "", ctx ? mi_last_error(ctx) : "");
    exit(1);
}

inline int env_int(const char* name, int def) { const char* v = getenv(name); return v ? atoi(v) : def; }

// tag: "cuda" or "mega"; mode: MI_DECODE_PER_PHASE or MI_DECODE_PERSISTENT
inline int driver_main(int argc, char** argv, const char* tag, int mode) {
    if (argc < 4) { fprintf(stderr, "usage: %s <model.gguf> <n_gen> <id...>\n", argv[0]); return 1; }
    const int n_gen = atoi(argv[2]);
    std::vector<int32_t> ids;
    for (int i = 3; i < argc; i++) ids.push_back(atoi(argv[i]));
    const int teacher = env_int("TEACHER", 0);
    int tchunk = env_int("TCHUNK", 16);
    tchunk = tchunk < 1 ? 1 : tchunk > 16 ? 16 : tchunk;
    if (env_int("PROFILE", 0)) setenv("MINFER_PROFILE", "1", 1);
    const bool raw_ids = env_int("RAWIDS", 0) != 0;
    // text mode: the vocabulary pieces and the end-of-sequence id come from the model file
    GgufFile vocab_file;
    int eos_id = -1;
    if (!raw_ids) {
        vocab_file.keep_token_strings(true);
        const std::string err = vocab_file.open(argv[1]);
        if (!err.empty()) { fprintf(stderr, "minfer-%s: %s\n", tag, err.c_str()); return 1; }
        eos_id = (int)vocab_file.num("tokenizer.ggml.eos_token_id", 151645);
    }
    const std::vector<std::string>& vocab = vocab_file.tokens();
    auto emit = [&](int id) {
        if (raw_ids) { printf("%d ", id); return; }
        if (id == eos_id || id < 0 || id >= (int)vocab.size()) return;
        const std::string& piece = vocab[(size_t)id];
        std::string text(piece.size(), '\0');
        const int64_t n = mi_detok_piece(piece.data(), (int64_t)piece.size(), &text[0], (int64_t)text.size());
        if (n > 0) fwrite(text.data(), 1, (size_t)n, stdout);
        fflush(stdout);
    };

    mi_ctx* ctx = nullptr;
    int st = mi_ctx_create(env_int("GPU", 0), &ctx);
    if (st) die(nullptr, "mi_ctx_create (is there a B200?)", st);
    const int P = (int)ids.size();
    const int maxseq = env_int("MAXSEQ", P + n_gen + 8);
    mi_model* model = nullptr;
    if ((st = mi_model_load_gguf(ctx, argv[1], maxseq, &model))) die(ctx, "mi_model_load_gguf", st);
    mi_model_config c;
    mi_model_info(model, &c);
    fprintf(stderr, "minfer-%s: qwen2 L=%d d=%d ff=%d H=%d/%d hd=%d vocab=%d maxseq=%d | q4_0 weights %.1f MB/token, fp16 KV %lld B/position | %d CTAs\n",
            tag, c.n_layer, c.n_embd, c.n_ff, c.n_head, c.n_head_kv, c.head_dim, c.n_vocab, c.max_seq,
            c.q4_weight_bytes_per_token / 1e6, (long long)c.kv_bytes_per_position, c.grid_ctas);

    const bool stop_eos = !raw_ids && !teacher && eos_id >= 0 && eos_id < c.n_vocab;
    for (int w = env_int("WARMUP", 2); w > 0; w--) {             // untimed: clocks, instruction cache, first-touch
        int32_t tok = ids[0], out;
        if ((st = mi_decode(ctx, model, &tok, 1, 1, 0, &out, nullptr, mode, nullptr))) die(ctx, "mi_decode (warm-up)", st);
    }

    if (teacher) {
        // every position is forced; prediction s is compared with ids[s+1] from position teacher-1 on
        std::vector<int32_t> pred(P);
        float* logits = nullptr;
        if ((st = mi_device_malloc(ctx, (size_t)P * c.n_vocab * sizeof(float), (void**)&logits))) die(ctx, "mi_device_malloc", st);
        float ms = 0;
        if (tchunk == 1) {
            if ((st = mi_decode(ctx, model, ids.data(), P, P, 0, pred.data(), logits, mode, &ms))) die(ctx, "mi_decode", st);
        } else {
            for (int i = 0; i < P; i += tchunk) {                // tchunk tokens per weight pass: same logits, bit for bit
                const int mtok = P - i < tchunk ? P - i : tchunk;
                float cms = 0;
                if ((st = mi_verify(ctx, model, ids.data() + i, mtok, i, pred.data() + i, logits + (size_t)i * c.n_vocab, &cms))) die(ctx, "mi_verify", st);
                ms += cms;
            }
        }
        std::vector<float> h((size_t)P * c.n_vocab);
        if ((st = mi_memcpy_to_host(ctx, h.data(), logits, h.size() * sizeof(float)))) die(ctx, "mi_memcpy_to_host", st);
        auto margin_at = [&](int i) {                            // top-1 minus top-2 logit of position i
            const float* lg = h.data() + (size_t)i * c.n_vocab;
            float b1 = -INFINITY, b2 = -INFINITY;
            for (int v = 0; v < c.n_vocab; v++) { if (lg[v] > b1) { b2 = b1; b1 = lg[v]; } else if (lg[v] > b2) b2 = lg[v]; }
            return b1 - b2;
        };
        int agree = 0, total = 0;
        for (int i = teacher - 1; i + 1 < P; i++, total++) {
            if (pred[i] == ids[i + 1]) { agree++; continue; }
            fprintf(stderr, "  pos %d: ref %d, %s %d (%s margin %.4f)\n", i + 1, ids[i + 1], tag, pred[i], tag, margin_at(i));
        }
        // FNV-1a over the bits of every logit of every position: equal hashes mean bit-identical logits
        unsigned long long hsh = 1469598103934665603ull;
        const unsigned char* b = reinterpret_cast<const unsigned char*>(h.data());
        for (size_t i = 0; i < h.size() * 4; i++) { hsh ^= b[i]; hsh *= 1099511628211ull; }
        fprintf(stderr, "teacher-forced top-1 agreement: %d/%d | %d positions in %.1f ms (%.2f ms per %d-token step) | logit hash %016llx\n", agree, total, P,
                ms, ms * tchunk / P, tchunk, hsh);
        mi_device_free(ctx, logits);
        mi_model_free(ctx, model); mi_ctx_destroy(ctx);
        return 0;
    }

    const bool persistent = mode == MI_DECODE_PERSISTENT;
    const int spec = env_int("SPEC", persistent ? 1 : 0);
    const int ngmax = env_int("NGMAX", env_int("NG", 3)), draftk = env_int("DRAFTK", 4);
    std::vector<int32_t> gen;                 // the n_gen generated ids
    std::vector<float> margin;                // their logit margins (where the step kind reports one)
    std::vector<unsigned long long> stamp;    // GPU time of each (ring path)
    double dms = 0, ttft = -1;
    long long n_steps = 0, n_drafted = 0, n_accepted = 0;
    if (stop_eos && (st = mi_model_set_stop_token(model, eos_id))) die(ctx, "mi_model_set_stop_token", st);
    int n_out = n_gen;                        // tokens actually generated: fewer when the end-of-sequence token came up
    const auto t0 = std::chrono::steady_clock::now();
    auto since = [&]() { return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count(); };
    if (spec && n_gen > 0) {
        // lossless n-gram speculation: the library's loop over single-token steps and M-token verify passes
        gen.resize(n_gen); margin.resize(n_gen);
        int64_t stats[4] = {0, 0, 0, 0};
        if ((st = mi_generate_spec(ctx, model, ids.data(), P, n_gen, ngmax, spec >= 2 ? -draftk : draftk, gen.data(), margin.data(), stats))) die(ctx, "mi_generate_spec", st);
        n_out = mi_model_last_count(model);
        dms = since(); ttft = dms / (n_out > 0 ? n_out : 1);
        n_steps = stats[0]; n_drafted = stats[1]; n_accepted = stats[2];
        for (int i = 0; i < n_out; i++) emit(gen[i]);
        printf("\n");
        float minm = 1e30f; int mi = 0;
        for (int i = 0; i < n_out; i++) if (margin[i] < minm) { minm = margin[i]; mi = i; }
        fprintf(stderr, "minfer-%s decode: %d tok in %.1f ms = %.2f tok/s | first token after %.1f ms (prompt %d) | min logit margin %.4f at #%d | prompt included in the time; NGMAX=%d DRAFTK=%d\n",
                tag, n_out, dms, dms > 0 ? n_out * 1e3 / dms : 0.0, ttft, P, minm, mi, ngmax, draftk);
    } else if (n_gen > 0) {
        // prompt: all but its last token, tchunk per weight pass (or one step per token); the last prompt token is the
        // first step of the generation itself, so that every generated id comes with its margin
        float pms = 0;
        std::vector<int32_t> out(P > 0 ? P : 1);
        if (P > 1) {
            if (tchunk == 1) {
                if ((st = mi_decode(ctx, model, ids.data(), P - 1, P - 1, 0, out.data(), nullptr, mode, &pms))) die(ctx, "mi_decode (prefill)", st);
            } else {
                for (int i = 0; i < P - 1; i += tchunk) {
                    const int mtok = P - 1 - i < tchunk ? P - 1 - i : tchunk;
                    float cms = 0;
                    if ((st = mi_verify(ctx, model, ids.data() + i, mtok, i, out.data() + i, nullptr, &cms))) die(ctx, "mi_verify (prefill)", st);
                    pms += cms;
                }
            }
        }
        fprintf(stderr, "minfer-%s prefill: %d tok in %.1f ms (%d per pass)\n", tag, P - 1, pms, tchunk);
        gen.resize(n_gen); margin.resize(n_gen);
        if (persistent) {
            // one launch generates everything; the ids are printed as the kernel publishes them
            mi_token_ring* ring = nullptr;
            if ((st = mi_ring_create(ctx, n_gen, &ring))) die(ctx, "mi_ring_create", st);
            if ((st = mi_decode_run(ctx, model, &ids[P - 1], 1, n_gen, P - 1, ring))) die(ctx, "mi_decode_run", st);
            stamp.resize(n_gen);
            int seen = 0;
            const int32_t* rt; const float* rm; const uint64_t* rn;
            for (;;) {
                int cnt = 0;
                mi_ring_peek(ring, &cnt, &rt, &rm, &rn);
                for (; seen < cnt; seen++) {
                    if (ttft < 0) ttft = since();
                    gen[seen] = rt[seen]; margin[seen] = rm[seen]; stamp[seen] = rn[seen];
                    emit(gen[seen]); fflush(stdout);
                }
                if (seen >= n_gen || (stop_eos && seen > 0 && gen[seen - 1] == eos_id)) break;
                if (since() > 600e3) { fprintf(stderr, "minfer-%s: no token for ten minutes\n", tag); break; }
                std::this_thread::sleep_for(std::chrono::microseconds(100));
            }
            if ((st = mi_ctx_sync(ctx))) die(ctx, "mi_decode_run", st);
            mi_ring_destroy(ctx, ring);
            printf("\n");
            if (seen < n_gen && !(stop_eos && seen > 0 && gen[seen - 1] == eos_id)) return 1;
            n_out = seen;
            dms = n_out > 1 ? (double)(stamp[n_out - 1] - stamp[0]) / 1e6 : 0.0;          // first to last token, on the GPU's clock
        } else {
            float ms = 0;
            if ((st = mi_decode(ctx, model, &ids[P - 1], 1, n_gen, P - 1, gen.data(), nullptr, mode, &ms))) die(ctx, "mi_decode", st);
            n_out = mi_model_last_count(model);
            if ((st = mi_decode_margins(ctx, model, n_out, margin.data()))) die(ctx, "mi_decode_margins", st);
            ttft = since();
            dms = n_out > 1 ? ms * (n_out - 1) / n_out : 0.0;
            for (int i = 0; i < n_out; i++) emit(gen[i]);
            printf("\n");
        }
        n_steps = n_out;
        float minm = 1e30f; int mi = 0;
        for (int i = 0; i < n_out; i++) if (margin[i] < minm) { minm = margin[i]; mi = i; }
        const int timed = n_out - 1;
        fprintf(stderr, "minfer-%s decode: %d tok in %.1f ms = %.2f tok/s | first token after %.1f ms (prompt %d) | min logit margin %.4f at #%d\n", tag, timed,
                dms, dms > 0 ? timed * 1e3 / dms : 0.0, ttft, P, minm, mi);
        if (timed > 0 && dms > 0) {
            const double bytes = (double)c.q4_weight_bytes_per_token + (double)c.kv_bytes_per_position * (P + n_out / 2.0);
            fprintf(stderr, "minfer-%s: %.1f us/token, %.0f GB/s of weight + KV bytes (%.1f MB/token)\n", tag, dms * 1e3 / timed,
                    bytes * timed / (dms * 1e-3) / 1e9, bytes / 1e6);
        }
    }
    if (n_steps > 0)
        fprintf(stderr, "minfer-%s: %lld generation steps, %.2f tokens/step | drafted %lld, accepted %lld (%.0f%%)%s\n", tag, n_steps,
                (double)n_out / n_steps, n_drafted, n_accepted, n_drafted ? 100.0 * n_accepted / n_drafted : 0.0, spec ? "" : " [SPEC=0]");
    if (getenv("SEGMENTS") && !stamp.empty()) {                      // tok/s over consecutive windows: the slope with depth
        const int w = atoi(getenv("SEGMENTS"));
        for (int i = 0; w > 0 && i + w < n_out; i += w)
            fprintf(stderr, "  tokens %4d-%4d (pos %4d): %.1f tok/s\n", i, i + w, P + i, w * 1e9 / (double)(stamp[i + w] - stamp[i]));
    }
    if (env_int("PROFILE", 0)) {
        void* p = nullptr; int64_t nb = 0;
        if (mi_model_state_ptr(model, MI_STATE_PROFILE, &p, &nb) == MI_OK && p) {
            unsigned long long pr[32];
            mi_memcpy_to_host(ctx, pr, p, sizeof pr);
            // slots (csrc/decode_kernel.cuh): 2k = prologue of phase kind k, 2k+1 = its tail after the unit loop, 12 = waiting
            // for other CTAs' data, 13 = step prologue, 14..16 = attention (q staging, scan, fold + merge), 18 / 19 = tile loops and
            // fold + epilogue of the per-layer GEMV phases
            const char* ph[6] = {"P1 QKV", "P2 attention", "P3 Wo", "P4 gate/up", "P5 down", "lm_head"};
            const double steps = (double)(P + n_gen - 1 + env_int("WARMUP", 2));   // (with TCHUNK > 1 the prompt is not in the profile)
            auto us = [&](int k) { return pr[k] / 1e3 / steps; };
            double tot = 0;
            for (int k = 0; k < 6; k++) {
                const double stage = k == 1 ? us(14) : us(2 * k), work = k == 1 ? us(15) + us(16) + us(3) : us(2 * k + 1);
                fprintf(stderr, "  %-13s %8.1f %8.1f us/token (prologue, %s)\n", ph[k], stage, work, k == 1 ? "scan + fold" : k == 5 ? "lm_head rows + argmax" : "tail");
                tot += stage + work;
            }
            fprintf(stderr, "  %-13s %8.1f %8.1f us/token (tile loops, fold + epilogue of P1 / P3 / P4 / P5)\n", "GEMV units", us(18), us(19));
            tot += us(18) + us(19);
            fprintf(stderr, "  %-13s %8.1f us/token; step prologue %.1f; total %.1f us/position on the profiled CTA\n", "waits", us(12), us(13),
                    tot + us(12) + us(13));
        }
    }
    if (getenv("MARGINS") && !margin.empty())
        for (int i = 0; i < n_out; i++) fprintf(stderr, "%d:%d:%.4f%c", i, gen[i], margin[i], i + 1 < n_out ? ' ' : '\n');
    mi_model_free(ctx, model);
    mi_ctx_destroy(ctx);
    return 0;
}

}  // namespace mib200
