// Shared body of the two driver programs.  They keep the command line, environment
// knobs and stdout / stderr line shapes of the reference's drivers
//     <exe> <model.gguf> <n_gen> <id0> <id1> ...
// (reference src/cuda_infer.cu:844-1201 and src/mega.cu:1009-1259) and call the CUDA
// path only through the C ABI of minfer_b200.h.  Like the reference's CK()/REQUIRE()
// they print and exit on any error; the library itself never exits.
//
// stdout: the n_gen greedy ids separated by a space, then a newline (the first id
// is the prediction after the last prompt token: src/cpu_infer.cpp:161-167).
// Token ids are always printed (the reference's RAWIDS=1 form): detokenized text
// needs a real vocabulary and is outside this path.
//
// Environment: TEACHER=k (ids are a reference sequence whose first k are the
// prompt; report top-1 agreement at every later position, as
// src/cuda_infer.cu:1148-1160 / src/mega.cu:1192-1205), MAXSEQ=n (KV cache
// positions; default prompt + n_gen + 8), WARMUP=n (untimed steps before the run),
// PROFILE=1 (per-phase time on CTA 0, persistent engine), GPU=i (device index),
// TCHUNK=m (prompt / teacher-forced tokens per weight pass through the M-token step,
// 1..16, default 16; 1 = one decode step per token; src/cuda_infer.cu:1130-1144).
#pragma once
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

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
    if (!env_int("RAWIDS", 0)) fprintf(stderr, "minfer-%s: text output is outside this path; printing token ids (RAWIDS=1 form)\n", tag);

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
        int agree = 0, total = 0;
        for (int i = teacher - 1; i + 1 < P; i++, total++) {
            if (pred[i] == ids[i + 1]) { agree++; continue; }
            fprintf(stderr, "  pos %d: ref %d, %s %d\n", i + 1, ids[i + 1], tag, pred[i]);
        }
        // FNV-1a over the bits of every logit of every position: equal hashes mean bit-identical logits
        std::vector<float> h((size_t)P * c.n_vocab);
        if ((st = mi_memcpy_to_host(ctx, h.data(), logits, h.size() * sizeof(float)))) die(ctx, "mi_memcpy_to_host", st);
        unsigned long long hsh = 1469598103934665603ull;
        const unsigned char* b = reinterpret_cast<const unsigned char*>(h.data());
        for (size_t i = 0; i < h.size() * 4; i++) { hsh ^= b[i]; hsh *= 1099511628211ull; }
        fprintf(stderr, "teacher-forced top-1 agreement: %d/%d | %d positions in %.1f ms | logit hash %016llx\n", agree, total, P, ms, hsh);
        mi_device_free(ctx, logits);
        mi_model_free(ctx, model); mi_ctx_destroy(ctx);
        return 0;
    }

    // prefill: tchunk prompt tokens per weight pass (or one step per token); the last one predicts generated token #1
    std::vector<int32_t> out(P > 0 ? P : 1);
    float pms = 0;
    const auto t0 = std::chrono::steady_clock::now();
    if (tchunk == 1) {
        if ((st = mi_decode(ctx, model, ids.data(), P, P, 0, out.data(), nullptr, mode, &pms))) die(ctx, "mi_decode (prefill)", st);
    } else {
        for (int i = 0; i < P; i += tchunk) {
            const int mtok = P - i < tchunk ? P - i : tchunk;
            float cms = 0;
            if ((st = mi_verify(ctx, model, ids.data() + i, mtok, i, out.data() + i, nullptr, &cms))) die(ctx, "mi_verify (prefill)", st);
            pms += cms;
        }
    }
    const double ttft = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    fprintf(stderr, "minfer-%s prefill: %d tok in %.1f ms (%d per pass)\n", tag, P, pms, tchunk);
    std::vector<int32_t> gen;
    int32_t next = out[P - 1];
    gen.push_back(next);
    float dms = 0;
    if (n_gen > 1) {
        std::vector<int32_t> more(n_gen - 1);
        if ((st = mi_decode(ctx, model, &next, 1, n_gen - 1, P, more.data(), nullptr, mode, &dms))) die(ctx, "mi_decode", st);
        gen.insert(gen.end(), more.begin(), more.end());
    }
    for (int i = 0; i < n_gen && i < (int)gen.size(); i++) printf("%d ", gen[i]);
    printf("\n");
    const int timed = n_gen - 1;
    fprintf(stderr, "minfer-%s decode: %d tok in %.1f ms = %.2f tok/s | first token after %.1f ms (prompt %d)\n", tag, timed, dms,
            dms > 0 ? timed * 1e3 / dms : 0.0, ttft, P);
    if (timed > 0) {
        const double bytes = (double)c.q4_weight_bytes_per_token + (double)c.kv_bytes_per_position * (P + n_gen / 2.0);
        fprintf(stderr, "minfer-%s: %.1f us/token, %.0f GB/s of weight + KV bytes (%.1f MB/token)\n", tag, dms * 1e3 / timed,
                bytes * timed / (dms * 1e-3) / 1e9, bytes / 1e6);
    }
    if (env_int("PROFILE", 0)) {
        void* p = nullptr; int64_t nb = 0;
        if (mi_model_state_ptr(model, MI_STATE_PROFILE, &p, &nb) == MI_OK && p) {
            unsigned long long pr[32];
            mi_memcpy_to_host(ctx, pr, p, sizeof pr);
            // slots (csrc/decode_kernel.cuh): 2k = prologue of phase kind k, 2k+1 = its tail after the unit loop, 12 = grid
            // barrier, 13 = step prologue, 14..16 = attention (q staging, scan, fold + merge), 18 / 19 = tile loops and
            // fold + epilogue of the per-layer GEMV phases
            const char* ph[6] = {"P1 QKV", "P2 attention", "P3 Wo", "P4 gate/up", "P5 down", "lm_head"};
            const double steps = (double)(P + n_gen - 1 + env_int("WARMUP", 2));
            auto us = [&](int k) { return pr[k] / 1e3 / steps; };
            double tot = 0;
            for (int k = 0; k < 6; k++) {
                const double stage = k == 1 ? us(14) : us(2 * k), work = k == 1 ? us(15) + us(16) + us(3) : us(2 * k + 1);
                fprintf(stderr, "  %-13s %8.1f %8.1f us/token (prologue, %s)\n", ph[k], stage, work, k == 1 ? "scan + fold" : k == 5 ? "lm_head rows + argmax" : "tail");
                tot += stage + work;
            }
            fprintf(stderr, "  %-13s %8.1f %8.1f us/token (tile loops, fold + epilogue of P1 / P3 / P4 / P5)\n", "GEMV units", us(18), us(19));
            tot += us(18) + us(19);
            fprintf(stderr, "  %-13s %8.1f us/token; step prologue %.1f; total %.1f us/position on CTA 0\n", "grid barrier", us(12), us(13),
                    tot + us(12) + us(13));
        }
    }
    mi_model_free(ctx, model);
    mi_ctx_destroy(ctx);
    return 0;
}

}  // namespace mib200
