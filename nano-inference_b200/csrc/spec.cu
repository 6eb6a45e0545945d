// Lossless n-gram (prompt-lookup) speculative decoding on top of the two step kinds of this library: the single-token
// decode step and the M-token step, whose logits for a token are the same bits whatever else shares the pass.  A drafted
// token is kept only if it equals the greedy token the model itself produces at that position, so the output is, token
// for token, what plain greedy decoding gives.
//
// Follows the reference's host-side loop (src/cuda_infer.cu:1203-1292: draft from the latest earlier occurrence of the
// current suffix, verify cur + draft in one weight pass, accept the longest matching prefix, continue from the model's
// own token at the first mismatch, an acceptance estimate that switches drafting off while it does not pay and probes
// now and then) with the longest-suffix-first lookup of its in-kernel form (src/mega.cu:557-576: n-gram lengths
// ngmax .. 1) and that form's choice of the draft length (src/mega.cu:579-589): the K that maximizes expected tokens per
// unit of time for the current acceptance estimate, E(K) = (1 - a^(K+1)) / (1 - a).  The reference prices a step of K
// extra tokens with one constant slope; here the two step kinds are different code paths, so the loop prices them by what
// it has measured itself: the device time of its own single-token steps and of its own M-token passes.
#include "model.cuh"

#include <algorithm>
#include <vector>

using namespace mi;

namespace {

// the up to kmax tokens that followed the latest earlier occurrence of the last ng tokens of seq, ng = ngmax .. 1
int ngram_draft(const std::vector<int32_t>& seq, int ngmax, int kmax, int32_t* draft) {
    const int L = (int)seq.size();
    if (kmax <= 0) return 0;
    for (int ng = ngmax; ng >= 1; ng--) {
        if (L < ng + 1) continue;
        for (int j = L - ng - 1; j >= 0; j--) {
            bool m = true;
            for (int k = 0; k < ng && m; k++) m = seq[j + k] == seq[L - ng + k];
            if (m) {
                const int n = std::min(kmax, L - (j + ng));
                for (int k = 0; k < n; k++) draft[k] = seq[j + ng + k];
                return n;
            }
        }
    }
    return 0;
}

}  // namespace

extern "C" int mi_generate_spec(mi_ctx* ctx, mi_model* m, const int32_t* prompt_host, int n_prompt, int n_gen, int ngmax, int draftk,
                                int32_t* out_tokens_host, float* margins_host, int64_t* stats) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m || !prompt_host || !out_tokens_host || n_prompt < 1 || n_gen < 0) return set_error(ctx, MI_ERR_INVALID, "generate_spec: bad argument");
    if (m->tp_world != 1) return set_error(ctx, MI_ERR_UNSUPPORTED, "generate_spec: the M-token step runs on an unsharded model");
    if (n_prompt + n_gen > m->max_seq) return set_error(ctx, MI_ERR_LIMIT, "generate_spec: %d prompt + %d generated tokens exceed the KV cache of %d", n_prompt, n_gen, m->max_seq);
    constexpr int kMaxPass = 16;                                     // tokens per M-token pass
    ngmax = std::max(1, std::min(ngmax, 8));
    const bool forced = draftk < 0;                                   // draft whenever a draft exists, whatever it costs
    draftk = std::max(0, std::min(forced ? -draftk : draftk, kMaxPass - 1));
    int64_t n_steps = 0, n_drafted = 0, n_accepted = 0, n_specruns = 0;
    int st;
    // prompt: up to 16 tokens per weight pass; the last token's prediction is generated token #1
    std::vector<int32_t> seq(prompt_host, prompt_host + n_prompt);
    int32_t pred[kMaxPass];
    float prompt_ms[kMaxPass + 1] = {0.f};                           // device time of the prompt's passes, by pass size
    for (int i = 0; i < n_prompt; i += kMaxPass) {
        const int mt = std::min(kMaxPass, n_prompt - i);
        float pms = 0.f;
        if ((st = mi_verify(ctx, m, prompt_host + i, mt, i, pred, nullptr, &pms))) return st;
        prompt_ms[mt] = pms;
        if (i + mt == n_prompt) seq.push_back(pred[mt - 1]);
    }
    // margin of the token that is current: the logit margin of the step that predicted it
    float mg[kMaxPass], cur_margin = 0.f;
    if (margins_host) {
        const int last = (n_prompt - 1) % kMaxPass;
        if ((st = mi_verify_margins(ctx, m, last + 1, mg))) return st;
        cur_margin = mg[last];
    }
    int32_t cur = seq.back();
    int pos = n_prompt, n_emit = 0;
    // What a step costs, as measured by this loop (device milliseconds, running averages): a single-token step, and an
    // M-token pass for every M used so far; an M not yet seen is priced from the nearest seen one along the measured shape
    // of the pass time (about 0.49 + 0.032 M of the 16-token pass).
    float t_dec = 0.f, t_ver[kMaxPass + 1] = {0.f};
    auto learn = [](float& avg, float ms) { if (ms > 0.f) avg = avg > 0.f ? 0.8f * avg + 0.2f * ms : ms; };
    for (int M = 1; M <= kMaxPass; M++) t_ver[M] = prompt_ms[M];     // the prompt's own passes are the first measurements
    auto pass_ms = [&](int M) {
        if (t_ver[M] > 0.f) return t_ver[M];
        for (int d = 1; d <= kMaxPass; d++)
            for (int q : {M - d, M + d})
                if (q >= 1 && q <= kMaxPass && t_ver[q] > 0.f) return t_ver[q] * (0.49f + 0.032f * M) / (0.49f + 0.032f * q);
        return 0.f;
    };
    // acceptance probability of one drafted token (running estimate), and the draft length that pays best for it
    float alpha = 0.6f; long probe = 0;
    auto best_len = [&](int kmax) {
        if (t_dec <= 0.f) return 0;                                   // nothing to compare with yet: take a plain step and measure it
        int kb = 0; float vb = 1.f / t_dec, pw = alpha;
        for (int K = 1; K <= kmax; K++) {
            pw *= alpha;                                              // alpha^(K+1)
            const float tv = pass_ms(K + 1);
            if (tv <= 0.f) continue;
            const float expect = alpha < 0.999f ? (1.f - pw) / (1.f - alpha) : (float)(K + 1);
            if (expect / tv > vb) { vb = expect / tv; kb = K; }
        }
        return kb;
    };
    int32_t draft[kMaxPass], hb[kMaxPass], r[kMaxPass];
    const int stop = m->stop_token;                                   // generation ends with this token (src/cuda_infer.cu:1254,1272-1275)
    auto stopped = [&]() { return stop >= 0 && n_emit > 0 && out_tokens_host[n_emit - 1] == stop; };
    while (n_emit < n_gen && !stopped()) {
        int K = draftk > 0 ? ngram_draft(seq, ngmax, draftk, draft) : 0;
        K = std::min(K, m->max_seq - 1 - pos);                         // KV headroom
        K = std::min(K, n_gen - n_emit - 1);                          // nothing is gained by drafting past the end
        if (K > 0 && !forced) {
            const int want = best_len(K);
            // while drafting does not pay, every 32nd step still tests one drafted token, so that the estimate can recover
            // (src/cuda_infer.cu:1233-1243); a test that succeeds is followed by the next one at once
            if (want == 0 && t_dec > 0.f && (probe++ % 32) == 0) K = 1;
            else K = want;
        }
        if (K <= 0) {
            int32_t nxt; float ms = 0.f;
            if ((st = mi_decode(ctx, m, &cur, 1, 1, pos, &nxt, nullptr, MI_DECODE_PERSISTENT, &ms))) return st;
            learn(t_dec, ms);
            if (margins_host) { margins_host[n_emit] = cur_margin; if ((st = mi_decode_margins(ctx, m, 1, &cur_margin))) return st; }
            out_tokens_host[n_emit++] = cur;
            cur = nxt; pos++; seq.push_back(cur);
            n_steps++;
            continue;
        }
        const int T = K + 1;                                          // cur and the draft at positions pos .. pos+K
        hb[0] = cur;
        for (int k = 0; k < K; k++) hb[1 + k] = draft[k];
        float vms = 0.f;
        if ((st = mi_verify(ctx, m, hb, T, pos, r, nullptr, &vms))) return st;          // r[j] = the model's token after hb[j]
        learn(t_ver[T], vms);
        int a = 0;
        while (a < K && draft[a] == r[a]) a++;
        if (margins_host) {
            if ((st = mi_verify_margins(ctx, m, T, mg))) return st;
            margins_host[n_emit] = cur_margin;
            for (int k = 0; k < a && n_emit + 1 + k < n_gen; k++) margins_host[n_emit + 1 + k] = mg[k];      // draft[k] was predicted by pass row k
            cur_margin = mg[a];
        }
        out_tokens_host[n_emit++] = cur;
        for (int k = 0; k < a && n_emit < n_gen && !stopped(); k++) out_tokens_host[n_emit++] = draft[k];
        for (int k = 0; k < a; k++) seq.push_back(draft[k]);
        cur = r[a]; pos += a + 1; seq.push_back(cur);                  // the model's own token at the first mismatch
        alpha = 0.7f * alpha + 0.3f * ((float)a / (float)std::min(K, a + 1));       // a successes in the a (+1, if one failed) drafts that were tested
        if (a == K) probe = 0;
        n_steps++; n_specruns++; n_drafted += K; n_accepted += a;
    }
    m->last_count = n_emit;
    if (stats) { stats[0] = n_steps; stats[1] = n_drafted; stats[2] = n_accepted; stats[3] = n_specruns; }
    return MI_OK;
}
