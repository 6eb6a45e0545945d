// gguf_synth: writes a seeded, random-init Qwen2-architecture GGUF file (all q4_0 unless told otherwise)
// that the reference programs (cpu_infer / cuda_infer / mega) and this engine
// all accept.  It stands in for a published model file: there is no network for
// checkpoints, and the benchmark configurations ask for seeded normal weights.
//
//   gguf_synth <out.gguf> --preset {tiny|0.5b|1.5b|3b} [--seed S] [--std 0.02]
//              [--bias-std 0.02] [--norm-std 0] [--layers L --embd E --ff F
//              --heads H --kv-heads K --vocab V]
//              [--emb-type T] [--head-type T] [--down-type T] [--untied] [--eos ID]
//
// The last four make files shaped like published ones, which store the token embedding, the lm_head and ffn_down in
// other block formats (T = 2 Q4_0, 3 Q4_1, 8 Q8_0, 14 Q6_K).  --untied (implied when the head and embedding types
// differ) draws output.weight from its own random stream instead of repeating the embedding's bytes.
//
// File layout: the GGUF v3 subset the reference reader parses (reference
// src/gguf.h:183-222).  Metadata keys and tensor names are the ones the
// reference drivers look up (src/cpu_infer.cpp:71-98).  The vocabulary size is
// the length of tokenizer.ggml.tokens (src/cpu_infer.cpp:79), so V placeholder
// strings are written: token b < 256 is the byte-level BPE spelling of byte b (so that
// a detokenizer has every byte to decode), token i >= 256 is "t<i>" preceded by the
// spelling of a space.  tokenizer.ggml.eos_token_id is V-1 unless --eos says
// otherwise.  The lm_head is tied: the same q4_0 bytes are stored as
// token_embd.weight and as output.weight, which cpu_infer requires to exist
// (src/cpu_infer.cpp:85).
//
// Random numbers are counter based (splitmix64 of seed, tensor id and element
// index, Box-Muller on pairs), so any element can be regenerated independently
// and the result does not depend on the thread count.
//
// q4_0 quantization is ggml's published reference rule: per 32 values, take the
// value of largest magnitude with its sign, d = that / -8, store fp16(d); each
// nibble is min(15, trunc(x * (1/d) + 8.5)); elements 0..15 go to the low
// nibbles of the 16 bytes, elements 16..31 to the high nibbles.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

namespace {

struct Shape { int layers, embd, ff, heads, kv_heads, vocab; };

inline uint64_t splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// two independent N(0,1) values for pair index p of stream `key`
inline void normal_pair(uint64_t key, uint64_t p, float& a, float& b) {
    uint64_t r1 = splitmix64(key + 2 * p), r2 = splitmix64(key + 2 * p + 1);
    float u1 = ((float)(r1 >> 40) + 1.0f) * (1.0f / 16777217.0f);   // (0,1]
    float u2 = (float)(r2 >> 40) * (1.0f / 16777216.0f);             // [0,1)
    float r = std::sqrt(-2.0f * std::log(u1)), t = 6.28318530717958647692f * u2;
    a = r * std::cos(t); b = r * std::sin(t);
}

inline void fill_normal(float* out, int64_t n, uint64_t key, int64_t first, float std_) {
    // element e comes from pair e/2; first is the global element index of out[0] (even)
    for (int64_t i = 0; i < n; i += 2) {
        float a, b; normal_pair(key, (uint64_t)(first + i) / 2, a, b);
        out[i] = a * std_; if (i + 1 < n) out[i + 1] = b * std_;
    }
}

inline uint16_t f32_to_f16(float x) {
    uint32_t f; memcpy(&f, &x, 4);
    uint32_t sign = (f >> 16) & 0x8000u, e = (f >> 23) & 0xFFu, m = f & 0x7FFFFFu;
    if (e == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? 0x200u : 0));
    int32_t ne = (int32_t)e - 112;
    if (ne >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (ne <= 0) {
        if (ne < -10) return (uint16_t)sign;
        m |= 0x800000u;
        uint32_t sh = (uint32_t)(14 - ne), hm = m >> sh, rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
        if (rem > half || (rem == half && (hm & 1))) hm++;
        return (uint16_t)(sign | hm);
    }
    uint32_t hm = m >> 13, rem = m & 0x1FFFu;
    uint16_t o = (uint16_t)(sign | ((uint32_t)ne << 10) | hm);
    if (rem > 0x1000u || (rem == 0x1000u && (hm & 1))) o++;
    return o;
}

void quantize_row_q4_0(const float* x, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / 32; b++, out += 18) {
        const float* xb = x + b * 32;
        float amax = 0.f, mx = 0.f;
        for (int j = 0; j < 32; j++) { float a = std::fabs(xb[j]); if (a > amax) { amax = a; mx = xb[j]; } }
        const float d = mx / -8.f, id = d != 0.f ? 1.f / d : 0.f;
        const uint16_t dh = f32_to_f16(d); memcpy(out, &dh, 2);
        for (int j = 0; j < 16; j++) {
            int q0 = (int)(int8_t)(xb[j] * id + 8.5f), q1 = (int)(int8_t)(xb[j + 16] * id + 8.5f);
            if (q0 > 15) q0 = 15;
            if (q1 > 15) q1 = 15;
            out[2 + j] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

// ---- the other block formats.  Layouts as the reference reader decodes them (reference src/gguf.h:103-140); the
// quantization rules are plain nearest-value ones, stated here in full (any well-formed blocks serve the tests).

// Q8_0: fp16 d = amax / 127, 32 x int8 q = round(x / d)
void quantize_row_q8_0(const float* x, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / 32; b++, out += 34) {
        const float* xb = x + b * 32;
        float amax = 0.f;
        for (int j = 0; j < 32; j++) amax = std::fmax(amax, std::fabs(xb[j]));
        const float d = amax / 127.f, id = d != 0.f ? 1.f / d : 0.f;
        const uint16_t dh = f32_to_f16(d); memcpy(out, &dh, 2);
        for (int j = 0; j < 32; j++) out[2 + j] = (uint8_t)(int8_t)std::lrintf(xb[j] * id);
    }
}
// Q4_1: fp16 d = (max - min) / 15, fp16 m = min, nibbles q = min(15, trunc((x - min) / d + 0.5)); elements 0..15 low, 16..31 high
void quantize_row_q4_1(const float* x, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / 32; b++, out += 20) {
        const float* xb = x + b * 32;
        float mn = xb[0], mx = xb[0];
        for (int j = 1; j < 32; j++) { mn = std::fmin(mn, xb[j]); mx = std::fmax(mx, xb[j]); }
        const float d = (mx - mn) / 15.f, id = d != 0.f ? 1.f / d : 0.f;
        const uint16_t dh = f32_to_f16(d), mh = f32_to_f16(mn); memcpy(out, &dh, 2); memcpy(out + 2, &mh, 2);
        for (int j = 0; j < 16; j++) {
            int q0 = (int)((xb[j] - mn) * id + 0.5f), q1 = (int)((xb[j + 16] - mn) * id + 0.5f);
            q0 = q0 > 15 ? 15 : q0; q1 = q1 > 15 ? 15 : q1;
            out[4 + j] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}
// Q6_K: 256 elements = ql[128] | qh[64] | int8 scale[16] | fp16 d.  Each run of 16 elements j has scale[j];
// value = d * scale * (q - 32) with 6-bit q.  Rule: s_j = amax_j / 31, d = max_j s_j / 127, scale_j = round(s_j / d),
// q = clamp(round(x / (d * scale_j)), -32, 31) + 32.
void quantize_row_q6_k(const float* x, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / 256; b++, out += 210) {
        const float* xb = x + b * 256;
        float sj[16], smax = 0.f;
        for (int j = 0; j < 16; j++) {
            float a = 0.f;
            for (int i = 0; i < 16; i++) a = std::fmax(a, std::fabs(xb[j * 16 + i]));
            sj[j] = a / 31.f; smax = std::fmax(smax, sj[j]);
        }
        const float d = smax / 127.f;
        const uint16_t dh = f32_to_f16(d);
        memset(out, 0, 210); memcpy(out + 208, &dh, 2);
        for (int j = 0; j < 16; j++) {
            const int sc = d > 0.f ? (int)std::lrintf(sj[j] / d) : 0;
            out[192 + j] = (uint8_t)(int8_t)(sc > 127 ? 127 : sc);
            const float step = d * (float)(int8_t)out[192 + j], is = step > 0.f ? 1.f / step : 0.f;
            for (int i = 0; i < 16; i++) {
                const int e = j * 16 + i, nh = e >> 7, qd = (e >> 5) & 3, l = e & 31;
                int q = (int)std::lrintf(xb[e] * is); q = (q < -32 ? -32 : q > 31 ? 31 : q) + 32;
                out[64 * nh + l + 32 * (qd & 1)] |= (uint8_t)((q & 0x0F) << (qd < 2 ? 0 : 4));
                out[128 + 32 * nh + l] |= (uint8_t)((q >> 4) << (2 * qd));
            }
        }
    }
}

inline size_t type_row_bytes(uint32_t type, int64_t cols) {
    switch (type) {
        case 0: return (size_t)cols * 4;
        case 2: return (size_t)cols / 32 * 18;
        case 3: return (size_t)cols / 32 * 20;
        case 8: return (size_t)cols / 32 * 34;
        case 14: return (size_t)cols / 256 * 210;
    }
    return 0;
}

struct TensorSpec {
    std::string name; uint32_t type; int64_t cols, rows; uint64_t key; float std_; float mean;
    int alias = -1;            // index of the tensor whose bytes this one repeats
    uint64_t offset = 0; size_t nbytes = 0;
};

struct Writer {
    FILE* f; uint64_t pos = 0;
    void raw(const void* p, size_t n) { if (fwrite(p, 1, n, f) != n) { perror("gguf_synth: write"); exit(1); } pos += n; }
    template <typename T> void v(T x) { raw(&x, sizeof(T)); }
    void s(const std::string& x) { v<uint64_t>(x.size()); raw(x.data(), x.size()); }
    void kv_u32(const std::string& k, uint32_t x) { s(k); v<uint32_t>(4); v<uint32_t>(x); }
    void kv_f32(const std::string& k, float x) { s(k); v<uint32_t>(6); v<float>(x); }
    void kv_str(const std::string& k, const std::string& x) { s(k); v<uint32_t>(8); s(x); }
    void pad(uint64_t a) { static const char z[64] = {0}; while (pos % a) raw(z, 1); }
};

void gen_tensor(const TensorSpec& t, std::vector<uint8_t>& buf, unsigned nthreads) {
    buf.resize(t.nbytes);
    if (t.type == 0) {          // F32
        float* o = (float*)buf.data();
        fill_normal(o, t.cols * t.rows, t.key, 0, t.std_);
        if (t.mean != 0.f) for (int64_t i = 0; i < t.cols * t.rows; i++) o[i] += t.mean;
        return;
    }
    const int64_t row_bytes = (int64_t)type_row_bytes(t.type, t.cols);
    auto work = [&](int64_t r0, int64_t r1) {
        std::vector<float> row((size_t)t.cols);
        for (int64_t r = r0; r < r1; r++) {
            fill_normal(row.data(), t.cols, t.key, r * t.cols, t.std_);
            uint8_t* o = buf.data() + r * row_bytes;
            if (t.type == 3) quantize_row_q4_1(row.data(), t.cols, o);
            else if (t.type == 8) quantize_row_q8_0(row.data(), t.cols, o);
            else if (t.type == 14) quantize_row_q6_k(row.data(), t.cols, o);
            else quantize_row_q4_0(row.data(), t.cols, o);
        }
    };
    if (nthreads <= 1 || t.rows < 64) { work(0, t.rows); return; }
    std::vector<std::thread> th;
    for (unsigned i = 0; i < nthreads; i++)
        th.emplace_back(work, t.rows * i / nthreads, t.rows * (i + 1) / nthreads);
    for (auto& x : th) x.join();
}

}  // namespace

int main(int argc, char** argv) {
    if (argc < 2) {
        fprintf(stderr, "usage: %s <out.gguf> --preset {tiny|0.5b|1.5b|3b} [--seed S] [--std X] [--bias-std X] "
                        "[--norm-std X] [--layers L --embd E --ff F --heads H --kv-heads K --vocab V]\n", argv[0]);
        return 1;
    }
    Shape sh{2, 128, 256, 4, 2, 512};
    uint64_t seed = 1234; float wstd = 0.02f, bstd = 0.02f, nstd = 0.f;
    uint32_t emb_type = 2, head_type = 2, down_type = 2; bool untied = false; int eos = -1;
    auto block_type = [&](const char* v) -> uint32_t {
        const int t = atoi(v);
        if (t != 2 && t != 3 && t != 8 && t != 14) { fprintf(stderr, "gguf_synth: block type %d is not one of 2, 3, 8, 14\n", t); exit(1); }
        return (uint32_t)t;
    };
    for (int i = 2; i < argc; i++) {
        std::string a = argv[i];
        auto next = [&]() -> const char* { if (i + 1 >= argc) { fprintf(stderr, "missing value for %s\n", a.c_str()); exit(1); } return argv[++i]; };
        if (a == "--preset") {
            std::string p = next();
            if (p == "tiny") sh = {2, 128, 256, 4, 2, 512};
            else if (p == "0.5b") sh = {24, 896, 4864, 14, 2, 151936};
            else if (p == "1.5b") sh = {28, 1536, 8960, 12, 2, 151936};
            else if (p == "3b") sh = {36, 2048, 11008, 16, 2, 151936};
            else { fprintf(stderr, "unknown preset %s\n", p.c_str()); return 1; }
        }
        else if (a == "--seed") seed = strtoull(next(), nullptr, 10);
        else if (a == "--std") wstd = (float)atof(next());
        else if (a == "--bias-std") bstd = (float)atof(next());
        else if (a == "--norm-std") nstd = (float)atof(next());
        else if (a == "--layers") sh.layers = atoi(next());
        else if (a == "--embd") sh.embd = atoi(next());
        else if (a == "--ff") sh.ff = atoi(next());
        else if (a == "--heads") sh.heads = atoi(next());
        else if (a == "--kv-heads") sh.kv_heads = atoi(next());
        else if (a == "--vocab") sh.vocab = atoi(next());
        else if (a == "--emb-type") emb_type = block_type(next());
        else if (a == "--head-type") head_type = block_type(next());
        else if (a == "--down-type") down_type = block_type(next());
        else if (a == "--untied") untied = true;
        else if (a == "--eos") eos = atoi(next());
        else { fprintf(stderr, "unknown option %s\n", a.c_str()); return 1; }
    }
    if (sh.embd % 32 || sh.ff % 32 || sh.embd % sh.heads || sh.heads % sh.kv_heads) {
        fprintf(stderr, "gguf_synth: embd and ff must be multiples of 32; heads must divide embd; kv-heads must divide heads\n");
        return 1;
    }
    const int hd = sh.embd / sh.heads, kvd = hd * sh.kv_heads;
    if (((emb_type == 14 || head_type == 14) && sh.embd % 256) || (down_type == 14 && sh.ff % 256)) {
        fprintf(stderr, "gguf_synth: a Q6_K tensor needs a row length that is a multiple of 256\n");
        return 1;
    }
    if (head_type != emb_type) untied = true;

    std::vector<TensorSpec> ts;
    uint64_t tid = 0;
    auto add = [&](const std::string& n, uint32_t type, int64_t cols, int64_t rows, float sd, float mean) {
        TensorSpec t; t.name = n; t.type = type; t.cols = cols; t.rows = rows; t.std_ = sd; t.mean = mean;
        t.key = splitmix64(seed ^ splitmix64(++tid * 0xD1B54A32D192ED03ull));
        t.nbytes = (size_t)rows * type_row_bytes(type, cols);
        ts.push_back(t);
    };
    add("token_embd.weight", emb_type, sh.embd, sh.vocab, wstd, 0.f);
    add("output.weight", head_type, sh.embd, sh.vocab, wstd, 0.f); if (!untied) ts.back().alias = 0;
    add("output_norm.weight", 0, sh.embd, 1, nstd, 1.f);
    for (int l = 0; l < sh.layers; l++) {
        std::string p = "blk." + std::to_string(l) + ".";
        add(p + "attn_norm.weight", 0, sh.embd, 1, nstd, 1.f);
        add(p + "attn_q.weight", 2, sh.embd, sh.embd, wstd, 0.f);
        add(p + "attn_q.bias", 0, sh.embd, 1, bstd, 0.f);
        add(p + "attn_k.weight", 2, sh.embd, kvd, wstd, 0.f);
        add(p + "attn_k.bias", 0, kvd, 1, bstd, 0.f);
        add(p + "attn_v.weight", 2, sh.embd, kvd, wstd, 0.f);
        add(p + "attn_v.bias", 0, kvd, 1, bstd, 0.f);
        add(p + "attn_output.weight", 2, sh.embd, sh.embd, wstd, 0.f);
        add(p + "ffn_norm.weight", 0, sh.embd, 1, nstd, 1.f);
        add(p + "ffn_gate.weight", 2, sh.embd, sh.ff, wstd, 0.f);
        add(p + "ffn_up.weight", 2, sh.embd, sh.ff, wstd, 0.f);
        add(p + "ffn_down.weight", down_type, sh.ff, sh.embd, wstd, 0.f);
    }
    uint64_t off = 0;
    for (auto& t : ts) { t.offset = off; off += (t.nbytes + 31) / 32 * 32; }

    FILE* f = fopen(argv[1], "wb");
    if (!f) { perror("gguf_synth: open output"); return 1; }
    static char iobuf[1 << 22]; setvbuf(f, iobuf, _IOFBF, sizeof iobuf);
    Writer w{f};
    w.v<uint32_t>(0x46554747u); w.v<uint32_t>(3);
    w.v<uint64_t>(ts.size()); w.v<uint64_t>(12);
    w.kv_str("general.architecture", "qwen2");
    w.kv_str("general.name", "synthetic-qwen2-q4_0");
    w.kv_u32("general.alignment", 32);
    w.kv_u32("qwen2.block_count", (uint32_t)sh.layers);
    w.kv_u32("qwen2.embedding_length", (uint32_t)sh.embd);
    w.kv_u32("qwen2.feed_forward_length", (uint32_t)sh.ff);
    w.kv_u32("qwen2.attention.head_count", (uint32_t)sh.heads);
    w.kv_u32("qwen2.attention.head_count_kv", (uint32_t)sh.kv_heads);
    w.kv_f32("qwen2.rope.freq_base", 1e6f);
    w.kv_f32("qwen2.attention.layer_norm_rms_epsilon", 1e-6f);
    w.kv_u32("tokenizer.ggml.eos_token_id", (uint32_t)(eos >= 0 && eos < sh.vocab ? eos : sh.vocab - 1));
    w.s("tokenizer.ggml.tokens"); w.v<uint32_t>(9); w.v<uint32_t>(8); w.v<uint64_t>((uint64_t)sh.vocab);
    // byte-level BPE alphabet: printable non-space Latin-1 bytes spell themselves, the other 68 bytes take code points 256..
    auto spell = [](int byte) {
        int cp = byte, next = 256;
        for (int b = 0; b <= byte; b++) {
            const bool self = (b >= 0x21 && b <= 0x7E) || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
            if (!self) { if (b == byte) cp = next; next++; }
        }
        std::string u;
        if (cp < 0x80) u.push_back((char)cp);
        else { u.push_back((char)(0xC0 | (cp >> 6))); u.push_back((char)(0x80 | (cp & 0x3F))); }
        return u;
    };
    for (int i = 0; i < sh.vocab; i++) w.s(i < 256 ? spell(i) : spell(' ') + "t" + std::to_string(i));
    for (auto& t : ts) {
        w.s(t.name);
        if (t.rows == 1) { w.v<uint32_t>(1); w.v<uint64_t>((uint64_t)t.cols); }
        else { w.v<uint32_t>(2); w.v<uint64_t>((uint64_t)t.cols); w.v<uint64_t>((uint64_t)t.rows); }
        w.v<uint32_t>(t.type); w.v<uint64_t>(t.offset);
    }
    w.pad(32);
    const uint64_t data_start = w.pos;
    unsigned nth = std::thread::hardware_concurrency(); if (nth == 0) nth = 1; if (nth > 64) nth = 64;
    std::vector<uint8_t> buf, first;
    for (size_t i = 0; i < ts.size(); i++) {
        const TensorSpec& t = ts[i];
        if (w.pos - data_start != t.offset) { fprintf(stderr, "gguf_synth: internal offset mismatch\n"); return 1; }
        if (t.alias == 0) w.raw(first.data(), first.size());
        else {
            gen_tensor(t, buf, nth);
            w.raw(buf.data(), buf.size());
            if (i == 0) first = buf;
        }
        w.pad(32);
    }
    if (fclose(f) != 0) { perror("gguf_synth: close"); return 1; }
    fprintf(stderr, "gguf_synth: wrote %s: L=%d d=%d ff=%d H=%d/%d hd=%d vocab=%d seed=%llu std=%g (%llu bytes)\n",
            argv[1], sh.layers, sh.embd, sh.ff, sh.heads, sh.kv_heads, hd, sh.vocab,
            (unsigned long long)seed, wstd, (unsigned long long)w.pos);
    return 0;
}
