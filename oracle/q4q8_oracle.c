/*
 * CPU oracle for the quantized decode path of minfer (123-code/nano-inference).
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing on the product path may call, link or load
 * this file: it exists so that the CUDA kernels can be checked against a plain
 * scalar restatement of the reference arithmetic.  Only the test-suite, the
 * smoke check and the benchmark's CPU-baseline leg use it.
 *
 * Every function names the reference lines it restates (paths are relative to
 * the reference project root).  The fp32-activation mode restates the
 * reference's own CPU oracle src/cpu_infer.cpp and is pinned against that
 * program compiled unmodified (see oracle/Makefile, target _ref); the
 * q8_0-activation mode restates the integer arithmetic of the reference's GPU
 * kernels (src/cuda_infer.cu quant_x_q8 / gemv_dp4a, src/mega.cu blk_acc),
 * which has no CPU implementation in the reference.
 *
 * Arithmetic of the q8_0 mode.  A q8_0 quantizer is discontinuous: an ulp-sized
 * difference in its input (a different fp32 summation order, another libm's expf)
 * can flip one int8, and two engines that differ that way drift apart to about
 * 2e-3 on the logits.  The reference's own GPU engines each sum in their own
 * order, so the reference defines the formulas but no canonical rounding.  The
 * q8_0 mode therefore evaluates every reference formula in double precision
 * (block products dw*dx*isum are exact in double; exp / cos / sin through the
 * double libm) and rounds to fp32 once, where the reference stores an fp32
 * tensor.  A result obtained this way does not depend on the order of the sum,
 * so any engine that accumulates in double can match it bit for bit.
 *
 * Plain C99 + OpenMP (optional).  No dependencies.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- fp16 <-> fp32 */

/* Exact half -> float, subnormals included (src/gguf.h:37-52). */
ORC_API float orc_fp16_to_fp32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, f;
    if (e == 0) {
        if (m == 0) f = sign;
        else {
            int shift = 0;
            while (!(m & 0x400u)) { m <<= 1; shift++; }
            m &= 0x3FFu;
            f = sign | ((uint32_t)(127 - 15 + 1 - shift) << 23) | (m << 13);
        }
    } else if (e == 0x1F) f = sign | 0x7F800000u | (m << 13);
    else f = sign | ((e - 15 + 127) << 23) | (m << 13);
    float out; memcpy(&out, &f, 4); return out;
}

/* float -> half, round-to-nearest-even: what __float2half does on the GPU
 * (src/cuda_infer.cu:88 stores the activation scale through it). */
ORC_API uint16_t orc_fp32_to_fp16(float x) {
    uint32_t f; memcpy(&f, &x, 4);
    uint32_t sign = (f >> 16) & 0x8000u;
    uint32_t e = (f >> 23) & 0xFFu, m = f & 0x7FFFFFu;
    if (e == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? 0x200u : 0));
    int32_t ne = (int32_t)e - 127 + 15;
    if (ne >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (ne <= 0) {
        if (ne < -10) return (uint16_t)sign;
        m |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - ne);
        uint32_t hm = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (hm & 1))) hm++;
        return (uint16_t)(sign | hm);
    }
    uint32_t hm = m >> 13, rem = m & 0x1FFFu;
    uint16_t out = (uint16_t)(sign | ((uint32_t)ne << 10) | hm);
    if (rem > 0x1000u || (rem == 0x1000u && (hm & 1))) out++;
    return out;
}

/* ---------------------------------------------------------------- q4_0 blocks */

/* One row of a q4_0 matrix to fp32 (src/gguf.h:94-102): 18-byte blocks, fp16 d
 * then 16 bytes; element j is the low nibble of byte j, element j+16 the high. */
ORC_API void orc_dequant_row_q4_0(const uint8_t* row, int64_t nb, float* out) {
    for (int64_t b = 0; b < nb; b++, row += 18) {
        uint16_t dh; memcpy(&dh, row, 2);
        float d = orc_fp16_to_fp32(dh);
        const uint8_t* qs = row + 2; float* y = out + b * 32;
        for (int j = 0; j < 16; j++) {
            y[j]      = (float)((qs[j] & 0x0F) - 8) * d;
            y[j + 16] = (float)((qs[j] >> 4) - 8) * d;
        }
    }
}

/* One row of a Q4_1 / Q8_0 / Q6_K matrix to fp32 (src/gguf.h:103-140); ggml type ids 3, 8, 14.
 * Q4_1: 20-byte blocks {fp16 d, fp16 m, 16 bytes}: value = nibble * d + m.
 * Q8_0: 34-byte blocks {fp16 d, 32 int8}: value = q * d.
 * Q6_K: 210-byte super-blocks of 256 {ql[128], qh[64], int8 sc[16], fp16 d}: value = d * sc * (6-bit q - 32),
 *       multiplied left to right in fp32 as the reference writes it. */
ORC_API int orc_dequant_row_t(int type, const uint8_t* p, int64_t cols, float* out) {
    if (type == 3) {
        for (int64_t b = 0; b < cols / 32; b++, p += 20) {
            uint16_t dh, mh; memcpy(&dh, p, 2); memcpy(&mh, p + 2, 2);
            const float d = orc_fp16_to_fp32(dh), m = orc_fp16_to_fp32(mh);
            const uint8_t* qs = p + 4; float* y = out + b * 32;
            for (int j = 0; j < 16; j++) { y[j] = (float)(qs[j] & 0x0F) * d + m; y[j + 16] = (float)(qs[j] >> 4) * d + m; }
        }
        return 0;
    }
    if (type == 8) {
        for (int64_t b = 0; b < cols / 32; b++, p += 34) {
            uint16_t dh; memcpy(&dh, p, 2);
            const float d = orc_fp16_to_fp32(dh);
            const int8_t* qs = (const int8_t*)(p + 2); float* y = out + b * 32;
            for (int j = 0; j < 32; j++) y[j] = (float)qs[j] * d;
        }
        return 0;
    }
    if (type == 14) {
        for (int64_t b = 0; b < cols / 256; b++, p += 210) {
            const uint8_t* ql = p; const uint8_t* qh = p + 128; const int8_t* sc = (const int8_t*)(p + 192);
            uint16_t dh; memcpy(&dh, p + 208, 2);
            const float d = orc_fp16_to_fp32(dh);
            float* y = out + b * 256;
            for (int n = 0; n < 256; n += 128) {
                for (int l = 0; l < 32; l++) {
                    const int is = l / 16;
                    const int8_t q1 = (int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                    const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                    const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                    y[l] = d * sc[is + 0] * q1; y[l + 32] = d * sc[is + 2] * q2; y[l + 64] = d * sc[is + 4] * q3; y[l + 96] = d * sc[is + 6] * q4;
                }
                ql += 64; qh += 32; sc += 8; y += 128;
            }
        }
        return 0;
    }
    return 1;
}

/* The reference's own q4_0 re-quantizer for tensors stored in another type (src/mega.cu:924-936, the same arithmetic
 * as src/cuda_infer.cu:816-835): symmetric, d = amax / 7, q = clamp(lrintf(y / d) + 8, 0, 15), scale stored as fp16. */
ORC_API void orc_requant_row_q4_0(const float* y, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / 32; b++, y += 32, out += 18) {
        float amax = 0.f;
        for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(y[j]));
        const float d = amax / 7.f, inv = (d > 0.f) ? 1.f / d : 0.f;
        const uint16_t dh = orc_fp32_to_fp16(d); memcpy(out, &dh, 2);
        for (int j = 0; j < 16; j++) {
            int q0 = (int)lrintf(y[j] * inv) + 8;      q0 = q0 < 0 ? 0 : (q0 > 15 ? 15 : q0);
            int q1 = (int)lrintf(y[j + 16] * inv) + 8; q1 = q1 < 0 ? 0 : (q1 > 15 ? 15 : q1);
            out[2 + j] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

/* ggml's q4_0 quantizer, as the benchmark configuration states it: d = (signed
 * value of largest magnitude) / -8, q = min(15, trunc(x/d + 8.5)).  The scale is
 * stored as fp16; the division uses the fp32 d.  Not in the reference tree (the
 * reference consumes files quantized by llama.cpp); used to make test inputs. */
ORC_API void orc_quantize_row_q4_0(const float* x, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / 32; b++, out += 18) {
        const float* xb = x + b * 32;
        float amax = 0.f, mx = 0.f;
        for (int j = 0; j < 32; j++) { float a = fabsf(xb[j]); if (a > amax) { amax = a; mx = xb[j]; } }
        float d = mx / -8.f, id = d != 0.f ? 1.f / d : 0.f;
        uint16_t dh = orc_fp32_to_fp16(d); memcpy(out, &dh, 2);
        for (int j = 0; j < 16; j++) {
            int q0 = (int)(int8_t)(xb[j] * id + 8.5f), q1 = (int)(int8_t)(xb[j + 16] * id + 8.5f);
            if (q0 > 15) q0 = 15; if (q1 > 15) q1 = 15;
            out[2 + j] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

/* ---------------------------------------------------------------- q8_0 activations */

/* Per 32-element block: a = max|x|, inv = a > 0 ? 127/a : 0, xq = rint(x*inv)
 * (round half to even), xd = fp16(a/127)  (src/cuda_infer.cu:80-89). */
ORC_API void orc_quant_q8(const float* x, int64_t n, int8_t* xq, uint16_t* xd) {
    for (int64_t g = 0; g < n / 32; g++) {
        float a = 0.f;
        for (int i = 0; i < 32; i++) a = fmaxf(a, fabsf(x[g * 32 + i]));
        float inv = a > 0.f ? 127.f / a : 0.f;
        for (int i = 0; i < 32; i++) xq[g * 32 + i] = (int8_t)(int)nearbyintf(x[g * 32 + i] * inv);
        xd[g] = orc_fp32_to_fp16(a / 127.f);
    }
}

/* Integer part of one q4_0 block against 32 int8 activations:
 * sum_k n_k*xq_k - 8*sum_k xq_k with n the raw nibbles 0..15
 * (src/cuda_infer.cu:110-122, src/mega.cu:157-165). Exact. */
static inline int32_t block_isum(const uint8_t* blk18, const int8_t* xq) {
    const uint8_t* qs = blk18 + 2;
    int32_t acc = 0, sx = 0;
    for (int j = 0; j < 16; j++) {
        acc += (int32_t)(qs[j] & 0x0F) * xq[j] + (int32_t)(qs[j] >> 4) * xq[j + 16];
        sx += xq[j] + xq[j + 16];
    }
    return acc - 8 * sx;
}

/* All block sums of a matrix: isum[row*nb + b]. */
ORC_API void orc_block_isums(const uint8_t* W, int64_t rows, int64_t cols, const int8_t* xq, int32_t* isum) {
    const int64_t nb = cols / 32;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++)
        for (int64_t b = 0; b < nb; b++)
            isum[r * nb + b] = block_isum(W + (r * nb + b) * 18, xq + b * 32);
}

/* y[r] = fp32( sum_b (dw*dx) * isum ) + bias[r]: the sum of src/cuda_infer.cu:94-127
 * (src/mega.cu:151-155) with the accumulation carried in double.  dw*dx is exact in
 * fp32 (two fp16 values), its product with the integer is exact in double. */
ORC_API void orc_gemv_q4_q8(const uint8_t* W, int64_t rows, int64_t cols, const int8_t* xq,
                            const uint16_t* xd, const float* bias, float* y) {
    const int64_t nb = cols / 32;
    float* dx = (float*)malloc(sizeof(float) * (size_t)nb);
    for (int64_t b = 0; b < nb; b++) dx[b] = orc_fp16_to_fp32(xd[b]);
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        double acc = 0.0;
        for (int64_t b = 0; b < nb; b++) {
            const uint8_t* blk = W + (r * nb + b) * 18;
            uint16_t dh; memcpy(&dh, blk, 2);
            const float s = orc_fp16_to_fp32(dh) * dx[b];
            acc += (double)s * (double)block_isum(blk, xq + b * 32);
        }
        const float v = (float)acc;
        y[r] = bias ? v + bias[r] : v;
    }
    free(dx);
}

/* fp32-activation product of the reference CPU oracle (src/cpu_infer.cpp:22-32):
 * dequantize the row, then a sequential fp32 dot. */
ORC_API void orc_matvec_f32(const uint8_t* W, int64_t rows, int64_t cols, const float* x, float* y) {
    const int64_t nb = cols / 32;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        float row[16384];
        orc_dequant_row_q4_0(W + r * nb * 18, nb, row);
        float acc = 0.f;
        for (int64_t k = 0; k < cols; k++) acc += row[k] * x[k];
        y[r] = acc;
    }
}

/* ---------------------------------------------------------------- glue ops */

/* src/cpu_infer.cpp:40-46 (double sum of squares, float scale). */
ORC_API void orc_rmsnorm(const float* x, const float* w, int n, float eps, float* out) {
    double ss = 0; for (int i = 0; i < n; i++) ss += (double)x[i] * x[i];
    float scale = 1.f / sqrtf((float)(ss / n) + eps);
    for (int i = 0; i < n; i++) out[i] = x[i] * scale * w[i];
}

/* NEOX RoPE, pairs (i, i+hd/2) (src/cpu_infer.cpp:49-61). */
ORC_API void orc_rope(float* v, int n_head, int hd, int pos, float base) {
    int half = hd / 2;
    for (int h = 0; h < n_head; h++) {
        float* p = v + (size_t)h * hd;
        for (int i = 0; i < half; i++) {
            float theta = pos * powf(base, -2.f * i / hd);
            float c = cosf(theta), s = sinf(theta);
            float x0 = p[i], x1 = p[i + half];
            p[i] = x0 * c - x1 * s;
            p[i + half] = x0 * s + x1 * c;
        }
    }
}

/* q8_0 mode: the same rotation with cos/sin from the double libm and exact double
 * products, rounded to fp32 once per output. */
ORC_API void orc_rope_d(float* v, int n_head, int hd, int pos, float base) {
    int half = hd / 2;
    for (int h = 0; h < n_head; h++) {
        float* p = v + (size_t)h * hd;
        for (int i = 0; i < half; i++) {
            const float theta = pos * powf(base, -2.f * i / hd);
            const float c = (float)cos((double)theta), s = (float)sin((double)theta);
            const double x0 = p[i], x1 = p[i + half];
            p[i] = (float)(x0 * c - x1 * s);
            p[i + half] = (float)(x0 * s + x1 * c);
        }
    }
}

/* q8_0 mode: softmax attention (src/cpu_infer.cpp:121-140) carried in double:
 * score = fp32(q.k) * inv in fp32, weights exp(score - max) and both sums in double,
 * output fp32(sum / denominator). */
ORC_API void orc_attention_d(const float* q, const float* kc, const float* vc, int pos,
                             int n_head, int n_head_kv, int hd, float* att) {
    const int kv_dim = n_head_kv * hd, gqa = n_head / n_head_kv;
    const float inv = 1.f / sqrtf((float)hd);
    float* sc = (float*)malloc(sizeof(float) * (size_t)(pos + 1));
    double* o = (double*)malloc(sizeof(double) * (size_t)hd);
    for (int hh = 0; hh < n_head; hh++) {
        const int kvh = hh / gqa; const float* qh = q + (size_t)hh * hd;
        float mx = -INFINITY;
        for (int t = 0; t <= pos; t++) {
            const float* kt = kc + (size_t)t * kv_dim + (size_t)kvh * hd;
            double d = 0; for (int i = 0; i < hd; i++) d += (double)qh[i] * (double)kt[i];
            sc[t] = (float)d * inv; if (sc[t] > mx) mx = sc[t];
        }
        double sum = 0;
        for (int i = 0; i < hd; i++) o[i] = 0;
        for (int t = 0; t <= pos; t++) {
            const float* vt = vc + (size_t)t * kv_dim + (size_t)kvh * hd;
            const double e = exp((double)sc[t] - (double)mx);
            sum += e;
            for (int i = 0; i < hd; i++) o[i] = fma(e, (double)vt[i], o[i]);
        }
        for (int i = 0; i < hd; i++) att[(size_t)hh * hd + i] = (float)(o[i] / sum);
    }
    free(sc); free(o);
}

/* Causal GQA attention of one query over positions 0..pos of a cache laid out
 * [pos][kv_dim] (src/cpu_infer.cpp:121-140).  The cache is fp32; when the caller
 * wants fp16-cache semantics it stores values already rounded through fp16. */
ORC_API void orc_attention(const float* q, const float* kc, const float* vc, int pos,
                           int n_head, int n_head_kv, int hd, float* att) {
    const int kv_dim = n_head_kv * hd, gqa = n_head / n_head_kv;
    const float inv = 1.f / sqrtf((float)hd);
    float* sc = (float*)malloc(sizeof(float) * (size_t)(pos + 1));
    for (int hh = 0; hh < n_head; hh++) {
        const int kvh = hh / gqa; const float* qh = q + (size_t)hh * hd;
        float mx = -1e30f;
        for (int t = 0; t <= pos; t++) {
            const float* kt = kc + (size_t)t * kv_dim + (size_t)kvh * hd;
            float d = 0; for (int i = 0; i < hd; i++) d += qh[i] * kt[i];
            sc[t] = d * inv; if (sc[t] > mx) mx = sc[t];
        }
        float sum = 0; for (int t = 0; t <= pos; t++) { sc[t] = expf(sc[t] - mx); sum += sc[t]; }
        float* oh = att + (size_t)hh * hd;
        for (int i = 0; i < hd; i++) oh[i] = 0;
        for (int t = 0; t <= pos; t++) {
            const float* vt = vc + (size_t)t * kv_dim + (size_t)kvh * hd;
            float p = sc[t] / sum;
            for (int i = 0; i < hd; i++) oh[i] += p * vt[i];
        }
    }
    free(sc);
}

/* ---------------------------------------------------------------- whole forward */

typedef struct {
    int32_t n_layer, n_embd, n_ff, n_head, n_head_kv, head_dim, n_vocab;
    float rope_base, rms_eps;
    const uint8_t* tok_emb;      /* q4_0 [n_vocab][n_embd] */
    const uint8_t* out_w;        /* q4_0 [n_vocab][n_embd] */
    const float*   out_norm;
    /* per layer arrays of pointers */
    const float* const*   attn_norm; const float* const* ffn_norm;
    const uint8_t* const* wq; const uint8_t* const* wk; const uint8_t* const* wv; const uint8_t* const* wo;
    const float* const*   bq; const float* const* bk; const float* const* bv;
    const uint8_t* const* wg; const uint8_t* const* wu; const uint8_t* const* wd;
    int32_t tok_emb_type;        /* 0 or 2: q4_0 rows; 8: Q8_0 rows (34-byte blocks), which the reference's persistent
                                    engine reads without re-quantizing (src/mega.cu:639-646, 1110-1111) */
} orc_model;

typedef struct {
    int32_t max_seq, act_q8, kv_f16;
    float *kc, *vc;                       /* [layer][max_seq][kv_dim] */
    float *h, *xb, *q, *k, *v, *att, *proj, *gbuf, *ubuf;
    int8_t* xq; uint16_t* xd;
} orc_state;

ORC_API orc_state* orc_state_new(const orc_model* m, int max_seq, int act_q8, int kv_f16) {
    orc_state* s = (orc_state*)calloc(1, sizeof(orc_state));
    const size_t kv_dim = (size_t)m->n_head_kv * m->head_dim;
    s->max_seq = max_seq; s->act_q8 = act_q8; s->kv_f16 = kv_f16;
    s->kc = (float*)calloc((size_t)m->n_layer * max_seq * kv_dim, 4);
    s->vc = (float*)calloc((size_t)m->n_layer * max_seq * kv_dim, 4);
    s->h = (float*)calloc(m->n_embd, 4); s->xb = (float*)calloc(m->n_embd, 4);
    s->q = (float*)calloc((size_t)m->n_head * m->head_dim, 4);
    s->k = (float*)calloc(kv_dim, 4); s->v = (float*)calloc(kv_dim, 4);
    s->att = (float*)calloc((size_t)m->n_head * m->head_dim, 4);
    s->proj = (float*)calloc(m->n_embd, 4);
    s->gbuf = (float*)calloc(m->n_ff, 4); s->ubuf = (float*)calloc(m->n_ff, 4);
    size_t mx = (size_t)(m->n_ff > m->n_embd ? m->n_ff : m->n_embd);
    s->xq = (int8_t*)calloc(mx, 1); s->xd = (uint16_t*)calloc(mx / 32 + 1, 2);
    return s;
}

ORC_API void orc_state_free(orc_state* s) {
    if (!s) return;
    free(s->kc); free(s->vc); free(s->h); free(s->xb); free(s->q); free(s->k); free(s->v);
    free(s->att); free(s->proj); free(s->gbuf); free(s->ubuf); free(s->xq); free(s->xd); free(s);
}

/* y = W x through whichever activation mode the state selects.  In q8 mode the
 * input is quantized where the reference GPU step quantizes it
 * (src/cuda_infer.cu:1037,1062,1065,1069,1078): once per distinct input. */
static void mv(const orc_state* s, const uint8_t* W, int rows, int cols, const float* x,
               const float* bias, float* y, int requant) {
    if (s->act_q8) {
        if (requant) orc_quant_q8(x, cols, s->xq, s->xd);
        orc_gemv_q4_q8(W, rows, cols, s->xq, s->xd, bias, y);
    } else {
        orc_matvec_f32(W, rows, cols, x, y);
        if (bias) for (int i = 0; i < rows; i++) y[i] += bias[i];
    }
}

static void round_f16(float* v, int n) {
    for (int i = 0; i < n; i++) v[i] = orc_fp16_to_fp32(orc_fp32_to_fp16(v[i]));
}

/* One token at position pos (src/cpu_infer.cpp:109-156).  logits may be NULL.
 * hidden_out, when given, receives the residual stream after every layer
 * ([n_layer][n_embd]) for per-layer checks.  Returns the greedy token: strict '>'
 * in ascending order, so the lowest index wins ties (src/cpu_infer.cpp:153-154). */
ORC_API int orc_forward(const orc_model* m, orc_state* s, int token, int pos, float* logits, float* hidden_out) {
    const int E = m->n_embd, HD = m->head_dim, NH = m->n_head, NKV = m->n_head_kv;
    const int kv_dim = NKV * HD, FF = m->n_ff, V = m->n_vocab;
    const int64_t nbE = E / 32;
    if (m->tok_emb_type == 8) orc_dequant_row_t(8, m->tok_emb + (int64_t)token * nbE * 34, E, s->h);
    else orc_dequant_row_q4_0(m->tok_emb + (int64_t)token * nbE * 18, nbE, s->h);
    for (int l = 0; l < m->n_layer; l++) {
        orc_rmsnorm(s->h, m->attn_norm[l], E, m->rms_eps, s->xb);
        mv(s, m->wq[l], NH * HD, E, s->xb, m->bq[l], s->q, 1);
        mv(s, m->wk[l], kv_dim, E, s->xb, m->bk[l], s->k, 0);
        mv(s, m->wv[l], kv_dim, E, s->xb, m->bv[l], s->v, 0);
        if (s->act_q8) { orc_rope_d(s->q, NH, HD, pos, m->rope_base); orc_rope_d(s->k, NKV, HD, pos, m->rope_base); }
        else { orc_rope(s->q, NH, HD, pos, m->rope_base); orc_rope(s->k, NKV, HD, pos, m->rope_base); }
        if (s->kv_f16) { round_f16(s->k, kv_dim); round_f16(s->v, kv_dim); }
        float* kc = s->kc + (size_t)l * s->max_seq * kv_dim;
        float* vc = s->vc + (size_t)l * s->max_seq * kv_dim;
        memcpy(kc + (size_t)pos * kv_dim, s->k, sizeof(float) * kv_dim);
        memcpy(vc + (size_t)pos * kv_dim, s->v, sizeof(float) * kv_dim);
        if (s->act_q8) orc_attention_d(s->q, kc, vc, pos, NH, NKV, HD, s->att);
        else orc_attention(s->q, kc, vc, pos, NH, NKV, HD, s->att);
        mv(s, m->wo[l], E, NH * HD, s->att, NULL, s->proj, 1);
        for (int i = 0; i < E; i++) s->h[i] += s->proj[i];
        orc_rmsnorm(s->h, m->ffn_norm[l], E, m->rms_eps, s->xb);
        mv(s, m->wg[l], FF, E, s->xb, NULL, s->gbuf, 1);
        mv(s, m->wu[l], FF, E, s->xb, NULL, s->ubuf, 0);
        if (s->act_q8)
            for (int i = 0; i < FF; i++) { const double x = s->gbuf[i]; s->gbuf[i] = (float)((x / (1.0 + exp(-x))) * (double)s->ubuf[i]); }
        else
            for (int i = 0; i < FF; i++) { float x = s->gbuf[i]; s->gbuf[i] = (x / (1.f + expf(-x))) * s->ubuf[i]; }
        mv(s, m->wd[l], E, FF, s->gbuf, NULL, s->proj, 1);
        for (int i = 0; i < E; i++) s->h[i] += s->proj[i];
        if (hidden_out) memcpy(hidden_out + (size_t)l * E, s->h, sizeof(float) * E);
    }
    orc_rmsnorm(s->h, m->out_norm, E, m->rms_eps, s->xb);
    float* lg = logits ? logits : (float*)malloc(sizeof(float) * (size_t)V);
    mv(s, m->out_w, V, E, s->xb, NULL, lg, 1);
    int best = 0; float bv = lg[0];
    for (int i = 1; i < V; i++) if (lg[i] > bv) { bv = lg[i]; best = i; }
    if (!logits) free(lg);
    return best;
}

/* The fp32 KV cache of a state ([layer][max_seq][kv_dim]), for cache-content checks. */
ORC_API float* orc_state_kc(orc_state* s) { return s->kc; }
ORC_API float* orc_state_vc(orc_state* s) { return s->vc; }

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
