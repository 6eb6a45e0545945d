// Checker-side wrapper around the reference CPU oracle's own functions.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit textually includes the
// reference's src/cpu_infer.cpp from where it lies (the include path is given
// on the compiler command line by oracle/Makefile; no reference source is
// copied) with its main() renamed, and exports its static matvec / rmsnorm /
// rope / add_bias and GGUF::dequant_row through a C ABI so that the restatement
// in q4q8_oracle.c can be compared with the real thing, op by op.
// The reference uses the same trick in bench/breakdown.cu:10-12.
#define main minfer_cpu_infer_main
#include "cpu_infer.cpp"
#undef main

#include <cstdint>

static Tensor make_tensor(uint32_t type, int64_t cols, int64_t rows, const void* data) {
    Tensor t; t.type = type; t.ne = {cols, rows}; t.data = (const uint8_t*)data; return t;
}

extern "C" {

// src/cpu_infer.cpp:22-32 on a q4_0 matrix given as raw GGUF bytes.
__attribute__((visibility("default")))
void ref_matvec_q4_0(const uint8_t* raw, int64_t rows, int64_t cols, const float* x, float* y) {
    Tensor W = make_tensor(GT_Q4_0, cols, rows, raw);
    matvec(W, x, y);
}

// src/gguf.h:85-102
__attribute__((visibility("default")))
void ref_dequant_row_q4_0(const uint8_t* raw, int64_t rows, int64_t cols, int64_t r, float* out) {
    Tensor W = make_tensor(GT_Q4_0, cols, rows, raw);
    GGUF::dequant_row(W, r, out);
}

// src/gguf.h:85-140, any tensor type the reference reads (ggml type id)
__attribute__((visibility("default")))
void ref_dequant_row(uint32_t type, const uint8_t* raw, int64_t rows, int64_t cols, int64_t r, float* out) {
    Tensor W = make_tensor(type, cols, rows, raw);
    GGUF::dequant_row(W, r, out);
}

// src/cpu_infer.cpp:40-46
__attribute__((visibility("default")))
void ref_rmsnorm(const float* x, const float* w, int n, float eps, float* out) {
    Tensor T = make_tensor(GT_F32, n, 1, w);
    rmsnorm(x, T, n, eps, out);
}

// src/cpu_infer.cpp:49-61
__attribute__((visibility("default")))
void ref_rope(float* v, int n_head, int hd, int pos, float base) { rope(v, n_head, hd, pos, base); }

// src/cpu_infer.cpp:34-38
__attribute__((visibility("default")))
void ref_add_bias(float* y, const float* b, int n) {
    Tensor T = make_tensor(GT_F32, n, 1, b);
    add_bias(y, T, n);
}

// src/gguf.h:37-52
__attribute__((visibility("default")))
float ref_fp16_to_fp32(uint16_t h) { return fp16_to_fp32(h); }

}  // extern "C"
