// Checker-side wrapper around one host function of the reference's persistent-kernel driver.
//
// TEST INFRASTRUCTURE ONLY.  The reference's q4_0 re-quantizer for tensors stored in another type, quant_row_q4_0
// (src/mega.cu:924-936), is a static host function of a CUDA source file.  This translation unit textually includes
// src/mega.cu from where it lies (include path given by oracle/Makefile; no reference source is copied) with its main()
// renamed and exports that one function through a C ABI.  It is compiled with nvcc because the file it includes is a
// .cu; nothing in it runs on a GPU, and the library loads on a machine without one.
#define main minfer_mega_main
#include "mega.cu"
#undef main

extern "C" __attribute__((visibility("default")))
void ref_quant_row_q4_0(const float* y, int n, uint8_t* out) { quant_row_q4_0(y, n, out); }
