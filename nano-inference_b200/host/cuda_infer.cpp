// cuda_infer: the kernel-sequence engine.  Same command line as the reference's
// cuda_infer (src/cuda_infer.cu:6): every decode phase is its own launch in stream
// order, the analogue of the reference's per-token CUDA graph of kernels.
#include "driver_common.hpp"
int main(int argc, char** argv) { return mib200::driver_main(argc, argv, "cuda", MI_DECODE_PER_PHASE); }
