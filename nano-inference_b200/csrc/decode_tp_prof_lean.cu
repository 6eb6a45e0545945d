// The instrumented form of the tensor-parallel short-context build (see decode_tp_lean.cu and decode_prof.cu): where a
// sharded decode step spends its time, read on the GPUs themselves - a profiler that replays kernels cannot be used on
// kernels that wait for one another's data.
#define MI_TP 1
#define MI_PROF 1
#define MI_LEAN 1
#include "decode_kernel.cuh"

namespace mi {

const void* decode_kernel_tp_prof_lean(int HD, int G) {
    #define MI_PICK(hd, g) if (HD == hd && G == g) return (const void*)decode_kernel<hd, g>;
    MI_PICK(128, 6) MI_PICK(128, 8) MI_PICK(64, 2)      // head shapes of models whose embedding width this build takes (1024 < E <= 2048)
    #undef MI_PICK
    return nullptr;
}

}  // namespace mi
