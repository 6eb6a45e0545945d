// The instrumented build of the decode kernel (in-kernel profiler: nanoseconds per phase part on CTA 0, read back
// through MI_STATE_PROFILE).  decode.cu launches these instantiations when the model was loaded with MINFER_PROFILE set;
// otherwise it launches the build without any profiling code.
#define MI_PROF 1
#include "decode_kernel.cuh"

namespace mi {

const void* decode_kernel_prof(int HD, int G) {
    #define MI_PICK(hd, g) if (HD == hd && G == g) return (const void*)decode_kernel<hd, g>;
    MI_PICK(32, 2) MI_PICK(64, 2) MI_PICK(64, 7) MI_PICK(128, 6) MI_PICK(128, 8)
    #undef MI_PICK
    return nullptr;
}

}  // namespace mi
