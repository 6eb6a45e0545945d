// The short-context build of the decode kernel: what a launch runs whose steps all end within kShortAttnMax cached
// positions on a model with dedicated attention CTAs.  It contains no attention code besides those CTAs', so the loop of
// the GEMV CTAs compiles without the stack frame and the spills the other attention variants bring into the function.
#define MI_LEAN 1
#include "decode_kernel.cuh"

namespace mi {

const void* decode_kernel_lean(int HD, int G) {
    #define MI_PICK(hd, g) if (HD == hd && G == g) return (const void*)decode_kernel<hd, g>;
    MI_PICK(128, 6) MI_PICK(128, 8) MI_PICK(64, 2)      // head shapes of models whose embedding width this build takes (1024 < E <= 2048)
    #undef MI_PICK
    return nullptr;
}

}  // namespace mi
