// The build of the decode kernel for launches whose steps all have more than kPerHeadAttnMax cached positions: a whole GQA group per CTA and chunk.
// Like the short-context build (decode_lean.cu) it holds one attention variant and no call site in the step loop.
#define MI_LEAN 3
#include "decode_kernel.cuh"

namespace mi {

const void* decode_kernel_lean_long(int HD, int G) {
    #define MI_PICK(hd, g) if (HD == hd && G == g) return (const void*)decode_kernel<hd, g>;
    MI_PICK(128, 6) MI_PICK(128, 8) MI_PICK(64, 2)      // head shapes of models whose embedding width this build takes (1024 < E <= 2048)
    #undef MI_PICK
    return nullptr;
}

}  // namespace mi
