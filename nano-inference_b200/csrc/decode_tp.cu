// The tensor-parallel build of the decode kernel: the persistent loop with the exchange with the other GPUs inside it
// (every producing CTA stores its tagged words into the other GPUs' exchange blocks over NVLink as well as its own).
// decode.cu launches these instantiations for a sharded model whose peer buffers are mapped; the single-GPU build
// carries none of this code.
#define MI_TP 1
#include "decode_kernel.cuh"

namespace mi {

const void* decode_kernel_tp(int HD, int G) {
    #define MI_PICK(hd, g) if (HD == hd && G == g) return (const void*)decode_kernel<hd, g>;
    MI_PICK(32, 2) MI_PICK(64, 2) MI_PICK(64, 7) MI_PICK(128, 6) MI_PICK(128, 8)
    #undef MI_PICK
    return nullptr;
}

}  // namespace mi
