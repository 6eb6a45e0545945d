// mega: the persistent engine.  Same command line as the reference's mega
// (src/mega.cu:25): prompt and generation run inside cooperative launches of one
// persistent kernel, phases separated by a bounded-wait grid barrier.
#include "driver_common.hpp"
int main(int argc, char** argv) { return mib200::driver_main(argc, argv, "mega", MI_DECODE_PERSISTENT); }
