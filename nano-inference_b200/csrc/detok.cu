// Detokenizer of byte-level BPE vocabularies (GPT-2 style, as Qwen2 model files carry): host code, no GPU involved.
//
// Such a vocabulary spells every byte of the text as one printable code point: the 188 bytes that are printable and not a
// space in Latin-1 ('!'..'~', 0xA1..0xAC, 0xAE..0xFF) stand for themselves, the other 68 bytes, in ascending order, take
// the code points 256, 257, ... 323.  A piece is the UTF-8 spelling of those code points; decoding it means reading the
// code points back and emitting their bytes.  Replaces build_byte_decoder / detok_piece of the reference
// (src/detok.h:13-41), including its treatment of malformed input: a byte that cannot start a UTF-8 sequence is skipped,
// a sequence cut short by the end of the piece is decoded from the bytes that are there, and a code point outside the
// table emits nothing.
#include "minfer_b200.h"

#include <cstdint>

namespace {

struct ByteTable {
    int16_t byte_of[324];
    ByteTable() {
        for (int i = 0; i < 324; i++) byte_of[i] = -1;
        int next = 256;
        for (int b = 0; b < 256; b++) {
            const bool self = (b >= 0x21 && b <= 0x7E) || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
            if (self) byte_of[b] = (int16_t)b; else byte_of[next++] = (int16_t)b;
        }
    }
};

}  // namespace

extern "C" int64_t mi_detok_piece(const char* piece, int64_t n, char* out, int64_t cap) {
    static const ByteTable table;
    if (!piece || n < 0 || (cap > 0 && !out)) return -1;
    const unsigned char* p = reinterpret_cast<const unsigned char*>(piece);
    int64_t w = 0;
    for (int64_t i = 0; i < n;) {
        const unsigned c = p[i];
        int len; unsigned cp;
        if (c < 0x80) { len = 1; cp = c; }
        else if ((c & 0xE0) == 0xC0) { len = 2; cp = c & 0x1F; }
        else if ((c & 0xF0) == 0xE0) { len = 3; cp = c & 0x0F; }
        else if ((c & 0xF8) == 0xF0) { len = 4; cp = c & 0x07; }
        else { i++; continue; }                               // a stray continuation byte (or 0xF8..0xFF)
        for (int k = 1; k < len && i + k < n; k++) cp = (cp << 6) | (p[i + k] & 0x3F);
        i += len;
        if (cp < 324 && table.byte_of[cp] >= 0) {
            if (w < cap) out[w] = (char)table.byte_of[cp];
            w++;
        }
    }
    return w;
}
