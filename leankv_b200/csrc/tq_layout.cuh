// Bit layout of one pool chunk: the 16 tokens of a page for one KV head, K or V.
//
// A chunk is 192 32-bit words of codes followed by 16 fp16 norms (800 bytes). The words
// form 64 "units" of 3 words; word kk of unit ui sits at word index kk*64 + ui, so that
// the 32 lanes of a warp read consecutive words (no shared-memory bank conflicts) and a
// chunk can be brought into shared memory by one bulk copy without any re-ordering.
//
// A unit packs 32 codes e = 0..31 of 3 bits each:
//   e < 24 : word e/8, bits [4*(e%8), 4*(e%8)+2]           (one code per nibble)
//   e >= 24: bit b of the code sits in word b at bit 4*(e-24)+3  (the nibbles' spare bit)
// Masking a word with 0x77777777 therefore yields eight byte-permute selectors directly.
//
// Which 32 codes a unit holds follows the operand fragments of mma.m16n8k16:
//   K chunk: unit (slot s, quarter t) = coordinates 32t .. 32t+31 of token s; ui = 4s + t.
//            Lane (g,t) of the score MMA needs exactly the units of tokens g and g+8.
//   V chunk: unit (pair p, group g) = coordinates 16g .. 16g+15 of tokens 2p and 2p+1,
//            interleaved e = 2*(c%16) + (token&1); ui = 4g + p for p < 4, 32 + 4g + (p-4)
//            otherwise. Lane (g,t) of the value MMA needs units (t,g) and (t+4,g).
#pragma once

#include <stdint.h>

namespace leankv {

constexpr int kChunkWords = 192;
constexpr int kChunkBytes = LEANKV_TQ_CHUNK_BYTES;   // 768 + 16 * 2
constexpr int kNormOffsetBytes = 768;

struct CodeSlot {
    int ui;   // unit index 0..63
    int e;    // code index inside the unit 0..31
};

__host__ __device__ inline CodeSlot k_code_slot(int slot, int coord) {
    CodeSlot r;
    r.ui = slot * 4 + (coord >> 5);
    r.e = coord & 31;
    return r;
}

__host__ __device__ inline CodeSlot v_code_slot(int slot, int coord) {
    CodeSlot r;
    const int p = slot >> 1, g = coord >> 4;
    r.ui = p < 4 ? 4 * g + p : 32 + 4 * g + (p - 4);
    r.e = 2 * (coord & 15) + (slot & 1);
    return r;
}

// Extract one code from a chunk's words (generic pointer: global or shared).
__host__ __device__ inline int chunk_get_code(const uint32_t* words, CodeSlot cs) {
    if (cs.e < 24) return (words[(cs.e >> 3) * 64 + cs.ui] >> (4 * (cs.e & 7))) & 7;
    const int sh = 4 * (cs.e - 24) + 3;
    return ((words[cs.ui] >> sh) & 1) | (((words[64 + cs.ui] >> sh) & 1) << 1) |
           (((words[128 + cs.ui] >> sh) & 1) << 2);
}

// Contribution of code `c` at position e to word kk of its unit.
__host__ __device__ inline uint32_t unit_word_bits(int e, int kk, int c) {
    if (e < 24) return (e >> 3) == kk ? ((uint32_t)c << (4 * (e & 7))) : 0u;
    return (uint32_t)((c >> kk) & 1) << (4 * (e - 24) + 3);
}

}  // namespace leankv
