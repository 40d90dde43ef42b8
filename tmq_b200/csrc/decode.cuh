// Decoding one 32-bit word of the prepacked weight layouts (tmq_prepack) into tensor-core operands.
#pragma once
#include <stdint.h>

namespace tmq {

// bf16 format: bits [31-2j:30-2j] = (sign, nonzero) of k = 2j+1, bits [15-2j:14-2j] of k = 2j, j = 0..7.
// (w << 2j) & 0xC000C000 is then the bf16 pair {k=2j (low half), k=2j+1 (high half)} with values 0 / +2 / -2.
__device__ __forceinline__ void decode_word_bf16(uint32_t w, uint32_t (&r)[8]) {
#pragma unroll
    for (int j = 0; j < 8; j++) r[j] = (w << (2 * j)) & 0xC000C000u;
}

// int8 format: nibble-spaced reference codes (0 -> 0, 1 -> +1, 2 -> -1); a byte permute with the 4-entry table
// {0x00, 0x01, 0xFF, 0x00} turns four codes into four int8 values at once.
__device__ __forceinline__ void decode_word_i8(uint32_t w, uint32_t (&r)[4]) {
    const uint32_t table = 0x00FF0100u;
    const uint32_t lo = w & 0x33333333u, hi = (w >> 2) & 0x33333333u;
    r[0] = __byte_perm(table, 0u, lo);
    r[1] = __byte_perm(table, 0u, hi);
    r[2] = __byte_perm(table, 0u, lo >> 16);
    r[3] = __byte_perm(table, 0u, hi >> 16);
}

}  // namespace tmq
