// The prepared ("packed") weight layout read by the tensor-core GEMV kernels.
//
// A matrix [rows, cols] is cut into tiles of 16 rows x 128 columns (one scale
// group wide).  Tiles are stored row-block major: tile (rb, g) of a matrix with
// G = cols/128 groups lives at byte offset (rb*G + g) * kTileBytes.  Rows are
// padded up to a multiple of 16 with zero weights and zero scales.
//
//   bytes   0..511 : codes.  16 rows x 4 lanes x 2 words.  Word w (0/1) of lane t
//                    (0..3) of row r sits at (r*4 + t)*8 + w*4.  It holds the 16-bit
//                    selectors of MMA steps 2w (low half) and 2w+1 (high half).
//                    The selector of step m has four nibbles n = 0..3; nibble n
//                    encodes the PAIR of weights at group columns
//                        ka = 32m + 4t + n      and      kb = 32m + 16 + 4t + n
//                    as the 4-bit pattern pair_code(ta, tb) below.  That is the
//                    register layout of the A operand of mma.m16n8k32 (a0 = the
//                    four `a` weights, a2 = the four `b` weights of a lane), so one
//                    PRMT per operand register expands four weights.
//   bytes 512..543 : scales, FP16.  Rows r and r+8 (r = 0..7) are adjacent:
//                    half[2r] = scale of row r, half[2r+1] = scale of row r+8.
//
// pair_code: the eight pairs other than (0,0) take patterns 0..7 in the order
// (+,+) (+,0) (+,-) (0,+) (0,-) (-,+) (-,0) (-,-); the pair (0,0) is pattern 8.
// A PRMT selector nibble uses bits 0..2 as a byte index into an 8-byte table and
// bit 3 as "replicate the sign bit of the selected byte"; entry 0 of both tables
// is +1 (sign bit clear), so pattern 8 yields 0x00 for both weights.
//
// The layout keeps 2 bits per weight and all FP16 scales: it is exactly as large
// as the three reference arrays for 16-row-aligned matrices, and it is lossless
// for canonical masks (sign bit set only where the nonzero bit is set), which is
// all the reference's packer emits (ternarize/pack.py:135-138).
#pragma once
#include <cstdint>

namespace tllm {

constexpr int kTileRows = 16;
constexpr int kTileCodeBytes = 512;
constexpr int kTileBytes = 544;

// PRMT tables (bytes 0..3 in the low word, 4..7 in the high word), INT8 operands.
// index:            0     1     2     3     4     5     6     7
// weight a:        +1    +1    +1     0     0    -1    -1    -1
// weight b:        +1     0    -1    +1    -1    +1     0    -1
constexpr uint32_t kTabA_lo = 0x00010101u, kTabA_hi = 0xFFFFFF00u;
constexpr uint32_t kTabB_lo = 0x01FF0001u, kTabB_hi = 0xFF0001FFu;

// (ta, tb) in {-1,0,+1}^2 -> 4-bit pattern.
__host__ __device__ inline uint32_t pair_code(int ta, int tb)
{
    if (ta == 0 && tb == 0) return 8u;
    // rows of the table above: a = +1 -> 0..2, a = 0 -> 3..4, a = -1 -> 5..7
    if (ta > 0) return (uint32_t)(1 - tb);            // +1:0, 0:1, -1:2
    if (ta == 0) return tb > 0 ? 3u : 4u;
    return (uint32_t)(6 - tb);                        // +1:5, 0:6, -1:7
}

// 4-bit pattern -> (ta, tb); the inverse of pair_code (patterns 9..15 never occur).
__host__ __device__ inline void pair_decode(uint32_t p, int& ta, int& tb)
{
    const int8_t a[9] = {1, 1, 1, 0, 0, -1, -1, -1, 0};
    const int8_t b[9] = {1, 0, -1, 1, -1, 1, 0, -1, 0};
    const uint32_t i = p > 8u ? 8u : p;
    ta = a[i];
    tb = b[i];
}

}  // namespace tllm
