// The prepared ("packed") weight layout read by the streaming GEMV and the tcgen05 GEMM.
//
// A matrix [rows, cols] is cut into super-tiles of 64 rows x 128 columns (one scale
// group wide).  Super-tiles are stored row-block major: super-tile (rb, g) of a matrix
// with G = cols/128 groups lives at byte offset (rb*G + g) * kStBytes.  Rows are padded
// up to a multiple of 64 with zero weights and zero scales.
//
//   bytes    0..2047 : codes, 512 words of 32 bits.  A weight t in {-1,0,+1} is stored
//                      as the 2-bit OFFSET CODE c = t + 1 (0, 1, 2; 3 never occurs).
//                      Word (m, lane, i) at index (m*32 + lane)*4 + i, with
//                          m    = 0..3   the k32 step of mma.m16n8k32 inside the group
//                          lane = 0..31  the MMA lane, lane = gq*4 + t
//                          i    = 0..3   i = 2h + j2: row half h, column half j2
//                      holds sixteen codes: byte j (0..3), field f (0..3) at bits
//                      8j + 2f .. 8j + 2f + 1 is the weight at
//                          row    16f + gq + 8h
//                          column 32m + 16*j2 + 4t + j              (inside the group)
//                      So `word & (0x03030303 << 2f)` IS an A-operand register of the MMA
//                      whose 16 A rows are rows 16f .. 16f+15 of the super-tile (words
//                      i = 0,1,2,3 are registers a0,a2,a1,a3), as unsigned bytes scaled by
//                      4^f: one logic instruction per operand register, no shift, no
//                      table.  The 4^f factor is divided out in FP32 together with the
//                      scale, and sum(t*x) = sum(c*x) - sum(x).  The two words of one row
//                      (i = 2h, 2h+1) are adjacent: a thread that expands ONE row, as the
//                      GEMM's does, reads them with one 64-bit load per (m, t).
//   bytes 2048..2175 : scales, FP16.  half[gq*8 + f*2 + h] is the scale of row
//                      16f + gq + 8h: the eight scales an MMA lane needs are 16
//                      contiguous bytes.
//
// The layout keeps 2 bits per weight and all FP16 scales: it is exactly as large as
// the three reference arrays for matrices whose row count is a multiple of 64, and it
// is lossless for canonical masks (sign bit set only where the nonzero bit is set),
// which is all the reference's packer emits (ternarize/pack.py:135-138).
#pragma once
#include <cstdint>

namespace tllm {

constexpr int kStRows = 64;
constexpr int kStCodeBytes = 2048;
constexpr int kStScaleBytes = 128;
constexpr int kStBytes = kStCodeBytes + kStScaleBytes;   // 2176

// Weight (r64, c) of a super-tile, r64 = 0..63, c = 0..127: index of its code word and
// the bit position of its 2-bit code inside that word.
__host__ __device__ inline void st_locate(int r64, int c, int& word, int& shift)
{
    const int f = r64 >> 4, gq = r64 & 7, h = (r64 >> 3) & 1;
    const int m = c >> 5, j2 = (c >> 4) & 1, t = (c >> 2) & 3, j = c & 3;
    word = (m * 32 + gq * 4 + t) * 4 + 2 * h + j2;
    shift = 8 * j + 2 * f;
}

// Index of row r64's scale among the 64 FP16 scales of a super-tile.
__host__ __device__ inline int st_scale_index(int r64)
{
    return (r64 & 7) * 8 + (r64 >> 4) * 2 + ((r64 >> 3) & 1);
}

}  // namespace tllm
