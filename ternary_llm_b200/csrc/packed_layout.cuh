// The prepared ("packed") weight layout read by the streaming GEMV and the tcgen05 GEMM.
//
// A matrix [rows, cols] is cut into tiles of 16 rows x 128 columns (one scale group
// wide).  Tiles are stored row-block major: tile (rb, g) of a matrix with G = cols/128
// groups lives at byte offset (rb*G + g) * kTileBytes.  Rows are padded up to a multiple
// of 16 with zero weights and zero scales.
//
//   bytes   0..511 : codes, 128 words of 32 bits.  A weight t in {-1,0,+1} is stored as
//                    the 2-bit OFFSET CODE c = t + 1 (0, 1, 2; 3 never occurs).
//                    Word (lane, i) at index lane*4 + i, with
//                        lane = 0..31  the lane of mma.m16n8k32, lane = gq*4 + t
//                        i    = 0..3   i = 2h + j2: row half h, column half j2
//                    holds sixteen codes: byte j (0..3), field f (0..3) at bits
//                    8j + 2f .. 8j + 2f + 1 is the weight at
//                        row    gq + 8h
//                        column 32f + 16*j2 + 4t + j                (inside the group)
//                    So `word & (0x03030303 << 2f)` IS an A-operand register of the MMA
//                    that contracts columns 32f .. 32f+31 of the group (words i =
//                    0,1,2,3 are registers a0,a2,a1,a3), as unsigned bytes scaled by 4^f:
//                    one logic instruction per operand register, no shift, no table.
//                    The four MMAs of a tile are independent; their accumulators D_f
//                    are combined exactly in integers, ((D_0*4 + D_1)*4 + D_2)*4 + D_3 =
//                    64 * sum(c*x), the factor 64 is divided out in FP32 together with
//                    the scale, and sum(t*x) = sum(c*x) - sum(x).  The two words of
//                    one row (i = 2h, 2h+1) are adjacent: a thread that expands ONE
//                    row, as the GEMM's does, reads them with one 64-bit load per t.
//   bytes 512..543 : scales, FP16.  half[2*gq + h] is the scale of row gq + 8h: the two
//                    scales an MMA lane needs are one 32-bit word.
//
// The layout keeps 2 bits per weight and all FP16 scales: it is exactly as large as
// the three reference arrays for matrices whose row count is a multiple of 16, and it
// is lossless for canonical masks (sign bit set only where the nonzero bit is set),
// which is all the reference's packer emits (ternarize/pack.py:135-138).
#pragma once
#include <cstdint>

namespace tllm {

constexpr int kTileRows = 16;
constexpr int kTileCodeBytes = 512;
constexpr int kTileScaleBytes = 32;
constexpr int kTileBytes = kTileCodeBytes + kTileScaleBytes;   // 544

// Weight (r16, c) of a tile, r16 = 0..15, c = 0..127: index of its code word and the bit
// position of its 2-bit code inside that word.
__host__ __device__ inline void tile_locate(int r16, int c, int& word, int& shift)
{
    const int gq = r16 & 7, h = r16 >> 3;
    const int f = c >> 5, j2 = (c >> 4) & 1, t = (c >> 2) & 3, j = c & 3;
    word = (gq * 4 + t) * 4 + 2 * h + j2;
    shift = 8 * j + 2 * f;
}

// Index of row r16's scale among the 16 FP16 scales of a tile.
__host__ __device__ inline int tile_scale_index(int r16) { return 2 * (r16 & 7) + (r16 >> 3); }

}  // namespace tllm
