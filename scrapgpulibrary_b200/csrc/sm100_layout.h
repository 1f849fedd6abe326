// The B200 weight layout ("backend-packed", layout tag 1) shared by the host packer and the kernels.
//
// A quantized tensor W = [K, N] has B = K / block_elems blocks per row and T = N * B blocks in all,
// numbered t = n * B + b.  The natural (GGUF) layout stores whole blocks one after another, which
// puts a 2..16-byte header between every run of quants, so no quant run is 16-byte aligned for
// Q4_0 / Q8_0 / Q6_K.  The packed layout splits the tensor into planes, one per block field, each
// plane holding that field of all T blocks in block order.  The planes follow each other without
// padding, so the packed tensor has exactly the natural byte count and packing is a permutation.
//
//   Q4_K  (144 B):  Q plane  T x 128 B   the quant bytes in tensor-core tile order: rows are taken 16 at a
//                                        time (a row tile), K 64 weights at a time (a pair of 32-weight
//                                        sub-blocks = 32 quant bytes per row).  One 16-row x 64-weight tile is
//                                        512 contiguous bytes, 16 per lane of a warp: lane 4g + t holds
//                                        row g bytes [4t, 4t+4) and [16+4t, 16+4t+4) of the pair, then the same
//                                        bytes of row g + 8 -- exactly the A-fragment registers of two
//                                        mma.m16n8k16 steps per sub-block, so a warp reads a tile with one
//                                        16-byte load per lane.  Tiles are ordered [row tile][pair].  The
//                                        N % 16 rows left over follow in plain row-major order.
//                   H plane  T x  16 B   per (row, block), row-major: f16 d, f16 dmin, then the eight 6-bit
//                                        (scale, min) pairs re-encoded as four 24-bit little-endian fields,
//                                        field p = sc[2p] | m[2p] << 6 | sc[2p+1] << 12 | m[2p+1] << 18
//   Q6_K  (210 B):  L plane  T x 128 B   low nibbles, regrouped in four 32-byte units: unit u = 2h + c
//                                        holds ql[64h + 16c + i] then ql[64h + 32 + 16c + i], i < 16
//                   X plane  T x  64 B   the 2-bit high parts, natural order (unit u uses bytes 16u..16u+15)
//                   S plane  T x  16 B   int8 scales regrouped per unit: sc[8h + c + {0, 2, 4, 6}]
//                   D plane  T x   2 B   f16 d
//   Q4_0  (18 B):   Q plane  T x  16 B   quant bytes;  D plane  T x 2 B   f16 d
//   Q8_0  (34 B):   Q plane  T x  32 B   int8 quants;  D plane  T x 2 B   f16 d
//
// Every 16-byte quant unit is 16-byte aligned when the tensor base is (buffers are 256-byte aligned),
// each block's quants start on a 128-byte line for the K-quants, and rows [r0, r1) of any plane are one
// contiguous run, which is what bulk (TMA) copies and fully coalesced 16-byte loads want.
#pragma once

#include <cstdint>

#ifndef __CUDACC__
#define __host__
#define __device__
#endif

namespace sm100 {

struct Planes {
    // byte offsets of the planes from the tensor base, and bytes per block in each plane
    int64_t off[4];
    int32_t per_block[4];
    int32_t count;
    int64_t n_rows;          // N
    int64_t blocks_per_row;  // K / block elements
};

// byte offset inside the Q4_K Q plane of quant byte i (0..127) of block b of row r
__host__ __device__ inline int64_t q4k_q_offset(const Planes & p, int64_t r, int64_t b, int i) {
    const int64_t full = (p.n_rows / 16) * 16;
    if (r >= full) return full * p.blocks_per_row * 128 + ((r - full) * p.blocks_per_row + b) * 128 + i;
    const int64_t pairs = p.blocks_per_row * 4;
    const int64_t c = b * 4 + (i >> 5);
    const int i32 = i & 31, g = (int) (r & 7), hi8 = (int) ((r >> 3) & 1);
    return ((r >> 4) * pairs + c) * 512 + (g * 4 + ((i32 & 15) >> 2)) * 16 + hi8 * 8 + (i32 >> 4) * 4 + (i32 & 3);
}

inline Planes planes_for(int dtype, int64_t n_rows, int64_t k) {
    Planes p = {};
    const int64_t bpr = k / (dtype == 32 || dtype == 33 ? 256 : 32);
    const int64_t total_blocks = n_rows * bpr;
    p.n_rows = n_rows;
    p.blocks_per_row = bpr;
    const int32_t q4k[] = {128, 16}, q6k[] = {128, 64, 16, 2}, q40[] = {16, 2}, q80[] = {32, 2};
    const int32_t * f = nullptr;
    switch (dtype) {
        case 32: f = q4k; p.count = 2; break;
        case 33: f = q6k; p.count = 4; break;
        case 16: f = q40; p.count = 2; break;
        case 17: f = q80; p.count = 2; break;
        default: return p;
    }
    int64_t off = 0;
    for (int i = 0; i < p.count; ++i) {
        p.off[i] = off;
        p.per_block[i] = f[i];
        off += (int64_t) f[i] * total_blocks;
    }
    return p;
}

}  // namespace sm100
