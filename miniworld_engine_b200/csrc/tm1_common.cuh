// Constants and launch parameters shared by the c = 128 stage-1 kernels (tm1_pair_sm100.cuh, the
// default, and tm1_sm100.cuh, the lone-CTA form that also scatters).
#pragma once

#include "ptx_sm100.cuh"

namespace trimul {

constexpr int kT1C = 128;                 // channels
constexpr int kT1P = 128;                 // positions per tile
constexpr int kT1SubTile = 128 * 64 * 2;  // 16 KB: 128 rows x 64 bf16, one swizzle-row wide
constexpr int kT1XBytes = 2 * kT1SubTile; // one z tile
constexpr int kStageIdTm1 = 1;

struct Tm1Params {
    int B, c;
    int n_fixed;          // extent of the tile's fixed index (outgoing: rows, incoming: N)
    int n_run;            // extent of the running index     (outgoing: N,    incoming: rows)
    int tiles_per_fixed;  // ceil(n_run / 128)
    int total_tiles;      // B * n_fixed * tiles_per_fixed
    int incoming;         // 0 / 1
    int N, row0;          // full token count and global index of the slab's first z row
    int mask_kind;
    const uint8_t* mask;
    const float* gamma;
    const float* beta;
    float eps;
    int a_row_chunk, a_col_chunk, b_row_chunk, b_col_chunk;
    int planes_per_dest;  // scatter variants: planes of one destination (a multiple of 16; divides or is a multiple of 128)
    int32_t* status;
};

// Tile index -> (batch element, fixed index f, first running position t0); the running index is the
// fast one.  (Walking the tiles from the end of the tensor, to start on whatever the previous kernel
// left in L2, was measured and changed nothing.)
__device__ __forceinline__ void tm1_decode_tile(const Tm1Params& p, int tile, int& b, int& f, int& t0) {
    t0 = (tile % p.tiles_per_fixed) * kT1P;
    const int bf = tile / p.tiles_per_fixed;
    f = bf % p.n_fixed;
    b = bf / p.n_fixed;
}

}  // namespace trimul
