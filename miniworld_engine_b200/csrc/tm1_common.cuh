// Constants and launch parameters shared by the c = 128 stage-1 kernels (tm1_pair_sm100.cuh, the
// default, and tm1_sm100.cuh, the lone-CTA form).
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
    int step_q[2], step_r[2];   // tile strides of the pair kernel's roles (clusters, 2 x clusters) as q * tiles_per_fixed + r
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

// The same decode for a role that walks tiles first, first + stride, ...: the divisions are done once,
// every further tile costs a few adds (a decode per tile in every warp of every role was a measurable
// share of the LayerNorm warps' instructions).
struct Tm1Cursor {
    int b, f, ti;      // batch element, fixed index, tile index along the running index
    __device__ __forceinline__ void init(const Tm1Params& p, int first) {
        ti = first % p.tiles_per_fixed;
        const int bf = first / p.tiles_per_fixed;
        f = bf % p.n_fixed;
        b = bf / p.n_fixed;
    }
    // advance by stride k (p.step_q[k] * tiles_per_fixed + p.step_r[k] tiles)
    __device__ __forceinline__ void next(const Tm1Params& p, int k) {
        ti += p.step_r[k];
        f += p.step_q[k];
        if (ti >= p.tiles_per_fixed) {
            ti -= p.tiles_per_fixed;
            ++f;
        }
        while (f >= p.n_fixed) {
            f -= p.n_fixed;
            ++b;
        }
    }
    __device__ __forceinline__ int t0() const { return ti * kT1P; }
};

// Pair-mask value of running position `run` of a tile with fixed index f (reference.py:72-75):
// token masks: m[b, zr] & m[b, zc]; pair masks: m[b, zr, zc]; zr is the global z row, zc the z column.
// One or two byte loads; positions past the end of the running index are masked.
__device__ __forceinline__ bool tm1_keep(const Tm1Params& p, int b, int f, int run) {
    if (run >= p.n_run) return false;
    const int zr = p.row0 + (p.incoming ? run : f);
    const int zc = p.incoming ? f : run;
    const uint8_t* mb = p.mask + (size_t)b * p.N;
    if (p.mask_kind == 1) return (mb[zr] != 0) && (mb[zc] != 0);
    return p.mask[((size_t)b * p.N + zr) * p.N + zc] != 0;
}

}  // namespace trimul
