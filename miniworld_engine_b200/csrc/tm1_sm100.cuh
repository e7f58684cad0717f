// Stage 1 of the block on the tensor cores, c = 128: LayerNorm_in, pair mask and the two
// sigmoid-gated projections in ONE pass over z (reference.py:66-75), writing the operands a and b
// as channel-major planes for the contraction.
//
// Shape of the tensor-core work.  On a B200 a tcgen05.mma costs about 93 cycles however small it
// is, and operands are fetched from shared memory at about 75 bytes per cycle (both measured), so
// the only efficient instruction is the widest one: M = 128, N = 256, K = 16.  Each side (left = a,
// right = b) is therefore ONE accumulation chain D[position][p | g] = x_n . [W_proj ; W_gate]^T:
// the normalised tile is the A operand (128 positions, K-major as TMA wrote it), the projection and
// gate weights of the side are stacked into one 256-row B operand, and D is 256 TMEM columns
// (p/2 in [0,128), g/2 in [128,256): the weights are halved once in shared memory, exact in bf16, so
// p * sigmoid(g) = (p/2) * tanh(g/2) + p/2 is one MUFU and one FMA).  Eight UMMAs per side and tile
// instead of 16 of half the width; the two sides' accumulators fill the 512 TMEM columns, and the
// epilogue of one side overlaps the UMMAs of the other.
//
// A TMEM lane is a POSITION, so an epilogue thread holds all 128 channels of one position, while the
// destination is channel-major.  The 32 lanes of a warp are 32 consecutive positions, i.e. 64
// contiguous bytes of one plane row: the epilogue stores straight to global memory, one
// 2-byte store per channel and lane, each warp-wide store a full 64-byte segment.  No staging
// buffer, no transposition pass, no shared-memory traffic for the results at all — what this
// stage is short of is shared-memory bandwidth (the UMMA operand fetch alone uses most of it), not
// store instructions.  For the same reason the LayerNorm is warp-cooperative (eight lanes per
// row): every value is read from shared memory once, stays in registers between statistics and
// normalisation, and gamma / beta are register-resident.
//
// Persistent kernel, one CTA per SM, 576 threads, 128-position tiles:
//   warp 0        TMA producer: the four weight matrices once, then z tiles into a 3-stage ring
//   warp 1        UMMA issuer: per tile 8 UMMAs (128 x 256 x 16) per side
//   warps 2..9    LayerNorm (+ mask): all eight warps on the same tile, 16 rows each, in place in the
//                 swizzled tile (the TMA SWIZZLE_128B image is the UMMA K-major layout); a masked
//                 position is written as a zero row, which makes both projections of that position
//                 exactly zero, so the epilogue needs no mask
//   warps 10..13  epilogue of the left side, warps 14..17 of the right side, thread = position:
//                 TMEM -> p * sigmoid(g) -> bf16 -> global
//
// kScatter = true: the planes are split over several destination buffers, planes_per_dest planes
// each (a multiple of 16 that divides or is a multiple of 128) — the multi-GPU exchange of the
// channel-sharded contraction, done by this kernel's own stores into the consumer's memory.
//
// A tile is 128 consecutive positions along the index that becomes the contraction's k: for the
// outgoing direction z row f, columns t0..t0+127; for the incoming direction z column f, rows
// t0..t0+127 (a strided TMA box), so both directions store plane element (f, t0+p).
#pragma once

#include "ptx_sm100.cuh"

namespace trimul {

constexpr int kT1C = 128;                 // channels
constexpr int kT1P = 128;                 // positions per tile
constexpr int kT1Threads = 576;
constexpr int kT1LnWarps = 8;             // warps 2..9
constexpr int kT1SubTile = 128 * 64 * 2;  // 16 KB: 128 rows x 64 bf16, one swizzle-row wide
constexpr int kT1XBytes = 2 * kT1SubTile; // one z tile
constexpr int kT1WBytes = 8 * kT1SubTile; // per side and K half: [W_proj rows | W_gate rows] = 32 KB
#ifndef TRIMUL_T1_XSTAGES
#define TRIMUL_T1_XSTAGES 3
#endif
constexpr int kT1XStages = TRIMUL_T1_XSTAGES;
constexpr int kT1OffX = kT1WBytes;
constexpr int kT1OffDest = kT1OffX + kT1XStages * kT1XBytes;   // scatter: [2 sides][8] destination base pointers
constexpr int kT1OffBars = kT1OffDest + 2 * 8 * 8;
constexpr int kT1SmemBytes = kT1OffBars + 256;
constexpr int kStageIdTm1 = 1;
constexpr int kT1LnBarrier = 2;           // named barrier of the eight LayerNorm warps
constexpr int kT1EpiBarrier = 3;          // 3: left side's four epilogue warps, 4: right side's
static_assert(kT1SmemBytes <= 232448, "stage 1 shared memory exceeds the 227 KB a CTA may use");

// Where one side's planes go: element (plane, r, q) of the logical [planes][rows][cols] array lies at
//   base + (r / row_chunk) * chunk_stride + plane * plane_stride + (r % row_chunk) * pitch + q      (row-chunked)
//   base + (q / col_chunk) * chunk_stride + plane * plane_stride + r * pitch + (q % col_chunk)      (col-chunked)
// in elements (at most one of the two is chunked; an unchunked extent has chunk == extent).
struct Tm1Dest {
    __nv_bfloat16* base[8];   // one per destination buffer (index 0 only unless scattering)
    long long plane_stride, chunk_stride;
    int pitch, row_chunk, col_chunk;
};

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
    int planes_per_dest;  // scatter variant: planes of one destination (a multiple of 16; divides or is a multiple of 128)
    int32_t* status;
    Tm1Dest dest[2];      // a, b
};

template <bool kScatter>
__global__ void __launch_bounds__(kT1Threads, 1)
tm1_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWl,
                 const __grid_constant__ CUtensorMap tmWlg, const __grid_constant__ CUtensorMap tmWr,
                 const __grid_constant__ CUtensorMap tmWrg, const __grid_constant__ Tm1Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm1, 900);
        return;
    }
    uint8_t* sW = smem;                                // [side][K half][proj rows | gate rows], 32 KB each
    uint8_t* sX = smem + kT1OffX;
    unsigned long long* sDest = reinterpret_cast<unsigned long long*>(smem + kT1OffDest);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kT1OffBars);
    uint64_t* w_full = bars;                           // weights landed
    uint64_t* w_ready = bars + 1;                      // weights halved (512 arrivals)
    uint64_t* x_full = bars + 2;                       // [stages] z tile landed
    uint64_t* xn_ready = x_full + kT1XStages;          // [stages] tile normalised (8 arrivals, one per warp)
    uint64_t* x_empty = xn_ready + kT1XStages;         // [stages] UMMAs that read the tile retired
    uint64_t* acc_full = x_empty + kT1XStages;         // [2] side's accumulators complete
    uint64_t* acc_empty = acc_full + 2;                // [2] side's accumulators drained (4 arrivals, one per warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    static_assert((3 * kT1XStages + 6) * 8 + 8 <= 256, "barrier block too small");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        mbar_init(w_ready, kT1Threads - 64);
        for (int s = 0; s < kT1XStages; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&xn_ready[s], kT1LnWarps);
            mbar_init(&x_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        *abort_flag = 0;
        fence_mbarrier_init();
        tma_prefetch_desc(&tmZ);
    }
    if (kScatter && threadIdx.x >= 64 && threadIdx.x < 64 + 16) {
        const int i = threadIdx.x - 64;
        sDest[i] = reinterpret_cast<unsigned long long>(p.dest[i >> 3].base[i & 7]);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Everything above touches no global memory; from here on the kernel reads what its
    // predecessor in the stream may have written.
    griddep_wait();
    griddep_launch_dependents();

    if (warp >= 2) {
        // every worker thread: halve its share of the weights once they have landed
        if (mbar_wait<true>(w_full, 0, abort_flag, p.status, kStageIdTm1, 150)) {
            halve_bf16_smem(sW, kT1WBytes, threadIdx.x - 64, kT1Threads - 64);
            fence_proxy_async_smem();
        }
        mbar_arrive(w_ready);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, kT1WBytes);
            const CUtensorMap* wm[4] = {&tmWl, &tmWlg, &tmWr, &tmWrg};
            for (int m = 0; m < 4; ++m)          // matrix m: side m >> 1, rows (m & 1) * 128 of the stacked operand
                for (int kh = 0; kh < 2; ++kh)
                    tma_load_2d(sW + ((m >> 1) * 2 + kh) * 2 * kT1SubTile + (m & 1) * kT1SubTile, wm[m], w_full,
                                kh * 64, 0);
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it % kT1XStages;
                const uint32_t ph = (it / kT1XStages) & 1u;
                if (!mbar_wait<true>(&x_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm1, 100 + s)) break;
                const int t0 = (tile % p.tiles_per_fixed) * kT1P;
                const int bf = tile / p.tiles_per_fixed;
                const int f = bf % p.n_fixed;
                const int b = bf / p.n_fixed;
                mbar_arrive_expect_tx(&x_full[s], kT1XBytes);
                uint8_t* dst = sX + s * kT1XBytes;
                // z viewed as (channel, column, row, batch); outgoing box = 128 columns of row f,
                // incoming box = 128 rows of column f
                const int col = p.incoming ? f : t0;
                const int row = p.incoming ? t0 : f;
                tma_load_4d(dst, &tmZ, &x_full[s], 0, col, row, b);
                tma_load_4d(dst + kT1SubTile, &tmZ, &x_full[s], 64, col, row, b);
                TRIMUL_STAMP(0, it, 0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(kT1P, 256);
            bool ok = mbar_wait<true>(w_ready, 0, abort_flag, p.status, kStageIdTm1, 200);
            tcgen05_fence_after();
            uint32_t it = 0;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it % kT1XStages;
                const uint32_t ph = (it / kT1XStages) & 1u;
                if (!mbar_wait<true>(&xn_ready[s], ph, abort_flag, p.status, kStageIdTm1, 210 + s)) break;
                tcgen05_fence_after();
                TRIMUL_STAMP(1, it, 0);
                const uint32_t xs = smem_u32(sX + s * kT1XBytes);
                for (int side = 0; side < 2; ++side) {
                    if (!mbar_wait<true>(&acc_empty[side], (it & 1u) ^ 1u, abort_flag, p.status, kStageIdTm1,
                                         220 + side)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t d = tmem_base + side * 256;
                    const uint32_t ws = smem_u32(sW + side * 4 * kT1SubTile);
#pragma unroll
                    for (int kk = 0; kk < kT1C / 16; ++kk) {
                        const uint64_t kofs = (kk & 3) * kDescKStep;
                        umma_bf16_ss(d, umma_smem_desc_sw128(xs + (kk >> 2) * kT1SubTile) + kofs,
                                     umma_smem_desc_sw128(ws + (kk >> 2) * 2 * kT1SubTile) + kofs, idesc, kk != 0);
                    }
                    umma_commit(&acc_full[side]);
                    TRIMUL_STAMP(1, it, 1 + side);
                }
                if (!ok) break;
                umma_commit(&x_empty[s]);   // both sides' UMMAs have read the tile when this fires
            }
        }
        __syncwarp();
    } else if (warp < 2 + kT1LnWarps) {
        // ------------------------------------------------------------------ LayerNorm (+ mask)
        // warp lw owns rows [16 lw, 16 lw + 16) of every tile; lane l row 16 lw + 4 i + (l >> 3) in
        // iteration i, 16-byte chunk l & 7 of both 64-channel sub-tiles
        const int lw = warp - 2;
        const int rr = lane >> 3;
        const int j = lane & 7;
        f32x2 gb[16];
        {
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(p.gamma + 8 * j));
            const float4 g1 = __ldg(reinterpret_cast<const float4*>(p.gamma + 8 * j + 4));
            const float4 g2 = __ldg(reinterpret_cast<const float4*>(p.gamma + 64 + 8 * j));
            const float4 g3 = __ldg(reinterpret_cast<const float4*>(p.gamma + 64 + 8 * j + 4));
            const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.beta + 8 * j));
            const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.beta + 8 * j + 4));
            const float4 b2 = __ldg(reinterpret_cast<const float4*>(p.beta + 64 + 8 * j));
            const float4 b3 = __ldg(reinterpret_cast<const float4*>(p.beta + 64 + 8 * j + 4));
            gb[0] = f2_pack(g0.x, g0.y); gb[1] = f2_pack(g0.z, g0.w); gb[2] = f2_pack(g1.x, g1.y); gb[3] = f2_pack(g1.z, g1.w);
            gb[4] = f2_pack(g2.x, g2.y); gb[5] = f2_pack(g2.z, g2.w); gb[6] = f2_pack(g3.x, g3.y); gb[7] = f2_pack(g3.z, g3.w);
            gb[8] = f2_pack(b0.x, b0.y); gb[9] = f2_pack(b0.z, b0.w); gb[10] = f2_pack(b1.x, b1.y); gb[11] = f2_pack(b1.z, b1.w);
            gb[12] = f2_pack(b2.x, b2.y); gb[13] = f2_pack(b2.z, b2.w); gb[14] = f2_pack(b3.x, b3.y); gb[15] = f2_pack(b3.z, b3.w);
        }
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it % kT1XStages;
            const uint32_t ph = (it / kT1XStages) & 1u;
            // pair-mask bits of this lane's four rows (independent of the tile data: do it first)
            uint32_t zero_bits = 0u;
            if (p.mask_kind != 0) {
                const int t0 = (tile % p.tiles_per_fixed) * kT1P;
                const int bf = tile / p.tiles_per_fixed;
                const int f = bf % p.n_fixed;
                const int b = bf / p.n_fixed;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int run = t0 + 16 * lw + 4 * i + rr;
                    bool keep = false;
                    if (run < p.n_run) {
                        const int zr = p.row0 + (p.incoming ? run : f);   // global z row
                        const int zc = p.incoming ? f : run;              // z column
                        if (p.mask_kind == 1)
                            keep = (p.mask[(size_t)b * p.N + zr] != 0) && (p.mask[(size_t)b * p.N + zc] != 0);
                        else
                            keep = p.mask[((size_t)b * p.N + zr) * p.N + zc] != 0;
                    }
                    if (!keep) zero_bits |= 1u << i;
                }
            }
            // ONE thread of the eight warps polls; the others park at the group's named barrier
            if (!group_wait<true>(&x_full[s], ph, threadIdx.x == 64, kT1LnBarrier, 32 * kT1LnWarps, abort_flag,
                                  p.status, kStageIdTm1, 300 + s))
                break;
            if (lw == 0 && lane == 0) TRIMUL_STAMP(2, it, 0);
            ln_rows_warp<4>(sX + s * kT1XBytes, kT1SubTile, 16 * lw, lane, gb, p.eps, zero_bits);
            fence_proxy_async_smem();   // normalised rows -> visible to the UMMA (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive(&xn_ready[s]);
            if (lw == 0 && lane == 0) TRIMUL_STAMP(2, it, 1);
        }
    } else {
        // ------------------------------------------------------------------ epilogue, one side per group
        const int side = (warp - 10) >> 2;
        const int q = warp & 3;
        const int pos = q * 32 + lane;                // position inside the tile == TMEM lane
        const Tm1Dest& dst = p.dest[side];
        const uint32_t t_p = tmem_base + side * 256 + ((uint32_t)(q * 32) << 16);   // p/2; g/2 128 columns on
        const long long pstride = dst.plane_stride;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int t0 = (tile % p.tiles_per_fixed) * kT1P;
            const int bf = tile / p.tiles_per_fixed;
            const int f = bf % p.n_fixed;
            const int b = bf / p.n_fixed;
            // where this thread's position lies inside a plane (elements)
            const int run = t0 + pos;
            const bool valid = run < p.n_run;
            const long long in_plane = (long long)(f / dst.row_chunk + run / dst.col_chunk) * dst.chunk_stride +
                                       (long long)(f % dst.row_chunk) * dst.pitch + run % dst.col_chunk;
            if (!group_wait<true>(&acc_full[side], it & 1u, q == 2 && lane == 0, kT1EpiBarrier + side, 128, abort_flag,
                                  p.status, kStageIdTm1, 400 + side))
                break;
            tcgen05_fence_after();
            if (q == 2 && lane == 0) TRIMUL_STAMP(4 + side, it, 0);
            // 16 channels at a time; the TMEM loads of the next 16 are in flight while the current 16 are
            // gated, rounded and stored.  A warp-wide store covers 32 consecutive positions of one plane row.
            auto emit16 = [&](int c16, const uint32_t (&rp)[16], const uint32_t (&rg)[16]) {
                const int plane0 = b * kT1C + c16 * 16;
                __nv_bfloat16* base;
                int pin = plane0;
                if (kScatter) {
                    const int d = plane0 / p.planes_per_dest;
                    pin = plane0 - d * p.planes_per_dest;
                    base = reinterpret_cast<__nv_bfloat16*>(sDest[side * 8 + d]);
                } else {
                    base = dst.base[0];
                }
                unsigned short* o = reinterpret_cast<unsigned short*>(base + (long long)pin * pstride + in_plane);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t w = gate2_bf16(__uint_as_float(rp[2 * e]), __uint_as_float(rg[2 * e]),
                                                  __uint_as_float(rp[2 * e + 1]), __uint_as_float(rg[2 * e + 1]));
#ifdef TRIMUL_T1_NO_STORE
                    if (valid && w == 0x12345678u) o[0] = (unsigned short)w;      // timing experiment: no stores
#else
                    if (valid) {
                        o[(long long)(2 * e) * pstride] = (unsigned short)(w & 0xffffu);
                        o[(long long)(2 * e + 1) * pstride] = (unsigned short)(w >> 16);
                    }
#endif
                }
            };
            uint32_t rpA[16], rgA[16], rpB[16], rgB[16];
            tmem_ld_32x16(t_p, rpA);
            tmem_ld_32x16(t_p + 128, rgA);
#pragma unroll 1
            for (int c16 = 0; c16 < 8; c16 += 2) {
                tmem_ld_wait();
                tmem_ld_32x16(t_p + (c16 + 1) * 16, rpB);
                tmem_ld_32x16(t_p + 128 + (c16 + 1) * 16, rgB);
                emit16(c16, rpA, rgA);
                tmem_ld_wait();
                if (c16 + 2 < 8) {
                    tmem_ld_32x16(t_p + (c16 + 2) * 16, rpA);
                    tmem_ld_32x16(t_p + 128 + (c16 + 2) * 16, rgA);
                } else {
                    // every TMEM read of this warp's lanes has completed: hand the accumulators back early
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[side]);
                    if (q == 2 && lane == 0) TRIMUL_STAMP(4 + side, it, 1);
                }
                emit16(c16 + 1, rpB, rgB);
            }
        }
    }

    if (*abort_flag != 0) {
        for (int i = 0; i < 256; ++i) __nanosleep(1000);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace trimul
