// Stage 1 of the block, THREAD-PER-POSITION variant (TRIMUL_FLAG_DIRECT_STORE_STAGE1), c = 128: LayerNorm_in, pair mask and the two
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
// Persistent kernel, one CTA per SM, 832 threads, 128-position tiles:
//   warp 0        TMA producer: the four weight matrices once, then z tiles into a 3-stage ring
//   warp 1        UMMA issuer: per tile 8 UMMAs (128 x 256 x 16) per side
//   warps 2..9    LayerNorm (+ mask): all eight warps on the same tile, 16 rows each, in place in the
//                 swizzled tile (the TMA SWIZZLE_128B image is the UMMA K-major layout); a masked
//                 position is written as a zero row, which makes both projections of that position
//                 exactly zero, so the epilogue needs no mask
//   warps 10..17  epilogue of the left side, warps 18..25 of the right side, thread = position and
//                 half of the channels (the epilogue is bound by latency, not by issue slots: eight
//                 warps per side hide it, four did not):
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

#include "tm1_common.cuh"

namespace trimul {

constexpr int kD1Threads = 832;
constexpr int kD1LnWarps = 8;             // warps 2..9
constexpr int kD1WBytes = 8 * kT1SubTile; // per side and K half: [W_proj rows | W_gate rows] = 32 KB
#ifndef TRIMUL_D1_XSTAGES
#define TRIMUL_D1_XSTAGES 3
#endif
constexpr int kD1XStages = TRIMUL_D1_XSTAGES;
constexpr int kD1OffX = kD1WBytes;
constexpr int kD1OffDest = kD1OffX + kD1XStages * kT1XBytes;   // scatter: [2 sides][8] destination base pointers
constexpr int kD1OffBars = kD1OffDest + 2 * 8 * 8;
constexpr int kD1SmemBytes = kD1OffBars + 256;
constexpr int kD1LnBarrier = 2;           // named barrier of the eight LayerNorm warps
constexpr int kD1EpiWarps = 8;            // per side
constexpr int kD1EpiBarrier = 3;          // 3: left side's eight epilogue warps, 4: right side's
static_assert(kD1SmemBytes <= 232448, "stage 1 shared memory exceeds the 227 KB a CTA may use");

template <bool kScatter>
__global__ void __launch_bounds__(kD1Threads, 1)
tm1_direct_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWl,
                 const __grid_constant__ CUtensorMap tmWlg, const __grid_constant__ CUtensorMap tmWr,
                 const __grid_constant__ CUtensorMap tmWrg, const __grid_constant__ Tm1Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm1, 900);
        return;
    }
    uint8_t* sW = smem;                                // [side][K half][proj rows | gate rows], 32 KB each
    uint8_t* sX = smem + kD1OffX;
    unsigned long long* sDest = reinterpret_cast<unsigned long long*>(smem + kD1OffDest);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kD1OffBars);
    uint64_t* w_full = bars;                           // weights landed
    uint64_t* w_ready = bars + 1;                      // weights halved (512 arrivals)
    uint64_t* x_full = bars + 2;                       // [stages] z tile landed
    uint64_t* xn_ready = x_full + kD1XStages;          // [stages] tile normalised (8 arrivals, one per warp)
    uint64_t* x_empty = xn_ready + kD1XStages;         // [stages] UMMAs that read the tile retired
    uint64_t* acc_full = x_empty + kD1XStages;         // [2] side's accumulators complete
    uint64_t* acc_empty = acc_full + 2;                // [2] side's accumulators drained (8 arrivals, one per warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    static_assert((3 * kD1XStages + 6) * 8 + 8 <= 256, "barrier block too small");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        mbar_init(w_ready, kD1Threads - 64);
        for (int s = 0; s < kD1XStages; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&xn_ready[s], kD1LnWarps);
            mbar_init(&x_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], kD1EpiWarps);
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
            halve_bf16_smem(sW, kD1WBytes, threadIdx.x - 64, kD1Threads - 64);
            fence_proxy_async_smem();
        }
        mbar_arrive(w_ready);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, kD1WBytes);
            const CUtensorMap* wm[4] = {&tmWl, &tmWlg, &tmWr, &tmWrg};
            for (int m = 0; m < 4; ++m)          // matrix m: side m >> 1, rows (m & 1) * 128 of the stacked operand
                for (int kh = 0; kh < 2; ++kh)
                    tma_load_2d(sW + ((m >> 1) * 2 + kh) * 2 * kT1SubTile + (m & 1) * kT1SubTile, wm[m], w_full,
                                kh * 64, 0);
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it % kD1XStages;
                const uint32_t ph = (it / kD1XStages) & 1u;
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
                const int s = it % kD1XStages;
                const uint32_t ph = (it / kD1XStages) & 1u;
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
    } else if (warp < 2 + kD1LnWarps) {
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
            const int s = it % kD1XStages;
            const uint32_t ph = (it / kD1XStages) & 1u;
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
            if (!group_wait<true>(&x_full[s], ph, threadIdx.x == 64, kD1LnBarrier, 32 * kD1LnWarps, abort_flag,
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
        const int ew = warp - 10;
        const int side = ew >> 3;
        const int q = warp & 3;                       // TMEM lane quarter this warp may read
        const int hch = (ew >> 2) & 1;                // channel half: channels [64 hch, 64 hch + 64)
        const int pos = q * 32 + lane;                // position inside the tile == TMEM lane
        const Tm1Dest& dst = p.dest[side];
        // p/2 of this thread's channels; g/2 128 columns on
        const uint32_t t_p = tmem_base + side * 256 + hch * 64 + ((uint32_t)(q * 32) << 16);
        const long long pstride = dst.plane_stride;
        const bool poller = (ew & 7) == 0 && lane == 0;
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
            if (!group_wait<true>(&acc_full[side], it & 1u, poller, kD1EpiBarrier + side, 32 * kD1EpiWarps, abort_flag,
                                  p.status, kStageIdTm1, 400 + side))
                break;
            tcgen05_fence_after();
            if (poller) TRIMUL_STAMP(4 + side, it, 0);
            // 8 channels at a time; the TMEM loads of the next 8 are in flight while the current 8 are
            // gated, rounded and stored.  A warp-wide store covers 32 consecutive positions of one plane row.
            auto emit8 = [&](int c8, const uint32_t (&rp)[8], const uint32_t (&rg)[8]) {
                const int plane0 = b * kT1C + hch * 64 + c8 * 8;
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
                for (int e = 0; e < 4; ++e) {
                    const uint32_t w = gate2_bf16(__uint_as_float(rp[2 * e]), __uint_as_float(rg[2 * e]),
                                                  __uint_as_float(rp[2 * e + 1]), __uint_as_float(rg[2 * e + 1]));
                    if (valid) {
                        o[(long long)(2 * e) * pstride] = (unsigned short)w;
                        o[(long long)(2 * e + 1) * pstride] = (unsigned short)(w >> 16);
                    }
                }
            };
            uint32_t rpA[8], rgA[8], rpB[8], rgB[8];
            tmem_ld_32x8(t_p, rpA);
            tmem_ld_32x8(t_p + 128, rgA);
#pragma unroll 1
            for (int c8 = 0; c8 < 8; c8 += 2) {
                tmem_ld_wait();
                tmem_ld_32x8(t_p + (c8 + 1) * 8, rpB);
                tmem_ld_32x8(t_p + 128 + (c8 + 1) * 8, rgB);
                emit8(c8, rpA, rgA);
                tmem_ld_wait();
                if (c8 + 2 < 8) {
                    tmem_ld_32x8(t_p + (c8 + 2) * 8, rpA);
                    tmem_ld_32x8(t_p + 128 + (c8 + 2) * 8, rgA);
                } else {
                    // every TMEM read of this warp's share has completed: hand the accumulators back early
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[side]);
                    if (poller) TRIMUL_STAMP(4 + side, it, 1);
                }
                emit8(c8 + 1, rpB, rgB);
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
