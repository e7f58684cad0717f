// Stage 1 of the block on the tensor cores for c = h = 64 (the narrowest case of the reference's
// d_pair sweep): LayerNorm_in, pair mask and the two sigmoid-gated projections in one pass over z
// (reference.py:66-75), writing a and b as channel-major planes.
//
// Transposed like the other stage-1 kernels (D^T[channel][position], TMEM lane = output channel,
// epilogue thread = one channel and a run of positions -> swizzled staging box -> TMA store), but a
// side has only 64 output channels, and a tcgen05.mma wants M = 128: the LEFT and RIGHT weights are
// stacked into one A operand, [W_left ; W_right] for the projections and [W_left_gate ;
// W_right_gate] for the gates, so lanes 0..63 of the accumulators are the channels of a and lanes
// 64..127 those of b.  A tile is then 8 UMMAs (K = 64) into 2 x 128 TMEM columns; the accumulators
// are double-buffered, the four 8 KB weight matrices stay in shared memory (halved once, exact in
// bf16, for the tanh form of the gate) and the z ring is four 16 KB tiles deep.
//
// Persistent kernel, one CTA per SM, 576 threads, 128-position tiles:
//   warp 0        TMA producer: the weights once, then z tiles
//   warp 1        UMMA issuer
//   warps 2..9    LayerNorm: two groups of four warps on alternate tiles, one thread per position,
//                 in place in the swizzled tile; a masked position becomes a zero row
//   warps 10..13  epilogue of the even tiles, warps 14..17 of the odd tiles
#pragma once

#include "tm1_common.cuh"

namespace trimul {

constexpr int kN1C = 64;
constexpr int kN1Threads = 576;
constexpr int kN1LnThreads = 256;
constexpr int kN1XBytes = kT1SubTile;               // one z tile: [128 positions][64 channels] = 16 KB
constexpr int kN1XStages = 4;
constexpr int kN1WBytes = 2 * kT1SubTile;           // stacked proj operand + stacked gate operand
constexpr int kN1OffX = kN1WBytes;
constexpr int kN1OffStaging = kN1OffX + kN1XStages * kN1XBytes;     // one [128 lanes][64 positions] box per epilogue group
constexpr int kN1OffAffine = kN1OffStaging + 2 * kT1SubTile;
constexpr int kN1OffBars = kN1OffAffine + 2 * kN1C * 4;
constexpr int kN1SmemBytes = kN1OffBars + 256;
constexpr int kN1LnBarrier = 2;        // 2, 3: the two LayerNorm groups
constexpr int kN1EpiBarrier = 4;       // 4, 5: the two epilogue groups
constexpr int kN1AffineBarrier = 6;

__global__ void __launch_bounds__(kN1Threads, 1)
tm1_narrow_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWl,
                        const __grid_constant__ CUtensorMap tmWlg, const __grid_constant__ CUtensorMap tmWr,
                        const __grid_constant__ CUtensorMap tmWrg, const __grid_constant__ CUtensorMap tmA,
                        const __grid_constant__ CUtensorMap tmB, const __grid_constant__ Tm1Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm1, 900);
        return;
    }
    uint8_t* sW = smem;                       // [0, 16 KB): [W_left ; W_right], [16, 32 KB): [W_left_gate ; W_right_gate]
    uint8_t* sX = smem + kN1OffX;
    uint8_t* sOut = smem + kN1OffStaging;
    float* sGamma = reinterpret_cast<float*>(smem + kN1OffAffine);
    float* sBeta = sGamma + kN1C;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kN1OffBars);
    uint64_t* w_full = bars;                          // weights landed
    uint64_t* w_ready = bars + 1;                     // weights halved (512 arrivals)
    uint64_t* x_full = bars + 2;                      // [stages]
    uint64_t* xn_ready = x_full + kN1XStages;         // [stages] (128 arrivals)
    uint64_t* x_empty = xn_ready + kN1XStages;        // [stages]
    uint64_t* acc_full = x_empty + kN1XStages;        // [2]
    uint64_t* acc_empty = acc_full + 2;               // [2] (4 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    static_assert((6 + 3 * kN1XStages) * 8 + 8 <= 256, "barrier block too small");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        mbar_init(w_ready, kN1Threads - 64);
        for (int s = 0; s < kN1XStages; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&xn_ready[s], kN1LnThreads / 2);
            mbar_init(&x_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        *abort_flag = 0;
        fence_mbarrier_init();
        tma_prefetch_desc(&tmZ);
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
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

    if (warp >= 2 && warp < 10) {
        if (threadIdx.x < 64 + kN1C) {
            sGamma[threadIdx.x - 64] = p.gamma[threadIdx.x - 64];
            sBeta[threadIdx.x - 64] = p.beta[threadIdx.x - 64];
        }
        named_barrier_sync(kN1AffineBarrier, kN1LnThreads);
    }
    if (warp >= 2) {
        // every worker thread: halve its share of the weights once they have landed
        if (mbar_wait<true>(w_full, 0, abort_flag, p.status, kStageIdTm1, 150)) {
            halve_bf16_smem(sW, kN1WBytes, threadIdx.x - 64, kN1Threads - 64);
            fence_proxy_async_smem();
        }
        mbar_arrive(w_ready);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, kN1WBytes);
            // box = [64 rows][64 k] = 8 KB: left matrix into rows 0..63, right matrix into rows 64..127
            tma_load_2d(sW, &tmWl, w_full, 0, 0);
            tma_load_2d(sW + 8192, &tmWr, w_full, 0, 0);
            tma_load_2d(sW + kT1SubTile, &tmWlg, w_full, 0, 0);
            tma_load_2d(sW + kT1SubTile + 8192, &tmWrg, w_full, 0, 0);
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it % kN1XStages;
                const uint32_t ph = (it / kN1XStages) & 1u;
                if (!mbar_wait<true>(&x_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm1, 100 + s)) break;
                const int t0 = (tile % p.tiles_per_fixed) * kT1P;
                const int bf = tile / p.tiles_per_fixed;
                const int f = bf % p.n_fixed;
                const int b = bf / p.n_fixed;
                mbar_arrive_expect_tx(&x_full[s], kN1XBytes);
                tma_load_4d(sX + s * kN1XBytes, &tmZ, &x_full[s], 0, p.incoming ? f : t0, p.incoming ? t0 : f, b);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(128, kT1P);
            bool ok = mbar_wait<true>(w_ready, 0, abort_flag, p.status, kStageIdTm1, 200);
            tcgen05_fence_after();
            const uint32_t wp = smem_u32(sW), wg = smem_u32(sW + kT1SubTile);
            uint32_t it = 0;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it % kN1XStages;
                const uint32_t ph = (it / kN1XStages) & 1u;
                const int acc = it & 1;
                if (!mbar_wait<true>(&xn_ready[s], ph, abort_flag, p.status, kStageIdTm1, 210 + s)) break;
                if (!mbar_wait<true>(&acc_empty[acc], ((it >> 1) & 1u) ^ 1u, abort_flag, p.status, kStageIdTm1, 220 + acc))
                    break;
                tcgen05_fence_after();
                const uint32_t xs = smem_u32(sX + s * kN1XBytes);
                const uint32_t d_p = tmem_base + acc * 256, d_g = d_p + 128;
#pragma unroll
                for (int kk = 0; kk < kN1C / 16; ++kk) {
                    const uint64_t kofs = kk * kDescKStep;
                    const uint64_t db = umma_smem_desc_sw128(xs) + kofs;
                    umma_bf16_ss(d_p, umma_smem_desc_sw128(wp) + kofs, db, idesc, kk != 0);
                    umma_bf16_ss(d_g, umma_smem_desc_sw128(wg) + kofs, db, idesc, kk != 0);
                }
                umma_commit(&acc_full[acc]);
                umma_commit(&x_empty[s]);
            }
        }
        __syncwarp();
    } else if (warp < 10) {
        // ------------------------------------------------------------------ LayerNorm (+ mask)
        const int g = (warp - 2) >> 2;
        const int pos = threadIdx.x - 64 - g * 128;    // 0..127, row of the tile
        uint32_t it = g;
        for (int tile = blockIdx.x + g * gridDim.x; tile < p.total_tiles; tile += 2 * gridDim.x, it += 2) {
            const int s = it % kN1XStages;
            const uint32_t ph = (it / kN1XStages) & 1u;
            bool keep = true;
            if (p.mask_kind != 0) {
                const int t0 = (tile % p.tiles_per_fixed) * kT1P;
                const int bf = tile / p.tiles_per_fixed;
                const int f = bf % p.n_fixed;
                const int b = bf / p.n_fixed;
                const int run = t0 + pos;
                keep = false;
                if (run < p.n_run) {
                    const int zr = p.row0 + (p.incoming ? run : f);   // global z row
                    const int zc = p.incoming ? f : run;              // z column
                    if (p.mask_kind == 1)
                        keep = (p.mask[(size_t)b * p.N + zr] != 0) && (p.mask[(size_t)b * p.N + zc] != 0);
                    else
                        keep = p.mask[((size_t)b * p.N + zr) * p.N + zc] != 0;
                }
            }
            if (!group_wait<true>(&x_full[s], ph, pos == 0, kN1LnBarrier + g, 128, abort_flag, p.status, kStageIdTm1,
                                  300 + s))
                break;
            ln_row_inplace<1>(sX + s * kN1XBytes, kT1SubTile, pos, sGamma, sBeta, p.eps, !keep);
            fence_proxy_async_smem();
            mbar_arrive(&xn_ready[s]);
        }
    } else {
        // ------------------------------------------------------------------ epilogue, alternate tiles per group
        const int grp = (warp - 10) >> 2;             // == accumulator pair == parity of the local tile index
        const int q = warp & 3;
        const int ln = q * 32 + lane;                 // TMEM lane: 0..63 channels of a, 64..127 channels of b
        const bool leader = ((warp - 10) & 3) == 0 && lane == 0;
        const int bar_id = kN1EpiBarrier + grp;
        uint8_t* stg = sOut + grp * kT1SubTile;
        const uint32_t t_p = tmem_base + grp * 256 + ((uint32_t)(q * 32) << 16);
        uint32_t it = grp;
        for (int tile = blockIdx.x + grp * gridDim.x; tile < p.total_tiles; tile += 2 * gridDim.x, it += 2) {
            const int t0 = (tile % p.tiles_per_fixed) * kT1P;
            const int bf = tile / p.tiles_per_fixed;
            const int f = bf % p.n_fixed;
            const int b = bf / p.n_fixed;
            if (!group_wait<true>(&acc_full[grp], (it >> 1) & 1u, leader, bar_id, 128, abort_flag, p.status, kStageIdTm1,
                                  400 + grp))
                break;
            tcgen05_fence_after();
            auto emit16 = [&](int c16, const uint32_t (&rp)[16], const uint32_t (&rg)[16]) {
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i0 = k * 8 + 2 * e;
                        o[e] = gate2_bf16(__uint_as_float(rp[i0]), __uint_as_float(rg[i0]),
                                          __uint_as_float(rp[i0 + 1]), __uint_as_float(rg[i0 + 1]));
                    }
                    const int chunk = ((c16 & 3) * 2 + k) ^ (ln & 7);
                    *reinterpret_cast<uint4*>(stg + ln * 128 + (chunk << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            };
            uint32_t rpA[16], rgA[16], rpB[16], rgB[16];
            tmem_ld_32x16(t_p, rpA);
            tmem_ld_32x16(t_p + 128, rgA);
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                if (leader) tma_store_wait_read<0>();      // the previous stores have read the staging box
                named_barrier_sync(bar_id, 128);
#pragma unroll 1
                for (int cp = 0; cp < 2; ++cp) {
                    const int c16 = half * 4 + cp * 2;
                    tmem_ld_wait();
                    tmem_ld_32x16(t_p + (c16 + 1) * 16, rpB);
                    tmem_ld_32x16(t_p + 128 + (c16 + 1) * 16, rgB);
                    emit16(c16, rpA, rgA);
                    tmem_ld_wait();
                    if (c16 + 2 < 8) {
                        tmem_ld_32x16(t_p + (c16 + 2) * 16, rpA);
                        tmem_ld_32x16(t_p + 128 + (c16 + 2) * 16, rgA);
                    } else {
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[grp]);
                    }
                    emit16(c16 + 1, rpB, rgB);
                }
                fence_proxy_async_smem();
                named_barrier_sync(bar_id, 128);
                if (leader) {
                    const int col0 = t0 + half * 64;
                    if (col0 < p.n_run) {
                        // rows 0..63 of the box are the planes of a, rows 64..127 those of b
                        tma_store_4d(&tmA, stg, col0 % p.a_col_chunk, f % p.a_row_chunk, b * kN1C,
                                     col0 / p.a_col_chunk + f / p.a_row_chunk);
                        tma_store_4d(&tmB, stg + 64 * 128, col0 % p.b_col_chunk, f % p.b_row_chunk, b * kN1C,
                                     col0 / p.b_col_chunk + f / p.b_row_chunk);
                        tma_store_commit();
                    }
                }
            }
        }
        if (leader) tma_store_wait_all<0>();
        __syncwarp();
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
