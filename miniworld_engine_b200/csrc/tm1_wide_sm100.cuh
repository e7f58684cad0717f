// Stage 1 of the block on the tensor cores for c = h = 256 (the widest case of the reference's
// d_pair sweep): LayerNorm_in, pair mask and the two sigmoid-gated projections in one pass over z
// (reference.py:66-75), writing a and b as channel-major planes.
//
// Same transposed formulation as the c = 128 kernel (tm1_sm100.cuh): D^T[channel][position] =
// W[channel][:] . x_n[position][:], weights as the UMMA A operand in their [out,in] layout, the
// normalised tile as the B operand, TMEM lane = output channel, epilogue thread = one channel and a
// run of consecutive positions -> swizzled staging box -> TMA store.  What differs is size: the
// four 256 x 256 weight matrices are 512 KB and do not stay in shared memory, so they are STREAMED
// from L2 through a ring of [128 rows][64 k] slots beside the z ring, and a tile is worked off in four
// UNITS (side, channel half): per unit 128 output channels of proj and of gate (2 x 128 TMEM columns)
// over K = 256, i.e. 32 UMMAs of 128 x 128 x 16.  Two units' accumulators fit in tensor memory, so
// the epilogue of one unit overlaps the UMMAs of the next.  The streamed weights cannot be halved
// once, so the epilogue applies the two factors 1/2 of the tanh form of the gate itself.
//
// Persistent kernel, one CTA per SM, 608 threads, 128-position tiles:
//   warp 0        TMA producer of the z tiles (four 64-channel sub-tiles each) into a 2-stage ring
//   warp 1        UMMA issuer
//   warps 2..9    LayerNorm: two groups of four warps on alternate tiles, one thread per position,
//                 in place in the swizzled tile; a masked position becomes a zero row
//   warps 10..13  epilogue of the units with channel half 0, warps 14..17 of those with half 1
//   warp 18       TMA producer of the weight slots
//
// A tile is 128 consecutive positions along the index that becomes the contraction's k, exactly as
// in tm1_sm100.cuh (outgoing: z row f, columns t0..; incoming: z column f, rows t0.. through a
// strided TMA box).
#pragma once

#include "tm1_common.cuh"

namespace trimul {

constexpr int kW1C = 256;
constexpr int kW1Sub = kW1C / 64;                   // 64-channel sub-tiles per z tile
constexpr int kW1Threads = 608;
constexpr int kW1LnThreads = 256;                   // warps 2..9
constexpr int kW1XBytes = kW1Sub * kT1SubTile;      // one z tile: 64 KB
constexpr int kW1XStages = 2;
constexpr int kW1WSlots = 4;                        // weight ring: [128 rows][64 k] = 16 KB per slot
constexpr int kW1OffW = kW1XStages * kW1XBytes;
constexpr int kW1OffStaging = kW1OffW + kW1WSlots * kT1SubTile;     // one [128 channels][64 positions] box per epilogue group
constexpr int kW1OffAffine = kW1OffStaging + 2 * kT1SubTile;        // gamma[256], beta[256] fp32
constexpr int kW1OffBars = kW1OffAffine + 2 * kW1C * 4;
constexpr int kW1SmemBytes = kW1OffBars + 256;
constexpr int kW1LnBarrier = 2;        // 2, 3: the two LayerNorm groups
constexpr int kW1EpiBarrier = 4;       // 4, 5: the two epilogue groups
constexpr int kW1AffineBarrier = 6;
static_assert(kW1SmemBytes <= 232448, "wide stage 1 shared memory exceeds the 227 KB a CTA may use");

__global__ void __launch_bounds__(kW1Threads, 1)
tm1_wide_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWl,
                      const __grid_constant__ CUtensorMap tmWlg, const __grid_constant__ CUtensorMap tmWr,
                      const __grid_constant__ CUtensorMap tmWrg, const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const __grid_constant__ Tm1Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm1, 900);
        return;
    }
    uint8_t* sX = smem;
    uint8_t* sW = smem + kW1OffW;
    uint8_t* sOut = smem + kW1OffStaging;
    float* sGamma = reinterpret_cast<float*>(smem + kW1OffAffine);
    float* sBeta = sGamma + kW1C;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kW1OffBars);
    uint64_t* x_full = bars;                  // [2] z tile landed
    uint64_t* xn_ready = bars + 2;            // [2] tile normalised (128 arrivals)
    uint64_t* x_empty = bars + 4;             // [2] every UMMA that reads the tile has retired
    uint64_t* w_full = bars + 6;              // [slots] weight slot landed
    uint64_t* w_empty = w_full + kW1WSlots;   // [slots] the UMMAs that read the slot retired
    uint64_t* acc_full = w_empty + kW1WSlots; // [2] unit's accumulators complete
    uint64_t* acc_empty = acc_full + 2;       // [2] unit's accumulators drained (4 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    static_assert((10 + 2 * kW1WSlots) * 8 + 8 <= 256, "barrier block too small");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&xn_ready[s], kW1LnThreads / 2);
            mbar_init(&x_empty[s], 1);
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        for (int s = 0; s < kW1WSlots; ++s) {
            mbar_init(&w_full[s], 1);
            mbar_init(&w_empty[s], 1);
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
        // the LayerNorm warps bring gamma and beta into shared memory for themselves
        sGamma[threadIdx.x - 64] = p.gamma[threadIdx.x - 64];
        sBeta[threadIdx.x - 64] = p.beta[threadIdx.x - 64];
        named_barrier_sync(kW1AffineBarrier, kW1LnThreads);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ z tile producer
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1u;
                if (!mbar_wait<true>(&x_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm1, 100 + s)) break;
                const int t0 = (tile % p.tiles_per_fixed) * kT1P;
                const int bf = tile / p.tiles_per_fixed;
                const int f = bf % p.n_fixed;
                const int b = bf / p.n_fixed;
                mbar_arrive_expect_tx(&x_full[s], kW1XBytes);
                uint8_t* dst = sX + s * kW1XBytes;
                const int col = p.incoming ? f : t0;
                const int row = p.incoming ? t0 : f;
                for (int ks = 0; ks < kW1Sub; ++ks)
                    tma_load_4d(dst + ks * kT1SubTile, &tmZ, &x_full[s], ks * 64, col, row, b);
            }
        }
        __syncwarp();
    } else if (warp == 18) {
        // ------------------------------------------------------------------ weight slot producer
        // per tile and unit u = (side, channel half): for every K slice the proj slot, then the gate slot
        if (lane == 0) {
            const CUtensorMap* wm[4] = {&tmWl, &tmWlg, &tmWr, &tmWrg};
            uint32_t cnt = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
                for (int u = 0; ok && u < 4; ++u) {
                    const int side = u >> 1, chalf = u & 1;
                    for (int ks = 0; ks < kW1Sub; ++ks) {
                        for (int m = 0; m < 2; ++m, ++cnt) {
                            const int s = cnt % kW1WSlots;
                            const uint32_t ph = (cnt / kW1WSlots) & 1u;
                            if (!mbar_wait<true>(&w_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm1, 500 + s)) {
                                ok = false;
                                break;
                            }
                            mbar_arrive_expect_tx(&w_full[s], kT1SubTile);
                            tma_load_2d(sW + s * kT1SubTile, wm[side * 2 + m], &w_full[s], ks * 64, chalf * 128);
                        }
                        if (!ok) break;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(128, kT1P);
            uint32_t it = 0, cnt = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1u;
                if (!mbar_wait<true>(&xn_ready[s], ph, abort_flag, p.status, kStageIdTm1, 210 + s)) break;
                tcgen05_fence_after();
                TRIMUL_STAMP(1, it, 0);
                const uint32_t xs = smem_u32(sX + s * kW1XBytes);
                for (int u = 0; ok && u < 4; ++u) {
                    // accumulator pair u & 1; its use counter is 2 * it + (u >> 1)
                    const int acc = u & 1;
                    if (!mbar_wait<true>(&acc_empty[acc], ((uint32_t)(u >> 1) & 1u) ^ 1u, abort_flag, p.status,
                                         kStageIdTm1, 220 + acc)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    TRIMUL_STAMP(3, it, u);
                    const uint32_t d_p = tmem_base + acc * 256;
                    const uint32_t d_g = d_p + 128;
                    for (int ks = 0; ks < kW1Sub; ++ks, cnt += 2) {
                        const int sp = cnt % kW1WSlots, sg = (cnt + 1) % kW1WSlots;
                        if (!mbar_wait<true>(&w_full[sp], (cnt / kW1WSlots) & 1u, abort_flag, p.status, kStageIdTm1,
                                             230 + sp) ||
                            !mbar_wait<true>(&w_full[sg], ((cnt + 1) / kW1WSlots) & 1u, abort_flag, p.status,
                                             kStageIdTm1, 230 + sg)) {
                            ok = false;
                            break;
                        }
                        tcgen05_fence_after();
                        const uint32_t wp = smem_u32(sW + sp * kT1SubTile);
                        const uint32_t wg = smem_u32(sW + sg * kT1SubTile);
                        const uint32_t xk = xs + ks * kT1SubTile;
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint64_t kofs = kk * kDescKStep;
                            const uint64_t db = umma_smem_desc_sw128(xk) + kofs;
                            umma_bf16_ss(d_p, umma_smem_desc_sw128(wp) + kofs, db, idesc, (ks | kk) != 0);
                            umma_bf16_ss(d_g, umma_smem_desc_sw128(wg) + kofs, db, idesc, (ks | kk) != 0);
                        }
                        umma_commit(&w_empty[sp]);
                        umma_commit(&w_empty[sg]);
                    }
                    if (!ok) break;
                    umma_commit(&acc_full[acc]);
                    if (u != 2) TRIMUL_STAMP(1, it, u == 3 ? 3 : u + 1);
                }
                if (!ok) break;
                umma_commit(&x_empty[s]);   // every UMMA that reads the tile has retired when this fires
            }
        }
        __syncwarp();
    } else if (warp < 10) {
        // ------------------------------------------------------------------ LayerNorm (+ mask)
        const int g = (warp - 2) >> 2;
        const int pos = threadIdx.x - 64 - g * 128;    // 0..127, row of the tile
        uint32_t it = g;
        for (int tile = blockIdx.x + g * gridDim.x; tile < p.total_tiles; tile += 2 * gridDim.x, it += 2) {
            const uint32_t ph = (it >> 1) & 1u;
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
            if (!group_wait<true>(&x_full[g], ph, pos == 0, kW1LnBarrier + g, 128, abort_flag, p.status, kStageIdTm1,
                                  300 + g))
                break;
            if (pos == 0) TRIMUL_STAMP(2, it, 0);
            ln_row_inplace<kW1Sub>(sX + g * kW1XBytes, kT1SubTile, pos, sGamma, sBeta, p.eps, !keep);
            fence_proxy_async_smem();   // normalised tile -> visible to the UMMA (async proxy)
            mbar_arrive(&xn_ready[g]);
            if (pos == 0) TRIMUL_STAMP(2, it, 1);
        }
    } else {
        // ------------------------------------------------------------------ epilogue, one channel half per group
        const int grp = (warp - 10) >> 2;             // == channel half == accumulator pair
        const int q = warp & 3;
        const int ch = q * 32 + lane;                 // output channel inside the half == TMEM lane
        const bool leader = ((warp - 10) & 3) == 0 && lane == 0;
        const int bar_id = kW1EpiBarrier + grp;
        uint8_t* stg = sOut + grp * kT1SubTile;
        const uint32_t t_p = tmem_base + grp * 256 + ((uint32_t)(q * 32) << 16);
        uint32_t use = 0;
        bool alive = true;
        for (int tile = blockIdx.x; alive && tile < p.total_tiles; tile += gridDim.x) {
            const int t0 = (tile % p.tiles_per_fixed) * kT1P;
            const int bf = tile / p.tiles_per_fixed;
            const int f = bf % p.n_fixed;
            const int b = bf / p.n_fixed;
#pragma unroll 1
            for (int side = 0; side < 2; ++side, ++use) {
                const CUtensorMap* om = side == 0 ? &tmA : &tmB;
                const int rc = side == 0 ? p.a_row_chunk : p.b_row_chunk;
                const int cc = side == 0 ? p.a_col_chunk : p.b_col_chunk;
                if (!group_wait<true>(&acc_full[grp], use & 1u, leader, bar_id, 128, abort_flag, p.status, kStageIdTm1,
                                      400 + grp)) {
                    alive = false;
                    break;
                }
                tcgen05_fence_after();
                auto emit16 = [&](int c16, const uint32_t (&rp)[16], const uint32_t (&rg)[16]) {
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        uint32_t o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int i0 = k * 8 + 2 * e;
                            o[e] = gate2_full_bf16(__uint_as_float(rp[i0]), __uint_as_float(rg[i0]),
                                                   __uint_as_float(rp[i0 + 1]), __uint_as_float(rg[i0 + 1]));
                        }
                        const int chunk = ((c16 & 3) * 2 + k) ^ (ch & 7);
                        *reinterpret_cast<uint4*>(stg + ch * 128 + (chunk << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                };
                uint32_t rpA[16], rgA[16], rpB[16], rgB[16];
                tmem_ld_32x16(t_p, rpA);
                tmem_ld_32x16(t_p + 128, rgA);
#pragma unroll 1
                for (int half = 0; half < 2; ++half) {
                    if (leader) tma_store_wait_read<0>();      // the previous store has read the staging box
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
                            // every TMEM read of this unit's accumulators has completed: hand them back early
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
                            tma_store_4d(om, stg, col0 % cc, f % rc, b * kW1C + grp * 128, col0 / cc + f / rc);
                            tma_store_commit();
                        }
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
