// Stage 1 of the block on the tensor cores, c = 128: LayerNorm_in, pair mask and the two
// sigmoid-gated projections in ONE pass over z (reference.py:66-75), writing the operands a and b
// as channel-major planes for the contraction.
//
// The projections are computed transposed, D^T[channel][position] = W[channel][:] . x_n[position][:],
// so the weights are the UMMA A operand in their native nn.Linear [out,in] layout, the normalised
// activations are the B operand in their native row-major layout, and a TMEM lane is an output
// channel: each epilogue thread owns one channel and a run of consecutive positions, which is
// exactly a row of the channel-major destination (16-byte shared-memory stores into a swizzled
// staging box, then one TMA store per box).
//
// Persistent kernel, one CTA per SM, 576 threads, 128-position tiles:
//   warp 0        TMA producer: the four weight matrices once, then z tiles into a 2-stage ring
//   warp 1        UMMA issuer: per tile, left pair (proj, gate) then right pair, 128x128x16 each,
//                 into four 128-column TMEM accumulators
//   warps 2..9    LayerNorm: two groups of four warps on alternate tiles, eight lanes per position,
//                 normalise the 128 channels in place inside the swizzled tile (the TMA SWIZZLE_128B
//                 image is the UMMA K-major layout) and round to bf16; a masked position is written
//                 as a zero row, which makes both projections of that position exactly zero, so the
//                 epilogue needs no mask
//   warps 10..13  epilogue of the left side, warps 14..17 of the right side:
//                 TMEM -> p * sigmoid(g) -> bf16 -> swizzled staging -> TMA store
// All worker warps first halve the weight matrices in shared memory (exact in bf16), so the
// accumulators hold p/2 and g/2 and p*sigmoid(g) = (p/2)*tanh(g/2) + p/2 is one MUFU + one FMA.
//
// What bounds the stage (measured on a B200, csrc/microbench_sm100.cu): a tcgen05.mma of this shape
// is bound by its operand fetch from shared memory (about 75 bytes per cycle: 107 cycles instead of
// the ideal 64, 1.7 us of UMMAs per tile) and the z ring is only two tiles deep beside 128 KB of
// weights, so the tile period is half the life of a ring slot — load (2.0 us under load), LayerNorm
// (2.3 us), the UMMAs of both sides (2.0 us including their waits for the accumulators): 3.1 us
// against 2.2 us for the HBM traffic of a tile.  Neither tensor memory reads (130-320 bytes per
// cycle and SM) nor the hardware tanh (16 per cycle and SM, 1.0 us per tile) are the limit.
// tm1_direct_sm100.cuh is the variant that halves the number of UMMAs (N = 256) and has a
// three-deep ring at the price of a thread-per-position epilogue; it is slower.
//
// A tile is 128 consecutive positions along the index that becomes the contraction's k: for the
// outgoing direction z row f, columns t0..t0+127; for the incoming direction z column f, rows
// t0..t0+127 (a strided TMA box), so both directions store plane element (f, t0+p).
#pragma once

#include "tm1_common.cuh"

namespace trimul {

constexpr int kT1Threads = 576;
constexpr int kT1LnThreads = 256;      // warps 2..9
constexpr int kT1EpiThreads = 128;     // per side
constexpr int kT1WBytes = 8 * kT1SubTile;         // 4 matrices x 2 K halves
constexpr int kT1XStages = 2;
constexpr int kT1StagingBytes = 2 * kT1SubTile;   // one [128 channels][64 positions] store box per side
constexpr int kT1OffX = kT1WBytes;
constexpr int kT1OffStaging = kT1OffX + kT1XStages * kT1XBytes;
constexpr int kT1OffBars = kT1OffStaging + kT1StagingBytes;
constexpr int kT1SmemBytes = kT1OffBars + 192;
constexpr int kT1LnBarrier = 2;
constexpr int kT1EpiBarrier = 3;       // 3: left side, 4: right side
constexpr int kT1LnBarrier2 = 5;       // second LayerNorm group

__global__ void __launch_bounds__(kT1Threads, 1)
tm1_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWl,
                 const __grid_constant__ CUtensorMap tmWlg, const __grid_constant__ CUtensorMap tmWr,
                 const __grid_constant__ CUtensorMap tmWrg, const __grid_constant__ CUtensorMap tmA,
                 const __grid_constant__ CUtensorMap tmB, const Tm1Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm1, 900);
        return;
    }
    uint8_t* sW = smem;
    uint8_t* sX = smem + kT1OffX;
    uint8_t* sOut = smem + kT1OffStaging;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kT1OffBars);
    uint64_t* w_full = bars;            // weights landed
    uint64_t* x_full = bars + 1;        // [2] z tile landed
    uint64_t* xn_ready = bars + 3;      // [2] tile normalised (256 arrivals)
    uint64_t* x_empty = bars + 5;       // [2] UMMAs that read the tile retired
    uint64_t* acc_full = bars + 7;      // [2] side's accumulators complete
    uint64_t* acc_empty = bars + 9;     // [2] side's accumulators drained (4 arrivals)
    uint64_t* w_ready = bars + 11;      // weights halved (512 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        mbar_init(w_ready, kT1LnThreads + 2 * kT1EpiThreads);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&xn_ready[s], kT1LnThreads / 2);
            mbar_init(&x_empty[s], 1);
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

    if (warp >= 2) {
        // every worker thread: halve its share of the weights once they have landed
        if (mbar_wait(w_full, 0, abort_flag, p.status, kStageIdTm1, 150)) {
            halve_bf16_smem(sW, kT1WBytes, threadIdx.x - 64, kT1LnThreads + 2 * kT1EpiThreads);
            fence_proxy_async_smem();
        }
        mbar_arrive(w_ready);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, kT1WBytes);
            const CUtensorMap* wm[4] = {&tmWl, &tmWlg, &tmWr, &tmWrg};
            for (int m = 0; m < 4; ++m)
                for (int kh = 0; kh < 2; ++kh)
                    tma_load_2d(sW + (m * 2 + kh) * kT1SubTile, wm[m], w_full, kh * 64, 0);
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1u;
                if (!mbar_wait(&x_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm1, 100 + s)) break;
                int b, f, t0;
                tm1_decode_tile(p, tile, b, f, t0);
                mbar_arrive_expect_tx(&x_full[s], kT1XBytes);
                uint8_t* dst = sX + s * kT1XBytes;
                // z viewed as (channel, column, row, batch); outgoing box = 128 columns of row f,
                // incoming box = 128 rows of column f
                const int col = p.incoming ? f : t0;
                const int row = p.incoming ? t0 : f;
                tma_load_4d(dst, &tmZ, &x_full[s], 0, col, row, b);
                tma_load_4d(dst + kT1SubTile, &tmZ, &x_full[s], 64, col, row, b);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(128, kT1P);
            bool ok = mbar_wait(w_ready, 0, abort_flag, p.status, kStageIdTm1, 200);
            tcgen05_fence_after();
            uint32_t it = 0;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1u;
                if (!mbar_wait(&xn_ready[s], ph, abort_flag, p.status, kStageIdTm1, 210 + s)) break;
                tcgen05_fence_after();
                const uint32_t xs = smem_u32(sX + s * kT1XBytes);
                for (int side = 0; side < 2; ++side) {
                    if (!mbar_wait(&acc_empty[side], (it & 1u) ^ 1u, abort_flag, p.status, kStageIdTm1,
                                   220 + side)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t d_p = tmem_base + side * 256;
                    const uint32_t d_g = d_p + 128;
                    const uint32_t wp = smem_u32(sW + (side * 4) * kT1SubTile);       // proj: 2 K halves
                    const uint32_t wg = smem_u32(sW + (side * 4 + 2) * kT1SubTile);   // gate: 2 K halves
#pragma unroll
                    for (int kk = 0; kk < kT1C / 16; ++kk) {
                        const uint32_t sub = (kk >> 2) * kT1SubTile;
                        const uint64_t kofs = (kk & 3) * kDescKStep;
                        const uint64_t db = umma_smem_desc_sw128(xs + sub) + kofs;
                        umma_bf16_ss(d_p, umma_smem_desc_sw128(wp + sub) + kofs, db, idesc, kk != 0);
                        umma_bf16_ss(d_g, umma_smem_desc_sw128(wg + sub) + kofs, db, idesc, kk != 0);
                    }
                    umma_commit(&acc_full[side]);
                }
                if (!ok) break;
                umma_commit(&x_empty[s]);   // both sides' UMMAs have read the tile when this fires
            }
        }
        __syncwarp();
    } else if (warp < 10) {
        // ------------------------------------------------------------------ LayerNorm (+ mask)
        // two groups of four warps; group g takes the tiles with (local tile index & 1) == g, which
        // are the ones in stage g; warp lw of a group owns rows [32 lw, 32 lw + 32): lane l row
        // 32 lw + 4 i + (l >> 3) in iteration i, 16-byte chunk l & 7 of both 64-channel sub-tiles
        // (the same summation order as the CTA-pair kernel, so the two give identical results)
        const int g = (warp - 2) >> 2;
        const int lw = (warp - 2) & 3;
        const int rr = lane >> 3;
        const int bar_id = g == 0 ? kT1LnBarrier : kT1LnBarrier2;
        f32x2 gb[16];
        ln_load_affine<2>(gb, p.gamma, p.beta, lane);
        uint32_t it = g;
        for (int tile = blockIdx.x + g * gridDim.x; tile < p.total_tiles; tile += 2 * gridDim.x, it += 2) {
            const uint32_t ph = (it >> 1) & 1u;
            // pair-mask bits of this lane's eight rows (independent of the tile data: do it first).  Lane l
            // looks up position 32 lw + l of the tile — one or two byte loads — and a ballot hands every
            // lane the bits of its own rows.
            bool keep = true;
            if (p.mask_kind != 0) {
                int b, f, t0;
                tm1_decode_tile(p, tile, b, f, t0);
                keep = tm1_keep(p, b, f, t0 + 32 * lw + lane);
            }
            if (!group_wait(&x_full[g], ph, lw == 0 && lane == 0, bar_id, 128, abort_flag, p.status, kStageIdTm1, 300 + g))
                break;
            uint32_t zero_bits = 0u;
            if (p.mask_kind != 0) {
                const uint32_t drop = ~__ballot_sync(0xffffffffu, keep);
#pragma unroll
                for (int i = 0; i < 8; ++i) zero_bits |= ((drop >> (4 * i + rr)) & 1u) << i;
            }
            ln_rows_warp<8>(sX + g * kT1XBytes, kT1SubTile, 32 * lw, lane, gb, p.eps, zero_bits);
            fence_proxy_async_smem();   // normalised tile -> visible to the UMMA (async proxy)
            mbar_arrive(&xn_ready[g]);
        }
    } else {
        // ------------------------------------------------------------------ epilogue, one side per group
        const int side = (warp - 10) >> 2;
        const int q = warp & 3;
        const int ch = q * 32 + lane;                 // output channel == TMEM lane
        const bool leader = ((warp - 10) & 3) == 0 && lane == 0;
        const int bar_id = kT1EpiBarrier + side;
        uint8_t* stg = sOut + side * kT1SubTile;
        const CUtensorMap* om = side == 0 ? &tmA : &tmB;
        const int rc = side == 0 ? p.a_row_chunk : p.b_row_chunk;
        const int cc = side == 0 ? p.a_col_chunk : p.b_col_chunk;
        const uint32_t t_p = tmem_base + side * 256 + ((uint32_t)(q * 32) << 16);
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            int b, f, t0;
            tm1_decode_tile(p, tile, b, f, t0);
            if (!group_wait(&acc_full[side], it & 1u, leader, bar_id, kT1EpiThreads, abort_flag, p.status,
                            kStageIdTm1, 400 + side))
                break;
            tcgen05_fence_after();
            // 16 positions at a time; the TMEM loads of the next 16 are in flight while the current
            // 16 are gated, rounded and written to the staging box (64 positions per TMA store)
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
                named_barrier_sync(bar_id, kT1EpiThreads);
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
                        // every TMEM read of this side's accumulators has completed: hand them back early
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[side]);
                    }
                    emit16(c16 + 1, rpB, rgB);
                }
                fence_proxy_async_smem();
                named_barrier_sync(bar_id, kT1EpiThreads);
                if (leader) {
                    const int col0 = t0 + half * 64;
                    if (col0 < p.n_run) {
                        tma_store_4d(om, stg, col0 % cc, f % rc, b * kT1C, col0 / cc + f / rc);
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
