// Stage 3 of the block with BOTH LayerNorms folded into the projections, c = 128
// (reference.py:76-83): out = sigmoid(Wg . LN_in(z)) * (Wo . LN_out(tri)) [+ z].
//
//   W . LN(x) = rstd * (W*gamma) . x  +  t * rowsum(W*gamma)  +  W . beta,      t = -mean * rstd
//
// The tensor cores multiply the RAW z tile and the RAW tri tile by weights that carry gamma (and
// the factor 1/2 of the tanh form of the gate); mean and rstd of every position enter in the
// epilogue as one FMA per value.  Nothing is normalised in place any more, so
//   * the UMMAs start the moment a tile lands, the statistics are computed beside them,
//   * each tile is read once by the statistics warps instead of read, re-read and rewritten,
//   * the z tile is still intact when the epilogue runs: the result is written IN PLACE over it
//     (the swizzled [128 positions][128 channels] image of the z tile is exactly the layout of the
//     TMA store box) and the residual `+ z` is read from the same bytes.  No staging buffer.
// The result differs from the reference's bf16 path only by where the rounding to bf16 happens
// (W*gamma instead of LN(x)); against an fp32 evaluation it is closer than the reference's own
// bf16 path.
//
// A z buffer lives long (load, statistics, epilogue, store), a tri buffer only until its UMMAs
// and statistics are done, so the z ring is three deep and the tri ring two.  The statistics of a
// tile travel to the epilogue through the first 2 KB of the tile's own tri buffer, which is dead
// by then; that leaves shared memory for the third z buffer.
//
// Persistent kernel, one CTA per SM, 640 threads, 128-position tiles (z row r, columns j0..j0+127):
//   warp 0        TMA producer: Wg, Wo once; per tile the z tile and the tri tile [128 channels]
//                 [128 positions] (channel-major, as the contraction wrote it)
//   warp 1        UMMA issuer: gate = z . Wg'^T (z K-major), proj = tri . Wo'^T (tri MN-major, used as
//                 it lies), 128x128x16 each, into a double-buffered pair of TMEM accumulators
//   warp 2        store warp: TMA-stores each 64-channel half of a finished tile and hands the z
//                 buffer back to the producer once the store has read it
//   warp 3        idle
//   warps 4..11   epilogue, thread = position; warps 4..7 own channels 0..63, warps 8..11 channels
//                 64..127: TMEM -> statistics -> gate -> (+ z) -> bf16 -> in place -> store warp
//   warps 12..15  statistics of the z tile, one thread per position
//   warps 16..19  statistics of the tri tile: a thread owns 8 positions of 16 channel rows, the 8
//                 lanes that share the positions combine by a halving butterfly, so each lane ends
//                 up with the sums of ONE position
// Before the first tile the epilogue threads fold gamma and 1/2 into Wg and Wo in shared memory
// and leave per-channel (rowsum, bias) pairs for the epilogue.
//
// kDropScale: the row-broadcast dropout scale of the reference module in training mode multiplies
// the block output before the residual (a template parameter: the inference instantiations carry
// no trace of it).
//
// kKH = 2 is the last stage of the BIDIRECTIONAL block (bidirectional.py:150-156): tri has 256
// channel planes per batch ([outgoing | incoming]), LayerNorm_out runs over all 256 and Wo is
// [128, 256].  The tri tile then arrives as two 128-channel halves, each in one slot of the tri
// ring (so a tile occupies the whole ring and the z ring is two deep: Wo takes 32 KB more); the
// projection accumulates over both halves and the tri statistics are summed over both.
#pragma once

#include "tm2_sm100.cuh"

namespace trimul {

constexpr int kG2Threads = 640;
constexpr int kG2EpiThreads = 256;      // warps 4..11, two groups of 128
constexpr int kG2StatThreads = 128;     // each of the two statistics groups
template <int kKH>
struct G2Layout {
    static constexpr int kWBytes = (2 + 2 * kKH) * kT2SubTile;   // Wg: 2 K sub-tiles, Wo: 2 per 128 hidden channels
    static constexpr int kZStages = kKH == 1 ? 3 : 2;
    static constexpr int kOffZ = kWBytes;                        // z ring, 32 KB per stage
    static constexpr int kOffT = kOffZ + kZStages * kT2XBytes;   // 2 x 32 KB tri ring; once a tile's tri data is dead the
                                                                 // first 2 KB of its last slot hold [128 positions]
                                                                 // (r_in, t_in, r_out, t_out)
    static constexpr int kOffConst = kOffT + 2 * kT2TBytes;      // [2 matrices][64 channel pairs] (s0, s1, b0, b1)
    static constexpr int kOffBars = kOffConst + 2048;
    static constexpr int kSmemBytes = kOffBars + 256;
};
constexpr int kG2StatInBarrier = 2;
constexpr int kG2StatOutBarrier = 3;
constexpr int kG2EpiBarrier = 4;        // 4: channels 0..63, 5: channels 64..127

struct Tm2FoldParams {
    Tm2Params base;
    int residual_is_z;    // add the z tile to the result (the block's `pair + update` form)
    const __nv_bfloat16* drop_scale;   // [B, 1, N, 128] row-broadcast multiplier of the block output
                                       // (module.py:332-337), applied before the residual; or null
};

template <bool kResidualIsZ, int kKH, bool kDropScale>
__global__ void __launch_bounds__(kG2Threads, 1)
tm2_fold_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWg,
                      const __grid_constant__ CUtensorMap tmWo, const __grid_constant__ CUtensorMap tmOut,
                      const __grid_constant__ CUtensorMap tmTri, const Tm2FoldParams fp) {
    const Tm2Params& p = fp.base;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm2, 900);
        return;
    }
    using L = G2Layout<kKH>;
    constexpr int kG2ZStages = L::kZStages;
    uint8_t* sW = smem;
    uint8_t* sZ = smem + L::kOffZ;
    uint8_t* sT = smem + L::kOffT;
    float4* sConst = reinterpret_cast<float4*>(smem + L::kOffConst);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBars);
    uint64_t* w_full = bars;            // weights landed
    uint64_t* w_ready = bars + 1;       // weights folded (256 arrivals)
    uint64_t* z_full = bars + 2;        // [3] z tile landed
    uint64_t* z_empty = bars + 5;       // [3] the store of the tile written over the z tile has read it (1 arrival)
    uint64_t* box_ready = bars + 8;     // [3 stages][2 halves] result half written (4 arrivals)
    uint64_t* t_full = bars + 14;       // [2] tri slot landed (a slot = 128 channel planes of a tile)
    uint64_t* tri_dead = bars + 16;     // [2] the slot's UMMAs retired + its 128 statistics threads done reading
    uint64_t* t_empty = bars + 18;      // [2] the epilogue has taken the statistics out of the slot (8 arrivals)
    uint64_t* acc_full = bars + 20;     // [2]
    uint64_t* acc_empty = bars + 22;    // [2] (8 arrivals)
    uint64_t* stat_in = bars + 24;      // [2] z statistics written into the tri buffer (128 arrivals)
    uint64_t* stat_out = bars + 26;     // [2] tri statistics written (128 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 28);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        mbar_init(w_ready, kG2EpiThreads);
        for (int s = 0; s < kG2ZStages; ++s) {
            mbar_init(&z_full[s], 1);
            mbar_init(&z_empty[s], 1);
            mbar_init(&box_ready[2 * s], 4);
            mbar_init(&box_ready[2 * s + 1], 4);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&t_full[s], 1);
            mbar_init(&tri_dead[s], 1 + kG2StatThreads);
            mbar_init(&t_empty[s], 8);
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 8);
            mbar_init(&stat_in[s], kG2StatThreads);
            mbar_init(&stat_out[s], kG2StatThreads);
        }
        *abort_flag = 0;
        fence_mbarrier_init();
        tma_prefetch_desc(&tmZ);
        tma_prefetch_desc(&tmOut);
        tma_prefetch_desc(&tmTri);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up done without touching global memory: now wait for the producer of tri (and of z)
    griddep_wait();
    griddep_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, L::kWBytes);
            for (int kh = 0; kh < 2; ++kh) tma_load_2d(sW + kh * kT2SubTile, &tmWg, w_full, kh * 64, 0);
            for (int kh = 0; kh < 2 * kKH; ++kh) tma_load_2d(sW + (2 + kh) * kT2SubTile, &tmWo, w_full, kh * 64, 0);
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int zs = it % kG2ZStages;
                const uint32_t zph = (it / kG2ZStages) & 1u;
                const int j0 = (tile % p.tiles_per_row) * kT2P;
                const int br = tile / p.tiles_per_row;
                const int r = br % p.rows;
                const int b = br / p.rows;
                bool okp = true;
                for (int h = 0; h < kKH; ++h) {
                    // tri slot of this 128-channel half: slots are used round-robin, use n = u >> 1
                    const uint32_t u = it * kKH + h;
                    const int ts = u & 1;
                    const uint32_t tph = (u >> 1) & 1u;
                    // a tile's LAST slot carries the statistics and is released by the epilogue; any
                    // other slot is free as soon as its readers are done (so the next tile's first half
                    // streams in while this tile's last half is still being worked on)
                    uint64_t* freed = h == kKH - 1 ? &t_empty[ts] : &tri_dead[ts];
                    if (!mbar_wait<true>(freed, tph ^ 1u, abort_flag, p.status, kStageIdTm2, 100 + ts)) {
                        okp = false;
                        break;
                    }
                    // tri planes viewed as (column, row, plane, chunk): 64 columns x 128 planes per box
                    mbar_arrive_expect_tx(&t_full[ts], kT2TBytes);
                    uint8_t* dt = sT + ts * kT2TBytes;
                    tma_load_4d(dt, &tmTri, &t_full[ts], j0, r, (b * kKH + h) * kT2C, 0);
                    tma_load_4d(dt + kT2SubTile, &tmTri, &t_full[ts], j0 + 64, r, (b * kKH + h) * kT2C, 0);
                }
                if (!okp) break;
                if (!mbar_wait<true>(&z_empty[zs], zph ^ 1u, abort_flag, p.status, kStageIdTm2, 110 + zs)) break;
                TRIMUL_STAMP(0, it, 0);
                mbar_arrive_expect_tx(&z_full[zs], kT2XBytes);
                uint8_t* dz = sZ + zs * kT2XBytes;
                tma_load_4d(dz, &tmZ, &z_full[zs], 0, j0, r, b);
                tma_load_4d(dz + kT2SubTile, &tmZ, &z_full[zs], 64, j0, r, b);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(kT2P, kT2C);
            constexpr uint32_t idesc_mn = umma_idesc_bf16(kT2P, kT2C, 1, 0);   // A (tri) is MN-major
            bool ok = mbar_wait<true>(w_ready, 0, abort_flag, p.status, kStageIdTm2, 200);
            tcgen05_fence_after();
            uint32_t it = 0;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1u;
                // accumulator pair `s` was last used by tile it-2
                if (!mbar_wait<true>(&acc_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm2, 210 + s)) break;
                const uint32_t wg = smem_u32(sW);
                const uint32_t wo = wg + 2 * kT2SubTile;
                const uint32_t d_g = tmem_base + s * 256;
                const uint32_t d_p = d_g + 128;
                for (int h = 0; ok && h < kKH; ++h) {
                    const uint32_t u = it * kKH + h;
                    const int tsl = u & 1;
                    if (!mbar_wait<true>(&t_full[tsl], (u >> 1) & 1u, abort_flag, p.status, kStageIdTm2, 230 + tsl)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    TRIMUL_STAMP(1, it, 0);
                    const uint32_t ts = smem_u32(sT + tsl * kT2TBytes);
                    const uint32_t woh = wo + h * 2 * kT2SubTile;       // Wo columns of this half
#pragma unroll 2
                    for (int kk = 0; kk < kT2C / 16; ++kk) {
                        // tri slot: rows are channels (K), 128 bytes = 64 positions per row, the second
                        // 64 positions one sub-tile further; a K step of 16 is two 8-row groups = 2048 B
                        umma_bf16_ss(d_p, umma_smem_desc_mn_sw128(ts + kk * 2048, kT2SubTile, 1024),
                                     umma_smem_desc_sw128(woh + (kk >> 2) * kT2SubTile) + (kk & 3) * kDescKStep,
                                     idesc_mn, (kk | h) != 0);
                    }
                    umma_commit(&tri_dead[tsl]);
                }
                if (!ok) break;
                const int zs = it % kG2ZStages;
                if (!mbar_wait<true>(&z_full[zs], (it / kG2ZStages) & 1u, abort_flag, p.status, kStageIdTm2, 220 + zs)) break;
                tcgen05_fence_after();
                TRIMUL_STAMP(1, it, 1);
                const uint32_t xs = smem_u32(sZ + zs * kT2XBytes);
#pragma unroll 2
                for (int kk = 0; kk < kT2C / 16; ++kk) {
                    const uint32_t sub = (kk >> 2) * kT2SubTile;
                    const uint64_t kofs = (kk & 3) * kDescKStep;
                    umma_bf16_ss(d_g, umma_smem_desc_sw128(xs + sub) + kofs, umma_smem_desc_sw128(wg + sub) + kofs,
                                 idesc, kk != 0);
                }
                umma_commit(&acc_full[s]);
                TRIMUL_STAMP(1, it, 2);
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ------------------------------------------------------------------ store warp
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it % kG2ZStages;
                const uint32_t ph = (it / kG2ZStages) & 1u;
                const int j0 = (tile % p.tiles_per_row) * kT2P;
                const int br = tile / p.tiles_per_row;
                const int r = br % p.rows;
                const int b = br / p.rows;
                const uint8_t* src = sZ + s * kT2XBytes;
                if (!mbar_wait<true>(&box_ready[2 * s], ph, abort_flag, p.status, kStageIdTm2, 600 + s)) break;
                tma_store_4d(&tmOut, src, 0, j0, r, b);
                tma_store_commit();
                if (!mbar_wait<true>(&box_ready[2 * s + 1], ph, abort_flag, p.status, kStageIdTm2, 610 + s)) break;
                tma_store_4d(&tmOut, src + kT2SubTile, 64, j0, r, b);
                tma_store_commit();
                tma_store_wait_read<0>();
                TRIMUL_STAMP(2, it, 0);
                mbar_arrive(&z_empty[s]);        // the producer may refill the z buffer
            }
            tma_store_wait_all<0>();
        }
        __syncwarp();
    } else if (warp == 3) {
        // idle
    } else if (warp < 12) {
        // ------------------------------------------------------------------ epilogue
        const int e = threadIdx.x - 128;               // 0..255
        const int grp = e >> 7;                        // channel half: 0 -> channels 0..63, 1 -> 64..127
        const int q = warp & 3;
        const int row = q * 32 + lane;                 // position inside the tile == TMEM lane
        const bool leader = (e & 127) == 0;
        const int bar_id = kG2EpiBarrier + grp;
        // fold gamma and 1/2 into the weights: thread e takes matrix e >> 7 (0: Wg with LN_in,
        // 1: Wo with LN_out), output channel e & 127
        bool run = mbar_wait<true>(w_full, 0, abort_flag, p.status, kStageIdTm2, 150);
        if (run) {
            const int m = e >> 7, n = e & 127;
            float s_, b_;
            fold_row_smem(sW + m * 2 * kT2SubTile, kT2SubTile, n, m == 0 ? p.gamma_in : p.gamma_out,
                          m == 0 ? p.beta_in : p.beta_out, m == 0 ? 2 : 2 * kKH, s_, b_);
            float* c = reinterpret_cast<float*>(&sConst[m * 64 + (n >> 1)]);
            c[n & 1] = s_;
            c[2 + (n & 1)] = b_;
            fence_proxy_async_smem();      // folded weights -> visible to the UMMA (async proxy)
        }
        mbar_arrive(w_ready);
        // every channel's constants are needed by every epilogue thread
        run = run && mbar_wait<true>(w_ready, 0, abort_flag, p.status, kStageIdTm2, 160);
        // one verdict per group: a thread that gave up must not leave the others at the group's barrier
        run = named_barrier_all(bar_id, 128, run);

        const uint32_t lane_bits = (uint32_t)(q * 32) << 16;
        const ulonglong2* cG = reinterpret_cast<const ulonglong2*>(sConst) + grp * 32;
        const ulonglong2* cO = cG + 64;
        uint32_t it = 0;
        for (int tile = blockIdx.x; run && tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it & 1;
            const uint32_t ph = (it >> 1) & 1u;
            const int zs = it % kG2ZStages;
            bool ok = true;
            if (leader) {
                ok = mbar_wait<true>(&acc_full[s], ph, abort_flag, p.status, kStageIdTm2, 400 + s) &&
                     mbar_wait<true>(&stat_in[s], ph, abort_flag, p.status, kStageIdTm2, 410 + s) &&
                     mbar_wait<true>(&stat_out[s], ph, abort_flag, p.status, kStageIdTm2, 420 + s);
            }
            if (!named_barrier_all(bar_id, 128, ok)) break;
            tcgen05_fence_after();
            if (e == 0) TRIMUL_STAMP(4, it, 0);
            const int slot0 = (it * kKH + kKH - 1) & 1;     // the tile's last tri slot carries its statistics
            const float4 st = reinterpret_cast<const float4*>(sT + slot0 * kT2TBytes)[row];
            __syncwarp();
            if (lane == 0) mbar_arrive(&t_empty[slot0]);    // this warp has its statistics: the slot may be refilled
            const f32x2 rin = f2_pack(st.x, st.x), tin = f2_pack(st.y, st.y);
            const f32x2 rout = f2_pack(st.z, st.z), tout = f2_pack(st.w, st.w);
            const uint32_t t_g = tmem_base + s * 256 + grp * 64 + lane_bits;     // gate; proj 128 columns on
            uint8_t* tile_row = sZ + zs * kT2XBytes + grp * kT2SubTile + row * 128;
            // this position's 64 drop-scale values (it is column j0 + row of z row r, any r)
            const __nv_bfloat16* ds_row = nullptr;
            if (kDropScale) {
                const int j0 = (tile % p.tiles_per_row) * kT2P;
                const int b = (tile / p.tiles_per_row) / p.rows;
                if (j0 + row < p.N) ds_row = fp.drop_scale + ((size_t)b * p.N + j0 + row) * kT2C + grp * 64;
            }
            // 8 output channels (one 16-byte chunk) at a time; the TMEM loads of the next 8 are in
            // flight while the current 8 get their statistics, are gated, rounded and written over the
            // z tile.  The loop stays rolled to keep the code small.
            auto emit8 = [&](int c8, const uint32_t (&rg)[8], const uint32_t (&rp)[8]) {
                uint4* dst = reinterpret_cast<uint4*>(tile_row + ((c8 ^ (row & 7)) << 4));
                uint32_t res[4] = {0u, 0u, 0u, 0u};
                if (kResidualIsZ) {
                    const uint4 rv = *dst;
                    res[0] = rv.x; res[1] = rv.y; res[2] = rv.z; res[3] = rv.w;
                }
                uint32_t dsw[4] = {0u, 0u, 0u, 0u};
                if (kDropScale && ds_row != nullptr) {
                    const uint4 dv = __ldg(reinterpret_cast<const uint4*>(ds_row + c8 * 8));
                    dsw[0] = dv.x; dsw[1] = dv.y; dsw[2] = dv.z; dsw[3] = dv.w;
                }
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const ulonglong2 kg = cG[c8 * 4 + k], ko = cO[c8 * 4 + k];     // channel pair's constants
                    const f32x2 hg = f2_fma(f2_pack(__uint_as_float(rg[2 * k]), __uint_as_float(rg[2 * k + 1])), rin,
                                            f2_fma(tin, kg.x, kg.y));
                    const f32x2 ho = f2_fma(f2_pack(__uint_as_float(rp[2 * k]), __uint_as_float(rp[2 * k + 1])), rout,
                                            f2_fma(tout, ko.x, ko.y));
                    float g0, g1;
                    f2_unpack(hg, g0, g1);
                    o[k] = f2_to_bf16x2(f2_fma(ho, f2_pack(tanh_fast(g0), tanh_fast(g1)), ho));
                    if (kDropScale && ds_row != nullptr)   // the scale multiplies the rounded block output, like `out * scale`
                        o[k] = f2_to_bf16x2(f2_mul(f2_from_bf16x2(o[k]), f2_from_bf16x2(dsw[k])));
                    if (kResidualIsZ)   // the reference rounds the block output to bf16 before `out + pair`
                        o[k] = f2_to_bf16x2(f2_add(f2_from_bf16x2(o[k]), f2_from_bf16x2(res[k])));
                }
                *dst = make_uint4(o[0], o[1], o[2], o[3]);
            };
            uint32_t rgA[8], rpA[8], rgB[8], rpB[8];
            tmem_ld_32x8(t_g, rgA);
            tmem_ld_32x8(t_g + 128, rpA);
#pragma unroll 1
            for (int c8 = 0; c8 < 8; c8 += 2) {
                tmem_ld_wait();
                tmem_ld_32x8(t_g + (c8 + 1) * 8, rgB);
                tmem_ld_32x8(t_g + 128 + (c8 + 1) * 8, rpB);
                emit8(c8, rgA, rpA);
                tmem_ld_wait();
                if (c8 + 2 < 8) {
                    tmem_ld_32x8(t_g + (c8 + 2) * 8, rgA);
                    tmem_ld_32x8(t_g + 128 + (c8 + 2) * 8, rpA);
                } else {
                    // every TMEM read of this warp's share of the accumulators has completed
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[s]);
                }
                emit8(c8 + 1, rgB, rpB);
            }
            fence_proxy_async_smem();      // result half -> visible to the TMA store (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive(&box_ready[2 * zs + grp]);
            if (e == 0) TRIMUL_STAMP(4, it, 1);
        }
    } else if (warp < 16) {
        // ------------------------------------------------------------------ statistics of the z tile
        const int pos = threadIdx.x - 384;             // 0..127, row of the tile
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it & 1;
            const int zs = it % kG2ZStages;
            if (!group_wait<true>(&z_full[zs], (it / kG2ZStages) & 1u, pos == 0, kG2StatInBarrier, kG2StatThreads, abort_flag,
                            p.status, kStageIdTm2, 300 + zs))
                break;
            if (pos == 0) TRIMUL_STAMP(3, it, 0);
            float rstd, t;
            row_stats(sZ + zs * kT2XBytes, kT2SubTile, pos, p.eps_in, rstd, t);
            // the statistics go into the tile's last tri slot once nothing reads the tri data there any more
            const uint32_t u0 = it * kKH + kKH - 1;
            const int slot0 = u0 & 1;
            if (!group_wait<true>(&tri_dead[slot0], (u0 >> 1) & 1u, pos == 0, kG2StatInBarrier, kG2StatThreads,
                                  abort_flag, p.status, kStageIdTm2, 310 + slot0))
                break;
            *reinterpret_cast<float2*>(reinterpret_cast<float4*>(sT + slot0 * kT2TBytes) + pos) = make_float2(rstd, t);
            mbar_arrive(&stat_in[s]);
            if (pos == 0) TRIMUL_STAMP(3, it, 1);
        }
    } else {
        // ------------------------------------------------------------------ statistics of the tri tile
        // The tile is [128 channel rows][128 positions] as two 64-position sub-tiles, 16-byte chunk c
        // of row r stored at chunk c ^ (r & 7).  Thread (tw, ql, rs): position chunk cq = 4 tw + ql
        // (positions 8 cq .. 8 cq + 7), channel rows rs, rs + 8, ..., rs + 120; all its rows have
        // r & 7 == rs, so its 16 bytes sit at the same offset in every row.
        const int tid = threadIdx.x - 512;             // 0..127
        const int tw = tid >> 5;
        const int ql = lane >> 3;
        const int rs = lane & 7;
        const int cq = 4 * tw + ql;
        const uint32_t col_off = (uint32_t)(cq >> 3) * kT2SubTile + ((((uint32_t)cq & 7u) ^ (uint32_t)rs) << 4);
        const float inv_c = 1.0f / (float)(kT2C * kKH);
        uint32_t it = 0;
        bool alive = true;
        for (int tile = blockIdx.x; alive && tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it & 1;
            uint32_t sh[4] = {0u, 0u, 0u, 0u};
            f32x2 nsh[4] = {0ull, 0ull, 0ull, 0ull}, a[4] = {0ull, 0ull, 0ull, 0ull}, qq[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll 1
            for (int h = 0; h < kKH; ++h) {           // the tile's 128-channel halves, one tri slot each
                const uint32_t u = it * kKH + h;
                const int ts = u & 1;
                if (!group_wait<true>(&t_full[ts], (u >> 1) & 1u, tid == 0, kG2StatOutBarrier, kG2StatThreads, abort_flag,
                                      p.status, kStageIdTm2, 500 + ts)) {
                    alive = false;
                    break;
                }
                if (tid == 0) TRIMUL_STAMP(5, it, 0);
                const uint8_t* base = sT + ts * kT2TBytes + col_off + rs * 128;
                if (h == 0) {
                    // common shift of each position: its channel 0 (row 0, held by the rs == 0 lane)
                    const uint4 v0 = *reinterpret_cast<const uint4*>(base);
                    sh[0] = __shfl_sync(0xffffffffu, v0.x, lane & 24);
                    sh[1] = __shfl_sync(0xffffffffu, v0.y, lane & 24);
                    sh[2] = __shfl_sync(0xffffffffu, v0.z, lane & 24);
                    sh[3] = __shfl_sync(0xffffffffu, v0.w, lane & 24);
#pragma unroll
                    for (int w = 0; w < 4; ++w) nsh[w] = f2_pack(-bf16_lo(sh[w]), -bf16_hi(sh[w]));
                }
#pragma unroll 4
                for (int m = 0; m < 16; ++m) {
                    const uint4 v = *reinterpret_cast<const uint4*>(base + m * 1024);
                    const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const f32x2 d = f2_add(f2_from_bf16x2(w4[w]), nsh[w]);
                        a[w] = f2_add(a[w], d);
                        qq[w] = f2_fma(d, d, qq[w]);
                    }
                }
                mbar_arrive(&tri_dead[ts]);             // this thread is done with the slot's tri data
            }
            if (!alive) break;
            float s1[8], s2[8];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                f2_unpack(a[w], s1[2 * w], s1[2 * w + 1]);
                f2_unpack(qq[w], s2[2 * w], s2[2 * w + 1]);
            }
            // halving butterfly over the 8 lanes that share the positions: after the three steps lane
            // rs holds the complete sums of position rs of the chunk
#pragma unroll
            for (int half = 4; half >= 1; half >>= 1) {
                const bool up = (rs & half) != 0;
#pragma unroll
                for (int i = 0; i < half; ++i) {
                    const float send1 = up ? s1[i] : s1[i + half], keep1 = up ? s1[i + half] : s1[i];
                    const float send2 = up ? s2[i] : s2[i + half], keep2 = up ? s2[i + half] : s2[i];
                    s1[i] = keep1 + __shfl_xor_sync(0xffffffffu, send1, half);
                    s2[i] = keep2 + __shfl_xor_sync(0xffffffffu, send2, half);
                }
            }
            const uint32_t shw = (rs >> 1) == 0 ? sh[0] : (rs >> 1) == 1 ? sh[1] : (rs >> 1) == 2 ? sh[2] : sh[3];
            const float shift = (rs & 1) ? bf16_hi(shw) : bf16_lo(shw);
            const float m1 = s1[0] * inv_c;
            const float rstd = rsqrtf(fmaxf(fmaf(-m1, m1, s2[0] * inv_c), 0.f) + p.eps_out);
            const float t = -(shift + m1) * rstd;
            // the statistics go into the tile's last tri slot once nothing reads the tri data there any more
            const uint32_t u0 = it * kKH + kKH - 1;
            const int slot0 = u0 & 1;
            if (!group_wait<true>(&tri_dead[slot0], (u0 >> 1) & 1u, tid == 0, kG2StatOutBarrier, kG2StatThreads, abort_flag,
                                  p.status, kStageIdTm2, 510 + slot0))
                break;
            // position 8 cq + rs == tid
            *(reinterpret_cast<float2*>(reinterpret_cast<float4*>(sT + slot0 * kT2TBytes) + tid) + 1) = make_float2(rstd, t);
            mbar_arrive(&stat_out[s]);
            if (tid == 0) TRIMUL_STAMP(5, it, 1);
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
