// Stage 1 of the block on CTA PAIRS (tcgen05 cta_group::2), c = 128: LayerNorm_in, pair mask and
// the two sigmoid-gated projections in one pass over z, writing a and b as channel-major planes.
// Same arithmetic and layouts as tm1_sm100_kernel; what changes is how the work is split.
//
// A pair of CTAs (a cluster of two) processes a 128-position tile together:
//   * each CTA loads and normalises ITS 64 positions of the tile (the UMMA B operand, N = 128,
//     is read half from each CTA's shared memory) — LayerNorm work is split, not duplicated;
//   * the UMMA has M = 256: rows 0..127 are the LEFT projection (or gate) weights held by the
//     leader CTA, rows 128..255 the RIGHT ones held by the other CTA.  So each CTA keeps only two
//     of the four weight matrices (64 KB), and its TMEM receives its own side's accumulators for
//     all 128 positions: proj and gate, 128 columns each;
//   * that leaves room for TWO accumulator sets per CTA (the epilogue of tile t overlaps the UMMAs
//     of tile t+1) and a 6-deep ring of 16 KB position tiles (loads run far ahead), which the
//     single-CTA kernel cannot afford (4 x 128 TMEM columns, 128 KB of weights).
//
// Roles per CTA (832 threads):
//   warp 0        TMA producer: this CTA's two weight matrices, then its 64-position tiles
//   warp 1        UMMA issuer (leader CTA only; the other CTA's warp 1 only allocates TMEM)
//   warps 2..9    LayerNorm, four groups of two warps taking every fourth tile, one thread per position
//   warps 10..25  epilogue of this CTA's side, four groups of four warps: (accumulator set, half tile):
//                 TMEM -> p * sigmoid(g) -> bf16 -> swizzled staging -> TMA store
// Cross-CTA signalling (no TMA multicast anywhere):
//   xn_ready[s]   in the leader, 2 arrivals: each CTA's LayerNorm group reports its half (remote arrive)
//   x_empty[s]    in each CTA: tcgen05.commit multicast once the UMMAs that read stage s retire
//   acc_full[b]   in each CTA: commit multicast
//   acc_empty[b]  in the leader, 16 arrivals: eight epilogue warps of each CTA (remote arrive)
//   w_all         in the leader, 2 arrivals: each CTA's weights are loaded and halved
#pragma once

#include "tm1_sm100.cuh"

namespace trimul {

constexpr int kP1Threads = 832;
constexpr int kP1Stages = 6;
constexpr int kP1HalfPos = 64;                          // positions per CTA per tile
constexpr int kP1SubTile = kP1HalfPos * 64 * 2;         // 8 KB: 64 positions x 64 channels
constexpr int kP1XBytes = 2 * kP1SubTile;               // 16 KB: this CTA's half tile, two K halves
constexpr int kP1WSub = 128 * 64 * 2;                   // 16 KB: 128 weight rows x 64 input channels
constexpr int kP1WBytes = 4 * kP1WSub;                  // proj + gate of this CTA's side
constexpr int kP1BoxBytes = 128 * 64 * 2;               // 16 KB store box: 128 channels x 64 positions
constexpr int kP1OffX = kP1WBytes;
constexpr int kP1OffStaging = kP1OffX + kP1Stages * kP1XBytes;
constexpr int kP1OffAffine = kP1OffStaging + 4 * kP1BoxBytes;   // two boxes per epilogue group
constexpr int kP1OffBars = kP1OffAffine + 2 * kT1C * 4;
constexpr int kP1SmemBytes = kP1OffBars + 320;
constexpr int kP1LnBarrier = 2;        // 2..5: the four LayerNorm groups
constexpr int kP1EpiBarrier = 6;       // 6..9: the four epilogue groups

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kP1Threads, 1)
tm1_pair_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWp,
                      const __grid_constant__ CUtensorMap tmWg, const __grid_constant__ CUtensorMap tmWp2,
                      const __grid_constant__ CUtensorMap tmWg2, const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const Tm1Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm1, 901);
        return;
    }
    uint8_t* sW = smem;                                  // [proj K0, proj K1, gate K0, gate K1]
    uint8_t* sX = smem + kP1OffX;
    uint8_t* sOut = smem + kP1OffStaging;
    float* sGamma = reinterpret_cast<float*>(smem + kP1OffAffine);
    float* sBeta = sGamma + kT1C;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kP1OffBars);
    uint64_t* x_full = bars;                             // [stages] this CTA's half tile landed
    uint64_t* xn_ready = bars + kP1Stages;               // [stages] leader: both halves normalised
    uint64_t* x_empty = bars + 2 * kP1Stages;            // [stages] UMMAs that read the stage retired
    uint64_t* acc_full = bars + 3 * kP1Stages;           // [2]
    uint64_t* acc_empty = acc_full + 2;                  // [2] leader, 8 arrivals
    uint64_t* w_full = acc_empty + 2;                    // this CTA's weights landed
    uint64_t* w_ready = w_full + 1;                      // ... and halved (all worker threads)
    uint64_t* w_all = w_ready + 1;                       // leader: both CTAs' weights ready
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_all + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();             // 0 = leader = left side, 1 = right side
    const bool is_leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kP1Stages; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&xn_ready[s], 2);
            mbar_init(&x_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 16);
        }
        mbar_init(w_full, 1);
        mbar_init(w_ready, kP1Threads - 64);
        mbar_init(w_all, 2);
        *abort_flag = 0;
        fence_mbarrier_init();
        tma_prefetch_desc(&tmZ);
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (threadIdx.x >= 64 && threadIdx.x < 64 + kT1C) {
        sGamma[threadIdx.x - 64] = p.gamma[threadIdx.x - 64];
        sBeta[threadIdx.x - 64] = p.beta[threadIdx.x - 64];
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // pair tiles: 128 positions (this CTA: 64 of them) along the running index
    const int tiles_per_fixed = (p.n_run + 127) / 128;
    const int total_tiles = p.B * p.n_fixed * tiles_per_fixed;
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;

    if (warp >= 2) {
        // every worker thread: halve its share of this CTA's weights once they have landed
        if (mbar_wait(w_full, 0, abort_flag, p.status, kStageIdTm1, 1150)) {
            halve_bf16_smem(sW, kP1WBytes, threadIdx.x - 64, kP1Threads - 64);
            fence_proxy_async_smem();
        }
        mbar_arrive(w_ready);
        if (threadIdx.x == 64) {
            // one thread reports this CTA's weights to the leader's UMMA issuer
            mbar_wait(w_ready, 0, abort_flag, p.status, kStageIdTm1, 1151);
            mbar_arrive_cluster(map_to_cta(smem_u32(w_all), 0));
        }
        __syncwarp();
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, kP1WBytes);
            const CUtensorMap* wp = is_leader ? &tmWp : &tmWp2;
            const CUtensorMap* wg = is_leader ? &tmWg : &tmWg2;
            for (int kh = 0; kh < 2; ++kh) {
                tma_load_2d(sW + kh * kP1WSub, wp, w_full, kh * 64, 0);
                tma_load_2d(sW + (2 + kh) * kP1WSub, wg, w_full, kh * 64, 0);
            }
            uint32_t it = 0;
            for (int tile = cluster_id; tile < total_tiles; tile += num_clusters, ++it) {
                const int s = it % kP1Stages;
                const uint32_t ph = (it / kP1Stages) & 1u;
                if (!mbar_wait(&x_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm1, 1100 + s)) break;
                const int t0 = (tile % tiles_per_fixed) * 128 + (int)rank * kP1HalfPos;
                const int bf = tile / tiles_per_fixed;
                const int f = bf % p.n_fixed;
                const int b = bf / p.n_fixed;
                if (is_leader) TRIMUL_STAMP(0, it, 0);
                mbar_arrive_expect_tx(&x_full[s], kP1XBytes);
                uint8_t* dst = sX + s * kP1XBytes;
                const int col = p.incoming ? f : t0;
                const int row = p.incoming ? t0 : f;
                tma_load_4d(dst, &tmZ, &x_full[s], 0, col, row, b);
                tma_load_4d(dst + kP1SubTile, &tmZ, &x_full[s], 64, col, row, b);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer (leader)
        if (lane == 0 && is_leader) {
            constexpr uint32_t idesc = umma_idesc_bf16(256, 128);
            bool ok = mbar_wait(w_all, 0, abort_flag, p.status, kStageIdTm1, 1200);
            tcgen05_fence_after();
            const uint32_t wp = smem_u32(sW), wg = smem_u32(sW + 2 * kP1WSub);
            uint32_t it = 0;
            for (int tile = cluster_id; ok && tile < total_tiles; tile += num_clusters, ++it) {
                const int s = it % kP1Stages;
                const uint32_t ph = (it / kP1Stages) & 1u;
                const uint32_t buf = it & 1u;
                if (!mbar_wait(&acc_empty[buf], ((it >> 1) & 1u) ^ 1u, abort_flag, p.status, kStageIdTm1, 1210 + buf))
                    break;
                if (!mbar_wait(&xn_ready[s], ph, abort_flag, p.status, kStageIdTm1, 1220 + s)) break;
                tcgen05_fence_after();
                TRIMUL_STAMP(2, it, 0);
                const uint32_t xs = smem_u32(sX + s * kP1XBytes);
                const uint32_t d_p = tmem_base + buf * 256;
                const uint32_t d_g = d_p + 128;
#pragma unroll
                for (int kk = 0; kk < kT1C / 16; ++kk) {
                    const uint64_t kofs = (kk & 3) * kDescKStep;
                    const uint64_t db = umma_smem_desc_sw128(xs + (kk >> 2) * kP1SubTile) + kofs;
                    umma_bf16_ss_pair(d_p, umma_smem_desc_sw128(wp + (kk >> 2) * kP1WSub) + kofs, db, idesc, kk != 0);
                    umma_bf16_ss_pair(d_g, umma_smem_desc_sw128(wg + (kk >> 2) * kP1WSub) + kofs, db, idesc, kk != 0);
                }
                umma_commit_pair(&x_empty[s]);
                umma_commit_pair(&acc_full[buf]);
            }
        }
        __syncwarp();
    } else if (warp < 10) {
        // ------------------------------------------------------------------ LayerNorm (+ mask)
        // four groups of two warps; group g takes the tiles with (local tile index & 3) == g; one
        // thread per position of this CTA's half tile
        const int g = (warp - 2) >> 1;
        const int pos = threadIdx.x - 64 - g * 64;     // 0..63
        const int bar_id = kP1LnBarrier + g;
        uint32_t it = g;
        for (int tile = cluster_id + g * num_clusters; tile < total_tiles; tile += 4 * num_clusters, it += 4) {
            const int s = it % kP1Stages;
            const uint32_t ph = (it / kP1Stages) & 1u;
            bool keep = true;
            if (p.mask_kind != 0) {
                const int t0 = (tile % tiles_per_fixed) * 128 + (int)rank * kP1HalfPos;
                const int bf = tile / tiles_per_fixed;
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
            if (!group_wait(&x_full[s], ph, pos == 0, bar_id, 64, abort_flag, p.status, kStageIdTm1, 1300 + s)) break;
            if (pos == 0 && is_leader) TRIMUL_STAMP(1, it, 0);
            ln_row_inplace(sX + s * kP1XBytes, kP1SubTile, pos, sGamma, sBeta, p.eps, !keep);
            fence_proxy_async_smem();          // normalised half tile -> visible to the UMMA (async proxy)
            named_barrier_sync(bar_id, 64);    // the whole half is written ...
            if (pos == 0 && is_leader) TRIMUL_STAMP(1, it, 1);
            if (pos == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&xn_ready[s]), 0));   // ... tell the leader
        }
    } else {
        // ------------------------------------------------------------------ epilogue of this CTA's side
        // four groups of four warps: group (eb, half) drains positions [64*half, 64*half+64) of
        // accumulator set eb, i.e. of the tiles with (local tile index & 1) == eb
        const int ge = (warp - 10) >> 2;
        const int eb = ge >> 1;
        const int half = ge & 1;
        const int q = warp & 3;
        const int ch = q * 32 + lane;                  // output channel == TMEM lane
        const bool leader_thread = ((warp - 10) & 3) == 0 && lane == 0;
        const int bar_id = kP1EpiBarrier + ge;
        uint8_t* box = sOut + ge * kP1BoxBytes;
        const CUtensorMap* om = is_leader ? &tmA : &tmB;
        const int rc = is_leader ? p.a_row_chunk : p.b_row_chunk;
        const int cc = is_leader ? p.a_col_chunk : p.b_col_chunk;
        const uint32_t t_p = tmem_base + eb * 256 + half * 64 + ((uint32_t)(q * 32) << 16);
        uint32_t it = eb;
        for (int tile = cluster_id + eb * num_clusters; tile < total_tiles; tile += 2 * num_clusters, it += 2) {
            const int t0 = (tile % tiles_per_fixed) * 128;
            const int bf = tile / tiles_per_fixed;
            const int f = bf % p.n_fixed;
            const int b = bf / p.n_fixed;
            if (!group_wait(&acc_full[eb], (it >> 1) & 1u, leader_thread, bar_id, 128, abort_flag, p.status,
                            kStageIdTm1, 1400 + ge))
                break;
            tcgen05_fence_after();
            if (leader_thread && is_leader && half == 0) TRIMUL_STAMP(3, it, 0);
            if (leader_thread) tma_store_wait_read<0>();    // this group's previous store (two tiles ago)
            named_barrier_sync(bar_id, 128);
#pragma unroll 1
            for (int c16 = 0; c16 < 4; ++c16) {
                uint32_t rp[16], rg[16];
                if (leader_thread && is_leader && half == 0 && c16 == 1) TRIMUL_STAMP(4, it, 0);
                tmem_ld_32x16(t_p + c16 * 16, rp);
                tmem_ld_32x16(t_p + 128 + c16 * 16, rg);
                tmem_ld_wait();
                if (leader_thread && is_leader && half == 0 && c16 == 1) TRIMUL_STAMP(4, it, 1);
                if (c16 == 3) {
                    // every TMEM read of this group's share has completed: hand it back to the leader
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[eb]), 0));
                    if (leader_thread && is_leader && half == 0) TRIMUL_STAMP(3, it, 1);
                }
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i0 = k * 8 + 2 * e;
                        o[e] = gate2_bf16(__uint_as_float(rp[i0]), __uint_as_float(rg[i0]),
                                          __uint_as_float(rp[i0 + 1]), __uint_as_float(rg[i0 + 1]));
                    }
                    const int chunk = (c16 * 2 + k) ^ (ch & 7);
                    if (leader_thread && is_leader && half == 0 && c16 == 1 && k == 1) TRIMUL_STAMP(4, it, 2);
                    *reinterpret_cast<uint4*>(box + ch * 128 + (chunk << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
                if (leader_thread && is_leader && half == 0 && c16 == 1) TRIMUL_STAMP(4, it, 3);
            }
            fence_proxy_async_smem();
            named_barrier_sync(bar_id, 128);
            if (leader_thread) {
                const int col0 = t0 + half * 64;
                if (col0 < p.n_run) {
                    tma_store_4d(om, box, col0 % cc, f % rc, b * kT1C, col0 / cc + f / rc);
                    tma_store_commit();
                }
            }
        }
        if (leader_thread) tma_store_wait_all<0>();
        __syncwarp();
    }

    if (*abort_flag != 0) {
        for (int i = 0; i < 256; ++i) __nanosleep(1000);
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

}  // namespace trimul
