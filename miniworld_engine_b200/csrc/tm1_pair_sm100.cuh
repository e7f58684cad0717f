// Stage 1 of the block on CTA PAIRS (tcgen05 cta_group::2), c = 128: LayerNorm_in, pair mask and
// the two sigmoid-gated projections in one pass over z (reference.py:66-75), writing a and b as
// channel-major planes for the contraction.  Same arithmetic and layouts as tm1_sm100.cuh; what
// changes is how the work is split, and with it what fits on an SM.
//
// A pair of CTAs (a cluster of two) processes a 128-position tile together:
//   * each CTA loads and normalises ITS 64 positions of the tile (the UMMA B operand, N = 128, is
//     read half from each CTA's shared memory) — LayerNorm work is split, not duplicated;
//   * the UMMA has M = 256: rows 0..127 are the LEFT projection (or gate) weights held by the leader
//     CTA, rows 128..255 the RIGHT ones held by the other CTA.  So each CTA keeps only two of the
//     four weight matrices (64 KB), and its TMEM receives its own side's accumulators for all 128
//     positions: proj and gate, 128 columns each;
//   * that leaves room for TWO accumulator sets per CTA (the epilogue of tile t overlaps the UMMAs
//     of tile t+1), a 6-deep ring of 16 KB position tiles (loads run far ahead) and four store
//     boxes, none of which the single-CTA kernel can afford (4 x 128 TMEM columns, 128 KB of weights).
//
// Roles per CTA (832 threads):
//   warp 0        TMA producer: this CTA's two weight matrices, then its 64-position tiles
//   warp 1        UMMA issuer (leader CTA only; the other CTA's warp 1 only allocates TMEM)
//   warps 2..9    LayerNorm (+ mask): two groups of four warps on alternate tiles, 16 rows per warp,
//                 eight lanes per row, in place in the swizzled tile; a masked position is written as
//                 a zero row
//   warps 10..25  epilogue of this CTA's side, sixteen independent warps: warp = (accumulator set,
//                 position half, TMEM lane quarter); TMEM -> p * sigmoid(g) -> bf16 -> the warp's own
//                 swizzled [32 channels][64 positions] box -> the warp's own TMA store
// Cross-CTA signalling (no TMA multicast anywhere):
//   xn_ready[s]   in the leader, 8 arrivals: the four LayerNorm warps of the tile's group in both CTAs
//   x_empty[s]    in each CTA: tcgen05.commit multicast once the UMMAs that read stage s retire
//   acc_full[b]   in each CTA: commit multicast
//   acc_empty[b]  in the leader, 16 arrivals: the set's eight epilogue warps of each CTA (remote arrive)
//   w_all         in the leader, 2 arrivals: each CTA's weights are loaded and halved
//
// kScatter = true: a warp's 32 planes are stored in segments of planes_per_dest planes (16 or 32),
// each through the tensor map of the destination buffer that holds those planes — the multi-GPU
// exchange of the channel-sharded contraction, done by this kernel's own TMA stores.
#pragma once

#include "tm1_common.cuh"

namespace trimul {

constexpr int kP1Threads = 832;
constexpr int kP1Stages = 6;
constexpr int kP1LnWarps = 8;
constexpr int kP1EpiWarps = 16;
constexpr int kP1HalfPos = 64;                          // positions per CTA per tile
constexpr int kP1SubTile = kP1HalfPos * 64 * 2;         // 8 KB: 64 positions x 64 channels
constexpr int kP1XBytes = 2 * kP1SubTile;               // 16 KB: this CTA's half tile, two K halves
constexpr int kP1WSub = 128 * 64 * 2;                   // 16 KB: 128 weight rows x 64 input channels
constexpr int kP1WBytes = 4 * kP1WSub;                  // proj + gate of this CTA's side
constexpr int kP1WarpBoxBytes = 32 * 64 * 2;            // 4 KB store box of one epilogue warp: 32 channels x 64 positions
constexpr int kP1OffX = kP1WBytes;
constexpr int kP1OffStaging = kP1OffX + kP1Stages * kP1XBytes;
constexpr int kP1OffBars = kP1OffStaging + kP1EpiWarps * kP1WarpBoxBytes;
constexpr int kP1SmemBytes = kP1OffBars + 320;
constexpr int kP1LnBarrier = 2;        // 2, 3: the two LayerNorm groups
constexpr int kP1EpiBarrier = 4;       // 4, 5: the eight epilogue warps of accumulator set 0, 1
static_assert(kP1SmemBytes <= 232448, "stage 1 shared memory exceeds the 227 KB a CTA may use");

template <bool kScatter>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kP1Threads, 1)
tm1_pair_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWl,
                      const __grid_constant__ CUtensorMap tmWlg, const __grid_constant__ CUtensorMap tmWr,
                      const __grid_constant__ CUtensorMap tmWrg, const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const __grid_constant__ Tm1Params p,
                      const __grid_constant__ ScatterMaps scA, const __grid_constant__ ScatterMaps scB) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        // both CTAs of a pair see the same offset, so both leave here and nobody waits for the other
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm1, 901);
        return;
    }
    uint8_t* sW = smem;                                  // [proj K0, proj K1, gate K0, gate K1]
    uint8_t* sX = smem + kP1OffX;
    uint8_t* sOut = smem + kP1OffStaging;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kP1OffBars);
    uint64_t* x_full = bars;                             // [stages] this CTA's half tile landed
    uint64_t* xn_ready = bars + kP1Stages;               // [stages] leader: both halves normalised
    uint64_t* x_empty = bars + 2 * kP1Stages;            // [stages] UMMAs that read the stage retired
    uint64_t* acc_full = bars + 3 * kP1Stages;           // [2]
    uint64_t* acc_empty = acc_full + 2;                  // [2] leader
    uint64_t* w_full = acc_empty + 2;                    // this CTA's weights landed
    uint64_t* w_ready = w_full + 1;                      // ... and halved (all worker threads)
    uint64_t* w_all = w_ready + 1;                       // leader: both CTAs' weights ready
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_all + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    static_assert((3 * kP1Stages + 7) * 8 + 8 <= 320, "barrier block too small");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) TRIMUL_STAMP(7, TRIMUL_TRACE_FIRST, 0);
    const uint32_t rank = cluster_ctarank();             // 0 = leader = left side, 1 = right side
    const bool is_leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kP1Stages; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&xn_ready[s], kP1LnWarps);        // four warps of each CTA per tile
            mbar_init(&x_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], kP1EpiWarps);      // eight warps of each CTA per set
        }
        mbar_init(w_full, 1);
        mbar_init(w_ready, kP1Threads - 64);
        mbar_init(w_all, 2);
        *abort_flag = 0;
        fence_mbarrier_init();
        tma_prefetch_desc(&tmZ);
        tma_prefetch_desc(is_leader ? &tmA : &tmB);
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

    // Everything above touches no global memory; from here on the kernel reads what its
    // predecessor in the stream may have written.
    griddep_wait();
    griddep_launch_dependents();
    if (threadIdx.x == 0) TRIMUL_STAMP(7, TRIMUL_TRACE_FIRST, 1);

    // pair tiles: 128 positions (this CTA: 64 of them) along the running index
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;

    if (warp >= 2) {
        // every worker thread: halve its share of this CTA's weights once they have landed
        if (mbar_wait<true>(w_full, 0, abort_flag, p.status, kStageIdTm1, 1150)) {
            halve_bf16_smem(sW, kP1WBytes, threadIdx.x - 64, kP1Threads - 64);
            fence_proxy_async_smem();
        }
        mbar_arrive(w_ready);
        if (threadIdx.x == 64) {
            // one thread reports this CTA's weights to the leader's UMMA issuer
            mbar_wait<true>(w_ready, 0, abort_flag, p.status, kStageIdTm1, 1151);
            mbar_arrive_remote(map_to_cta(smem_u32(w_all), 0));
        }
        __syncwarp();
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, kP1WBytes);
            const CUtensorMap* wp = is_leader ? &tmWl : &tmWr;
            const CUtensorMap* wg = is_leader ? &tmWlg : &tmWrg;
            for (int kh = 0; kh < 2; ++kh) {
                tma_load_2d(sW + kh * kP1WSub, wp, w_full, kh * 64, 0);
                tma_load_2d(sW + (2 + kh) * kP1WSub, wg, w_full, kh * 64, 0);
            }
            uint32_t it = 0;
            Tm1Cursor cur;
            cur.init(p, cluster_id);
            for (int tile = cluster_id; tile < p.total_tiles; tile += num_clusters, ++it, cur.next(p, 0)) {
                const int s = it % kP1Stages;
                const uint32_t ph = (it / kP1Stages) & 1u;
                if (!mbar_wait<true>(&x_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm1, 1100 + s)) break;
                const int b = cur.b, f = cur.f, t0 = cur.t0() + (int)rank * kP1HalfPos;
                if (is_leader) TRIMUL_STAMP(0, it, 0);
                mbar_arrive_expect_tx(&x_full[s], kP1XBytes);
                uint8_t* dst = sX + s * kP1XBytes;
                // z viewed as (channel, column, row, batch); outgoing box = 64 columns of row f,
                // incoming box = 64 rows of column f (positions past the end read as zeros)
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
            bool ok = mbar_wait<true>(w_all, 0, abort_flag, p.status, kStageIdTm1, 1200);
            TRIMUL_STAMP(7, TRIMUL_TRACE_FIRST, 2);
            tcgen05_fence_after();
            const uint32_t wp = smem_u32(sW), wg = smem_u32(sW + 2 * kP1WSub);
            uint32_t it = 0;
            for (int tile = cluster_id; ok && tile < p.total_tiles; tile += num_clusters, ++it) {
                const int s = it % kP1Stages;
                const uint32_t ph = (it / kP1Stages) & 1u;
                const uint32_t buf = it & 1u;
                if (!mbar_wait<true>(&acc_empty[buf], ((it >> 1) & 1u) ^ 1u, abort_flag, p.status, kStageIdTm1,
                                     1210 + buf))
                    break;
                TRIMUL_STAMP(1, it, 0);
                if (!mbar_wait<true>(&xn_ready[s], ph, abort_flag, p.status, kStageIdTm1, 1220 + s)) break;
                tcgen05_fence_after();
                TRIMUL_STAMP(1, it, 1);
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
                TRIMUL_STAMP(1, it, 2);
            }
        }
        __syncwarp();
    } else if (warp < 2 + kP1LnWarps) {
        // ------------------------------------------------------------------ LayerNorm (+ mask)
        // two groups of four warps on alternate tiles (a group has two tile periods for its half tile, and
        // nobody waits for the slowest of eight warps); warp lw of a group owns rows [16 lw, 16 lw + 16):
        // lane l row 16 lw + 4 i + (l >> 3) in iteration i, 16-byte chunk l & 7 of both 64-channel sub-tiles
        const int lg = (warp - 2) >> 2;
        const int lw = (warp - 2) & 3;
        const int rr = lane >> 3;
        f32x2 gb[16];
        ln_load_affine<2>(gb, p.gamma, p.beta, lane);
        uint32_t it = lg;
        Tm1Cursor cur;
        cur.init(p, cluster_id + lg * num_clusters);
        // Pair mask: lane l < 16 looks up position 16 lw + l of the half tile — one or two byte loads,
        // issued ONE TILE AHEAD so that their latency (the mask of a large pair tensor streams from L2
        // or DRAM) hides behind the LayerNorm of the current tile — and a ballot hands every lane the
        // bits of its own rows.
        const int my_pos = (int)rank * kP1HalfPos + 16 * lw + lane;
        bool keep_next = true;
        if (p.mask_kind != 0 && lane < 16 && cluster_id + lg * num_clusters < p.total_tiles)
            keep_next = tm1_keep(p, cur.b, cur.f, cur.t0() + my_pos);
        for (int tile = cluster_id + lg * num_clusters; tile < p.total_tiles; tile += 2 * num_clusters, it += 2) {
            const int s = it % kP1Stages;
            const uint32_t ph = (it / kP1Stages) & 1u;
            const bool keep = keep_next;
            cur.next(p, 1);
            if (p.mask_kind != 0 && lane < 16 && tile + 2 * num_clusters < p.total_tiles)
                keep_next = tm1_keep(p, cur.b, cur.f, cur.t0() + my_pos);
            // ONE thread of the group's four warps polls; the others park at the group's named barrier
            if (!group_wait<true>(&x_full[s], ph, lw == 0 && lane == 0, kP1LnBarrier + lg, 128, abort_flag, p.status,
                                  kStageIdTm1, 1300 + s))
                break;
            uint32_t zero_bits = 0u;
            if (p.mask_kind != 0) {
                const uint32_t drop = ~__ballot_sync(0xffffffffu, keep);
#pragma unroll
                for (int i = 0; i < 4; ++i) zero_bits |= ((drop >> (4 * i + rr)) & 1u) << i;
            }
            if (lw == 0 && lane == 0 && is_leader) TRIMUL_STAMP(2, it, 0);
            ln_rows_warp<4>(sX + s * kP1XBytes, kP1SubTile, 16 * lw, lane, gb, p.eps, zero_bits);
            fence_proxy_async_smem();   // normalised rows -> visible to the UMMA (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&xn_ready[s]), 0));
            if (lw == 0 && lane == 0 && is_leader) TRIMUL_STAMP(2, it, 1);
        }
    } else {
        // ------------------------------------------------------------------ epilogue of this CTA's side
        // Sixteen warps that meet only where a set's eight wait for its accumulators.  Warp = (accumulator set eb, position half,
        // TMEM lane quarter q): it drains 32 channels x 64 positions of every second tile into its own
        // 4 KB store box ([32 channels][64 positions], swizzled) and issues its own TMA store, so two
        // tiles are in the epilogue at any time and a slow warp delays nobody else.
        const int ew = warp - 10;
        const uint32_t eb = (uint32_t)ew >> 3;
        const int half = (ew >> 2) & 1;
        const int q = warp & 3;
        const int chl = lane;                          // channel inside the warp's quarter; TMEM lane q * 32 + lane
        uint8_t* box = sOut + ew * kP1WarpBoxBytes;
        const CUtensorMap* om = is_leader ? &tmA : &tmB;
        const int rc = is_leader ? p.a_row_chunk : p.b_row_chunk;
        const int cc = is_leader ? p.a_col_chunk : p.b_col_chunk;
        const uint32_t t_p = tmem_base + eb * 256 + half * 64 + ((uint32_t)(q * 32) << 16);
        uint32_t it = eb;
        Tm1Cursor cur;
        cur.init(p, cluster_id + (int)eb * num_clusters);
        for (int tile = cluster_id + (int)eb * num_clusters; tile < p.total_tiles;
             tile += 2 * num_clusters, it += 2, cur.next(p, 1)) {
            const int b = cur.b, f = cur.f, t0 = cur.t0();
            if (lane == 0) tma_store_wait_read<0>();   // this warp's previous store has read the box
            // ONE thread of the set's eight warps polls (every poller costs the working warps issue slots);
            // the others park at the set's named barrier
            if (!group_wait<true>(&acc_full[eb], (it >> 1) & 1u, (ew & 7) == 0 && lane == 0, kP1EpiBarrier + (int)eb, 256,
                                  abort_flag, p.status, kStageIdTm1, 1400 + (int)eb))
                break;
            tcgen05_fence_after();
            if (ew == 0 && lane == 0 && is_leader) TRIMUL_STAMP(3, it, 0);
            // 8 positions at a time; the TMEM loads of the next 8 are in flight while the current 8 are
            // gated, rounded and written to the box
            auto emit8 = [&](int c8, const uint32_t (&rp)[8], const uint32_t (&rg)[8]) {
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    o[e] = gate2_bf16(__uint_as_float(rp[2 * e]), __uint_as_float(rg[2 * e]),
                                      __uint_as_float(rp[2 * e + 1]), __uint_as_float(rg[2 * e + 1]));
                const int chunk = c8 ^ (chl & 7);
                *reinterpret_cast<uint4*>(box + chl * 128 + (chunk << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
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
                    // every TMEM read of this warp's share has completed: hand it back to the leader
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&acc_empty[eb]), 0));
                    if (ew == 0 && lane == 0 && is_leader) TRIMUL_STAMP(3, it, 1);
                }
                emit8(c8 + 1, rpB, rgB);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                const int col0 = t0 + half * 64;
                if (col0 < p.n_run) {
                    if (kScatter) {
                        // the warp's 32 planes in segments of one destination's share
                        const ScatterMaps* sm = is_leader ? &scA : &scB;
                        const int seg = p.planes_per_dest < 32 ? p.planes_per_dest : 32;
                        for (int k0 = 0; k0 < 32; k0 += seg) {
                            const int plane = b * kT1C + q * 32 + k0;
                            const int d = plane / p.planes_per_dest;
                            tma_store_4d(&sm->map[d], box + k0 * 128, col0 % cc, f % rc, plane - d * p.planes_per_dest,
                                         col0 / cc + f / rc);
                        }
                    } else {
                        tma_store_4d(om, box, col0 % cc, f % rc, b * kT1C + q * 32, col0 / cc + f / rc);
                    }
                    tma_store_commit();
                }
                if (ew == 0 && is_leader) TRIMUL_STAMP(3, it, 2);
            }
        }
        if (lane == 0) tma_store_wait_all<0>();
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
