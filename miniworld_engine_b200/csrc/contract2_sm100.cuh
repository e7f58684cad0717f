// Stage 2 of the block with CTA PAIRS: tri[p] = a[p] . b[p]^T per channel plane, 256 x 256 output
// tiles computed by two CTAs of a cluster with tcgen05.mma.cta_group::2 (UMMA M = 256, N = 256).
//
// Each CTA of the pair loads ITS half of both operands — 128 rows of A and 128 rows of B per
// 64-wide K slice, 32 KB per stage instead of the 48 KB a lone CTA needs for a 128 x 256 tile — so
// L2 -> SM traffic per FLOP drops by a third and the same shared memory holds a 6-deep ring.  The
// pair's UMMA reads the B halves from both CTAs' shared memory; no TMA multicast is involved.
// Each CTA's TMEM receives the accumulator rows of its own A half (128 lanes x 256 columns, two
// of them, so the epilogue overlaps the next tile).
//
// Roles per CTA (192 threads): warp 0 TMA producer (both CTAs), warp 1 UMMA issuer (leader CTA
// only; in the other CTA the warp just allocates TMEM), warps 2..5 epilogue (both CTAs).
// Cross-CTA signalling:
//   full[s]      lives in the leader; the leader's producer posts the pair's byte count, both
//                CTAs' TMA loads complete on it (cta_group::2 loads may signal the peer's barrier)
//   empty[s]     in each CTA; the leader's tcgen05.commit arrives on both (commit multicast)
//   acc_full[a]  in each CTA; commit multicast
//   acc_empty[a] in the leader, 8 arrivals: the four epilogue warps of each CTA (remote arrive with
//                CTA-scope release; the cluster-scope form held each warp for more than a microsecond
//                per tile: 18 % of the kernel at N = 384, 4 % at N = 2048)
//
// The bounded waits of this kernel are out of line (mbar_wait<true>): measured 2-7 % faster than
// the inlined polling loops (N = 768 ... 2048).
//
// kScatter = true: the output rows are split into row chunks of d_row_chunk rows and chunk d is
// stored through destination map d (the multi-GPU exchange of the channel-sharded contraction,
// done by the producing kernel's own TMA stores: chunk d is GPU d's slab of rows).
#pragma once

#include "contract_sm100.cuh"

namespace trimul {

constexpr int kC2Stages = 6;
constexpr int kC2HalfBytes = 128 * kCtBK * 2;            // 16 KB: 128 rows x 64 bf16
constexpr int kC2StageBytes = 2 * kC2HalfBytes;          // this CTA's A half + B half
constexpr int kC2SmemBytes = kC2Stages * kC2StageBytes + kCtStagingBytes + kCtBarBytes;
constexpr int kC2EpiBarrier = 1;

template <bool kScatter>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kCtThreads, 1)
contract2_sm100_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmD, const ContractParams p,
                       const __grid_constant__ ScatterMaps sc) {
    extern __shared__ __align__(1024) uint8_t smem[];
    // (a misaligned dynamic shared-memory base would be the same in both CTAs: uniform exit)
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdContract, 901);
        return;
    }
    uint8_t* staging = smem + kC2Stages * kC2StageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kCtStagingBytes);
    uint64_t* full = bars;                       // [kC2Stages] used in the leader
    uint64_t* empty = bars + kC2Stages;          // [kC2Stages] in each CTA
    uint64_t* acc_full = bars + 2 * kC2Stages;   // [2] in each CTA
    uint64_t* acc_empty = acc_full + 2;          // [2] used in the leader, 8 arrivals
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();     // 0 = leader
    const bool is_leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kC2Stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 8);
        }
        *abort_flag = 0;
        fence_mbarrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        tma_prefetch_desc(&tmD);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();          // both CTAs' barriers are initialised before anyone signals the peer
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up done without touching global memory: now wait for the producer of a and b
    griddep_wait();
    griddep_launch_dependents();

    // pair tiles: 256 rows x 256 columns of one plane
    const int tiles_m = (p.rows_a + 255) / 256;
    const int tiles_n = (p.rows_b + 255) / 256;
    const int tiles_per_plane = tiles_m * tiles_n;
    const int total_tiles = p.planes * tiles_per_plane;
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = cluster_id; ok && tile < total_tiles; tile += num_clusters) {
                const int plane = tile / tiles_per_plane;
                const int rem = tile - plane * tiles_per_plane;
                const int row_a = (rem / tiles_n) * 256 + (int)rank * 128;    // this CTA's halves
                const int row_b = (rem % tiles_n) * 256 + (int)rank * 128;
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % kC2Stages;
                    const uint32_t ph = (it / kC2Stages) & 1u;
                    if (!mbar_wait<true>(&empty[s], ph ^ 1u, abort_flag, p.status, kStageIdContract, 1100 + s)) {
                        ok = false;
                        break;
                    }
                    // the leader's barrier counts the bytes of both CTAs
                    if (is_leader) mbar_arrive_expect_tx(&full[s], 2 * kC2StageBytes);
                    const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
                    const int k0 = kb * kCtBK;
                    uint8_t* sa = smem + s * kC2StageBytes;
                    // rows past the operand's extent are out of range and read as zeros
                    tma_load_4d_pair(sa, &tmA, bar, k0 % p.a_k_chunk, row_a % p.a_row_chunk, plane,
                                     k0 / p.a_k_chunk + row_a / p.a_row_chunk);
                    tma_load_4d_pair(sa + kC2HalfBytes, &tmB, bar, k0 % p.b_k_chunk, row_b % p.b_row_chunk, plane,
                                     k0 / p.b_k_chunk + row_b / p.b_row_chunk);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && is_leader) {
            constexpr uint32_t idesc = umma_idesc_bf16(256, 256);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (int tile = cluster_id; ok && tile < total_tiles; tile += num_clusters, ++tile_it) {
                const uint32_t acc = tile_it & 1u;
                const uint32_t acc_ph = (tile_it >> 1) & 1u;
                if (!mbar_wait<true>(&acc_empty[acc], acc_ph ^ 1u, abort_flag, p.status, kStageIdContract, 1200 + acc)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * 256;
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % kC2Stages;
                    const uint32_t ph = (it / kC2Stages) & 1u;
                    if (!mbar_wait<true>(&full[s], ph, abort_flag, p.status, kStageIdContract, 1300 + s)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(smem + s * kC2StageBytes);
                    const uint64_t da = umma_smem_desc_sw128(sa);
                    const uint64_t db = umma_smem_desc_sw128(sa + kC2HalfBytes);
#pragma unroll
                    for (int kk = 0; kk < kCtBK / 16; ++kk)
                        umma_bf16_ss_pair(d_tmem, da + kk * kDescKStep, db + kk * kDescKStep, idesc,
                                          (kb | kk) != 0 ? 1u : 0u);
                    umma_commit_pair(&empty[s]);
                }
                if (ok) umma_commit_pair(&acc_full[acc]);
            }
        }
        __syncwarp();
    } else {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool leader_thread = (threadIdx.x == 64);
        uint32_t tile_it = 0, store_it = 0;
        for (int tile = cluster_id; tile < total_tiles; tile += num_clusters, ++tile_it) {
            const int plane = tile / tiles_per_plane;
            const int rem = tile - plane * tiles_per_plane;
            const int row_d = (rem / tiles_n) * 256 + (int)rank * 128;
            const int col_d = (rem % tiles_n) * 256;
            const uint32_t acc = tile_it & 1u;
            const uint32_t acc_ph = (tile_it >> 1) & 1u;
            if (!group_wait<true>(&acc_full[acc], acc_ph, leader_thread, kC2EpiBarrier, 128, abort_flag, p.status,
                            kStageIdContract, 1400 + acc))
                break;
            tcgen05_fence_after();
            const uint32_t t_acc = tmem_base + acc * 256 + ((uint32_t)(q * 32) << 16);
            const bool rows_valid = row_d < p.rows_a;       // uniform per CTA
#pragma unroll 1
            for (int box = 0; box < 4; ++box) {
                const int col0 = col_d + box * 64;
                if (col0 >= p.rows_b || !rows_valid) break;
                uint8_t* buf = staging + (store_it & 1u) * (kCtBM * 128);
                ++store_it;
                if (leader_thread) tma_store_wait_read<1>();
                named_barrier_sync(kC2EpiBarrier, 128);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t r[32];
                    tmem_ld_32x32(t_acc + box * 64 + half * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        uint4 v;
                        v.x = pack_bf16x2(__uint_as_float(r[cc * 8 + 0]), __uint_as_float(r[cc * 8 + 1]));
                        v.y = pack_bf16x2(__uint_as_float(r[cc * 8 + 2]), __uint_as_float(r[cc * 8 + 3]));
                        v.z = pack_bf16x2(__uint_as_float(r[cc * 8 + 4]), __uint_as_float(r[cc * 8 + 5]));
                        v.w = pack_bf16x2(__uint_as_float(r[cc * 8 + 6]), __uint_as_float(r[cc * 8 + 7]));
                        const int chunk = (half * 4 + cc) ^ (row & 7);
                        *reinterpret_cast<uint4*>(buf + row * 128 + chunk * 16) = v;
                    }
                }
                fence_proxy_async_smem();
                named_barrier_sync(kC2EpiBarrier, 128);
                if (leader_thread) {
                    if (kScatter)   // this CTA's 128 rows lie inside one destination's row chunk
                        tma_store_4d(&sc.map[row_d / p.d_row_chunk], buf, col0, row_d % p.d_row_chunk, plane, 0);
                    else
                        tma_store_4d(&tmD, buf, col0 % p.d_col_chunk, row_d % p.d_row_chunk, plane,
                                     col0 / p.d_col_chunk + row_d / p.d_row_chunk);
                    tma_store_commit();
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&acc_empty[acc]), 0));
        }
        if (leader_thread) tma_store_wait_all<0>();
        __syncwarp();
    }

    if (*abort_flag != 0) {
        for (int i = 0; i < 256; ++i) __nanosleep(1000);
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer may still be reading this CTA's shared memory / barriers
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

}  // namespace trimul
