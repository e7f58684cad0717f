// Stage 2 of the block on the tensor cores: tri[p][i][j] = sum_k a[p][i][k] * b[p][j][k] for
// every channel plane p (the einsum of the reference, reference.py:77-80, after stage 1 has
// laid both operands out K-contiguous for either direction).
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warp 0      TMA producer: 64-wide K slices of a 128-row A tile and a 256-row B tile into a
//               ring of shared-memory stages (SWIZZLE_128B, which is the UMMA K-major layout)
//   warp 1      UMMA issuer: 128x256x16 tcgen05.mma into one of two 256-column TMEM accumulators
//   warps 2..5  epilogue: TMEM -> registers -> bf16 -> swizzled staging -> TMA store, overlapping
//               the next tile's main loop through the second accumulator
// Tiles are enumerated plane-major, so the CTAs in flight share a few planes' operands in L2.
// Ragged sizes are handled by TMA: out-of-range loads read zeros, stores are clipped.
#pragma once

#include "ptx_sm100.cuh"

namespace trimul {

constexpr int kCtBM = 128;          // tile rows (UMMA M)
constexpr int kCtBN = 256;          // tile columns (UMMA N)
constexpr int kCtBK = 64;           // K slice per stage: one 128-byte swizzle row of bf16
constexpr int kCtStages = 4;
constexpr int kCtThreads = 192;
constexpr int kCtABytes = kCtBM * kCtBK * 2;           // 16 KB
constexpr int kCtBBytes = kCtBN * kCtBK * 2;           // 32 KB
constexpr int kCtStageBytes = kCtABytes + kCtBBytes;   // 48 KB
constexpr int kCtStagingBytes = 2 * kCtBM * 64 * 2;    // two 128x64 bf16 store boxes
constexpr int kCtBarBytes = 256;
constexpr int kCtSmemBytes = kCtStages * kCtStageBytes + kCtStagingBytes + kCtBarBytes;
constexpr int kCtEpiBarrier = 1;    // named barrier id of the 128 epilogue threads
constexpr int kStageIdContract = 2;

struct ContractParams {
    int planes, rows_a, rows_b, K;
    int tiles_m, tiles_n, num_kb;
    // chunk sizes of the 4-D tensor maps (== the full extent when the operand is not chunked)
    int a_row_chunk, a_k_chunk;
    int b_row_chunk, b_k_chunk;
    int d_row_chunk, d_col_chunk;
    int32_t* status;
};

__global__ void __launch_bounds__(kCtThreads, 1)
contract_sm100_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmD, const ContractParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {   // swizzled tiles need 1024-byte alignment; uniform exit
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdContract, 900);
        return;
    }
    uint8_t* staging = smem + kCtStages * kCtStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kCtStagingBytes);
    uint64_t* full = bars;                       // [kCtStages] TMA landed
    uint64_t* empty = bars + kCtStages;          // [kCtStages] UMMAs that read the stage retired
    uint64_t* acc_full = bars + 2 * kCtStages;   // [2] accumulator complete
    uint64_t* acc_empty = acc_full + 2;          // [2] accumulator drained by the epilogue
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kCtStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_mbarrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        tma_prefetch_desc(&tmD);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_per_plane = p.tiles_m * p.tiles_n;
    const int total_tiles = p.planes * tiles_per_plane;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int plane = tile / tiles_per_plane;
                const int rem = tile - plane * tiles_per_plane;
                const int row_a = (rem / p.tiles_n) * kCtBM;
                const int row_b = (rem % p.tiles_n) * kCtBN;
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % kCtStages;
                    const uint32_t ph = (it / kCtStages) & 1u;
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.status, kStageIdContract, 100 + s)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full[s], kCtStageBytes);
                    const int k0 = kb * kCtBK;
                    uint8_t* sa = smem + s * kCtStageBytes;
                    tma_load_4d(sa, &tmA, &full[s], k0 % p.a_k_chunk, row_a % p.a_row_chunk, plane,
                                k0 / p.a_k_chunk + row_a / p.a_row_chunk);
                    tma_load_4d(sa + kCtABytes, &tmB, &full[s], k0 % p.b_k_chunk, row_b % p.b_row_chunk, plane,
                                k0 / p.b_k_chunk + row_b / p.b_row_chunk);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(kCtBM, kCtBN);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tile_it) {
                const uint32_t acc = tile_it & 1u;
                const uint32_t acc_ph = (tile_it >> 1) & 1u;
                if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1u, abort_flag, p.status, kStageIdContract, 200 + acc)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kCtBN;
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % kCtStages;
                    const uint32_t ph = (it / kCtStages) & 1u;
                    if (!mbar_wait(&full[s], ph, abort_flag, p.status, kStageIdContract, 300 + s)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(smem + s * kCtStageBytes);
                    const uint64_t da = umma_smem_desc_sw128(sa);
                    const uint64_t db = umma_smem_desc_sw128(sa + kCtABytes);
#pragma unroll
                    for (int kk = 0; kk < kCtBK / 16; ++kk) {
                        umma_bf16_ss(d_tmem, da + kk * kDescKStep, db + kk * kDescKStep, idesc,
                                     (kb | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);   // stage reusable once these UMMAs have read it
                }
                if (ok) umma_commit(&acc_full[acc]);
            }
        }
        __syncwarp();
    } else {
        // epilogue: warp w may touch TMEM lanes [32*(w%4), 32*(w%4)+32)
        const int q = warp & 3;
        const int row = q * 32 + lane;              // row inside the tile == TMEM lane
        const bool leader = (threadIdx.x == 64);    // issues the TMA stores
        uint32_t tile_it = 0, store_it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++tile_it) {
            const int plane = tile / tiles_per_plane;
            const int rem = tile - plane * tiles_per_plane;
            const int row_d = (rem / p.tiles_n) * kCtBM;
            const int col_d = (rem % p.tiles_n) * kCtBN;
            const uint32_t acc = tile_it & 1u;
            const uint32_t acc_ph = (tile_it >> 1) & 1u;
            if (!group_wait(&acc_full[acc], acc_ph, leader, kCtEpiBarrier, 128, abort_flag, p.status, kStageIdContract,
                            400 + acc))
                break;
            tcgen05_fence_after();
            const uint32_t t_acc = tmem_base + acc * kCtBN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int box = 0; box < kCtBN / 64; ++box) {
                const int col0 = col_d + box * 64;
                if (col0 >= p.rows_b) break;        // uniform across the CTA
                // the two staging boxes alternate per store; the store issued two stores ago read
                // this one, so at most the latest store may still be reading
                uint8_t* buf = staging + (store_it & 1u) * (kCtBM * 128);
                ++store_it;
                if (leader) tma_store_wait_read<1>();
                named_barrier_sync(kCtEpiBarrier, 128);
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
                named_barrier_sync(kCtEpiBarrier, 128);
                if (leader) {
                    tma_store_4d(&tmD, buf, col0 % p.d_col_chunk, row_d % p.d_row_chunk, plane,
                                 col0 / p.d_col_chunk + row_d / p.d_row_chunk);
                    tma_store_commit();
                }
            }
            // all TMEM reads of this accumulator have completed (each load was waited for)
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
        if (leader) tma_store_wait_all<0>();
        __syncwarp();
    }

    // tear-down; after an abort give in-flight bulk copies time to land before shared memory
    // and TMEM are released
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
