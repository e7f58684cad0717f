// Stage 3 of the block on the tensor cores for c = h = 256 (reference.py:76-83):
// out = sigmoid(Wg . LN_in(z)) * (Wo . LN_out(tri)) [* drop_scale] [+ residual].
//
// Untransposed, D[position][output channel]: the normalised z tile is the K-major A operand of the
// gate projection, the normalised tri tile — [256 channel rows][128 positions], exactly as the
// contraction wrote it — is used AS IT LIES as the MN-major A operand of the output projection, a
// TMEM lane is a position and the epilogue writes row-major output.  The two 256 x 256 weight
// matrices (256 KB) are streamed from L2 through a ring of [128 rows][64 k] slots; a tile is worked
// off in two UNITS (output-channel halves): per unit 128 gate and 128 proj accumulator columns over
// K = 256, 32 UMMAs of 128 x 128 x 16, and the two units' accumulators alternate so the epilogue of
// one overlaps the UMMAs of the other.  Both LayerNorms are applied in place in shared memory
// (LN(x) is rounded to bf16, as the reference does); because that destroys the raw z tile, the
// residual (and the dropout scale) are read from global memory in the epilogue.  The streamed
// weights cannot be halved once, so the epilogue applies the factors 1/2 of the tanh form itself.
//
// One tile (z 64 KB + tri 64 KB) is resident at a time: the next tile is fetched as soon as the
// last UMMA of the current one retires, while its epilogue is still running.
//
// Persistent kernel, one CTA per SM, 608 threads, 128-position tiles (z row r, columns j0..j0+127):
//   warp 0        TMA producer of the tiles
//   warp 1        UMMA issuer
//   warps 2..5    LayerNorm_in, one thread per position, in place in the swizzled z tile
//   warps 6..13   LayerNorm_out in place in the swizzled tri tile: a thread owns 4 positions (8 bytes)
//                 of 32 channel rows; the per-position sums are combined over the 8 lanes that share
//                 the positions by warp shuffles (two passes over the tile: statistics, then normalise)
//   warps 14..17  epilogue, thread = position: TMEM -> gate -> (* scale) (+ residual) -> bf16 ->
//                 swizzled staging box [128 positions][64 channels] -> TMA store
//   warp 18       TMA producer of the weight slots
#pragma once

#include "tm2_sm100.cuh"

namespace trimul {

constexpr int kW2C = 256;
constexpr int kW2Threads = 608;
constexpr int kW2ZBytes = 4 * kT2SubTile;           // z tile: four [128 positions][64 channels] sub-tiles
constexpr int kW2TBytes = 4 * kT2SubTile;           // tri tile: two 128-channel blocks of two [128 rows][64 positions]
constexpr int kW2WSlots = 4;
constexpr int kW2OffT = kW2ZBytes;
constexpr int kW2OffW = kW2OffT + kW2TBytes;
constexpr int kW2OffStaging = kW2OffW + kW2WSlots * kT2SubTile;
constexpr int kW2OffAffine = kW2OffStaging + kT2SubTile;            // gamma_in, beta_in, gamma_out, beta_out (256 each)
constexpr int kW2OffBars = kW2OffAffine + 4 * kW2C * 4;
constexpr int kW2SmemBytes = kW2OffBars + 256;
constexpr int kW2LnBarrier = 2;
constexpr int kW2TriBarrier = 3;
constexpr int kW2EpiBarrier = 4;
constexpr int kW2AffineBarrier = 5;
static_assert(kW2SmemBytes <= 232448, "wide stage 3 shared memory exceeds the 227 KB a CTA may use");

struct Tm2WideParams {
    Tm2Params base;
    const __nv_bfloat16* residual;     // [B, rows, N, 256] or null
    const __nv_bfloat16* drop_scale;   // [B, 1, N, 256] or null
};

__global__ void __launch_bounds__(kW2Threads, 1)
tm2_wide_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWg,
                      const __grid_constant__ CUtensorMap tmWo, const __grid_constant__ CUtensorMap tmOut,
                      const __grid_constant__ CUtensorMap tmTri, const __grid_constant__ Tm2WideParams wp) {
    const Tm2Params& p = wp.base;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm2, 900);
        return;
    }
    uint8_t* sZ = smem;
    uint8_t* sT = smem + kW2OffT;
    uint8_t* sW = smem + kW2OffW;
    uint8_t* sOut = smem + kW2OffStaging;
    float* sAff = reinterpret_cast<float*>(smem + kW2OffAffine);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kW2OffBars);
    uint64_t* t_full = bars;                  // tile (z + tri) landed
    uint64_t* zn_ready = bars + 1;            // z tile normalised (128 arrivals)
    uint64_t* tn_ready = bars + 2;            // tri tile normalised (256 arrivals)
    uint64_t* tile_empty = bars + 3;          // every UMMA that reads the tile has retired
    uint64_t* w_full = bars + 4;              // [slots]
    uint64_t* w_empty = w_full + kW2WSlots;   // [slots]
    uint64_t* acc_full = w_empty + kW2WSlots; // [2]
    uint64_t* acc_empty = acc_full + 2;       // [2] (4 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    static_assert((8 + 2 * kW2WSlots) * 8 + 8 <= 256, "barrier block too small");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(t_full, 1);
        mbar_init(zn_ready, 128);
        mbar_init(tn_ready, 256);
        mbar_init(tile_empty, 1);
        for (int s = 0; s < kW2WSlots; ++s) {
            mbar_init(&w_full[s], 1);
            mbar_init(&w_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        *abort_flag = 0;
        fence_mbarrier_init();
        tma_prefetch_desc(&tmZ);
        tma_prefetch_desc(&tmTri);
        tma_prefetch_desc(&tmOut);
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

    if (warp >= 2 && warp < 14) {
        // the LayerNorm warps bring the four affine vectors into shared memory for themselves
        for (int i = threadIdx.x - 64; i < 4 * kW2C; i += 384) {
            const float* src = i < kW2C ? p.gamma_in : i < 2 * kW2C ? p.beta_in : i < 3 * kW2C ? p.gamma_out : p.beta_out;
            sAff[i] = src[i & (kW2C - 1)];
        }
        named_barrier_sync(kW2AffineBarrier, 384);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ tile producer
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                if (!mbar_wait<true>(tile_empty, (it & 1u) ^ 1u, abort_flag, p.status, kStageIdTm2, 100)) break;
                const int j0 = (tile % p.tiles_per_row) * kT2P;
                const int br = tile / p.tiles_per_row;
                const int r = br % p.rows;
                const int b = br / p.rows;
                mbar_arrive_expect_tx(t_full, kW2ZBytes + kW2TBytes);
                for (int ks = 0; ks < 4; ++ks) tma_load_4d(sZ + ks * kT2SubTile, &tmZ, t_full, ks * 64, j0, r, b);
                // tri planes viewed as (column, row, plane, chunk): 64 columns x 128 planes per box
                for (int kb = 0; kb < 2; ++kb) {
                    tma_load_4d(sT + (kb * 2) * kT2SubTile, &tmTri, t_full, j0, r, b * kW2C + kb * 128, 0);
                    tma_load_4d(sT + (kb * 2 + 1) * kT2SubTile, &tmTri, t_full, j0 + 64, r, b * kW2C + kb * 128, 0);
                }
            }
        }
        __syncwarp();
    } else if (warp == 18) {
        // ------------------------------------------------------------------ weight slot producer
        // per tile and unit (output-channel half): for every K slice the gate slot, then the proj slot
        if (lane == 0) {
            uint32_t cnt = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
                for (int u = 0; ok && u < 2; ++u) {
                    for (int ks = 0; ks < 4; ++ks) {
                        for (int m = 0; m < 2; ++m, ++cnt) {
                            const int s = cnt % kW2WSlots;
                            const uint32_t ph = (cnt / kW2WSlots) & 1u;
                            if (!mbar_wait<true>(&w_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm2, 600 + s)) {
                                ok = false;
                                break;
                            }
                            mbar_arrive_expect_tx(&w_full[s], kT2SubTile);
                            tma_load_2d(sW + s * kT2SubTile, m == 0 ? &tmWg : &tmWo, &w_full[s], ks * 64, u * 128);
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
            constexpr uint32_t idesc = umma_idesc_bf16(kT2P, 128);
            constexpr uint32_t idesc_mn = umma_idesc_bf16(kT2P, 128, 1, 0);   // A (tri_n) is MN-major
            uint32_t it = 0, cnt = 0;
            bool ok = true;
            const uint32_t zs = smem_u32(sZ), ts = smem_u32(sT);
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                if (!mbar_wait<true>(zn_ready, it & 1u, abort_flag, p.status, kStageIdTm2, 210) ||
                    !mbar_wait<true>(tn_ready, it & 1u, abort_flag, p.status, kStageIdTm2, 211))
                    break;
                tcgen05_fence_after();
                for (int u = 0; ok && u < 2; ++u) {
                    // accumulator pair u, used once per tile: use counter = it
                    if (!mbar_wait<true>(&acc_empty[u], (it & 1u) ^ 1u, abort_flag, p.status, kStageIdTm2, 220 + u)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t d_g = tmem_base + u * 256;
                    const uint32_t d_p = d_g + 128;
                    for (int ks = 0; ks < 4; ++ks, cnt += 2) {
                        const int sg = cnt % kW2WSlots, so = (cnt + 1) % kW2WSlots;
                        if (!mbar_wait<true>(&w_full[sg], (cnt / kW2WSlots) & 1u, abort_flag, p.status, kStageIdTm2,
                                             230 + sg) ||
                            !mbar_wait<true>(&w_full[so], ((cnt + 1) / kW2WSlots) & 1u, abort_flag, p.status,
                                             kStageIdTm2, 230 + so)) {
                            ok = false;
                            break;
                        }
                        tcgen05_fence_after();
                        const uint32_t wg = smem_u32(sW + sg * kT2SubTile), wo = smem_u32(sW + so * kT2SubTile);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint64_t kofs = kk * kDescKStep;
                            // gate: z_n sub-tile ks, K-major
                            umma_bf16_ss(d_g, umma_smem_desc_sw128(zs + ks * kT2SubTile) + kofs,
                                         umma_smem_desc_sw128(wg) + kofs, idesc, (ks | kk) != 0);
                            // proj: tri_n block ks >> 1 (two [128 rows][64 positions] sub-tiles, 16 KB apart), channel
                            // rows (ks & 1) * 64 + kk * 16 ..: a K step of 16 rows is two 8-row groups = 2048 B
                            umma_bf16_ss(d_p,
                                         umma_smem_desc_mn_sw128(ts + (ks >> 1) * 2 * kT2SubTile +
                                                                     ((ks & 1) * 4 + kk) * 2048, kT2SubTile, 1024),
                                         umma_smem_desc_sw128(wo) + kofs, idesc_mn, (ks | kk) != 0);
                        }
                        umma_commit(&w_empty[sg]);
                        umma_commit(&w_empty[so]);
                    }
                    if (!ok) break;
                    umma_commit(&acc_full[u]);
                }
                if (!ok) break;
                umma_commit(tile_empty);
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ------------------------------------------------------------------ LayerNorm_in
        const int pos = threadIdx.x - 64;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            if (!group_wait<true>(t_full, it & 1u, pos == 0, kW2LnBarrier, 128, abort_flag, p.status, kStageIdTm2, 300))
                break;
            ln_row_inplace<4>(sZ, kT2SubTile, pos, sAff, sAff + kW2C, p.eps_in, false);
            fence_proxy_async_smem();
            mbar_arrive(zn_ready);
        }
    } else if (warp < 14) {
        // ------------------------------------------------------------------ LayerNorm_out on the tri tile
        // Block kb of the tile is [128 channel rows][128 positions] as two 64-position sub-tiles, 16-byte
        // chunk c of row r at chunk c ^ (r & 7).  Thread (tw, ql, rs): position quad qd = 4 tw + ql
        // (positions 4 qd .. 4 qd + 3, half of chunk qd >> 1), channel rows rs, rs + 8, ... of both
        // blocks.  All its rows have r & 7 == rs, so its 8 bytes sit at the same offset in every row.
        const int tw = warp - 6;
        const int ql = lane >> 3;
        const int rs = lane & 7;
        const int qd = 4 * tw + ql;
        const int cc = qd >> 1;
        const float* sGamma = sAff + 2 * kW2C;
        const float* sBeta = sAff + 3 * kW2C;
        const uint32_t col_off = (uint32_t)(cc >> 3) * kT2SubTile + ((((uint32_t)cc & 7u) ^ (uint32_t)rs) << 4) +
                                 (uint32_t)(qd & 1) * 8u;
        const float inv_c = 1.0f / (float)kW2C;
        uint8_t* base = sT + col_off + rs * 128;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            if (!group_wait<true>(t_full, it & 1u, tw == 0 && lane == 0, kW2TriBarrier, 256, abort_flag, p.status,
                                  kStageIdTm2, 500))
                break;
            // common shift of each position: its channel 0 (block 0, row 0, held by the rs == 0 lane)
            const uint2 v0 = *reinterpret_cast<const uint2*>(base);
            const uint32_t shx = __shfl_sync(0xffffffffu, v0.x, lane & 24);
            const uint32_t shy = __shfl_sync(0xffffffffu, v0.y, lane & 24);
            const float shift[4] = {bf16_lo(shx), bf16_hi(shx), bf16_lo(shy), bf16_hi(shy)};
            const f32x2 nsh01 = f2_pack(-shift[0], -shift[1]), nsh23 = f2_pack(-shift[2], -shift[3]);
            f32x2 a01 = 0ull, a23 = 0ull, q01 = 0ull, q23 = 0ull;
#pragma unroll 1
            for (int kb = 0; kb < 2; ++kb) {
#pragma unroll 8
                for (int m = 0; m < 16; ++m) {
                    const uint2 v = *reinterpret_cast<const uint2*>(base + kb * 2 * kT2SubTile + m * 1024);
                    const f32x2 d01 = f2_add(f2_from_bf16x2(v.x), nsh01);
                    const f32x2 d23 = f2_add(f2_from_bf16x2(v.y), nsh23);
                    a01 = f2_add(a01, d01);
                    q01 = f2_fma(d01, d01, q01);
                    a23 = f2_add(a23, d23);
                    q23 = f2_fma(d23, d23, q23);
                }
            }
            float s1[4], s2[4];
            f2_unpack(a01, s1[0], s1[1]);
            f2_unpack(a23, s1[2], s1[3]);
            f2_unpack(q01, s2[0], s2[1]);
            f2_unpack(q23, s2[2], s2[3]);
            // combine the 8 row slots of a quad (lanes that differ in bits 0..2)
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s1[e] += __shfl_xor_sync(0xffffffffu, s1[e], o);
                    s2[e] += __shfl_xor_sync(0xffffffffu, s2[e], o);
                }
            }
            float rstd[4], nmr[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float m1 = s1[e] * inv_c;
                rstd[e] = rsqrtf(fmaxf(fmaf(-m1, m1, s2[e] * inv_c), 0.f) + p.eps_out);
                nmr[e] = -(shift[e] + m1) * rstd[e];
            }
            const f32x2 r01 = f2_pack(rstd[0], rstd[1]), r23 = f2_pack(rstd[2], rstd[3]);
            const f32x2 n01 = f2_pack(nmr[0], nmr[1]), n23 = f2_pack(nmr[2], nmr[3]);
#pragma unroll 1
            for (int kb = 0; kb < 2; ++kb) {
#pragma unroll 4
                for (int m = 0; m < 16; ++m) {
                    uint2* ptr = reinterpret_cast<uint2*>(base + kb * 2 * kT2SubTile + m * 1024);
                    const uint2 v = *ptr;
                    const float ga = sGamma[kb * 128 + rs + 8 * m], be = sBeta[kb * 128 + rs + 8 * m];
                    const f32x2 ga2 = f2_pack(ga, ga), be2 = f2_pack(be, be);
                    uint2 o;
                    o.x = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v.x), r01, n01), ga2, be2));
                    o.y = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v.y), r23, n23), ga2, be2));
                    *ptr = o;
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(tn_ready);
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;
        const int row = q * 32 + lane;                 // position inside the tile == TMEM lane
        const bool leader = (warp == 14 && lane == 0);
        const uint32_t lane_bits = (uint32_t)(q * 32) << 16;
        uint32_t it = 0;
        bool alive = true;
        for (int tile = blockIdx.x; alive && tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int j0 = (tile % p.tiles_per_row) * kT2P;
            const int br = tile / p.tiles_per_row;
            const int r = br % p.rows;
            const int b = br / p.rows;
            const bool in_range = j0 + row < p.N;
            const size_t out_row = (((size_t)b * p.rows + r) * p.N + j0 + row) * kW2C;
            const size_t ds_rowo = ((size_t)b * p.N + j0 + row) * kW2C;
#pragma unroll 1
            for (int u = 0; u < 2; ++u) {
                if (!group_wait<true>(&acc_full[u], it & 1u, leader, kW2EpiBarrier, 128, abort_flag, p.status, kStageIdTm2,
                                      400 + u)) {
                    alive = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t t_g = tmem_base + u * 256 + lane_bits;     // gate; proj 128 columns on
#pragma unroll 1
                for (int sub = 0; sub < 2; ++sub) {        // 64 output channels per staging box
                    if (leader) tma_store_wait_read<0>();  // the previous store has read the staging box
                    named_barrier_sync(kW2EpiBarrier, 128);
                    const int ch0 = u * 128 + sub * 64;
                    auto emit8 = [&](int c8, const uint32_t (&rg)[8], const uint32_t (&rp)[8]) {
                        uint32_t o[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            o[k] = gate2_full_bf16(__uint_as_float(rp[2 * k]), __uint_as_float(rg[2 * k]),
                                                   __uint_as_float(rp[2 * k + 1]), __uint_as_float(rg[2 * k + 1]));
                        if (wp.drop_scale != nullptr && in_range) {
                            const uint4 dv = __ldg(reinterpret_cast<const uint4*>(wp.drop_scale + ds_rowo + ch0 + c8 * 8));
                            const uint32_t dsw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                o[k] = f2_to_bf16x2(f2_mul(f2_from_bf16x2(o[k]), f2_from_bf16x2(dsw[k])));
                        }
                        if (wp.residual != nullptr && in_range) {
                            const uint4 rv = __ldg(reinterpret_cast<const uint4*>(wp.residual + out_row + ch0 + c8 * 8));
                            const uint32_t res[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                o[k] = f2_to_bf16x2(f2_add(f2_from_bf16x2(o[k]), f2_from_bf16x2(res[k])));
                        }
                        *reinterpret_cast<uint4*>(sOut + row * 128 + ((c8 ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    };
                    uint32_t rgA[8], rpA[8], rgB[8], rpB[8];
                    const uint32_t tg = t_g + sub * 64;
                    tmem_ld_32x8(tg, rgA);
                    tmem_ld_32x8(tg + 128, rpA);
#pragma unroll 1
                    for (int c8 = 0; c8 < 8; c8 += 2) {
                        tmem_ld_wait();
                        tmem_ld_32x8(tg + (c8 + 1) * 8, rgB);
                        tmem_ld_32x8(tg + 128 + (c8 + 1) * 8, rpB);
                        emit8(c8, rgA, rpA);
                        tmem_ld_wait();
                        if (c8 + 2 < 8) {
                            tmem_ld_32x8(tg + (c8 + 2) * 8, rgA);
                            tmem_ld_32x8(tg + 128 + (c8 + 2) * 8, rpA);
                        } else if (sub == 1) {
                            // every TMEM read of this unit's accumulators has completed
                            tcgen05_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&acc_empty[u]);
                        }
                        emit8(c8 + 1, rgB, rpB);
                    }
                    fence_proxy_async_smem();
                    named_barrier_sync(kW2EpiBarrier, 128);
                    if (leader) {
                        tma_store_4d(&tmOut, sOut, ch0, j0, r, b);
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
