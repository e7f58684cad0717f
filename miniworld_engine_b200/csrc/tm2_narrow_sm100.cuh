// Stage 3 of the block on the tensor cores for c = h = 64 (reference.py:76-83):
// out = sigmoid(Wg . LN_in(z)) * (Wo . LN_out(tri)) [* drop_scale] [+ residual].
//
// Untransposed, D[position][output channel], like the other stage-3 kernels: the normalised z tile
// is the K-major A operand of the gate projection, the normalised tri tile — [64 channel rows]
// [128 positions], as the contraction wrote it — the MN-major A operand of the output projection,
// a TMEM lane is a position and the epilogue writes row-major output.  Both 64 x 64 weight matrices
// stay in shared memory (halved once, exact in bf16, for the tanh form of the gate); both LayerNorms
// are applied in place in shared memory (LN(x) rounded to bf16, as the reference does), which destroys
// the raw z tile: the residual tile is TMA-loaded into the staging box the result is about to be
// written to, the (small, L2-resident) dropout scale is read from global memory in the epilogue.  A tile is 8 UMMAs of
// 128 x 64 x 16 into 2 x 64 TMEM columns, accumulators double-buffered, three (z, tri) tile pairs in
// flight.
//
// Persistent kernel, one CTA per SM, 576 threads, 128-position tiles (z row r, columns j0..j0+127):
//   warp 0        TMA producer: the weights once, then the tiles
//   warp 1        UMMA issuer
//   warps 2..5    LayerNorm_in, one thread per position, in place in the swizzled z tile
//   warps 6..13   LayerNorm_out in place in the swizzled tri tile: a thread owns 4 positions (8 bytes)
//                 of 8 channel rows; sums combined over the 8 lanes that share the positions
//   warps 14..17  epilogue, thread = position: TMEM -> gate -> (* scale) (+ residual) -> bf16 ->
//                 swizzled staging box [128 positions][64 channels] -> TMA store
#pragma once

#include "tm2_sm100.cuh"

namespace trimul {

constexpr int kN2C = 64;
constexpr int kN2Threads = 576;
constexpr int kN2ZBytes = kT2SubTile;               // [128 positions][64 channels]
constexpr int kN2TBytes = kT2SubTile;               // [64 channel rows][128 positions] as two 8 KB halves
constexpr int kN2Stages = 3;
constexpr int kN2StageBytes = kN2ZBytes + kN2TBytes;
constexpr int kN2WBytes = 2 * 8192;                 // Wg, Wo: [64 rows][64 k] each
constexpr int kN2OffStage = kN2WBytes;
constexpr int kN2OffStaging = kN2OffStage + kN2Stages * kN2StageBytes;
constexpr int kN2OffAffine = kN2OffStaging + 2 * kT2SubTile;
constexpr int kN2OffBars = kN2OffAffine + 4 * kN2C * 4;
constexpr int kN2SmemBytes = kN2OffBars + 256;
constexpr int kN2LnBarrier = 2;
constexpr int kN2TriBarrier = 3;
constexpr int kN2EpiBarrier = 4;
constexpr int kN2AffineBarrier = 5;

struct Tm2NarrowParams {
    Tm2Params base;
    const __nv_bfloat16* residual;     // [B, rows, N, 64] or null
    const __nv_bfloat16* drop_scale;   // [B, 1, N, 64] or null
};

__global__ void __launch_bounds__(kN2Threads, 1)
tm2_narrow_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWg,
                        const __grid_constant__ CUtensorMap tmWo, const __grid_constant__ CUtensorMap tmOut,
                        const __grid_constant__ CUtensorMap tmTri, const __grid_constant__ CUtensorMap tmRes,
                        const __grid_constant__ Tm2NarrowParams np) {
    const Tm2Params& p = np.base;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm2, 900);
        return;
    }
    uint8_t* sW = smem;                       // Wg at 0, Wo at 8 KB
    uint8_t* sStage = smem + kN2OffStage;     // per stage: z tile, then tri tile
    uint8_t* sOut = smem + kN2OffStaging;
    float* sAff = reinterpret_cast<float*>(smem + kN2OffAffine);   // gamma_in, beta_in, gamma_out, beta_out
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kN2OffBars);
    uint64_t* w_full = bars;
    uint64_t* w_ready = bars + 1;                     // weights halved (512 arrivals)
    uint64_t* t_full = bars + 2;                      // [stages] z + tri landed
    uint64_t* zn_ready = t_full + kN2Stages;          // [stages] (128 arrivals)
    uint64_t* tn_ready = zn_ready + kN2Stages;        // [stages] (256 arrivals)
    uint64_t* tile_empty = tn_ready + kN2Stages;      // [stages]
    uint64_t* acc_full = tile_empty + kN2Stages;      // [2]
    uint64_t* acc_empty = acc_full + 2;               // [2] (4 arrivals)
    uint64_t* res_full = acc_empty + 2;               // [2] residual tile landed in the staging box
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(res_full + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    static_assert((8 + 4 * kN2Stages) * 8 + 8 <= 256, "barrier block too small");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        mbar_init(w_ready, kN2Threads - 64);
        for (int s = 0; s < kN2Stages; ++s) {
            mbar_init(&t_full[s], 1);
            mbar_init(&zn_ready[s], 128);
            mbar_init(&tn_ready[s], 256);
            mbar_init(&tile_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
            mbar_init(&res_full[s], 1);
        }
        *abort_flag = 0;
        fence_mbarrier_init();
        tma_prefetch_desc(&tmZ);
        tma_prefetch_desc(&tmTri);
        tma_prefetch_desc(&tmOut);
        tma_prefetch_desc(&tmRes);
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
        if (threadIdx.x - 64 < 4 * kN2C) {
            const int i = threadIdx.x - 64;
            const float* src = i < kN2C ? p.gamma_in : i < 2 * kN2C ? p.beta_in : i < 3 * kN2C ? p.gamma_out : p.beta_out;
            sAff[i] = src[i & (kN2C - 1)];
        }
        named_barrier_sync(kN2AffineBarrier, 384);
    }
    if (warp >= 2) {
        if (mbar_wait<true>(w_full, 0, abort_flag, p.status, kStageIdTm2, 150)) {
            halve_bf16_smem(sW, kN2WBytes, threadIdx.x - 64, kN2Threads - 64);
            fence_proxy_async_smem();
        }
        mbar_arrive(w_ready);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, kN2WBytes);
            tma_load_2d(sW, &tmWg, w_full, 0, 0);
            tma_load_2d(sW + 8192, &tmWo, w_full, 0, 0);
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it % kN2Stages;
                const uint32_t ph = (it / kN2Stages) & 1u;
                if (!mbar_wait<true>(&tile_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm2, 100 + s)) break;
                const int j0 = (tile % p.tiles_per_row) * kT2P;
                const int br = tile / p.tiles_per_row;
                const int r = br % p.rows;
                const int b = br / p.rows;
                uint8_t* dz = sStage + s * kN2StageBytes;
                mbar_arrive_expect_tx(&t_full[s], kN2StageBytes);
                tma_load_4d(dz, &tmZ, &t_full[s], 0, j0, r, b);
                // tri planes viewed as (column, row, plane, chunk): 64 columns x 64 planes per box
                tma_load_4d(dz + kN2ZBytes, &tmTri, &t_full[s], j0, r, b * kN2C, 0);
                tma_load_4d(dz + kN2ZBytes + 8192, &tmTri, &t_full[s], j0 + 64, r, b * kN2C, 0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(kT2P, kN2C);
            constexpr uint32_t idesc_mn = umma_idesc_bf16(kT2P, kN2C, 1, 0);   // A (tri_n) is MN-major
            bool ok = mbar_wait<true>(w_ready, 0, abort_flag, p.status, kStageIdTm2, 200);
            tcgen05_fence_after();
            const uint32_t wg = smem_u32(sW), wo = smem_u32(sW + 8192);
            uint32_t it = 0;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it % kN2Stages;
                const uint32_t ph = (it / kN2Stages) & 1u;
                const int acc = it & 1;
                if (!mbar_wait<true>(&zn_ready[s], ph, abort_flag, p.status, kStageIdTm2, 210 + s) ||
                    !mbar_wait<true>(&tn_ready[s], ph, abort_flag, p.status, kStageIdTm2, 215 + s) ||
                    !mbar_wait<true>(&acc_empty[acc], ((it >> 1) & 1u) ^ 1u, abort_flag, p.status, kStageIdTm2, 220 + acc))
                    break;
                tcgen05_fence_after();
                const uint32_t zs = smem_u32(sStage + s * kN2StageBytes), ts = zs + kN2ZBytes;
                const uint32_t d_g = tmem_base + acc * 128, d_p = d_g + 64;
#pragma unroll
                for (int kk = 0; kk < kN2C / 16; ++kk) {
                    const uint64_t kofs = kk * kDescKStep;
                    umma_bf16_ss(d_g, umma_smem_desc_sw128(zs) + kofs, umma_smem_desc_sw128(wg) + kofs, idesc, kk != 0);
                    // tri_n: rows are channels (K), 128 bytes = 64 positions per row, the second 64
                    // positions 8 KB further; a K step of 16 rows is two 8-row groups = 2048 B
                    umma_bf16_ss(d_p, umma_smem_desc_mn_sw128(ts + kk * 2048, 8192, 1024),
                                 umma_smem_desc_sw128(wo) + kofs, idesc_mn, kk != 0);
                }
                umma_commit(&acc_full[acc]);
                umma_commit(&tile_empty[s]);
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ------------------------------------------------------------------ LayerNorm_in
        const int pos = threadIdx.x - 64;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it % kN2Stages;
            if (!group_wait<true>(&t_full[s], (it / kN2Stages) & 1u, pos == 0, kN2LnBarrier, 128, abort_flag, p.status,
                                  kStageIdTm2, 300 + s))
                break;
            ln_row_inplace<1>(sStage + s * kN2StageBytes, kT2SubTile, pos, sAff, sAff + kN2C, p.eps_in, false);
            fence_proxy_async_smem();
            mbar_arrive(&zn_ready[s]);
        }
    } else if (warp < 14) {
        // ------------------------------------------------------------------ LayerNorm_out on the tri tile
        // The tile is [64 channel rows][128 positions] as two 64-position halves (8 KB apart), 16-byte
        // chunk c of row r at chunk c ^ (r & 7).  Thread (tw, ql, rs): position quad qd = 4 tw + ql,
        // channel rows rs, rs + 8, ..., rs + 56; all its rows have r & 7 == rs.
        const int tw = warp - 6;
        const int ql = lane >> 3;
        const int rs = lane & 7;
        const int qd = 4 * tw + ql;
        const int cc = qd >> 1;
        const float* sGamma = sAff + 2 * kN2C;
        const float* sBeta = sAff + 3 * kN2C;
        const uint32_t col_off = (uint32_t)(cc >> 3) * 8192u + ((((uint32_t)cc & 7u) ^ (uint32_t)rs) << 4) +
                                 (uint32_t)(qd & 1) * 8u;
        const float inv_c = 1.0f / (float)kN2C;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it % kN2Stages;
            if (!group_wait<true>(&t_full[s], (it / kN2Stages) & 1u, tw == 0 && lane == 0, kN2TriBarrier, 256, abort_flag,
                                  p.status, kStageIdTm2, 500 + s))
                break;
            uint8_t* base = sStage + s * kN2StageBytes + kN2ZBytes + col_off + rs * 128;
            uint2 v[8];
#pragma unroll
            for (int m = 0; m < 8; ++m) v[m] = *reinterpret_cast<const uint2*>(base + m * 1024);
            const uint32_t shx = __shfl_sync(0xffffffffu, v[0].x, lane & 24);
            const uint32_t shy = __shfl_sync(0xffffffffu, v[0].y, lane & 24);
            const float shift[4] = {bf16_lo(shx), bf16_hi(shx), bf16_lo(shy), bf16_hi(shy)};
            const f32x2 nsh01 = f2_pack(-shift[0], -shift[1]), nsh23 = f2_pack(-shift[2], -shift[3]);
            f32x2 a01 = 0ull, a23 = 0ull, q01 = 0ull, q23 = 0ull;
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                const f32x2 d01 = f2_add(f2_from_bf16x2(v[m].x), nsh01);
                const f32x2 d23 = f2_add(f2_from_bf16x2(v[m].y), nsh23);
                a01 = f2_add(a01, d01);
                q01 = f2_fma(d01, d01, q01);
                a23 = f2_add(a23, d23);
                q23 = f2_fma(d23, d23, q23);
            }
            float s1[4], s2[4];
            f2_unpack(a01, s1[0], s1[1]);
            f2_unpack(a23, s1[2], s1[3]);
            f2_unpack(q01, s2[0], s2[1]);
            f2_unpack(q23, s2[2], s2[3]);
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
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                const float ga = sGamma[rs + 8 * m], be = sBeta[rs + 8 * m];
                const f32x2 ga2 = f2_pack(ga, ga), be2 = f2_pack(be, be);
                uint2 o;
                o.x = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v[m].x), r01, n01), ga2, be2));
                o.y = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v[m].y), r23, n23), ga2, be2));
                *reinterpret_cast<uint2*>(base + m * 1024) = o;
            }
            fence_proxy_async_smem();
            mbar_arrive(&tn_ready[s]);
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;
        const int row = q * 32 + lane;                 // position inside the tile == TMEM lane
        const bool leader = (warp == 14 && lane == 0);
        const uint32_t lane_bits = (uint32_t)(q * 32) << 16;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const int j0 = (tile % p.tiles_per_row) * kT2P;
            const int br = tile / p.tiles_per_row;
            const int r = br % p.rows;
            const int b = br / p.rows;
            const bool in_range = j0 + row < p.N;
            const size_t ds_rowo = ((size_t)b * p.N + j0 + row) * kN2C;
            uint8_t* stg = sOut + acc * kT2SubTile;
            bool ok = true;
            if (leader) {
                tma_store_wait_read<1>();              // the store two tiles ago has read this staging box
                if (np.residual != nullptr) {          // the residual tile goes where the result will be written
                    mbar_arrive_expect_tx(&res_full[acc], kT2SubTile);
                    tma_load_4d(stg, &tmRes, &res_full[acc], 0, j0, r, b);
                }
                ok = mbar_wait<true>(&acc_full[acc], (it >> 1) & 1u, abort_flag, p.status, kStageIdTm2, 400 + acc);
                if (ok && np.residual != nullptr)
                    ok = mbar_wait<true>(&res_full[acc], (it >> 1) & 1u, abort_flag, p.status, kStageIdTm2, 410 + acc);
            }
            if (!named_barrier_all(kN2EpiBarrier, 128, ok)) break;
            tcgen05_fence_after();
            const uint32_t t_g = tmem_base + acc * 128 + lane_bits;     // gate; proj 64 columns on
            auto emit8 = [&](int c8, const uint32_t (&rg)[8], const uint32_t (&rp)[8]) {
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    o[k] = gate2_bf16(__uint_as_float(rp[2 * k]), __uint_as_float(rg[2 * k]),
                                      __uint_as_float(rp[2 * k + 1]), __uint_as_float(rg[2 * k + 1]));
                if (np.drop_scale != nullptr && in_range) {
                    const uint4 dv = __ldg(reinterpret_cast<const uint4*>(np.drop_scale + ds_rowo + c8 * 8));
                    const uint32_t dsw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        o[k] = f2_to_bf16x2(f2_mul(f2_from_bf16x2(o[k]), f2_from_bf16x2(dsw[k])));
                }
                uint4* dst = reinterpret_cast<uint4*>(stg + row * 128 + ((c8 ^ (row & 7)) << 4));
                if (np.residual != nullptr) {
                    const uint4 rv = *dst;
                    const uint32_t res[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        o[k] = f2_to_bf16x2(f2_add(f2_from_bf16x2(o[k]), f2_from_bf16x2(res[k])));
                }
                *dst = make_uint4(o[0], o[1], o[2], o[3]);
            };
            uint32_t rgA[8], rpA[8], rgB[8], rpB[8];
            tmem_ld_32x8(t_g, rgA);
            tmem_ld_32x8(t_g + 64, rpA);
#pragma unroll 1
            for (int c8 = 0; c8 < 8; c8 += 2) {
                tmem_ld_wait();
                tmem_ld_32x8(t_g + (c8 + 1) * 8, rgB);
                tmem_ld_32x8(t_g + 64 + (c8 + 1) * 8, rpB);
                emit8(c8, rgA, rpA);
                tmem_ld_wait();
                if (c8 + 2 < 8) {
                    tmem_ld_32x8(t_g + (c8 + 2) * 8, rgA);
                    tmem_ld_32x8(t_g + 64 + (c8 + 2) * 8, rpA);
                } else {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[acc]);
                }
                emit8(c8 + 1, rgB, rpB);
            }
            fence_proxy_async_smem();
            named_barrier_sync(kN2EpiBarrier, 128);
            if (leader) {
                tma_store_4d(&tmOut, stg, 0, j0, r, b);
                tma_store_commit();
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
