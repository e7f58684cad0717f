// Stage 3 of the block on the tensor cores, c = 128: LayerNorm_out over the channels of the
// contraction result, the output projection, the output gate from a fresh LayerNorm_in of z
// (unmasked, reference.py:82-83), optional residual — one pass, row-major bf16 result.
//
// Persistent kernel, one CTA per SM, 704 threads, 128-position tiles (z row r, columns j0..j0+127):
//   warp 0        TMA producer: Wg, Wo once; per tile the z tile [128 positions][128 channels] and
//                 the tri tile [128 channels][128 positions] (channel-major, as the contraction
//                 wrote it), plus the residual tile when asked, into a 2-stage ring
//   warp 1        UMMA issuer: gate = x_n . Wg^T with x_n K-major, proj = tri_n . Wo^T with tri_n
//                 MN-major — the channel-major tile is used as the A operand AS IT LIES, so the
//                 channel-major -> row-major turn of the data costs nothing at all; 128x128x16
//                 each, into a double-buffered pair of 128-column TMEM accumulators
//   warps 2..9    LayerNorm_in: two groups of four warps on alternate tiles, one thread per
//                 position, in place in the swizzled z tile
//   warps 10..17  LayerNorm_out, in place in the swizzled tri tile: a thread owns 4 positions (8
//                 bytes) of 16 channel rows; the per-position sums are combined over the 8 lanes
//                 that share the positions by warp shuffles
//   warps 18..21  epilogue: TMEM -> sigmoid(g) * p (+ residual) -> bf16 -> swizzled staging -> TMA store
// The worker warps first halve Wg and Wo in shared memory (exact in bf16) so that
// p*sigmoid(g) = (p/2)*tanh(g/2) + p/2 costs one MUFU and one FMA.
#pragma once

#include "ptx_sm100.cuh"

namespace trimul {

constexpr int kT2C = 128;
constexpr int kT2P = 128;
constexpr int kT2Threads = 704;
constexpr int kT2LnThreads = 256;       // warps 2..9
constexpr int kT2TriThreads = 256;      // warps 10..17
constexpr int kT2EpiThreads = 128;      // warps 18..21
constexpr int kT2Workers = kT2LnThreads + kT2TriThreads + kT2EpiThreads;
constexpr int kT2SubTile = 128 * 64 * 2;          // 16 KB
constexpr int kT2WBytes = 4 * kT2SubTile;         // Wg, Wo: 2 K halves each
constexpr int kT2XBytes = 2 * kT2SubTile;         // z tile  -> x_n operand
constexpr int kT2TBytes = 2 * kT2SubTile;         // tri tile -> tri_n operand (MN-major)
constexpr int kT2StageBytes = kT2XBytes + kT2TBytes;
constexpr int kT2StagingBytes = 2 * kT2SubTile;   // [128 positions][128 channels] as two 64-wide boxes
constexpr int kT2OffStage = kT2WBytes;
constexpr int kT2OffStaging = kT2OffStage + 2 * kT2StageBytes;
constexpr int kT2OffAffine = kT2OffStaging + kT2StagingBytes;   // gamma_in, beta_in, gamma_out, beta_out
constexpr int kT2OffBars = kT2OffAffine + 4 * kT2C * 4;
constexpr int kT2SmemBytes = kT2OffBars + 192;
constexpr int kT2LnBarrier = 2;
constexpr int kT2TriBarrier = 3;
constexpr int kT2EpiBarrier = 4;
constexpr int kT2LnBarrier2 = 5;        // second LayerNorm_in group
constexpr int kStageIdTm2 = 3;

struct Tm2Params {
    int B, rows, N;
    int tiles_per_row;    // ceil(N / 128)
    int total_tiles;      // B * rows * tiles_per_row
    const float* gamma_in;
    const float* beta_in;
    const float* gamma_out;
    const float* beta_out;
    float eps_in, eps_out;
    int has_residual;
    int32_t* status;
};

__global__ void __launch_bounds__(kT2Threads, 1)
tm2_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWg,
                 const __grid_constant__ CUtensorMap tmWo, const __grid_constant__ CUtensorMap tmOut,
                 const __grid_constant__ CUtensorMap tmRes, const __grid_constant__ CUtensorMap tmTri,
                 const Tm2Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm2, 900);
        return;
    }
    uint8_t* sW = smem;
    uint8_t* sStage = smem + kT2OffStage;
    uint8_t* sOut = smem + kT2OffStaging;
    float* sAff = reinterpret_cast<float*>(smem + kT2OffAffine);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kT2OffBars);
    uint64_t* w_full = bars;            // weights landed
    uint64_t* x_full = bars + 1;        // [2] z tile landed
    uint64_t* xn_ready = bars + 3;      // [2] x_n operand ready (256 arrivals)
    uint64_t* tn_ready = bars + 5;      // [2] tri_n operand ready (256 arrivals)
    uint64_t* s_empty = bars + 7;       // [2] UMMAs that read the stage retired
    uint64_t* acc_full = bars + 9;      // [2]
    uint64_t* acc_empty = bars + 11;    // [2] (4 arrivals)
    uint64_t* res_full = bars + 13;     // residual tile landed in the staging buffer
    uint64_t* out_free = bars + 14;     // staging buffer released by the epilogue (1 arrival)
    uint64_t* w_ready = bars + 15;      // weights halved (all worker threads)
    uint64_t* t_full = bars + 16;       // [2] tri tile landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        mbar_init(w_ready, kT2Workers);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&t_full[s], 1);
            mbar_init(&xn_ready[s], kT2LnThreads / 2);
            mbar_init(&tn_ready[s], kT2TriThreads);
            mbar_init(&s_empty[s], 1);
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        mbar_init(res_full, 1);
        mbar_init(out_free, 1);
        *abort_flag = 0;
        fence_mbarrier_init();
        tma_prefetch_desc(&tmZ);
        tma_prefetch_desc(&tmOut);
        tma_prefetch_desc(&tmTri);
    }
    if (threadIdx.x >= 64 && threadIdx.x < 64 + kT2C) {
        const int i = threadIdx.x - 64;
        sAff[i] = p.gamma_in[i];
        sAff[kT2C + i] = p.beta_in[i];
        sAff[2 * kT2C + i] = p.gamma_out[i];
        sAff[3 * kT2C + i] = p.beta_out[i];
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= 2) {
        if (mbar_wait(w_full, 0, abort_flag, p.status, kStageIdTm2, 150)) {
            halve_bf16_smem(sW, kT2WBytes, threadIdx.x - 64, kT2Workers);
            fence_proxy_async_smem();
        }
        mbar_arrive(w_ready);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, kT2WBytes);
            for (int kh = 0; kh < 2; ++kh) {
                tma_load_2d(sW + kh * kT2SubTile, &tmWg, w_full, kh * 64, 0);
                tma_load_2d(sW + (2 + kh) * kT2SubTile, &tmWo, w_full, kh * 64, 0);
            }
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1u;
                const int j0 = (tile % p.tiles_per_row) * kT2P;
                const int br = tile / p.tiles_per_row;
                const int r = br % p.rows;
                const int b = br / p.rows;
                if (!mbar_wait(&s_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm2, 100 + s)) break;
                TRIMUL_STAMP(0, it, 0);
                mbar_arrive_expect_tx(&x_full[s], kT2XBytes);
                uint8_t* dst = sStage + s * kT2StageBytes;
                tma_load_4d(dst, &tmZ, &x_full[s], 0, j0, r, b);
                tma_load_4d(dst + kT2SubTile, &tmZ, &x_full[s], 64, j0, r, b);
                // tri planes viewed as (column, row, plane, chunk): 64 columns x 128 planes per box
                mbar_arrive_expect_tx(&t_full[s], kT2TBytes);
                tma_load_4d(dst + kT2XBytes, &tmTri, &t_full[s], j0, r, b * kT2C, 0);
                tma_load_4d(dst + kT2XBytes + kT2SubTile, &tmTri, &t_full[s], j0 + 64, r, b * kT2C, 0);
                if (p.has_residual) {
                    // the residual tile is fetched into the output staging buffer once the
                    // epilogue has released it (its previous store has finished reading it)
                    if (!mbar_wait(out_free, (it & 1u) ^ 1u, abort_flag, p.status, kStageIdTm2, 110)) break;
                    mbar_arrive_expect_tx(res_full, kT2StagingBytes);
                    tma_load_4d(sOut, &tmRes, res_full, 0, j0, r, b);
                    tma_load_4d(sOut + kT2SubTile, &tmRes, res_full, 64, j0, r, b);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(kT2P, kT2C);
            constexpr uint32_t idesc_mn = umma_idesc_bf16(kT2P, kT2C, 1, 0);   // A (tri_n) is MN-major
            bool ok = mbar_wait(w_ready, 0, abort_flag, p.status, kStageIdTm2, 200);
            tcgen05_fence_after();
            uint32_t it = 0;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1u;
                // accumulator pair `s` was last used by tile it-2
                if (!mbar_wait(&acc_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm2, 210 + s)) break;
                if (!mbar_wait(&xn_ready[s], ph, abort_flag, p.status, kStageIdTm2, 220 + s)) break;
                if (!mbar_wait(&tn_ready[s], ph, abort_flag, p.status, kStageIdTm2, 230 + s)) break;
                tcgen05_fence_after();
                TRIMUL_STAMP(2, it, 0);
                const uint32_t xs = smem_u32(sStage + s * kT2StageBytes);
                const uint32_t ts = xs + kT2XBytes;
                const uint32_t wg = smem_u32(sW);
                const uint32_t wo = wg + 2 * kT2SubTile;
                const uint32_t d_g = tmem_base + s * 256;
                const uint32_t d_p = d_g + 128;
#pragma unroll
                for (int kk = 0; kk < kT2C / 16; ++kk) {
                    const uint32_t sub = (kk >> 2) * kT2SubTile;
                    const uint64_t kofs = (kk & 3) * kDescKStep;
                    umma_bf16_ss(d_g, umma_smem_desc_sw128(xs + sub) + kofs, umma_smem_desc_sw128(wg + sub) + kofs,
                                 idesc, kk != 0);
                    // tri_n tile: rows are channels (K), 128 bytes = 64 positions per row, the second
                    // 64 positions one sub-tile further; a K step of 16 is two 8-row groups = 2048 B
                    umma_bf16_ss(d_p, umma_smem_desc_mn_sw128(ts + kk * 2048, kT2SubTile, 1024),
                                 umma_smem_desc_sw128(wo + sub) + kofs, idesc_mn, kk != 0);
                }
                umma_commit(&s_empty[s]);
                umma_commit(&acc_full[s]);
            }
        }
        __syncwarp();
    } else if (warp < 10) {
        // ------------------------------------------------------------------ LayerNorm_in, in place
        // two groups of four warps; group g takes the tiles in stage g; one thread per position
        const int g = (warp - 2) >> 2;
        const int pos = threadIdx.x - 64 - g * 128;
        const int bar_id = g == 0 ? kT2LnBarrier : kT2LnBarrier2;
        uint32_t it = g;
        for (int tile = blockIdx.x + g * gridDim.x; tile < p.total_tiles; tile += 2 * gridDim.x, it += 2) {
            const uint32_t ph = (it >> 1) & 1u;
            if (!group_wait(&x_full[g], ph, pos == 0, bar_id, 128, abort_flag, p.status, kStageIdTm2, 300 + g)) break;
            if (pos == 0) TRIMUL_STAMP(1, it, 0);
            ln_row_inplace(sStage + g * kT2StageBytes, kT2SubTile, pos, sAff, sAff + kT2C, p.eps_in, false);
            fence_proxy_async_smem();
            if (pos == 0) TRIMUL_STAMP(1, it, 1);
            mbar_arrive(&xn_ready[g]);
        }
    } else if (warp < 18) {
        // ------------------------------------------------------------------ LayerNorm_out, in place
        // The tile is [128 channel rows][128 positions] as two 64-position sub-tiles, 16-byte chunk c
        // of row r stored at chunk c ^ (r & 7).  Thread (w, ql, rs) of the group: position quad
        // qd = 4w + ql (positions 4qd .. 4qd+3, half of chunk qd >> 1), channel rows rs, rs+8, ...,
        // rs+120.  All its rows have r & 7 == rs, so its 8 bytes sit at the same offset in every row.
        const int tw = warp - 10;
        const int ql = lane >> 3;
        const int rs = lane & 7;
        const int qd = 4 * tw + ql;
        const int cc = qd >> 1;
        const float* sGamma = sAff + 2 * kT2C;
        const float* sBeta = sAff + 3 * kT2C;
        const uint32_t col_off = (uint32_t)(cc >> 3) * kT2SubTile + ((((uint32_t)cc & 7u) ^ (uint32_t)rs) << 4) +
                                 (uint32_t)(qd & 1) * 8u;
        const float inv_c = 1.0f / (float)kT2C;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it & 1;
            const uint32_t ph = (it >> 1) & 1u;
            if (!group_wait(&t_full[s], ph, tw == 0 && lane == 0, kT2TriBarrier, kT2TriThreads, abort_flag, p.status,
                            kStageIdTm2, 500 + s))
                break;
            if (tw == 0 && lane == 0) TRIMUL_STAMP(3, it, 0);
            uint8_t* base = sStage + s * kT2StageBytes + kT2XBytes + col_off + rs * 128;
            uint2 v[16];
#pragma unroll
            for (int m = 0; m < 16; ++m) v[m] = *reinterpret_cast<const uint2*>(base + m * 1024);
            // common shift of each position: its channel 0 (row 0, held by the rs == 0 lane)
            const uint32_t shx = __shfl_sync(0xffffffffu, v[0].x, lane & 24);
            const uint32_t shy = __shfl_sync(0xffffffffu, v[0].y, lane & 24);
            const float shift[4] = {bf16_lo(shx), bf16_hi(shx), bf16_lo(shy), bf16_hi(shy)};
            // positions (0,1) and (2,3) of the quad as packed fp32 pairs
            const f32x2 nsh01 = f2_pack(-shift[0], -shift[1]), nsh23 = f2_pack(-shift[2], -shift[3]);
            f32x2 a01 = 0ull, a23 = 0ull, q01 = 0ull, q23 = 0ull;
#pragma unroll
            for (int m = 0; m < 16; ++m) {
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
            if (tw == 0 && lane == 0) TRIMUL_STAMP(3, it, 1);
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                const float ga = sGamma[rs + 8 * m], be = sBeta[rs + 8 * m];
                const f32x2 ga2 = f2_pack(ga, ga), be2 = f2_pack(be, be);
                uint2 o;
                o.x = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v[m].x), r01, n01), ga2, be2));
                o.y = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v[m].y), r23, n23), ga2, be2));
                *reinterpret_cast<uint2*>(base + m * 1024) = o;
            }
            fence_proxy_async_smem();
            if (tw == 0 && lane == 0) TRIMUL_STAMP(3, it, 2);
            mbar_arrive(&tn_ready[s]);
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;
        const int row = q * 32 + lane;                 // position inside the tile == TMEM lane
        const bool leader = (warp == 18 && lane == 0);
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it & 1;
            const uint32_t ph = (it >> 1) & 1u;
            const int j0 = (tile % p.tiles_per_row) * kT2P;
            const int br = tile / p.tiles_per_row;
            const int r = br % p.rows;
            const int b = br / p.rows;
            bool ok = true;
            if (leader) {
                ok = mbar_wait(&acc_full[s], ph, abort_flag, p.status, kStageIdTm2, 400 + s);
                if (ok && p.has_residual) ok = mbar_wait(res_full, it & 1u, abort_flag, p.status, kStageIdTm2, 410);
            }
            if (!named_barrier_all(kT2EpiBarrier, kT2EpiThreads, ok)) break;
            tcgen05_fence_after();
            if (leader) TRIMUL_STAMP(5, it, 0);
            // The staging tile is two 64-channel boxes, each stored (and committed) on its own.  Before
            // a box is rewritten only ITS previous store must have finished reading it; the other
            // box's store, issued later, may still be in flight (at most one group pending).
            if (!p.has_residual) {
                if (leader) tma_store_wait_read<1>();
                named_barrier_sync(kT2EpiBarrier, kT2EpiThreads);
            }
            if (leader) TRIMUL_STAMP(5, it, 2);
            const uint32_t t_g = tmem_base + s * 256 + ((uint32_t)(q * 32) << 16);
            // 16 output channels at a time; the TMEM loads of the next 16 are in flight while the
            // current 16 are gated, rounded and written to the staging tile
            auto emit16 = [&](int c16, const uint32_t (&rg)[16], const uint32_t (&rp)[16]) {
                uint8_t* base = sOut + (c16 >> 2) * kT2SubTile + row * 128;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int chunk = ((c16 & 3) * 2 + cc) ^ (row & 7);
                    uint4* dst = reinterpret_cast<uint4*>(base + (chunk << 4));
                    uint32_t res[4] = {0u, 0u, 0u, 0u};
                    if (p.has_residual) {
                        const uint4 rv = *dst;
                        res[0] = rv.x; res[1] = rv.y; res[2] = rv.z; res[3] = rv.w;
                    }
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i0 = cc * 8 + 2 * e;
                        o[e] = gate2_bf16(__uint_as_float(rp[i0]), __uint_as_float(rg[i0]),
                                          __uint_as_float(rp[i0 + 1]), __uint_as_float(rg[i0 + 1]));
                        if (p.has_residual)   // the reference rounds the block output to bf16 before `out + pair`
                            o[e] = f2_to_bf16x2(f2_add(f2_from_bf16x2(o[e]), f2_from_bf16x2(res[e])));
                    }
                    *dst = make_uint4(o[0], o[1], o[2], o[3]);
                }
            };
            uint32_t rgA[16], rpA[16], rgB[16], rpB[16];
            tmem_ld_32x16(t_g, rgA);
            tmem_ld_32x16(t_g + 128, rpA);
#pragma unroll 1
            for (int c16 = 0; c16 < 8; c16 += 2) {
                if (c16 == 4) {
                    if (leader) TRIMUL_STAMP(5, it, 3);
                    // box 0 (channels 0..63) is complete: store it, then make sure box 1 is free
                    fence_proxy_async_smem();
                    named_barrier_sync(kT2EpiBarrier, kT2EpiThreads);
                    if (leader && !p.has_residual) {
                        tma_store_4d(&tmOut, sOut, 0, j0, r, b);
                        tma_store_commit();
                        tma_store_wait_read<1>();
                    }
                    named_barrier_sync(kT2EpiBarrier, kT2EpiThreads);
                }
                tmem_ld_wait();
                tmem_ld_32x16(t_g + (c16 + 1) * 16, rgB);
                tmem_ld_32x16(t_g + 128 + (c16 + 1) * 16, rpB);
                emit16(c16, rgA, rpA);
                tmem_ld_wait();
                if (c16 + 2 < 8) {
                    tmem_ld_32x16(t_g + (c16 + 2) * 16, rgA);
                    tmem_ld_32x16(t_g + 128 + (c16 + 2) * 16, rpA);
                } else {
                    // every TMEM read of this accumulator pair has completed: hand it back early
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[s]);
                }
                emit16(c16 + 1, rgB, rpB);
            }
            if (leader) TRIMUL_STAMP(5, it, 1);
            fence_proxy_async_smem();
            named_barrier_sync(kT2EpiBarrier, kT2EpiThreads);
            if (leader) {
                if (p.has_residual) tma_store_4d(&tmOut, sOut, 0, j0, r, b);
                tma_store_4d(&tmOut, sOut + kT2SubTile, 64, j0, r, b);
                tma_store_commit();
                if (p.has_residual) {
                    tma_store_wait_read<0>();
                    mbar_arrive(out_free);   // the producer may fetch the next residual tile
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
