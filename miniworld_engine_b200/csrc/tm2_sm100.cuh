// Stage 3 of the block on the tensor cores, c = 128: LayerNorm_out over the channels of the
// contraction result, the output projection, the output gate from a fresh LayerNorm_in of z
// (unmasked, reference.py:82-83), optional residual — one pass, row-major bf16 result.
//
// Persistent kernel, one CTA per SM, 448 threads, 128-position tiles (z row r, columns j0..j0+127):
//   warp 0        TMA producer: Wg, Wo once; z tiles (and residual tiles) into a 2-stage ring
//   warp 1        UMMA issuer: gate = x_n . Wg^T and proj = tri_n . Wo^T, 128x128x16 each, into a
//                 double-buffered pair of 128-column TMEM accumulators (TMEM lane = position)
//   warps 2..5    LayerNorm_in: one thread per position, in place in the swizzled z tile
//   warps 6..9    LayerNorm_out: read tri straight from global memory along the contiguous
//                 position axis of each channel plane (coalesced 4-byte pairs), keep the 64x2
//                 values in registers, normalise, and write them TRANSPOSED into the K-major
//                 swizzled operand tile — the channel-major -> row-major turn costs no extra pass
//   warps 10..13  epilogue: TMEM -> sigmoid(g) * p (+ residual) -> bf16 -> swizzled staging -> TMA store
#pragma once

#include "ptx_sm100.cuh"

namespace trimul {

constexpr int kT2C = 128;
constexpr int kT2P = 128;
constexpr int kT2Threads = 448;
constexpr int kT2SubTile = 128 * 64 * 2;          // 16 KB
constexpr int kT2WBytes = 4 * kT2SubTile;         // Wg, Wo: 2 K halves each
constexpr int kT2XBytes = 2 * kT2SubTile;         // z tile  -> x_n operand
constexpr int kT2TBytes = 2 * kT2SubTile;         // tri_n operand
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
constexpr int kStageIdTm2 = 3;

struct Tm2Params {
    int B, rows, N;
    int tiles_per_row;    // ceil(N / 128)
    int total_tiles;      // B * rows * tiles_per_row
    const __nv_bfloat16* tri;   // planes [B*128][rows][pitch]
    long long tri_pitch, tri_plane_stride;
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
                 const __grid_constant__ CUtensorMap tmRes, const Tm2Params p) {
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
    uint64_t* xn_ready = bars + 3;      // [2] x_n operand ready (128 arrivals)
    uint64_t* tn_ready = bars + 5;      // [2] tri_n operand ready (128 arrivals)
    uint64_t* s_empty = bars + 7;       // [2] UMMAs that read the stage retired
    uint64_t* acc_full = bars + 9;      // [2]
    uint64_t* acc_empty = bars + 11;    // [2] (4 arrivals)
    uint64_t* res_full = bars + 13;     // residual tile landed in the staging buffer
    uint64_t* out_free = bars + 14;     // staging buffer released by the epilogue (1 arrival)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&xn_ready[s], 128);
            mbar_init(&tn_ready[s], 128);
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
                mbar_arrive_expect_tx(&x_full[s], kT2XBytes);
                uint8_t* dst = sStage + s * kT2StageBytes;
                tma_load_4d(dst, &tmZ, &x_full[s], 0, j0, r, b);
                tma_load_4d(dst + kT2SubTile, &tmZ, &x_full[s], 64, j0, r, b);
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
            bool ok = mbar_wait(w_full, 0, abort_flag, p.status, kStageIdTm2, 200);
            uint32_t it = 0;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1u;
                // accumulator pair `s` was last used by tile it-2
                if (!mbar_wait(&acc_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm2, 210 + s)) break;
                if (!mbar_wait(&xn_ready[s], ph, abort_flag, p.status, kStageIdTm2, 220 + s)) break;
                if (!mbar_wait(&tn_ready[s], ph, abort_flag, p.status, kStageIdTm2, 230 + s)) break;
                tcgen05_fence_after();
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
                    umma_bf16_ss(d_p, umma_smem_desc_sw128(ts + sub) + kofs, umma_smem_desc_sw128(wo + sub) + kofs,
                                 idesc, kk != 0);
                }
                umma_commit(&s_empty[s]);
                umma_commit(&acc_full[s]);
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ------------------------------------------------------------------ LayerNorm_in, in place
        const int pos = threadIdx.x - 64;
        const float inv_c = 1.0f / (float)kT2C;
        const float* sGamma = sAff;
        const float* sBeta = sAff + kT2C;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it & 1;
            const uint32_t ph = (it >> 1) & 1u;
            bool ok = mbar_wait(&x_full[s], ph, abort_flag, p.status, kStageIdTm2, 300 + s);
            ok = named_barrier_all(kT2LnBarrier, 128, ok);
            if (!ok) break;
            uint8_t* xrow = sStage + s * kT2StageBytes + pos * 128;
            uint4 v[16];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    v[h * 8 + j] = *reinterpret_cast<const uint4*>(xrow + h * kT2SubTile + ((j ^ (pos & 7)) << 4));
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                sum += bf16_lo(v[i].x) + bf16_hi(v[i].x) + bf16_lo(v[i].y) + bf16_hi(v[i].y);
                sum += bf16_lo(v[i].z) + bf16_hi(v[i].z) + bf16_lo(v[i].w) + bf16_hi(v[i].w);
            }
            const float mean = sum * inv_c;
            float sq = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float d0 = bf16_lo(w4[e]) - mean, d1 = bf16_hi(w4[e]) - mean;
                    sq = fmaf(d0, d0, sq);
                    sq = fmaf(d1, d1, sq);
                }
            }
            const float rstd = rsqrtf(sq * inv_c + p.eps_in);
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = h * 8 + j;
                    const int ch = h * 64 + j * 8;
                    const uint32_t w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
                    uint32_t o4[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float y0 = fmaf((bf16_lo(w4[e]) - mean) * rstd, sGamma[ch + 2 * e], sBeta[ch + 2 * e]);
                        const float y1 =
                            fmaf((bf16_hi(w4[e]) - mean) * rstd, sGamma[ch + 2 * e + 1], sBeta[ch + 2 * e + 1]);
                        o4[e] = pack_bf16x2(y0, y1);
                    }
                    *reinterpret_cast<uint4*>(xrow + h * kT2SubTile + ((j ^ (pos & 7)) << 4)) =
                        make_uint4(o4[0], o4[1], o4[2], o4[3]);
                }
            fence_proxy_async_smem();
            mbar_arrive(&xn_ready[s]);
        }
    } else if (warp < 10) {
        // ------------------------------------------------------------------ LayerNorm_out + transpose
        // lane l of warp w: positions 2*pp, 2*pp+1 with pp = 16*w + (l & 15); channel half h = l >> 4
        const int tw = warp - 6;
        const int pp = tw * 16 + (lane & 15);
        const int h = lane >> 4;
        const float inv_c = 1.0f / (float)kT2C;
        const float* sGamma = sAff + 2 * kT2C + h * 64;
        const float* sBeta = sAff + 3 * kT2C + h * 64;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it & 1;
            const uint32_t ph = (it >> 1) & 1u;
            const int j0 = (tile % p.tiles_per_row) * kT2P;
            const int br = tile / p.tiles_per_row;
            const int r = br % p.rows;
            const int b = br / p.rows;
            const int j = j0 + 2 * pp;
            const bool v0ok = j < p.N, v1ok = (j + 1) < p.N;
            const uint32_t keep = (v0ok ? 0x0000FFFFu : 0u) | (v1ok ? 0xFFFF0000u : 0u);
            const __nv_bfloat16* src =
                p.tri + ((long long)b * kT2C + h * 64) * p.tri_plane_stride + (long long)r * p.tri_pitch + j;
            uint32_t v[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                uint32_t x = 0;
                if (v0ok) x = __ldg(reinterpret_cast<const unsigned int*>(src + (long long)i * p.tri_plane_stride));
                v[i] = x & keep;
            }
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                s0 += bf16_lo(v[i]);
                s1 += bf16_hi(v[i]);
            }
            s0 += __shfl_xor_sync(0xffffffffu, s0, 16);
            s1 += __shfl_xor_sync(0xffffffffu, s1, 16);
            const float m0 = s0 * inv_c, m1 = s1 * inv_c;
            float q0 = 0.f, q1 = 0.f;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                const float d0 = bf16_lo(v[i]) - m0, d1 = bf16_hi(v[i]) - m1;
                q0 = fmaf(d0, d0, q0);
                q1 = fmaf(d1, d1, q1);
            }
            q0 += __shfl_xor_sync(0xffffffffu, q0, 16);
            q1 += __shfl_xor_sync(0xffffffffu, q1, 16);
            const float r0 = rsqrtf(q0 * inv_c + p.eps_out), r1 = rsqrtf(q1 * inv_c + p.eps_out);

            // the operand tile of this stage is free once the UMMAs of tile it-2 have retired
            bool ok = mbar_wait(&s_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm2, 500 + s);
            ok = named_barrier_all(kT2TriBarrier, 128, ok);
            if (!ok) break;
            uint8_t* trow0 = sStage + s * kT2StageBytes + kT2XBytes + h * kT2SubTile + (2 * pp) * 128;
            uint8_t* trow1 = trow0 + 128;
#pragma unroll
            for (int jc = 0; jc < 8; ++jc) {
                uint32_t o0[4], o1[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = jc * 8 + 2 * e;
                    const float g0 = sGamma[i], g1 = sGamma[i + 1], be0 = sBeta[i], be1 = sBeta[i + 1];
                    o0[e] = pack_bf16x2(fmaf((bf16_lo(v[i]) - m0) * r0, g0, be0),
                                        fmaf((bf16_lo(v[i + 1]) - m0) * r0, g1, be1));
                    o1[e] = pack_bf16x2(fmaf((bf16_hi(v[i]) - m1) * r1, g0, be0),
                                        fmaf((bf16_hi(v[i + 1]) - m1) * r1, g1, be1));
                }
                *reinterpret_cast<uint4*>(trow0 + ((jc ^ ((2 * pp) & 7)) << 4)) = make_uint4(o0[0], o0[1], o0[2], o0[3]);
                *reinterpret_cast<uint4*>(trow1 + ((jc ^ ((2 * pp + 1) & 7)) << 4)) =
                    make_uint4(o1[0], o1[1], o1[2], o1[3]);
            }
            fence_proxy_async_smem();
            mbar_arrive(&tn_ready[s]);
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;
        const int row = q * 32 + lane;                 // position inside the tile == TMEM lane
        const bool leader = (threadIdx.x == 320);
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it & 1;
            const uint32_t ph = (it >> 1) & 1u;
            const int j0 = (tile % p.tiles_per_row) * kT2P;
            const int br = tile / p.tiles_per_row;
            const int r = br % p.rows;
            const int b = br / p.rows;
            bool ok = mbar_wait(&acc_full[s], ph, abort_flag, p.status, kStageIdTm2, 400 + s);
            if (ok && p.has_residual) ok = mbar_wait(res_full, it & 1u, abort_flag, p.status, kStageIdTm2, 410);
            ok = named_barrier_all(kT2EpiBarrier, 128, ok);
            if (!ok) break;
            tcgen05_fence_after();
            if (!p.has_residual) {
                if (leader) tma_store_wait_read<0>();      // previous tile's store has read the staging
                named_barrier_sync(kT2EpiBarrier, 128);
            }
            const uint32_t t_g = tmem_base + s * 256 + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c32 = 0; c32 < 4; ++c32) {
                uint32_t rg[32], rp[32];
                tmem_ld_32x32(t_g + c32 * 32, rg);
                tmem_ld_32x32(t_g + 128 + c32 * 32, rp);
                tmem_ld_wait();
                uint8_t* base = sOut + (c32 >> 1) * kT2SubTile + row * 128;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const int chunk = ((c32 & 1) * 4 + cc) ^ (row & 7);
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
                        float v0 = __uint_as_float(rp[i0]) * sigmoid_fast(__uint_as_float(rg[i0]));
                        float v1 = __uint_as_float(rp[i0 + 1]) * sigmoid_fast(__uint_as_float(rg[i0 + 1]));
                        if (p.has_residual) {
                            // the reference rounds the block output to bf16 before `out + pair`
                            v0 = __bfloat162float(__float2bfloat16_rn(v0)) + bf16_lo(res[e]);
                            v1 = __bfloat162float(__float2bfloat16_rn(v1)) + bf16_hi(res[e]);
                        }
                        o[e] = pack_bf16x2(v0, v1);
                    }
                    *dst = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[s]);
            fence_proxy_async_smem();
            named_barrier_sync(kT2EpiBarrier, 128);
            if (leader) {
                tma_store_4d(&tmOut, sOut, 0, j0, r, b);
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
