// Stage 3 of the block on the tensor cores, c = 128: LayerNorm_out over the channels of the
// contraction result, the output projection, the output gate from a fresh LayerNorm_in of z
// (unmasked, reference.py:82-83), optional residual — one pass, row-major bf16 result.
//
// Persistent kernel, one CTA per SM, 704 threads, 128-position tiles (z row r, columns j0..j0+127):
//   warp 0        TMA producer: Wg, Wo once; z tiles (and residual tiles) into a 2-stage ring
//   warp 1        UMMA issuer: gate = x_n . Wg^T and proj = tri_n . Wo^T, 128x128x16 each, into a
//                 double-buffered pair of 128-column TMEM accumulators (TMEM lane = position)
//   warps 2..9    LayerNorm_in: two threads per position, in place in the swizzled z tile
//   warps 10..17  LayerNorm_out, two groups of four warps that take alternate tiles (one group per
//                 stage): read tri straight from global memory along the contiguous position axis
//                 of each channel plane (coalesced 4-byte pairs), accumulate the statistics while
//                 parking the raw values TRANSPOSED in the K-major swizzled operand tile, then
//                 normalise that tile in place — the channel-major -> row-major turn costs no
//                 extra pass over memory
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
constexpr int kT2TriThreads = 128;      // per group, warps 10..13 and 14..17
constexpr int kT2EpiThreads = 128;      // warps 18..21
constexpr int kT2Workers = kT2LnThreads + 2 * kT2TriThreads + kT2EpiThreads;
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
constexpr int kT2TriBarrier = 3;        // 3, 4: the two LayerNorm_out groups
constexpr int kT2EpiBarrier = 5;
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
    uint64_t* xn_ready = bars + 3;      // [2] x_n operand ready (256 arrivals)
    uint64_t* tn_ready = bars + 5;      // [2] tri_n operand ready (128 arrivals)
    uint64_t* s_empty = bars + 7;       // [2] UMMAs that read the stage retired
    uint64_t* acc_full = bars + 9;      // [2]
    uint64_t* acc_empty = bars + 11;    // [2] (4 arrivals)
    uint64_t* res_full = bars + 13;     // residual tile landed in the staging buffer
    uint64_t* out_free = bars + 14;     // staging buffer released by the epilogue (1 arrival)
    uint64_t* w_ready = bars + 15;      // weights halved (all worker threads)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        mbar_init(w_ready, kT2Workers);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&xn_ready[s], kT2LnThreads);
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
    } else if (warp < 10) {
        // ------------------------------------------------------------------ LayerNorm_in, in place
        const int lt = threadIdx.x - 64;
        const int pos = lt >> 1;
        const int h = lt & 1;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int s = it & 1;
            const uint32_t ph = (it >> 1) & 1u;
            if (!group_wait(&x_full[s], ph, lt == 0, kT2LnBarrier, kT2LnThreads, abort_flag, p.status,
                            kStageIdTm2, 300 + s))
                break;
            ln_half_row_inplace(sStage + s * kT2StageBytes, kT2SubTile, pos, h, sAff, sAff + kT2C, p.eps_in, false);
            fence_proxy_async_smem();
            mbar_arrive(&xn_ready[s]);
        }
    } else if (warp < 18) {
        // ------------------------------------------------------------------ LayerNorm_out + transpose
        // group g owns stage g and the tiles with (local tile index & 1) == g.
        // lane l of group-warp w: positions 2*pp, 2*pp+1 with pp = 16*w + (l & 15); channel half h = l >> 4
        const int g = (warp - 10) >> 2;
        const int tw = (warp - 10) & 3;
        const int pp = tw * 16 + (lane & 15);
        const int h = lane >> 4;
        const int bar_id = kT2TriBarrier + g;
        const float* sGamma = sAff + 2 * kT2C + h * 64;
        const float* sBeta = sAff + 3 * kT2C + h * 64;
        uint8_t* trow0 = sStage + g * kT2StageBytes + kT2XBytes + h * kT2SubTile + (2 * pp) * 128;
        uint8_t* trow1 = trow0 + 128;
        const uint32_t swz0 = (uint32_t)((2 * pp) & 7), swz1 = (uint32_t)((2 * pp + 1) & 7);
        uint32_t it = g;
        for (int tile = blockIdx.x + g * gridDim.x; tile < p.total_tiles; tile += 2 * gridDim.x, it += 2) {
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
            // the operand tile of this stage is free once the UMMAs of the group's previous tile retired
            if (!group_wait(&s_empty[g], ph ^ 1u, tw == 0 && lane == 0, bar_id, kT2TriThreads, abort_flag, p.status,
                            kStageIdTm2, 500 + g))
                break;
            // pass 1: global -> (statistics, raw transposed copy in the operand tile)
            float sh0 = 0.f, sh1 = 0.f, a0 = 0.f, a1 = 0.f, q0 = 0.f, q1 = 0.f;
#pragma unroll 1
            for (int jc = 0; jc < 8; ++jc) {
                uint32_t v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    uint32_t x = 0;
                    if (v0ok)
                        x = __ldg(reinterpret_cast<const unsigned int*>(src + (long long)(jc * 8 + i) * p.tri_plane_stride));
                    v[i] = x & keep;
                }
                if (jc == 0) {
                    // common shift of the row: channel 0, held by the h = 0 lane of the pair
                    sh0 = __shfl_sync(0xffffffffu, bf16_lo(v[0]), lane & 15);
                    sh1 = __shfl_sync(0xffffffffu, bf16_hi(v[0]), lane & 15);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float d0 = bf16_lo(v[i]) - sh0, d1 = bf16_hi(v[i]) - sh1;
                    a0 += d0;
                    q0 = fmaf(d0, d0, q0);
                    a1 += d1;
                    q1 = fmaf(d1, d1, q1);
                }
                // transpose 8 (position-pair) words into one 16-byte chunk per position
                uint4 c0, c1;
                c0.x = __byte_perm(v[0], v[1], 0x5410); c1.x = __byte_perm(v[0], v[1], 0x7632);
                c0.y = __byte_perm(v[2], v[3], 0x5410); c1.y = __byte_perm(v[2], v[3], 0x7632);
                c0.z = __byte_perm(v[4], v[5], 0x5410); c1.z = __byte_perm(v[4], v[5], 0x7632);
                c0.w = __byte_perm(v[6], v[7], 0x5410); c1.w = __byte_perm(v[6], v[7], 0x7632);
                *reinterpret_cast<uint4*>(trow0 + ((((uint32_t)jc) ^ swz0) << 4)) = c0;
                *reinterpret_cast<uint4*>(trow1 + ((((uint32_t)jc) ^ swz1) << 4)) = c1;
            }
            a0 += __shfl_xor_sync(0xffffffffu, a0, 16);
            a1 += __shfl_xor_sync(0xffffffffu, a1, 16);
            q0 += __shfl_xor_sync(0xffffffffu, q0, 16);
            q1 += __shfl_xor_sync(0xffffffffu, q1, 16);
            const float inv_c = 1.0f / (float)kT2C;
            const float m0 = a0 * inv_c, m1 = a1 * inv_c;
            const float r0 = rsqrtf(fmaxf(fmaf(-m0, m0, q0 * inv_c), 0.f) + p.eps_out);
            const float r1 = rsqrtf(fmaxf(fmaf(-m1, m1, q1 * inv_c), 0.f) + p.eps_out);
            const float n0 = -(sh0 + m0) * r0, n1 = -(sh1 + m1) * r1;
            // pass 2: normalise the parked values in place (each thread re-reads only what it wrote)
#pragma unroll 1
            for (int jc = 0; jc < 8; ++jc) {
                const float4 g0 = *reinterpret_cast<const float4*>(sGamma + jc * 8);
                const float4 g1 = *reinterpret_cast<const float4*>(sGamma + jc * 8 + 4);
                const float4 b0 = *reinterpret_cast<const float4*>(sBeta + jc * 8);
                const float4 b1 = *reinterpret_cast<const float4*>(sBeta + jc * 8 + 4);
                uint4* p0 = reinterpret_cast<uint4*>(trow0 + ((((uint32_t)jc) ^ swz0) << 4));
                uint4* p1 = reinterpret_cast<uint4*>(trow1 + ((((uint32_t)jc) ^ swz1) << 4));
                const uint4 x0 = *p0, x1 = *p1;
                uint4 o0, o1;
                o0.x = pack_bf16x2(fmaf(fmaf(bf16_lo(x0.x), r0, n0), g0.x, b0.x), fmaf(fmaf(bf16_hi(x0.x), r0, n0), g0.y, b0.y));
                o0.y = pack_bf16x2(fmaf(fmaf(bf16_lo(x0.y), r0, n0), g0.z, b0.z), fmaf(fmaf(bf16_hi(x0.y), r0, n0), g0.w, b0.w));
                o0.z = pack_bf16x2(fmaf(fmaf(bf16_lo(x0.z), r0, n0), g1.x, b1.x), fmaf(fmaf(bf16_hi(x0.z), r0, n0), g1.y, b1.y));
                o0.w = pack_bf16x2(fmaf(fmaf(bf16_lo(x0.w), r0, n0), g1.z, b1.z), fmaf(fmaf(bf16_hi(x0.w), r0, n0), g1.w, b1.w));
                o1.x = pack_bf16x2(fmaf(fmaf(bf16_lo(x1.x), r1, n1), g0.x, b0.x), fmaf(fmaf(bf16_hi(x1.x), r1, n1), g0.y, b0.y));
                o1.y = pack_bf16x2(fmaf(fmaf(bf16_lo(x1.y), r1, n1), g0.z, b0.z), fmaf(fmaf(bf16_hi(x1.y), r1, n1), g0.w, b0.w));
                o1.z = pack_bf16x2(fmaf(fmaf(bf16_lo(x1.z), r1, n1), g1.x, b1.x), fmaf(fmaf(bf16_hi(x1.z), r1, n1), g1.y, b1.y));
                o1.w = pack_bf16x2(fmaf(fmaf(bf16_lo(x1.w), r1, n1), g1.z, b1.z), fmaf(fmaf(bf16_hi(x1.w), r1, n1), g1.w, b1.w));
                *p0 = o0;
                *p1 = o1;
            }
            fence_proxy_async_smem();
            mbar_arrive(&tn_ready[g]);
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
            if (!p.has_residual) {
                if (leader) tma_store_wait_read<0>();      // previous tile's store has read the staging
                named_barrier_sync(kT2EpiBarrier, kT2EpiThreads);
            }
            const uint32_t t_g = tmem_base + s * 256 + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c16 = 0; c16 < 8; ++c16) {
                uint32_t rg[16], rp[16];
                tmem_ld_32x16(t_g + c16 * 16, rg);
                tmem_ld_32x16(t_g + 128 + c16 * 16, rp);
                tmem_ld_wait();
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
                        float v0 = gate_from_halves(__uint_as_float(rp[i0]), __uint_as_float(rg[i0]));
                        float v1 = gate_from_halves(__uint_as_float(rp[i0 + 1]), __uint_as_float(rg[i0 + 1]));
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
            named_barrier_sync(kT2EpiBarrier, kT2EpiThreads);
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
