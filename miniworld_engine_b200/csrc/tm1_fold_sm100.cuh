// Stage 1 of the block with the LayerNorm FOLDED into the projections, c = 128 (reference.py:66-75).
//
//   W . LN(x) = rstd * (W*gamma) . x  -  rstd*mean * rowsum(W*gamma)  +  W . beta
//
// so the tensor cores multiply the RAW z tile by weights that carry gamma, and the per-position
// statistics enter in the epilogue as one FMA per value:
//   pre[ch][pos] = acc[ch][pos] * rstd[pos] + (t[pos] * s[ch] + bias[ch]),   t = -mean * rstd,
//   s[ch] = sum_k bf16(W[ch][k] * gamma[k]) (the rounded values the UMMA really multiplies, so the
//   mean term cancels exactly), bias[ch] = sum_k W[ch][k] * beta[k].
// Nothing is written back into the z tile: the UMMAs start the moment the tile lands, the
// statistics are computed beside them, and the tile costs one shared-memory read pass instead of
// two reads and a write.  The result differs from the reference's bf16 path only by WHERE the
// rounding to bf16 happens (W*gamma instead of LN(x)); against an fp32 evaluation it is closer
// than the reference's own bf16 path.
//
// The folded weights live in TENSOR MEMORY as the UMMA A operand (tcgen05.mma with A in TMEM):
// 4 matrices x 64 columns (two bf16 per 32-bit column), written once per CTA by the epilogue
// threads, which fold their own channel's rows straight from global memory.  That halves the
// shared-memory traffic of the UMMAs (only the z tile is read from shared memory) and frees
// 128 KB of shared memory for a four-deep z ring and double-buffered store boxes.
//
// The other 256 TMEM columns hold the accumulators of HALF a tile (64 positions): per side
// (left = a, right = b) 64 columns of p/2 and 64 of g/2 — the weights are halved while folding, so
// p*sigmoid(g) = (p/2)*tanh(g/2) + p/2.  Order of work per 128-position tile:
// (a, half 0), (b, half 0), (a, half 1), (b, half 1); a side's epilogue drains its 128 columns
// while the tensor cores work on the other side.
//
// Persistent kernel, one CTA per SM, 576 threads:
//   warp 0        TMA producer: z tiles into a 4-stage ring
//   warp 1        UMMA issuer: per (half, side) 2 x 8 UMMAs of 128 x 64 x 16
//   warps 2..9    statistics: two groups of four warps on alternate tiles, one thread per position:
//                 mean and rstd of its 128 channels and the pair-mask bit, into an 8-slot ring
//   warps 10..13  epilogue of the left side, warps 14..17 of the right side:
//                 TMEM -> statistics -> gate -> bf16 -> swizzled staging -> TMA store
//
// A tile is 128 consecutive positions along the index that becomes the contraction's k: for the
// outgoing direction z row f, columns t0..t0+127; for the incoming direction z column f, rows
// t0..t0+127 (a strided TMA box), so both directions store plane element (f, t0+p).
#pragma once

#include "tm1_sm100.cuh"

namespace trimul {

constexpr int kF1Threads = 576;
constexpr int kF1StatThreads = 256;       // warps 2..9
constexpr int kF1EpiThreads = 128;        // per side
constexpr int kF1XStages = 4;
constexpr int kF1StatSlots = 8;
constexpr int kF1XBytes = 2 * kT1SubTile;                 // one z tile: two 64-channel halves
constexpr int kF1BoxBytes = kT1SubTile;                   // [128 channels][64 positions] store box
constexpr int kF1OffStaging = kF1XStages * kF1XBytes;     // 4 boxes: side x 2
constexpr int kF1OffStats = kF1OffStaging + 4 * kF1BoxBytes;      // per slot 64 x (r0, r1, t0, t1)
constexpr int kF1OffMaskWords = kF1OffStats + kF1StatSlots * 1024;  // per slot 128 x u16
constexpr int kF1OffAffine = kF1OffMaskWords + kF1StatSlots * 256;  // gamma[128], beta[128] fp32
constexpr int kF1OffBars = kF1OffAffine + 2 * kT1C * 4;
constexpr int kF1SmemBytes = kF1OffBars + 256;
constexpr int kF1StatBarrier = 2;      // 2, 3: the two statistics groups
constexpr int kF1EpiBarrier = 4;       // 4: left side, 5: right side
constexpr uint32_t kF1WeightCols = 256;   // TMEM columns [0,256): folded weights; [256,512): accumulators

struct Tm1FoldParams {
    Tm1Params base;
    const __nv_bfloat16* w[4];     // to_left, to_left_gate, to_right, to_right_gate ([out][in], 16-byte aligned)
};

// D[tmem] (+)= A[tmem] * B[smem]^T: A is 128 lanes (rows) x 16 bf16 per UMMA, two per 32-bit column.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// registers -> TMEM: thread t of the warp writes 16 consecutive 32-bit columns of lane
// (warp_id % 4) * 32 + t
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Fold one weight row (128 bf16, [out][in] layout) with gamma and 0.5, write it into this
// thread's TMEM lane at `tcol` (64 columns), and return s = sum of the folded (rounded) row and
// bias = 0.5 * sum_k W[k] * beta[k].
__device__ __forceinline__ void fold_row_to_tmem(const __nv_bfloat16* wrow, const float* sGamma, const float* sBeta,
                                                 uint32_t tcol, float& s, float& bias) {
    float ssum = 0.f, bsum = 0.f;
#pragma unroll 1
    for (int blk = 0; blk < 4; ++blk) {           // 32 input channels = 16 columns per block
        uint32_t packed[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k0 = blk * 32 + q * 8;
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(wrow + k0));
            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float w0 = bf16_lo(w4[e]), w1 = bf16_hi(w4[e]);
                const int k = k0 + 2 * e;
                const uint32_t f = pack_bf16x2(w0 * sGamma[k] * 0.5f, w1 * sGamma[k + 1] * 0.5f);
                ssum += bf16_lo(f) + bf16_hi(f);
                bsum = fmaf(w0, sBeta[k], fmaf(w1, sBeta[k + 1], bsum));
                packed[q * 4 + e] = f;
            }
        }
        tmem_st_32x16(tcol + blk * 16, packed);
    }
    s = ssum;
    bias = 0.5f * bsum;
}

__global__ void __launch_bounds__(kF1Threads, 1)
tm1_fold_sm100_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const Tm1FoldParams fp) {
    const Tm1Params& p = fp.base;
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, kStageIdTm1, 900);
        return;
    }
    uint8_t* sX = smem;
    uint8_t* sOut = smem + kF1OffStaging;
    uint8_t* sStats = smem + kF1OffStats;
    uint8_t* sMaskW = smem + kF1OffMaskWords;
    float* sGamma = reinterpret_cast<float*>(smem + kF1OffAffine);
    float* sBeta = sGamma + kT1C;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kF1OffBars);
    uint64_t* x_full = bars;                         // [4] z tile landed
    uint64_t* x_empty = bars + 4;                    // [4] UMMAs retired + 128 statistics threads done
    uint64_t* stat_ready = bars + 8;                 // [8] slot written (128 arrivals)
    uint64_t* acc_full = bars + 16;                  // [2] side's accumulators complete
    uint64_t* acc_empty = bars + 18;                 // [2] side's accumulators drained (4 arrivals)
    uint64_t* w_ready = bars + 20;                   // folded weights are in TMEM (256 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kF1XStages; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&x_empty[s], 1 + kF1StatThreads / 2);
        }
        for (int s = 0; s < kF1StatSlots; ++s) mbar_init(&stat_ready[s], kF1StatThreads / 2);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        mbar_init(w_ready, 2 * kF1EpiThreads);
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
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_acc = tmem_base + kF1WeightCols;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it % kF1XStages;
                const uint32_t ph = (it / kF1XStages) & 1u;
                if (!mbar_wait<true>(&x_empty[s], ph ^ 1u, abort_flag, p.status, kStageIdTm1, 100 + s)) break;
                const int t0 = (tile % p.tiles_per_fixed) * kT1P;
                const int bf = tile / p.tiles_per_fixed;
                const int f = bf % p.n_fixed;
                const int b = bf / p.n_fixed;
                mbar_arrive_expect_tx(&x_full[s], kF1XBytes);
                uint8_t* dst = sX + s * kF1XBytes;
                // z viewed as (channel, column, row, batch); outgoing box = 128 columns of row f,
                // incoming box = 128 rows of column f
                const int col = p.incoming ? f : t0;
                const int row = p.incoming ? t0 : f;
                tma_load_4d(dst, &tmZ, &x_full[s], 0, col, row, b);
                tma_load_4d(dst + kT1SubTile, &tmZ, &x_full[s], 64, col, row, b);
                TRIMUL_STAMP(0, it, 0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(128, 64);
            bool ok = mbar_wait<true>(w_ready, 0, abort_flag, p.status, kStageIdTm1, 200);
            tcgen05_fence_after();
            uint32_t it = 0;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
                const int s = it % kF1XStages;
                const uint32_t ph = (it / kF1XStages) & 1u;
                if (!mbar_wait<true>(&x_full[s], ph, abort_flag, p.status, kStageIdTm1, 210 + s)) break;
                tcgen05_fence_after();
                TRIMUL_STAMP(1, it, 0);
                const uint32_t xs = smem_u32(sX + s * kF1XBytes);
                for (int half = 0; ok && half < 2; ++half) {
                    for (int side = 0; side < 2; ++side) {
                        // use counter of this side's accumulators: 2 * it + half, so the parity is `half`
                        if (!mbar_wait<true>(&acc_empty[side], (uint32_t)half ^ 1u, abort_flag, p.status, kStageIdTm1,
                                       220 + side)) {
                            ok = false;
                            break;
                        }
                        tcgen05_fence_after();
                        const uint32_t d_p = tmem_acc + side * 128;
                        const uint32_t d_g = d_p + 64;
                        const uint32_t a_p = tmem_base + (side * 2) * 64;
                        const uint32_t a_g = a_p + 64;
#pragma unroll 2
                        for (int kk = 0; kk < kT1C / 16; ++kk) {
                            // B operand: positions half*64 .. +63 (64 rows of 128 bytes = 8 KB per half)
                            const uint64_t db = umma_smem_desc_sw128(xs + (kk >> 2) * kT1SubTile + half * 8192) +
                                                (kk & 3) * kDescKStep;
                            umma_bf16_ts(d_p, a_p + kk * 8, db, idesc, kk != 0);
                            umma_bf16_ts(d_g, a_g + kk * 8, db, idesc, kk != 0);
                        }
                        umma_commit(&acc_full[side]);
                        TRIMUL_STAMP(1, it, 1 + half);
                    }
                }
                if (!ok) break;
                umma_commit(&x_empty[s]);   // every UMMA that reads the tile has retired when this fires
            }
        }
        __syncwarp();
    } else if (warp < 10) {
        // ------------------------------------------------------------------ statistics (+ mask)
        const int g = (warp - 2) >> 2;
        const int pos = threadIdx.x - 64 - g * 128;    // 0..127, row of the tile
        const int bar_id = kF1StatBarrier + g;
        uint32_t it = g;
        for (int tile = blockIdx.x + g * gridDim.x; tile < p.total_tiles; tile += 2 * gridDim.x, it += 2) {
            const int s = it % kF1XStages;
            const uint32_t ph = (it / kF1XStages) & 1u;
            const int slot = it % kF1StatSlots;
            bool keep = true;
            if (p.mask_kind != 0) {
                const int t0 = (tile % p.tiles_per_fixed) * kT1P;
                const int bf = tile / p.tiles_per_fixed;
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
            if (!group_wait<true>(&x_full[s], ph, pos == 0, bar_id, 128, abort_flag, p.status, kStageIdTm1, 300 + s)) break;
            if (pos == 0) TRIMUL_STAMP(2 + g, it, 0);
            float rstd, t;
            row_stats(sX + s * kF1XBytes, kT1SubTile, pos, p.eps, rstd, t);
            mbar_arrive(&x_empty[s]);                  // this thread is done with the tile
            // slot `it % 8` was last read by the epilogues of tile it - 8, which finished before the
            // UMMAs of tile it - 4 could retire, which this tile's load had to wait for
            float* rec = reinterpret_cast<float*>(sStats + slot * 1024) + (pos >> 1) * 4 + (pos & 1);
            rec[0] = rstd;
            rec[2] = t;
            reinterpret_cast<uint16_t*>(sMaskW + slot * 256)[pos] = keep ? (uint16_t)0xFFFFu : (uint16_t)0u;
            mbar_arrive(&stat_ready[slot]);
            if (pos == 0) TRIMUL_STAMP(2 + g, it, 1);
        }
    } else {
        // ------------------------------------------------------------------ epilogue, one side per group
        const int side = (warp - 10) >> 2;
        const int q = warp & 3;
        const int ch = q * 32 + lane;                 // output channel == TMEM lane
        const bool leader = ((warp - 10) & 3) == 0 && lane == 0;
        const int bar_id = kF1EpiBarrier + side;
        const CUtensorMap* om = side == 0 ? &tmA : &tmB;
        const int rc = side == 0 ? p.a_row_chunk : p.b_row_chunk;
        const int cc = side == 0 ? p.a_col_chunk : p.b_col_chunk;
        const uint32_t lane_bits = (uint32_t)(q * 32) << 16;

        // fold this channel's projection and gate rows into TMEM
        float s_p, b_p, s_g, b_g;
        const __nv_bfloat16* w_proj = side == 0 ? fp.w[0] : fp.w[2];
        const __nv_bfloat16* w_gate = side == 0 ? fp.w[1] : fp.w[3];
        fold_row_to_tmem(w_proj + ch * kT1C, sGamma, sBeta, tmem_base + lane_bits + (side * 2) * 64, s_p, b_p);
        fold_row_to_tmem(w_gate + ch * kT1C, sGamma, sBeta, tmem_base + lane_bits + (side * 2 + 1) * 64, s_g, b_g);
        tmem_st_wait();
        tcgen05_fence_before();
        mbar_arrive(w_ready);
        const f32x2 sp2 = f2_pack(s_p, s_p), bp2 = f2_pack(b_p, b_p);
        const f32x2 sg2 = f2_pack(s_g, s_g), bg2 = f2_pack(b_g, b_g);

        const uint32_t t_p = tmem_acc + side * 128 + lane_bits;
        const bool masked = p.mask_kind != 0;
        uint32_t it = 0, use = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++it) {
            const int t0 = (tile % p.tiles_per_fixed) * kT1P;
            const int bf = tile / p.tiles_per_fixed;
            const int f = bf % p.n_fixed;
            const int b = bf / p.n_fixed;
            const int slot = it % kF1StatSlots;
            const uint8_t* stats = sStats + slot * 1024;
            const uint32_t* maskw = reinterpret_cast<const uint32_t*>(sMaskW + slot * 256);
#pragma unroll 1
            for (int half = 0; half < 2; ++half, ++use) {
                bool mine = true;
                if (leader) {
                    mine = mbar_wait<true>(&acc_full[side], use & 1u, abort_flag, p.status, kStageIdTm1, 400 + side);
                    if (mine && half == 0)
                        mine = mbar_wait<true>(&stat_ready[slot], (it / kF1StatSlots) & 1u, abort_flag, p.status,
                                         kStageIdTm1, 410 + slot);
                    // the store issued two boxes ago has read its staging box
                    tma_store_wait_read<1>();
                }
                if (!named_barrier_all(bar_id, kF1EpiThreads, mine)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                if (leader) TRIMUL_STAMP(4 + side, it, half * 2);
                uint8_t* stg = sOut + (side * 2 + (use & 1u)) * kF1BoxBytes;
                // 8 positions (one 16-byte chunk) at a time; the TMEM loads of the next 8 are in flight
                // while the current 8 get their statistics, are gated, rounded and written to the staging
                // box.  The loop stays rolled to keep the code small.
                auto emit8 = [&](int c8, const uint32_t (&rp)[8], const uint32_t (&rg)[8]) {
                    const int pair0 = half * 32 + c8 * 4;       // first position pair of the 8
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const ulonglong2 st = *reinterpret_cast<const ulonglong2*>(stats + (pair0 + e) * 16);
                        const f32x2 r2 = st.x, t2 = st.y;
                        const f32x2 hp = f2_fma(f2_pack(__uint_as_float(rp[2 * e]), __uint_as_float(rp[2 * e + 1])), r2,
                                                f2_fma(t2, sp2, bp2));
                        const f32x2 hg = f2_fma(f2_pack(__uint_as_float(rg[2 * e]), __uint_as_float(rg[2 * e + 1])), r2,
                                                f2_fma(t2, sg2, bg2));
                        float g0, g1;
                        f2_unpack(hg, g0, g1);
                        uint32_t w = f2_to_bf16x2(f2_fma(hp, f2_pack(tanh_fast(g0), tanh_fast(g1)), hp));
                        if (masked) w &= maskw[pair0 + e];
                        o[e] = w;
                    }
                    *reinterpret_cast<uint4*>(stg + ch * 128 + ((c8 ^ (ch & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                };
                uint32_t rpA[8], rgA[8], rpB[8], rgB[8];
                tmem_ld_32x8(t_p, rpA);
                tmem_ld_32x8(t_p + 64, rgA);
#pragma unroll 1
                for (int c8 = 0; c8 < 8; c8 += 2) {
                    tmem_ld_wait();
                    tmem_ld_32x8(t_p + (c8 + 1) * 8, rpB);
                    tmem_ld_32x8(t_p + 64 + (c8 + 1) * 8, rgB);
                    emit8(c8, rpA, rgA);
                    tmem_ld_wait();
                    if (c8 + 2 < 8) {
                        tmem_ld_32x8(t_p + (c8 + 2) * 8, rpA);
                        tmem_ld_32x8(t_p + 64 + (c8 + 2) * 8, rgA);
                    } else {
                        // every TMEM read of this side's accumulators has completed: hand them back early
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[side]);
                        if (leader) TRIMUL_STAMP(4 + side, it, half * 2 + 1);
                    }
                    emit8(c8 + 1, rpB, rgB);
                }
                fence_proxy_async_smem();
                named_barrier_sync(bar_id, kF1EpiThreads);
                if (leader) {
                    const int col0 = t0 + half * 64;
                    if (col0 < p.n_run) {
                        tma_store_4d(om, stg, col0 % cc, f % rc, b * kT1C, col0 / cc + f / rc);
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
