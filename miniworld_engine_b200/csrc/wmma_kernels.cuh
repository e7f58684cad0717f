// Warp-level tensor-core kernels for stages 1 and 3 at the channel widths the tcgen05 kernels
// do not cover (bf16, c and h multiples of 16 up to 256, other than the c = h = 128 case).
//
// They keep the layouts and the bf16 rounding points of the other kernels (x_n, a, b, tri_n, out
// rounded to bf16, fp32 accumulation and fp32 LayerNorm / gate arithmetic in between) and use the
// warp-wide 16x16x16 MMA through nvcuda::wmma: one block owns 64 positions, normalises them into
// shared memory once, and each warp multiplies a 32- or 64-position slice against the weight
// matrices, whose 16x16 fragments it reads straight from global memory (they stay in L2: at most
// 4 x 256 x 256 bf16).  These are not tuned like the c = 128 kernels; they exist so that the other
// widths of the reference's d_pair sweep do not fall back to the scalar CUDA-core kernels.
#pragma once

#include <mma.h>

#include "plain_kernels.cuh"

namespace trimul {

constexpr int kWmPos = 64;          // positions per block
constexpr int kWmThreads = 256;     // 8 warps: 2 position halves x 4 residue classes of 16-channel groups
constexpr int kWmScratch = 8 * 4 * 256 * (int)sizeof(float);     // per warp 4 accumulator tiles

inline int wmma_xn_bytes(int width) { return (kWmPos * (width + 8) * 2 + 127) / 128 * 128; }
inline int wmma_tm1_smem(int c) { return wmma_xn_bytes(c) + kWmScratch + kWmPos * (int)sizeof(float); }
inline int wmma_tm2_smem(int c, int h) { return wmma_xn_bytes(c) + wmma_xn_bytes(h) + kWmScratch; }

// LayerNorm of one row of `width` values (held by one warp, lane l has channels l + 32 i in v[i]);
// the normalised, affine-transformed, bf16-rounded row goes to dst[ch].  width <= 256.
__device__ __forceinline__ void wmma_ln_regs(const float (&v)[8], int width, const float* __restrict__ gamma,
                                             const float* __restrict__ beta, float eps, __nv_bfloat16* dst) {
    const int lane = threadIdx.x & 31;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s / (float)width;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float d = (lane + 32 * i) < width ? v[i] - mean : 0.f;
        q = fmaf(d, d, q);
    }
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float rstd = 1.0f / sqrtf(q / (float)width + eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int ch = lane + 32 * i;
        if (ch < width) dst[ch] = __float2bfloat16_rn((v[i] - mean) * rstd * gamma[ch] + beta[ch]);
    }
}

// `get(ch)` returns the raw value of channel ch of the row
template <typename Get>
__device__ __forceinline__ void wmma_ln_row(Get get, int width, const float* __restrict__ gamma,
                                            const float* __restrict__ beta, float eps, __nv_bfloat16* dst) {
    const int lane = threadIdx.x & 31;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (lane + 32 * i) < width ? get(lane + 32 * i) : 0.f;
    wmma_ln_regs(v, width, gamma, beta, eps, dst);
}

// LayerNorm_in of the block's 64 z rows into xn (rows past npos are zero-filled).  Each warp owns
// rows warp, warp + 8, ...; it fetches four of them before normalising any, so that four rows'
// worth of global loads are in flight.  `row_of(q)` returns the address of row q.
template <typename RowOf>
__device__ __forceinline__ void wmma_ln_tile(RowOf row_of, int npos, int c, int ldx, const float* __restrict__ gamma,
                                             const float* __restrict__ beta, float eps, __nv_bfloat16* xn) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int g = 0; g < 2; ++g) {
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int q = warp + 8 * (4 * g + u);
            const __nv_bfloat16* row = q < npos ? row_of(q) : nullptr;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                v[u][i] = (row != nullptr && (lane + 32 * i) < c) ? __bfloat162float(row[lane + 32 * i]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int q = warp + 8 * (4 * g + u);
            __nv_bfloat16* dst = xn + q * ldx;
            if (q < npos) {
                wmma_ln_regs(v[u], c, gamma, beta, eps, dst);
            } else {
                for (int ch = lane; ch < c; ch += 32) dst[ch] = __float2bfloat16_rn(0.f);
            }
        }
    }
}

using WmA = nvcuda::wmma::fragment<nvcuda::wmma::matrix_a, 16, 16, 16, __nv_bfloat16, nvcuda::wmma::row_major>;
using WmB = nvcuda::wmma::fragment<nvcuda::wmma::matrix_b, 16, 16, 16, __nv_bfloat16, nvcuda::wmma::col_major>;
using WmC = nvcuda::wmma::fragment<nvcuda::wmma::accumulator, 16, 16, 16, float>;

// Stage 1.  Outgoing: a block owns 64 consecutive columns s of one z row r, and writes plane
// elements (r, s).  Incoming: 64 consecutive rows r of one column s, plane elements (s, r) — in both
// cases the 64 positions are contiguous along the plane's column axis.
// grid: B * (outgoing ? rows : N) * ceil((outgoing ? N : rows) / 64); dynamic smem wmma_tm1_smem(c).
// kMT = 16-position tiles per warp: 2 (a warp owns 32 positions and every 4th 16-channel group) for
// narrow outputs, 4 (all 64 positions, every 8th group) once there are at least 8 groups.
template <int kMT>
__global__ void __launch_bounds__(kWmThreads, 2) wmma_tm1_kernel(const __nv_bfloat16* __restrict__ z, PlainTm1Params p) {
    extern __shared__ __align__(128) unsigned char wm_smem[];
    const int c = p.c, h = p.h, ldx = c + 8;
    __nv_bfloat16* xn = reinterpret_cast<__nv_bfloat16*>(wm_smem);
    float* scr_all = reinterpret_cast<float*>(wm_smem + (kWmPos * ldx * 2 + 127) / 128 * 128);
    float* keep = scr_all + 8 * 4 * 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int F = p.incoming ? p.rows : p.N;        // extent of the axis the tile runs along
    const int O = p.incoming ? p.N : p.rows;        // extent of the other axis
    const int tiles = (F + kWmPos - 1) / kWmPos;
    const int f0 = (blockIdx.x % tiles) * kWmPos;
    const int bo = blockIdx.x / tiles;
    const int o = bo % O, b = bo / O;
    const int npos = min(kWmPos, F - f0);

    // element offsets of the 64 positions inside a plane, computed once: PlaneView::offset divides
    // 64-bit integers, far too slow to repeat per channel
    __shared__ long long ofs_a[kWmPos], ofs_b[kWmPos];
    if (threadIdx.x < kWmPos) {
        const long long col = min(f0 + (int)threadIdx.x, F - 1);
        ofs_a[threadIdx.x] = p.a.offset(0, o, col);
        ofs_b[threadIdx.x] = p.b.offset(0, o, col);
        float k = 0.f;
        if (threadIdx.x < npos) {
            const int r = p.incoming ? f0 + threadIdx.x : o, s = p.incoming ? o : f0 + threadIdx.x;
            const int zr = p.row0 + r;
            k = 1.f;
            if (p.mask_kind == 1)
                k = (p.mask[(long long)b * p.N + zr] != 0 && p.mask[(long long)b * p.N + s] != 0) ? 1.f : 0.f;
            else if (p.mask_kind == 2)
                k = p.mask[((long long)b * p.N + zr) * p.N + s] != 0 ? 1.f : 0.f;
        }
        keep[threadIdx.x] = k;
    }
    wmma_ln_tile(
        [&](int q) {
            const int r = p.incoming ? f0 + q : o, s = p.incoming ? o : f0 + q;
            return z + (((long long)b * p.rows + r) * p.N + s) * c;
        },
        npos, c, ldx, p.gamma, p.beta, p.eps, xn);
    __syncthreads();

    // Two passes, one gated projection each (left -> a, right -> b): a warp holds the value and the
    // gate accumulators of kMT position tiles, so a weight fragment fetched from L2 serves 16 kMT
    // positions.
    constexpr int kClasses = 2 * kMT;                    // residue classes of the 16-channel groups: 8 warps / (4 / kMT) slices
    const int mp = kMT == 2 ? (warp & 1) : 0;            // first position of the warp's slice / 32
    const int cls = kMT == 2 ? (warp >> 1) : warp;
    float* scr = scr_all + warp * 4 * 256;
    for (int pass = 0; pass < 2; ++pass) {
        const __nv_bfloat16* Wv = static_cast<const __nv_bfloat16*>(pass ? p.w_right : p.w_left);
        const __nv_bfloat16* Wg = static_cast<const __nv_bfloat16*>(pass ? p.w_right_gate : p.w_left_gate);
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(pass ? p.b.base : p.a.base);
        const long long dst_plane = pass ? p.b.plane_stride : p.a.plane_stride;
        const long long* ofs = pass ? ofs_b : ofs_a;
        for (int nf = cls; nf < h / 16; nf += kClasses) {
            WmC av[kMT], ag[kMT];
#pragma unroll
            for (int t = 0; t < kMT; ++t) {
                nvcuda::wmma::fill_fragment(av[t], 0.f);
                nvcuda::wmma::fill_fragment(ag[t], 0.f);
            }
#pragma unroll 2
            for (int k0 = 0; k0 < c; k0 += 16) {
                WmB bv, bg;
                nvcuda::wmma::load_matrix_sync(bv, Wv + (long long)nf * 16 * c + k0, c);
                nvcuda::wmma::load_matrix_sync(bg, Wg + (long long)nf * 16 * c + k0, c);
#pragma unroll
                for (int t = 0; t < kMT; ++t) {
                    WmA a;
                    nvcuda::wmma::load_matrix_sync(a, xn + (mp * 32 + t * 16) * ldx + k0, ldx);
                    nvcuda::wmma::mma_sync(av[t], a, bv, av[t]);
                    nvcuda::wmma::mma_sync(ag[t], a, bg, ag[t]);
                }
            }
#pragma unroll
            for (int t = 0; t < kMT; ++t) {      // column-major: element (position i, channel j) at j * 16 + i
                nvcuda::wmma::store_matrix_sync(scr, av[t], 16, nvcuda::wmma::mem_col_major);
                nvcuda::wmma::store_matrix_sync(scr + 256, ag[t], 16, nvcuda::wmma::mem_col_major);
                __syncwarp();
                const int i = lane & 15;
                const int q = mp * 32 + t * 16 + i;
                if (q < npos) {
                    const float kq = keep[q];
                    // plane element: outgoing (r, s) = (o, f0 + q); incoming (s, r) = (o, f0 + q)
                    for (int j = lane >> 4; j < 16; j += 2) {
                        const float val = scr[j * 16 + i] * sigmoid_ref(scr[256 + j * 16 + i]) * kq;
                        dst[((long long)b * h + nf * 16 + j) * dst_plane + ofs[q]] = __float2bfloat16_rn(val);
                    }
                }
                __syncwarp();
            }
        }
    }
}

// Stage 3.  A block owns 64 consecutive columns of one row of the slab.
// grid: B * rows * ceil(N / 64); dynamic smem wmma_tm2_smem(c, h).  kMT as in stage 1.
template <int kMT>
__global__ void __launch_bounds__(kWmThreads, 2)
wmma_tm2_kernel(const __nv_bfloat16* __restrict__ z, __nv_bfloat16* __restrict__ out,
                const __nv_bfloat16* __restrict__ residual, PlainTm2Params p) {
    extern __shared__ __align__(128) unsigned char wm_smem[];
    const int c = p.c, h = p.h, ldx = c + 8, ldt = h + 8;
    __nv_bfloat16* xn = reinterpret_cast<__nv_bfloat16*>(wm_smem);
    __nv_bfloat16* tn = reinterpret_cast<__nv_bfloat16*>(wm_smem + (kWmPos * ldx * 2 + 127) / 128 * 128);
    float* scr_all = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(tn) + (kWmPos * ldt * 2 + 127) / 128 * 128);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int tiles = (p.N + kWmPos - 1) / kWmPos;
    const int s0 = (blockIdx.x % tiles) * kWmPos;
    const int br = blockIdx.x / tiles;
    const int r = br % p.rows, b = br / p.rows;
    const int npos = min(kWmPos, p.N - s0);
    const long long pos0 = ((long long)b * p.rows + r) * p.N + s0;

    // raw tri tile, transposed into [position][channel]: consecutive threads walk the contiguous position axis
    {
        const int q = threadIdx.x & 63;
        // the position's offset inside a plane once (PlaneView::offset divides 64-bit integers)
        const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.tri.base) + p.tri.offset(0, r, min(s0 + q, p.N - 1));
#pragma unroll 4
        for (int ch = threadIdx.x >> 6; ch < h; ch += 4)
            tn[q * ldt + ch] = q < npos ? src[((long long)b * h + ch) * p.tri.plane_stride] : __float2bfloat16_rn(0.f);
    }
    wmma_ln_tile([&](int q) { return z + (pos0 + q) * c; }, npos, c, ldx, p.gamma_in, p.beta_in, p.eps_in, xn);
    __syncthreads();
    for (int q = warp; q < npos; q += 8) {
        __nv_bfloat16* row = tn + q * ldt;       // in place: every lane holds its values before any is overwritten
        wmma_ln_row([&](int ch) { return __bfloat162float(row[ch]); }, h, p.gamma_out, p.beta_out, p.eps_out, row);
    }
    __syncthreads();

    const __nv_bfloat16* Wg = static_cast<const __nv_bfloat16*>(p.w_gate);
    const __nv_bfloat16* Wo = static_cast<const __nv_bfloat16*>(p.w_out);
    constexpr int kClasses = 2 * kMT;
    const int mp = kMT == 2 ? (warp & 1) : 0;
    const int cls = kMT == 2 ? (warp >> 1) : warp;
    float* scr = scr_all + warp * 4 * 256;
    for (int nf = cls; nf < c / 16; nf += kClasses) {
        WmC g[kMT], v[kMT];
#pragma unroll
        for (int t = 0; t < kMT; ++t) {
            nvcuda::wmma::fill_fragment(g[t], 0.f);
            nvcuda::wmma::fill_fragment(v[t], 0.f);
        }
#pragma unroll 2
        for (int k0 = 0; k0 < c; k0 += 16) {
            WmB bf;
            nvcuda::wmma::load_matrix_sync(bf, Wg + (long long)nf * 16 * c + k0, c);
#pragma unroll
            for (int t = 0; t < kMT; ++t) {
                WmA a;
                nvcuda::wmma::load_matrix_sync(a, xn + (mp * 32 + t * 16) * ldx + k0, ldx);
                nvcuda::wmma::mma_sync(g[t], a, bf, g[t]);
            }
        }
#pragma unroll 2
        for (int k0 = 0; k0 < h; k0 += 16) {
            WmB bf;
            nvcuda::wmma::load_matrix_sync(bf, Wo + (long long)nf * 16 * h + k0, h);
#pragma unroll
            for (int t = 0; t < kMT; ++t) {
                WmA a;
                nvcuda::wmma::load_matrix_sync(a, tn + (mp * 32 + t * 16) * ldt + k0, ldt);
                nvcuda::wmma::mma_sync(v[t], a, bf, v[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < kMT; ++t) {      // row-major: element (position i, channel j) at i * 16 + j
            nvcuda::wmma::store_matrix_sync(scr, g[t], 16, nvcuda::wmma::mem_row_major);
            nvcuda::wmma::store_matrix_sync(scr + 256, v[t], 16, nvcuda::wmma::mem_row_major);
            __syncwarp();
            const int j = lane & 15;
            for (int i = lane >> 4; i < 16; i += 2) {
                const int q = mp * 32 + t * 16 + i;
                if (q < npos) {
                    float y = sigmoid_ref(scr[i * 16 + j]) * scr[256 + i * 16 + j];
                    const long long e = (pos0 + q) * c + nf * 16 + j;
                    if (p.drop_scale != nullptr)
                        y = __bfloat162float(__float2bfloat16_rn(y)) *
                            __bfloat162float(static_cast<const __nv_bfloat16*>(p.drop_scale)[((long long)b * p.N + s0 + q) * c + nf * 16 + j]);
                    if (residual != nullptr) y = __bfloat162float(__float2bfloat16_rn(y)) + __bfloat162float(residual[e]);
                    out[e] = __float2bfloat16_rn(y);
                }
            }
            __syncwarp();
        }
    }
}

}  // namespace trimul
