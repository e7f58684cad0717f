// CUDA-core kernels for the three stages of the block, templated on the storage type.
//
// T = float is the fp32 path (IEEE fp32 FMA throughout, no TF32, expf-based sigmoid): it has to
// meet a 1e-5 relative tolerance against the fp32 reference, which rules the tensor cores out.
// T = __nv_bfloat16 uses the same layouts and the same bf16 rounding points as the tensor-core
// kernels (x_n, a, b, tri, tri_n, out) with fp32 arithmetic in between; it serves channel widths
// the tensor-core kernels do not cover and is the stage-by-stage cross-check for them.
//
// All three read/write the channel-major operand planes through PlaneView, which implements the
// chunked addressing of trimul_planes, so they work on gathered multi-GPU operands unchanged.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace trimul {

struct PlaneView {
    void* base;
    long long rows, cols, pitch, plane_stride, chunk_stride, row_chunk, col_chunk;
    __device__ __forceinline__ long long offset(long long p, long long r, long long q) const {
        const long long chunk = r / row_chunk + q / col_chunk;   // at most one of the two is non-zero
        return chunk * chunk_stride + p * plane_stride + (r % row_chunk) * pitch + (q % col_chunk);
    }
};

template <typename T> __device__ __forceinline__ float load_f(const T* p);
template <> __device__ __forceinline__ float load_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float load_f<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat162float(*p);
}
template <typename T> __device__ __forceinline__ T store_t(float v);
template <> __device__ __forceinline__ float store_t<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 store_t<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}
// value as it would be after a round trip through storage type T
template <typename T> __device__ __forceinline__ float round_t(float v);
template <> __device__ __forceinline__ float round_t<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_t<__nv_bfloat16>(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ float sigmoid_ref(float x) { return 1.0f / (1.0f + expf(-x)); }

constexpr int kPlainPos = 8;       // positions per block
constexpr int kPlainThreads = 128;
constexpr int kPlainMaxC = 256;

// LayerNorm of `npos` rows of c channels held at xs[pos*c + ch] (fp32, raw values on entry,
// normalised, affine-transformed and storage-rounded values on exit).  One warp per row.
template <typename T>
__device__ __forceinline__ void plain_layernorm_rows(float* xs, int npos, int c, const float* gamma,
                                                     const float* beta, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int pos = warp; pos < npos; pos += nwarps) {
        float* x = xs + pos * c;
        float s = 0.f;
        for (int ch = lane; ch < c; ch += 32) s += x[ch];
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float mean = s / (float)c;
        float q = 0.f;
        for (int ch = lane; ch < c; ch += 32) {
            const float d = x[ch] - mean;
            q = fmaf(d, d, q);
        }
        for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
        const float rstd = 1.0f / sqrtf(q / (float)c + eps);
        for (int ch = lane; ch < c; ch += 32)
            x[ch] = round_t<T>((x[ch] - mean) * rstd * gamma[ch] + beta[ch]);
    }
}

struct PlainTm1Params {
    int B, rows, N, c, row0, incoming, mask_kind;
    int h;      // planes per batch element = rows of the four [h, c] projection matrices
    const uint8_t* mask;
    const float *gamma, *beta;
    float eps;
    const void *w_left, *w_left_gate, *w_right, *w_right_gate;
    PlaneView a, b;
};

// grid: B * rows * ceil(N / kPlainPos); block kPlainThreads
template <typename T>
__global__ void __launch_bounds__(kPlainThreads) plain_tm1_kernel(const T* __restrict__ z, PlainTm1Params p) {
    __shared__ float xs[kPlainPos * kPlainMaxC];
    __shared__ float keep[kPlainPos];
    const int c = p.c;
    const int tiles = (p.N + kPlainPos - 1) / kPlainPos;
    const int s0 = (blockIdx.x % tiles) * kPlainPos;
    const int br = blockIdx.x / tiles;
    const int r = br % p.rows;
    const int b = br / p.rows;
    const int npos = min(kPlainPos, p.N - s0);
    const T* zrow = z + (((long long)b * p.rows + r) * p.N + s0) * c;
    for (int i = threadIdx.x; i < npos * c; i += blockDim.x) xs[i] = load_f<T>(zrow + i);
    if (threadIdx.x < npos) {
        const int zr = p.row0 + r, zc = s0 + threadIdx.x;
        float k = 1.f;
        if (p.mask_kind == 1)
            k = (p.mask[(long long)b * p.N + zr] != 0 && p.mask[(long long)b * p.N + zc] != 0) ? 1.f : 0.f;
        else if (p.mask_kind == 2)
            k = p.mask[((long long)b * p.N + zr) * p.N + zc] != 0 ? 1.f : 0.f;
        keep[threadIdx.x] = k;
    }
    __syncthreads();
    plain_layernorm_rows<T>(xs, npos, c, p.gamma, p.beta, p.eps);
    __syncthreads();
    const T* W[4] = {(const T*)p.w_left, (const T*)p.w_left_gate, (const T*)p.w_right, (const T*)p.w_right_gate};
    for (int o = threadIdx.x; o < p.h; o += blockDim.x) {
        float acc[4][kPlainPos];
#pragma unroll
        for (int m = 0; m < 4; ++m)
#pragma unroll
            for (int q = 0; q < kPlainPos; ++q) acc[m][q] = 0.f;
        for (int k = 0; k < c; ++k) {
            float w[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) w[m] = load_f<T>(W[m] + (long long)o * c + k);
#pragma unroll
            for (int q = 0; q < kPlainPos; ++q) {
                const float x = xs[q * c + k];
#pragma unroll
                for (int m = 0; m < 4; ++m) acc[m][q] = fmaf(w[m], x, acc[m][q]);
            }
        }
        const long long plane = (long long)b * p.h + o;
        for (int q = 0; q < npos; ++q) {
            const float left = acc[0][q] * sigmoid_ref(acc[1][q]) * keep[q];
            const float right = acc[2][q] * sigmoid_ref(acc[3][q]) * keep[q];
            // outgoing: plane element (r, s);  incoming: stored transposed, element (s, r)
            const long long pr = p.incoming ? (s0 + q) : r;
            const long long pc = p.incoming ? r : (s0 + q);
            ((T*)p.a.base)[p.a.offset(plane, pr, pc)] = store_t<T>(left);
            ((T*)p.b.base)[p.b.offset(plane, pr, pc)] = store_t<T>(right);
        }
    }
}

// tri[p][i][j] = sum_k a[p][i][k] * b[p][j][k]; grid (ceil(rows_b/32), ceil(rows_a/32), planes), block 16x16,
// each thread a 2x2 patch, K staged through shared memory 32 at a time.
template <typename T>
__global__ void __launch_bounds__(256) plain_contract_kernel(PlaneView a, PlaneView b, PlaneView d) {
    __shared__ float sa[32][33];
    __shared__ float sb[32][33];
    const long long plane = blockIdx.z;
    const int i0 = blockIdx.y * 32, j0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long long K = a.cols;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (long long k0 = 0; k0 < K; k0 += 32) {
        for (int e = threadIdx.x; e < 1024; e += 256) {
            const int rr = e >> 5, kk = e & 31;
            const long long k = k0 + kk;
            sa[rr][kk] = (i0 + rr < a.rows && k < K) ? load_f<T>((const T*)a.base + a.offset(plane, i0 + rr, k)) : 0.f;
            sb[rr][kk] = (j0 + rr < b.rows && k < K) ? load_f<T>((const T*)b.base + b.offset(plane, j0 + rr, k)) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
            const float a0 = sa[ty][kk], a1 = sa[ty + 16][kk];
            const float b0 = sb[tx][kk], b1 = sb[tx + 16][kk];
            acc[0][0] = fmaf(a0, b0, acc[0][0]);
            acc[0][1] = fmaf(a0, b1, acc[0][1]);
            acc[1][0] = fmaf(a1, b0, acc[1][0]);
            acc[1][1] = fmaf(a1, b1, acc[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            const long long i = i0 + ty + 16 * u, j = j0 + tx + 16 * v;
            if (i < d.rows && j < d.cols) ((T*)d.base)[d.offset(plane, i, j)] = store_t<T>(acc[u][v]);
        }
}

struct PlainTm2Params {
    int B, rows, N, c;
    int h;      // channels of tri / LayerNorm_out / in_features of w_out (c, or 2c for the bidirectional block)
    const float *gamma_in, *beta_in, *gamma_out, *beta_out;
    float eps_in, eps_out;
    const void *w_gate, *w_out;
    PlaneView tri;
    const void* drop_scale;   // [B, 1, N, c] row-broadcast multiplier of the block output, or null
};

// grid: B * rows * ceil(N / kPlainPos); block kPlainThreads
template <typename T>
__global__ void __launch_bounds__(kPlainThreads)
plain_tm2_kernel(const T* __restrict__ z, T* __restrict__ out, const T* __restrict__ residual, PlainTm2Params p) {
    __shared__ float xs[kPlainPos * kPlainMaxC];
    __shared__ float ts[kPlainPos * kPlainMaxC];
    const int c = p.c, h = p.h;
    const int tiles = (p.N + kPlainPos - 1) / kPlainPos;
    const int s0 = (blockIdx.x % tiles) * kPlainPos;
    const int br = blockIdx.x / tiles;
    const int r = br % p.rows;
    const int b = br / p.rows;
    const int npos = min(kPlainPos, p.N - s0);
    const long long pos0 = (((long long)b * p.rows + r) * p.N + s0);
    for (int i = threadIdx.x; i < npos * c; i += blockDim.x) xs[i] = load_f<T>(z + pos0 * c + i);
    for (int i = threadIdx.x; i < npos * h; i += blockDim.x) {
        const int ch = i / npos, q = i % npos;   // consecutive threads walk the contiguous position axis
        ts[q * h + ch] = load_f<T>((const T*)p.tri.base + p.tri.offset((long long)b * h + ch, r, s0 + q));
    }
    __syncthreads();
    plain_layernorm_rows<T>(xs, npos, c, p.gamma_in, p.beta_in, p.eps_in);
    plain_layernorm_rows<T>(ts, npos, h, p.gamma_out, p.beta_out, p.eps_out);
    __syncthreads();
    const T* Wg = (const T*)p.w_gate;
    const T* Wo = (const T*)p.w_out;
    for (int o = threadIdx.x; o < c; o += blockDim.x) {
        float g[kPlainPos], v[kPlainPos];
#pragma unroll
        for (int q = 0; q < kPlainPos; ++q) g[q] = v[q] = 0.f;
        for (int k = 0; k < c; ++k) {
            const float wg = load_f<T>(Wg + (long long)o * c + k);
#pragma unroll
            for (int q = 0; q < kPlainPos; ++q) g[q] = fmaf(wg, xs[q * c + k], g[q]);
        }
        for (int k = 0; k < h; ++k) {
            const float wo = load_f<T>(Wo + (long long)o * h + k);
#pragma unroll
            for (int q = 0; q < kPlainPos; ++q) v[q] = fmaf(wo, ts[q * h + k], v[q]);
        }
        for (int q = 0; q < npos; ++q) {
            float y = sigmoid_ref(g[q]) * v[q];
            if (p.drop_scale != nullptr)   // applied to the rounded block output, as out * scale would
                y = round_t<T>(y) * load_f<T>((const T*)p.drop_scale + ((long long)b * p.N + s0 + q) * c + o);
            if (residual != nullptr) y = round_t<T>(y) + load_f<T>(residual + (pos0 + q) * c + o);
            out[(pos0 + q) * c + o] = store_t<T>(y);
        }
    }
}

}  // namespace trimul
