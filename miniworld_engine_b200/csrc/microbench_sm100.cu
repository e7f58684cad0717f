// Micro-benchmarks of the sm_100a resources that bound the stage kernels of this library, one CTA
// per SM; what they print is what the tile shapes in tm1_sm100.cuh / tm1_direct_sm100.cuh and the
// polling rules in ptx_sm100.cuh are based on.
//   1. cycles per tcgen05.mma (kind::f16, M = 128, cta_group::1), A operand in shared memory (ss) or
//      in tensor memory (ts), N = 64 / 128 / 256, issued back to back by one thread;
//   2. the warp-cooperative LayerNorm of a [128][128] bf16 tile by 8 warps, alone and beside the UMMAs;
//   3. tensor memory -> registers (tcgen05.ld 32x32b.x16) with 4, 8 and 16 warps: bytes per cycle and SM;
//   4. the hardware tanh in its f32, f16x2 and bf16x2 forms: results per cycle and SM.
// Build and run:  python -m miniworld_engine_b200.build --microbench && ./miniworld_engine_b200/microbench_sm100
// Every wait is bounded; nothing here can hang.
#include <cstdio>

#include "ptx_sm100.cuh"
using namespace trimul;

__global__ void __launch_bounds__(320, 1) k_umma(int mode_ts, int N, int iters, int with_ln, long long* out) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag = 0; fence_mbarrier_init(); }
    if (warp == 1) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
    for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u + i;
    fence_proxy_async_smem();
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (warp == 1) {
        if (lane == 0 && iters > 0) {
            const uint32_t idesc = umma_idesc_bf16(128, N);
            const uint32_t a_s = smem_u32(smem);             // A: 128 rows x 64 k (16 KB)
            const uint32_t b_s = smem_u32(smem + 32768);     // B: up to 256 rows x 64 k (32 KB)
            const long long t0 = clock64();
            for (int it = 0; it < iters; ++it) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t db = umma_smem_desc_sw128(b_s) + kk * kDescKStep;
                    if (mode_ts) umma_bf16_ts(tmem_base + 256, tmem_base + kk * 8, db, idesc, 1);
                    else umma_bf16_ss(tmem_base + 256, umma_smem_desc_sw128(a_s) + kk * kDescKStep, db, idesc, 1);
                }
            }
            umma_commit(&bar);
            mbar_wait(&bar, 0, &abort_flag, nullptr, 0, 0);
            out[blockIdx.x * 4 + 0] = clock64() - t0;
        }
        __syncwarp();
    } else if (warp >= 2 && with_ln) {
        f32x2 gb[16];
        for (int i = 0; i < 16; ++i) gb[i] = f2_pack(1.f + i, 0.5f);
        const int lw = warp - 2;
        const long long s0 = clock64();
        for (int r = 0; r < with_ln; ++r) {
            ln_rows_warp<4>(smem + 96 * 1024, 16384, 16 * lw, lane, gb, 1e-5f, 0u);
            fence_proxy_async_smem();
            __syncwarp();
        }
        if (lw == 0 && lane == 0) out[blockIdx.x * 4 + 1] = clock64() - s0;
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) { tcgen05_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// `nwarps` warps (4, 8 or 16) read all 512 columns of their TMEM lane quarter `iters` times
__global__ void __launch_bounds__(576, 1) k_tmem_ld(int nwarps, int iters, long long* out, float* sink) {
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5;
    if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (warp >= 2 && warp < 2 + nwarps) {
        const uint32_t t = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        float acc = 0.f;
        const long long t0 = clock64();
        for (int it = 0; it < iters; ++it) {
#pragma unroll 1
            for (int c = 0; c < 512; c += 32) {
                uint32_t a[16], b[16];
                tmem_ld_32x16(t + c, a);
                tmem_ld_32x16(t + c + 16, b);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) acc += __uint_as_float(a[i] ^ b[i]);
            }
        }
        const long long dt = clock64() - t0;
        if (threadIdx.x == 64) out[blockIdx.x] = dt;
        sink[blockIdx.x * blockDim.x + threadIdx.x] = acc;
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) { tcgen05_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int MODE>
__global__ void k_tanh(float* out, int iters) {
    float x[8]; unsigned h[8];
    for (int i = 0; i < 8; ++i) { x[i] = 0.01f * (threadIdx.x + i); h[i] = 0x38003800u + threadIdx.x + i; }
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (MODE == 0) asm volatile("tanh.approx.f32 %0, %0;" : "+f"(x[i]));
            if (MODE == 1) asm volatile("tanh.approx.f16x2 %0, %0;" : "+r"(h[i]));
            if (MODE == 2) asm volatile("tanh.approx.bf16x2 %0, %0;" : "+r"(h[i]));
        }
    }
    float s = 0; for (int i = 0; i < 8; ++i) s += x[i] + __uint_as_float(h[i]);
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}
template <int MODE> void run_tanh(const char* name, float* out, int per_instr, double ghz) {
    const int iters = 4096; cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    k_tanh<MODE><<<148 * 2, 512>>>(out, iters); cudaDeviceSynchronize();
    cudaEventRecord(e0); k_tanh<MODE><<<148 * 2, 512>>>(out, iters); cudaEventRecord(e1); cudaDeviceSynchronize();
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    const double instr = 148.0 * 2 * 512 * 8.0 * iters;
    printf("%-20s %.1f results per cycle and SM (at %.3f GHz)\n", name, per_instr * instr / (ms * 1e-3) / 148 / (ghz * 1e9), ghz);
}

int main() {
    int khz = 0; cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, 0);
    const double ghz = khz * 1e-6;
    long long* out; cudaMalloc(&out, 148 * 4 * 8);
    float* sink; cudaMalloc(&sink, 148 * 2 * 576 * 4);
    cudaFuncSetAttribute(k_umma, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    long long h[148 * 4];
    const int iters = 2000;
    printf("1./2. tcgen05.mma 128 x N x 16, bf16, one accumulator, 8000 in a row; LayerNorm of a 128x128 tile by 8 warps\n");
    for (int ts = 0; ts < 2; ++ts)
        for (int N = 64; N <= 256; N *= 2)
            for (int ln = 0; ln <= 200; ln += 200) {
                cudaMemset(out, 0, sizeof(h));
                k_umma<<<148, 320, 160 * 1024>>>(ts, N, iters, ln, out);
                const cudaError_t e = cudaDeviceSynchronize();
                cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
                printf("  A in %s, N=%3d%s: %6.1f cycles per UMMA (ideal %3d)", ts ? "TMEM" : "smem", N,
                       ln ? ", LayerNorm warps busy" : "                      ", (double)h[0] / (iters * 4), N / 2);
                if (ln) printf(";  LayerNorm %5.0f cycles per tile", (double)h[1] / ln);
                printf("  [%s]\n", cudaGetErrorString(e));
            }
    cudaMemset(out, 0, sizeof(h));
    k_umma<<<148, 320, 160 * 1024>>>(0, 64, 0, 200, out);
    cudaDeviceSynchronize();
    cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
    printf("  LayerNorm alone: %5.0f cycles per tile\n", (double)h[1] / 200);
    printf("3. tcgen05.ld 32x32b.x16, every warp reads the 512 columns of its lane quarter 200 times\n");
    for (int nw = 4; nw <= 16; nw *= 2) {
        cudaMemset(out, 0, sizeof(h));
        k_tmem_ld<<<148, 576>>>(nw, 200, out, sink);
        const cudaError_t e = cudaDeviceSynchronize();
        cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
        const double bytes = (double)nw * 32 * 512 * 4 * 200;
        printf("  %2d warps: %6.1f bytes per cycle and SM  [%s]\n", nw, bytes / (double)h[0], cudaGetErrorString(e));
    }
    printf("4. hardware tanh\n");
    run_tanh<0>("  tanh.approx.f32", sink, 1, ghz);
    run_tanh<1>("  tanh.approx.f16x2", sink, 2, ghz);
    run_tanh<2>("  tanh.approx.bf16x2", sink, 2, ghz);
    return 0;
}
