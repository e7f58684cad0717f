// Thin inline-PTX wrappers for the sm_100a features the tensor-core kernels use:
// mbarrier, TMA (cp.async.bulk.tensor, no multicast anywhere), tcgen05 (TMEM allocation,
// UMMA issue/commit, TMEM loads) and the shared-memory / instruction descriptors.
//
// Every wait in this file is bounded: it gives up after a fixed time, raises a
// CTA-wide abort flag and reports through the caller's status words, so a protocol bug
// ends the kernel instead of hanging the device.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace trimul {

// ---------------------------------------------------------------------------------------
// status reporting (4 int32 words in global memory, may be null)
// ---------------------------------------------------------------------------------------
constexpr int kErrDeviceTimeout = -5;

__device__ __forceinline__ void report_timeout(int32_t* status, int stage, int detail) {
    if (status != nullptr) {
        if (atomicCAS(status, 0, kErrDeviceTimeout) == 0) {
            status[1] = stage;
            status[2] = (int)blockIdx.x;
            status[3] = detail;
        }
    }
}

// ---------------------------------------------------------------------------------------
// optional timeline tracing (compiled in only with -DTRIMUL_TRACE): block 0 stamps the global
// nanosecond timer for sixteen local tile indices (from 8 unless TRIMUL_TRACE_FIRST says otherwise) into a device array that a debug entry point
// copies out.  Layout: [role][tile - 8][event], 8 roles x 16 tiles x 4 events.
// ---------------------------------------------------------------------------------------
#ifdef TRIMUL_TRACE
#ifndef TRIMUL_TRACE_FIRST
#define TRIMUL_TRACE_FIRST 8u
#endif
__device__ unsigned long long g_trace[8 * 16 * 4];
#define TRIMUL_STAMP(role, it, ev)                                                             \
    do {                                                                                       \
        if (blockIdx.x == 0 && (it) >= TRIMUL_TRACE_FIRST && (it) < TRIMUL_TRACE_FIRST + 16u) { \
            unsigned long long t_;                                                             \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                             \
            g_trace[((role) * 16 + ((it) - TRIMUL_TRACE_FIRST)) * 4 + (ev)] = t_;              \
        }                                                                                      \
    } while (0)
#else
#define TRIMUL_STAMP(role, it, ev) do { } while (0)
#endif

// ---------------------------------------------------------------------------------------
// shared-memory addresses, fences
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Make generic-proxy writes to shared memory visible to the async proxy (TMA stores, UMMA reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_mbarrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(pred));
    return pred;
}

// Named barrier among a subset of warps (ids 1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

// One poll.  The suspend-time hint lets the hardware park the thread (no issue slots used)
// until the phase completes or the hint (nanoseconds) runs out, whichever comes first.
constexpr uint32_t kTryWaitHintNs = 20000u;

__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kTryWaitHintNs)
        : "memory");
    return done;
}

// Time budget of one wait.  A polling thread costs issue slots that the working warps of the same
// scheduler need (the suspend hint does not park it for long): after a handful of immediate
// polls each further poll is preceded by a short sleep, and every 64th poll compares the global
// nanosecond timer with the moment the slow path was entered.  One second is far beyond any
// legitimate wait in these kernels and short enough that a protocol bug returns control to the
// host with the context intact.  For the same reason a group of warps never polls with more
// than one thread (group_wait below).
#ifndef TRIMUL_HOT_POLLS
#define TRIMUL_HOT_POLLS 8
#endif
#ifndef TRIMUL_POLL_SLEEP_NS
#define TRIMUL_POLL_SLEEP_NS 32
#endif
constexpr uint32_t kHotPolls = TRIMUL_HOT_POLLS;
constexpr uint32_t kPollSleepNs = TRIMUL_POLL_SLEEP_NS;
constexpr uint64_t kWaitNs = 1000ull * 1000ull * 1000ull;

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  `abort_flag` is a CTA-shared word: once any thread of the CTA has timed out,
// every other wait in the CTA returns false promptly, and all roles fall through to the
// kernel's tear-down.  Returns true when the phase completed.
// kOutOfLine = true keeps the polling loop out of line.  Kernels that wait in dozens of places
// and have large epilogues can outgrow the SM's instruction cache when the loop is inlined
// everywhere (instruction-cache hit rates of 60-90 % and the instruction-fetch path near its
// peak were measured); for them the call is cheaper than the misses.
__device__ __forceinline__ bool mbar_wait_loop(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               int32_t* status, int stage, int detail, uint64_t limit_ns = kWaitNs) {
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it >= kHotPolls) {
            __nanosleep(kPollSleepNs);
            if ((it & 63u) == 0u) {
                if (*abort_flag != 0) return false;
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > limit_ns) break;
            }
        }
    }
    *abort_flag = 1;
    report_timeout(status, stage, detail);
    return false;
}
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                            int32_t* status, int stage, int detail, uint64_t limit_ns) {
    return mbar_wait_loop(bar, parity, abort_flag, status, stage, detail, limit_ns);
}
template <bool kOutOfLine = false>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* status, int stage, int detail, uint64_t limit_ns = kWaitNs) {
    if (kOutOfLine) {
        if (mbar_try_wait(bar, parity)) return true;
        return mbar_wait_slow(bar, parity, abort_flag, status, stage, detail, limit_ns);
    }
    return mbar_wait_loop(bar, parity, abort_flag, status, stage, detail, limit_ns);
}

// Collective AND over the `nthreads` threads that share named barrier `id`: every one of them
// gets the same answer, so a group either continues together or leaves together.
__device__ __forceinline__ bool named_barrier_all(int id, int nthreads, bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "bar.red.and.pred q, %2, %3, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t"
        "}\n"
        : "=r"(r)
        : "r"((uint32_t)ok), "r"(id), "r"(nthreads)
        : "memory");
    return r != 0;
}

// Wait of a whole warp group on one mbarrier phase: ONE thread polls (bounded), the others park
// at the group's named barrier, which costs them no issue slots; the barrier also hands the
// poller's verdict and its view of memory to every thread of the group.
template <bool kOutOfLine = false>
__device__ __forceinline__ bool group_wait(uint64_t* bar, uint32_t parity, bool poller, int bar_id, int nthreads,
                                           volatile int* abort_flag, int32_t* status, int stage, int detail,
                                           uint64_t limit_ns = kWaitNs) {
    bool ok = true;
    if (poller) ok = mbar_wait<kOutOfLine>(bar, parity, abort_flag, status, stage, detail, limit_ns);
    return named_barrier_all(bar_id, nthreads, ok);
}

// ---------------------------------------------------------------------------------------
// TMA (tensor maps are passed as __grid_constant__ kernel parameters)
// ---------------------------------------------------------------------------------------
// Destination maps of the scattering kernel variants: one tensor map per destination buffer
// (another GPU's memory, mapped into this process, or a local buffer).  Only STORES go through
// these maps.
constexpr int kMaxDest = 8;
struct ScatterMaps {
    CUtensorMap map[kMaxDest];
};

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, "
        "%6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* src, int c0, int c1, int c2,
                                             int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Wait until at most N of this thread's bulk store groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Wait until at most N of this thread's bulk store groups are incomplete (writes performed).
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------
// tcgen05: TMEM allocation (one warp, .sync.aligned), fences, commit
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrive on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---------------------------------------------------------------------------------------
// UMMA descriptors
// ---------------------------------------------------------------------------------------
// Shared-memory operand descriptor for a K-major bf16 tile stored as rows of 64 elements
// (128 bytes) with the 128-byte swizzle — exactly what a TMA load with SWIZZLE_128B and a
// 64-element inner box writes.  Eight rows form a 1024-byte group; groups are contiguous.
//   bits [0,14)  start address >> 4          bits [16,30) leading byte offset >> 4 (unused here: 1)
//   bits [32,46) stride byte offset >> 4 (1024 B between 8-row groups)
//   bits [46,48) descriptor version = 1 on sm_100        bits [61,64) layout: 2 = SWIZZLE_128B
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Shared-memory operand descriptor for an MN-major bf16 tile with the 128-byte swizzle: each
// row is one K index and holds 64 consecutive M (or N) elements (128 bytes) — what a TMA load
// with SWIZZLE_128B and a 64-element inner box writes when the contiguous tensor dimension is
// the operand's M/N dimension.  Eight K rows form a 1024-byte group.
//   leading byte offset = distance between consecutive 64-element blocks along M/N
//   stride  byte offset = distance between consecutive 8-row groups along K
// One UMMA (K = 16) consumes two 8-row groups, so stepping K by 16 adds 2 * sbo_bytes.
__device__ __forceinline__ uint64_t umma_smem_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Advancing a K-major SWIZZLE_128B descriptor by one UMMA K step (16 bf16 = 32 bytes) inside the
// 128-byte row: add 32 >> 4 to the start-address field.
constexpr uint64_t kDescKStep = 32u >> 4;

// Instruction descriptor for kind::f16 with bf16 A/B (both K-major), fp32 accumulate.
//   [4,6) D format: 1 = f32    [7,10) A format: 1 = bf16    [10,13) B format: 1 = bf16
//   [15] A major: 0 = K        [16] B major: 0 = K          [17,23) N >> 3        [24,29) M >> 4
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int a_mn_major = 0, int b_mn_major = 0) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by ONE thread.
__device__ __forceinline__ void umma_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]^T: the A operand is read from tensor memory, 128 lanes (rows) x 16
// bf16 per UMMA stored two per 32-bit column (8 columns per K step of 16).
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

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization
// attribute may start while the kernel before it in the stream is still running; nothing the
// predecessor wrote may be read (and nothing it reads may be overwritten) before
// griddep_wait() returns, which happens once the predecessor has completed and its memory
// operations are visible.  Without the launch attribute both instructions are no-ops.
// griddep_launch_dependents() lets the NEXT kernel in the stream be scheduled as soon as every
// CTA of this grid has executed it (its CTAs then take over SMs as this grid's CTAs retire).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------------------
// TMEM -> registers: 32 lanes x 32 consecutive fp32 columns; thread t of the warp gets lane
// (warp_id % 4) * 32 + t.  The address carries the lane in bits [16,32) and the column in [0,16).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// Same, 16 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// Same, 8 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// small math helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// sigmoid(x) = 0.5 * tanh(0.5 x) + 0.5 with the hardware tanh: one MUFU operation per value
// (absolute error ~5e-4 of tanh.approx, i.e. ~2.5e-4 on the gate — a quarter of a bf16 ulp at 1).
__device__ __forceinline__ float sigmoid_fast(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(0.5f, t, 0.5f);
}

// ---------------------------------------------------------------------------------------
// CTA pairs (clusters of two, tcgen05 cta_group::2).  No TMA multicast is used anywhere: a pair's
// loads land in the issuing CTA and only their completion is signalled across the pair.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// Arrive on a barrier of the PEER CTA, with release semantics at CTA scope (what the instruction
// defaults to).  That is enough when what the arrival publishes is this CTA's own shared or tensor
// memory, which the pair's UMMAs read in place, and far cheaper than `.release.cluster`, which was
// measured to hold the arriving warp for more than a microsecond.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of a CTA pair: data lands in this CTA, completion is signalled on `bar_cluster_addr`
// (a shared::cluster address, here always the leader's barrier).  No multicast.
__device__ __forceinline__ void tma_load_4d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
        "%4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A . B^T with A, B halves in both CTAs' shared memory; ONE thread of
// the leader CTA issues it.
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                  uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the barrier at the same offset in BOTH CTAs once the pair's UMMAs issued so far retire.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"(mask)
        : "memory");
}


// ---------------------------------------------------------------------------------------
// Packed fp32 pairs (sm_100 executes add/mul/fma on two fp32 lanes per instruction).  A pair
// lives in a 64-bit register; the helpers below are what the LayerNorm and gate code is
// written in, which halves its arithmetic instruction count.
// ---------------------------------------------------------------------------------------
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 f2_pack(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// bf16x2 word -> (lo, hi) as fp32 pair, and back with round-to-nearest-even
__device__ __forceinline__ f32x2 f2_from_bf16x2(uint32_t w) { return f2_pack(bf16_lo(w), bf16_hi(w)); }
__device__ __forceinline__ uint32_t f2_to_bf16x2(f32x2 v) {
    float lo, hi;
    f2_unpack(v, lo, hi);
    return pack_bf16x2(lo, hi);
}
__device__ __forceinline__ float f2_hsum(f32x2 v) {
    float lo, hi;
    f2_unpack(v, lo, hi);
    return lo + hi;
}

__device__ __forceinline__ float tanh_fast(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
    return t;
}

// p * sigmoid(g) from HALVED inputs hp = p/2, hg = g/2:  p*sigmoid(g) = hp*tanh(hg) + hp.
// The kernels halve the weight matrices once in shared memory (exact in bf16), so the
// accumulators already hold hp and hg and the gate costs one MUFU and one FMA per value.
__device__ __forceinline__ float gate_from_halves(float hp, float hg) { return fmaf(hp, tanh_fast(hg), hp); }
// two gates at once, result rounded to a bf16x2 word
__device__ __forceinline__ uint32_t gate2_bf16(float hp0, float hg0, float hp1, float hg1) {
    const f32x2 hp = f2_pack(hp0, hp1);
    return f2_to_bf16x2(f2_fma(hp, f2_pack(tanh_fast(hg0), tanh_fast(hg1)), hp));
}

// the same from UNHALVED p and g (kernels that stream their weights and cannot halve them once)
__device__ __forceinline__ uint32_t gate2_full_bf16(float p0, float g0, float p1, float g1) {
    const f32x2 half2 = f2_pack(0.5f, 0.5f);
    const f32x2 hp = f2_mul(f2_pack(p0, p1), half2);
    return f2_to_bf16x2(f2_fma(hp, f2_pack(tanh_fast(0.5f * g0), tanh_fast(0.5f * g1)), hp));
}

// Multiply `nbytes` of bf16 data in shared memory by 0.5 in place (exact: only the exponent
// changes), work split over `nthreads` cooperating threads with rank `tid`.
__device__ __forceinline__ void halve_bf16_smem(uint8_t* base, int nbytes, int tid, int nthreads) {
    const __nv_bfloat162 half2 = __floats2bfloat162_rn(0.5f, 0.5f);
    for (int i = tid; i < nbytes / 16; i += nthreads) {
        uint4 v = *reinterpret_cast<uint4*>(base + i * 16);
        __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) e[k] = __hmul2(e[k], half2);
        *reinterpret_cast<uint4*>(base + i * 16) = v;
    }
}

// ---------------------------------------------------------------------------------------
// LayerNorm of one 128-channel row of a tile pair stored as two [128 rows][64 ch] SWIZZLE_128B
// sub-tiles (`sub_bytes` apart), done IN PLACE by two cooperating threads that sit in adjacent
// lanes: thread h (0/1) owns 16-byte chunks 4h..4h+3 of each sub-tile, i.e. channels
// [32h, 32h+32) and [64+32h, 64+32h+32).  Two passes over shared memory with small loop bodies:
//   1. shifted sums (shift = the row's first element) -> mean, variance without cancellation
//   2. normalise, affine, round to bf16, store back
// `zero_row` stores zeros instead (masked position: the projections of a zero row are exactly 0);
// such a thread still runs both passes, because the pair exchanges partial sums by warp shuffle.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void ln_half_row_inplace(uint8_t* tile, int sub_bytes, int row, int h,
                                                    const float* sGamma, const float* sBeta, float eps,
                                                    bool zero_row) {
    const uint32_t swz = (uint32_t)(row & 7);
    uint8_t* rowp = tile + row * 128;
    // NOTE: no early exit for masked rows — the shuffles below need every lane of the warp.
    // shift: channel 0 lives in chunk 0 of sub-tile 0
    const uint32_t first = *reinterpret_cast<const uint32_t*>(rowp + (swz << 4));
    const float shift = bf16_lo(first);
    const f32x2 nshift = f2_pack(-shift, -shift);
    f32x2 s1 = 0ull, s2 = 0ull;   // (even, odd) element lanes; 0ull is the pair (+0.f, +0.f)
#pragma unroll 1
    for (int s = 0; s < 2; ++s) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const uint4 v = *reinterpret_cast<const uint4*>(rowp + s * sub_bytes + ((((uint32_t)(4 * h + jj)) ^ swz) << 4));
            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const f32x2 d = f2_add(f2_from_bf16x2(w4[e]), nshift);
                s1 = f2_add(s1, d);
                s2 = f2_fma(d, d, s2);
            }
        }
    }
    float t1 = f2_hsum(s1), t2 = f2_hsum(s2);
    t1 += __shfl_xor_sync(0xffffffffu, t1, 1);
    t2 += __shfl_xor_sync(0xffffffffu, t2, 1);
    const float m1 = t1 * (1.0f / 128.0f);
    const float var = fmaxf(fmaf(-m1, m1, t2 * (1.0f / 128.0f)), 0.f);
    const float rstd = rsqrtf(var + eps);
    const float nmr = -(shift + m1) * rstd;   // y = x*rstd + nmr
    const f32x2 rstd2 = f2_pack(rstd, rstd), nmr2 = f2_pack(nmr, nmr);
#pragma unroll 1
    for (int s = 0; s < 2; ++s) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int j = 4 * h + jj;
            uint4* p = reinterpret_cast<uint4*>(rowp + s * sub_bytes + ((((uint32_t)j) ^ swz) << 4));
            const uint4 v = *p;
            const int ch = s * 64 + j * 8;
            const float4 g0 = *reinterpret_cast<const float4*>(sGamma + ch);
            const float4 g1 = *reinterpret_cast<const float4*>(sGamma + ch + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(sBeta + ch);
            const float4 b1 = *reinterpret_cast<const float4*>(sBeta + ch + 4);
            uint4 o;
            o.x = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v.x), rstd2, nmr2), f2_pack(g0.x, g0.y), f2_pack(b0.x, b0.y)));
            o.y = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v.y), rstd2, nmr2), f2_pack(g0.z, g0.w), f2_pack(b0.z, b0.w)));
            o.z = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v.z), rstd2, nmr2), f2_pack(g1.x, g1.y), f2_pack(b1.x, b1.y)));
            o.w = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v.w), rstd2, nmr2), f2_pack(g1.z, g1.w), f2_pack(b1.z, b1.w)));
            if (zero_row) o = make_uint4(0u, 0u, 0u, 0u);
            *p = o;
        }
    }
}

// ---------------------------------------------------------------------------------------
// LayerNorm of one 128-channel row by ONE thread, in place, same tile layout as above.  All lanes
// of a warp work on the same chunk index at the same time, so the gamma/beta vector loads are
// warp-uniform (one shared-memory wavefront each) and the tile accesses are conflict-free:
// this variant moves about a third of the shared-memory wavefronts of the two-thread one, which
// matters because these kernels are bound by shared-memory bandwidth, not by arithmetic.
// ---------------------------------------------------------------------------------------
template <int kSub = 2>
__device__ __forceinline__ void ln_row_inplace(uint8_t* tile, int sub_bytes, int row, const float* sGamma,
                                               const float* sBeta, float eps, bool zero_row) {
    // kSub = number of 64-channel sub-tiles of a row (2: 128 channels, 4: 256 channels)
    constexpr float kInvC = 1.0f / (64.0f * kSub);
    const uint32_t swz = (uint32_t)(row & 7);
    uint8_t* rowp = tile + row * 128;
    const uint32_t first = *reinterpret_cast<const uint32_t*>(rowp + (swz << 4));
    const float shift = bf16_lo(first);
    const f32x2 nshift = f2_pack(-shift, -shift);
    // four independent accumulator pairs keep the dependent add/fma chains short
    f32x2 s1[4] = {0ull, 0ull, 0ull, 0ull}, s2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll 1
    for (int s = 0; s < kSub; ++s) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint4 v = *reinterpret_cast<const uint4*>(rowp + s * sub_bytes + ((((uint32_t)j) ^ swz) << 4));
            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const f32x2 d = f2_add(f2_from_bf16x2(w4[e]), nshift);
                s1[e] = f2_add(s1[e], d);
                s2[e] = f2_fma(d, d, s2[e]);
            }
        }
    }
    const float m1 = f2_hsum(f2_add(f2_add(s1[0], s1[1]), f2_add(s1[2], s1[3]))) * kInvC;
    const float q1 = f2_hsum(f2_add(f2_add(s2[0], s2[1]), f2_add(s2[2], s2[3])));
    const float var = fmaxf(fmaf(-m1, m1, q1 * kInvC), 0.f);
    const float rstd = rsqrtf(var + eps);
    const float nmr = -(shift + m1) * rstd;
    const f32x2 rstd2 = f2_pack(rstd, rstd), nmr2 = f2_pack(nmr, nmr);
#pragma unroll 1
    for (int s = 0; s < kSub; ++s) {
#pragma unroll 4
        for (int j = 0; j < 8; ++j) {
            uint4* p = reinterpret_cast<uint4*>(rowp + s * sub_bytes + ((((uint32_t)j) ^ swz) << 4));
            const uint4 v = *p;
            const int ch = s * 64 + j * 8;
            const float4 g0 = *reinterpret_cast<const float4*>(sGamma + ch);
            const float4 g1 = *reinterpret_cast<const float4*>(sGamma + ch + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(sBeta + ch);
            const float4 b1 = *reinterpret_cast<const float4*>(sBeta + ch + 4);
            uint4 o;
            o.x = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v.x), rstd2, nmr2), f2_pack(g0.x, g0.y), f2_pack(b0.x, b0.y)));
            o.y = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v.y), rstd2, nmr2), f2_pack(g0.z, g0.w), f2_pack(b0.z, b0.w)));
            o.z = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v.z), rstd2, nmr2), f2_pack(g1.x, g1.y), f2_pack(b1.x, b1.y)));
            o.w = f2_to_bf16x2(f2_fma(f2_fma(f2_from_bf16x2(v.w), rstd2, nmr2), f2_pack(g1.z, g1.w), f2_pack(b1.z, b1.w)));
            if (zero_row) o = make_uint4(0u, 0u, 0u, 0u);
            *p = o;
        }
    }
}

// ---------------------------------------------------------------------------------------
// LayerNorm of 4 * kIters consecutive rows (first row `row0`, a multiple of 8) of a tile of
// 64 * kSub channels (kSub swizzled 64-channel sub-tiles, `sub_bytes` apart) by ONE WARP, in place.
// Eight lanes share a row: lane l works on row row0 + 4 i + (l >> 3) in iteration i and owns 16-byte
// chunk l & 7 of every sub-tile, i.e. channels [64 s + 8 j, 64 s + 8 j + 8), j = l & 7.  Every value
// is read from shared memory ONCE and stays in registers between the statistics and the
// normalisation; gamma and beta of the lane's channels live in registers (`gb`: gamma pairs
// [0, 4 kSub), beta pairs [4 kSub, 8 kSub), see ln_load_affine), so no affine vector is fetched per
// row; the row sums are combined by a three-step butterfly over the eight lanes.  A quarter warp
// reads or writes one whole 128-byte swizzled row segment: conflict-free.  Bit i of `zero_bits` set
// -> the lane's row of iteration i is a masked position and is written as zeros.
// ---------------------------------------------------------------------------------------
template <int kIters, int kSub = 2>
__device__ __forceinline__ void ln_rows_warp(uint8_t* tile, int sub_bytes, int row0, int lane,
                                             const f32x2 (&gb)[8 * kSub], float eps, uint32_t zero_bits) {
    const int rr = lane >> 3;
    const uint32_t j = (uint32_t)lane & 7u;
    constexpr float kInvC = 1.0f / (64.0f * kSub);
#pragma unroll 2
    for (int i = 0; i < kIters; ++i) {
        const int r = row0 + 4 * i + rr;
        const uint32_t off = (uint32_t)r * 128u + ((j ^ ((uint32_t)r & 7u)) << 4);
        uint4 v[kSub];
#pragma unroll
        for (int s = 0; s < kSub; ++s) v[s] = *reinterpret_cast<const uint4*>(tile + s * sub_bytes + off);
        // common shift of the row: its channel 0 (held by the lane with j == 0)
        const float shift = bf16_lo(__shfl_sync(0xffffffffu, v[0].x, lane & 24));
        const f32x2 ns = f2_pack(-shift, -shift);
        f32x2 d[4 * kSub];
#pragma unroll
        for (int s = 0; s < kSub; ++s) {
            d[4 * s + 0] = f2_add(f2_from_bf16x2(v[s].x), ns);
            d[4 * s + 1] = f2_add(f2_from_bf16x2(v[s].y), ns);
            d[4 * s + 2] = f2_add(f2_from_bf16x2(v[s].z), ns);
            d[4 * s + 3] = f2_add(f2_from_bf16x2(v[s].w), ns);
        }
        // per 64-channel sub-tile: a short sum tree and a four-deep FMA chain, then the sub-tiles added up
        // (for two sub-tiles this is the order (s0 + s1), the same in every kernel that normalises 128 channels)
        f32x2 sum = 0ull, sq = 0ull;
#pragma unroll
        for (int s = 0; s < kSub; ++s) {
            const f32x2 sa = f2_add(f2_add(d[4 * s], d[4 * s + 1]), f2_add(d[4 * s + 2], d[4 * s + 3]));
            const f32x2 qa = f2_fma(d[4 * s], d[4 * s],
                                    f2_fma(d[4 * s + 1], d[4 * s + 1],
                                           f2_fma(d[4 * s + 2], d[4 * s + 2], f2_fma(d[4 * s + 3], d[4 * s + 3], 0ull))));
            sum = s == 0 ? sa : f2_add(sum, sa);
            sq = s == 0 ? qa : f2_add(sq, qa);
        }
        float t1 = f2_hsum(sum), t2 = f2_hsum(sq);
#pragma unroll
        for (int o = 4; o >= 1; o >>= 1) {
            t1 += __shfl_xor_sync(0xffffffffu, t1, o);
            t2 += __shfl_xor_sync(0xffffffffu, t2, o);
        }
        const float m1 = t1 * kInvC;
        const float var = fmaxf(fmaf(-m1, m1, t2 * kInvC), 0.f);
        const float rstd = rsqrtf(var + eps);
        const float nm = -m1 * rstd;                       // y = d * rstd + nm
        const f32x2 r2 = f2_pack(rstd, rstd), n2 = f2_pack(nm, nm);
        const bool zero = (zero_bits >> i) & 1u;
#pragma unroll
        for (int s = 0; s < kSub; ++s) {
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
                o[k] = zero ? 0u
                            : f2_to_bf16x2(f2_fma(f2_fma(d[4 * s + k], r2, n2), gb[4 * s + k], gb[4 * kSub + 4 * s + k]));
            *reinterpret_cast<uint4*>(tile + s * sub_bytes + off) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// gamma and beta of a lane's channels for ln_rows_warp, from global memory: lane chunk j = lane & 7 owns
// channels [64 s + 8 j, 64 s + 8 j + 8) of every sub-tile s.
template <int kSub>
__device__ __forceinline__ void ln_load_affine(f32x2 (&gb)[8 * kSub], const float* gamma, const float* beta, int lane) {
    const int j = lane & 7;
#pragma unroll
    for (int s = 0; s < kSub; ++s) {
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + 64 * s + 8 * j));
        const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma + 64 * s + 8 * j + 4));
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta + 64 * s + 8 * j));
        const float4 b1 = __ldg(reinterpret_cast<const float4*>(beta + 64 * s + 8 * j + 4));
        gb[4 * s + 0] = f2_pack(g0.x, g0.y); gb[4 * s + 1] = f2_pack(g0.z, g0.w);
        gb[4 * s + 2] = f2_pack(g1.x, g1.y); gb[4 * s + 3] = f2_pack(g1.z, g1.w);
        gb[4 * kSub + 4 * s + 0] = f2_pack(b0.x, b0.y); gb[4 * kSub + 4 * s + 1] = f2_pack(b0.z, b0.w);
        gb[4 * kSub + 4 * s + 2] = f2_pack(b1.x, b1.y); gb[4 * kSub + 4 * s + 3] = f2_pack(b1.z, b1.w);
    }
}

// Mean / rstd of one 128-channel row of a swizzled z tile (one pass, sums shifted by the row's
// first element so the variance does not cancel).  Returns rstd and t = -mean * rstd.
__device__ __forceinline__ void row_stats(const uint8_t* tile, int sub_bytes, int row, float eps, float& rstd,
                                          float& t) {
    const uint32_t swz = (uint32_t)(row & 7);
    const uint8_t* rowp = tile + row * 128;
    const uint32_t first = *reinterpret_cast<const uint32_t*>(rowp + (swz << 4));
    const float shift = bf16_lo(first);
    const f32x2 nshift = f2_pack(-shift, -shift);
    f32x2 s1[4] = {0ull, 0ull, 0ull, 0ull}, s2[4] = {0ull, 0ull, 0ull, 0ull};
    // (short loop bodies on purpose: see the note on instruction-cache pressure at mbar_wait_slow)
#pragma unroll 1
    for (int s = 0; s < 2; ++s) {
#pragma unroll 4
        for (int j = 0; j < 8; ++j) {
            const uint4 v = *reinterpret_cast<const uint4*>(rowp + s * sub_bytes + ((((uint32_t)j) ^ swz) << 4));
            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const f32x2 d = f2_add(f2_from_bf16x2(w4[e]), nshift);
                s1[e] = f2_add(s1[e], d);
                s2[e] = f2_fma(d, d, s2[e]);
            }
        }
    }
    const float m1 = f2_hsum(f2_add(f2_add(s1[0], s1[1]), f2_add(s1[2], s1[3]))) * (1.0f / 128.0f);
    const float q1 = f2_hsum(f2_add(f2_add(s2[0], s2[1]), f2_add(s2[2], s2[3])));
    const float var = fmaxf(fmaf(-m1, m1, q1 * (1.0f / 128.0f)), 0.f);
    rstd = rsqrtf(var + eps);
    t = -(shift + m1) * rstd;
}


// Fold one row (output channel n) of a weight matrix that lies in shared memory as `nsub` swizzled
// 64-column sub-tiles (`sub_bytes` apart): w[k] <- bf16(w[k] * gamma[k] / 2).  Returns the sum of the rounded row and
// 0.5 * sum_k w[k] * beta[k].
__device__ __forceinline__ void fold_row_smem(uint8_t* wbase, int sub_bytes, int n, const float* gamma,
                                              const float* beta, int nsub, float& s, float& bias) {
    float ssum = 0.f, bsum = 0.f;
    const uint32_t swz = (uint32_t)(n & 7);
#pragma unroll 1
    for (int kh = 0; kh < nsub; ++kh) {
#pragma unroll 2
        for (int j = 0; j < 8; ++j) {
            uint4* ptr = reinterpret_cast<uint4*>(wbase + kh * sub_bytes + n * 128 + ((((uint32_t)j) ^ swz) << 4));
            const uint4 v = *ptr;
            const int k0 = kh * 64 + j * 8;
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + k0));
            const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma + k0 + 4));
            const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta + k0));
            const float4 b1 = __ldg(reinterpret_cast<const float4*>(beta + k0 + 4));
            const float ga[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            const float be[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float w0 = bf16_lo(w4[e]), w1 = bf16_hi(w4[e]);
                const uint32_t f = pack_bf16x2(w0 * ga[2 * e] * 0.5f, w1 * ga[2 * e + 1] * 0.5f);
                ssum += bf16_lo(f) + bf16_hi(f);
                bsum = fmaf(w0, be[2 * e], fmaf(w1, be[2 * e + 1], bsum));
                o[e] = f;
            }
            *ptr = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    s = ssum;
    bias = 0.5f * bsum;
}


}  // namespace trimul
