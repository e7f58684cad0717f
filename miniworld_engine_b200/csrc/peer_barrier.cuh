// Cross-GPU barrier of the collective-free multi-GPU block, and a self-test of the bounded waits.
//
// peer_barrier_kernel: every rank owns an array of `world` 32-bit flags in memory that all ranks
// of the node can write (peer-mapped).  Barrier number `epoch` (1, 2, 3, ... — the same on every
// rank, counted by the host) is: thread t stores `epoch` into flag [rank] of rank t's array with
// release semantics at system scope, then polls flag [t] of its OWN array with acquire semantics
// until it holds at least `epoch`.  Launched in stream order between two stages, it makes every
// peer's stores of the stage before visible before the stage after reads them.  The poll is
// bounded: after `timeout_ns` the thread writes {TRIMUL_E_DEVICE_TIMEOUT, stage 9, rank it waited
// for, epoch} to the status words and returns, so a rank that stopped between steps cannot leave
// its peers spinning.  Plain peer loads and stores only: no multicast objects are involved.
//
// expire_wait_kernel: initialises an mbarrier that nothing will ever complete and waits on it
// with the given limit — the wait gives up, reports through the status words and the kernel
// returns normally.  It exists so that a test can see the report path work.
#pragma once

#include "ptx_sm100.cuh"

namespace trimul {

constexpr int kStageIdBarrier = 9;
constexpr int kStageIdSelfTest = 10;

struct PeerFlags {
    int32_t* flags[kMaxDest];   // flags[r]: rank r's flag array (world entries), writable from this GPU
};

__global__ void peer_barrier_kernel(const PeerFlags pf, int rank, int world, uint32_t epoch, uint64_t timeout_ns,
                                    int32_t* status) {
    const int t = threadIdx.x;
    if (t >= world) return;
    // everything this GPU wrote before the barrier (the stage before, in stream order) is ordered
    // before the flag by the release; the fence covers stores issued through other proxies
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pf.flags[t] + rank), "r"(epoch) : "memory");
    const int32_t* mine = pf.flags[rank] + t;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t it = 0;; ++it) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int32_t)(v - epoch) >= 0) return;
        __nanosleep(64);
        if ((it & 15u) == 15u && global_timer_ns() - t0 > timeout_ns) break;
    }
    if (status != nullptr && atomicCAS(status, 0, kErrDeviceTimeout) == 0) {
        status[1] = kStageIdBarrier;
        status[2] = t;                  // the rank that never arrived
        status[3] = (int32_t)epoch;
    }
}

__global__ void expire_wait_kernel(uint64_t timeout_ns, int32_t* status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_mbarrier_init();
    }
    __syncthreads();
    // one poller, the rest of the warp group parked at a named barrier: the shape every wait of
    // the stage kernels has
    const bool ok = group_wait<true>(&bar, 0, threadIdx.x == 0, 1, (int)blockDim.x, &abort_flag, status,
                                     kStageIdSelfTest, 77, timeout_ns);
    if (!ok && threadIdx.x == 0 && status != nullptr) atomicAdd(status + 3, 1000);   // detail 77 -> 1077: tear-down ran
}

}  // namespace trimul
