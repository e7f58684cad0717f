// C-ABI of the B200 TriangleMultiplication block: argument validation, tensor-map
// construction, workspace layout and kernel launches.  Declarations and the reference
// interfaces each entry point replaces are in include/trimul_b200.h.
//
// Nothing here allocates device memory, synchronises or throws.  Tensor maps are built on the
// host per call (a pure CPU encode) and passed by value as kernel parameters, so the entry
// points can be captured in CUDA graphs.

#include "../../include/trimul_b200.h"

#include <atomic>
#include <cstddef>
#include <cstring>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <utility>

#include "contract_sm100.cuh"
#include "contract2_sm100.cuh"
#include "peer_barrier.cuh"
#include "plain_kernels.cuh"
#include "tm1_sm100.cuh"
#include "tm1_pair_sm100.cuh"
#include "tm2_sm100.cuh"
#include "tm2_fold_sm100.cuh"
#include "tm1_wide_sm100.cuh"
#include "tm2_wide_sm100.cuh"
#include "tm1_narrow_sm100.cuh"
#include "tm2_narrow_sm100.cuh"
#include "wmma_kernels.cuh"

using namespace trimul;

// Scratch for trimul_b200_forward_static: the a/b/tri planes of callers that cannot allocate.
// It is part of the device image, so every GPU that loads this library carries it until the
// process exits.  In HOST code this name is only a handle for cudaGetSymbolAddress — it is not
// a device address and must never be passed to a kernel as one.
static __device__ __align__(256) unsigned char g_static_scratch[TRIMUL_B200_STATIC_SCRATCH_BYTES];

namespace {

// ---------------------------------------------------------------------------------------
// driver entry point for tensor-map encoding (resolved at run time: no link against libcuda)
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// bf16 tensor of up to 4 dimensions, innermost first; strides in ELEMENTS for dims 1..3.
bool encode_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_elems,
                 const uint32_t* box, int swizzle_bytes) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t gdim[4];
    cuuint64_t gstride[3];
    cuuint32_t bdim[4];
    cuuint32_t estr[4];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        estr[i] = 1;
    }
    for (int i = 0; i + 1 < rank; ++i) gstride[i] = strides_elems[i] * 2;
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride,
                    bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                    : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                          : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Channel-major planes as a 4-D tensor (col, row-in-chunk, plane, chunk) with the given box.
bool encode_planes(CUtensorMap* map, const trimul_planes& pl, int planes, uint32_t box_cols, uint32_t box_rows,
                   uint32_t box_planes, int swizzle_bytes = 128) {
    const bool row_chunked = pl.row_chunk < pl.rows;
    const bool col_chunked = pl.col_chunk < pl.cols;
    const uint64_t chunks = row_chunked ? (uint64_t)((pl.rows + pl.row_chunk - 1) / pl.row_chunk)
                          : col_chunked ? (uint64_t)((pl.cols + pl.col_chunk - 1) / pl.col_chunk)
                                        : 1;
    const uint64_t dims[4] = {(uint64_t)(col_chunked ? pl.col_chunk : pl.cols),
                              (uint64_t)(row_chunked ? pl.row_chunk : pl.rows), (uint64_t)planes, chunks};
    const uint64_t chunk_stride = chunks > 1 ? (uint64_t)pl.chunk_stride : (uint64_t)pl.plane_stride * planes;
    const uint64_t strides[3] = {(uint64_t)pl.pitch, (uint64_t)pl.plane_stride, chunk_stride};
    const uint32_t box[4] = {box_cols, box_rows, box_planes, 1};
    return encode_bf16(map, pl.base, 4, dims, strides, box, swizzle_bytes);
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 148;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// Opt the kernel in to `bytes` of dynamic shared memory — once per kernel and device: the
// attribute call is not free and these entry points sit on latency-sensitive host paths.
bool ensure_smem_once(const void* fn, int bytes) {
    struct Entry { const void* fn; uint64_t devices; };
    static Entry table[32];
    static int used = 0;
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    std::lock_guard<std::mutex> lock(mu);
    Entry* e = nullptr;
    for (int i = 0; i < used; ++i)
        if (table[i].fn == fn) e = &table[i];
    if (e != nullptr && dev < 64 && ((e->devices >> dev) & 1u)) return true;
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
    if (e == nullptr && used < 32) { e = &table[used++]; e->fn = fn; e->devices = 0; }
    if (e != nullptr && dev < 64) e->devices |= 1ull << dev;
    return true;
}
template <typename K>
bool ensure_smem(K kernel, int bytes) {
    return ensure_smem_once(reinterpret_cast<const void*>(kernel), bytes);
}

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// ---------------------------------------------------------------------------------------
// validation
// ---------------------------------------------------------------------------------------
// The descriptor grew by one trailing field (drop_scale); a caller built against the shorter
// form passes its own size in struct_bytes and simply has no such field.
constexpr uint32_t kDescBytesV1 = (uint32_t)offsetof(trimul_desc, drop_scale);

inline const void* desc_drop_scale(const trimul_desc* d) {
    return d->struct_bytes >= sizeof(trimul_desc) ? d->drop_scale : nullptr;
}

int check_desc(const trimul_desc* d) {
    if (d == nullptr || (d->struct_bytes != sizeof(trimul_desc) && d->struct_bytes != kDescBytesV1))
        return TRIMUL_E_INVALID;
    if (desc_drop_scale(d) != nullptr && (reinterpret_cast<uintptr_t>(d->drop_scale) & 15u) != 0) return TRIMUL_E_INVALID;
    if (d->B <= 0 || d->N <= 0 || d->c <= 0 || d->rows <= 0 || d->row0 < 0) return TRIMUL_E_INVALID;
    if (d->row0 + d->rows > d->N) return TRIMUL_E_INVALID;
    if (d->dtype != TRIMUL_DTYPE_BF16 && d->dtype != TRIMUL_DTYPE_FP32) return TRIMUL_E_INVALID;
    if (d->direction != TRIMUL_OUTGOING && d->direction != TRIMUL_INCOMING) return TRIMUL_E_INVALID;
    if (d->mask_kind < TRIMUL_MASK_NONE || d->mask_kind > TRIMUL_MASK_PAIR) return TRIMUL_E_INVALID;
    if (!(d->eps_in > 0.f) || !(d->eps_out > 0.f)) return TRIMUL_E_INVALID;
    if (d->c_hidden <= 0) return TRIMUL_E_INVALID;
    if (d->c > kPlainMaxC || d->c_hidden > kPlainMaxC || (d->c % 8) != 0 || (d->c_hidden % 8) != 0)
        return TRIMUL_E_UNSUPPORTED;
    if ((int64_t)d->B * d->c_hidden > 65535) return TRIMUL_E_UNSUPPORTED;
    if (d->N > 16384) return TRIMUL_E_UNSUPPORTED;
    return TRIMUL_OK;
}

int check_weights(const trimul_weights* w) {
    if (w == nullptr) return TRIMUL_E_INVALID;
    if (!w->ln_in_weight || !w->ln_in_bias || !w->w_left || !w->w_left_gate || !w->w_right || !w->w_right_gate ||
        !w->ln_out_weight || !w->ln_out_bias || !w->w_gate || !w->w_out)
        return TRIMUL_E_INVALID;
    const void* ws[6] = {w->w_left, w->w_left_gate, w->w_right, w->w_right_gate, w->w_gate, w->w_out};
    for (const void* p : ws)
        if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return TRIMUL_E_INVALID;
    return TRIMUL_OK;
}

int check_planes(const trimul_planes* pl, int64_t rows, int64_t cols) {
    if (pl == nullptr || pl->base == nullptr) return TRIMUL_E_INVALID;
    if (pl->rows != rows || pl->cols != cols) return TRIMUL_E_INVALID;
    if (pl->pitch < 0 || pl->plane_stride <= 0 || pl->row_chunk <= 0 || pl->col_chunk <= 0) return TRIMUL_E_INVALID;
    if ((pl->pitch % 8) || (pl->plane_stride % 8) || (pl->chunk_stride % 8)) return TRIMUL_E_INVALID;
    if ((reinterpret_cast<uintptr_t>(pl->base) & 15u) != 0) return TRIMUL_E_INVALID;
    const bool rc = pl->row_chunk < rows, cc = pl->col_chunk < cols;
    if (rc && cc) return TRIMUL_E_INVALID;
    if (pl->pitch < (cc ? pl->col_chunk : cols)) return TRIMUL_E_INVALID;
    if ((rc || cc) && pl->chunk_stride <= 0) return TRIMUL_E_INVALID;
    return TRIMUL_OK;
}

PlaneView view_of(const trimul_planes& pl) {
    PlaneView v;
    v.base = pl.base;
    v.rows = pl.rows;
    v.cols = pl.cols;
    v.pitch = pl.pitch;
    v.plane_stride = pl.plane_stride;
    v.chunk_stride = pl.chunk_stride;
    v.row_chunk = pl.row_chunk < pl.rows ? pl.row_chunk : (pl.rows > 0 ? pl.rows : 1);
    v.col_chunk = pl.col_chunk < pl.cols ? pl.col_chunk : (pl.cols > 0 ? pl.cols : 1);
    return v;
}

// chunk sizes as the tensor-core kernels use them: the full extent when not chunked
inline int eff_chunk(int64_t chunk, int64_t extent) { return (int)(chunk < extent ? chunk : extent); }

// bf16 with 128 channels of z; each stage adds its own condition on c_hidden
bool tensor_core_path(const trimul_desc* d) {
    return d->dtype == TRIMUL_DTYPE_BF16 && d->c == 128 && (d->flags & TRIMUL_FLAG_PLAIN_KERNELS) == 0;
}

// bf16 with c = h = 256: the streamed-weight tensor-core kernels of stages 1 and 3
bool wide_tensor_core_path(const trimul_desc* d) {
    return d->dtype == TRIMUL_DTYPE_BF16 && d->c == 256 && d->c_hidden == 256 &&
           (d->flags & TRIMUL_FLAG_PLAIN_KERNELS) == 0;
}

// bf16 with c = h = 64: the stacked-operand tensor-core kernels of stages 1 and 3
bool narrow_tensor_core_path(const trimul_desc* d) {
    return d->dtype == TRIMUL_DTYPE_BF16 && d->c == 64 && d->c_hidden == 64 &&
           (d->flags & TRIMUL_FLAG_PLAIN_KERNELS) == 0;
}

int launch_status() { return cudaGetLastError() == cudaSuccess ? TRIMUL_OK : TRIMUL_E_CUDA; }

// Launch of a tensor-core stage kernel.  `overlap` asks for programmatic dependent launch: the
// kernel may be scheduled while its predecessor in the stream is still draining, runs its set-up
// (barriers, tensor memory, descriptor prefetch) and then blocks in griddepcontrol.wait until the
// predecessor has completed, so launch latency and set-up disappear from the critical path.  Every
// kernel launched this way executes that wait before it touches global memory.
template <typename... KArgs, typename... Args>
int launch_stage(void (*kernel)(KArgs...), int grid, int block, int smem, cudaStream_t st, bool overlap,
                 Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)block, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1u : 0u;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...) == cudaSuccess ? TRIMUL_OK : TRIMUL_E_CUDA;
}
inline bool overlap_launches(uint32_t flags) { return (flags & TRIMUL_FLAG_SERIAL_LAUNCH) == 0; }

// ---------------------------------------------------------------------------------------
// stage 1
// ---------------------------------------------------------------------------------------
template <typename T>
int run_plain_tm1(const trimul_desc* d, const void* z, const uint8_t* mask, const trimul_weights* w,
                  const trimul_planes* a, const trimul_planes* b, cudaStream_t st) {
    PlainTm1Params p;
    p.B = d->B; p.rows = d->rows; p.N = d->N; p.c = d->c; p.row0 = d->row0; p.h = d->c_hidden;
    p.incoming = d->direction == TRIMUL_INCOMING;
    p.mask_kind = mask ? d->mask_kind : 0;
    p.mask = mask;
    p.gamma = w->ln_in_weight; p.beta = w->ln_in_bias; p.eps = d->eps_in;
    p.w_left = w->w_left; p.w_left_gate = w->w_left_gate; p.w_right = w->w_right; p.w_right_gate = w->w_right_gate;
    p.a = view_of(*a); p.b = view_of(*b);
    const int64_t grid = (int64_t)d->B * d->rows * ((d->N + kPlainPos - 1) / kPlainPos);
    plain_tm1_kernel<T><<<(unsigned)grid, kPlainThreads, 0, st>>>(static_cast<const T*>(z), p);
    return launch_status();
}

// Warp-MMA kernels: bf16, c and h multiples of 16, weight matrices 32-byte aligned (fragment loads).
bool wmma_ok(const trimul_desc* d, const void* const* mats, int n) {
    if (d->dtype != TRIMUL_DTYPE_BF16 || (d->flags & TRIMUL_FLAG_PLAIN_KERNELS) != 0) return false;
    if ((d->c % 16) != 0 || (d->c_hidden % 16) != 0) return false;
    for (int i = 0; i < n; ++i)
        if ((reinterpret_cast<uintptr_t>(mats[i]) & 31u) != 0) return false;
    return true;
}

int run_wmma_tm1(const trimul_desc* d, const void* z, const uint8_t* mask, const trimul_weights* w,
                 const trimul_planes* a, const trimul_planes* b, cudaStream_t st) {
    PlainTm1Params p;
    p.B = d->B; p.rows = d->rows; p.N = d->N; p.c = d->c; p.row0 = d->row0; p.h = d->c_hidden;
    p.incoming = d->direction == TRIMUL_INCOMING;
    p.mask_kind = mask ? d->mask_kind : 0;
    p.mask = mask;
    p.gamma = w->ln_in_weight; p.beta = w->ln_in_bias; p.eps = d->eps_in;
    p.w_left = w->w_left; p.w_left_gate = w->w_left_gate; p.w_right = w->w_right; p.w_right_gate = w->w_right_gate;
    p.a = view_of(*a); p.b = view_of(*b);
    const int smem = wmma_tm1_smem(d->c);
    auto kernel = d->c_hidden >= 128 ? wmma_tm1_kernel<4> : wmma_tm1_kernel<2>;
    if (!ensure_smem(kernel, wmma_tm1_smem(kPlainMaxC))) return TRIMUL_E_CUDA;   // opt in once, for the widest case
    const int64_t along = p.incoming ? d->rows : d->N, other = p.incoming ? d->N : d->rows;
    const int64_t grid = (int64_t)d->B * other * ((along + kWmPos - 1) / kWmPos);
    kernel<<<(unsigned)grid, kWmThreads, smem, st>>>(static_cast<const __nv_bfloat16*>(z), p);
    return launch_status();
}

// `n_dest` == 0: a and b are single plane sets.  `n_dest` > 0: a[k] and b[k], k < n_dest, are the
// buffers that receive planes [k * P, (k + 1) * P), P = B * 128 / n_dest (identical geometry).
int run_fast_tm1(const trimul_desc* d, const void* z, const uint8_t* mask, const trimul_weights* w,
                 const trimul_planes* a, const trimul_planes* b, cudaStream_t st, int32_t* status, int n_dest = 0) {
    const bool inc = d->direction == TRIMUL_INCOMING;
    CUtensorMap tmZ, tmW[4];
    {
        const uint64_t dims[4] = {128, (uint64_t)d->N, (uint64_t)d->rows, (uint64_t)d->B};
        const uint64_t strides[3] = {128, (uint64_t)d->N * 128, (uint64_t)d->rows * d->N * 128};
        const uint32_t box_out[4] = {64, 128, 1, 1};
        const uint32_t box_in[4] = {64, 1, 128, 1};
        if (!encode_bf16(&tmZ, z, 4, dims, strides, inc ? box_in : box_out, 128)) return TRIMUL_E_CUDA;
    }
    const void* ws[4] = {w->w_left, w->w_left_gate, w->w_right, w->w_right_gate};
    for (int m = 0; m < 4; ++m) {
        const uint64_t dims[2] = {128, 128};
        const uint64_t strides[1] = {128};
        const uint32_t box[2] = {64, 128};
        if (!encode_bf16(&tmW[m], ws[m], 2, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    }
    const int planes = d->B * 128;
    const int planes_per_dest = n_dest > 0 ? planes / n_dest : planes;

    Tm1Params p;
    p.B = d->B; p.c = 128;
    p.n_fixed = inc ? d->N : d->rows;
    p.n_run = inc ? d->rows : d->N;
    p.tiles_per_fixed = (p.n_run + kT1P - 1) / kT1P;
    const int64_t total = (int64_t)d->B * p.n_fixed * p.tiles_per_fixed;
    if (total > 0x7fffffff) return TRIMUL_E_UNSUPPORTED;
    p.total_tiles = (int)total;
    p.incoming = inc;
    p.N = d->N; p.row0 = d->row0;
    p.mask_kind = mask ? d->mask_kind : 0;
    p.mask = mask;
    p.gamma = w->ln_in_weight; p.beta = w->ln_in_bias; p.eps = d->eps_in;
    p.a_row_chunk = eff_chunk(a->row_chunk, a->rows); p.a_col_chunk = eff_chunk(a->col_chunk, a->cols);
    p.b_row_chunk = eff_chunk(b->row_chunk, b->rows); p.b_col_chunk = eff_chunk(b->col_chunk, b->cols);
    p.planes_per_dest = planes_per_dest;
    p.status = status;
    const int grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
    const bool overlap = overlap_launches(d->flags);
    if ((d->flags & TRIMUL_FLAG_SINGLE_CTA_STAGE1) == 0 && sm_count() >= 2) {
        // CTA pairs: each CTA holds one side's weights and normalises 64 positions of a tile
        CUtensorMap tmZh, tmA, tmB;
        ScatterMaps scA{}, scB{};
        const uint64_t dims[4] = {128, (uint64_t)d->N, (uint64_t)d->rows, (uint64_t)d->B};
        const uint64_t strides[3] = {128, (uint64_t)d->N * 128, (uint64_t)d->rows * d->N * 128};
        const uint32_t box_out[4] = {64, 64, 1, 1};
        const uint32_t box_in[4] = {64, 1, 64, 1};
        if (!encode_bf16(&tmZh, z, 4, dims, strides, inc ? box_in : box_out, 128)) return TRIMUL_E_CUDA;
        const int pairs = p.total_tiles < sm_count() / 2 ? p.total_tiles : sm_count() / 2;
        for (int k = 0; k < 2; ++k) {
            p.step_q[k] = (k + 1) * pairs / p.tiles_per_fixed;
            p.step_r[k] = (k + 1) * pairs % p.tiles_per_fixed;
        }
        if (n_dest > 0) {
            // one epilogue warp stores 64 positions x 32 planes, in segments of one destination's share
            const uint32_t seg = planes_per_dest < 32 ? planes_per_dest : 32;
            for (int k = 0; k < n_dest; ++k) {
                if (!encode_planes(&scA.map[k], a[k], planes_per_dest, 64, 1, seg)) return TRIMUL_E_CUDA;
                if (!encode_planes(&scB.map[k], b[k], planes_per_dest, 64, 1, seg)) return TRIMUL_E_CUDA;
            }
            tmA = scA.map[0];
            tmB = scB.map[0];
            if (!ensure_smem(tm1_pair_sm100_kernel<true>, kP1SmemBytes)) return TRIMUL_E_CUDA;
            return launch_stage(tm1_pair_sm100_kernel<true>, 2 * pairs, kP1Threads, kP1SmemBytes, st, overlap, tmZh,
                                tmW[0], tmW[1], tmW[2], tmW[3], tmA, tmB, p, scA, scB);
        }
        // one epilogue warp stores 64 positions x 32 planes
        if (!encode_planes(&tmA, *a, planes, 64, 1, 32)) return TRIMUL_E_CUDA;
        if (!encode_planes(&tmB, *b, planes, 64, 1, 32)) return TRIMUL_E_CUDA;
        if (!ensure_smem(tm1_pair_sm100_kernel<false>, kP1SmemBytes)) return TRIMUL_E_CUDA;
        return launch_stage(tm1_pair_sm100_kernel<false>, 2 * pairs, kP1Threads, kP1SmemBytes, st, overlap, tmZh,
                            tmW[0], tmW[1], tmW[2], tmW[3], tmA, tmB, p, scA, scB);
    }
    // lone CTAs: all four weight matrices per SM, results staged in shared memory and TMA-stored
    if (n_dest > 0) return TRIMUL_E_UNSUPPORTED;       // only the pair kernel scatters
    CUtensorMap tmA, tmB;
    // stores of a and b: 64 positions x 128 planes per box
    if (!encode_planes(&tmA, *a, planes, 64, 1, 128)) return TRIMUL_E_CUDA;
    if (!encode_planes(&tmB, *b, planes, 64, 1, 128)) return TRIMUL_E_CUDA;
    if (!ensure_smem(tm1_sm100_kernel, kT1SmemBytes)) return TRIMUL_E_CUDA;
    return launch_stage(tm1_sm100_kernel, grid, kT1Threads, kT1SmemBytes, st, overlap, tmZ, tmW[0], tmW[1], tmW[2],
                        tmW[3], tmA, tmB, p);
}

// c = h = 64: left and right weights stacked into one UMMA operand (tm1_narrow_sm100.cuh)
int run_narrow_tm1(const trimul_desc* d, const void* z, const uint8_t* mask, const trimul_weights* w,
                   const trimul_planes* a, const trimul_planes* b, cudaStream_t st, int32_t* status) {
    const bool inc = d->direction == TRIMUL_INCOMING;
    CUtensorMap tmZ, tmW[4], tmA, tmB;
    {
        const uint64_t dims[4] = {kN1C, (uint64_t)d->N, (uint64_t)d->rows, (uint64_t)d->B};
        const uint64_t strides[3] = {kN1C, (uint64_t)d->N * kN1C, (uint64_t)d->rows * d->N * kN1C};
        const uint32_t box_out[4] = {64, 128, 1, 1};
        const uint32_t box_in[4] = {64, 1, 128, 1};
        if (!encode_bf16(&tmZ, z, 4, dims, strides, inc ? box_in : box_out, 128)) return TRIMUL_E_CUDA;
    }
    const void* ws[4] = {w->w_left, w->w_left_gate, w->w_right, w->w_right_gate};
    for (int m = 0; m < 4; ++m) {
        const uint64_t dims[2] = {kN1C, kN1C};
        const uint64_t strides[1] = {kN1C};
        const uint32_t box[2] = {64, 64};
        if (!encode_bf16(&tmW[m], ws[m], 2, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    }
    const int planes = d->B * kN1C;
    if (!encode_planes(&tmA, *a, planes, 64, 1, 64)) return TRIMUL_E_CUDA;
    if (!encode_planes(&tmB, *b, planes, 64, 1, 64)) return TRIMUL_E_CUDA;
    Tm1Params p = {};
    p.B = d->B; p.c = kN1C;
    p.n_fixed = inc ? d->N : d->rows;
    p.n_run = inc ? d->rows : d->N;
    p.tiles_per_fixed = (p.n_run + kT1P - 1) / kT1P;
    const int64_t total = (int64_t)d->B * p.n_fixed * p.tiles_per_fixed;
    if (total > 0x7fffffff) return TRIMUL_E_UNSUPPORTED;
    p.total_tiles = (int)total;
    p.incoming = inc;
    p.N = d->N; p.row0 = d->row0;
    p.mask_kind = mask ? d->mask_kind : 0;
    p.mask = mask;
    p.gamma = w->ln_in_weight; p.beta = w->ln_in_bias; p.eps = d->eps_in;
    p.a_row_chunk = eff_chunk(a->row_chunk, a->rows); p.a_col_chunk = eff_chunk(a->col_chunk, a->cols);
    p.b_row_chunk = eff_chunk(b->row_chunk, b->rows); p.b_col_chunk = eff_chunk(b->col_chunk, b->cols);
    p.planes_per_dest = planes;
    p.status = status;
    const int grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
    if (!ensure_smem(tm1_narrow_sm100_kernel, kN1SmemBytes)) return TRIMUL_E_CUDA;
    return launch_stage(tm1_narrow_sm100_kernel, grid, kN1Threads, kN1SmemBytes, st, overlap_launches(d->flags), tmZ,
                        tmW[0], tmW[1], tmW[2], tmW[3], tmA, tmB, p);
}

// c = h = 256: weights streamed through shared memory (tm1_wide_sm100.cuh)
int run_wide_tm1(const trimul_desc* d, const void* z, const uint8_t* mask, const trimul_weights* w,
                 const trimul_planes* a, const trimul_planes* b, cudaStream_t st, int32_t* status) {
    const bool inc = d->direction == TRIMUL_INCOMING;
    CUtensorMap tmZ, tmW[4], tmA, tmB;
    {
        const uint64_t dims[4] = {kW1C, (uint64_t)d->N, (uint64_t)d->rows, (uint64_t)d->B};
        const uint64_t strides[3] = {kW1C, (uint64_t)d->N * kW1C, (uint64_t)d->rows * d->N * kW1C};
        const uint32_t box_out[4] = {64, 128, 1, 1};
        const uint32_t box_in[4] = {64, 1, 128, 1};
        if (!encode_bf16(&tmZ, z, 4, dims, strides, inc ? box_in : box_out, 128)) return TRIMUL_E_CUDA;
    }
    const void* ws[4] = {w->w_left, w->w_left_gate, w->w_right, w->w_right_gate};
    for (int m = 0; m < 4; ++m) {
        const uint64_t dims[2] = {kW1C, kW1C};
        const uint64_t strides[1] = {kW1C};
        const uint32_t box[2] = {64, 128};
        if (!encode_bf16(&tmW[m], ws[m], 2, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    }
    const int planes = d->B * kW1C;
    if (!encode_planes(&tmA, *a, planes, 64, 1, 128)) return TRIMUL_E_CUDA;
    if (!encode_planes(&tmB, *b, planes, 64, 1, 128)) return TRIMUL_E_CUDA;
    Tm1Params p = {};
    p.B = d->B; p.c = kW1C;
    p.n_fixed = inc ? d->N : d->rows;
    p.n_run = inc ? d->rows : d->N;
    p.tiles_per_fixed = (p.n_run + kT1P - 1) / kT1P;
    const int64_t total = (int64_t)d->B * p.n_fixed * p.tiles_per_fixed;
    if (total > 0x7fffffff) return TRIMUL_E_UNSUPPORTED;
    p.total_tiles = (int)total;
    p.incoming = inc;
    p.N = d->N; p.row0 = d->row0;
    p.mask_kind = mask ? d->mask_kind : 0;
    p.mask = mask;
    p.gamma = w->ln_in_weight; p.beta = w->ln_in_bias; p.eps = d->eps_in;
    p.a_row_chunk = eff_chunk(a->row_chunk, a->rows); p.a_col_chunk = eff_chunk(a->col_chunk, a->cols);
    p.b_row_chunk = eff_chunk(b->row_chunk, b->rows); p.b_col_chunk = eff_chunk(b->col_chunk, b->cols);
    p.planes_per_dest = planes;
    p.status = status;
    const int grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
    if (!ensure_smem(tm1_wide_sm100_kernel, kW1SmemBytes)) return TRIMUL_E_CUDA;
    return launch_stage(tm1_wide_sm100_kernel, grid, kW1Threads, kW1SmemBytes, st, overlap_launches(d->flags), tmZ,
                        tmW[0], tmW[1], tmW[2], tmW[3], tmA, tmB, p);
}

// ---------------------------------------------------------------------------------------
// stage 2
// ---------------------------------------------------------------------------------------
template <typename T>
int run_plain_contract(int planes, const trimul_planes* a, const trimul_planes* b, const trimul_planes* t,
                       cudaStream_t st) {
    dim3 grid((unsigned)((b->rows + 31) / 32), (unsigned)((a->rows + 31) / 32), (unsigned)planes);
    plain_contract_kernel<T><<<grid, 256, 0, st>>>(view_of(*a), view_of(*b), view_of(*t));
    return launch_status();
}

bool fast_contract_ok(const trimul_planes* a, const trimul_planes* b, const trimul_planes* t, bool pair) {
    // a chunk boundary must not cut through a tile (a CTA's half tile for the pair kernel) or a K slice
    if (a->row_chunk < a->rows && (a->row_chunk % kCtBM)) return false;
    if (b->row_chunk < b->rows && (b->row_chunk % (pair ? 128 : kCtBN))) return false;
    // K chunks: whole K slices per chunk, and the last chunk full (the tensor map gives every chunk
    // the extent col_chunk, so a ragged last chunk would read its padding instead of zeros)
    if (a->col_chunk < a->cols && ((a->col_chunk % kCtBK) || (a->cols % a->col_chunk))) return false;
    if (b->col_chunk < b->cols && ((b->col_chunk % kCtBK) || (b->cols % b->col_chunk))) return false;
    if (t->row_chunk < t->rows && (t->row_chunk % kCtBM)) return false;
    if (t->col_chunk < t->cols && (t->col_chunk % 64)) return false;
    if ((reinterpret_cast<uintptr_t>(a->base) | reinterpret_cast<uintptr_t>(b->base) |
         reinterpret_cast<uintptr_t>(t->base)) & 127u)
        return false;
    return true;
}

// `n_dest` == 0: t is one plane set.  `n_dest` > 0 (pair kernel only): t[k], k < n_dest, receives
// output rows [k * R, (k + 1) * R), R = rows_a / n_dest (identical geometry, R a multiple of 128).
int run_fast_contract(int planes, const trimul_planes* a, const trimul_planes* b, const trimul_planes* t,
                      cudaStream_t st, int32_t* status, bool pair, uint32_t flags, int n_dest = 0) {
    CUtensorMap tmA, tmB, tmD;
    ScatterMaps sc{};
    if (!encode_planes(&tmA, *a, planes, kCtBK, kCtBM, 1)) return TRIMUL_E_CUDA;
    if (!encode_planes(&tmB, *b, planes, kCtBK, pair ? 128 : kCtBN, 1)) return TRIMUL_E_CUDA;
    for (int k = 0; k < n_dest; ++k)
        if (!encode_planes(&sc.map[k], t[k], planes, 64, kCtBM, 1)) return TRIMUL_E_CUDA;
    if (n_dest > 0) tmD = sc.map[0];
    else if (!encode_planes(&tmD, *t, planes, 64, kCtBM, 1)) return TRIMUL_E_CUDA;
    ContractParams p;
    p.planes = planes;
    p.rows_a = (int)a->rows; p.rows_b = (int)b->rows; p.K = (int)a->cols;
    p.tiles_m = (p.rows_a + kCtBM - 1) / kCtBM;
    p.tiles_n = (p.rows_b + kCtBN - 1) / kCtBN;
    p.num_kb = (p.K + kCtBK - 1) / kCtBK;
    p.a_row_chunk = eff_chunk(a->row_chunk, a->rows); p.a_k_chunk = eff_chunk(a->col_chunk, a->cols);
    p.b_row_chunk = eff_chunk(b->row_chunk, b->rows); p.b_k_chunk = eff_chunk(b->col_chunk, b->cols);
    p.d_row_chunk = eff_chunk(t->row_chunk, t->rows); p.d_col_chunk = eff_chunk(t->col_chunk, t->cols);
    if (n_dest > 0) { p.d_row_chunk = (int)t->rows; p.d_col_chunk = (int)t->cols; }
    p.status = status;
    if (pair) {
        // CTA pairs: 256 x 256 tiles, one cluster of two CTAs per tile
        const int64_t pair_tiles = (int64_t)planes * ((p.rows_a + 255) / 256) * ((p.rows_b + 255) / 256);
        if (pair_tiles > 0x3fffffff) return TRIMUL_E_UNSUPPORTED;
        const int max_clusters = sm_count() / 2;
        const int clusters = pair_tiles < max_clusters ? (int)pair_tiles : max_clusters;
        const bool overlap = overlap_launches(flags);
        if (n_dest > 0) {
            if (!ensure_smem(contract2_sm100_kernel<true>, kC2SmemBytes)) return TRIMUL_E_CUDA;
            return launch_stage(contract2_sm100_kernel<true>, 2 * clusters, kCtThreads, kC2SmemBytes, st, overlap, tmA,
                                tmB, tmD, p, sc);
        }
        if (!ensure_smem(contract2_sm100_kernel<false>, kC2SmemBytes)) return TRIMUL_E_CUDA;
        return launch_stage(contract2_sm100_kernel<false>, 2 * clusters, kCtThreads, kC2SmemBytes, st, overlap, tmA,
                            tmB, tmD, p, sc);
    }
    if (n_dest > 0) return TRIMUL_E_UNSUPPORTED;
    const int64_t total = (int64_t)planes * p.tiles_m * p.tiles_n;
    if (total > 0x7fffffff) return TRIMUL_E_UNSUPPORTED;
    if (!ensure_smem(contract_sm100_kernel, kCtSmemBytes)) return TRIMUL_E_CUDA;
    const int grid = total < sm_count() ? (int)total : sm_count();
    contract_sm100_kernel<<<grid, kCtThreads, kCtSmemBytes, st>>>(tmA, tmB, tmD, p);
    return launch_status();
}

// ---------------------------------------------------------------------------------------
// stage 3
// ---------------------------------------------------------------------------------------
template <typename T>
int run_plain_tm2(const trimul_desc* d, const void* z, const trimul_planes* tri, const trimul_weights* w, void* out,
                  const void* residual, cudaStream_t st) {
    PlainTm2Params p;
    p.B = d->B; p.rows = d->rows; p.N = d->N; p.c = d->c; p.h = d->c_hidden;
    p.gamma_in = w->ln_in_weight; p.beta_in = w->ln_in_bias;
    p.gamma_out = w->ln_out_weight; p.beta_out = w->ln_out_bias;
    p.eps_in = d->eps_in; p.eps_out = d->eps_out;
    p.w_gate = w->w_gate; p.w_out = w->w_out;
    p.tri = view_of(*tri);
    p.drop_scale = desc_drop_scale(d);
    const int64_t grid = (int64_t)d->B * d->rows * ((d->N + kPlainPos - 1) / kPlainPos);
    plain_tm2_kernel<T><<<(unsigned)grid, kPlainThreads, 0, st>>>(static_cast<const T*>(z), static_cast<T*>(out),
                                                                   static_cast<const T*>(residual), p);
    return launch_status();
}

int run_wmma_tm2(const trimul_desc* d, const void* z, const trimul_planes* tri, const trimul_weights* w, void* out,
                 const void* residual, cudaStream_t st) {
    PlainTm2Params p;
    p.B = d->B; p.rows = d->rows; p.N = d->N; p.c = d->c; p.h = d->c_hidden;
    p.gamma_in = w->ln_in_weight; p.beta_in = w->ln_in_bias;
    p.gamma_out = w->ln_out_weight; p.beta_out = w->ln_out_bias;
    p.eps_in = d->eps_in; p.eps_out = d->eps_out;
    p.w_gate = w->w_gate; p.w_out = w->w_out;
    p.tri = view_of(*tri);
    p.drop_scale = desc_drop_scale(d);
    const int smem = wmma_tm2_smem(d->c, d->c_hidden);
    auto kernel = d->c >= 128 ? wmma_tm2_kernel<4> : wmma_tm2_kernel<2>;
    if (!ensure_smem(kernel, wmma_tm2_smem(kPlainMaxC, kPlainMaxC))) return TRIMUL_E_CUDA;
    const int64_t grid = (int64_t)d->B * d->rows * ((d->N + kWmPos - 1) / kWmPos);
    kernel<<<(unsigned)grid, kWmThreads, smem, st>>>(
        static_cast<const __nv_bfloat16*>(z), static_cast<__nv_bfloat16*>(out),
        static_cast<const __nv_bfloat16*>(residual), p);
    return launch_status();
}

int run_fast_tm2(const trimul_desc* d, const void* z, const trimul_planes* tri, const trimul_weights* w, void* out,
                 const void* residual, cudaStream_t st, int32_t* status) {
    CUtensorMap tmZ, tmWg, tmWo, tmOut, tmRes, tmTri;
    const uint64_t dims[4] = {128, (uint64_t)d->N, (uint64_t)d->rows, (uint64_t)d->B};
    const uint64_t strides[3] = {128, (uint64_t)d->N * 128, (uint64_t)d->rows * d->N * 128};
    const uint32_t box[4] = {64, 128, 1, 1};
    if (!encode_bf16(&tmZ, z, 4, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    if (!encode_bf16(&tmOut, out, 4, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    if (!encode_bf16(&tmRes, residual ? residual : z, 4, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    const int kh = d->c_hidden / 128;          // 1, or 2 for the bidirectional block's last stage
    const uint64_t wdims[2] = {128, 128};
    const uint64_t wstrides[1] = {128};
    const uint64_t wodims[2] = {(uint64_t)d->c_hidden, 128};
    const uint64_t wostrides[1] = {(uint64_t)d->c_hidden};
    const uint32_t wbox[2] = {64, 128};
    if (!encode_bf16(&tmWg, w->w_gate, 2, wdims, wstrides, wbox, 128)) return TRIMUL_E_CUDA;
    if (!encode_bf16(&tmWo, w->w_out, 2, wodims, wostrides, wbox, 128)) return TRIMUL_E_CUDA;
    Tm2Params p;
    p.B = d->B; p.rows = d->rows; p.N = d->N;
    p.tiles_per_row = (d->N + kT2P - 1) / kT2P;
    const int64_t total = (int64_t)d->B * d->rows * p.tiles_per_row;
    if (total > 0x7fffffff) return TRIMUL_E_UNSUPPORTED;
    p.total_tiles = (int)total;
    if (!encode_planes(&tmTri, *tri, d->B * d->c_hidden, 64, 1, 128)) return TRIMUL_E_CUDA;
    p.gamma_in = w->ln_in_weight; p.beta_in = w->ln_in_bias;
    p.gamma_out = w->ln_out_weight; p.beta_out = w->ln_out_bias;
    p.eps_in = d->eps_in; p.eps_out = d->eps_out;
    p.has_residual = residual != nullptr;
    p.status = status;
    const int grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
    if ((d->flags & TRIMUL_FLAG_INPLACE_NORM_STAGE3) == 0 && (residual == nullptr || residual == z)) {
        // default: both LayerNorms folded into the weights, result written in place over the z tile
        // (a residual other than z itself needs a tile buffer this kernel does not have)
        Tm2FoldParams fp;
        fp.base = p;
        fp.residual_is_z = residual != nullptr;
        fp.drop_scale = static_cast<const __nv_bfloat16*>(desc_drop_scale(d));
#define TRIMUL_LAUNCH_TM2_FOLD(RES, KH, DS)                                                                       \
    do {                                                                                                           \
        if (!ensure_smem(tm2_fold_sm100_kernel<RES, KH, DS>, G2Layout<KH>::kSmemBytes)) return TRIMUL_E_CUDA;       \
        return launch_stage(tm2_fold_sm100_kernel<RES, KH, DS>, grid, kG2Threads, G2Layout<KH>::kSmemBytes, st,     \
                            overlap_launches(d->flags), tmZ, tmWg, tmWo, tmOut, tmTri, fp);                        \
    } while (0)
#define TRIMUL_LAUNCH_TM2_FOLD_RK(RES, KH)                  \
    do {                                                    \
        if (fp.drop_scale != nullptr) TRIMUL_LAUNCH_TM2_FOLD(RES, KH, true); \
        else TRIMUL_LAUNCH_TM2_FOLD(RES, KH, false);        \
    } while (0)
        if (kh == 2) {
            if (residual != nullptr) TRIMUL_LAUNCH_TM2_FOLD_RK(true, 2);
            else TRIMUL_LAUNCH_TM2_FOLD_RK(false, 2);
        } else {
            if (residual != nullptr) TRIMUL_LAUNCH_TM2_FOLD_RK(true, 1);
            else TRIMUL_LAUNCH_TM2_FOLD_RK(false, 1);
        }
#undef TRIMUL_LAUNCH_TM2_FOLD_RK
#undef TRIMUL_LAUNCH_TM2_FOLD
    }
    if (kh != 1) return TRIMUL_E_UNSUPPORTED;      // the in-place variant below is 128 hidden channels only
    if (desc_drop_scale(d) != nullptr) return TRIMUL_E_UNSUPPORTED;   // ... and has no drop-scale operand
    if (!ensure_smem(tm2_sm100_kernel, kT2SmemBytes)) return TRIMUL_E_CUDA;
    tm2_sm100_kernel<<<grid, kT2Threads, kT2SmemBytes, st>>>(tmZ, tmWg, tmWo, tmOut, tmRes, tmTri, p);
    return launch_status();
}

// c = h = 64 (tm2_narrow_sm100.cuh)
int run_narrow_tm2(const trimul_desc* d, const void* z, const trimul_planes* tri, const trimul_weights* w, void* out,
                   const void* residual, cudaStream_t st, int32_t* status) {
    CUtensorMap tmZ, tmWg, tmWo, tmOut, tmTri;
    const uint64_t dims[4] = {kN2C, (uint64_t)d->N, (uint64_t)d->rows, (uint64_t)d->B};
    const uint64_t strides[3] = {kN2C, (uint64_t)d->N * kN2C, (uint64_t)d->rows * d->N * kN2C};
    const uint32_t box[4] = {64, 128, 1, 1};
    if (!encode_bf16(&tmZ, z, 4, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    if (!encode_bf16(&tmOut, out, 4, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    const uint64_t wdims[2] = {kN2C, kN2C};
    const uint64_t wstrides[1] = {kN2C};
    const uint32_t wbox[2] = {64, 64};
    if (!encode_bf16(&tmWg, w->w_gate, 2, wdims, wstrides, wbox, 128)) return TRIMUL_E_CUDA;
    if (!encode_bf16(&tmWo, w->w_out, 2, wdims, wstrides, wbox, 128)) return TRIMUL_E_CUDA;
    if (!encode_planes(&tmTri, *tri, d->B * kN2C, 64, 1, 64)) return TRIMUL_E_CUDA;
    CUtensorMap tmRes;
    if (!encode_bf16(&tmRes, residual ? residual : z, 4, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    Tm2NarrowParams np = {};
    Tm2Params& p = np.base;
    p.B = d->B; p.rows = d->rows; p.N = d->N;
    p.tiles_per_row = (d->N + kT2P - 1) / kT2P;
    const int64_t total = (int64_t)d->B * d->rows * p.tiles_per_row;
    if (total > 0x7fffffff) return TRIMUL_E_UNSUPPORTED;
    p.total_tiles = (int)total;
    p.gamma_in = w->ln_in_weight; p.beta_in = w->ln_in_bias;
    p.gamma_out = w->ln_out_weight; p.beta_out = w->ln_out_bias;
    p.eps_in = d->eps_in; p.eps_out = d->eps_out;
    p.has_residual = residual != nullptr;
    p.status = status;
    np.residual = static_cast<const __nv_bfloat16*>(residual);
    np.drop_scale = static_cast<const __nv_bfloat16*>(desc_drop_scale(d));
    const int grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
    if (!ensure_smem(tm2_narrow_sm100_kernel, kN2SmemBytes)) return TRIMUL_E_CUDA;
    return launch_stage(tm2_narrow_sm100_kernel, grid, kN2Threads, kN2SmemBytes, st, overlap_launches(d->flags), tmZ,
                        tmWg, tmWo, tmOut, tmTri, tmRes, np);
}

// c = h = 256: weights streamed through shared memory (tm2_wide_sm100.cuh)
int run_wide_tm2(const trimul_desc* d, const void* z, const trimul_planes* tri, const trimul_weights* w, void* out,
                 const void* residual, cudaStream_t st, int32_t* status) {
    CUtensorMap tmZ, tmWg, tmWo, tmOut, tmTri;
    const uint64_t dims[4] = {kW2C, (uint64_t)d->N, (uint64_t)d->rows, (uint64_t)d->B};
    const uint64_t strides[3] = {kW2C, (uint64_t)d->N * kW2C, (uint64_t)d->rows * d->N * kW2C};
    const uint32_t box[4] = {64, 128, 1, 1};
    if (!encode_bf16(&tmZ, z, 4, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    if (!encode_bf16(&tmOut, out, 4, dims, strides, box, 128)) return TRIMUL_E_CUDA;
    const uint64_t wdims[2] = {kW2C, kW2C};
    const uint64_t wstrides[1] = {kW2C};
    const uint32_t wbox[2] = {64, 128};
    if (!encode_bf16(&tmWg, w->w_gate, 2, wdims, wstrides, wbox, 128)) return TRIMUL_E_CUDA;
    if (!encode_bf16(&tmWo, w->w_out, 2, wdims, wstrides, wbox, 128)) return TRIMUL_E_CUDA;
    if (!encode_planes(&tmTri, *tri, d->B * kW2C, 64, 1, 128)) return TRIMUL_E_CUDA;
    Tm2WideParams wp = {};
    Tm2Params& p = wp.base;
    p.B = d->B; p.rows = d->rows; p.N = d->N;
    p.tiles_per_row = (d->N + kT2P - 1) / kT2P;
    const int64_t total = (int64_t)d->B * d->rows * p.tiles_per_row;
    if (total > 0x7fffffff) return TRIMUL_E_UNSUPPORTED;
    p.total_tiles = (int)total;
    p.gamma_in = w->ln_in_weight; p.beta_in = w->ln_in_bias;
    p.gamma_out = w->ln_out_weight; p.beta_out = w->ln_out_bias;
    p.eps_in = d->eps_in; p.eps_out = d->eps_out;
    p.has_residual = residual != nullptr;
    p.status = status;
    wp.residual = static_cast<const __nv_bfloat16*>(residual);
    wp.drop_scale = static_cast<const __nv_bfloat16*>(desc_drop_scale(d));
    const int grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
    if (!ensure_smem(tm2_wide_sm100_kernel, kW2SmemBytes)) return TRIMUL_E_CUDA;
    return launch_stage(tm2_wide_sm100_kernel, grid, kW2Threads, kW2SmemBytes, st, overlap_launches(d->flags), tmZ, tmWg,
                        tmWo, tmOut, tmTri, wp);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// =========================================================================================
// exported entry points
// =========================================================================================
extern "C" {

#ifdef TRIMUL_TRACE
// debug builds only: copy the timeline stamps of the last kernel that wrote them to the host
int trimul_b200_debug_trace(void* host, size_t n) { return (int)cudaMemcpyFromSymbol(host, trimul::g_trace, n); }
#endif

int trimul_b200_abi_version(void) { return TRIMUL_B200_ABI_VERSION; }

const char* trimul_b200_strerror(int code) {
    switch (code) {
        case TRIMUL_OK: return "success";
        case TRIMUL_E_INVALID: return "invalid argument (null pointer, bad size or enum, misaligned buffer)";
        case TRIMUL_E_UNSUPPORTED: return "unsupported configuration";
        case TRIMUL_E_WORKSPACE: return "workspace too small";
        case TRIMUL_E_CUDA: return "CUDA call failed (kernel launch or tensor-map encode)";
        case TRIMUL_E_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
        case TRIMUL_E_STATIC_SCRATCH:
            return "problem needs more scratch than the library's built-in array holds "
                   "(TRIMUL_B200_STATIC_SCRATCH_BYTES); use trimul_b200_forward with your own workspace";
        default: return "unknown error code";
    }
}

int trimul_b200_workspace_bytes(const trimul_desc* desc, size_t* bytes, trimul_planes* a, trimul_planes* b,
                                trimul_planes* tri) {
    int rc = check_desc(desc);
    if (rc != TRIMUL_OK) return rc;
    if (bytes == nullptr) return TRIMUL_E_INVALID;
    const int64_t esz = desc->dtype == TRIMUL_DTYPE_BF16 ? 2 : 4;
    const int64_t planes = (int64_t)desc->B * desc->c_hidden;
    const bool inc = desc->direction == TRIMUL_INCOMING;
    // a, b: outgoing [planes][rows][N], incoming [planes][N][rows];  tri: [planes][rows][N]
    const int64_t ab_rows = inc ? desc->N : desc->rows, ab_cols = inc ? desc->rows : desc->N;
    const int64_t ab_pitch = round_up(ab_cols, 8), t_pitch = round_up(desc->N, 8);
    const int64_t ab_plane = ab_rows * ab_pitch, t_plane = (int64_t)desc->rows * t_pitch;
    const int64_t ab_bytes = round_up(planes * ab_plane * esz, 1024), t_bytes = round_up(planes * t_plane * esz, 1024);
    trimul_planes pa = {nullptr, ab_rows, ab_cols, ab_pitch, ab_plane, 0, ab_rows, ab_cols};
    trimul_planes pb = pa;
    pb.base = reinterpret_cast<void*>((uintptr_t)ab_bytes);
    trimul_planes pt = {reinterpret_cast<void*>((uintptr_t)(2 * ab_bytes)), desc->rows, desc->N, t_pitch, t_plane, 0,
                        desc->rows, desc->N};
    if (a) *a = pa;
    if (b) *b = pb;
    if (tri) *tri = pt;
    *bytes = (size_t)(2 * ab_bytes + t_bytes);
    return TRIMUL_OK;
}

int trimul_b200_tm1(const trimul_desc* desc, const void* z, const uint8_t* mask, const trimul_weights* w,
                    const trimul_planes* a, const trimul_planes* b, void* stream, int32_t* status) {
    int rc = check_desc(desc);
    if (rc != TRIMUL_OK) return rc;
    if ((rc = check_weights(w)) != TRIMUL_OK) return rc;
    if (z == nullptr || !aligned16(z)) return TRIMUL_E_INVALID;
    if (desc->mask_kind != TRIMUL_MASK_NONE && mask == nullptr) return TRIMUL_E_INVALID;
    const bool inc = desc->direction == TRIMUL_INCOMING;
    const int64_t prow = inc ? desc->N : desc->rows, pcol = inc ? desc->rows : desc->N;
    if ((rc = check_planes(a, prow, pcol)) != TRIMUL_OK) return rc;
    if ((rc = check_planes(b, prow, pcol)) != TRIMUL_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (desc->dtype == TRIMUL_DTYPE_FP32) return run_plain_tm1<float>(desc, z, mask, w, a, b, st);
    const bool chunks_ok = (a->col_chunk >= a->cols || a->col_chunk % 64 == 0) &&
                           (b->col_chunk >= b->cols || b->col_chunk % 64 == 0) &&
                           ((reinterpret_cast<uintptr_t>(a->base) | reinterpret_cast<uintptr_t>(b->base)) & 127u) == 0;
    if (tensor_core_path(desc) && desc->c_hidden == 128 && chunks_ok)
        return run_fast_tm1(desc, z, mask, w, a, b, st, status);
    if (wide_tensor_core_path(desc) && chunks_ok) return run_wide_tm1(desc, z, mask, w, a, b, st, status);
    if (narrow_tensor_core_path(desc) && chunks_ok) return run_narrow_tm1(desc, z, mask, w, a, b, st, status);
    const void* mats[4] = {w->w_left, w->w_left_gate, w->w_right, w->w_right_gate};
    if (wmma_ok(desc, mats, 4)) return run_wmma_tm1(desc, z, mask, w, a, b, st);
    return run_plain_tm1<__nv_bfloat16>(desc, z, mask, w, a, b, st);
}

int trimul_b200_contract(int32_t dtype, uint32_t flags, int32_t planes, const trimul_planes* a,
                         const trimul_planes* b, const trimul_planes* tri, void* stream, int32_t* status) {
    if (a == nullptr || b == nullptr || tri == nullptr) return TRIMUL_E_INVALID;
    if (planes <= 0 || planes > 65535) return TRIMUL_E_INVALID;
    if (dtype != TRIMUL_DTYPE_BF16 && dtype != TRIMUL_DTYPE_FP32) return TRIMUL_E_INVALID;
    int rc;
    if ((rc = check_planes(a, a->rows, a->cols)) != TRIMUL_OK) return rc;
    if ((rc = check_planes(b, b->rows, a->cols)) != TRIMUL_OK) return rc;
    if ((rc = check_planes(tri, a->rows, b->rows)) != TRIMUL_OK) return rc;
    if (a->rows <= 0 || b->rows <= 0 || a->cols <= 0) return TRIMUL_E_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == TRIMUL_DTYPE_FP32) return run_plain_contract<float>(planes, a, b, tri, st);
    if ((flags & TRIMUL_FLAG_PLAIN_KERNELS) == 0) {
        const bool pair = (flags & TRIMUL_FLAG_SINGLE_CTA_CONTRACT) == 0 && sm_count() >= 2;
        if (fast_contract_ok(a, b, tri, pair)) return run_fast_contract(planes, a, b, tri, st, status, pair, flags);
        if (pair && fast_contract_ok(a, b, tri, false))
            return run_fast_contract(planes, a, b, tri, st, status, false, flags);
    }
    return run_plain_contract<__nv_bfloat16>(planes, a, b, tri, st);
}

namespace {
// all destination buffers of a scattering call must share one geometry (only the base differs)
bool same_geometry(const trimul_planes* v, int n) {
    for (int k = 1; k < n; ++k)
        if (v[k].rows != v[0].rows || v[k].cols != v[0].cols || v[k].pitch != v[0].pitch ||
            v[k].plane_stride != v[0].plane_stride || v[k].chunk_stride != v[0].chunk_stride ||
            v[k].row_chunk != v[0].row_chunk || v[k].col_chunk != v[0].col_chunk)
            return false;
    return true;
}
}  // namespace

int trimul_b200_tm1_scatter(const trimul_desc* desc, const void* z, const uint8_t* mask, const trimul_weights* w,
                            int32_t n_dest, const trimul_planes* a_dest, const trimul_planes* b_dest, void* stream,
                            int32_t* status) {
    int rc = check_desc(desc);
    if (rc != TRIMUL_OK) return rc;
    if ((rc = check_weights(w)) != TRIMUL_OK) return rc;
    if (z == nullptr || !aligned16(z) || a_dest == nullptr || b_dest == nullptr) return TRIMUL_E_INVALID;
    if (desc->mask_kind != TRIMUL_MASK_NONE && mask == nullptr) return TRIMUL_E_INVALID;
    if (n_dest < 1 || n_dest > kMaxDest) return TRIMUL_E_INVALID;
    const int64_t planes = (int64_t)desc->B * desc->c;
    if (planes % n_dest != 0) return TRIMUL_E_INVALID;
    const int64_t per = planes / n_dest;
    const bool inc = desc->direction == TRIMUL_INCOMING;
    const int64_t prow = inc ? desc->N : desc->rows, pcol = inc ? desc->rows : desc->N;
    for (int k = 0; k < n_dest; ++k) {
        if ((rc = check_planes(&a_dest[k], prow, pcol)) != TRIMUL_OK) return rc;
        if ((rc = check_planes(&b_dest[k], prow, pcol)) != TRIMUL_OK) return rc;
        if (((reinterpret_cast<uintptr_t>(a_dest[k].base) | reinterpret_cast<uintptr_t>(b_dest[k].base)) & 127u) != 0)
            return TRIMUL_E_INVALID;
    }
    if (!same_geometry(a_dest, n_dest) || !same_geometry(b_dest, n_dest)) return TRIMUL_E_INVALID;
    // tensor-core kernel only: a destination's share must be whole 16-plane groups of a 128-plane tile
    if (!tensor_core_path(desc) || desc->c_hidden != 128) return TRIMUL_E_UNSUPPORTED;
    if (per % 16 != 0 || !(128 % per == 0 || per % 128 == 0)) return TRIMUL_E_UNSUPPORTED;
    if ((a_dest->col_chunk < a_dest->cols && a_dest->col_chunk % 64) ||
        (b_dest->col_chunk < b_dest->cols && b_dest->col_chunk % 64))
        return TRIMUL_E_UNSUPPORTED;
    return run_fast_tm1(desc, z, mask, w, a_dest, b_dest, static_cast<cudaStream_t>(stream), status, n_dest);
}

int trimul_b200_contract_scatter(int32_t dtype, uint32_t flags, int32_t planes, const trimul_planes* a,
                                 const trimul_planes* b, int32_t n_dest, const trimul_planes* tri_dest, void* stream,
                                 int32_t* status) {
    if (a == nullptr || b == nullptr || tri_dest == nullptr) return TRIMUL_E_INVALID;
    if (planes <= 0 || planes > 65535) return TRIMUL_E_INVALID;
    if (dtype != TRIMUL_DTYPE_BF16 && dtype != TRIMUL_DTYPE_FP32) return TRIMUL_E_INVALID;
    if (n_dest < 1 || n_dest > kMaxDest) return TRIMUL_E_INVALID;
    int rc;
    if ((rc = check_planes(a, a->rows, a->cols)) != TRIMUL_OK) return rc;
    if ((rc = check_planes(b, b->rows, a->cols)) != TRIMUL_OK) return rc;
    if (a->rows <= 0 || b->rows <= 0 || a->cols <= 0 || a->rows % n_dest != 0) return TRIMUL_E_INVALID;
    const int64_t R = a->rows / n_dest;
    for (int k = 0; k < n_dest; ++k) {
        if ((rc = check_planes(&tri_dest[k], R, b->rows)) != TRIMUL_OK) return rc;
        if ((reinterpret_cast<uintptr_t>(tri_dest[k].base) & 127u) != 0) return TRIMUL_E_INVALID;
        if (tri_dest[k].row_chunk < R || tri_dest[k].col_chunk < b->rows) return TRIMUL_E_UNSUPPORTED;
    }
    if (!same_geometry(tri_dest, n_dest)) return TRIMUL_E_INVALID;
    // CTA-pair tensor-core kernel only; each CTA's 128 output rows must lie in one destination
    if (dtype != TRIMUL_DTYPE_BF16 || sm_count() < 2 || R % 128 != 0) return TRIMUL_E_UNSUPPORTED;
    trimul_planes shape = tri_dest[0];        // operand checks of the tile geometry use the full extent
    shape.rows = a->rows; shape.row_chunk = a->rows;
    if (!fast_contract_ok(a, b, &shape, true)) return TRIMUL_E_UNSUPPORTED;
    return run_fast_contract(planes, a, b, tri_dest, static_cast<cudaStream_t>(stream), status, true, flags, n_dest);
}

int trimul_b200_tm2(const trimul_desc* desc, const void* z, const trimul_planes* tri, const trimul_weights* w,
                    void* out, const void* residual, void* stream, int32_t* status) {
    int rc = check_desc(desc);
    if (rc != TRIMUL_OK) return rc;
    if ((rc = check_weights(w)) != TRIMUL_OK) return rc;
    if (z == nullptr || out == nullptr || out == z || !aligned16(z) || !aligned16(out)) return TRIMUL_E_INVALID;
    if (residual != nullptr && (!aligned16(residual) || residual == out)) return TRIMUL_E_INVALID;
    if ((rc = check_planes(tri, desc->rows, desc->N)) != TRIMUL_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (desc->dtype == TRIMUL_DTYPE_FP32) return run_plain_tm2<float>(desc, z, tri, w, out, residual, st);
    const bool plain_layout = tri->row_chunk >= tri->rows && tri->col_chunk >= tri->cols &&
                              (reinterpret_cast<uintptr_t>(tri->base) & 127u) == 0;
    if (tensor_core_path(desc) && plain_layout && (desc->c_hidden == 128 || desc->c_hidden == 256)) {
        // the wide (2c) form exists only in the folded kernel, which takes no residual but z itself
        const bool wide = desc->c_hidden != desc->c;
        const bool folded_ok = (desc->flags & TRIMUL_FLAG_INPLACE_NORM_STAGE3) == 0 && (residual == nullptr || residual == z);
        if (!wide || folded_ok) return run_fast_tm2(desc, z, tri, w, out, residual, st, status);
    }
    if (wide_tensor_core_path(desc) && plain_layout) return run_wide_tm2(desc, z, tri, w, out, residual, st, status);
    if (narrow_tensor_core_path(desc) && plain_layout) return run_narrow_tm2(desc, z, tri, w, out, residual, st, status);
    const void* mats[2] = {w->w_gate, w->w_out};
    if (wmma_ok(desc, mats, 2)) return run_wmma_tm2(desc, z, tri, w, out, residual, st);
    return run_plain_tm2<__nv_bfloat16>(desc, z, tri, w, out, residual, st);
}

int trimul_b200_forward(const trimul_desc* desc, const void* z, const uint8_t* mask, const trimul_weights* w,
                        void* out, const void* residual, void* workspace, size_t workspace_bytes, void* stream,
                        int32_t* status) {
    int rc = check_desc(desc);
    if (rc != TRIMUL_OK) return rc;
    if (desc->rows != desc->N || desc->row0 != 0) return TRIMUL_E_INVALID;
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return TRIMUL_E_INVALID;
    size_t need = 0;
    trimul_planes a, b, t;
    if ((rc = trimul_b200_workspace_bytes(desc, &need, &a, &b, &t)) != TRIMUL_OK) return rc;
    if (workspace_bytes < need) return TRIMUL_E_WORKSPACE;
    const uintptr_t base = reinterpret_cast<uintptr_t>(workspace);
    a.base = reinterpret_cast<void*>(base + reinterpret_cast<uintptr_t>(a.base));
    b.base = reinterpret_cast<void*>(base + reinterpret_cast<uintptr_t>(b.base));
    t.base = reinterpret_cast<void*>(base + reinterpret_cast<uintptr_t>(t.base));
    // validate everything before the first launch, so an error leaves nothing enqueued
    if ((rc = check_weights(w)) != TRIMUL_OK) return rc;
    if (z == nullptr || out == nullptr || out == z || !aligned16(z) || !aligned16(out)) return TRIMUL_E_INVALID;
    if (residual != nullptr && (!aligned16(residual) || residual == out)) return TRIMUL_E_INVALID;
    if (desc->mask_kind != TRIMUL_MASK_NONE && mask == nullptr) return TRIMUL_E_INVALID;
    // the one combination the tensor-core last stage has no kernel for (see trimul_desc.drop_scale)
    if (desc_drop_scale(desc) != nullptr && residual != nullptr && residual != z && tensor_core_path(desc) &&
        desc->c_hidden == 128)
        return TRIMUL_E_UNSUPPORTED;
    if ((rc = trimul_b200_tm1(desc, z, mask, w, &a, &b, stream, status)) != TRIMUL_OK) return rc;
    if ((rc = trimul_b200_contract(desc->dtype, desc->flags, desc->B * desc->c_hidden, &a, &b, &t, stream, status)) !=
        TRIMUL_OK)
        return rc;
    return trimul_b200_tm2(desc, z, &t, w, out, residual, stream, status);
}

int trimul_b200_bidir_workspace_bytes(const trimul_desc* desc, size_t* bytes) {
    int rc = check_desc(desc);
    if (rc != TRIMUL_OK) return rc;
    if (bytes == nullptr || desc->c_hidden % 16 != 0) return TRIMUL_E_INVALID;   // 2h, h a multiple of 8
    if (desc->rows != desc->N || desc->row0 != 0) return TRIMUL_E_INVALID;
    const int64_t esz = desc->dtype == TRIMUL_DTYPE_BF16 ? 2 : 4;
    const int64_t set_bytes = round_up((int64_t)desc->B * desc->c_hidden * desc->N * round_up(desc->N, 8) * esz, 1024);
    *bytes = (size_t)(3 * set_bytes);
    return TRIMUL_OK;
}

int trimul_b200_forward_bidir(const trimul_desc* desc, const void* z, const uint8_t* mask, const trimul_weights* w,
                              void* out, int32_t add_residual, void* workspace, size_t workspace_bytes, void* stream,
                              int32_t* status) {
    size_t need = 0;
    int rc = trimul_b200_bidir_workspace_bytes(desc, &need);
    if (rc != TRIMUL_OK) return rc;
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return TRIMUL_E_INVALID;
    if (workspace_bytes < need) return TRIMUL_E_WORKSPACE;
    if ((rc = check_weights(w)) != TRIMUL_OK) return rc;
    if (z == nullptr || out == nullptr || out == z || !aligned16(z) || !aligned16(out)) return TRIMUL_E_INVALID;
    if (desc->mask_kind != TRIMUL_MASK_NONE && mask == nullptr) return TRIMUL_E_INVALID;
    const int64_t esz = desc->dtype == TRIMUL_DTYPE_BF16 ? 2 : 4;
    const int64_t N = desc->N, c = desc->c, h = desc->c_hidden / 2, pitch = round_up(N, 8), plane = N * pitch;
    const int64_t set_bytes = (int64_t)(need / 3);
    uint8_t* base = static_cast<uint8_t*>(workspace);
    // stage 1: per batch element and direction, with that direction's rows of the [2h, c] weights
    trimul_desc d1 = {};
    memcpy(&d1, desc, desc->struct_bytes < sizeof(trimul_desc) ? desc->struct_bytes : sizeof(trimul_desc));
    d1.B = 1;
    d1.c_hidden = (int32_t)h;
    for (int bi = 0; bi < desc->B; ++bi) {
        const uint8_t* zb = static_cast<const uint8_t*>(z) + (int64_t)bi * N * N * c * esz;
        const uint8_t* mb = mask == nullptr ? nullptr
                          : mask + (int64_t)bi * (desc->mask_kind == TRIMUL_MASK_PAIR ? N * N : N);
        for (int dir = 0; dir < 2; ++dir) {
            d1.direction = dir == 0 ? TRIMUL_OUTGOING : TRIMUL_INCOMING;
            trimul_weights w1 = *w;
            const int64_t wofs = (int64_t)dir * h * c * esz;
            w1.w_left = static_cast<const uint8_t*>(w->w_left) + wofs;
            w1.w_left_gate = static_cast<const uint8_t*>(w->w_left_gate) + wofs;
            w1.w_right = static_cast<const uint8_t*>(w->w_right) + wofs;
            w1.w_right_gate = static_cast<const uint8_t*>(w->w_right_gate) + wofs;
            const int64_t first = ((int64_t)bi * 2 * h + (int64_t)dir * h) * plane * esz;
            trimul_planes pa = {base + first, N, N, pitch, plane, 0, N, N};
            trimul_planes pb = pa;
            pb.base = base + set_bytes + first;
            if ((rc = trimul_b200_tm1(&d1, zb, mb, &w1, &pa, &pb, stream, status)) != TRIMUL_OK) return rc;
        }
    }
    // stage 2: one contraction over all B * 2h planes; stage 3: LayerNorm_out over 2h channels
    trimul_planes a = {base, N, N, pitch, plane, 0, N, N};
    trimul_planes b = a, t = a;
    b.base = base + set_bytes;
    t.base = base + 2 * set_bytes;
    if ((rc = trimul_b200_contract(desc->dtype, desc->flags, desc->B * desc->c_hidden, &a, &b, &t, stream, status)) !=
        TRIMUL_OK)
        return rc;
    return trimul_b200_tm2(desc, z, &t, w, out, add_residual ? z : nullptr, stream, status);
}

int trimul_b200_peer_barrier(int32_t rank, int32_t world, int32_t* const* peer_flags, uint32_t epoch,
                             uint32_t timeout_us, void* stream, int32_t* status) {
    if (world < 1 || world > kMaxDest || rank < 0 || rank >= world || peer_flags == nullptr || epoch == 0 ||
        timeout_us == 0)
        return TRIMUL_E_INVALID;
    PeerFlags pf{};
    for (int r = 0; r < world; ++r) {
        if (peer_flags[r] == nullptr || (reinterpret_cast<uintptr_t>(peer_flags[r]) & 3u) != 0) return TRIMUL_E_INVALID;
        pf.flags[r] = peer_flags[r];
    }
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pf, rank, world, epoch,
                                                                        (uint64_t)timeout_us * 1000ull, status);
    return launch_status();
}

int trimul_b200_selftest_expiring_wait(uint32_t timeout_us, void* stream, int32_t* status) {
    if (timeout_us == 0 || status == nullptr) return TRIMUL_E_INVALID;
    expire_wait_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>((uint64_t)timeout_us * 1000ull, status);
    return launch_status();
}

// ---------------------------------------------------------------------------------------
// built-in scratch: device address of g_static_scratch, looked up once per device
// ---------------------------------------------------------------------------------------
namespace {

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the static scratch array on the CURRENT device.  The first call per device
// asks the runtime for it (which also loads the device image there); later calls hit the cache.
int static_scratch_address(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TRIMUL_E_CUDA;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return TRIMUL_E_CUDA;
        }
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return TRIMUL_OK;
}

}  // namespace

int trimul_b200_forward_static(const trimul_desc* desc, const void* z, const uint8_t* mask, const trimul_weights* w,
                               void* out, const void* residual, void* stream, int32_t* status) {
    size_t need = 0;
    int rc = trimul_b200_workspace_bytes(desc, &need, nullptr, nullptr, nullptr);
    if (rc != TRIMUL_OK) return rc;
    if (need > (size_t)TRIMUL_B200_STATIC_SCRATCH_BYTES) return TRIMUL_E_STATIC_SCRATCH;
    void* scratch = nullptr;
    if ((rc = static_scratch_address(&scratch)) != TRIMUL_OK) return rc;
    return trimul_b200_forward(desc, z, mask, w, out, residual, scratch, (size_t)TRIMUL_B200_STATIC_SCRATCH_BYTES,
                               stream, status);
}

}  // extern "C"
