/*
 * trimul_b200 — C ABI of the B200 (sm_100a) TriangleMultiplication block.
 *
 * One block call computes, for a pair tensor z[B,N,N,c]:
 *
 *   x_n   = LayerNorm_in(z)                                   (over c, fp32 statistics)
 *   a     = sigmoid(x_n Wlg^T) * (x_n Wl^T) * pairmask        (left operand)
 *   b     = sigmoid(x_n Wrg^T) * (x_n Wr^T) * pairmask        (right operand)
 *   tri   = outgoing: sum_k a[i,k,:] * b[j,k,:]    incoming: sum_k a[k,i,:] * b[k,j,:]
 *   out   = sigmoid(x_n Wg^T) * (LayerNorm_out(tri) Wo^T)     (+ residual when asked)
 *
 * which is the arithmetic of the reference's ground truth,
 * src/miniworld_engine/modules/triangle_multiplication/reference.py:62-83 (module form) and
 * :86-122 (functional form, pair mask).  All Linear weights are [out,in] row-major
 * (nn.Linear), bias-free; LayerNorm parameters are fp32 whatever the activation type
 * (src/miniworld_engine/modules/primitives.py:70-88).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller; nothing here allocates,
 *     frees, synchronises or throws;  work is enqueued on `stream` (a cudaStream_t);
 *   - return value: 0 on success, a negative TRIMUL_E_* code otherwise (see
 *     trimul_b200_strerror);  errors are detected before anything is enqueued;
 *   - `status` (optional, may be NULL) points to 4 caller-owned int32 words on the device,
 *     zeroed by the caller.  A kernel whose bounded wait expires writes
 *     {TRIMUL_E_DEVICE_TIMEOUT, stage id, block index, detail} there and returns
 *     early instead of hanging; the caller reads it after synchronising the stream;
 *   - entry points are re-entrant across streams as long as workspaces are distinct.
 *
 * The functions replace, behind the reference's own module / functional interface, the
 * launch sequence of its sm_100 fast path
 * (src/miniworld_engine/modules/triangle_multiplication/module.py:399-459).
 */
#ifndef TRIMUL_B200_H_
#define TRIMUL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRIMUL_B200_ABI_VERSION 2

/* error codes */
#define TRIMUL_OK                 0
#define TRIMUL_E_INVALID         -1   /* NULL pointer, bad size, bad enum, misaligned buffer        */
#define TRIMUL_E_UNSUPPORTED     -2   /* valid request that this build has no kernel for            */
#define TRIMUL_E_WORKSPACE       -3   /* workspace smaller than trimul_b200_workspace_bytes says    */
#define TRIMUL_E_CUDA            -4   /* a CUDA runtime/driver call failed (launch, tensor map)     */
#define TRIMUL_E_DEVICE_TIMEOUT  -5   /* only ever written to the device status words               */
#define TRIMUL_E_STATIC_SCRATCH  -6   /* problem too large for the library's built-in scratch array */

/* dtype of activations and Linear weights */
#define TRIMUL_DTYPE_BF16 0           /* bf16 storage, fp32 accumulate, tensor-core kernels         */
#define TRIMUL_DTYPE_FP32 1           /* fp32 storage and arithmetic (no TF32), CUDA-core kernels   */

/* direction: reference.py:77-80 */
#define TRIMUL_OUTGOING 0
#define TRIMUL_INCOMING 1

/* mask kind */
#define TRIMUL_MASK_NONE  0
#define TRIMUL_MASK_TOKEN 1           /* uint8 [B,N];   pair mask = m[i] & m[k]  (reference.py:72-75)  */
#define TRIMUL_MASK_PAIR  2           /* uint8 [B,N,N]; functional form          (reference.py:108-111) */

/* flags */
#define TRIMUL_FLAG_PLAIN_KERNELS 1u  /* run the CUDA-core kernels even where tensor-core ones exist
                                         (cross-checking aid; same layouts, same rounding points)   */
#define TRIMUL_FLAG_SINGLE_CTA_CONTRACT 2u /* contraction on lone CTAs (128x256 tiles) instead of CTA
                                         pairs (256x256 tiles, cta_group::2); cross-checking aid    */
#define TRIMUL_FLAG_SINGLE_CTA_STAGE1 4u /* stage 1 (c = 128) on lone CTAs (all four weight matrices and a
                                         two-deep tile ring per SM) instead of CTA pairs (cta_group::2:
                                         each CTA holds one side's weights and normalises half of a
                                         tile); same arithmetic, results equal to the last bf16 bit of
                                         a few elements; slower                                      */
#define TRIMUL_FLAG_INPLACE_NORM_STAGE3 16u /* stage 3 with both LayerNorms applied in place in shared
                                         memory before the projections (rounds LN(x) to bf16 like the
                                         reference) instead of the default kernel, which folds them
                                         into the weights; cross-checking aid, slower               */
#define TRIMUL_FLAG_SERIAL_LAUNCH 32u  /* launch the tensor-core stages without programmatic dependent
                                         launch.  By default a stage may be scheduled while its
                                         predecessor in the stream drains and waits on the device
                                         (griddepcontrol.wait) before it touches global memory; the
                                         results are the same either way                            */

/*
 * Problem description.  `rows`/`row0` select a horizontal slab of z for the row-sharded
 * multi-GPU form: this call sees z rows [row0, row0+rows) of the N x N grid, as a dense
 * [B, rows, N, c] tensor, and produces the matching [B, rows, N, c] slab of the output.
 * The whole-block entry point requires rows == N and row0 == 0.
 */
typedef struct trimul_desc {
    uint32_t struct_bytes;   /* sizeof(trimul_desc), for ABI evolution                              */
    int32_t  B;              /* batch                                                               */
    int32_t  N;              /* tokens: z is N x N positions per batch                              */
    int32_t  c;              /* d_pair = channels of z and of the output                            */
    int32_t  c_hidden;       /* h = d_hidden: the number of a/b/tri planes per batch element, the rows
                                of the four input projections, the width of LayerNorm_out and the
                                in_features of w_out (kernels/trimul_inproj/whole_op.py:203-209).  A
                                multiple of 8, at most 256; the reference module only ever builds
                                h == c (reference.py:51-59), the functional op and the bidirectional
                                block (bidirectional.py:73-84, where this field is 2 * d_hidden) also
                                other widths.  tcgen05 kernels exist for bf16 with c == 128 (stage 1:
                                h == 128; stage 3: h == 128 or 256) and, for the reference's d_pair
                                sweep, c == h == 64 and c == h == 256; other bf16 widths that are
                                multiples of 16 run that stage on warp-MMA kernels, the rest (and
                                fp32) on CUDA-core kernels; the contraction is on tcgen05 at every
                                bf16 width                                                          */
    int32_t  dtype;          /* TRIMUL_DTYPE_*                                                      */
    int32_t  direction;      /* TRIMUL_OUTGOING / TRIMUL_INCOMING                                   */
    int32_t  mask_kind;      /* TRIMUL_MASK_*                                                       */
    float    eps_in;         /* LayerNorm_in epsilon  (1e-5 in the reference)                       */
    float    eps_out;        /* LayerNorm_out epsilon                                               */
    uint32_t flags;          /* TRIMUL_FLAG_*                                                       */
    int32_t  rows;           /* z rows in this call (N for the unsharded block)                     */
    int32_t  row0;           /* global index of the first of them                                   */
    const void* drop_scale;  /* optional (NULL = none): the reference module's row-broadcast dropout
                                scale, a DEVICE pointer to [B, 1, N, c] values of the activation
                                dtype, 16-byte aligned (module.py:332-337).  The last stage multiplies
                                the block output by it before the residual is added, as the
                                reference's gate kernel does (kernels/trimul_inproj/triton/
                                gate_elem.py:41-78).  Not available together with a residual that is
                                a different tensor from z on the tensor-core path
                                (TRIMUL_E_UNSUPPORTED).  Callers built against the descriptor
                                without this field pass the shorter struct_bytes and are served
                                as before                                                            */
} trimul_desc;

/* Parameters, named as in reference.py:51-59.  Linear weights have the activation dtype;
 * the four ln_* vectors are always fp32. */
typedef struct trimul_weights {
    const float* ln_in_weight;    /* ln_pair.weight  [c] */
    const float* ln_in_bias;      /* ln_pair.bias    [c] */
    const void*  w_left;          /* to_left.weight        [h,c]   (h = c_hidden) */
    const void*  w_left_gate;     /* to_left_gate.weight   [h,c] */
    const void*  w_right;         /* to_right.weight       [h,c] */
    const void*  w_right_gate;    /* to_right_gate.weight  [h,c] */
    const float* ln_out_weight;   /* ln_out.weight   [h] */
    const float* ln_out_bias;     /* ln_out.bias     [h] */
    const void*  w_gate;          /* to_gate.weight        [c,c] */
    const void*  w_out;           /* to_out.weight         [c,h] */
} trimul_weights;

/*
 * Channel-major operand planes: the layout of a, b and tri between the stages.
 * Logical shape [planes = B*c_hidden][rows][cols]; element (p, r, q) lives at
 *     base + (r / row_chunk) * chunk_stride + p * plane_stride + (r % row_chunk) * pitch + q       (row-chunked)
 *     base + (q / col_chunk) * chunk_stride + p * plane_stride + r * pitch + (q % col_chunk)       (col-chunked)
 * in elements.  row_chunk == rows and col_chunk == cols (chunk_stride ignored) is the plain
 * single-GPU layout; at most one of the two may be chunked.  Chunked forms are what an
 * all-gather / all-to-all of per-rank slabs leaves in memory, so the contraction can read the
 * gathered operand in place.  pitch, plane_stride and chunk_stride must be multiples of 8
 * elements and `base` 16-byte aligned (128 for the tensor-core kernels).
 */
typedef struct trimul_planes {
    void*   base;
    int64_t rows;
    int64_t cols;
    int64_t pitch;
    int64_t plane_stride;
    int64_t chunk_stride;
    int64_t row_chunk;
    int64_t col_chunk;
} trimul_planes;

/* ABI version of the loaded library (TRIMUL_B200_ABI_VERSION it was built with). */
int trimul_b200_abi_version(void);

/* Human-readable text for a TRIMUL_E_* code.  Never NULL. */
const char* trimul_b200_strerror(int code);

/*
 * Bytes of device workspace trimul_b200_forward needs for `desc` (the a, b and tri planes),
 * and — when the out-pointers are non-NULL — the three plane descriptors the block uses
 * inside a workspace that starts at address 0 (add the real base to each `base`).
 * Replaces the per-call torch.empty intermediates of the reference fast path
 * (module.py:431-452).
 */
int trimul_b200_workspace_bytes(const trimul_desc* desc, size_t* bytes,
                                trimul_planes* a, trimul_planes* b, trimul_planes* tri);

/*
 * The whole block.  z, out (and residual when non-NULL): [B,N,N,c] dense, activation dtype,
 * 16-byte aligned; out must not alias z.  mask: per desc->mask_kind, or NULL.  residual
 * non-NULL adds it to the result (the reference module's `out + pair`, module.py:453);
 * NULL gives reference.py's output.  Drop-in for TriangleMultiplication._forward_cute_free
 * (module.py:399-459) and for triangle_multiplicative_update_cute
 * (src/miniworld_engine/modules/triangle_multiplication/interface.py:8-22).
 */
int trimul_b200_forward(const trimul_desc* desc, const void* z, const uint8_t* mask,
                        const trimul_weights* w, void* out, const void* residual,
                        void* workspace, size_t workspace_bytes,
                        void* stream, int32_t* status);

/*
 * Stage 1: LayerNorm_in + mask + the two sigmoid-gated projections.  Reads the z slab
 * [B, rows, N, c]; writes a and b as channel-major planes.  Outgoing: plane element
 * (r, k) is position (row0+r, k), planes are [B*c_hidden][rows][N].  Incoming: the planes are
 * stored transposed, element (i, k) is position (row0+k, i), planes are [B*c_hidden][N][rows],
 * so that the contraction is "rows times rows over a contiguous k" in both directions.
 * Replaces fused_ln_mask + tm1_cute_forward(out_layout="bdll_sm100")
 * (module.py:422-438; kernels/tm1/cute/sm100_gate_gemm_collective.py:586-647).
 */
int trimul_b200_tm1(const trimul_desc* desc, const void* z, const uint8_t* mask,
                    const trimul_weights* w, const trimul_planes* a, const trimul_planes* b,
                    void* stream, int32_t* status);

/*
 * Stage 2: tri[p][i][j] = sum_k a[p][i][k] * b[p][j][k] for every plane p, fp32
 * accumulation.  a: [planes][rows_a][K], b: [planes][rows_b][K], tri: [planes][rows_a][rows_b].
 * `dtype` is TRIMUL_DTYPE_*.  Replaces the einsum / cuBLAS bmm of module.py:439-442.
 */
int trimul_b200_contract(int32_t dtype, uint32_t flags, int32_t planes,
                         const trimul_planes* a, const trimul_planes* b, const trimul_planes* tri,
                         void* stream, int32_t* status);

/*
 * Scattering variants of stages 1 and 2, for a contraction that is sharded over channel planes
 * across several GPUs of one node.  They have NO counterpart in the reference, which runs on a
 * single GPU: they are the exchange steps of the multi-GPU plan, performed by the producing
 * kernels' own stores instead of by separate collectives.
 *
 * trimul_b200_tm1_scatter: as trimul_b200_tm1, but planes [k*P, (k+1)*P), P = B*c / n_dest, are
 * written to a_dest[k] / b_dest[k] (plane index inside a destination counts from 0).
 * trimul_b200_contract_scatter: as trimul_b200_contract, but output rows [k*R, (k+1)*R),
 * R = rows_a / n_dest, are written to tri_dest[k] (row index inside a destination counts from 0).
 * Destination buffers may lie in another GPU's memory that is mapped into this process (peer
 * access); all destinations of one call share one geometry and only differ in `base`.
 * The calls order nothing between GPUs: the caller puts a cross-GPU barrier between a scattering
 * stage and the stage that consumes what other GPUs scattered.  1 <= n_dest <= 8.  Only the
 * tensor-core kernels scatter: bf16, c = 128, P a multiple of 16 that divides or is a multiple of
 * 128, R a multiple of 128; anything else returns TRIMUL_E_UNSUPPORTED and the caller falls back
 * to the plain stages plus a collective.
 */
int trimul_b200_tm1_scatter(const trimul_desc* desc, const void* z, const uint8_t* mask,
                            const trimul_weights* w, int32_t n_dest, const trimul_planes* a_dest,
                            const trimul_planes* b_dest, void* stream, int32_t* status);
int trimul_b200_contract_scatter(int32_t dtype, uint32_t flags, int32_t planes,
                                 const trimul_planes* a, const trimul_planes* b, int32_t n_dest,
                                 const trimul_planes* tri_dest, void* stream, int32_t* status);

/*
 * Barrier over the `world` GPUs of one node for the scattering stages above, enqueued on `stream`.
 * (No counterpart in the reference, which has no multi-GPU code.)  peer_flags[r], r < world, is
 * the DEVICE address — valid on this GPU, i.e. peer-mapped for r != rank — of rank r's flag array:
 * `world` int32 words, zero before the first barrier.  `epoch` numbers the barriers 1, 2, 3, ...
 * and must be the same on every rank for the same barrier.  The kernel stores `epoch` into word
 * [rank] of every rank's array (release, system scope) and waits until every word of its own array
 * has reached `epoch` (acquire).  The wait is bounded by `timeout_us`: when it runs out the kernel
 * writes {TRIMUL_E_DEVICE_TIMEOUT, 9, missing rank, epoch} to `status` and returns, so the caller —
 * who reads the status words after synchronising — learns that a peer never arrived instead of
 * hanging.  Plain peer loads and stores; no multicast.
 */
int trimul_b200_peer_barrier(int32_t rank, int32_t world, int32_t* const* peer_flags, uint32_t epoch,
                             uint32_t timeout_us, void* stream, int32_t* status);

/*
 * Self-test of the bounded device-side waits.  (No counterpart in the reference.)  Launches one
 * small kernel that waits, with a limit of `timeout_us`, on a barrier nothing will ever complete:
 * the wait gives up, the kernel writes {TRIMUL_E_DEVICE_TIMEOUT, 10, 0, 1077} to `status` and returns
 * normally; the context stays usable.  `status` must be non-NULL and zeroed.
 */
int trimul_b200_selftest_expiring_wait(uint32_t timeout_us, void* stream, int32_t* status);

/*
 * Stage 3: LayerNorm_out over the channels of tri, the output projection, the output gate
 * computed from a fresh LayerNorm_in of the z slab (unmasked, reference.py:83), optional
 * residual; writes out [B, rows, N, c].  tri planes are [B*c_hidden][rows][N] for both directions.
 * Replaces trimul_back_split_sm100 + the residual add (module.py:445-453;
 * kernels/trimul_inproj/cute/back_split_sm100.py:26-34).
 */
int trimul_b200_tm2(const trimul_desc* desc, const void* z, const trimul_planes* tri,
                    const trimul_weights* w, void* out, const void* residual,
                    void* stream, int32_t* status);

/*
 * The whole BIDIRECTIONAL block (bidirectional.py:93-156): one input LayerNorm, the four gated
 * projections of width 2h (rows [0,h) of each weight feed an outgoing contraction, rows [h,2h) an
 * incoming one), one LayerNorm over the 2h result channels, to_out [c,2h] gated by to_gate(x_n);
 * `add_residual` != 0 adds z (what the reference module always returns).
 * `desc`: c_hidden = 2h (h = d_hidden a multiple of 8, 2h <= 256), rows = N, row0 = 0; `direction`
 * is ignored; mask kinds as in the single-direction block.  `w`: w_left, w_left_gate, w_right,
 * w_right_gate are [2h, c]; ln_out_* have 2h entries; w_gate is [c, c]; w_out is [c, 2h].  The
 * workspace holds three plane sets of B*2h planes (trimul_b200_bidir_workspace_bytes); per batch
 * element planes [0,h) belong to the outgoing half and [h,2h) to the incoming half.  bf16 with
 * c = h = 128 runs every stage on the tensor cores.  Replaces the sm_100 path
 * BidirectionalTriangleMultiplication._forward_cute (bidirectional.py:118-132;
 * kernels/trimul_inproj/cute/bidirectional_sm100.py:33-71).
 */
int trimul_b200_bidir_workspace_bytes(const trimul_desc* desc, size_t* bytes);
int trimul_b200_forward_bidir(const trimul_desc* desc, const void* z, const uint8_t* mask,
                              const trimul_weights* w, void* out, int32_t add_residual,
                              void* workspace, size_t workspace_bytes, void* stream, int32_t* status);

/*
 * The whole block for callers that have no device memory to offer as a workspace.
 * (No counterpart in the reference: its launchers allocate their intermediates with torch.)
 *
 * Some hosts of this library cannot hand over a workspace: a serving process that gave all
 * device memory to its own pool at start-up, where a cudaMalloc issued from a plugin fails
 * or eats into someone else's budget; a latency-critical loop that must not hit cudaMalloc's
 * device-wide synchronisation; a foreign-function boundary that passes inputs and outputs
 * only.  For them the a/b/tri planes live in a fixed array that is part of the library's
 * device image, TRIMUL_B200_STATIC_SCRATCH_BYTES large.  Every GPU on which the library is
 * used holds that array from the moment the library's device code is loaded there until the
 * process exits, whether or not this function is ever called.
 *
 * Same arguments and results as trimul_b200_forward, minus the workspace.  Differences:
 *   - a problem whose planes need more than TRIMUL_B200_STATIC_SCRATCH_BYTES (see
 *     trimul_b200_workspace_bytes; N <= 208 at c = 128 in bf16 with B = 1) is refused
 *     with TRIMUL_E_STATIC_SCRATCH before anything is enqueued;
 *   - the first call on each device looks up the array's device address (once per device,
 *     with that device current).  Make that first call before any stream capture begins;
 *   - there is ONE array per device, shared by every call and every stream, and it keeps
 *     whatever the previous call left in it.  The kernels overwrite every element they later
 *     read, so nothing needs clearing between calls, but two calls whose kernels overlap on
 *     the GPU (different streams, no dependency between them) race on it and both results
 *     are then undefined.  Order such calls yourself;
 *   - it calls no cudaMalloc, cudaFree or other allocating routine, and needs no torch.
 */
#define TRIMUL_B200_STATIC_SCRATCH_BYTES (32u << 20)

int trimul_b200_forward_static(const trimul_desc* desc, const void* z, const uint8_t* mask,
                               const trimul_weights* w, void* out, const void* residual,
                               void* stream, int32_t* status);

#ifdef __cplusplus
}
#endif
#endif /* TRIMUL_B200_H_ */
