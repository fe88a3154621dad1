/*
 * b2_w4a16.h - C ABI of the B200 (sm_100a) W4A16 quantized-linear engine.
 *
 * Plain pointers and sizes only: no torch types, no C++ types, no exceptions.  Every
 * function returns an int status (B2_OK == 0); b2_w4a16_last_error() gives the text of
 * the calling thread's last failure.  All pointers except `*_host` arguments are device
 * pointers on the CURRENT device; `stream` is a cudaStream_t passed as void* (NULL = the
 * legacy default stream).  Calls are asynchronous, never synchronize, never read tensor
 * values on the host and allocate nothing, so they may be captured into a CUDA graph.
 *
 * Each entry point names the reference interface it stands in for (paths inside the
 * reference project, dandan-ops).
 *
 * Tensor conventions (row-major, contiguous unless a leading dimension is given):
 *   packed  int32  [N, ceil(K/8)]   eight unsigned 4-bit codes per word, code j in bits 4j..4j+3
 *   scales  float  [N, ceil(K/64)]  one step per output row and group of 64 inputs
 *   zeros   int32  [N, ceil(K/64)]  zero points in 0..15
 *   x       fp16   [M, K]  (row stride ldx elements)
 *   y       fp16   [M, N]  (row stride ldy elements)
 *   weight  w[n,k] = fp16_rn( fp32(code - zero) * step ),  y = fp16_rn( sum_k fp32(x)*fp32(w) )
 * Only group size 64 exists in this ABI.
 */
#ifndef B2_W4A16_H
#define B2_W4A16_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_OK 0
#define B2_ERR_ARGUMENT 1    /* null pointer, non-positive size, misaligned native buffer */
#define B2_ERR_CUDA 2        /* a CUDA runtime call or a kernel launch failed */
#define B2_ERR_WORKSPACE 3   /* workspace smaller than b2_w4a16_workspace_bytes() */
#define B2_ERR_RANGE 4       /* dimensions exceed the kernel index range */
#define B2_ERR_UNSUPPORTED 5 /* device is not sm_100 or the requested route does not apply */

/* Kernel families selectable through b2_w4a16_linear_route(). */
#define B2_ROUTE_AUTO 0      /* by size: tile kernel for M <= 16 on layers up to ~10 MB, streaming kernel up to
                                B2_STREAM_MAX_M rows (32 rows on layers above ~10 MB), tensor-memory GEMM above */
#define B2_ROUTE_STREAM 1    /* persistent weight-streaming kernel (any M, re-reads the weights every 64 rows) */
#define B2_ROUTE_TCGEN05 2   /* TMA + tcgen05 GEMM with in-kernel INT4->FP16 converter */
#define B2_ROUTE_TILE 3      /* one CTA (or a cluster of 2 or 4 CTAs that split K) per 16-row tile, the whole K range
                                in flight at once (M <= 16; K as far as it fits in shared memory) */

/* Largest M the weight-streaming kernel takes in one launch; B2_ROUTE_AUTO hands larger
 * batches to the tensor-memory GEMM. */
#define B2_STREAM_MAX_M 64

/* Every workspace starts with this many bytes of arrival counters (one per 16-row tile;
 * K is only split when a layer has fewer row tiles than this). */
#define B2_W4A16_TICKET_BYTES 32768

/* Contract version of the packed format and numerics; 2, as the reference's
 * `w4a16_contract_version` op (dandan_ops/csrc/operators.cu:260). */
int b2_w4a16_contract_version(void);

/* Text of the calling thread's last error ("" if none). */
const char* b2_w4a16_last_error(void);

/* Bytes of the device-native weight image for an [N, K] layer (0 on bad sizes).
 * The image holds the 4-bit codes, FP32 steps and 4-bit zero points tiled in
 * 16-row x 256-column blocks of 2336 bytes: 0.5703 bytes per weight when N and K are
 * multiples of 16 and 256.  The reference keeps 0.625 bytes per weight
 * (QuantizedLinear.storage_bytes, dandan_ops/quantized_linear.py:176-178). */
int64_t b2_w4a16_native_bytes(int64_t n, int64_t k);

/* Reference layout -> native image.  `native` must be 256-byte aligned and
 * b2_w4a16_native_bytes(n,k) long.  Replaces the layout half of pack_int4
 * (dandan_ops/quantization.py:85-103): the reference kernels read that layout
 * directly, this engine reads the tiled image. */
int b2_w4a16_repack(const int32_t* packed, const float* scales, const int32_t* zeros,
                    int64_t n, int64_t k, void* native, void* stream);

/* Native image -> reference layout (exact inverse of b2_w4a16_repack; codes beyond K
 * in the last word come back as 0, as pack_int4 writes them). */
int b2_w4a16_unrepack(const void* native, int64_t n, int64_t k, int32_t* packed,
                      float* scales, int32_t* zeros, void* stream);

/* uint8 codes [N,K] (values 0..15) -> packed int32 [N, ceil(K/8)].
 * Replaces pack_int4 (dandan_ops/quantization.py:85-103). */
int b2_w4a16_pack(const uint8_t* codes, int64_t n, int64_t k, int32_t* packed, void* stream);

/* Native image -> FP32 weights [N,K] (row stride ldo), bit-identical to
 * dequantize_int4 (dandan_ops/quantization.py:124-143). */
int b2_w4a16_dequantize(const void* native, int64_t n, int64_t k, float* out, int64_t ldo,
                        void* stream);

/* Same, rounded once more to FP16: the weights the linear kernels multiply by
 * (`dequantize_int4(...).half()`, dandan_ops/quantized_linear.py:75-76). */
int b2_w4a16_dequantize_fp16(const void* native, int64_t n, int64_t k, void* out_fp16,
                             int64_t ldo, void* stream);

/* Scratch bytes b2_w4a16_linear needs for this problem on the current device (always > 0).
 * The first B2_W4A16_TICKET_BYTES bytes hold per-tile arrival counters: they must be
 * ZERO before the first call that uses the buffer and every call leaves them zero (the
 * last word of that area is a sticky status word, see b2_w4a16_status), so one buffer can
 * serve any number of calls (and graph replays) on one stream.  Calls that may overlap on
 * the GPU need separate workspaces.  b2_w4a16_linear always needs a workspace. */
int64_t b2_w4a16_workspace_bytes(int64_t m, int64_t n, int64_t k);

/* Reads the workspace's sticky status word into *status_host (0 = every kernel that used
 * the workspace ran to completion; bit 0 = a warp gave up waiting for a weight copy and
 * the outputs of that call are undefined).  workspace == NULL reads the word of the scratch built
 * into the library (b2_w4a16_linear_static).  SYNCHRONIZES the stream; diagnostics only. */
int b2_w4a16_status(const void* workspace, void* stream, unsigned* status_host);

/* y = x @ W^T for one layer.  Replaces the four reference ops
 *   w4a16_gemv        dandan_ops/csrc/operators.cu:122-137
 *   w4a16_gemm        dandan_ops/csrc/operators.cu:90-120
 *   w4a16_small       dandan_ops/csrc/hgemm.cu:70-86
 *   w4a16_tensorcore  dandan_ops/csrc/hgemm.cu:63-68
 * with one engine that picks the kernel by M.  m == 0 returns B2_OK without a launch.
 * Limits (as check_w4a16, dandan_ops/csrc/gemm_checks.h:22-25): m*k, m*n and n*k must
 * each fit in int32. */
int b2_w4a16_linear(const void* x, int64_t ldx, const void* native, void* y, int64_t ldy,
                    int64_t m, int64_t n, int64_t k, void* workspace, int64_t workspace_bytes,
                    void* stream);

/* No counterpart in the reference.  y = x @ W^T for at most B2_STREAM_MAX_M rows of x, with
 * the scratch memory built into the library instead of a caller-supplied workspace.
 *
 * For callers that cannot hand over device memory of their own and must not allocate:
 * an operator slot whose interface passes only inputs and outputs (no workspace
 * argument), a runtime whose memory is planned ahead and frozen, code running where
 * cudaMalloc would stall the device or is simply forbidden.  This call allocates
 * nothing - no cudaMalloc/cudaFree, no allocating library routine - and needs nothing
 * from the caller beyond x, the weight image and y.
 *
 * The scratch is one fixed array of B2_W4A16_STATIC_SCRATCH_BYTES in device memory; every
 * GPU that loads this library holds it until the process exits.  Limits and rules:
 *   - m <= B2_STREAM_MAX_M, and the tickets plus split-K partial tiles of the streaming kernel's
 *     plan for (m,n,k) must fit in B2_W4A16_STATIC_SCRATCH_BYTES (never more than
 *     b2_w4a16_workspace_bytes(m,n,k)); otherwise B2_ERR_RANGE with a message naming both sizes
 *     (the call always uses the streaming kernel);
 *   - the first call on a device looks up the array's device address (one runtime query, no
 *     allocation); make that first call before starting any stream capture;
 *   - all calls on a device share the array and it keeps the previous call's contents; each
 *     call re-zeroes the part that must start at zero (an async memset on `stream`); the sticky
 *     status word is kept and b2_w4a16_status(NULL, stream, &word) reads it;
 *   - two calls that overlap on the GPU (different streams, or graphs replayed concurrently)
 *     race on the array: serialize them, or give one of them b2_w4a16_linear and a workspace. */
#define B2_W4A16_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int b2_w4a16_linear_static(const void* x, int64_t ldx, const void* native, void* y, int64_t ldy,
                           int64_t m, int64_t n, int64_t k, void* stream);

/* Same with an explicit kernel family (B2_ROUTE_*), for tests and benchmarks. */
int b2_w4a16_linear_route(const void* x, int64_t ldx, const void* native, void* y, int64_t ldy,
                          int64_t m, int64_t n, int64_t k, void* workspace,
                          int64_t workspace_bytes, void* stream, int route);

/* y = fp16(x @ W^T) + bias, the bias add fused into the kernels' output stage with the
 * reference's rounding order: the product is rounded to FP16 first, then the FP16 bias is added
 * in FP16 (`y + bias.to(y.dtype)`, dandan_ops/quantized_linear.py:81, a separate elementwise
 * launch there).  `bias_fp16` is [N] FP16, 4-byte aligned, or NULL for no bias. */
int b2_w4a16_linear_bias(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* y,
                         int64_t ldy, int64_t m, int64_t n, int64_t k, void* workspace,
                         int64_t workspace_bytes, void* stream, int route);

/* Same with layer flags.  B2_FLAG_FP16_STEPS: the caller asserts that EVERY step (scale) of the layer is
 * exactly representable in FP16 - true for checkpoints that store FP16 scales.  The decode kernels (M <= 16,
 * 16-byte aligned x) and the converters of the pair GEMM (16-byte aligned y) then dequantize with two FP16 instructions per weight pair instead of the mixed-precision
 * chain: (code - zero) * step has at most 15 significant bits, so fp16_rn(fp32(code - zero) * step) ==
 * hmul2(code - zero, step) and the weights are bit-identical to the general path.  The flag changes speed only;
 * set on a layer with other steps it gives wrong weights.  No counterpart in the reference (its kernels
 * multiply in FP32 throughout, kernels/w4a16_small.cuh:39). */
#define B2_FLAG_FP16_STEPS 1
/* B2_FLAG_OVERLAP_LAUNCH: the decode kernels (tile and streaming) may start before the previous kernel of the
 * stream has finished (programmatic dependent launch).  As that kernel drains, CTAs of this one move in, set
 * up their barriers and request their weight blocks (the tile kernel all of them, the streaming kernel the
 * first ring); they touch x, bias, y and the workspace only after the previous kernel has completed and its
 * writes are visible (griddepcontrol.wait).  The caller asserts that the weight IMAGE is not being written by
 * work still in flight on the stream (it is constant after the layer was built).  Hides the launch latency and
 * the first trip of the weights behind the previous kernel's tail; results are unchanged.  The tensor-core
 * GEMM ignores the flag. */
#define B2_FLAG_OVERLAP_LAUNCH 2
int b2_w4a16_linear_flags(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* y,
                          int64_t ldy, int64_t m, int64_t n, int64_t k, void* workspace,
                          int64_t workspace_bytes, void* stream, int route, int flags);

/* Fused gate/up projection of a gated MLP: y[M, N/2] = SiLU(g) * u with g, u = the FP16 outputs
 * (bias included) of the gate and up rows, rounded as the reference's separate launch does
 * (`silu_and_mul`: SiLU rounded to FP16 before the multiplication, dandan_ops/elementwise.py:168-173,
 * dandan_ops/csrc/elementwise.cu:70-73).  The image must be built from rows in PAIR ORDER: every
 * 16-row tile holds 8 gate rows followed by the 8 up rows of the same output columns
 * (N % 16 == 0), and `bias_fp16` follows the same order.  The product and the activation never
 * leave the SM: the decode kernels hold a gate/up pair in one thread, the pair GEMM exchanges
 * the two sums between lanes l and l ^ 8 of its epilogue warps.  b2_w4a16_silu_mul_is_fused() tells
 * whether a problem runs this way (everything except batches above 64 rows whose GEMM tile shape is a
 * single-CTA one); the others call b2_w4a16_linear on the same image and then
 * b2_w4a16_silu_mul_pairs, and this function returns B2_ERR_UNSUPPORTED for them. */
int b2_w4a16_linear_silu_mul(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* y,
                             int64_t ldy, int64_t m, int64_t n, int64_t k, void* workspace,
                             int64_t workspace_bytes, void* stream);
/* Same with the layer flags of b2_w4a16_linear_flags (FP16-step dequantization, overlap launch). */
int b2_w4a16_linear_silu_mul_flags(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* y,
                                   int64_t ldy, int64_t m, int64_t n, int64_t k, void* workspace,
                                   int64_t workspace_bytes, void* stream, int flags);
int b2_w4a16_silu_mul_is_fused(int64_t m, int64_t n, int64_t k);

/* Residual add + RMSNorm in front of a projection (the step before the qkv projection of a decoder
 * layer):  s = fp16(x + residual)  (residual may be NULL: s = x),  xn = fp16(fp16(s * rsqrt(mean(s^2)
 * + eps)) * norm_weight),  y = xn @ W^T (+ bias) - the rounding order of the reference's
 * `residual_rms_norm` (dandan_ops/elementwise.py:156-165, dandan_ops/csrc/elementwise.cu:39-62).
 * `summed` (optional, [M, K], row stride lds) receives s for the residual stream; `xn_scratch`
 * ([M, K] FP16, row stride K) receives xn.  Two launches on `stream`: the norm kernel below, then
 * b2_w4a16_linear.  (A variant that normalized the tile kernel's shared-memory copy of x inside the
 * projection launch was measured and dropped: every CTA repeats the norm, which cost more than the
 * second launch.)  K, ldx, ldr, lds multiples of 8; pointers 16-byte aligned. */
int b2_w4a16_rmsnorm_linear(const void* x, int64_t ldx, const void* residual, int64_t ldr, const void* norm_weight,
                            float eps, void* summed, int64_t lds, void* xn_scratch, const void* native,
                            const void* bias_fp16, void* y, int64_t ldy, int64_t m, int64_t n, int64_t k,
                            void* workspace, int64_t workspace_bytes, void* stream);

/* The norm alone (the first launch of b2_w4a16_rmsnorm_linear):
 * summed = fp16(x + residual) (optional output), out = RMSNorm(summed) * norm_weight. */
int b2_w4a16_residual_rms_norm(const void* x, int64_t ldx, const void* residual, int64_t ldr, const void* norm_weight,
                               float eps, void* summed, int64_t lds, void* out, int64_t ldo, int64_t m, int64_t k,
                               void* stream);

/* out[M, N/2] = SiLU(in[m][16j+g]) * in[m][16j+8+g] for out column 8j+g: the elementwise form of
 * the epilogue above, for outputs of b2_w4a16_linear on a pair-ordered image. */
int b2_w4a16_silu_mul_pairs(const void* y_pairs, int64_t ld_in, void* out, int64_t ld_out, int64_t m, int64_t n,
                            void* stream);

/* Which kernel family B2_ROUTE_AUTO picks for this problem (a B2_ROUTE_* value) and,
 * through the optional out-parameters, the launch plan: K-splits, grid size, rows of x
 * handled per launch.  Pure host arithmetic; used by execution_info(). */
int b2_w4a16_plan(int64_t m, int64_t n, int64_t k, int* route, int* k_splits, int* grid,
                  int* rows_per_launch);

/* Tile shape of the tensor-memory GEMM (B2_ROUTE_TCGEN05).  B2_GEMM_SHAPE_AUTO picks per call
 * by a cost model (waves x cost per tile); the others force one shape for every later call of
 * the process, for tests and tuning.  The single-CTA shapes are rows of x by output columns per
 * CTA; the PAIR shapes run on two SMs per tile (tcgen05 cta_group::2, weights through tensor
 * memory): 256 output columns by 256 or 192 rows of x.  No counterpart in the reference, whose
 * route table is fixed offline (dandan_ops/_dispatch.py). */
#define B2_GEMM_SHAPE_AUTO 0
#define B2_GEMM_SHAPE_128x128 1
#define B2_GEMM_SHAPE_256x128 2
#define B2_GEMM_SHAPE_256x192 3
#define B2_GEMM_SHAPE_PAIR_256 4
#define B2_GEMM_SHAPE_PAIR_192 5
/* k_splits: CTAs along K per tile of the PAIR shapes, 1..8, or 0 = by the cost model (K is split
 * when a layer has fewer tiles than SM pairs; the FP32 partial tiles meet in the workspace and
 * are added in split order, so results do not depend on timing).  A split the problem or the
 * workspace cannot take (fewer than four 256-column blocks per CTA, too many tiles for the ticket
 * area, workspace smaller than b2_w4a16_workspace_bytes()) is reduced. */
int b2_w4a16_set_gemm_shape(int shape, int k_splits);

/* Multi-GPU: all-gather of the column slices of an [M, N] FP16 output over NVLink.  No counterpart in
 * the reference, which is single-GPU; it is the collective step of the column-sharded layer (each rank
 * owns the output columns of its rows of W).  Rank q owns the columns [q * slice_cols, min(n_total,
 * (q + 1) * slice_cols)).  Every rank has its own copy of the [m, ld] buffer in memory that all peers can
 * write (peer-mapped / symmetric memory) and has written its slice into its own copy - the projection
 * stores there directly.  One launch; when the kernel ends, the local copy holds every rank's slice.
 * Nothing reads remote memory, no TMA or bulk copy touches a peer, nothing is multicast.
 *   y_ranks[q], flag_blocks[q]  HOST arrays of `world` device pointers as mapped into this process
 *                               (entry [rank] is this rank's own).  A flag block is
 *                               b2_w4a16_gather_block_bytes(world, mailbox_slice_bytes) of zero-initialised,
 *                               8-byte aligned memory, one per rank and process, shared by every gathered
 *                               layer; all ranks must issue the same sequence of gathers with the same
 *                               mailbox_slice_bytes.
 * Two forms, chosen by size (the same way on every rank):
 *   - a rank's slice (m * slice_cols * 2 bytes) fits in mailbox_slice_bytes and the slices are 4-byte
 *     aligned: every word travels as an 8-byte packet {word, epoch} into the peer's mailbox, and the
 *     receiving kernel polls the packets and copies the words into its buffer - one NVLink crossing, no
 *     fence, ~5 us per gather (latency is all that matters at decode sizes);
 *   - otherwise: the slice is pushed straight into every peer's buffer with 16-byte stores, then the last
 *     CTA publishes this call's epoch in every peer's flag block (st.release.sys) and waits for theirs.
 * Every wait is bounded by the clock (five seconds by default, b2_w4a16_gather_wait_limit): if a peer's data
 * does not arrive, bit 2 of the flag block's status word is set (b2_w4a16_gather_status reads it,
 * synchronizing) and the kernel returns.  Reuse of one buffer: a peer may start writing the next call's slice
 * as soon as it has finished this call, so between two gathers into the SAME buffer a rank must issue at
 * least one other gather (or alternate two buffers). */
int64_t b2_w4a16_gather_block_bytes(int world, int64_t mailbox_slice_bytes);
int b2_w4a16_gather(void* const* y_ranks, void* const* flag_blocks, int64_t mailbox_slice_bytes, int rank, int world,
                    int64_t m, int64_t ld, int64_t n_total, int64_t slice_cols, void* stream);
int b2_w4a16_gather_status(const void* flag_block, void* stream, unsigned* status_host);
int b2_w4a16_gather_wait_limit(int64_t microseconds);      /* <= 0 restores the default */

/* Column-sharded projection and all-gather as ONE call: y_ranks[rank][:, :n_total] = x W^T (+bias) on every
 * rank, where this rank's `native` image holds its rows [rank * slice_cols, min(n_total, (rank + 1) *
 * slice_cols)) of W and `bias_fp16` (optional) those entries of the bias.  Arguments as b2_w4a16_gather and
 * b2_w4a16_linear_flags; `ld` is the row stride of the gathered buffers.
 * Decode sizes (m <= 16, a slice that fits a mailbox half, K % 8 == 0, an aligned x) run as one launch.
 * Layers of the streaming kernel, w4a16_stream_gather_kernel: the warp that completes a 16-column tile stores it
 * into the local buffer and sends it to every peer's mailbox as {word, epoch} packets while the rest of the
 * weight stream is still running; CTAs that have finished their range poll the packets the peers sent.
 * Layers of the tile kernel, w4a16_tile_gather_kernel: every CTA sends its tile, and the last CTA to finish
 * collects the peers' packets - taken while that is a single round of four packets per thread.
 * The transfer overlaps the math tile by tile and the launch, fence and flag round trip of a separate gather
 * disappear.  Everything else runs the projection (b2_w4a16_linear_flags into the local slice) followed by
 * b2_w4a16_gather - same result, two launches; b2_w4a16_linear_gather_launches() says which (0 = bad arguments).
 * All ranks must make the same sequence of calls; waits are bounded as in b2_w4a16_gather. */
int b2_w4a16_linear_gather(const void* x, int64_t ldx, const void* native, const void* bias_fp16, void* const* y_ranks,
                           void* const* flag_blocks, int64_t mailbox_slice_bytes, int rank, int world, int64_t m,
                           int64_t ld, int64_t n_total, int64_t slice_cols, int64_t k, void* workspace,
                           int64_t workspace_bytes, void* stream, int flags);
int b2_w4a16_linear_gather_launches(int64_t m, int64_t n_total, int64_t slice_cols, int64_t k, int rank, int world,
                                    int64_t mailbox_slice_bytes);

/* Launches an empty kernel on `stream`: the floor of one graph node, for benchmarks. */
int b2_w4a16_noop(void* stream);

/* Test hooks, no counterpart in the reference.  wait_limit: polls after which a kernel's bounded
 * wait for a weight copy gives up (<= 0 restores the default, about a million).  skip_copy >= 0: the
 * NEXT decode-kernel launch (tile or streaming) arms the barrier of that copy of its first CTA but does
 * not issue the copy, so the wait runs out, the warp records bit 0 in the status word, drains its other
 * copies and the kernel returns - nothing hangs; -1 = off.  stream_variant: 0 or 1 = the shipped
 * streaming kernel; 2 / 3 = the double-buffered form with 32 / 16 warps per CTA, 4 = the chunk-major
 * two-dimensional split (all M <= 16), kept for measurements. */
int b2_w4a16_test_hooks(int wait_limit, int skip_copy, int stream_variant);

/* Number of kernels this library has launched from the calling process so far. */
int64_t b2_w4a16_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B2_W4A16_H */
