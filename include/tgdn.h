/* C ABI of libtgdn_b200: hand-written sm_100a CUDA kernels for the Triadic Gated DeltaNet hot path.
 *
 * Conventions shared by every entry point
 *   - every pointer is a device pointer unless its name starts with host_; the caller owns every buffer
 *     (PyTorch in the Python package), the library never allocates or frees device memory and never synchronises;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call returns at once;
 *   - the return value is 0 on success, a negative TGDN_ERR_* code for a rejected argument, or
 *     -(1000 + cudaError) for a CUDA runtime error at launch; tgdn_error_string() explains either;
 *   - bf16 tensors are raw 16-bit words; "token layout" means the caller's (B, T, H, X) contiguous tensors, "chunk
 *     layout" means (B, NC, H, ...) with NC = T/64 for dense rows or the chunk-map capacity for packed rows;
 *   - packed rows (B = 1) pass the chunk map built by tgdn_metadata; dense rows pass NULL.
 *
 * The reference package has no C interface: its boundary is Python.  Each entry point below names the reference
 * function (path inside the reference project) whose device work it replaces.
 */
#ifndef TGDN_H_
#define TGDN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TGDN_OK 0
#define TGDN_ERR_SHAPE (-1)       /* unsupported or inconsistent sizes */
#define TGDN_ERR_NULL (-2)        /* a required pointer is NULL */
#define TGDN_ERR_ALIGN (-3)       /* a pointer or stride breaks the 16-byte alignment the kernels need */
#define TGDN_ERR_DRIVER (-4)      /* the CUDA driver entry point for tensor maps is unavailable or failed */
#define TGDN_ERR_SCRATCH (-5)     /* scratch buffer missing or too small */
#define TGDN_ERR_DEVICE (-6)      /* the current device is not compute capability 10.x */
#define TGDN_ERR_STATIC_LIMIT (-7) /* the problem needs more scratch than the library's built-in static buffer holds */

/* Human-readable text for a return code of this library. */
const char* tgdn_error_string(int code);

/* Version of this ABI (major * 100 + minor). */
int tgdn_abi_version(void);

/* Blocking read-and-clear of the device status word of the current device: 0 = no kernel gave up on a wait;
 * 1 = a load barrier timed out, 2 = an MMA barrier timed out, 3 = a chunk map entry was out of range.
 * Synchronises the device; meant for tests and debugging, not for the hot path. */
int tgdn_device_status(int* host_status);

/* ---- convolution pre-pass -----------------------------------------------------------------------------------------
 * Width-4 causal depthwise convolution, f32 accumulation, SiLU on channels [0, act_channels), one bf16 rounding.
 * x (B, T, C) bf16 with element strides (stride_b, stride_t, 1); weight (C, 4) bf16 contiguous; y (B, T, C) contiguous.
 * cu_seqlens: NULL, or n_docs+1 int32 offsets of a packed row (B = 1); the window restarts at every document.
 * Replaces: cute_triadic_gdn/ops/conv_split_act.py:20-55 (_fwd_kernel), :133-146 (_forward, conv_split_act_fwd). */
int tgdn_conv_fwd(const void* x, const void* weight, void* y, const int32_t* cu_seqlens, int n_docs, int B, int T, int C,
                  int64_t stride_b, int64_t stride_t, int act_channels, void* stream);

/* Bytes of f32 scratch tgdn_conv_bwd needs for its per-tile weight-gradient partials. */
int64_t tgdn_conv_bwd_scratch_bytes(int B, int T, int C);

/* Backward of the convolution: dx (B, T, C) bf16 contiguous and dw (C, 4) bf16.  dy has element strides
 * (dy_stride_b, dy_stride_t, 1).  The SiLU derivative is evaluated at the bf16-rounded pre-activation, recomputed in
 * the same kernel; dw is summed in f32 over token tiles in a fixed order and rounded once.
 * Replaces: cute_triadic_gdn/ops/conv_split_act.py:58-107 (_bwd_kernel), :154-168 (conv_split_act_bwd). */
int tgdn_conv_bwd(const void* x, const void* weight, const void* dy, void* dx, void* dw, const int32_t* cu_seqlens,
                  int n_docs, int B, int T, int C, int64_t stride_b, int64_t stride_t, int64_t dy_stride_b,
                  int64_t dy_stride_t, int act_channels, void* scratch, int64_t scratch_bytes, void* stream);

/* Size of the scratch array built into the library for tgdn_conv_bwd_static (held on every GPU that loads the library). */
#define TGDN_CONV_STATIC_SCRATCH_BYTES (8u << 20)

/* tgdn_conv_bwd_static: tgdn_conv_bwd for callers that cannot give it scratch memory because they are not allowed to
 * allocate on the device (a host with a fixed, externally owned memory arena; a thread on which cudaMalloc is forbidden
 * or too slow because it may synchronise the device).  Same arguments and results as tgdn_conv_bwd without the scratch
 * pair; the weight-gradient partials go to a TGDN_CONV_STATIC_SCRATCH_BYTES array inside the library image.
 * Limit: tgdn_conv_bwd_scratch_bytes(B, T, C) must not exceed that size, otherwise TGDN_ERR_STATIC_LIMIT is returned
 * and nothing is launched.  The first call on each device looks up the array's device address (make it outside any
 * stream capture); the array is shared by all calls on a device, so calls that overlap on the GPU race with each other.
 * After the first call on a device (a warm-up that loads the library's CUDA module with its array and looks the address
 * up, which the CUDA runtime may answer with allocations of its own), neither this call nor anything under it allocates
 * or frees memory.
 * No counterpart in the reference (its wrappers always allocate with torch). */
int tgdn_conv_bwd_static(const void* x, const void* weight, const void* dy, void* dx, void* dw, const int32_t* cu_seqlens,
                         int n_docs, int B, int T, int C, int64_t stride_b, int64_t stride_t, int64_t dy_stride_b,
                         int64_t dy_stride_t, int act_channels, void* stream);

/* ---- packed-document metadata -------------------------------------------------------------------------------------
 * Chunk-map capacity for n_docs documents over T tokens: ceil(T/64) + n_docs - 1 rounded up to a multiple of 16.
 * Replaces: cute_triadic_gdn/ops/joint_packing.py:16-20 (chunk_capacity). */
int tgdn_chunk_capacity(int T, int n_docs);

/* Builds, on the device and without reading the offsets on the host: offsets (n_docs+1) int32 = first chunk of every
 * document; mapping (3, capacity) int32 = [first token of chunk | valid rows of chunk | documents longest first];
 * valid (1 byte) = offsets start at 0, end at T and strictly increase.  Never writes out of bounds for bad offsets.
 * cu_seqlens holds int32 (cu_is_int64 = 0) or int64 values.
 * Replaces: cute_triadic_gdn/kernels/sm90_joint_packed.py:64-129 (metadata_kernel, joint_metadata). */
int tgdn_metadata(const void* cu_seqlens, int cu_is_int64, int n_docs, int T, int32_t* offsets, int32_t* mapping,
                  int capacity, uint8_t* valid, void* stream);

/* ---- Triadic GDN core ----------------------------------------------------------------------------------------------
 * Shapes: q, k, v, o (B, T, H, 128) bf16; k2, q2, g (B, T, H, E) f32; beta (B, T, H) f32; E in {1,2,4,8,12,16}.
 * Dense rows: T % 64 == 0, NC = T/64, chunk_map = doc_offsets = NULL.  Packed rows: B = 1, NC = chunk-map capacity,
 * chunk_map / doc_offsets from tgdn_metadata, n_docs documents; the state restarts at every document.
 * Chunk-layout intermediates, indexed by item = (b*NC + n)*H + h:
 *   gc f32 [item][tgdn_gate_item_floats(E) = 256 E + 16]: the gates of the chunk in five blocks, with gL = gc[63] and
 *      zeros in rows past a document end: [0, 64E) gc[t][e] cumulative log gate; [64E, 128E) a = k2 exp(gc);
 *      [128E, 192E) r = k2 exp(gL - gc); [192E, 256E) c = scale q2 exp(gc); [256E, 256E + 16) d[e] = exp(gL), zero padded;
 *   AP bf16 [item][128*64] ([A; Pm A] operand image);  Pm bf16 [item][64*64];
 *   W, U, dU bf16 [item][64][128];  h, ds bf16 [item][E][16][128][8] (state slice as [v/8][d][v%8]).
 *
 * tgdn_masks: chunk-local cumulative log gate, the gate factors of the recurrences, UT transform and intra-chunk
 * operators of every chunk.
 * Replaces: cute_triadic_gdn/kernels/sm90_joint_scan.py:92-110 (joint_scan, forward) and
 * cute_triadic_gdn/kernels/sm100_joint_masks.py:291-323 (joint_masks_sm100). */
int tgdn_gate_item_floats(int E);
int tgdn_masks(const void* q, const void* k, const float* k2, const float* q2, const float* g, const float* beta,
               float scale, const int32_t* chunk_map, int B, int T, int H, int E, int NC, float* gc, void* AP, void* Pm,
               void* stream);

/* tgdn_fwd: the forward chunk recurrence; writes o and, unless NULL, the tensors the backward needs (W, U, h).
 * gc is the tensor tgdn_masks wrote with the same scale (the recurrences read the gate factors a, r, c, d from it; k2 and
 * q2 stay in the signature as the inputs those factors came from and are not read again); k2, q2 and gc must be 16-byte
 * aligned.
 * Replaces: cute_triadic_gdn/kernels/sm100_joint_fwd.py:569-618 (joint_fwd_sm100). */
int tgdn_fwd(const void* q, const void* k, const void* v, const float* k2, const float* q2, const float* beta,
             const float* gc, const void* AP, float scale, const int32_t* doc_offsets, const int32_t* chunk_map,
             int n_docs, int B, int T, int H, int E, int NC, void* o, void* W, void* U, void* h, void* stream);

/* tgdn_fwd_state: tgdn_fwd with the recurrent state handed in and out, for inference that continues a sequence:
 * state_in / state_out are f32 [sequence][H][E][128 key rows][128 value columns] (sequence = batch row, or document of a
 * packed row), 16-byte aligned; NULL state_in starts from zero, NULL state_out discards the final state.
 * No counterpart in the reference (its forward always starts from a zero state and drops the final one:
 * cute_triadic_gdn/kernels/sm100_joint_fwd.py:190-206). */
int tgdn_fwd_state(const void* q, const void* k, const void* v, const float* k2, const float* q2, const float* beta,
                   const float* gc, const void* AP, float scale, const int32_t* doc_offsets, const int32_t* chunk_map,
                   int n_docs, int B, int T, int H, int E, int NC, void* o, void* W, void* U, void* h,
                   const float* state_in, float* state_out, void* stream);

/* tgdn_glue_fwd: the convolution with the layer glue that follows it fused in.  x bf16 (B, T, C) with element strides
 * (stride_b, stride_t, 1), C = H (3*128 + 2E) channels laid out [q: H x 128 | k: H x 128 | v: H x 128 | k2: H x E | q2: H x E];
 * weight bf16 (C, 4); writes q, k = l2norm(SiLU(conv)) and v = SiLU(conv) as bf16 (B, T, H, 128) and k2, q2 =
 * l2norm(softplus(conv)) as f32 (B, T, H, E), l2norm(s) = s * rsqrt(sum s^2 + eps) over the last axis.  Packed rows as in
 * tgdn_conv_fwd.  The reference describes this glue (cute_triadic_gdn/ops/conv_split_act.py:3-5) and leaves it to the caller.
 * tgdn_glue_bwd_norm: the backward of that glue up to the convolution: from the gradients of q, k, v, k2, q2 (same layouts)
 * it writes dy bf16 (B, T, C) contiguous, the gradient tgdn_conv_bwd takes with act_channels = 3*H*128. */
int tgdn_glue_fwd(const void* x, const void* weight, const int32_t* cu_seqlens, int n_docs, int B, int T, int C,
                  int64_t stride_b, int64_t stride_t, int H, int E, float eps, void* q, void* k, void* v, float* k2, float* q2,
                  void* stream);
int tgdn_glue_bwd_norm(const void* x, const void* weight, const int32_t* cu_seqlens, int n_docs, int B, int T, int C,
                       int64_t stride_b, int64_t stride_t, int H, int E, float eps, const void* dq, const void* dk,
                       const void* dv, const float* dk2, const float* dq2, void* dy, void* stream);

/* tgdn_decode_step: one token of the recurrence on a resident state (decode).  q, k, v bf16 (B, H, 128); k2, q2, g f32
 * (B, H, E); beta f32 (B, H); state f32 (B, H, E, 128 key rows, 128 value columns), 16-byte aligned, updated in place (the
 * form tgdn_fwd_state hands out); o bf16 (B, H, 128).  Token-by-token definition of
 * cute_triadic_gdn/ops/gdn_joint.py:45-90; the reference itself has no decode entry. */
int tgdn_decode_step(const void* q, const void* k, const void* v, const float* k2, const float* q2, const float* g,
                     const float* beta, float scale, int B, int H, int E, float* state, void* o, void* stream);

/* tgdn_bwd_recurrent: the reverse chunk recurrence.  Reads the upstream gradient dO (token layout) and the forward's
 * gc, AP, Pm, U; writes dV (token layout; the gradient of v), dU (chunk layout), dr f32 [item][128/VC][64][E]
 * (VC = 32 for E <= 8, 16 for E = 12 and 16), dkg, per value block the part of dK that contracts the gradient state over the
 * value axis, sum_e G_e (r_e U)^T, as a bf16 operand image [item][128/VC][token / 8][128 key rows][token % 8] (16 KB per
 * block), and ds (chunk layout, dL/dS at the end of a chunk, same form as h) for those slices only whose chunk decay
 * exp(gc[63][e]) is at least 2^-24 (the other slices of ds are left untouched; nothing reads them).
 * Replaces: cute_triadic_gdn/kernels/sm100_joint_bwd_recurrent.py:561-609 (joint_bwd_recurrent_sm100, recurrence part)
 * and the (r U) G^T product of cute_triadic_gdn/kernels/sm100_joint_state_grads.py:373-378. */
int tgdn_bwd_recurrent(const void* q, const void* k, const void* dO, const float* k2, const float* q2, const float* beta,
                       const float* gc, const void* AP, const void* Pm, const void* U, float scale,
                       const int32_t* doc_offsets, const int32_t* chunk_map, int n_docs, int B, int T, int H, int E,
                       int NC, void* dV, void* dU, void* ds, void* dkg, float* dr, void* stream);

/* tgdn_bwd_recurrent_state: tgdn_bwd_recurrent with the gradient of the recurrent state handed in and out, for sequences
 * that are processed in segments (context parallelism): grad_state_in is dL/dS after the segment's last token (NULL: zero),
 * grad_state_out receives dL/dS before its first token (NULL: discarded); both f32 [sequence][H][E][128][128], 16-byte
 * aligned, the form of tgdn_fwd_state's states.  No counterpart in the reference. */
int tgdn_bwd_recurrent_state(const void* q, const void* k, const void* dO, const float* k2, const float* q2,
                             const float* beta, const float* gc, const void* AP, const void* Pm, const void* U, float scale,
                             const int32_t* doc_offsets, const int32_t* chunk_map, int n_docs, int B, int T, int H, int E,
                             int NC, void* dV, void* dU, void* ds, void* dkg, float* dr, const float* grad_state_in,
                             float* grad_state_out, void* stream);

/* tgdn_bwd_state_grads: per (chunk, head), the gradient terms that contract the saved forward states h (chunk start)
 * over the value axis, plus the sum of the value-block images dkg of the reverse recurrence.  Writes dkq, a bf16 image
 * [item][column / 8][128 rows][column % 8] (32 KB per item; rows 0..63: state part of dK, rows 64..127: of dQ; 16-byte
 * aligned), da, dc f32 [item][64][E] (gradients of the gate tables a = k2 exp(gc), c = scale q2 exp(gc)) and dd f32
 * [item][E], the gradient <h_e, G_e> of the chunk decay exp(gL_e), which is zero for slices whose chunk decay is below
 * 2^-24 (ds is read for the other slices only).
 * Replaces: cute_triadic_gdn/kernels/sm100_joint_state_grads.py:480-520 (joint_state_grads_sm100). */
int tgdn_bwd_state_grads(const void* q, const void* k, const void* dO, const void* dV, const void* h, const void* ds,
                         const void* dkg, const float* k2, const float* q2, const float* gc, float scale,
                         const int32_t* chunk_map, int B, int T, int H, int E, int NC, void* dkq, float* da, float* dc,
                         float* dd, void* stream);

/* tgdn_bwd_matrix: per (chunk, head), the matrix gradients through the chunk operators, the mask gradients, and the
 * final assembly: dq, dk (bf16, token layout; local part + dkq), dk2, dq2, dg, dbeta (f32, token layout).  dg is the
 * reverse chunk-local cumulative sum of the gradient of gc.
 * Replaces: cute_triadic_gdn/kernels/sm100_joint_bwd_parallel.py:442-491 (joint_bwd_parallel_sm100: matrix_kernel and
 * mask_grad_kernel) and the reverse cute_triadic_gdn/kernels/sm90_joint_scan.py:92-110 (joint_scan(reverse=True)). */
int tgdn_bwd_matrix(const void* q, const void* k, const void* dO, const void* dU, const void* W, const void* U,
                    const void* AP, const float* k2, const float* q2, const float* beta, const float* gc,
                    const void* dkq, const float* da, const float* dc, const float* dd, const float* dr, float scale,
                    const int32_t* chunk_map, int B, int T, int H, int E, int NC, void* dq, void* dk, float* dk2,
                    float* dq2, float* dg, float* dbeta, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TGDN_H_ */
