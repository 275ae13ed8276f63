/*
 * sigattn_b200.h - C ABI of the B200 (sm_100a) sigmoid-attention library.
 *
 * O = sigmoid(scale * Q K^T + bias[b] (+ score_mod[b, key])) V on (B, T, H, D) tensors,
 * with optional causal masking (top-left aligned) and per-batch valid lengths, plus the
 * recomputation backward producing dQ, dK, dV.
 *
 * The reference project (MSDLLCpapers/triton-sigmoid) has no native boundary: its device
 * code is JIT-compiled from Python.  Each entry point below names the reference routine
 * whose work it takes over (paths relative to that repository).
 *
 * Conventions
 *  - Every pointer in SigAttnParams is a DEVICE pointer owned by the caller.  The attention entry
 *    points allocate no device memory (only the diagnostic self-test does, 4 bytes for the duration
 *    of its call); the library pins one 4 KB page of its own host data the first time it is used
 *    (host-visible copies of the devices' health words, see sigattn_device_status).  All launches are
 *    asynchronous on `stream`.  The first call on each device does a little set-up (symbol addresses,
 *    kernel attributes): make it outside any stream capture.
 *  - Strides are in ELEMENTS; the head dimension is contiguous (stride 1).  Base pointers
 *    must be 16-byte aligned and every stride times the element size a multiple of 16 bytes.
 *  - The tensor-core kernels are persistent (one CTA per SM draws work items from a counter).  Each
 *    launch takes the next of a ring of counter pairs built into the library's device image and leaves
 *    it at zero when it ends (the pair is chosen on the host when the call is made): 768 pairs serve
 *    ordinary launches, so up to 768 of them may be in flight per device at a time; launches recorded
 *    into a stream capture draw from 256 pairs of their own (a captured launch keeps its pair for every
 *    replay), so a graph may hold up to 256 launches of this library and two graphs that share a pair
 *    must not run at the same time.
 *  - Return value -5: a kernel of this library gave up on a bounded wait on this device earlier; nothing
 *    is launched until sigattn_device_status() has been called (which reports and clears the failure).
 *  - Return value 0 = launched; negative = rejected before any launch, with a message
 *    available from sigattn_last_error() on the calling thread.
 *  - Supported: dtype fp16 / bf16 / fp32, D in {64, 128}, 1 <= H, B, Tq, Tk (zero-sized problems
 *    return 0 without launching).
 */
#ifndef SIGATTN_B200_H_
#define SIGATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SIGATTN_ABI_VERSION 2

/* fp16 / bf16: tensor-core kernels.  fp32: exact single-precision kernels on the FMA pipe (the
 * reference accepts float32, src/triton_sigmoid/__init__.py:48, and tests it to 1e-5); they need no
 * workspace, and base pointers / strides must be multiples of 16 bytes as for the other types. */
enum SigAttnDtype { SIGATTN_FP16 = 0, SIGATTN_BF16 = 1, SIGATTN_FP32 = 2 };

enum SigAttnFlags {
  SIGATTN_CAUSAL = 1u << 0,   /* key j visible to query i only if j <= i */
  /* Accurate sigmoid in the tensor-core kernels: exponential and reciprocal both on the special-function
   * unit (relative error ~2^-22) instead of the default one-exponential form with a polynomial
   * reciprocal or a short series.  Counterpart of the reference's TRITON_SIGMOID_ACCURATE switch
   * (src/triton_sigmoid/kernel_utils.py:190-193, 236-237); slower.  Ignored for fp32 (always exact). */
  SIGATTN_ACCURATE = 1u << 1,
  /* Backward only: use the pair of streaming kernels (dK/dV with the keys stationary, then dQ with the
   * queries stationary; 7 GEMMs per tile pair like the reference's split, sigmoid_triton_dense.py:162-467)
   * instead of the default fused kernel (5 GEMMs, dQ accumulated with fp32 reductions into `workspace`).
   * The split needs no workspace, uses no atomics and is run-to-run deterministic; the fused kernel was
   * measured faster and is therefore the default. */
  SIGATTN_BWD_SPLIT = 1u << 2,
  /* The default bias of the padded and packed entry points, computed on the device: bias of batch element b
   * = -log(number of valid keys of b) (the reference's sigmoid_triton_padded.py:995-998, which does it with a
   * few small tensor kernels before the launch); `bias` and `bias_scalar` are ignored.  An element without
   * keys gets +inf, where every probability is masked anyway. */
  SIGATTN_BIAS_NEG_LOG_LK = 1u << 3,
};

enum SigAttnQuery {
  SIGATTN_Q_ABI_VERSION = 0,
  SIGATTN_Q_SM_ARCH = 1,        /* 100: the only architecture the kernels are built for */
  SIGATTN_Q_MAX_HEAD_DIM = 2,   /* 128 */
  SIGATTN_Q_PARAMS_SIZE = 3     /* sizeof(SigAttnParams), for binding sanity checks */
};

typedef struct SigAttnParams {
  uint32_t struct_bytes; /* must be sizeof(SigAttnParams) */
  int32_t dtype;         /* SigAttnDtype of q, k, v, o, dout, dq, dk, dv */
  int32_t B, H, D;
  int32_t Tq, Tk;
  uint32_t flags;        /* SigAttnFlags */
  float scale;           /* multiplies Q K^T */
  float bias_scalar;     /* used for every batch when `bias` is NULL */
  int32_t device;        /* CUDA device ordinal the pointers live on */
  int32_t reserved0;

  const void *q, *k, *v; /* (B,Tq,H,D), (B,Tk,H,D), (B,Tk,H,D) */
  void *o;               /* forward output (B,Tq,H,D); unused by backward */
  const void *dout;      /* backward only: dO (B,Tq,H,D) */
  void *dq, *dk, *dv;    /* backward outputs, shaped like q, k, v */

  /* element strides {batch, token, head} */
  int64_t q_strides[3], k_strides[3], v_strides[3], o_strides[3];
  int64_t do_strides[3], dq_strides[3], dk_strides[3], dv_strides[3];

  const int32_t *seq_lens_q; /* [B] valid query rows, or NULL = Tq; clamped to [0,Tq] */
  const int32_t *seq_lens_k; /* [B] valid key rows,   or NULL = Tk; clamped to [0,Tk] */
  const float *bias;         /* [B] fp32 additive bias, or NULL = bias_scalar */
  const float *score_mod;    /* [B,Tk] fp32 per-key additive bias (contiguous), or NULL */

  void *workspace;           /* backward: >= sigattn_bwd_workspace_bytes() (unused with SIGATTN_BWD_SPLIT); forward: unused */
  size_t workspace_bytes;
  void *stream;              /* cudaStream_t */

  /* Optional cudaEvent_t pair (NULL = off), recorded on `stream` immediately before and after
   * the launch of the main attention kernel of the call, so that a caller can time that
   * kernel alone (the backward call also zero-fills and converts the dQ accumulator). */
  void *ev_main_start;
  void *ev_main_stop;

  /* Packed (variable-length) layout, optional.  (No counterpart in the reference, whose padded entry
   * point takes (B,T,H,D) tensors plus lengths; this is the layout of the flash-attention provider of
   * its benchmark, benchmarks/benchmark_sigmoid.py:116-134.)  When both pointers are non-NULL, sequence b
   * occupies rows cu_seqlens_q[b] .. cu_seqlens_q[b+1]-1 of q, o, dout, dq, which are (total_q, H, D),
   * and rows cu_seqlens_k[b] .. cu_seqlens_k[b+1]-1 of k, v, dk, dv, which are (total_k, H, D).  Then B is
   * the number of sequences, Tq / Tk are upper bounds of the sequence lengths (longer sequences are cut
   * there), the batch strides are ignored, seq_lens_* must be NULL, score_mod is [total_k], the backward
   * workspace is sigattn_bwd_workspace_bytes(1, total_q, H, D) bytes (none for fp32), and only rows of
   * the sequences are written: rows of q-side / k-side tensors that belong to no sequence (gaps, rows behind
 * the last sequence, rows of a sequence beyond Tq / Tk) are left untouched in o, dq, dk, dv - pre-zero
 * them if they are read afterwards. */
  const int32_t *cu_seqlens_q; /* [B+1] device, non-decreasing, cu_seqlens_q[B] <= total_q */
  const int32_t *cu_seqlens_k; /* [B+1] device */
  int32_t total_q, total_k;
} SigAttnParams;

/* Forward pass.  Replaces sigmoid_attention_fwd_op + _fwd_dense_kernel
 * (src/triton_sigmoid/sigmoid_triton_dense.py:23-154, 475-562) and, when seq_lens_* are
 * given, sigmoid_attn_padded_fwd_op + _fwd_padded_kernel
 * (src/triton_sigmoid/sigmoid_triton_padded.py:24-171, 517-623).  Rows at or beyond
 * seq_lens_q[b] are written as zeros. */
int sigattn_fwd(const SigAttnParams *p);

/* Backward pass (recomputes P; nothing but q, k, v, dO is read).  Replaces
 * sigmoid_attention_bwd_op + _bwd_dense_dq_kernel + _bwd_dense_dkdv_kernel
 * (sigmoid_triton_dense.py:162-467, 565-688) and the padded counterparts
 * (sigmoid_triton_padded.py:179-509, 626-772).  dQ rows >= seq_lens_q[b] and dK/dV rows
 * >= seq_lens_k[b] are written as zeros.  The default (fused) kernel keeps its fp32 dQ accumulator in
 * `workspace`; with SIGATTN_BWD_SPLIT the two streaming kernels run instead and `workspace` is unused. */
int sigattn_bwd(const SigAttnParams *p);

/* Backward pass for callers that cannot hand the library a workspace.  (No counterpart in the
 * reference: its backward needs no scratch memory because it recomputes S in two kernels.)
 *
 * Some hosts of this library are not allowed to allocate device memory at the moment they call
 * it: a plugin running inside an inference server or a framework whose memory pool is fixed at
 * start-up, code between the begin and end of a stream capture, a real-time loop that must not
 * enter the driver's allocator.  For them this entry point keeps the fp32 dQ accumulator in a
 * fixed array inside the library's own device image (SIGATTN_STATIC_SCRATCH_ELEMS floats, 32 MiB,
 * resident on every GPU that loads the library until the process exits) and ignores
 * p->workspace / p->workspace_bytes.  Everything else - inputs, outputs, semantics, results - is
 * as for sigattn_bwd.  It calls no cudaMalloc / cudaFree or other allocating routine.
 *
 *  - Limit: B * Tq * H * D <= SIGATTN_STATIC_SCRATCH_ELEMS, otherwise the call is rejected
 *    (negative return, message from sigattn_last_error()) before anything is launched.
 *  - The first call on each device looks up the device address of the array; make that first
 *    call outside any stream capture.
 *  - All calls on one device share the one array.  Each call zero-fills the part it uses on
 *    p->stream before its kernels run, so leftovers of earlier calls never matter; but two calls
 *    whose GPU work overlaps in time (different streams, no dependency) race on it.  Serialise
 *    them on one stream or with events. */
#define SIGATTN_STATIC_SCRATCH_ELEMS (8u * 1024u * 1024u)
int sigattn_bwd_static_scratch(const SigAttnParams *p);

/* Bytes of `workspace` sigattn_bwd needs for this problem (fp32 dQ accumulator). */
size_t sigattn_bwd_workspace_bytes(int32_t B, int32_t Tq, int32_t H, int32_t D);

/* Message for the last failed call made by this host thread ("" if none). */
const char *sigattn_last_error(void);

/* Static facts about the build; `what` is a SigAttnQuery.  Unknown -> -1. */
int sigattn_query(int what);

/* Device-side health word of `device`: 0 = no kernel of this library has given up on a
 * bounded wait since the last call; otherwise a code identifying the wait (the results of
 * launches since the last call are then undefined; while the word is set further launches
 * are refused with return value -5, and kernels already queued return at once).  Reading a non-zero
 * word clears it and the kernels' work-item counters, so the library can be used again.  Synchronises
 * the device.  Negative = CUDA error (see sigattn_last_error). */
int sigattn_device_status(int device);

/* Diagnostic (no counterpart in the reference): launches a one-warp kernel that waits, with a limit
 * of `limit_ms` milliseconds (1..1000), on a barrier nothing arrives on, the way a kernel of this
 * library would wait for a lost signal.  Returns 1 when the wait gave up in an orderly way (the
 * expected outcome; the health word of the device is then set, see sigattn_device_status), 0 if
 * it did not, negative on a CUDA error.  Allocates 4 bytes of device memory for the duration of
 * the call and synchronises the device. */
int sigattn_selftest_bounded_wait(int device, int limit_ms);

#ifdef __cplusplus
}
#endif
#endif /* SIGATTN_B200_H_ */
