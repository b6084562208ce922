/*
 * kda_b200 — C ABI of the B200 (sm_100a) Kimi Delta Attention kernels.
 *
 * One shared library (libkda_b200.so), extern "C", plain pointers and sizes only.  Every entry point
 *   - returns 0 on success, a negative KDA_E* code for an argument error (nothing was launched), or a
 *     positive cudaError_t value if a CUDA call failed;
 *   - launches on the stream it is given (a cudaStream_t passed as void*), never synchronises and,
 *     unless its comment says otherwise, never allocates: all outputs and scratch memory belong to
 *     the caller;
 *   - may be called from any host thread.
 *
 * The operator these entry points implement is the one published as `chunk_kda` / `fused_recurrent_kda`
 * in flash-linear-attention 0.5.1 (third-party; the NVlabs/kda repository has no native interface for
 * this path, so the citations below name the Python operator each entry point stands behind):
 *
 *     S_t = (I - beta_t k_t k_t^T) Diag(exp g_t) S_{t-1} + beta_t k_t v_t^T,      o_t = scale * S_t^T q_t
 *
 * Tensor layout: tokens are flattened, a tensor "[tokens, H, D]" is row-major with D contiguous;
 * sequence n owns tokens cu_seqlens[n] .. cu_seqlens[n+1]-1.  States are [N, H, K, V] fp32, V contiguous.
 */
#ifndef KDA_B200_H_
#define KDA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the entry points below are the library's only exports */
#endif

#define KDA_B200_ABI_VERSION 9
#define KDA_CHUNK 64 /* tokens per chunk of the chunked kernels */

/* io_dtype of q, k, v, o and of their gradients */
#define KDA_BF16 0
#define KDA_FP32 1

/* argument errors */
#define KDA_OK 0
#define KDA_E_NULL (-1)        /* a required pointer is NULL */
#define KDA_E_SHAPE (-2)       /* unsupported or inconsistent sizes */
#define KDA_E_DTYPE (-3)       /* unsupported io_dtype for this entry point */
#define KDA_E_ALIGN (-4)       /* a pointer is not 16-byte aligned */
#define KDA_E_WORKSPACE (-5)   /* workspace too small */
#define KDA_E_DEVICE (-6)      /* the current device is not sm_100 (compute capability 10.x) */
#define KDA_E_LIMIT (-7)       /* size beyond a documented fixed maximum */
#define KDA_E_TMAP (-8)        /* the driver refused to encode a TMA tensor map for one of the tensors */

int kda_b200_abi_version(void);
/* Text for a return code of this library (negative: argument error; positive: cudaGetErrorString). */
const char* kda_b200_strerror(int code);

/* ------------------------------------------------------------------------------------------------
 * Token-recurrent forward: decode (one token per sequence) and exact fp32 scans of any length.
 * Stands behind fused_recurrent_kda (fla/ops/kda/fused_recurrent.py:329-452) and its in-place
 * lower level fused_recurrent_kda_fwd (fla/ops/kda/fused_recurrent.py:229-325).
 * The state is kept in fp32 registers, decayed, delta-updated, then read out, token by token.
 * ------------------------------------------------------------------------------------------------ */
typedef struct kda_recurrent_args {
  const void* q;               /* [tokens, H, K] io_dtype */
  const void* k;               /* [tokens, H, K] io_dtype */
  const void* v;               /* [tokens, H, V] io_dtype */
  const float* g;              /* [tokens, H, K] fp32 log-decay (<= 0) */
  const float* beta;           /* [tokens, H]    fp32 */
  const float* h0;             /* [slots, H, K, V] fp32 initial states, or NULL for zeros */
  float* ht;                   /* [slots, H, K, V] fp32 final states, or NULL; may equal h0 (in place) */
  void* o;                     /* [tokens, H, V] io_dtype */
  const int32_t* cu_seqlens;   /* device [N+1] or NULL (then every sequence has T tokens) */
  const int32_t* state_indices;/* device, or NULL.  Continuous batching (fla/ops/kda/fused_recurrent.py:122-144,195-210):
                                  sequence n starts from slot state_indices[n * state_indices_stride + a], where
                                  a = num_accepted_tokens[n] - 1 (0 without it), and the state after its token t is
                                  written to slot state_indices[n * state_indices_stride + t]; needs ht == h0.
                                  With one token per sequence and stride 1 this is "slot state_indices[n]". */
  int64_t tokens;              /* total tokens */
  int32_t N;                   /* sequences */
  int32_t T;                   /* tokens per sequence when cu_seqlens is NULL */
  int32_t H, K, V;             /* K in {32,64,128,256}; V a multiple of 32 */
  int32_t io_dtype;            /* KDA_BF16 or KDA_FP32 */
  int32_t use_qk_l2norm;       /* x * rsqrt(sum x^2 + 1e-6) on q and k rows inside the kernel */
  float scale;
  const int32_t* num_accepted_tokens; /* device [N] or NULL: speculative decoding, see state_indices */
  int32_t state_indices_stride;       /* elements between two sequences' rows of state_indices (>= 1 when it is used) */
  int32_t transpose_state;            /* nonzero: states are [slots, H, V, K] (K contiguous), fla's transpose_state_layout;
                                         K in {64, 128} */
  int32_t HQ;                         /* grouped value heads (GVA): q and k have HQ heads, [tokens, HQ, K], and value head h reads
                                         q/k head h / (H / HQ); 0 or H: no grouping.  H must be a multiple of HQ. */
  /* Gate front end inside the kernel (USE_GATE_IN_KERNEL / APPLY_BETA_SIGMOID of fla/ops/kda/fused_recurrent.py:31-225),
   * all zero / NULL: g and beta are the activated fp32 values as described above. */
  const float* A_log;                 /* [H] or NULL.  Not NULL: `g` points to the RAW gate input [tokens, H, K] of dtype
                                         g_raw_dtype and the kernel uses g = -exp(A_log[h]) softplus(x + dt_bias[h, k]), or with
                                         use_lower_bound g = lower_bound sigmoid(exp(A_log[h]) (x + dt_bias[h, k])) */
  const float* dt_bias;               /* [H * K] or NULL */
  float lower_bound;
  int32_t use_lower_bound;
  int32_t g_raw_dtype;                /* KDA_BF16 or KDA_FP32; read only with A_log */
  int32_t beta_sigmoid;               /* nonzero: `beta` points to logits [tokens, H] of dtype beta_raw_dtype */
  int32_t beta_raw_dtype;             /* KDA_BF16 or KDA_FP32; read only with beta_sigmoid */
} kda_recurrent_args;

int kda_recurrent_fwd(const kda_recurrent_args* args, void* stream);

/* Large decode batches (one token per sequence, K = V = 128, at least four (sequence, head) units per SM) run on a
 * kernel that moves the states with the bulk-copy engine and waits for them on barriers with a bounded number of
 * polls.  This call copies the device status word of that kernel to *host_out and clears it (it synchronises with
 * the device: a diagnostic, not part of the step).  0: every wait completed; bit 0: a wait gave up and the outputs
 * of that step are incomplete. */
int kda_recurrent_status(uint32_t* host_out);

/* ------------------------------------------------------------------------------------------------
 * Token-recurrent backward in fp32: the exact gradients of the recurrence kda_recurrent_fwd computes
 * (fla/ops/kda/naive.py:12-66 differentiated), for training with float32 tensors.  Stands behind chunk_kda's
 * autograd function when the inputs are float32.  Whole sequences from their initial states (no slots, no gate
 * front end: g and beta are the activated fp32 values).  Deterministic: every sum has a fixed order.
 * ------------------------------------------------------------------------------------------------ */
typedef struct kda_recurrent_bwd_args {
  const void* q;               /* [tokens, HQ, K] fp32 */
  const void* k;               /* [tokens, HQ, K] fp32 */
  const void* v;               /* [tokens, H, V]  fp32 */
  const float* g;              /* [tokens, H, K] fp32 log-decay */
  const float* beta;           /* [tokens, H]    fp32 */
  const float* h0;             /* [N, H, K, V] fp32 or NULL */
  const int32_t* cu_seqlens;   /* device [N+1] or NULL (then every sequence has T tokens) */
  const void* d_o;             /* [tokens, H, V] fp32 */
  const float* d_ht;           /* [N, H, K, V] fp32 or NULL */
  void* dq;                    /* [tokens, HQ, K] fp32 (summed over each group of value heads) */
  void* dk;                    /* [tokens, HQ, K] fp32 */
  void* dv;                    /* [tokens, H, V]  fp32 */
  float* dg;                   /* [tokens, H, K] fp32 */
  float* dbeta;                /* [tokens, H]    fp32 */
  float* dh0;                  /* [N, H, K, V] fp32 or NULL */
  void* workspace;             /* >= kda_recurrent_bwd_workspace_bytes(..), 256-byte aligned */
  size_t workspace_bytes;
  int64_t tokens;
  int32_t N;
  int32_t T;                   /* tokens per sequence when cu_seqlens is NULL */
  int32_t H, K, V;             /* K, V in {32, 64, 128} */
  int32_t HQ;                  /* grouped value heads: heads of q and k; 0 or H: no grouping */
  int32_t io_dtype;            /* KDA_FP32 */
  int32_t use_qk_l2norm;       /* the forward normalised the rows of q and k; dq, dk go through that too */
  float scale;
} kda_recurrent_bwd_args;

/* Scratch for kda_recurrent_bwd: per-value-head dq, dk, the state at the start of every 64-token chunk
 * ((tokens / 64 + N + 1) x H x K x V x 4 bytes) and the per-token states of the chunks in flight. */
size_t kda_recurrent_bwd_workspace_bytes(int64_t tokens, int32_t N, int32_t H, int32_t K, int32_t V);
int kda_recurrent_bwd(const kda_recurrent_bwd_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Chunked forward / backward (chunk = 64 tokens), bf16 tensor-core path, K = V = 128.
 * Stand behind chunk_kda and its autograd function (fla/ops/kda/chunk.py:167-411, :22-162).
 *
 * The caller passes one scratch buffer ("workspace") of at least kda_chunk_workspace_bytes(...).
 * When save_for_backward != 0 the forward leaves in it what kda_chunk_bwd needs; the caller keeps the
 * buffer alive and unmodified until the backward call and passes the same pointer.
 * cu_seqlens is always required (for equal lengths pass 0, T, 2T, ...); chunks restart at every
 * sequence start and the last chunk of a sequence may be partial.
 * ------------------------------------------------------------------------------------------------ */
typedef struct kda_chunk_args {
  /* forward inputs */
  const void* q;               /* [tokens, H, K] bf16 */
  const void* k;               /* [tokens, H, K] bf16 */
  const void* v;               /* [tokens, H, V] bf16 */
  const float* g;              /* [tokens, H, K] fp32 log-decay */
  const float* beta;           /* [tokens, H]    fp32 */
  const float* h0;             /* [N, H, K, V] fp32 or NULL */
  const int32_t* cu_seqlens;   /* device [N+1] int32 */
  /* forward outputs */
  void* o;                     /* [tokens, H, V] bf16 */
  float* ht;                   /* [N, H, K, V] fp32 or NULL */
  /* backward inputs (kda_chunk_bwd only) */
  const void* d_o;             /* [tokens, H, V] bf16 */
  const float* d_ht;           /* [N, H, K, V] fp32 or NULL */
  /* backward outputs (kda_chunk_bwd only) */
  void* dq;                    /* [tokens, H, K] bf16 */
  void* dk;                    /* [tokens, H, K] bf16 */
  void* dv;                    /* [tokens, H, V] bf16 */
  float* dg;                   /* [tokens, H, K] fp32 */
  float* dbeta;                /* [tokens, H]    fp32 */
  float* dh0;                  /* [N, H, K, V] fp32 or NULL */
  /* scratch */
  void* workspace;             /* >= kda_chunk_workspace_bytes(..), 256-byte aligned */
  size_t workspace_bytes;
  void* bwd_workspace;         /* kda_chunk_bwd only: >= kda_chunk_bwd_workspace_bytes(..), 256-byte aligned */
  size_t bwd_workspace_bytes;
  /* sizes */
  int64_t tokens;
  int32_t N, H, K, V;
  int32_t io_dtype;            /* KDA_BF16 */
  int32_t use_qk_l2norm;
  int32_t save_for_backward;   /* bit 0: keep what kda_chunk_bwd reads in the workspace; bit 1 (with use_qk_l2norm): also keep
                                  the normalised q, k there, so that the backward does not recompute them.  Pass the same
                                  value to kda_chunk_workspace_bytes, kda_chunk_fwd and kda_chunk_bwd. */
  float scale;
  int32_t HQ;                  /* grouped value heads (GVA, fla/ops/kda/chunk.py:194-196,379-386): q, k, dq, dk have HQ heads
                                  ([tokens, HQ, K]) while v, g, beta, o, the states and their gradients have H; value head h reads
                                  q/k head h / (H / HQ), and dq, dk are summed over each group.  0 or H: no grouping. */
  int32_t scan_slices;         /* CTAs per (sequence, head) of the two state scans: 0 = chosen from N * H and the SM count (a call with
                                  at most a quarter as many units as SMs cuts every unit into 4 slices of 32 value columns, which
                                  shortens the chunk-to-chunk chain); 1 or 4 force a layout.  The results do not depend on it. */
  int32_t safe_gate;           /* nonzero: the caller promises g >= -5 for every token and channel (fla's safe_gate,
                                  fla/ops/kda/chunk.py:235-246, chunk_intra.py:659-761).  The forward then computes the diagonal 16 x 16
                                  blocks of the intra-chunk products on tensor cores too, factored around each block's middle row,
                                  instead of pairwise on CUDA cores.  With gates outside the bound the result may overflow; 0 is safe
                                  for any gate. */
} kda_chunk_args;

/* Upper bound on the number of chunks: every sequence adds at most one partial chunk. */
int64_t kda_chunk_max_chunks(int64_t tokens, int32_t N);
/* Bytes of scratch kda_chunk_fwd needs (more when it must keep what the backward reads). */
size_t kda_chunk_workspace_bytes(int64_t tokens, int32_t N, int32_t H, int32_t K, int32_t V, int32_t save_for_backward);
/* Bytes of the backward's own scratch (args->bwd_workspace); it need not outlive the backward call.
 * use_qk_l2norm is a flag word here: bit 0 = q/k are L2-normalised in the kernels, bit 1 = grouped value heads
 * (HQ < H), which needs room for the per-value-head dq, dk before they are summed, bit 2 = the forward kept the
 * normalised q, k (save_for_backward bit 1), so the backward needs no room for them. */
size_t kda_chunk_bwd_workspace_bytes(int64_t tokens, int32_t N, int32_t H, int32_t K, int32_t V, int32_t use_qk_l2norm);

int kda_chunk_fwd(const kda_chunk_args* args, void* stream);
int kda_chunk_bwd(const kda_chunk_args* args, void* stream);

/* Status word of the chunked kernels (diagnostic; no counterpart in fla, whose Triton kernels have no bounded waits).
 * Every device-side wait of these kernels (on a bulk copy or on a tensor-core product) polls a bounded number of
 * times; a wait that runs out makes its CTA stop and sets a bit, and the outputs of that call are then incomplete.
 * kda_chunk_fwd clears the word at its start and also reports an inconsistent cu_seqlens there; kda_chunk_bwd adds
 * its bits to the word of the forward whose workspace it is given.  This call copies the word to *host_out; it waits
 * for the device (cudaMemcpy), so it is a check to make after a step, not part of one.  workspace == NULL reads the
 * word of the fixed array kda_chunk_fwd_noalloc uses on the current device.  0: nothing to report. */
#define KDA_STATUS_SCAN_LOAD_WAIT 0x1u      /* forward scan: operand tiles of a chunk did not arrive */
#define KDA_STATUS_SCAN_MMA_WAIT 0x2u       /* forward scan: a product did not complete */
#define KDA_STATUS_BWD_SCAN_LOAD_WAIT 0x4u  /* reverse scan: operand tiles of a chunk did not arrive */
#define KDA_STATUS_BWD_SCAN_MMA_WAIT 0x8u   /* reverse scan: a product did not complete */
#define KDA_STATUS_BWD_MAIN_LOAD_WAIT 0x20u /* per-chunk backward: a tile's loads did not arrive */
#define KDA_STATUS_BWD_MAIN_MMA_WAIT 0x40u  /* per-chunk backward: a product did not complete */
#define KDA_STATUS_BAD_CU_SEQLENS 0x100u    /* cu_seqlens is not a non-decreasing sequence within [0, tokens]: nothing was computed */
int kda_chunk_status(const void* workspace, uint32_t* host_out);

/* ------------------------------------------------------------------------------------------------
 * Forward for callers that must not allocate.  It has no counterpart in the reference or in fla: their
 * host functions always allocate their intermediates with torch.empty.
 *
 * Who needs it: a serving process that handed every free byte of HBM to its state / KV-cache pool at
 * start-up, a host thread inside a region where the framework forbids allocator calls (an allocation
 * there can fail, or can stall the whole device while the allocator synchronises), or a plain C caller
 * that owns no device allocator at all.  Such a caller still passes its inputs and outputs (q, k, v, g,
 * beta, h0, cu_seqlens, o, ht) but no workspace: args->workspace / workspace_bytes are ignored, and the
 * per-chunk tiles go to a fixed KDA_NOALLOC_SCRATCH_BYTES array that lives in the library's device
 * image (every GPU that loads the library holds those bytes until the process exits).
 *
 *  - forward only: args->save_for_backward must be 0 (KDA_E_SHAPE otherwise), since the next call
 *    overwrites the array;
 *  - the problem must fit: kda_chunk_workspace_bytes(tokens, N, H, K, V, 0) <= KDA_NOALLOC_SCRATCH_BYTES,
 *    else KDA_E_LIMIT and nothing is launched (72.5 KiB per (chunk, head): e.g. 14 chunks of 32 heads);
 *  - the first call on each device looks the array's device address up (with that device current) and
 *    caches it; make that first call during start-up, before any stream capture begins;
 *  - all calls on a device share the one array: two calls that overlap on the GPU (different streams)
 *    race, so keep them on one stream or order them with events.  Nothing in the array has to start
 *    at zero: each call rewrites the tables, the status word and every tile it reads
 *    (kda_chunk_status(NULL, ..) reads that status word).
 *  - it calls no cudaMalloc / cudaFree and no allocating library routine.
 * ------------------------------------------------------------------------------------------------ */
#define KDA_NOALLOC_SCRATCH_BYTES (32u << 20)
int kda_chunk_fwd_noalloc(const kda_chunk_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Intermediate states for inference engines: chunk_kda(..., return_intermediate_states=True)
 * (fla/ops/kda/chunk.py:95-98; fla/ops/common/chunk_delta_h.py stores the state at the START of every chunk).
 * Reads the workspace of a kda_chunk_fwd call made with save_for_backward != 0 (same tokens, N, H) and writes
 * h_out [chunks, H, K, V] bf16, chunks in sequence order (a sequence of length L owns ceil(L / 64) of them).
 * h_out must hold kda_chunk_max_chunks(tokens, N) * H * 128 * 128 elements; chunks beyond the real count stay untouched.
 * ------------------------------------------------------------------------------------------------ */
int kda_chunk_export_states(const void* workspace, size_t workspace_bytes, int64_t tokens, int32_t N, int32_t H, void* h_out,
                            void* stream);

/* ------------------------------------------------------------------------------------------------
 * Gate front end: the decay activation and the beta sigmoid that the layer applies in front of the
 * operator, and their backward.  Stands behind chunk_kda(..., use_gate_in_kernel=True, A_log=..., dt_bias=...,
 * use_beta_sigmoid_in_kernel=True, lower_bound=...) (fla/ops/kda/chunk.py:176-177,225-240,365-378) and
 * fused_kda_gate / kda_gate_fwd / kda_gate_bwd (fla/ops/kda/gate.py:26-69,88-127,144-207,210-279,321-344):
 *
 *     x = g_raw + dt_bias[h, k]
 *     g = -exp(A_log[h]) * softplus(x)                  softplus(x) = x for x > 20        (lower bound off)
 *     g = lower_bound * sigmoid(exp(A_log[h]) * x)                                       (lower bound on)
 *     beta = sigmoid(beta_raw)
 *
 * kda_gate_fwd writes g (and beta when beta_raw is given) in fp32, the types the chunked entry points read.
 * kda_gate_bwd turns dg (and dbeta) into dg_raw (dbeta_raw) in the dtype of the raw tensors and reduces
 * dA_log [H] and, when ddt_bias is non-NULL, ddt_bias [H*K] over all tokens; the reduction runs through
 * per-CTA partial sums in `workspace` and is summed in a fixed order (bit-reproducible).
 * K must be a multiple of 8; g_raw, dt_bias, g, dg, dg_raw and the workspace 16-byte aligned.
 * g_raw == NULL with beta_raw != NULL runs the beta sigmoid alone (use_beta_sigmoid_in_kernel without the gate).
 * ------------------------------------------------------------------------------------------------ */
typedef struct kda_gate_args {
  const void* g_raw;     /* [tokens, H, K] g_dtype: gate input before the activation, or NULL */
  const float* A_log;    /* [H] */
  const float* dt_bias;  /* [H*K] or NULL */
  const void* beta_raw;  /* [tokens, H] beta_dtype: beta logits, or NULL (no beta sigmoid) */
  float* g;              /* out, forward: [tokens, H, K] fp32 */
  float* beta;           /* out, forward: [tokens, H] fp32 (needed iff beta_raw) */
  const float* dg;       /* in, backward: [tokens, H, K] fp32 */
  const float* dbeta;    /* in, backward: [tokens, H] fp32 (needed iff beta_raw) */
  void* dg_raw;          /* out, backward: [tokens, H, K] g_dtype */
  void* dbeta_raw;       /* out, backward: [tokens, H] beta_dtype (needed iff beta_raw) */
  float* dA_log;         /* out, backward: [H] */
  float* ddt_bias;       /* out, backward: [H*K] or NULL */
  void* workspace;       /* backward scratch of kda_gate_bwd_workspace_bytes() bytes */
  size_t workspace_bytes;
  int64_t tokens;
  int32_t H, K;
  int32_t g_dtype, beta_dtype; /* KDA_BF16 or KDA_FP32 */
  int32_t use_lower_bound;
  float lower_bound;
} kda_gate_args;

size_t kda_gate_bwd_workspace_bytes(int64_t tokens, int32_t H, int32_t K);
int kda_gate_fwd(const kda_gate_args* args, void* stream);
int kda_gate_bwd(const kda_gate_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Strided host <-> device copy for the host-resident pipeline (no counterpart in the Python operator): `rows`
 * rows of `width_bytes`, `spitch` / `dpitch` bytes apart, on `stream` (cudaMemcpy2DAsync, direction inferred from the
 * pointers).  Lets a head range [h0, h1) of a pinned [tokens, H, D] tensor travel as one copy.
 * ------------------------------------------------------------------------------------------------ */
int kda_copy_rows_async(void* dst, size_t dpitch, const void* src, size_t spitch, size_t width_bytes, size_t rows, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Per-kernel timing for benchmarks (no counterpart in the Python operator; fla times whole calls).
 * While enabled, kda_chunk_fwd / kda_chunk_bwd / kda_gate_fwd / kda_gate_bwd record a CUDA event on the call's stream before their
 * first kernel and after each kernel.  The events live in a fixed ring owned by the library (created
 * on the first enable; this is the one place the library creates CUDA objects).  kda_b200_profile_read
 * waits for the recorded events and returns, per stage, the summed milliseconds and the launch count
 * since the last reset.  Stage ids below.  Not meant to be left on in production.
 * ------------------------------------------------------------------------------------------------ */
#define KDA_STAGE_TABLES 0
#define KDA_STAGE_PREPARE 1
#define KDA_STAGE_SCAN 2
#define KDA_STAGE_BWD_SCAN 3
#define KDA_STAGE_BWD_MAIN 4
#define KDA_STAGE_L2NORM 5
#define KDA_STAGE_GATE_FWD 6
#define KDA_STAGE_GATE_BWD 7
#define KDA_NUM_STAGES 8
int kda_b200_profile_enable(int on);
int kda_b200_profile_read(float* stage_ms, int* stage_launches, int reset);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* KDA_B200_H_ */
