/*
 * pe_attn.h -- C ABI of the fused positional-encoding causal attention forward
 * for NVIDIA B200 (sm_100a).
 *
 * One call computes, for every (batch, head), the attention core that the
 * reference's attention modules run between their input projections and their
 * output projection: the positional transform of Q and K, softmax_causal(scale *
 * Q K^T [+ bias]) and the product with V.  Nothing but the output is written to
 * device memory: no transformed Q/K, no GQA copy, no score matrix.
 *
 * What each entry point replaces in the reference (paths inside that project):
 *   pe_attn_forward, variant PE_ATTN_NOPE / PE_ATTN_ROTARY
 *       src/model/attention.py:77-96   (rope.py:35-57 rotation, QKNorm, GQA repeat,
 *                                       F.scaled_dot_product_attention)
 *   pe_attn_forward, variant PE_ATTN_ALIBI
 *       src/model/alibi.py:137-160     (QKNorm, GQA repeat, scores + bias, mask,
 *                                       softmax, @ V)
 *   pe_attn_forward, variant PE_ATTN_POPE
 *       src/model/fpope_attention.py:145-177 with src/model/pope.py:124-183 or
 *       src/model/fpope.py:107-146,266-338 (softplus magnitudes, position x
 *       frequency phases, clamped key phase bias, cos/sin expansion, concat, GQA
 *       repeat, F.scaled_dot_product_attention)
 *   The reference's own native ABI for this path (extension "fpope_cuda",
 *   setup.py:36-46, Python-level fpope_attention_forward(q, k, v, freqs,
 *   phase_bias, start_pos, causal), tests/test_fpope.py:222-226) is no longer in
 *   its tree; this header is what a binding for the path links against instead.
 *
 * Conventions
 *   - All tensor pointers are DEVICE pointers owned by the caller; the library
 *     allocates no device memory.  Work is enqueued on the given stream and the
 *     call does not synchronise.
 *   - Tensors are addressed as base + b*stride[0] + h*stride[1] + s*stride[2] + d
 *     in ELEMENTS, innermost dimension contiguous.  Both [B,S,H,d] and [B,H,S,d]
 *     storage are therefore accepted without a copy.
 *   - Query head h reads key/value head h / (H / Hkv)  (repeat_interleave
 *     semantics, src/model/attention.py:87-89).
 *   - Query row r sits at position q_pos0 + r, key row s at k_pos0 + s; key s is
 *     visible to query r iff s <= r + (Sk - Sq).
 *   - Return value: 0 on success, otherwise a pe_attn_status code; a message for
 *     the calling thread's last failure is available from pe_attn_last_error().
 */
#ifndef PE_ATTN_H_
#define PE_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PE_ATTN_ABI_VERSION 4

typedef enum pe_attn_variant {
  PE_ATTN_NOPE = 0,   /* no positional transform                                            */
  PE_ATTN_ROTARY = 1, /* interleaved-pair rotation by a (cos, sin) table: RoPE, NTK, YaRN,    */
                      /* FoPE-rotary                                                        */
  PE_ATTN_ALIBI = 2,  /* logits - slope[h] * |t - s|                                        */
  PE_ATTN_POPE = 3    /* content half + softplus-magnitude / phase half: PoPE, PoPE-floor,  */
                      /* FoPE+PoPE                                                          */
} pe_attn_variant;

typedef enum pe_attn_dtype {
  PE_ATTN_BF16 = 0, /* bf16 tensors, tcgen05 tensor-core path, fp32 accumulate and softmax  */
  PE_ATTN_FP32 = 1  /* fp32 tensors, FFMA path in the reference's fp32 operation order      */
} pe_attn_dtype;

enum pe_attn_flags {
  PE_ATTN_QK_NORM = 1 << 0,           /* x / (||x||_2 + eps) on q and k rows, after the rotation   */
  PE_ATTN_FOURIER_MIX = 1 << 1,       /* POPE: freqs[] are base frequencies; mix them with         */
                                      /* fourier_coeffs[] inside the kernel (fpope.py:107-146)     */
  PE_ATTN_FOURIER_NORMALIZE = 1 << 2, /* L1-normalise each row of coefficients first               */
  PE_ATTN_FOURIER_CEILING = 1 << 3,   /* clamp effective frequencies to +-ceil_freq                */
  PE_ATTN_TABLE_GEOMETRIC = 1 << 4,   /* ROTARY: row i of rotary_table is (cos, sin)(i * angle_c),  */
                                      /* as every table of rope.py is (plain, NTK, YaRN): the       */
                                      /* decode kernel may then advance a key's rotation from tile  */
                                      /* to tile instead of reading every row                       */
  PE_ATTN_SIMT_CHECK = 1 << 8,        /* bf16 only: run the FFMA kernel on the bf16 tensors (an    */
                                      /* on-device cross-check for the tensor-core kernels)        */
  PE_ATTN_SINGLE_CTA = 1 << 9         /* bf16 only: keep the two-tile single-CTA tcgen05 kernel     */
                                      /* where the CTA-pair (d_v = 128, Sq > 256) or the four-tile */
                                      /* kernel (d_v = 64) would be chosen                         */
};

typedef enum pe_attn_status {
  PE_ATTN_OK = 0,
  PE_ATTN_ERR_NULL = 1,        /* a required pointer is null                                */
  PE_ATTN_ERR_VARIANT = 2,     /* unknown variant / dtype / struct size                     */
  PE_ATTN_ERR_SHAPE = 3,       /* unsupported or inconsistent dimensions                    */
  PE_ATTN_ERR_ALIGNMENT = 4,   /* base pointer or stride not 16-byte aligned                */
  PE_ATTN_ERR_LAUNCH = 5,      /* CUDA reported an error at launch or descriptor encoding   */
  PE_ATTN_ERR_DEVICE = 6,      /* no sm_100 device current                                  */
  PE_ATTN_ERR_TOO_LARGE = 7    /* a size exceeds what an entry point supports               */
} pe_attn_status;

typedef struct pe_attn_args {
  uint32_t struct_size; /* sizeof(pe_attn_args), checked                                    */
  int32_t variant;      /* pe_attn_variant                                                  */
  int32_t dtype;        /* pe_attn_dtype                                                    */
  uint32_t flags;       /* pe_attn_flags                                                    */

  int32_t B, H, Hkv;    /* batch, query heads, key/value heads (H % Hkv == 0)               */
  int32_t Sq, Sk;       /* query rows, key rows (Sk >= Sq)                                  */
  int32_t d_c;          /* content (or plain) head dim of q and k; 0 = position-only PoPE   */
  int32_t d_r;          /* PoPE position dim BEFORE the cos/sin expansion; 0 otherwise      */
  int32_t d_v;          /* value / output head dim                                          */
  int32_t q_pos0;       /* position of query row 0 (the reference's start_pos)              */
  int32_t k_pos0;       /* position of key row 0                                            */

  float scale;          /* logit scale, e.g. (d_c + 2 d_r)^-1/2                             */
  float qk_norm_eps;    /* QKNorm epsilon (reference: 1e-6)                                 */
  float mscale;         /* ROTARY: q and k are multiplied by this after rotation (YaRN); 1  */

  const void* q;        /* [B,H,Sq,d_c]  content / plain queries (null if d_c == 0)         */
  const void* k;        /* [B,Hkv,Sk,d_c]                                                   */
  const void* v;        /* [B,Hkv,Sk,d_v]                                                   */
  void* out;            /* [B,H,Sq,d_v]                                                     */
  const void* q_r;      /* POPE: [B,H,Sq,d_r] position queries, pre-softplus                */
  const void* k_r;      /* POPE: [B,Hkv,Sk,d_r]                                             */
  int64_t q_stride[3], k_stride[3], v_stride[3], out_stride[3], qr_stride[3], kr_stride[3];

  const float* rotary_table;  /* ROTARY: [table_rows, d_c/2, 2] fp32 (cos, sin); row i is     */
  int32_t table_pos0;         /* position table_pos0 + i                                     */
  int32_t table_rows;
  const float* alibi_slopes;  /* ALIBI: [H] fp32                                             */
  const float* freqs;         /* POPE: [d_r] fp32 effective (or, with FOURIER_MIX, base)     */
  const float* delta;         /* POPE: [d_r] fp32 raw key phase bias (clamped to [-2pi, 0]   */
                              /* inside, as the reference does at use); null = 0             */
  const float* fourier_coeffs;/* POPE + FOURIER_MIX: [d_r, n_fourier] fp32                   */
  int32_t n_fourier;
  float floor_freq;           /* FOURIER_MIX: |eff| < floor_freq -> 0  (2 pi / T)            */
  float ceil_freq;            /* FOURIER_CEILING: clamp bound (2 pi)                         */

  int32_t* device_status;     /* optional [1] int32 on the device: the tensor-core kernel     */
                              /* ORs a non-zero code into it if one of its bounded waits      */
                              /* expires (the output is then invalid); never written on      */
                              /* success.  May be null.                                      */
  float* lse;                 /* optional [B, H, Sq] fp32, contiguous: natural-log logsumexp  */
                              /* of each query row's scaled, biased, masked logits -- what    */
                              /* pe_attn_backward needs to rebuild the probabilities.  May    */
                              /* be null.                                                    */
  void* workspace;            /* optional device scratch for pe_attn_forward (16-byte         */
  uint64_t workspace_bytes;   /* aligned), see pe_attn_forward_workspace_bytes; may be null   */
} pe_attn_args;

/* ABI version of the loaded library (PE_ATTN_ABI_VERSION at build time). */
int pe_attn_version(void);

/* Validate ``args`` and enqueue the forward on ``stream`` (a cudaStream_t; null = default
 * stream) of the current device.  Replaces the reference code listed at the top. */
int pe_attn_forward(const pe_attn_args* args, void* stream);

/* Scratch that pe_attn_forward can use for ``args`` (0 for most calls).  A causal launch with
 * few (batch, head) problems cannot fill the GPU evenly: its longest query blocks decide the run
 * time.  Given this much workspace the CTA-pair kernel cuts those blocks in two along the keys
 * and merges the halves (bit-level results differ from the unsplit kernel by fp32 rounding of
 * the merge; both are within the tolerances).  Without it the call runs unsplit.  An fp32 call
 * with a positional transform and at least 128 query rows uses its workspace for the transformed
 * keys ([B][Hkv][Sk][d_qk] fp32, built once by a kernel in front of the attention kernel instead
 * of once per query block; identical results).  The workspace is only used during the call's
 * own kernels (stream-ordered). */
size_t pe_attn_forward_workspace_bytes(const pe_attn_args* args);

/* Validate only: same checks and return codes as pe_attn_forward, touches no GPU. */
int pe_attn_validate(const pe_attn_args* args);

/* Name of the kernel family pe_attn_forward would pick for ``args``: "tcgen05" (single CTA),
 * "tcgen05-pair" (two CTAs share every K/V tile through cta_group::2 MMAs) or "ffma";
 * null if ``args`` does not validate. */
const char* pe_attn_kernel_name(const pe_attn_args* args);

/* Message for the calling thread's most recent non-zero return ("" if none). */
const char* pe_attn_last_error(void);

/* Static name of a status code. */
const char* pe_attn_status_string(int status);

/* Algorithmic FLOPs of one call: B * H * (causal pairs) * 2 * (d_c + 2 d_r + d_v). */
double pe_attn_flops(const pe_attn_args* args);

/* Decode step against a cached K/V (the per-token call of the reference's cache modules,
 * src/model/fpope_attention.py:180-271: new rows appended to the cache, the new queries attend
 * to all of it).  Same arguments, variants and result as pe_attn_forward (bf16 only), for calls
 * with at most 8 query rows per K/V head (H / Hkv * Sq <= 8): the keys of every (batch,
 * K/V head) are cut into splits that separate CTAs stream from memory once, and a second
 * kernel merges the splits' partial outputs by their logsumexp.  ``workspace`` is device
 * memory of at least pe_attn_decode_workspace_bytes(args) bytes (16-byte aligned) that the
 * call may overwrite; it must stay untouched until the stream has run the call.
 * pe_attn_decode_workspace_bytes returns 0 when ``args`` does not validate or is not such a
 * call (pe_attn_last_error says why); pe_attn_decode then returns the error code. */
size_t pe_attn_decode_workspace_bytes(const pe_attn_args* args);
int pe_attn_decode(const pe_attn_args* args, void* workspace, size_t workspace_bytes, void* stream);

/* Failure-reporting self-test (no counterpart in the reference).  Launches one warp that
 * waits, with the same bounded wait the attention kernels use, on a barrier nothing ever
 * signals.  After ``limit_cycles`` SM clocks the wait gives up, the kernel ORs
 * PE_ATTN_SELFTEST_WAIT_EXPIRED into *device_status and returns normally; the context stays
 * usable.  Shows on a live GPU that an expired wait is reported, not hung on. */
#define PE_ATTN_SELFTEST_WAIT_EXPIRED 0x40000000
int pe_attn_selftest_wait_expiry(int32_t* device_status, int64_t limit_cycles, void* stream);

/* ---- attention backward (the gradient autograd derives from the SDPA call) ------------------
 *
 * Gradients of  out = softmax_causal(scale * Q K^T + bias) V  with respect to Q, K and V, for
 * bf16 or fp32 operands that already carry their positional transform: the quantity PyTorch's
 * autograd produces for F.scaled_dot_product_attention at src/model/attention.py:91-96,
 * src/model/fpope_attention.py:171-177 and for the explicit softmax of
 * src/model/alibi.py:145-160 (bias = -slope_h * (t - s) when alibi_slopes is given).  The
 * reference's deleted extension exposed the same step as the backward of
 * fpope_attention_forward (debug_backward.py:108-124; gradient tolerances 1e-2 there).
 * The backward of the positional transform itself is left to the caller (the Python host
 * differentiates its own restatement of the transform).
 *
 * q [B,H,Sq,d_qk], k [B,Hkv,Sk,d_qk], v [B,Hkv,Sk,d_v], out / dout [B,H,Sq,d_v]: ``dtype``,
 * element strides (batch, head, seq), 16-byte aligned, strides multiples of 8.  lse: the forward's
 * logsumexp output [B,H,Sq] fp32.  dq_accum: fp32 [B,Sq,H,d_qk] contiguous -- cleared and
 * then accumulated into by the call (TMA reductions in an order that is not fixed: bitwise
 * results vary between runs);
 * dk / dv: outputs of type ``dtype`` shaped and strided like k / v (each written exactly once);
 * dvec: fp32 [B,H,Sq] workspace.  bf16 with (d_qk, d_v) in {(64,64), (128,64), (128,128)} runs on
 * the tensor cores; every other multiple of 8 up to (256, 128), and every fp32 call, on the CUDA
 * cores (fixed summation order).  Causal rule as in the forward: key s is visible to query row
 * r iff s <= r + (Sk - Sq). */
typedef struct pe_attn_bwd_args {
  uint32_t struct_size;       /* sizeof(pe_attn_bwd_args), checked                            */
  int32_t B, H, Hkv, Sq, Sk, d_qk, d_v;
  float scale;
  const void *q, *k, *v, *out, *dout;
  int64_t q_stride[3], k_stride[3], v_stride[3], out_stride[3], dout_stride[3];
  const float* lse;
  const float* alibi_slopes;  /* [H] fp32 or null                                            */
  float* dq_accum;
  void* dk;
  void* dv;
  int64_t dk_stride[3], dv_stride[3];
  float* dvec;
  int32_t* device_status;     /* as in pe_attn_args; may be null                             */
  int32_t dtype;              /* pe_attn_dtype of q, k, v, out, dout, dk, dv                  */
} pe_attn_bwd_args;

int pe_attn_backward(const pe_attn_bwd_args* args, void* stream);

/* The PoPE-family transform as stand-alone steps of the training path (the backward kernel
 * reads transformed operands from memory; the forward never writes them).
 *
 * pe_pope_expand restates PoPEEmbedding / FoPEPoPEEmbedding .forward_query / .forward_key
 * (src/model/pope.py:124-183, src/model/fpope.py:266-338) with the content half prepended as
 * src/model/fpope_attention.py:166-167 does:
 *   out[b,s,h,:] = [ x_c | softplus(x_r) cos(phi) | softplus(x_r) sin(phi) ],
 *   phi = fl(fl((pos0 + s) * omega) + clamp(delta, -2 pi, 0))      (delta null: queries).
 * pe_pope_expand_backward is what autograd derives from it: given grad = d/d out (bf16 or
 * fp32, PE_ATTN_BF16 / PE_ATTN_FP32) it writes d x_c and d x_r (bf16) and ACCUMULATES
 * d_omega[c] += sum pos * d phi and d_delta[c] += sum d phi where -2 pi <= delta[c] <= 0 (fp64
 * [d_r]; d_delta is the gradient of the RAW bias: the clamp passes it on inside the interval
 * only; it may be null; zero both before the first call).
 * All tensors [B,S,H,*] by element strides (batch, head, seq), 16-byte aligned, strides
 * multiples of 8; d_r 32 or 64, d_c a multiple of 8 (0 = position-only).  omega: the
 * effective frequencies [d_r] fp32. */
int pe_pope_expand(const void* x_c, const int64_t* xc_stride, const void* x_r, const int64_t* xr_stride, void* out,
                   const int64_t* out_stride, int B, int S, int H, int d_c, int d_r, int pos0, const float* omega,
                   const float* delta, void* stream);
int pe_pope_expand_backward(const void* grad, int grad_dtype, const int64_t* grad_stride, const void* x_r,
                            const int64_t* xr_stride, void* dx_c, const int64_t* dxc_stride, void* dx_r,
                            const int64_t* dxr_stride, int B, int S, int H, int d_c, int d_r, int pos0,
                            const float* omega, const float* delta, double* d_omega, double* d_delta, void* stream);

/* FoPE's collapse of base frequencies and Fourier coefficients into one effective frequency
 * per position dimension (FoPEPoPEEmbedding._compute_effective_freqs, src/model/fpope.py:107-146)
 * and its gradient: omega[c] = base[c] * sum_j a^[c,j] j + base[c], a^ = a / (sum_j |a| + 1e-8)
 * with PE_ATTN_FOURIER_NORMALIZE, |omega| < floor_freq -> 0, clamp to +-ceil_freq with
 * PE_ATTN_FOURIER_CEILING.  The backward takes d_omega (fp64 [d_r], as pe_pope_expand_backward
 * accumulates it) and writes d_coeffs [d_r, n_fourier] and, if not null, d_base [d_r]. */
int pe_fope_effective_freqs(const float* base, const float* coeffs, int d_r, int n_fourier, unsigned flags,
                            float floor_freq, float ceil_freq, float* omega, void* stream);
int pe_fope_effective_freqs_backward(const float* base, const float* coeffs, int d_r, int n_fourier, unsigned flags,
                                     float floor_freq, float ceil_freq, const double* d_omega, float* d_coeffs,
                                     float* d_base, void* stream);

/* The same two steps for the rotary family and QKNorm (src/model/rope.py:35-57 and
 * rope.py:216-217 for YaRN's mscale, src/model/normalization.py:44-56):
 *   out = normalise(mscale * rotate(x)),  rotate by rows table_row0 .. of ``table``
 *   ([table_rows, D/2, 2] fp32 (cos, sin); null = no rotation), normalise = x / (|x|_2 + eps)
 *   when qk_norm != 0; rounding to bf16 after each step, as the forward kernel does.
 * The backward takes grad = d/d out (bf16 or fp32) and writes d x (bf16); the roundings are
 * treated as the identity.  x, out, grad, dx: [B,S,H,D] by element strides (batch, head, seq),
 * D 64 or 128. */
int pe_rotary_norm_expand(const void* x, const int64_t* x_stride, void* out, const int64_t* out_stride, int B, int S,
                          int H, int D, const float* table, int table_row0, int table_rows, float mscale, int qk_norm,
                          float eps, void* stream);
int pe_rotary_norm_expand_backward(const void* grad, int grad_dtype, const int64_t* grad_stride, const void* x,
                                   const int64_t* x_stride, void* dx, const int64_t* dx_stride, int B, int S, int H,
                                   int D, const float* table, int table_row0, int table_rows, float mscale,
                                   int qk_norm, float eps, void* stream);

/* ---- perplexity evaluation: next-token cross-entropy as loss sums ------------------------
 *
 * Replaces, for the evaluation path, F.cross_entropy on the shifted logits
 * (src/model/transformer.py:362-370) together with the per-window weighting
 * total_loss += loss * n_tokens of scripts/evaluate_ppl_degradation.py:96-108: instead of a
 * mean per call it accumulates the two sums a sharded evaluation reduces.
 *
 *   out[0] += sum over rows with target != ignore_index of
 *             logsumexp(logits[r, 0:vocab]) - logits[r, target[r]]
 *   out[1] += number of such rows
 *
 * Like F.cross_entropy, a row whose logits hold NaN or +inf makes the sum non-finite (it is
 * not dropped) and -inf logits count as probability zero.  A target outside [0, vocab) that
 * is not ignore_index is the caller's error: its row is scored as NaN, so the sums come out
 * NaN (torch raises a device assert there).
 *
 * logits: device [n_rows, vocab] of ``dtype`` (pe_attn_dtype), rows ``row_stride`` elements
 * apart (16-byte aligned rows are read fastest; any element-aligned pitch works).  targets:
 * device int64 [n_rows].  out: device double[2], accumulated (zero it before the first chunk).  scratch: device buffer of
 * pe_ce_scratch_bytes(n_rows) bytes, 256-byte aligned, whose first 256 bytes are zero on
 * entry (the kernel leaves them zero, so one cudaMemset after allocation is enough).
 * Calls that share a scratch buffer must be ordered on one stream. */
size_t pe_ce_scratch_bytes(int n_rows);
int pe_ce_loss_sums(const void* logits, int dtype, int64_t row_stride, const int64_t* targets, int n_rows, int vocab,
                    int ignore_index, void* scratch, double* out, void* stream);

/* ---- the memory-bound neighbours of attention on the evaluation path -------------------------
 *
 * pe_rmsnorm_forward replaces RMSNorm.forward (src/model/normalization.py:22-27) followed by
 * the cast the next linear layer's autocast applies: y = cast(cast(x * rsqrt(mean(x^2) + eps))
 * * weight), one read and one write of the activation.  x, y: device [rows, dim] of ``dtype``
 * (bf16: 16-byte aligned rows; fp32: 32-byte), rows ``x_stride`` / ``y_stride`` elements
 * apart, dim a multiple of 8; weight: device fp32 [dim].
 *
 * pe_swiglu_forward replaces SwiGLU.forward (src/model/ffn.py:8-27, called at ffn.py:68):
 * y = cast(cast(silu(gate)) * up) over ``n`` contiguous elements (a multiple of 8). */
int pe_rmsnorm_forward(const void* x, const float* weight, void* y, int dtype, int rows, int dim, int64_t x_stride,
                       int64_t y_stride, float eps, void* stream);
int pe_swiglu_forward(const void* gate, const void* up, void* y, int dtype, int64_t n, void* stream);

/* ---- the two GEMMs of the evaluation path whose results need not exist in HBM ------------------
 *
 * One persistent tcgen05 kernel (CTA pairs, 256 x 256 accumulator tiles in TMEM, TMA-staged
 * operands) with the consumer of the product in its epilogue.  bf16 operands with K contiguous,
 * 16-byte aligned bases, row strides that are multiples of 8 elements, K >= 64 and a multiple
 * of 8; fp32 accumulation.
 * ``device_status`` as in pe_attn_args (may be null).
 *
 * pe_lm_head_ce_loss_sums replaces the language-model head followed by the cross-entropy
 * (src/model/transformer.py:358-371, the evaluation's F.cross_entropy on the head's output):
 *   logits = round_bf16(hidden [n_rows, hidden_dim] * weight [vocab, hidden_dim]^T)
 *   out[0] += sum over scored rows of (logsumexp(logits[r, :]) - logits[r, targets[r]])
 *   out[1] += number of scored rows (targets[r] != ignore_index)
 * with the semantics of pe_ce_loss_sums for non-finite logits and out-of-range targets; the
 * logits are never written.  ``workspace``: 256-byte aligned device buffer of
 * pe_lm_head_ce_workspace_bytes(n_rows, vocab) bytes (per-tile partial results: 8 bytes per row
 * and 256 vocabulary entries), used only by the call's own kernels; calls that share one must be
 * ordered on one stream.
 *
 * pe_swiglu_gemm replaces the feed-forward's two input projections and SwiGLU
 * (src/model/ffn.py:30-68): y [n_rows, ffn_dim] = cast(cast(silu(cast(x w_gate^T))) * cast(x w_up^T)),
 * the roundings of the two bf16 projections followed by pe_swiglu_forward.  w_gate, w_up:
 * [ffn_dim, hidden_dim] with one common row stride.
 *
 * pe_gemm_nt: c [m, n] = cast(a [m, k] * b [n, k]^T), the same kernel with a plain store; with
 * ``residual`` [m, n] (may be null; may be ``c`` itself) c = cast(cast(a b^T) + residual), the
 * output projection (wo, w2) together with the block's residual add
 * (src/model/transformer.py:176-177). */
size_t pe_lm_head_ce_workspace_bytes(int n_rows, int vocab);
int pe_lm_head_ce_loss_sums(const void* hidden, int64_t hidden_stride, const void* weight, int64_t weight_stride,
                            const int64_t* targets, int n_rows, int hidden_dim, int vocab, int ignore_index,
                            void* workspace, size_t workspace_bytes, double* out, int32_t* device_status, void* stream);
int pe_swiglu_gemm(const void* x, int64_t x_stride, const void* w_gate, const void* w_up, int64_t w_stride, void* y,
                   int64_t y_stride, int n_rows, int hidden_dim, int ffn_dim, int32_t* device_status, void* stream);
int pe_gemm_nt(const void* a, int64_t a_stride, const void* b, int64_t b_stride, void* c, int64_t c_stride,
               const void* residual, int64_t residual_stride, int m, int n, int k, int32_t* device_status, void* stream);

/* Same computation as pe_ce_loss_sums for callers that must not allocate.  No counterpart
 * in the reference.
 *
 * Who needs it: an evaluation loop embedded in a process that handed all of its device
 * memory to a pool at start-up, or one that runs where cudaMalloc is off limits because it
 * synchronises the whole device (a serving thread sharing the GPU with latency-bound work).
 * Such a caller has nowhere to get the scratch buffer from, so this entry point keeps one
 * inside the library: a fixed device array of 256 + 4 * pe_ce_static_max_rows() bytes
 * (64.25 KiB) that every GPU loading the library carries until the process ends.  The call
 * itself allocates and frees nothing, on the device or through any library.
 *
 *   - n_rows above pe_ce_static_max_rows() (16384) is refused with PE_ATTN_ERR_TOO_LARGE:
 *     feed the logits in smaller chunks, ``out`` accumulates across calls.
 *   - The first call on each device looks up the array's device address (a one-time host
 *     step); make that first call during set-up, before any stream capture starts.
 *   - All calls on a device share the one array.  Each call clears the part that has to
 *     start at zero and the rest is overwritten before it is read, so consecutive calls
 *     on one stream are safe; calls that can overlap on the GPU (different streams, or
 *     several host threads) would race on it and must be serialised by the caller.
 *     A call that is refused (bad arguments, too many rows) touches nothing of the array.
 *   - logits / targets / out as for pe_ce_loss_sums; the caller still owns all three. */
int pe_ce_static_max_rows(void);
int pe_ce_loss_sums_static(const void* logits, int dtype, int64_t row_stride, const int64_t* targets, int n_rows,
                           int vocab, int ignore_index, double* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PE_ATTN_H_ */
