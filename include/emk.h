/*
 * emk.h — C ABI of the B200 (sm_100a) kernel backend for emmy's compiler hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream; none of them allocates,
 * frees or synchronises (except where stated), so every compute call can be captured in a CUDA graph.
 * All calls return an emk_status_t (0 = success). Paths in the comments are relative to the root of the
 * reference project (cloudrift-ai/deplodock, Python package "emmy").
 *
 * What this interface replaces: the reference lowers each fused Torch-IR op to generated CUDA text
 * (emmy/compiler/ir/kernel/render.py:407-515, emmy/compiler/pipeline/passes/lowering/cuda/010_lower_kernelop.py:63-112),
 * compiles it with nvcc at run time (emmy/compiler/backend/cuda/nvcc.py:118-177) and launches it through cupy
 * (emmy/compiler/backend/cuda/program.py:394-424, :960-1035). Here each op is one hand-written kernel behind one
 * export; the Python Backend shim (deplodock_b200/backend.py) binds them with ctypes.
 */
#ifndef EMK_H_
#define EMK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EMK_VERSION 100

/* Status codes. The Python shim maps them onto the exception types the reference raises
 * (emmy/compiler/backend/cuda/program.py:379-384 ValueError, :525 HungKernelError, :1027-1031 RuntimeError). */
typedef enum {
  EMK_OK = 0,
  EMK_ERR_SHAPE = 1,     /* a dimension is zero/negative or unsupported by the kernel          */
  EMK_ERR_DTYPE = 2,     /* unknown dtype token                                                 */
  EMK_ERR_ALIGN = 3,     /* pointer or leading dimension not aligned as the kernel requires     */
  EMK_ERR_WORKSPACE = 4, /* caller-provided workspace too small                                 */
  EMK_ERR_CUDA = 5,      /* a CUDA runtime/driver call failed; see emk_last_error               */
  EMK_ERR_TIMEOUT = 6,   /* a bounded device-side wait ran out (read back by emk_device_status) */
  EMK_ERR_ARG = 7,       /* null pointer / bad enum                                             */
  EMK_ERR_LIMIT = 8,     /* size beyond a stated fixed maximum of the entry point               */
  EMK_ERR_BOUNDS = 9     /* bounds-check build only: a token id, rotary position or cu_seqlens entry was out of
                            range (the access was clamped or dropped); read back by emk_device_status */
} emk_status_t;

/* dtype tokens: same names as the reference's graph dtypes (emmy/compiler/dtype.py:61-69). */
typedef enum { EMK_F32 = 0, EMK_BF16 = 1, EMK_F16 = 2 } emk_dtype_t;

/* Layout of the second GEMM operand.
 *   EMK_W_NK: W is [N,K] row-major, y = x·Wᵀ   — LinearOp (emmy/compiler/ir/frontend/ir.py:202-217).
 *   EMK_W_KN: W is [K,N] row-major, y = x·W    — MatmulOp (emmy/compiler/ir/frontend/ir.py:221-237). */
typedef enum { EMK_W_NK = 0, EMK_W_KN = 1 } emk_wlayout_t;

/* Fused GEMM epilogues (the reference folds these as fragment epilogues, emmy/compiler/ir/kernel/ir.py:1266-1288).
 *   EMK_EPI_NONE     y = bf16(acc)
 *   EMK_EPI_RESIDUAL y = bf16(bf16(acc) + residual)          residual is [M,N] bf16
 *   EMK_EPI_SWIGLU   W rows interleaved (gate_j, up_j); y[M,N/2] = bf16(bf16(silu(g)) * u), g,u = bf16(acc)
 *   EMK_EPI_BIAS     y = bf16(acc + bias[n])                  bias is [N] bf16 passed as `residual` */
typedef enum {
  EMK_EPI_NONE = 0,
  EMK_EPI_RESIDUAL = 1,
  EMK_EPI_SWIGLU = 2,
  EMK_EPI_BIAS = 3,
  EMK_EPI_QKNORM_ROPE = 4 /* emk_gemm_bf16_fused / emk_linear_bf16_qknorm_rope only */
} emk_epilogue_t;

typedef struct emk_handle_s* emk_handle_t;
typedef void* emk_stream_t; /* a cudaStream_t */

/* Library identity and error text. Replaces nothing in the reference (bookkeeping for the binding). */
int emk_version(void);
const char* emk_status_string(int status);
/* 1 in the bounds-check build of the library (compiled with -DEMK_BOUNDS_CHECK: indices that come from data — token
 * ids, rotary positions, cu_seqlens — are checked on the device and a violation is reported by emk_device_status as
 * EMK_ERR_BOUNDS), 0 in the normal build (same clamping, nothing recorded). The reference has no counterpart: its
 * generated kernels are checked with compute-sanitizer in its own test runs. */
int emk_bounds_check_enabled(void);

/* Per-device handle: holds the device id, SM count, the driver entry point used to encode TMA tensor maps
 * (the reference calls cuTensorMapEncodeTiled through ctypes, emmy/compiler/backend/cuda/_tma.py:91-170) and a
 * host-mapped status word that kernels write when a bounded wait runs out. */
int emk_create(int device, emk_handle_t* out);
int emk_destroy(emk_handle_t h);
const char* emk_last_error(emk_handle_t h);

/* Synchronises `stream`, then returns EMK_ERR_TIMEOUT if any kernel since the last call recorded an expired wait
 * (and clears the word), EMK_ERR_CUDA on a launch/runtime error, else EMK_OK. Same role as the reference's per-launch
 * polling watchdog `_wait_for_event` (emmy/compiler/backend/cuda/program.py:574-605). */
int emk_device_status(emk_handle_t h, emk_stream_t stream);

/* Limit, in milliseconds, of every device-side mbarrier wait (default 2000). */
int emk_set_wait_limit_ms(emk_handle_t h, int ms);

/* Programmatic dependent launch for the model-path kernels launched through this handle from now on: on (the
 * default, unless EMK_OVERLAP_LAUNCH=0) a kernel may become resident and run its set-up while the kernel before it in
 * the stream drains; off, kernels follow each other the ordinary way. Returns the previous setting (0 / 1), or a
 * negative status. Plans that chain their projections (emk_gemm_bf16_chain) measured 1.5-2 % faster with it off,
 * plans of separately launched GEMMs up to 3 % faster with it on. No counterpart in the reference. */
int emk_set_launch_overlap(emk_handle_t h, int on);

/* RMSNorm over the last axis: y = x * rsqrt(mean(x^2) + eps) * w, statistics in fp32.
 * Replaces the emitted k_rms_norm_<hash> kernel (RmsNormOp, emmy/compiler/ir/frontend/ir.py:296-312;
 * decomposition emmy/compiler/pipeline/passes/frontend/decomposition/080_rms_norm.py:17-60).
 * x,y: [rows, cols] of `dtype` (EMK_F32 or EMK_BF16), row-major; w: [cols] of `dtype`. */
int emk_rmsnorm(emk_handle_t h, const void* x, const void* w, void* y, int64_t rows, int64_t cols, float eps,
                int dtype, emk_stream_t stream);

/* Softmax over the last axis, fp32 statistics, one read and one write of the tensor.
 * Replaces the emitted k_softmax_<hash> kernel (SoftmaxOp, emmy/compiler/ir/frontend/ir.py:343-358;
 * emmy/compiler/pipeline/passes/lowering/tile/_softmax.py:123). -inf entries give 0; a fully -inf row gives NaN
 * exactly as torch does. dtype EMK_F32 or EMK_BF16. */
int emk_softmax_lastdim(emk_handle_t h, const void* x, void* y, int64_t rows, int64_t cols, int dtype,
                        emk_stream_t stream);

/* y[M,N] = x[M,K] · W (+ epilogue), bf16 operands, fp32 accumulation in tensor memory, bf16 output.
 * Replaces the emitted k_linear_<hash> kernels (LinearOp/MatmulOp above; TMA ring + mma.sync lowering in
 * emmy/compiler/pipeline/passes/lowering/kernel/_stage.py:345-450 and _atom.py:598-715).
 * K and N must be multiples of 8 (16-byte rows for TMA and vector stores); otherwise EMK_ERR_ALIGN.
 * `residual` is the [M,N] bf16 addend (EMK_EPI_RESIDUAL), the [N] bias (EMK_EPI_BIAS) or NULL.
 * For EMK_EPI_SWIGLU, y is [M,N/2]. */
int emk_linear_bf16(emk_handle_t h, const void* x, const void* w, const void* residual, void* y, int64_t M,
                    int64_t N, int64_t K, int wlayout, int epilogue, emk_stream_t stream);

/* Same contraction with e4m3 weights [N,K] and one fp32 scale per output channel:
 * y[m,n] = bf16( scale[n] * sum_k x[m,k] * float(Wq[n,k]) ). Two routes with identical arithmetic (e4m3 -> bf16 is
 * exact, the products accumulate in fp32, the scale is applied to the accumulator): with ws == NULL, or for
 * M <= 256, the weight tile is converted to bf16 inside the tensor-core main loop (no scratch, the weight crosses
 * HBM as bytes); with a workspace of emk_linear_bf16_w8_workspace_bytes(N, K) bytes (32-byte aligned) and M > 256 the
 * weight is expanded to bf16 once into ws and the bf16 tensor-core GEMM runs on it. The workspace holds nothing
 * between calls: one buffer sized for the largest layer serves a whole model. No counterpart kernel exists in the
 * reference (it has no fp8 path). */
int emk_linear_bf16_w8(emk_handle_t h, const void* x, const void* w_e4m3, const float* scale, void* y, int64_t M,
                       int64_t N, int64_t K, void* ws, int64_t ws_bytes, emk_stream_t stream);
int64_t emk_linear_bf16_w8_workspace_bytes(int64_t N, int64_t K);

/* Causal grouped-query attention, bf16, head_dim 128: O = softmax(Q·Kᵀ·scale + causal)·V with fp32 online softmax.
 * Replaces the emitted k_scaled_dot_product_attention kernel (SdpaOp, emmy/compiler/ir/frontend/ir.py:241-275;
 * decomposition .../decomposition/010_sdpa.py:52-141; flash lowering .../lowering/kernel/_twist.py:229).
 * q,o: [B,Hq,S,128]; k,v: [B,Hkv,S,128]; all contiguous bf16. Hq must be a multiple of Hkv. */
int emk_sdpa_causal_gqa_bf16(emk_handle_t h, const void* q, const void* k, const void* v, void* o, int64_t B,
                             int64_t Hq, int64_t Hkv, int64_t S, int64_t D, float scale, emk_stream_t stream);

/* The fused QKV projection with the q/k-norm + RoPE of emk_qknorm_rope applied in the GEMM epilogue (each thread of
 * the epilogue owns whole heads of its output row, so both are thread-local): y[M, (Hq+2*Hkv)*128] = x[M,K]·Wᵀ, then per
 * head RMSNorm(qw / kw, eps) and rotate-half RoPE on the query and key heads; position of row m is m % S.
 * `rope_chunk_major` is the cos/sin table re-laid for coalesced reads by the epilogue (lanes = consecutive rows):
 * bf16 [8][S][16], entry [q][s] = cos(s, 8q..8q+7) followed by sin(s, 8q..8q+7) for the first 64 elements of the
 * head (element i + 64 uses the same angle). Replaces k_linear_* plus k_mean_linear_reduce_* plus the RoPE pointwise
 * kernel of the reference's lowering of the traced layer. M must be a multiple of S. */
int emk_linear_bf16_qknorm_rope(emk_handle_t h, const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K,
                                const void* qw, const void* kw, const void* rope_chunk_major, int64_t S, int64_t Hq,
                                int64_t Hkv, float eps, emk_stream_t stream);

/* One descriptor for the tcgen05 GEMM with everything that can be fused around it; unused pointers are NULL.
 * Besides the epilogues of emk_linear_bf16 it can fold an RMSNorm across two GEMMs (the reference fuses norm -> linear
 * as k_linear_mean_reduce_* / k_mean_linear_reduce_*, emmy/compiler/pipeline/passes/loop/fusion/010_merge_loop_ops.py:131):
 * the GEMM that PRODUCES a hidden state writes partial sums of squares of every stored row to row_sumsq_out, fp32
 * [M][ceil(N/128)], one slot per 128 output columns (plain stores by the thread that owns the columns: no atomics, no
 * clearing, the same bits on every run); the GEMM that CONSUMES the hidden state reads row_sumsq_in [M][norm_dim/128]
 * and scales its accumulator rows by rsqrt(sum_s row_sumsq_in[m][s] / norm_dim + norm_eps) before its epilogue, with
 * the norm weight folded into W by the caller (W' = W * diag(w_norm)). The sum-of-squares buffers are scratch memory
 * owned by the caller. */
typedef struct {
  const void* x;        /* [M,K] bf16 */
  const void* w;        /* [N,K] (EMK_W_NK) or [K,N] (EMK_W_KN) bf16 */
  const void* residual; /* [M,N] (EMK_EPI_RESIDUAL) or [N] bias (EMK_EPI_BIAS) */
  void* y;              /* [M,N] bf16, [M,N/2] for EMK_EPI_SWIGLU */
  int64_t M, N, K;
  int wlayout, epilogue;
  const float* row_sumsq_in; /* fp32 [M][norm_dim/128] */
  int64_t norm_dim;          /* multiple of 128 */
  float norm_eps;
  float* row_sumsq_out;      /* fp32 [M][ceil(N/128)], overwritten */
  /* EMK_EPI_QKNORM_ROPE (see emk_linear_bf16_qknorm_rope) */
  const void* q_norm_weight;
  const void* k_norm_weight;
  const void* rope_chunk_major;
  int64_t seq_len, num_q_heads, num_kv_heads;
  float qk_eps;
  /* optional, EMK_EPI_QKNORM_ROPE: rotary position of every row, int32 [M] on the device (packed sequences of
   * different lengths, the "positions" of the reference's packed serving seam, emmy/serving/packed.py:6-34); seq_len
   * is then the number of positions the table holds and M need not be a multiple of it. NULL: position = m % seq_len */
  const int32_t* positions;
} emk_gemm_desc_t;
int emk_gemm_bf16_fused(emk_handle_t h, const emk_gemm_desc_t* desc, emk_stream_t stream);

/* A chain of 1 to 4 GEMMs of emk_gemm_bf16_fused, each reading as x the y of the one before it (descs[p].x ==
 * descs[p-1].y, K == its columns), run as ONE persistent launch: the 256x256 tiles of all phases form one list that
 * the CTA pairs walk together, a tile waiting only for the 256-row block of its input to be final (a device-side
 * counter per phase and row block), so the launches, pipeline fills, exposed last epilogues and partial last waves of
 * separate calls disappear — the o_proj -> gate/up -> down -> next-layer QKV sequence of a decoder layer, whose
 * counterpart in the reference is four separately launched k_linear_* kernels. Every phase: the same M, W [N,K]
 * (EMK_W_NK), N > 128, epilogue EMK_EPI_RESIDUAL, EMK_EPI_SWIGLU or EMK_EPI_QKNORM_ROPE. Besides its x, a phase may read (residual, row_sumsq_in) only what an EARLIER phase of the chain
 * wrote or what the chain does not write; y may alias the phase's own residual.
 * `workspace` (emk_gemm_bf16_chain_workspace_bytes(M) bytes, 16-byte aligned, device memory) holds the counters: it
 * must be zero before the first launch, and every launch that completes leaves it zero again (after
 * EMK_ERR_TIMEOUT the caller zeroes it). Launches that share a workspace must not overlap. */
int64_t emk_gemm_bf16_chain_workspace_bytes(int64_t M);
int emk_gemm_bf16_chain(emk_handle_t h, const emk_gemm_desc_t* descs, int n, void* workspace, int64_t workspace_bytes,
                        emk_stream_t stream);

/* y_hidden = bf16(bf16(x·Wᵀ) + residual) [M,N] and y_norm = RMSNorm(y_hidden; norm_weight, eps) [M,N], W [N,K], all
 * bf16 — the "projection + residual, then norm" step of a decoder layer in one call that allocates NOTHING: the
 * scratch between its two kernels (partial row sums of squares) is a fixed 4 MiB array inside the library, held by
 * every GPU that loads it. For callers that cannot call cudaMalloc: plugins inside a server that owns the whole device
 * heap, code under stream capture, latency-critical loops. Limit: M * ceil(N/128) <= 1048576, else EMK_ERR_LIMIT.
 * All calls on a device share the array, so calls that overlap on the GPU race; nothing in it needs zeroing. The
 * first call on a device resolves the array's address, and the first call of each shape class (M <= 128 or larger,
 * N <= 128 or larger, M and N both multiples of 256 or not: each selects its own GEMM kernel) sets that kernel's
 * attributes: make a warm-up call of the same shape class before any stream capture.
 * This entry point has no counterpart in the reference. */
int emk_linear_residual_rmsnorm_bf16_noalloc(emk_handle_t h, const void* x, const void* w, const void* residual,
                                             const void* norm_weight, void* y_hidden, void* y_norm, int64_t M,
                                             int64_t N, int64_t K, float eps, emk_stream_t stream);

/* fp32 LinearOp / MatmulOp on the tensor cores: y[M,N] (fp32) = x[M,K] · W (+ bias[N]), all fp32 in memory. Each
 * operand is split exactly into three bf16 terms, the six partial products that matter are summed by ONE bf16 tcgen05
 * GEMM with a 6K-long reduction axis and fp32 accumulation, and the accumulator is stored unrounded. The tensor core
 * accumulates with truncation, so the result sits about 1e-6 (K = 1024) to 3e-6 (K = 3072) of the output scale
 * below a correctly rounded sum — inside the 5e-5 the reference's tests allow for fp32 matmul. Replaces the reference's scalar-tier k_matmul_* / k_linear_*
 * kernels for fp32 graphs (the shapes its perf suite drives, tests/perf/cases.py:60-74). K and N multiples of 8.
 * `workspace` (device, 16-byte aligned, emk_linear_f32_tc_workspace_bytes(M, N, K) bytes = 12 (M + N) K) receives
 * the split operands and holds nothing between calls. */
int64_t emk_linear_f32_tc_workspace_bytes(int64_t M, int64_t N, int64_t K);
int emk_linear_f32_tc(emk_handle_t h, const float* x, const float* w, const float* bias, float* y, int64_t M,
                      int64_t N, int64_t K, int wlayout, void* workspace, int64_t workspace_bytes,
                      emk_stream_t stream);

/* Embedding row gather: out[t,:] = table[ids[t],:] (bf16 rows of `hidden` elements, hidden*2 a multiple of 16).
 * Replaces the GatherOp kernel of the traced trunk (emmy/compiler/trace/huggingface.py:17-186). ids are int64. */
int emk_embed_gather(emk_handle_t h, const void* table, const int64_t* ids, void* out, int64_t tokens,
                     int64_t hidden, int64_t vocab, emk_stream_t stream);
/* Same gather that also writes the sum of squares of every gathered row in the partial layout of emk_gemm_desc_t
 * (fp32 [tokens][hidden/128]: slot 0 holds the row's total, the other slots zero): the statistic the first folded
 * RMSNorm of the trunk needs. hidden must be a multiple of 128. */
int emk_embed_gather_sumsq(emk_handle_t h, const void* table, const int64_t* ids, void* out, float* row_sumsq,
                           int64_t tokens, int64_t hidden, int64_t vocab, emk_stream_t stream);

/* Same attention over token-major operands, so the fused QKV projection output can be consumed without a transpose:
 * q[(b*S+s)*ld_q + h*128 + d], likewise k, v (head index over Hkv) and o; ld_* are row pitches in elements
 * (multiples of 8). This is the layout of the traced layer before its transpose(1,2) nodes. */
int emk_sdpa_causal_gqa_bf16_tok(emk_handle_t h, const void* q, const void* k, const void* v, void* o, int64_t B,
                                 int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int64_t ld_q, int64_t ld_k,
                                 int64_t ld_v, int64_t ld_o, float scale, emk_stream_t stream);

/* Causal GQA attention over PACKED sequences of different lengths (the follow-up the reference names for its serving
 * path: cu_seqlens-aware attention tiles, one launch at mixed lengths, emmy/serving/ARCHITECTURE.md:133-137;
 * emmy/serving/packed.py:6-34 defines the packed stream). Token-major operands as in emk_sdpa_causal_gqa_bf16_tok over
 * `total_tokens` rows; sequence b occupies rows cu_seqlens[b] .. cu_seqlens[b+1]-1 (int32 [B+1] ON THE DEVICE, so the
 * call can be replayed from a CUDA graph with new lengths); no sequence may be longer than max_seqlen (<= 131072).
 * Rows not covered by any sequence are not written. `workspace` (device, 16-byte aligned, at least
 * emk_sdpa_varlen_workspace_bytes(B, total_tokens)) receives the table of 128-row query blocks a small kernel
 * builds from cu_seqlens before the attention kernel runs. */
int64_t emk_sdpa_varlen_workspace_bytes(int64_t B, int64_t total_tokens);
int emk_sdpa_causal_gqa_bf16_varlen(emk_handle_t h, const void* q, const void* k, const void* v, void* o,
                                    const int32_t* cu_seqlens, int64_t B, int64_t total_tokens, int64_t max_seqlen,
                                    int64_t Hq, int64_t Hkv, int64_t D, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                                    int64_t ld_o, float scale, void* workspace, int64_t workspace_bytes,
                                    emk_stream_t stream);

/* Pooling for packed sequences: out[b,:] = L2-normalise(RMSNorm(hidden_states[cu_seqlens[b+1]-1, :]; w, eps)), the
 * last token of every sequence (emk_pool_norm_l2 with per-sequence lengths). Empty sequences give zero rows. */
int emk_pool_norm_l2_varlen(emk_handle_t h, const void* hidden_states, const void* w, float* out,
                            const int32_t* cu_seqlens, int64_t B, int64_t hidden, float eps, emk_stream_t stream);

/* In place on the fused QKV projection output [T, (Hq+2*Hkv)*128] (T tokens, bf16, position of token t = t % S):
 * per-head RMSNorm (weights qw, kw [128] bf16, eps) on the Hq query heads and Hkv key heads, then rotate-half RoPE
 * with cos/sin tables [S,128] bf16 (the eager bf16 module multiplies by bf16 tables); the value heads are left untouched. Replaces the k_mean_linear_reduce_* q/k-norm
 * kernels and the k_cat_slice_transpose_unsqueeze_pointwise_* RoPE kernel of the reference's lowering of the traced
 * layer (traced pattern: emmy/compiler/trace/huggingface.py:17-186). */
int emk_qknorm_rope(emk_handle_t h, void* qkv, const void* qw, const void* kw, const void* cos_table,
                    const void* sin_table, int64_t tokens, int64_t S, int64_t Hq, int64_t Hkv, float eps,
                    emk_stream_t stream);

/* Same-shape pointwise ops that reach the backend as Torch-IR nodes of their own (the reference's perf suite drives
 * `torch.matmul(x,w)+r` and `F.silu(x@wg)*(x@wu)`, tests/perf/cases.py:60-74; ElementwiseOp add / multiply / silu):
 * y = a + b, a * b, silu(a), or silu(a) * b; n elements of `dtype` (EMK_F32 or EMK_BF16), no broadcasting.
 * Inside the model plan these are GEMM epilogues instead. */
typedef enum { EMK_EW_ADD = 0, EMK_EW_MUL = 1, EMK_EW_SILU = 2, EMK_EW_SILU_MUL = 3 } emk_elementwise_op_t;
int emk_elementwise(emk_handle_t h, int op, const void* a, const void* b, void* y, int64_t n, int dtype,
                    emk_stream_t stream);

/* Last-token pooling + final RMSNorm + L2 normalisation: for each sequence b, takes row (b*S + S-1) of hidden
 * [B*S, hidden] (bf16), applies RMSNorm(w, eps) rounding to bf16 as the eager module does, then divides by its L2
 * norm; writes fp32 [B, hidden]. Stands for the final norm of the trunk plus the pooler the reference leaves to
 * vLLM (emmy/serving/vllm_model.py:50-58). */
int emk_pool_norm_l2(emk_handle_t h, const void* hidden_states, const void* w, float* out, int64_t B, int64_t S,
                     int64_t hidden, float eps, emk_stream_t stream);

/* Plain CUDA-core GEMM used for operand shapes the tensor-core path rejects (K or N not a multiple of 8) and by
 * the tests as an independent check of the tcgen05 kernels. Same arguments and epilogues as emk_linear_bf16. */
int emk_linear_bf16_simt(emk_handle_t h, const void* x, const void* w, const void* residual, void* y, int64_t M,
                         int64_t N, int64_t K, int wlayout, int epilogue, emk_stream_t stream);

/* fp32 LinearOp / MatmulOp (+ optional bias [N]) on CUDA cores, for fp32 graphs (the reference's scalar tier,
 * emmy/compiler/pipeline/passes/lowering/kernel/_atom.py:572-597). Same layouts as emk_linear_bf16. */
int emk_linear_f32_simt(emk_handle_t h, const float* x, const float* w, const float* bias, float* y, int64_t M,
                        int64_t N, int64_t K, int wlayout, emk_stream_t stream);

/* The fp32 contraction behind the reference's Loop-IR kernel records (kernels/k_linear_*_reduce*.json,
 * k_add_3_reduce.json, k_add_5_reduce.json, k_mul_8_reduce.json; LoopOp bodies as in
 * emmy/compiler/ir/stmt/leaves.py:96-469): y[m,n] = e(sum_k x[m,k] * W[n,k]) with W [N,K] row-major, y and the
 * optional epilogue operand [M,N] row-major, e = identity, "+ residual[m,n]" or "* silu(gate[m,n])" (at most one of
 * residual / gate non-NULL). x[m,k] is read at (k / x_inner) * x_stride_outer + m * x_stride_m + k % x_inner:
 * (K, 0, K) for a row-major activation, (D, M*D, D) for the [heads, M, D] attention output the o_proj record reads. */
int emk_loop_linear_f32(emk_handle_t h, const float* x, const float* w, const float* residual, const float* gate,
                        float* y, int64_t M, int64_t N, int64_t K, int64_t x_inner, int64_t x_stride_outer,
                        int64_t x_stride_m, emk_stream_t stream);

/* The two halves of the reference's unfused attention lowering, as its Loop-IR records state them
 * (kernels/k_scaled_dot_product_attention_masked_reduce.json, ..._reduce_reduce.json), fp32:
 *   scores[h,i,j] = scale * sum_d rope(q)[i,h,d] * rope(k)[j,h/g,d] + (j <= i ? mask_zero : mask_fill),
 *   rope(x)[d] = x[d] * cos[pos,d] + (d < D/2 ? -x[d+D/2] : x[d-D/2]) * sin[pos,d];
 *   o[h,i,d] = sum_j softmax_j(scores[h,i,:])[j] * v[j,h/g,d].
 * q [S,H*D], k and v [S,Hkv*D], cos/sin [S,D], scores [H,S,S], o [H,S,D]; g = H/Hkv; D even and <= 128 for the
 * scores, S <= 1536 for the second half (EMK_ERR_LIMIT beyond). */
int emk_loop_rope_scores_f32(emk_handle_t h, const float* q, const float* k, const float* cos_table,
                             const float* sin_table, float* scores, int64_t S, int64_t H, int64_t Hkv, int64_t D,
                             float scale, float mask_zero, float mask_fill, emk_stream_t stream);
int emk_loop_softmax_pv_f32(emk_handle_t h, const float* scores, const float* v, float* o, int64_t S, int64_t H,
                            int64_t Hkv, int64_t D, emk_stream_t stream);

/* Generic attention on CUDA cores (one warp per query row, fp32 online softmax): any head_dim <= 256, causal or
 * full, EMK_F32 or EMK_BF16, q/o [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] contiguous. Takes the SdpaOp shapes the tensor-core
 * kernel rejects (fp32 inputs, head_dim != 128, non-causal: the reference's scalar flash tier,
 * emmy/compiler/pipeline/passes/lowering/kernel/_factor.py) and is the device-side cross-check in the tests. */
int emk_sdpa_simt(emk_handle_t h, const void* q, const void* k, const void* v, void* o, int64_t B, int64_t Hq,
                  int64_t Hkv, int64_t Sq, int64_t Skv, int64_t D, float scale, int causal, int dtype,
                  emk_stream_t stream);

/* Launches a one-warp kernel that waits on an mbarrier nobody arrives at, with the given limit; the kernel returns
 * by itself and records the expiry, so the next emk_device_status returns EMK_ERR_TIMEOUT. Exercises the same
 * bounded-wait code the GEMM and attention kernels use (the reference's counterpart is the host watchdog test
 * tests/compiler/backend/test_hung_kernel_watchdog.py, which needs a kernel that never ends; this one always ends). */
int emk_selftest_wait_expiry(emk_handle_t h, int limit_ms, emk_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* EMK_H_ */
