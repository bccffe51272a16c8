// Memory-bound pointwise / gather kernels of the Qwen3-shaped embedding forward: embedding row gather, per-head
// q/k RMSNorm + rotary embedding applied in place on the fused QKV projection, and last-token pooling with the final
// RMSNorm and L2 normalisation.
//
// In the reference these arrive as GatherOp, pow/mean/rsqrt/multiply chains and slice/negative/cat/multiply/add
// chains of the traced HF module (emmy/compiler/trace/huggingface.py:17-186) and lower to k_mean_linear_reduce_* and
// k_cat_slice_transpose_unsqueeze_pointwise_* kernels plus layout kernels; the transposes to [B,H,S,D] disappear here
// because the attention kernel reads the token-major buffer through strided TMA tensor maps.
//
// Rounding follows the eager bf16 module step by step (normalised value -> bf16, * weight -> bf16, each RoPE product
// -> bf16, sum -> bf16) so the only differences left against the CPU oracle come from fp32 summation order.
#include "emk_common.cuh"

namespace {

using namespace emk;

// out[t,:] = table[ids[t],:]; one warp per token, 16-byte vectors.
__global__ void __launch_bounds__(256) embed_gather_kernel(const uint4* __restrict__ table,
                                                           const int64_t* __restrict__ ids, uint4* __restrict__ out,
                                                           float* __restrict__ row_sumsq, int64_t tokens,
                                                           int vec_per_row, int64_t vocab, int* status) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  grid_dependency_wait();
  grid_launch_dependents();
  if (warp >= tokens) return;
  int64_t id = ids[warp];
  if (id < 0 || id >= vocab) {
    if (lane == 0) emk_record_bounds(status, EMK_DEV_BOUNDS_TOKEN_ID);
    id = id < 0 ? 0 : vocab - 1;  // clamp instead of reading out of bounds
  }
  const uint4* src = table + id * vec_per_row;
  uint4* dst = out + warp * vec_per_row;
  float ss = 0.f;
  for (int i = lane; i < vec_per_row; i += 32) {
    const uint4 v = __ldg(src + i);
    dst[i] = v;
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      ss = fmaf(bf16_lo(u[e]), bf16_lo(u[e]), ss);
      ss = fmaf(bf16_hi(u[e]), bf16_hi(u[e]), ss);
    }
  }
  if (row_sumsq != nullptr) {
    ss = warp_sum(ss);
    const int nslots = vec_per_row / 16;  // one slot per 128 columns; slot 0 takes the total
    for (int k = lane; k < nslots; k += 32) row_sumsq[warp * nslots + k] = k == 0 ? ss : 0.f;
  }
}

// Sixteen lanes per (token, head): a head is 128 bf16, lane j of the group owns elements 8j..8j+7 (one 16-byte
// access); its rotate-half partner (element +-64) lives in lane j^8. Each thread handles two heads per pass so two
// loads are in flight. cos/sin tables are bf16 [S,128] (the eager bf16 module multiplies by bf16 tables).
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

// A CTA has 16 lanes per q/k head of a token (blockDim = 16 * (Hq + Hkv) rounded up to a warp, at most 512) and
// handles QKR_TOKENS_PER_CTA tokens: all their 16-byte loads are issued first (HBM latency is paid once, with enough
// bytes in flight per SM), the cos/sin rows come from L1/L2 when each token is processed. No division per element:
// the head comes from the thread index, the position from one 32-bit remainder per token.
constexpr int QKR_TOKENS_PER_CTA = 4;

__global__ void __launch_bounds__(512, 2) qknorm_rope_kernel(__nv_bfloat16* __restrict__ qkv,
                                                             const __nv_bfloat16* __restrict__ qw,
                                                             const __nv_bfloat16* __restrict__ kw,
                                                             const __nv_bfloat16* __restrict__ cosb,
                                                             const __nv_bfloat16* __restrict__ sinb, int tokens, int S,
                                                             int Hq, int Hkv, float eps) {
  const int sub = threadIdx.x & 15;
  const int nh = Hq + Hkv;
  const int head_raw = threadIdx.x >> 4;
  const bool live = head_raw < nh;          // padding groups of the last warp compute on head nh-1 and store nothing
  const int head = live ? head_raw : nh - 1;
  const int ld = (Hq + 2 * Hkv) * 128;
  const int t_base = blockIdx.x * QKR_TOKENS_PER_CTA;
  uint4 x[QKR_TOKENS_PER_CTA];
#pragma unroll
  for (int i = 0; i < QKR_TOKENS_PER_CTA; ++i) {
    const int t = min(t_base + i, tokens - 1);
    x[i] = *reinterpret_cast<const uint4*>(qkv + (int64_t)t * ld + head * 128 + sub * 8);
  }
  // Everything after the fp32 statistic runs on packed bf16 pairs: a bf16x2 multiply/add rounds once to bf16, which
  // is exactly what the eager bf16 module does at every step, at a quarter of the instructions of unpack-to-fp32.
  const uint4 wv = __ldg(reinterpret_cast<const uint4*>((head < Hq ? qw : kw) + sub * 8));
  const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
  for (int i = 0; i < QKR_TOKENS_PER_CTA; ++i) {
    const int t = min(t_base + i, tokens - 1);
    const int s = t % S;
    const uint4 cv = __ldg(reinterpret_cast<const uint4*>(cosb + s * 128 + sub * 8));
    const uint4 sv = __ldg(reinterpret_cast<const uint4*>(sinb + s * 128 + sub * 8));
    const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&cv);
    const __nv_bfloat162* s2 = reinterpret_cast<const __nv_bfloat162*>(&sv);
    float xf[8];
    unpack8(x[i], xf);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(xf[e], xf[e], ss);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = 1.0f / sqrtf(ss * (1.0f / 128.0f) + eps);
    uint4 ov;
    uint32_t* o32 = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 n = __hmul2_rn(w2[e], __floats2bfloat162_rn(xf[2 * e] * r, xf[2 * e + 1] * r));
      uint32_t nb = *reinterpret_cast<const uint32_t*>(&n);
      uint32_t pb = __shfl_xor_sync(0xffffffffu, nb, 8);
      if (sub < 8) pb ^= 0x80008000u;  // rotate_half: first half takes -x[i+64], second half x[i-64]
      const __nv_bfloat162 rot = *reinterpret_cast<const __nv_bfloat162*>(&pb);
      const __nv_bfloat162 out = __hadd2_rn(__hmul2_rn(n, c2[e]), __hmul2_rn(rot, s2[e]));
      o32[e] = *reinterpret_cast<const uint32_t*>(&out);
    }
    if (live && t_base + i < tokens)
      *reinterpret_cast<uint4*>(qkv + (int64_t)t * ld + head * 128 + sub * 8) = ov;
  }
}

// One CTA per sequence: RMSNorm of the last token's hidden row, rounded to bf16 like the module output, then L2
// normalisation in fp32.
// `cu_seqlens` null: sequence b is rows b*S .. b*S+S-1; else its last row is cu_seqlens[b+1]-1 (packed sequences).
__global__ void __launch_bounds__(256) pool_norm_l2_kernel(const __nv_bfloat16* __restrict__ hs,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           float* __restrict__ out, int S, int hidden, float eps,
                                                           const int* __restrict__ cu_seqlens) {
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int64_t b = blockIdx.x;
  grid_dependency_wait();
  grid_launch_dependents();
  int64_t last = b * S + (S - 1);
  if (cu_seqlens != nullptr) {
    last = (int64_t)cu_seqlens[b + 1] - 1;
    if (cu_seqlens[b + 1] <= cu_seqlens[b]) {   // empty sequence: a zero row
      for (int c = threadIdx.x; c < hidden; c += 256) out[b * hidden + c] = 0.f;
      return;
    }
  }
  const __nv_bfloat16* row = hs + last * (int64_t)hidden;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += 256) {
    const float f = __bfloat162float(row[c]);
    ss = fmaf(f, f, ss);
  }
  ss = warp_sum(ss);
  if (lane == 0) red[wid] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  __syncthreads();
  const float r = 1.0f / sqrtf(tot / (float)hidden + eps);
  float l2 = 0.f;
  for (int c = threadIdx.x; c < hidden; c += 256) {
    const float n = bf16_round(__bfloat162float(w[c]) * bf16_round(__bfloat162float(row[c]) * r));
    l2 = fmaf(n, n, l2);
  }
  l2 = warp_sum(l2);
  if (lane == 0) red[wid] = l2;
  __syncthreads();
  float tot2 = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot2 += red[i];
  const float inv = 1.0f / fmaxf(sqrtf(tot2), 1e-12f);
  for (int c = threadIdx.x; c < hidden; c += 256) {
    const float n = bf16_round(__bfloat162float(w[c]) * bf16_round(__bfloat162float(row[c]) * r));
    out[b * hidden + c] = n * inv;
  }
}

// Same-shape pointwise ops of the frontend IR (ElementwiseOp add / multiply / silu, emmy/compiler/ir/tensor/ir.py;
// silu decomposed by the reference as x * reciprocal(1 + exp(-x)), .../decomposition/020_silu.py:11-36), with
// silu(a) * b as one fused form. 16 bytes per thread and step; fp32 math; bf16 results rounded once.
template <typename T, int OP>
__device__ __forceinline__ float ew_apply(float a, float b) {
  if (OP == EMK_EW_ADD) return a + b;
  if (OP == EMK_EW_MUL) return a * b;
  const float sa = a * (1.0f / (1.0f + expf(-a)));
  return OP == EMK_EW_SILU ? sa : sa * b;
}

template <typename T, int OP>
__global__ void __launch_bounds__(256) elementwise_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                          T* __restrict__ y, int64_t n) {
  constexpr int V = 16 / (int)sizeof(T);
  const int64_t nvec = n / V;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const uint4 va = reinterpret_cast<const uint4*>(a)[i];
    uint4 vb = va;
    if (OP != EMK_EW_SILU) vb = reinterpret_cast<const uint4*>(b)[i];
    uint4 vy;
    const T* pa = reinterpret_cast<const T*>(&va);
    const T* pb = reinterpret_cast<const T*>(&vb);
    T* py = reinterpret_cast<T*>(&vy);
#pragma unroll
    for (int e = 0; e < V; ++e) py[e] = (T)ew_apply<T, OP>((float)pa[e], (float)pb[e]);
    reinterpret_cast<uint4*>(y)[i] = vy;
  }
  for (int64_t i = nvec * V + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = (T)ew_apply<T, OP>((float)a[i], OP != EMK_EW_SILU ? (float)b[i] : 0.f);
}

template <typename T>
int elementwise_launch(emk_handle_t h, int op, const void* a, const void* b, void* y, int64_t n, cudaStream_t s) {
  int64_t blocks = (n / (16 / (int64_t)sizeof(T)) + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > (int64_t)h->sm_count * 16) blocks = (int64_t)h->sm_count * 16;
  const T *pa = (const T*)a, *pb = (const T*)b;
  T* py = (T*)y;
  switch (op) {
    case EMK_EW_ADD: elementwise_kernel<T, EMK_EW_ADD><<<(unsigned)blocks, 256, 0, s>>>(pa, pb, py, n); break;
    case EMK_EW_MUL: elementwise_kernel<T, EMK_EW_MUL><<<(unsigned)blocks, 256, 0, s>>>(pa, pb, py, n); break;
    case EMK_EW_SILU: elementwise_kernel<T, EMK_EW_SILU><<<(unsigned)blocks, 256, 0, s>>>(pa, pb, py, n); break;
    case EMK_EW_SILU_MUL: elementwise_kernel<T, EMK_EW_SILU_MUL><<<(unsigned)blocks, 256, 0, s>>>(pa, pb, py, n); break;
    default: return EMK_ERR_ARG;
  }
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

}  // namespace

extern "C" int emk_embed_gather_sumsq(emk_handle_t h, const void* table, const int64_t* ids, void* out, float* row_sumsq,
                                      int64_t tokens, int64_t hidden, int64_t vocab, emk_stream_t stream);

extern "C" int emk_embed_gather(emk_handle_t h, const void* table, const int64_t* ids, void* out, int64_t tokens,
                                int64_t hidden, int64_t vocab, emk_stream_t stream) {
  return emk_embed_gather_sumsq(h, table, ids, out, nullptr, tokens, hidden, vocab, stream);
}

extern "C" int emk_embed_gather_sumsq(emk_handle_t h, const void* table, const int64_t* ids, void* out, float* row_sumsq,
                                      int64_t tokens, int64_t hidden, int64_t vocab, emk_stream_t stream) {
  if (!h || !table || !ids || !out) return EMK_ERR_ARG;
  if (tokens <= 0 || hidden <= 0 || vocab <= 0) return EMK_ERR_SHAPE;
  if ((hidden * 2) % 16 != 0 || (((uintptr_t)table | (uintptr_t)out) & 15u)) return EMK_ERR_ALIGN;
  if (row_sumsq != nullptr && hidden % 128 != 0) return EMK_ERR_SHAPE;
  const int64_t grid = (tokens + 7) / 8;
  EMK_CUDA_TRY(h, launch_after_prologue(embed_gather_kernel, (unsigned)grid, 256u, 0, (cudaStream_t)stream,
                                        h->overlap_launch != 0, (const uint4*)table, ids, (uint4*)out, row_sumsq, tokens,
                                        (int)(hidden / 8), vocab, h->status_dev));
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_qknorm_rope(emk_handle_t h, void* qkv, const void* qw, const void* kw, const void* cosb,
                               const void* sinb, int64_t tokens, int64_t S, int64_t Hq, int64_t Hkv, float eps,
                               emk_stream_t stream) {
  if (!h || !qkv || !qw || !kw || !cosb || !sinb) return EMK_ERR_ARG;
  if (tokens <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0) return EMK_ERR_SHAPE;
  if ((((uintptr_t)qkv | (uintptr_t)qw | (uintptr_t)kw | (uintptr_t)cosb | (uintptr_t)sinb) & 15u)) return EMK_ERR_ALIGN;
  if (tokens > 0x7fffffffLL / 2 || (Hq + Hkv) > 32) return EMK_ERR_SHAPE;
  const int threads = (int)(((Hq + Hkv) * 16 + 31) / 32 * 32);
  const int64_t grid = (tokens + QKR_TOKENS_PER_CTA - 1) / QKR_TOKENS_PER_CTA;
  qknorm_rope_kernel<<<(unsigned)grid, threads, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)qkv, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, (const __nv_bfloat16*)cosb,
      (const __nv_bfloat16*)sinb, (int)tokens, (int)S, (int)Hq, (int)Hkv, eps);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_pool_norm_l2(emk_handle_t h, const void* hidden_states, const void* w, float* out, int64_t B,
                                int64_t S, int64_t hidden, float eps, emk_stream_t stream) {
  if (!h || !hidden_states || !w || !out) return EMK_ERR_ARG;
  if (B <= 0 || S <= 0 || hidden <= 0) return EMK_ERR_SHAPE;
  EMK_CUDA_TRY(h, launch_after_prologue(pool_norm_l2_kernel, (unsigned)B, 256u, 0, (cudaStream_t)stream,
                                        h->overlap_launch != 0, (const __nv_bfloat16*)hidden_states,
                                        (const __nv_bfloat16*)w, out, (int)S, (int)hidden, eps,
                                        (const int*)nullptr));
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_pool_norm_l2_varlen(emk_handle_t h, const void* hidden_states, const void* w, float* out,
                                       const int32_t* cu_seqlens, int64_t B, int64_t hidden, float eps,
                                       emk_stream_t stream) {
  if (!h || !hidden_states || !w || !out || !cu_seqlens) return EMK_ERR_ARG;
  if (B <= 0 || hidden <= 0) return EMK_ERR_SHAPE;
  EMK_CUDA_TRY(h, launch_after_prologue(pool_norm_l2_kernel, (unsigned)B, 256u, 0, (cudaStream_t)stream,
                                        h->overlap_launch != 0, (const __nv_bfloat16*)hidden_states,
                                        (const __nv_bfloat16*)w, out, 0, (int)hidden, eps, (const int*)cu_seqlens));
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_elementwise(emk_handle_t h, int op, const void* a, const void* b, void* y, int64_t n, int dtype,
                               emk_stream_t stream) {
  if (!h || !a || !y || (op != EMK_EW_SILU && !b)) return EMK_ERR_ARG;
  if (n <= 0) return EMK_ERR_SHAPE;
  if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)y) & 15u) != 0) return EMK_ERR_ALIGN;
  if (dtype == EMK_F32) return elementwise_launch<float>(h, op, a, b, y, n, (cudaStream_t)stream);
  if (dtype == EMK_BF16) return elementwise_launch<__nv_bfloat16>(h, op, a, b, y, n, (cudaStream_t)stream);
  return EMK_ERR_DTYPE;
}
