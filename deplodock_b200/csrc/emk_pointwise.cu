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
                                                           int64_t tokens, int vec_per_row, int64_t vocab) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (warp >= tokens) return;
  int64_t id = ids[warp];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // clamp instead of reading out of bounds
  const uint4* src = table + id * vec_per_row;
  uint4* dst = out + warp * vec_per_row;
  for (int i = lane; i < vec_per_row; i += 32) dst[i] = __ldg(src + i);
}

// One CTA (8 warps) per token; warp w handles heads w, w+8, ... of the Hq query heads followed by the Hkv key heads.
// A head is 128 bf16: lane l owns elements 4l..4l+3, its rotate-half partner (element +-64) lives in lane l^16.
__global__ void __launch_bounds__(256) qknorm_rope_kernel(__nv_bfloat16* __restrict__ qkv,
                                                          const __nv_bfloat16* __restrict__ qw,
                                                          const __nv_bfloat16* __restrict__ kw,
                                                          const float* __restrict__ cosb, const float* __restrict__ sinb,
                                                          int64_t tokens, int S, int Hq, int Hkv, float eps) {
  const int64_t t = blockIdx.x;
  if (t >= tokens) return;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int s = (int)(t % S);
  const int ld = (Hq + 2 * Hkv) * 128;
  __nv_bfloat16* row = qkv + t * ld;
  const float4 c4 = *reinterpret_cast<const float4*>(cosb + (int64_t)s * 128 + lane * 4);
  const float4 s4 = *reinterpret_cast<const float4*>(sinb + (int64_t)s * 128 + lane * 4);
  const float cs[4] = {c4.x, c4.y, c4.z, c4.w};
  const float sn[4] = {s4.x, s4.y, s4.z, s4.w};
  const uint2 qwv = *reinterpret_cast<const uint2*>(qw + lane * 4);
  const uint2 kwv = *reinterpret_cast<const uint2*>(kw + lane * 4);
  for (int head = wid; head < Hq + Hkv; head += 8) {
    const uint2 wv = head < Hq ? qwv : kwv;
    const float wf[4] = {bf16_lo(wv.x), bf16_hi(wv.x), bf16_lo(wv.y), bf16_hi(wv.y)};
    __nv_bfloat16* p = row + head * 128 + lane * 4;
    const uint2 xv = *reinterpret_cast<const uint2*>(p);
    float xf[4] = {bf16_lo(xv.x), bf16_hi(xv.x), bf16_lo(xv.y), bf16_hi(xv.y)};
    float ss = xf[0] * xf[0] + xf[1] * xf[1] + xf[2] * xf[2] + xf[3] * xf[3];
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss * (1.0f / 128.0f) + eps);
    float nrm[4], out[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) nrm[e] = bf16_round(wf[e] * bf16_round(xf[e] * r));
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float partner = __shfl_xor_sync(0xffffffffu, nrm[e], 16);
      // rotate_half: first half takes -x[i+64], second half takes x[i-64]
      const float rot = lane < 16 ? -partner : partner;
      out[e] = bf16_round(bf16_round(nrm[e] * cs[e]) + bf16_round(rot * sn[e]));
    }
    uint2 o;
    o.x = pack_bf16x2(out[0], out[1]);
    o.y = pack_bf16x2(out[2], out[3]);
    *reinterpret_cast<uint2*>(p) = o;
  }
}

// One CTA per sequence: RMSNorm of the last token's hidden row, rounded to bf16 like the module output, then L2
// normalisation in fp32.
__global__ void __launch_bounds__(256) pool_norm_l2_kernel(const __nv_bfloat16* __restrict__ hs,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           float* __restrict__ out, int S, int hidden, float eps) {
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int64_t b = blockIdx.x;
  const __nv_bfloat16* row = hs + (b * S + (S - 1)) * (int64_t)hidden;
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

}  // namespace

extern "C" int emk_embed_gather(emk_handle_t h, const void* table, const int64_t* ids, void* out, int64_t tokens,
                                int64_t hidden, int64_t vocab, emk_stream_t stream) {
  if (!h || !table || !ids || !out) return EMK_ERR_ARG;
  if (tokens <= 0 || hidden <= 0 || vocab <= 0) return EMK_ERR_SHAPE;
  if ((hidden * 2) % 16 != 0 || (((uintptr_t)table | (uintptr_t)out) & 15u)) return EMK_ERR_ALIGN;
  const int64_t grid = (tokens + 7) / 8;
  embed_gather_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)table, ids, (uint4*)out, tokens,
                                                                       (int)(hidden / 8), vocab);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_qknorm_rope(emk_handle_t h, void* qkv, const void* qw, const void* kw, const float* cosb,
                               const float* sinb, int64_t tokens, int64_t S, int64_t Hq, int64_t Hkv, float eps,
                               emk_stream_t stream) {
  if (!h || !qkv || !qw || !kw || !cosb || !sinb) return EMK_ERR_ARG;
  if (tokens <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0) return EMK_ERR_SHAPE;
  if ((((uintptr_t)qkv | (uintptr_t)qw | (uintptr_t)kw | (uintptr_t)cosb | (uintptr_t)sinb) & 15u)) return EMK_ERR_ALIGN;
  qknorm_rope_kernel<<<(unsigned)tokens, 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)qkv, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, cosb, sinb, tokens, (int)S, (int)Hq,
      (int)Hkv, eps);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_pool_norm_l2(emk_handle_t h, const void* hidden_states, const void* w, float* out, int64_t B,
                                int64_t S, int64_t hidden, float eps, emk_stream_t stream) {
  if (!h || !hidden_states || !w || !out) return EMK_ERR_ARG;
  if (B <= 0 || S <= 0 || hidden <= 0) return EMK_ERR_SHAPE;
  pool_norm_l2_kernel<<<(unsigned)B, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)hidden_states,
                                                                    (const __nv_bfloat16*)w, out, (int)S, (int)hidden,
                                                                    eps);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}
