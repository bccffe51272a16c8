// fp32 LinearOp / MatmulOp on the tcgen05 tensor cores by operand splitting.
//
// The reference runs fp32 graphs on its scalar FMA tier (its perf suite drives the Qwen3 projections as fp32
// torch.matmul expressions, tests/perf/cases.py:60-74, and its emitted kernel for them is a CUDA-core tile loop). The
// fifth-generation tensor cores have no fp32 operand type, but an fp32 value is exactly the sum of three bf16 values
// (8 + 8 + 8 significand bits): x = x1 + x2 + x3, x1 = bf16(x), x2 = bf16(x - x1), x3 = bf16(x - x1 - x2). A product
// x·w then needs the six partial products whose weight is at least 2^-16 of the leading one,
//     (x1w3 + x2w2 + x3w1) + (x1w2 + x2w1) + x1w1,
// each exact in fp32 (two 8-bit significands), accumulated in fp32 by the tensor core; the three dropped products are
// below 2^-24 relative. That is one bf16 GEMM with a six times longer reduction axis over operands laid out as
//     A' [M, 6K] = [x1 | x2 | x3 | x1 | x2 | x1],   W' = [w3 | w2 | w1 | w2 | w1 | w1] along k
// (for W given as [K,N] the six blocks are stacked along the rows, which needs no transpose), with the fp32
// accumulator stored unrounded. The blocks run smallest terms first: the tensor core adds each instruction's partial
// sum into its accumulator with truncation, not rounding (measured: results biased towards zero by about half an ulp
// per 16-deep accumulation step), and that loss is relative to the accumulator's magnitude — with the leading block
// last, only its K/16 steps see a full-size accumulator (measured: 1.3e-6 of the output scale at K = 1024 and 3.4e-6
// at K = 3072, where leading-block-first gave 1.4e-5; a scalar fp32 FMA loop is at a few 1e-7, and the reference's
// own tests allow 5e-5 for fp32 matmul, tests/compiler/e2e/test_ops_vs_torch.py:303). Two streaming kernels write A' and W' into a caller workspace, then the
// ordinary tcgen05 GEMM of this library runs on them: 6x the bf16 flops at tensor-core rate instead of 1x at
// CUDA-core rate.
#include "emk_common.cuh"

int emk_gemm_bf16_f32out_launch(emk_handle_t h, const void* x, const void* w, const float* bias, float* y, int64_t M,
                                int64_t N, int64_t K, int wlayout, cudaStream_t s);

namespace {

using namespace emk;

// Which of the three terms goes into each of the six blocks: A' = [x1 x2 x3 x1 x2 x1], W' = [w3 w2 w1 w2 w1 w1].
// A compile-time function of the unrolled block index, so the terms stay in registers.
template <bool IS_W>
__device__ __forceinline__ constexpr int split_term(int b) {
  return IS_W ? (b == 0 ? 2 : (b == 1 || b == 3) ? 1 : 0) : ((b == 0 || b == 3 || b == 5) ? 0 : (b == 2) ? 2 : 1);
}
static_assert(split_term<false>(0) == 0 && split_term<false>(1) == 1 && split_term<false>(2) == 2 &&
              split_term<false>(3) == 0 && split_term<false>(4) == 1 && split_term<false>(5) == 0, "A' pattern");
static_assert(split_term<true>(0) == 2 && split_term<true>(1) == 1 && split_term<true>(2) == 0 &&
              split_term<true>(3) == 1 && split_term<true>(4) == 0 && split_term<true>(5) == 0, "W' pattern");

// in [R, C] fp32 row-major. STACKED = false: out [R, 6C] bf16, block b of row r at columns [bC, bC + C) (the A'
// layout, and W' for W [N,K]); STACKED = true: out [6R, C], block b at rows [bR, bR + R) (W' for W [K,N]).
// One thread converts 8 consecutive elements of a row: two 128-bit loads, six 128-bit stores.
template <bool STACKED, bool IS_W>
__global__ void __launch_bounds__(256) split6_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                                          int64_t R, int64_t C) {
  const int64_t groups_per_row = C / 8;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= R * groups_per_row) return;
  const int64_t r = gid / groups_per_row, c = (gid % groups_per_row) * 8;
  const float4 lo = __ldg(reinterpret_cast<const float4*>(in + r * C + c));
  const float4 hi = __ldg(reinterpret_cast<const float4*>(in + r * C + c + 4));
  const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  uint32_t t[3][4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float p[2][3];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const float x = v[2 * e + k];
      const float x1 = bf16_round(x);
      const float r1 = x - x1;          // exact
      const float x2 = bf16_round(r1);
      const float x3 = bf16_round(r1 - x2);
      p[k][0] = x1; p[k][1] = x2; p[k][2] = x3;
    }
#pragma unroll
    for (int term = 0; term < 3; ++term) t[term][e] = pack_bf16x2(p[0][term], p[1][term]);
  }
#pragma unroll
  for (int b = 0; b < 6; ++b) {
    const int term = split_term<IS_W>(b);
    __nv_bfloat16* dst = STACKED ? out + ((int64_t)b * R + r) * C + c : out + r * (6 * C) + (int64_t)b * C + c;
    *reinterpret_cast<uint4*>(dst) = make_uint4(t[term][0], t[term][1], t[term][2], t[term][3]);
  }
}

template <bool STACKED, bool IS_W>
cudaError_t launch_split(const float* in, void* out, int64_t R, int64_t C, cudaStream_t s) {
  const int64_t groups = R * (C / 8);
  split6_bf16_kernel<STACKED, IS_W><<<(unsigned)((groups + 255) / 256), 256, 0, s>>>(in, (__nv_bfloat16*)out, R, C);
  return cudaGetLastError();
}

int64_t round256(int64_t b) { return (b + 255) / 256 * 256; }

}  // namespace

extern "C" int64_t emk_linear_f32_tc_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return round256(M * 6 * K * 2) + round256(N * 6 * K * 2);
}

extern "C" int emk_linear_f32_tc(emk_handle_t h, const float* x, const float* w, const float* bias, float* y,
                                 int64_t M, int64_t N, int64_t K, int wlayout, void* workspace,
                                 int64_t workspace_bytes, emk_stream_t stream) {
  if (!h || !x || !w || !y || !workspace) return EMK_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || 6 * K > 0x7fffffffLL) return EMK_ERR_SHAPE;
  if (wlayout != EMK_W_NK && wlayout != EMK_W_KN) return EMK_ERR_ARG;
  if ((K % 8) != 0 || (N % 8) != 0) {
    EMK_SET_ERR(h, "emk_linear_f32_tc: K and N must be multiples of 8; got K=%lld N=%lld (use emk_linear_f32_simt)",
                (long long)K, (long long)N);
    return EMK_ERR_ALIGN;
  }
  if ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)bias | (uintptr_t)workspace) & 15u) != 0)
    return EMK_ERR_ALIGN;
  if (workspace_bytes < emk_linear_f32_tc_workspace_bytes(M, N, K)) {
    EMK_SET_ERR(h, "emk_linear_f32_tc: workspace of %lld bytes, %lld needed", (long long)workspace_bytes,
                (long long)emk_linear_f32_tc_workspace_bytes(M, N, K));
    return EMK_ERR_WORKSPACE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  uint8_t* a6 = (uint8_t*)workspace;
  uint8_t* w6 = a6 + round256(M * 6 * K * 2);
  EMK_CUDA_TRY(h, (launch_split<false, false>(x, a6, M, K, s)));
  if (wlayout == EMK_W_NK)
    EMK_CUDA_TRY(h, (launch_split<false, true>(w, w6, N, K, s)));
  else
    EMK_CUDA_TRY(h, (launch_split<true, true>(w, w6, K, N, s)));
  return emk_gemm_bf16_f32out_launch(h, a6, w6, bias, y, M, N, 6 * K, wlayout, s);
}
