// CUDA-core GEMM with the same arguments and epilogues as the tensor-core path. Two uses: operand shapes the TMA
// path cannot take (K or N not a multiple of 8), and an independent device-side check of the tcgen05 kernels in the
// tests (the reference keeps the same triangulation idea: staged paths are asserted equal to the direct path,
// tests/compiler/e2e/test_matmul_coverage.py:300,938-1068).
#include "emk_common.cuh"

#include <math_constants.h>

namespace {

using namespace emk;

__device__ __forceinline__ float simt_dot(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                          int64_t m, int64_t n, int64_t N, int64_t K, int wl) {
  float acc = 0.f;
  const __nv_bfloat16* xr = x + m * K;
  if (wl == EMK_W_NK) {
    const __nv_bfloat16* wr = w + n * K;
    for (int64_t k = 0; k < K; ++k) acc = fmaf(__bfloat162float(xr[k]), __bfloat162float(wr[k]), acc);
  } else {
    for (int64_t k = 0; k < K; ++k) acc = fmaf(__bfloat162float(xr[k]), __bfloat162float(w[k * N + n]), acc);
  }
  return acc;
}

__global__ void __launch_bounds__(256) gemm_simt_kernel(const __nv_bfloat16* __restrict__ x,
                                                        const __nv_bfloat16* __restrict__ w,
                                                        const __nv_bfloat16* __restrict__ residual,
                                                        __nv_bfloat16* __restrict__ y, int64_t M, int64_t N,
                                                        int64_t K, int wl, int epi) {
  const int64_t ncols_out = (epi == EMK_EPI_SWIGLU) ? N / 2 : N;
  const int64_t total = M * ncols_out;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / ncols_out, j = i % ncols_out;
    float out;
    if (epi == EMK_EPI_SWIGLU) {
      const float gate = bf16_round(simt_dot(x, w, m, 2 * j, N, K, wl));
      const float up = bf16_round(simt_dot(x, w, m, 2 * j + 1, N, K, wl));
      out = bf16_round(gate / (1.0f + __expf(-gate))) * up;
    } else {
      const float acc = simt_dot(x, w, m, j, N, K, wl);
      if (epi == EMK_EPI_RESIDUAL) out = bf16_round(acc) + __bfloat162float(residual[m * N + j]);
      else if (epi == EMK_EPI_BIAS) out = acc + __bfloat162float(residual[j]);
      else out = acc;
    }
    y[i] = __float2bfloat16_rn(out);
  }
}


// Generic attention on CUDA cores: one warp per (batch, query head, query row), online softmax in fp32, any head_dim
// up to 256, causal or full, fp32 or bf16 operands. Covers SdpaOp shapes the tensor-core kernel does not take and
// serves the tests as an independent device-side check of it.
template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void st_from_float(T* p, float v);
template <>
__device__ __forceinline__ void st_from_float<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void st_from_float<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) sdpa_simt_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                        const T* __restrict__ v, T* __restrict__ o, int64_t B,
                                                        int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv, int D,
                                                        float scale, int causal) {
  const int lane = threadIdx.x & 31;
  const int64_t row_id = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row_id >= B * Hq * Sq) return;
  const int64_t i = row_id % Sq;
  const int64_t hq = (row_id / Sq) % Hq;
  const int64_t b = row_id / (Sq * Hq);
  const int64_t hkv = hq / (Hq / Hkv);
  const T* qr = q + row_id * D;
  const T* kb = k + (b * Hkv + hkv) * Skv * D;
  const T* vb = v + (b * Hkv + hkv) * Skv * D;
  float qv[8], acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int d = lane + 32 * e;
    qv[e] = d < D ? ld_as_float<T>(qr + d) : 0.f;
    acc[e] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  // causal: torch aligns the mask to the top-left corner (key j visible to query i iff j <= i)
  const int64_t jend = causal ? (i + 1 < Skv ? i + 1 : Skv) : Skv;
  for (int64_t j = 0; j < jend; ++j) {
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int d = lane + 32 * e;
      if (d < D) dot = fmaf(qv[e], ld_as_float<T>(kb + j * D + d), dot);
    }
    dot = warp_sum(dot) * scale;
    const float m_new = fmaxf(m, dot);
    const float alpha = expf(m - m_new);
    const float p = expf(dot - m_new);
    l = l * alpha + p;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int d = lane + 32 * e;
      if (d < D) acc[e] = acc[e] * alpha + p * ld_as_float<T>(vb + j * D + d);
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int d = lane + 32 * e;
    if (d < D) st_from_float<T>(o + row_id * D + d, acc[e] * inv);
  }
}

// fp32 LinearOp / MatmulOp (+ bias) on CUDA cores: fp32 graphs (the reference's scalar FMA tier) have no tensor-core
// path here; one thread per output element.
__global__ void __launch_bounds__(256) gemm_f32_simt_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                            const float* __restrict__ bias, float* __restrict__ y,
                                                            int64_t M, int64_t N, int64_t K, int wl) {
  const int64_t total = M * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / N, n = i % N;
    const float* xr = x + m * K;
    float acc = 0.f;
    if (wl == EMK_W_NK) {
      const float* wr = w + n * K;
      for (int64_t k = 0; k < K; ++k) acc = fmaf(xr[k], wr[k], acc);
    } else {
      for (int64_t k = 0; k < K; ++k) acc = fmaf(xr[k], w[k * N + n], acc);
    }
    y[i] = bias ? acc + bias[n] : acc;
  }
}

// Register-tiled fp32 contraction on CUDA cores: y[m,n] = e(sum_k x[m,k] * W), W [N,K] (WL = 0) or [K,N] (WL = 1),
// e = identity | + bias[n] | + residual[m,n] | * silu(gate[m,n]). The reference's perf suite drives exactly these
// shapes in fp32 (tests/perf/cases.py:60-74: the Qwen3 projections as torch.matmul, matmul + r, silu(x@wg) * (x@wu))
// and its emitted kernel for them is a 2x4-outputs-per-thread tile loop fed by TMA; this one keeps 4x4 outputs per
// thread in registers over a 64x64 CTA tile, stages 16-deep K slices of both operands through double-buffered
// shared memory (128-bit global loads, the activation slice stored transposed so a thread's four rows come back as
// one 128-bit shared load) and keeps the next two slices in flight into registers under the FMAs. Every
// output is still one fmaf chain over k in ascending order, i.e. bit-for-bit the serial reduce loop of the records.
// x[m,k] may live at (k / x_inner) * x_stride_outer + m * x_stride_m + k % x_inner (the blocked activation layout of
// the o_proj record); plain row-major is x_inner = K.
constexpr int FT_M = 64, FT_N = 64, FT_K = 16, FT_LD = 68, FT_PF = 2;

template <int WL>
__global__ void __launch_bounds__(256) gemm_f32_tiled_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                             const float* __restrict__ bias,
                                                             const float* __restrict__ residual,
                                                             const float* __restrict__ gate, float* __restrict__ y,
                                                             int M, int N, int K, int64_t x_inner,
                                                             int64_t x_stride_outer, int64_t x_stride_m,
                                                             int k_per_split) {
  __shared__ __align__(16) float As[2][FT_K][FT_LD];
  __shared__ __align__(16) float Bs[2][FT_K][FT_LD];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * FT_M, n0 = blockIdx.x * FT_N;
  // loader roles: activations (and [N,K] weights) as 64 rows x 4 quads of k; [K,N] weights as 16 k-rows x 16 quads of n
  const int lrow = tid >> 2, lkq = (tid & 3) * 4;
  const int bk = tid >> 4, bnq = (tid & 15) * 4;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const int xin = (int)x_inner;
  // split-K (gridDim.z > 1, few output tiles): this CTA sums k in [k_begin, k_lim) and adds its partial result to y,
  // which the host zeroed; with one split the result is stored and every output is one fmaf chain over all of k
  const int k_begin = (int)blockIdx.z * k_per_split;
  const int k_lim = min(K, k_begin + k_per_split);

  auto load_a = [&](int k0) -> float4 {
    const int m = m0 + lrow, k = k0 + lkq;
    if (m >= M || k >= k_lim) return zero4;
    const int kq = k / xin;   // 32-bit division: the 64-bit one cost as much as the slice's FMAs
    const int64_t off = (int64_t)kq * x_stride_outer + (int64_t)m * x_stride_m + (k - kq * xin);
    return __ldg(reinterpret_cast<const float4*>(x + off));
  };
  auto load_b = [&](int k0) -> float4 {
    if (WL == 0) {
      const int n = n0 + lrow, k = k0 + lkq;
      if (n >= N || k >= k_lim) return zero4;
      return __ldg(reinterpret_cast<const float4*>(w + (int64_t)n * K + k));
    }
    const int k = k0 + bk, n = n0 + bnq;
    if (k >= k_lim || n >= N) return zero4;
    return __ldg(reinterpret_cast<const float4*>(w + (int64_t)k * N + n));
  };
  auto store_tiles = [&](int buf, const float4& a, const float4& b) {
    As[buf][lkq + 0][lrow] = a.x; As[buf][lkq + 1][lrow] = a.y; As[buf][lkq + 2][lrow] = a.z; As[buf][lkq + 3][lrow] = a.w;
    if (WL == 0) {
      Bs[buf][lkq + 0][lrow] = b.x; Bs[buf][lkq + 1][lrow] = b.y; Bs[buf][lkq + 2][lrow] = b.z; Bs[buf][lkq + 3][lrow] = b.w;
    } else {
      *reinterpret_cast<float4*>(&Bs[buf][bk][bnq]) = b;
    }
  };

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int nk = (k_lim - k_begin + FT_K - 1) / FT_K;
  if (nk <= 0) return;
  // FT_PF K slices are on their way from global memory into registers at any time (a lone CTA per SM otherwise
  // spends most of each slice waiting for its loads: a 64-CTA problem ran at 9 TFLOP/s with one slice in flight);
  // a slice is written to the shared buffer of its parity right before it is used, one barrier per slice
  float4 ra[FT_PF], rb[FT_PF];
#pragma unroll
  for (int p = 0; p < FT_PF; ++p) {
    ra[p] = load_a(k_begin + p * FT_K);   // slices past the range read zeros
    rb[p] = load_b(k_begin + p * FT_K);
  }
  for (int kt = 0; kt < nk; kt += FT_PF) {
#pragma unroll
    for (int p = 0; p < FT_PF; ++p) {
      const int tile = kt + p;
      if (tile < nk) {   // uniform over the CTA
        const int buf = tile & 1;
        store_tiles(buf, ra[p], rb[p]);
        __syncthreads();
        ra[p] = load_a(k_begin + (tile + FT_PF) * FT_K);
        rb[p] = load_b(k_begin + (tile + FT_PF) * FT_K);
#pragma unroll
        for (int k = 0; k < FT_K; ++k) {
          const float4 a = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
          const float4 b = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
          const float av[4] = {a.x, a.y, a.z, a.w};
          const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
      }
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      const int64_t idx = (int64_t)m * N + n;
      float v = acc[i][j];
      if (gridDim.z > 1) {   // partial sum of one K range; y was initialised by the host (zeros, or the residual)
        if (blockIdx.z == 0 && bias != nullptr) v = v + bias[n];
        atomicAdd(y + idx, v);
        continue;
      }
      if (bias != nullptr) v = v + bias[n];
      if (residual != nullptr) v = residual[idx] + v;
      if (gate != nullptr) {
        const float gv = gate[idx];
        v = (gv * (1.0f / (1.0f + expf(-gv)))) * v;   // x * reciprocal(1 + exp(-x)), as the record spells silu
      }
      y[idx] = v;
    }
  }
}

// The tiled kernel needs 16-byte loads to be legal: k (and for [K,N] weights n) quads must not straddle rows.
inline bool f32_tiled_ok(const float* x, const float* w, int64_t N, int64_t K, int wl, int64_t x_inner,
                         int64_t x_stride_outer, int64_t x_stride_m) {
  if ((((uintptr_t)x | (uintptr_t)w) & 15u) != 0) return false;
  if ((K % 4) != 0 || (x_inner % 4) != 0 || (x_stride_outer % 4) != 0 || (x_stride_m % 4) != 0) return false;
  if (wl == EMK_W_KN && (N % 4) != 0) return false;
  return true;
}

// `sm_count` > 0 allows split-K when the output has too few tiles to fill the GPU (the K loop of a lone CTA is bound
// by the latency of its loads): y is zeroed and the splits add their partial sums with atomics, so the result is
// then no longer the serial chain, only equal to it within fp32 rounding. With a residual, y starts as a copy of it;
// a contraction with the multiplicative gate epilogue is never split.
template <int WL>
inline cudaError_t launch_f32_tiled(const float* x, const float* w, const float* bias, const float* residual,
                                    const float* gate, float* y, int64_t M, int64_t N, int64_t K, int64_t x_inner,
                                    int64_t x_stride_outer, int64_t x_stride_m, cudaStream_t s, int sm_count = 0) {
  dim3 grid((unsigned)((N + FT_N - 1) / FT_N), (unsigned)((M + FT_M - 1) / FT_M), 1);
  int64_t k_per_split = K;
  const int64_t tiles = (int64_t)grid.x * grid.y;
  if (sm_count > 0 && gate == nullptr && residual != y && tiles < 3 * (int64_t)sm_count && K >= 8 * FT_K) {
    int64_t splits = (4 * (int64_t)sm_count + tiles - 1) / tiles;   // about four 8-warp CTAs per SM hide the load latency
    if (splits > 16) splits = 16;
    k_per_split = ((K + splits - 1) / splits + FT_K - 1) / FT_K * FT_K;
    grid.z = (unsigned)((K + k_per_split - 1) / k_per_split);
    if (grid.z > 1) {
      // the splits add into y: it starts as zeros, or as the residual (which the sum is then added to)
      cudaError_t e = residual != nullptr
                          ? cudaMemcpyAsync(y, residual, (size_t)(M * N) * sizeof(float), cudaMemcpyDeviceToDevice, s)
                          : cudaMemsetAsync(y, 0, (size_t)(M * N) * sizeof(float), s);
      if (e != cudaSuccess) return e;
      residual = nullptr;
    }
  }
  gemm_f32_tiled_kernel<WL><<<grid, 256, 0, s>>>(x, w, bias, residual, gate, y, (int)M, (int)N, (int)K, x_inner,
                                                 x_stride_outer, x_stride_m, (int)k_per_split);
  return cudaSuccess;
}

// fp32 contraction of the Loop-IR kernel records (one LoopOp of the reference = one launch here):
//   y[m,n] = epilogue( sum_k x[m,k] * W[n,k] ),  epilogue = identity | + r[m,n] | * silu(g[m,n]).
// x[m,k] lives at (k / x_inner) * x_stride_outer + m * x_stride_m + k % x_inner, which covers the plain row-major
// activation (x_inner = K) and the [K/D, M, D] head-major attention output the o_proj record reads through a
// div/mod index. 32x32 output tile per CTA, K in steps of 32 through shared memory (coalesced loads of both operands),
// accumulation in k order like the reference's serial reduce loop.
__global__ void __launch_bounds__(1024) loop_linear_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                               const float* __restrict__ residual,
                                                               const float* __restrict__ gate, float* __restrict__ y,
                                                               int64_t M, int64_t N, int64_t K, int64_t x_inner,
                                                               int64_t x_stride_outer, int64_t x_stride_m) {
  __shared__ float sx[32][33];
  __shared__ float sw[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t m0 = (int64_t)blockIdx.y * 32, n0 = (int64_t)blockIdx.x * 32;
  float acc = 0.f;
  for (int64_t k0 = 0; k0 < K; k0 += 32) {
    const int64_t k = k0 + tx;
    const int64_t m = m0 + ty, n = n0 + ty;
    sx[ty][tx] = (m < M && k < K) ? x[(k / x_inner) * x_stride_outer + m * x_stride_m + k % x_inner] : 0.f;
    sw[ty][tx] = (n < N && k < K) ? w[n * K + k] : 0.f;
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) acc = fmaf(sx[ty][kk], sw[tx][kk], acc);
    __syncthreads();
  }
  const int64_t m = m0 + ty, n = n0 + tx;
  if (m < M && n < N) {
    const int64_t i = m * N + n;
    if (residual != nullptr) acc = residual[i] + acc;
    if (gate != nullptr) {
      const float gv = gate[i];
      acc = (gv * (1.0f / (1.0f + expf(-gv)))) * acc;   // x * reciprocal(1 + exp(-x)), as the record spells silu
    }
    y[i] = acc;
  }
}

// The reference's unfused attention, first half (kernels/k_scaled_dot_product_attention_masked_reduce.json):
//   s[h,i,j] = scale * sum_d rope(q)[i,h,d] * rope(k)[j,h/g,d] + (j <= i ? mask_zero : mask_fill),
//   rope(x)[d] = x[d] * cos[pos,d] + (d < D/2 ? -x[d + D/2] : x[d - D/2]) * sin[pos,d].
// q [S, H*D], k [S, Hkv*D], cos/sin [S, D], s [H, S, S]. One CTA per 32x32 tile of (i, j) and head: the rotated rows
// are built once in shared memory, then every thread takes one dot product over d in ascending order.
__global__ void __launch_bounds__(1024) loop_rope_scores_f32_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                                   const float* __restrict__ cosb,
                                                                   const float* __restrict__ sinb, float* __restrict__ y,
                                                                   int S, int H, int Hkv, int D, float scale,
                                                                   float mask_zero, float mask_fill) {
  extern __shared__ float rs_smem[];
  float* rq = rs_smem;                    // [32][D + 1]
  float* rk = rs_smem + 32 * (D + 1);     // [32][D + 1]
  const int h = blockIdx.z, hk = h / (H / Hkv);
  const int i0 = blockIdx.y * 32, j0 = blockIdx.x * 32;
  const int half = D / 2;
  for (int e = threadIdx.x; e < 32 * D; e += blockDim.x) {
    const int row = e / D, d = e % D;
    const int dr = d < half ? d + half : d - half;
    const int i = i0 + row, j = j0 + row;
    float vq = 0.f, vk = 0.f;
    if (i < S) {
      const float* qr = q + (int64_t)i * H * D + (int64_t)h * D;
      const float rot = d < half ? -qr[dr] : qr[dr];
      vq = qr[d] * cosb[(int64_t)i * D + d] + rot * sinb[(int64_t)i * D + d];
    }
    if (j < S) {
      const float* kr = k + (int64_t)j * Hkv * D + (int64_t)hk * D;
      const float rot = d < half ? -kr[dr] : kr[dr];
      vk = kr[d] * cosb[(int64_t)j * D + d] + rot * sinb[(int64_t)j * D + d];
    }
    rq[row * (D + 1) + d] = vq;
    rk[row * (D + 1) + d] = vk;
  }
  __syncthreads();
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int i = i0 + ty, j = j0 + tx;
  if (i < S && j < S) {
    float acc = 0.f;
    for (int d = 0; d < D; ++d) acc += rq[ty * (D + 1) + d] * rk[tx * (D + 1) + d];
    y[((int64_t)h * S + i) * S + j] = acc * scale + (j <= i ? mask_zero : mask_fill);
  }
}

// Second half (kernels/k_scaled_dot_product_attention_reduce_reduce.json):
//   o[h,i,d] = sum_j (exp(s[h,i,j] - max_j s) / sum_j exp(s[h,i,j] - max_j s)) * v[j,h/g,d].
// s [H, S, S], v [S, Hkv*D], o [H, S, D]. One warp per (h, i) row; the row's weights go through shared memory.
__global__ void __launch_bounds__(256) loop_softmax_pv_f32_kernel(const float* __restrict__ sc, const float* __restrict__ v,
                                                                 float* __restrict__ o, int S, int H, int Hkv, int D) {
  extern __shared__ float pv_smem[];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float* p = pv_smem + wid * S;
  const int64_t row = (int64_t)blockIdx.x * 8 + wid;
  if (row >= (int64_t)H * S) return;
  const int h = (int)(row / S), hk = h / (H / Hkv);
  const float* srow = sc + row * S;
  float mx = -CUDART_INF_F;
  for (int j = lane; j < S; j += 32) mx = fmaxf(mx, srow[j]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int j = lane; j < S; j += 32) {
    const float e = expf(srow[j] - mx);
    p[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  __syncwarp();
  for (int d = lane; d < D; d += 32) {
    float acc = 0.f;
    for (int j = 0; j < S; ++j) acc += (p[j] / sum) * v[(int64_t)j * Hkv * D + (int64_t)hk * D + d];
    o[row * D + d] = acc;
  }
}

}  // namespace

extern "C" int emk_loop_rope_scores_f32(emk_handle_t h, const float* q, const float* k, const float* cosb,
                                        const float* sinb, float* y, int64_t S, int64_t H, int64_t Hkv, int64_t D,
                                        float scale, float mask_zero, float mask_fill, emk_stream_t stream) {
  if (!h || !q || !k || !cosb || !sinb || !y) return EMK_ERR_ARG;
  if (S <= 0 || H <= 0 || Hkv <= 0 || D <= 0 || (D % 2) != 0 || H % Hkv != 0) return EMK_ERR_SHAPE;
  if (D > 128 || H > 65535 || S > 65535 * 32) return EMK_ERR_LIMIT;
  const unsigned t = (unsigned)((S + 31) / 32);
  const size_t smem = (size_t)2 * 32 * (D + 1) * sizeof(float);
  loop_rope_scores_f32_kernel<<<dim3(t, t, (unsigned)H), 1024, smem, (cudaStream_t)stream>>>(
      q, k, cosb, sinb, y, (int)S, (int)H, (int)Hkv, (int)D, scale, mask_zero, mask_fill);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_loop_softmax_pv_f32(emk_handle_t h, const float* scores, const float* v, float* o, int64_t S,
                                       int64_t H, int64_t Hkv, int64_t D, emk_stream_t stream) {
  if (!h || !scores || !v || !o) return EMK_ERR_ARG;
  if (S <= 0 || H <= 0 || Hkv <= 0 || D <= 0 || H % Hkv != 0) return EMK_ERR_SHAPE;
  if (S > 1536) {
    EMK_SET_ERR(h, "emk_loop_softmax_pv_f32: row length %lld exceeds the 1536 floats per warp of shared memory",
                (long long)S);
    return EMK_ERR_LIMIT;
  }
  const int64_t blocks = (H * S + 7) / 8;
  if (blocks > 0x7fffffffLL) return EMK_ERR_SHAPE;
  loop_softmax_pv_f32_kernel<<<(unsigned)blocks, 256, (size_t)8 * S * sizeof(float), (cudaStream_t)stream>>>(
      scores, v, o, (int)S, (int)H, (int)Hkv, (int)D);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_loop_linear_f32(emk_handle_t h, const float* x, const float* w, const float* residual,
                                   const float* gate, float* y, int64_t M, int64_t N, int64_t K, int64_t x_inner,
                                   int64_t x_stride_outer, int64_t x_stride_m, emk_stream_t stream) {
  if (!h || !x || !w || !y) return EMK_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || x_inner <= 0 || K % x_inner != 0 || x_stride_m <= 0 || x_stride_outer < 0)
    return EMK_ERR_SHAPE;
  if (residual != nullptr && gate != nullptr) return EMK_ERR_ARG;
  if (M <= 0x7fffffffLL && N <= 0x7fffffffLL && K <= 0x7fffffffLL && (M + FT_M - 1) / FT_M <= 65535 &&
      f32_tiled_ok(x, w, N, K, EMK_W_NK, x_inner, x_stride_outer, x_stride_m)) {
    EMK_CUDA_TRY(h, launch_f32_tiled<0>(x, w, nullptr, residual, gate, y, M, N, K, x_inner, x_stride_outer,
                                        x_stride_m, (cudaStream_t)stream, h->sm_count));
    EMK_LAUNCH_CHECK(h);
    return EMK_OK;
  }
  const int64_t gx = (N + 31) / 32, gy = (M + 31) / 32;
  if (gx > 0x7fffffffLL || gy > 65535) return EMK_ERR_SHAPE;
  loop_linear_f32_kernel<<<dim3((unsigned)gx, (unsigned)gy), 1024, 0, (cudaStream_t)stream>>>(
      x, w, residual, gate, y, M, N, K, x_inner, x_stride_outer, x_stride_m);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_linear_bf16_simt(emk_handle_t h, const void* x, const void* w, const void* residual, void* y,
                                    int64_t M, int64_t N, int64_t K, int wlayout, int epilogue, emk_stream_t stream) {
  if (!h || !x || !w || !y) return EMK_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0) return EMK_ERR_SHAPE;
  if (wlayout != EMK_W_NK && wlayout != EMK_W_KN) return EMK_ERR_ARG;
  if (epilogue < EMK_EPI_NONE || epilogue > EMK_EPI_BIAS) return EMK_ERR_ARG;
  if ((epilogue == EMK_EPI_RESIDUAL || epilogue == EMK_EPI_BIAS) && !residual) return EMK_ERR_ARG;
  if (epilogue == EMK_EPI_SWIGLU && (N % 2) != 0) return EMK_ERR_SHAPE;
  const int64_t total = M * ((epilogue == EMK_EPI_SWIGLU) ? N / 2 : N);
  int64_t blocks = (total + 255) / 256;
  if (blocks > (int64_t)h->sm_count * 32) blocks = (int64_t)h->sm_count * 32;
  gemm_simt_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, M, N, K,
      wlayout, epilogue);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_sdpa_simt(emk_handle_t h, const void* q, const void* k, const void* v, void* o, int64_t B,
                             int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv, int64_t D, float scale, int causal,
                             int dtype, emk_stream_t stream) {
  if (!h || !q || !k || !v || !o) return EMK_ERR_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || D <= 0 || D > 256 || Hq % Hkv != 0) return EMK_ERR_SHAPE;
  const int64_t rows = B * Hq * Sq;
  const int64_t blocks = (rows + 7) / 8;
  if (blocks > 0x7fffffffLL) return EMK_ERR_SHAPE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == EMK_F32)
    sdpa_simt_kernel<float><<<(unsigned)blocks, 256, 0, s>>>((const float*)q, (const float*)k, (const float*)v,
                                                             (float*)o, B, Hq, Hkv, Sq, Skv, (int)D, scale, causal);
  else if (dtype == EMK_BF16)
    sdpa_simt_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)o, B, Hq, Hkv, Sq,
        Skv, (int)D, scale, causal);
  else
    return EMK_ERR_DTYPE;
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

extern "C" int emk_linear_f32_simt(emk_handle_t h, const float* x, const float* w, const float* bias, float* y,
                                   int64_t M, int64_t N, int64_t K, int wlayout, emk_stream_t stream) {
  if (!h || !x || !w || !y) return EMK_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0) return EMK_ERR_SHAPE;
  if (wlayout != EMK_W_NK && wlayout != EMK_W_KN) return EMK_ERR_ARG;
  if (M <= 0x7fffffffLL && N <= 0x7fffffffLL && K <= 0x7fffffffLL && (M + FT_M - 1) / FT_M <= 65535 &&
      f32_tiled_ok(x, w, N, K, wlayout, K, 0, K)) {
    if (wlayout == EMK_W_NK)
      EMK_CUDA_TRY(h, launch_f32_tiled<0>(x, w, bias, nullptr, nullptr, y, M, N, K, K, 0, K, (cudaStream_t)stream,
                                          h->sm_count));
    else
      EMK_CUDA_TRY(h, launch_f32_tiled<1>(x, w, bias, nullptr, nullptr, y, M, N, K, K, 0, K, (cudaStream_t)stream,
                                          h->sm_count));
    EMK_LAUNCH_CHECK(h);
    return EMK_OK;
  }
  // odd sizes or unaligned operands: one thread per output
  int64_t blocks = (M * N + 255) / 256;
  if (blocks > (int64_t)h->sm_count * 32) blocks = (int64_t)h->sm_count * 32;
  gemm_f32_simt_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(x, w, bias, y, M, N, K, wlayout);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}
