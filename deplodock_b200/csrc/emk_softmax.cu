// Softmax over the last axis: y = exp(x - max) / sum(exp(x - max)), one read and one write of the tensor.
//
// Reference behaviour: SoftmaxOp (emmy/compiler/ir/frontend/ir.py:343-358), decomposed by
// emmy/compiler/pipeline/passes/frontend/decomposition/100_softmax.py:11-18 and lowered as an online (max, sum)
// carrier (emmy/compiler/pipeline/passes/lowering/tile/_softmax.py:123); its cold schedule gives one thread a whole
// row and reads the row twice with an 8 KB stride between neighbouring threads. Here one warp owns a row, keeps it in
// registers, reduces with shuffles, and every access is a coalesced 128-bit streaming load/store, so HBM traffic is
// exactly one read plus one write. Rows longer than 8 vectors per lane are shared by two or four warps. The reference seeds the running
// max with -1e30 (emmy/compiler/ir/elementwise.py:75-76); -inf is used here so -inf inputs behave as in torch.
#include "emk_common.cuh"

#include <math_constants.h>

namespace {

using namespace emk;

template <typename T>
struct Row16;
template <>
struct Row16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) {
    float4 v = __ldcs(reinterpret_cast<const float4*>(p));
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* f) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(f[0], f[1], f[2], f[3]));
  }
};
template <>
struct Row16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    uint4 v = __ldcs(reinterpret_cast<const uint4*>(p));
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* f) {
    uint4 v;
    v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]);
    v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
    __stcs(reinterpret_cast<uint4*>(p), v);
  }
};

// One warp per row, NV 16-byte vectors per lane held in registers between the reduce and the write.
template <typename T, int NV>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows,
                                                           int cols) {
  constexpr int E = Row16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int nvec = cols / E;
  for (int64_t row = warp; row < rows; row += nwarps) {
    const T* xr = x + row * cols;
    float v[NV][E];
    float m = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
        Row16<T>::load(xr + (int64_t)vi * E, v[i]);
#pragma unroll
        for (int e = 0; e < E; ++e) m = fmaxf(m, v[i][e]);
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) v[i][e] = -CUDART_INF_F;
      }
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
      for (int e = 0; e < E; ++e) {
        // x - m is NaN only when the whole row is -inf (m = -inf): torch returns NaN there too.
        v[i][e] = expf(v[i][e] - m);
        sum += v[i][e];
      }
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    T* yr = y + row * cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
        float o[E];
#pragma unroll
        for (int e = 0; e < E; ++e) o[e] = v[i][e] * inv;
        Row16<T>::store(yr + (int64_t)vi * E, o);
      }
    }
  }
}


// Long rows, many rows: WPR warps share a row (NV vectors per lane each), so a 2048-float row costs 32 data registers
// per lane instead of 64 and three to four CTAs fit an SM — the kernel is bound by HBM latency, and with one warp per
// row (16 resident warps) it reached 80 % of the copy bandwidth, with 24-32 resident warps 90 %. The two reductions
// cross the warps of a row through shared memory and two CTA barriers per row.
template <typename T, int NV, int WPR>
__global__ void __launch_bounds__(256, 4) softmax_multiwarp_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                   int64_t rows, int cols) {
  constexpr int E = Row16<T>::N;
  constexpr int RPC = 8 / WPR;  // rows per CTA
  __shared__ float red[2][RPC][WPR];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int r_in_cta = warp / WPR;
  const int wr = warp % WPR;
  const int nvec = cols / E;
  const int64_t row_stride = (int64_t)gridDim.x * RPC;
  const int64_t n_trips = (rows + row_stride - 1) / row_stride;  // same for every thread: barriers stay uniform
  for (int64_t trip = 0; trip < n_trips; ++trip) {
    const int64_t row = trip * row_stride + (int64_t)blockIdx.x * RPC + r_in_cta;
    const bool live = row < rows;
    const T* xr = x + (live ? row : 0) * cols;
    float v[NV][E];
    float m = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = (i * WPR + wr) * 32 + lane;
      if (live && vi < nvec) {
        Row16<T>::load(xr + (int64_t)vi * E, v[i]);
#pragma unroll
        for (int e = 0; e < E; ++e) m = fmaxf(m, v[i][e]);
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) v[i][e] = -CUDART_INF_F;
      }
    }
    m = warp_max(m);
    if (lane == 0) red[0][r_in_cta][wr] = m;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < WPR; ++k) m = fmaxf(m, red[0][r_in_cta][k]);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
      for (int e = 0; e < E; ++e) {
        v[i][e] = expf(v[i][e] - m);
        sum += v[i][e];
      }
    }
    sum = warp_sum(sum);
    if (lane == 0) red[1][r_in_cta][wr] = sum;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < WPR; ++k) tot += red[1][r_in_cta][k];
    const float inv = 1.0f / tot;
    T* yr = y + (live ? row : 0) * cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = (i * WPR + wr) * 32 + lane;
      if (live && vi < nvec) {
        float o[E];
#pragma unroll
        for (int e = 0; e < E; ++e) o[e] = v[i][e] * inv;
        Row16<T>::store(yr + (int64_t)vi * E, o);
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ float ld_f(const T* p);
template <>
__device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void st_f(T* p, float v);
template <>
__device__ __forceinline__ void st_f<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// Any row length / alignment: one CTA per row, three scalar sweeps (max, sum, write).
template <typename T>
__global__ void __launch_bounds__(256) softmax_generic_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                              int64_t rows, int64_t cols) {
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    float m = -CUDART_INF_F;
    for (int64_t c = threadIdx.x; c < cols; c += 256) m = fmaxf(m, ld_f<T>(xr + c));
    m = warp_max(m);
    if (lane == 0) red[wid] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    __syncthreads();
    float sum = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += 256) sum += expf(ld_f<T>(xr + c) - m);
    sum = warp_sum(sum);
    if (lane == 0) red[wid] = sum;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    __syncthreads();
    const float inv = 1.0f / tot;
    T* yr = y + row * cols;
    for (int64_t c = threadIdx.x; c < cols; c += 256) st_f<T>(yr + c, expf(ld_f<T>(xr + c) - m) * inv);
  }
}

template <typename T>
int launch_softmax(emk_handle_t h, const T* x, T* y, int64_t rows, int64_t cols, cudaStream_t s) {
  constexpr int E = Row16<T>::N;
  const bool vec_ok =
      (cols % E == 0) && (((uintptr_t)x | (uintptr_t)y) & 15u) == 0 && cols <= (int64_t)E * 1024;  // a row must fit the registers of four warps
  if (!vec_ok) {
    int grid = (int)(rows < 65535 * 16 ? rows : 65535 * 16);
    softmax_generic_kernel<T><<<grid, 256, 0, s>>>(x, y, rows, cols);
    EMK_LAUNCH_CHECK(h);
    return EMK_OK;
  }
  const int nvec = (int)(cols / E);
  const int64_t ctas = (rows + 7) / 8;
  const int grid = (int)(ctas < (int64_t)h->sm_count * 256 ? ctas : (int64_t)h->sm_count * 256);
  if (nvec <= 32) softmax_warp_kernel<T, 1><<<grid, 256, 0, s>>>(x, y, rows, (int)cols);
  else if (nvec <= 64) softmax_warp_kernel<T, 2><<<grid, 256, 0, s>>>(x, y, rows, (int)cols);
  else if (nvec <= 128) softmax_warp_kernel<T, 4><<<grid, 256, 0, s>>>(x, y, rows, (int)cols);
  else if (nvec <= 256) softmax_warp_kernel<T, 8><<<grid, 256, 0, s>>>(x, y, rows, (int)cols);
  else {
    // rows longer than 8 vectors per lane: two or four warps per row keep the register count low enough for four
    // CTAs per SM
    const int64_t cap = (int64_t)h->sm_count * 64;
    if (nvec <= 512) {
      const int64_t c2 = (rows + 3) / 4;
      softmax_multiwarp_kernel<T, 8, 2><<<(int)(c2 < cap ? c2 : cap), 256, 0, s>>>(x, y, rows, (int)cols);
    } else {
      const int64_t c4 = (rows + 1) / 2;
      softmax_multiwarp_kernel<T, 8, 4><<<(int)(c4 < cap ? c4 : cap), 256, 0, s>>>(x, y, rows, (int)cols);
    }
  }
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

}  // namespace

extern "C" int emk_softmax_lastdim(emk_handle_t h, const void* x, void* y, int64_t rows, int64_t cols, int dtype,
                                   emk_stream_t stream) {
  if (!h || !x || !y) return EMK_ERR_ARG;
  if (rows <= 0 || cols <= 0) return EMK_ERR_SHAPE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == EMK_F32) return launch_softmax<float>(h, (const float*)x, (float*)y, rows, cols, s);
  if (dtype == EMK_BF16)
    return launch_softmax<__nv_bfloat16>(h, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, cols, s);
  return EMK_ERR_DTYPE;
}
