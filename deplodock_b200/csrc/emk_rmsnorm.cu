// RMSNorm over the last axis: one read of x, one write of y, fp32 statistics.
//
// Reference behaviour: RmsNormOp (emmy/compiler/ir/frontend/ir.py:296-312) decomposed by
// emmy/compiler/pipeline/passes/frontend/decomposition/080_rms_norm.py:17-60 into acc = sum(x*x);
// r = rsqrt(acc * (1/N) + eps); y = x * r * w. The emitted kernel re-reads x from global memory for the second
// sweep; here each row stays in registers between the two sweeps, so the HBM traffic is the algorithmic minimum
// (x + y + w bytes). HBM-bound: 128-bit coalesced loads, shuffle-tree reductions, no shared-memory staging needed
// because a row fits the register file.
#include "emk_common.cuh"

namespace {

using namespace emk;

template <typename T>
struct Vec16;  // a 16-byte vector of T and its conversion to floats
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) {
    float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void load_stream(const float* p, float* f) {
    float4 v = __ldcs(reinterpret_cast<const float4*>(p));
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store_stream(float* p, const float* f) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(f[0], f[1], f[2], f[3]));
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(uint4 v, float* f) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
  }
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    unpack(*reinterpret_cast<const uint4*>(p), f);
  }
  static __device__ __forceinline__ void load_stream(const __nv_bfloat16* p, float* f) {
    unpack(__ldcs(reinterpret_cast<const uint4*>(p)), f);
  }
  static __device__ __forceinline__ void store_stream(__nv_bfloat16* p, const float* f) {
    uint4 v;
    v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]);
    v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
    __stcs(reinterpret_cast<uint4*>(p), v);
  }
};

// Output rounding. fp32: y = (x*r)*w. bf16: y = bf16(w * bf16(x*r)) — the normalised value is rounded to bf16 before
// the weight multiply, as the eager Qwen3 RMSNorm module does when its input is bf16.
template <typename T>
__device__ __forceinline__ float norm_out(float x, float r, float w);
template <>
__device__ __forceinline__ float norm_out<float>(float x, float r, float w) { return (x * r) * w; }
template <>
__device__ __forceinline__ float norm_out<__nv_bfloat16>(float x, float r, float w) { return bf16_round(x * r) * w; }

// Two neighbouring elements at a time. bf16: the two roundings of the normalised values are ONE packed conversion
// (cvt.rn.bf16x2.f32) instead of two scalar ones, which run at a quarter of the rate on the conversion pipe and were
// 43 % of its capacity in this kernel; the values are the same.
template <typename T>
__device__ __forceinline__ void norm_out2(const float* x, float r, const float* w, float* o);
template <>
__device__ __forceinline__ void norm_out2<float>(const float* x, float r, const float* w, float* o) {
  o[0] = (x[0] * r) * w[0];
  o[1] = (x[1] * r) * w[1];
}
template <>
__device__ __forceinline__ void norm_out2<__nv_bfloat16>(const float* x, float r, const float* w, float* o) {
  const uint32_t p = pack_bf16x2(x[0] * r, x[1] * r);
  o[0] = bf16_lo(p) * w[0];
  o[1] = bf16_hi(p) * w[1];
}

// One warp per row; each lane keeps NV 16-byte vectors of the row in registers. cols must be a multiple of the
// vector width; vectors past the end of the row are skipped.
template <typename T, int NV>
__global__ void __launch_bounds__(256) rmsnorm_warp_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                           T* __restrict__ y, int64_t rows, int cols, float eps) {
  constexpr int E = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int nvec = cols / E;
  for (int64_t row = warp; row < rows; row += nwarps) {
    const T* xr = x + row * cols;
    float v[NV][E];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
        Vec16<T>::load_stream(xr + (int64_t)vi * E, v[i]);
#pragma unroll
        for (int e = 0; e < E; ++e) ss = fmaf(v[i][e], v[i][e], ss);
      }
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)cols + eps);
    T* yr = y + row * cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
        float wv[E], o[E];
        Vec16<T>::load(w + (int64_t)vi * E, wv);
#pragma unroll
        for (int e = 0; e < E; e += 2) norm_out2<T>(&v[i][e], r, &wv[e], &o[e]);
        Vec16<T>::store_stream(yr + (int64_t)vi * E, o);
      }
    }
  }
}

// One CTA per row for short tensors with long rows (the [1,32,2048] fp32 case is 32 rows): more threads per row,
// so the latency of the single launch is one load, one block reduction and one store per thread.
template <typename T, int NV, int THREADS>
__global__ void __launch_bounds__(THREADS) rmsnorm_cta_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                              T* __restrict__ y, int64_t rows, int cols, float eps) {
  constexpr int E = Vec16<T>::N;
  __shared__ float red[THREADS / 32];
  const int nvec = cols / E;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    float v[NV][E];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = i * THREADS + threadIdx.x;
      if (vi < nvec) {
        Vec16<T>::load_stream(xr + (int64_t)vi * E, v[i]);
#pragma unroll
        for (int e = 0; e < E; ++e) ss = fmaf(v[i][e], v[i][e], ss);
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[wid] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < THREADS / 32; ++i) tot += red[i];
    __syncthreads();
    const float r = 1.0f / sqrtf(tot / (float)cols + eps);
    T* yr = y + row * cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = i * THREADS + threadIdx.x;
      if (vi < nvec) {
        float wv[E], o[E];
        Vec16<T>::load(w + (int64_t)vi * E, wv);
#pragma unroll
        for (int e = 0; e < E; e += 2) norm_out2<T>(&v[i][e], r, &wv[e], &o[e]);
        Vec16<T>::store_stream(yr + (int64_t)vi * E, o);
      }
    }
  }
}

// Any cols / any alignment: one CTA per row, scalar accesses, x read twice (second read hits L1/L2).
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_generic_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                              T* __restrict__ y, int64_t rows, int64_t cols,
                                                              float eps) {
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    float ss = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      float f = to_f<T>(xr[c]);
      ss = fmaf(f, f, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) red[wid] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    __syncthreads();
    const float r = 1.0f / sqrtf(tot / (float)cols + eps);
    T* yr = y + row * cols;
    for (int64_t c = threadIdx.x; c < cols; c += 256)
      yr[c] = from_f<T>(norm_out<T>(to_f<T>(xr[c]), r, to_f<T>(w[c])));
  }
}

template <typename T>
int launch_rmsnorm(emk_handle_t h, const T* x, const T* w, T* y, int64_t rows, int64_t cols, float eps,
                   cudaStream_t s) {
  constexpr int E = Vec16<T>::N;
  const bool vec_ok = (cols % E == 0) && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)w) & 15u) == 0 &&
                      cols <= (int64_t)E * 32 * 16;
  if (!vec_ok) {
    int grid = (int)(rows < 65535 * 16 ? rows : 65535 * 16);
    rmsnorm_generic_kernel<T><<<grid, 256, 0, s>>>(x, w, y, rows, cols, eps);
    EMK_LAUNCH_CHECK(h);
    return EMK_OK;
  }
  const int nvec = (int)(cols / E);
  // Few rows: spread each row over a whole CTA. Many rows: one warp per row, eight rows per CTA.
  if (rows < (int64_t)h->sm_count * 8) {
    const int grid = (int)rows;
    if (nvec <= 128) rmsnorm_cta_kernel<T, 1, 128><<<grid, 128, 0, s>>>(x, w, y, rows, (int)cols, eps);
    else if (nvec <= 256) rmsnorm_cta_kernel<T, 1, 256><<<grid, 256, 0, s>>>(x, w, y, rows, (int)cols, eps);
    else rmsnorm_cta_kernel<T, 2, 256><<<grid, 256, 0, s>>>(x, w, y, rows, (int)cols, eps);
  } else {
    const int64_t ctas = (rows + 7) / 8;
    const int grid = (int)(ctas < (int64_t)h->sm_count * 16 ? ctas : (int64_t)h->sm_count * 16);  // two resident rounds of CTAs, rows dealt evenly (one row per warp on an uncapped grid measured 3 % slower)
    if (nvec <= 32) rmsnorm_warp_kernel<T, 1><<<grid, 256, 0, s>>>(x, w, y, rows, (int)cols, eps);
    else if (nvec <= 64) rmsnorm_warp_kernel<T, 2><<<grid, 256, 0, s>>>(x, w, y, rows, (int)cols, eps);
    else if (nvec <= 128) rmsnorm_warp_kernel<T, 4><<<grid, 256, 0, s>>>(x, w, y, rows, (int)cols, eps);
    else if (nvec <= 256) rmsnorm_warp_kernel<T, 8><<<grid, 256, 0, s>>>(x, w, y, rows, (int)cols, eps);
    else rmsnorm_warp_kernel<T, 16><<<grid, 256, 0, s>>>(x, w, y, rows, (int)cols, eps);
  }
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

}  // namespace

extern "C" int emk_rmsnorm(emk_handle_t h, const void* x, const void* w, void* y, int64_t rows, int64_t cols,
                           float eps, int dtype, emk_stream_t stream) {
  if (!h || !x || !w || !y) return EMK_ERR_ARG;
  if (rows <= 0 || cols <= 0) return EMK_ERR_SHAPE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == EMK_F32) return launch_rmsnorm<float>(h, (const float*)x, (const float*)w, (float*)y, rows, cols, eps, s);
  if (dtype == EMK_BF16)
    return launch_rmsnorm<__nv_bfloat16>(h, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rows,
                                         cols, eps, s);
  return EMK_ERR_DTYPE;
}
