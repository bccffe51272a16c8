// emk_linear_residual_rmsnorm_bf16_noalloc: y_hidden = bf16(bf16(x·Wᵀ) + residual), y_norm = RMSNorm(y_hidden), for
// callers that must not allocate device memory.
//
// Who that is: a plugin running inside a host process that owns the whole device heap through its own pool (an
// inference server that grabbed "all free memory" at start-up and forbids cudaMalloc afterwards, so a late cudaMalloc
// fails or fragments the pool), code running while a stream is being captured (cudaMalloc is not capturable), and
// real-time callers that cannot take the implicit device synchronisation of cudaMalloc / cudaFree. The other entry
// points leave scratch to the caller; here the one piece of scratch the fused pair of kernels needs — the partial row
// sums of squares the GEMM epilogue hands to the normalising kernel — lives in a fixed array inside the library.
//
// Consequences the caller has to know:
//   * the array costs EMK_NOALLOC_MAX_SLOTS * 4 bytes (4 MiB) on every GPU that loads the library, until exit;
//   * sizes are limited: M * ceil(N / 128) <= EMK_NOALLOC_MAX_SLOTS, otherwise EMK_ERR_LIMIT;
//   * all calls on a device share the array: two calls that overlap on the GPU (different streams) race. The array
//     keeps the last call's contents; nothing in it has to start at zero because the GEMM epilogue overwrites every
//     slot it later reads;
//   * the first call on a device looks the array's device address up (cudaGetSymbolAddress), and the first call of
//     each shape class (M <= 128 or larger, N <= 128 or larger, M and N both multiples of 256 or not: each selects
//     its own GEMM kernel) sets that kernel's attributes: make a warm-up call of the same shape class before any stream capture.
// No counterpart exists in the reference (its runtime allocates through cupy, emmy/compiler/backend/cuda/program.py:340-364).
#include "emk_common.cuh"

#define EMK_NOALLOC_MAX_SLOTS (1 << 20)

// File-scope scratch. In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_noalloc_row_sumsq[EMK_NOALLOC_MAX_SLOTS];

namespace {

using namespace emk;

// y_norm[m,:] = bf16(w * bf16(h[m,:] * rsqrt(sum_s partial[m][s] / N + eps))): one warp per row, 16-byte accesses.
__global__ void __launch_bounds__(256) rmsnorm_from_partials_kernel(const __nv_bfloat16* __restrict__ hbuf,
                                                                    const __nv_bfloat16* __restrict__ w,
                                                                    const float* __restrict__ partial,
                                                                    __nv_bfloat16* __restrict__ y, int M, int N,
                                                                    int nslots, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= M) return;
  float tot = 0.f;
  for (int s = 0; s < nslots; ++s) tot += partial[(int64_t)row * nslots + s];
  const float r = 1.0f / sqrtf(tot / (float)N + eps);
  const __nv_bfloat16* hr = hbuf + (int64_t)row * N;
  __nv_bfloat16* yr = y + (int64_t)row * N;
  for (int c = lane * 8; c < N; c += 256) {
    const uint4 hv = *reinterpret_cast<const uint4*>(hr + c);
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + c));
    const uint32_t hh[4] = {hv.x, hv.y, hv.z, hv.w};
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = bf16_round(bf16_lo(hh[e]) * r) * bf16_lo(ww[e]);
      const float b = bf16_round(bf16_hi(hh[e]) * r) * bf16_hi(ww[e]);
      o[e] = pack_bf16x2(a, b);
    }
    *reinterpret_cast<uint4*>(yr + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Device address of the scratch array, looked up once per device with that device current.
int scratch_address(emk_handle_t h, float** out) {
  static float* addr[EMK_MAX_DEVICES] = {nullptr};
  static std::mutex mu;
  const int d = h->device;
  if (d < 0 || d >= EMK_MAX_DEVICES) return EMK_ERR_ARG;
  std::lock_guard<std::mutex> lk(mu);
  if (addr[d] == nullptr) {
    int cur = -1;
    EMK_CUDA_TRY(h, cudaGetDevice(&cur));
    if (cur != d) EMK_CUDA_TRY(h, cudaSetDevice(d));
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_row_sumsq);
    if (cur != d) (void)cudaSetDevice(cur);
    if (e != cudaSuccess || p == nullptr) {
      EMK_SET_ERR(h, "cudaGetSymbolAddress(g_noalloc_row_sumsq) failed: %s", cudaGetErrorString(e));
      return EMK_ERR_CUDA;
    }
    addr[d] = p;
  }
  *out = addr[d];
  return EMK_OK;
}

}  // namespace

extern "C" int emk_linear_residual_rmsnorm_bf16_noalloc(emk_handle_t h, const void* x, const void* w,
                                                        const void* residual, const void* norm_weight, void* y_hidden,
                                                        void* y_norm, int64_t M, int64_t N, int64_t K, float eps,
                                                        emk_stream_t stream) {
  if (!h || !x || !w || !residual || !norm_weight || !y_hidden || !y_norm) return EMK_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0) return EMK_ERR_SHAPE;
  if ((N % 8) != 0 || (K % 8) != 0) return EMK_ERR_ALIGN;
  if ((((uintptr_t)norm_weight | (uintptr_t)y_norm | (uintptr_t)y_hidden) & 15u) != 0) return EMK_ERR_ALIGN;
  const int64_t nslots = (N + 127) / 128;
  if (M * nslots > (int64_t)EMK_NOALLOC_MAX_SLOTS || M > 0x7fffffffLL) {
    EMK_SET_ERR(h,
                "emk_linear_residual_rmsnorm_bf16_noalloc: M * ceil(N/128) = %lld exceeds the built-in scratch of %d "
                "slots; use emk_gemm_bf16_fused with a caller-provided row_sumsq buffer",
                (long long)(M * nslots), EMK_NOALLOC_MAX_SLOTS);
    return EMK_ERR_LIMIT;
  }
  float* scratch = nullptr;
  int rc = scratch_address(h, &scratch);
  if (rc != EMK_OK) return rc;
  emk_gemm_desc_t d;
  memset(&d, 0, sizeof(d));
  d.x = x;
  d.w = w;
  d.residual = residual;
  d.y = y_hidden;
  d.M = M;
  d.N = N;
  d.K = K;
  d.wlayout = EMK_W_NK;
  d.epilogue = EMK_EPI_RESIDUAL;
  d.row_sumsq_out = scratch;  // a device address: the array's name itself must never reach a kernel from host code
  rc = emk_gemm_bf16_fused(h, &d, stream);
  if (rc != EMK_OK) return rc;
  const int64_t grid = (M + 7) / 8;
  rmsnorm_from_partials_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)y_hidden, (const __nv_bfloat16*)norm_weight, scratch, (__nv_bfloat16*)y_norm, (int)M, (int)N,
      (int)nslots, eps);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}
