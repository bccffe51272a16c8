// bf16-activation x e4m3-weight GEMM: y[m,n] = bf16(scale[n] * sum_k x[m,k] * float(Wq[n,k])).
//
// The reference has no fp8 path (nothing under emmy/ mentions fp8 or e4m3); the contraction itself is the LinearOp of
// emmy/compiler/ir/frontend/ir.py:202-217. tcgen05 kind::f16 needs both operands as 16-bit types, so the weight tile
// is dequantised inside the main loop: TMA lands the raw e4m3 tile (half the bytes of a bf16 tile) in shared memory,
// eight converter warps expand it to bf16 (exact: every e4m3 value is representable in bf16) directly into the
// 128-byte-swizzled K-major layout the tensor core reads, and the per-output-channel scale is applied once per
// output element in the epilogue (it commutes with the sum over k).
//
//   warps 0..3  epilogue (as in the bf16 kernel)      warp 4  TMA producer      warp 5  MMA issuer
//   warps 6..13 e4m3 -> bf16 converters
#include "emk_gemm_common.cuh"

#include <cuda_fp8.h>

namespace {

using namespace emk;

constexpr int W8_BN = 256;
constexpr int W8_STAGES = 3;
constexpr int W8_THREADS = 448;  // warps 0-3 epilogue, 4 TMA, 5 MMA, 6-13 converters
constexpr int W8_CVT_THREADS = 256;
constexpr int W8_RAW_BYTES = W8_BN * BK;       // e4m3 tile: 256 rows x 64 bytes
constexpr int W8_B_BYTES = W8_BN * BK * 2;     // bf16 tile
constexpr uint32_t W8_TX = A_STAGE_BYTES + W8_RAW_BYTES;
constexpr uint32_t W8_TMEM_COLS = 2 * W8_BN;
constexpr uint32_t W8_IDESC = make_idesc_bf16(BM, W8_BN, 0, 0);

struct __align__(8) W8Barriers {
  uint64_t full_raw[W8_STAGES];
  uint64_t full_cvt[W8_STAGES];
  uint64_t empty[W8_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// 4 e4m3 bytes (little endian, k ascending) -> two packed bf16 pairs.
__device__ __forceinline__ void cvt_e4m3x4_bf16(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xffffu), __NV_E4M3);
  const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
  const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
  const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
  lo = pack_bf16x2(f01.x, f01.y);
  hi = pack_bf16x2(f23.x, f23.y);
}

// Eight converter warps, not four: the conversion (one operation of the quarter-rate conversion pipe per element) is
// what paces the main loop, and two converter warps per scheduler hide its latency where one could not (4096 x 2048 x
// 6144: 158 -> 124 us; twelve warps: 130 us). Two routes around the conversion pipe were measured and dropped: the
// e4m3 bits shifted into a bf16's fields and scaled by a packed bf16 multiply (232 us), and cvt to f16 followed by the
// same shift-and-scale (184 us) — both exact, both slower than the plain conversions.
constexpr int W8_EXPAND_MIN_M = 256;  // above this many rows the weight is expanded once instead of per row tile

__global__ void __launch_bounds__(W8_THREADS, 1)
gemm_w8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_w,
               const GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = sA + W8_STAGES * A_STAGE_BYTES;
  uint8_t* sW = sB + W8_STAGES * W8_B_BYTES;
  W8Barriers* bars = reinterpret_cast<W8Barriers*>(sW + W8_STAGES * W8_RAW_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int ntiles = g.tiles_m * g.tiles_n;

  if (threadIdx.x == 0) {
    for (int i = 0; i < W8_STAGES; ++i) {
      mbar_init(&bars->full_raw[i], 1);
      mbar_init(&bars->full_cvt[i], W8_CVT_THREADS);
      mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 4);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_w);
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_base, W8_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  const WaitCtx wc{&bars->abort_flag, g.status, g.limit_ns};

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, g.tiles_m, g.tiles_n, 16, tm, tn);
        const int m0 = tm * BM;
        const int n0 = tn * W8_BN;
        for (int kb = 0; kb < g.kblocks; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1u, wc, EMK_DEV_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&bars->full_raw[stage], W8_TX);
          tma_load_2d(sA + stage * A_STAGE_BYTES, &tma_a, &bars->full_raw[stage], kb * BK, m0);
          tma_load_2d(sW + stage * W8_RAW_BYTES, &tma_w, &bars->full_raw[stage], kb * BK, n0);
          if (++stage == W8_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1u, wc, EMK_DEV_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * W8_BN);
        for (int kb = 0; kb < g.kblocks; ++kb) {
          if (!mbar_wait(&bars->full_raw[stage], phase, wc, EMK_DEV_TIMEOUT_MMA) ||
              !mbar_wait(&bars->full_cvt[stage], phase, wc, EMK_DEV_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * W8_B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_ss(d_tmem, make_smem_desc(a_addr + k * 32, 0, 1024), make_smem_desc(b_addr + k * 32, 0, 1024),
                    W8_IDESC, (uint32_t)((kb | k) != 0));
          }
          tc_commit(&bars->empty[stage]);
          if (++stage == W8_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(&bars->tmem_full[acc]);
      }
    }
  } else if (warp >= 6) {
    // ---------------- converters: e4m3 tile -> bf16 tile in the UMMA swizzled layout ----------------
    const int tid = threadIdx.x - 192;
    const int c = tid & 3;     // 16-byte chunk of the 64-byte e4m3 row -> bf16 chunks 2c, 2c+1
    const int r0 = tid >> 2;   // 0..63
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < g.kblocks; ++kb) {
        if (!mbar_wait_warp(&bars->full_raw[stage], phase, wc, EMK_DEV_TIMEOUT_CONVERT)) {
          ok = false;
          break;
        }
        const uint8_t* raw = sW + stage * W8_RAW_BYTES;
        uint8_t* dst = sB + stage * W8_B_BYTES;
#pragma unroll
        for (int i = 0; i < W8_BN / (W8_CVT_THREADS / 4); ++i) {
          const int r = r0 + (W8_CVT_THREADS / 4) * i;
          const uint4 v = *reinterpret_cast<const uint4*>(raw + r * 64 + c * 16);
          uint4 o0, o1;
          cvt_e4m3x4_bf16(v.x, o0.x, o0.y);
          cvt_e4m3x4_bf16(v.y, o0.z, o0.w);
          cvt_e4m3x4_bf16(v.z, o1.x, o1.y);
          cvt_e4m3x4_bf16(v.w, o1.z, o1.w);
          const int sw = r & 7;
          *reinterpret_cast<uint4*>(dst + r * 128 + (((2 * c) ^ sw) << 4)) = o0;
          *reinterpret_cast<uint4*>(dst + r * 128 + (((2 * c + 1) ^ sw) << 4)) = o1;
        }
        fence_proxy_async_smem();  // make the generic-proxy stores visible to the tensor core (async proxy)
        mbar_arrive(&bars->full_cvt[stage]);
        if (++stage == W8_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else {
    // ---------------- epilogue warps 0..3 ----------------
    int local = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
      if (!mbar_wait_warp(&bars->tmem_full[acc], acc_phase, wc, EMK_DEV_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      int tm, tn;
      tile_coords(tile, g.tiles_m, g.tiles_n, 16, tm, tn);
      const int m0 = tm * BM;
      const int n0 = tn * W8_BN;
      const int row = m0 + warp * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(acc * W8_BN);
      epilogue_drain<W8_BN / 32, EMK_EPI_NONE>(g, taddr, row, n0);   // the only epilogue of this kernel (+ channel scale)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_relaxed(&bars->tmem_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (bars->abort_flag) abort_drain();
  if (warp == 0) tmem_dealloc(tmem_base, W8_TMEM_COLS);
}

// e4m3 [rows of 16 bytes] -> bf16, exact (every e4m3 value is a bf16 value). One 16-byte load and one 32-byte store
// per thread and step; the grid covers the SMs a few times over and strides.
__global__ void __launch_bounds__(256) expand_e4m3_bf16_kernel(const uint4* __restrict__ src, uint32_t* __restrict__ dst,
                                                               int64_t n16) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 v = __ldg(src + i);
    uint32_t o[8];
    cvt_e4m3x4_bf16(v.x, o[0], o[1]);
    cvt_e4m3x4_bf16(v.y, o[2], o[3]);
    cvt_e4m3x4_bf16(v.z, o[4], o[5]);
    cvt_e4m3x4_bf16(v.w, o[6], o[7]);
    st_global_v8(dst + i * 8, o);
  }
}

constexpr int W8_SMEM = W8_STAGES * (A_STAGE_BYTES + W8_B_BYTES + W8_RAW_BYTES) + 1024 + (int)sizeof(W8Barriers);

}  // namespace

int emk_gemm_bf16_colscale_launch(emk_handle_t h, const void* x, const void* w, const float* scale, void* y, int64_t M,
                                  int64_t N, int64_t K, cudaStream_t s);

extern "C" int64_t emk_linear_bf16_w8_workspace_bytes(int64_t N, int64_t K) { return N > 0 && K > 0 ? N * K * 2 : 0; }

extern "C" int emk_linear_bf16_w8(emk_handle_t h, const void* x, const void* w_e4m3, const float* scale, void* y,
                                  int64_t M, int64_t N, int64_t K, void* ws, int64_t ws_bytes, emk_stream_t stream) {
  if (!h || !x || !w_e4m3 || !scale || !y) return EMK_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return EMK_ERR_SHAPE;
  if ((K % 16) != 0 || (N % 8) != 0) {
    EMK_SET_ERR(h, "emk_linear_bf16_w8: K must be a multiple of 16 and N of 8; got K=%lld N=%lld", (long long)K,
                (long long)N);
    return EMK_ERR_ALIGN;
  }
  if ((((uintptr_t)x | (uintptr_t)w_e4m3 | (uintptr_t)y | (uintptr_t)scale) & 15u) != 0) return EMK_ERR_ALIGN;
  if (ws != nullptr && M > W8_EXPAND_MIN_M) {
    // Many rows: every 128-row tile would convert the same weight tile again inside its main loop (M/128 times in
    // all). Expanding the weight once costs one pass over it at memory speed; the multiply then runs at bf16 rate.
    if (ws_bytes < N * K * 2) {
      EMK_SET_ERR(h, "emk_linear_bf16_w8: workspace of %lld bytes, %lld needed", (long long)ws_bytes,
                  (long long)(N * K * 2));
      return EMK_ERR_WORKSPACE;
    }
    if (((uintptr_t)ws & 31u) != 0) return EMK_ERR_ALIGN;
    const int64_t n16 = N * K / 16;
    int64_t blocks = (n16 + 255) / 256;
    if (blocks > (int64_t)h->sm_count * 16) blocks = (int64_t)h->sm_count * 16;
    expand_e4m3_bf16_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)w_e4m3, (uint32_t*)ws, n16);
    EMK_LAUNCH_CHECK(h);
    return emk_gemm_bf16_colscale_launch(h, x, ws, scale, y, M, N, K, (cudaStream_t)stream);
  }
  GemmArgs g = {};
  g.y = (__nv_bfloat16*)y;
  g.residual = nullptr;
  g.scale = scale;
  g.M = (int)M;
  g.N = (int)N;
  g.K = (int)K;
  g.ldy = (int)N;
  g.tiles_m = (int)((M + BM - 1) / BM);
  g.tiles_n = (int)((N + W8_BN - 1) / W8_BN);
  g.kblocks = (int)((K + BK - 1) / BK);
  g.epi = EMK_EPI_NONE;
  g.wide = ((N % 16) == 0 && ((uintptr_t)y & 31u) == 0) ? 1 : 0;
  g.status = h->status_dev;
  g.limit_ns = h->wait_limit_ns;
  CUtensorMap ta, tw;
  int rc = emk_make_tmap_2d(h, &ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2,
                            BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != EMK_OK) return rc;
  rc = emk_make_tmap_2d(h, &tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_e4m3, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK,
                        W8_BN, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != EMK_OK) return rc;
  static emk_device_once once;
  {
    std::lock_guard<std::mutex> lk(once.mu);
    if (!once.done[h->device]) {
      EMK_CUDA_TRY(h, cudaFuncSetAttribute(gemm_w8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W8_SMEM));
      once.done[h->device] = true;
    }
  }
  const int ntiles = g.tiles_m * g.tiles_n;
  const int grid = ntiles < h->sm_count ? ntiles : h->sm_count;
  gemm_w8_kernel<<<grid, W8_THREADS, W8_SMEM, (cudaStream_t)stream>>>(ta, tw, g);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}
