// bf16 GEMM on the 5th-generation tensor cores: y[M,N] = x[M,K] · W (+ fused epilogue), fp32 accumulation in tensor
// memory (TMEM), operands streamed by TMA into a 128-byte-swizzled shared-memory ring.
//
// Reference behaviour: LinearOp / MatmulOp (emmy/compiler/ir/frontend/ir.py:202-237), decomposed by
// emmy/compiler/pipeline/passes/frontend/decomposition/040_linear.py:16-43, scheduled as 128x128x16 mma.sync tiles
// with a 4-slot unswizzled TMA ring and a CTA-wide barrier every K step
// (emmy/compiler/pipeline/passes/lowering/tile/_schedule.py:735, lowering/kernel/_atom.py:598-715, _stage.py:345-450).
//
// This kernel instead is persistent (one CTA per SM, tiles strided over the grid) and warp-specialised:
//   warp 4      TMA producer: fills the ring, one mbarrier per slot counts the landed bytes
//   warp 5      MMA issuer: one thread issues tcgen05.mma 128xBNx16 per 16-wide K slice, commits slot release
//   warps 0..3  epilogue: tcgen05.ld the finished accumulator (thread = output row), apply the fused epilogue,
//               store bf16. Two accumulators live in TMEM so the epilogue of tile i overlaps the main loop of i+1.
// Every wait is bounded (emk::mbar_wait); after an expiry all roles fall through to the common teardown.
#include "emk_gemm_common.cuh"

int emk_gemm2_launch(emk_handle_t h, const void* x, const void* w, emk::GemmArgs g, int wlayout, cudaStream_t s);

namespace {

using namespace emk;

constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 16;

struct __align__(8) GemmBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// WL = 0: W is [N,K] (K contiguous, K-major B operand); WL = 1: W is [K,N] (N contiguous, MN-major B operand).
template <int BN, int STAGES, int WL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmArgs g) {
  constexpr int B_STAGE_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_TX = A_STAGE_BYTES + B_STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t IDESC = make_idesc_bf16(BM, BN, 0, WL);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(sB + STAGES * B_STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int ntiles = g.tiles_m * g.tiles_n;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&bars->full[i], 1);
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
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
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
        tile_coords(tile, g.tiles_m, g.tiles_n, GROUP_M, tm, tn);
        const int m0 = tm * BM;
        const int n0 = tn * BN;
        for (int kb = 0; kb < g.kblocks; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1u, wc, EMK_DEV_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&bars->full[stage], STAGE_TX);
          tma_load_2d(sA + stage * A_STAGE_BYTES, &tma_a, &bars->full[stage], kb * BK, m0);
          if (WL == 0) {
            tma_load_2d(sB + stage * B_STAGE_BYTES, &tma_b, &bars->full[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + stage * B_STAGE_BYTES + c * (BK * 128), &tma_b, &bars->full[stage], n0 + c * 64,
                          kb * BK);
          }
          if (++stage == STAGES) {
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
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < g.kblocks; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, wc, EMK_DEV_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = make_smem_desc(a_addr + k * 32, 0, 1024);
            const uint64_t bdesc = (WL == 0) ? make_smem_desc(b_addr + k * 32, 0, 1024)
                                             : make_smem_desc(b_addr + k * 16 * 128, BK * 128, 1024);
            umma_ss(d_tmem, adesc, bdesc, IDESC, (uint32_t)((kb | k) != 0));
          }
          tc_commit(&bars->empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(&bars->tmem_full[acc]);
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
      tile_coords(tile, g.tiles_m, g.tiles_n, GROUP_M, tm, tn);
      const int m0 = tm * BM;
      const int n0 = tn * BN;
      const int row = m0 + warp * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(acc * BN);
epilogue_drain<BN / 32>(g, taddr, row, n0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_relaxed(&bars->tmem_empty[acc]);
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (bars->abort_flag) abort_drain();
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int BN, int STAGES, int WL>
int launch_gemm(emk_handle_t h, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, cudaStream_t s) {
  constexpr int SMEM = STAGES * (A_STAGE_BYTES + BN * BK * 2) + 1024 + (int)sizeof(GemmBarriers);
  static emk_device_once once;
  auto kern = gemm_bf16_kernel<BN, STAGES, WL>;
  {
    std::lock_guard<std::mutex> lk(once.mu);
    if (!once.done[h->device]) {
      EMK_CUDA_TRY(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
      once.done[h->device] = true;
    }
  }
  const int ntiles = g.tiles_m * g.tiles_n;
  const int grid = ntiles < h->sm_count ? ntiles : h->sm_count;
  kern<<<grid, GEMM_THREADS, SMEM, s>>>(ta, tb, g);
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

struct QkRopeArgs {
  const void *qw, *kw, *rope;
  int S, Hq, Hkv;
  float eps;
  const int* pos;
};

struct RowStatArgs {
  const float* ss_in;
  int in_segs;
  float inv_dim, eps;
  float* ss_out;
};

int gemm_dispatch(emk_handle_t h, const void* x, const void* w, const void* residual, const float* scale, void* y,
                  int64_t M, int64_t N, int64_t K, int wlayout, int epilogue, cudaStream_t s,
                  const QkRopeArgs* qk = nullptr, const RowStatArgs* rsx = nullptr, bool f32_out = false,
                  const float* f32_bias = nullptr, GemmArgs* args_only = nullptr) {
  // args_only: validate and fill the kernel arguments (tiling left to the caller) without launching anything
  if (!h || !x || !w || !y) return EMK_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return EMK_ERR_SHAPE;
  if (wlayout != EMK_W_NK && wlayout != EMK_W_KN) return EMK_ERR_ARG;
  if (epilogue < EMK_EPI_NONE || epilogue > EMK_EPI_BIAS) return EMK_ERR_ARG;
  if ((epilogue == EMK_EPI_RESIDUAL || epilogue == EMK_EPI_BIAS) && !residual) return EMK_ERR_ARG;
  if ((K % 8) != 0 || (N % 8) != 0 || (epilogue == EMK_EPI_SWIGLU && (N % 16) != 0)) {
    EMK_SET_ERR(h, "emk_linear_bf16: K and N must be multiples of 8 (16 for the SwiGLU epilogue); got K=%lld N=%lld",
                (long long)K, (long long)N);
    return EMK_ERR_ALIGN;
  }
  if ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)residual | (uintptr_t)scale) & 15u) != 0) {
    EMK_SET_ERR(h, "emk_linear_bf16: operands must be 16-byte aligned");
    return EMK_ERR_ALIGN;
  }
  // Few output tiles (the fp32-output route runs a 6x longer K loop over small M x N): 128-wide single-CTA tiles
  // put more SMs to work than 256-wide ones.
  const bool narrow = f32_out && ((M + BM - 1) / BM) * ((N + 255) / 256) < h->sm_count / 2;
  const int BN = (N > 128 && !narrow) ? 256 : 128;
  GemmArgs g = {};
  g.y = (__nv_bfloat16*)y;
  g.residual = (const __nv_bfloat16*)residual;
  g.scale = scale;
  g.M = (int)M;
  g.N = (int)N;
  g.K = (int)K;
  g.ldy = (epilogue == EMK_EPI_SWIGLU) ? (int)(N / 2) : (int)N;
  g.tiles_m = (int)((M + BM - 1) / BM);
  g.tiles_n = (int)((N + BN - 1) / BN);
  g.kblocks = (int)((K + BK - 1) / BK);
  g.epi = epilogue;
  g.wide = ((g.ldy % 16) == 0 && ((uintptr_t)y & 31u) == 0 && ((uintptr_t)residual & 31u) == 0) ? 1 : 0;
  g.status = h->status_dev;
  g.limit_ns = h->wait_limit_ns;

  if (rsx) {
    g.ss_in = rsx->ss_in;
    g.ss_in_segs = rsx->in_segs;
    g.ss_inv_dim = rsx->inv_dim;
    g.ss_eps = rsx->eps;
    g.ss_out = rsx->ss_out;
  }
  g.qk_qw = g.qk_kw = g.qk_rope = nullptr;
  g.qk_pos = nullptr;
  g.f32_bias = nullptr;
  if (f32_out) {
    if ((((uintptr_t)y | (uintptr_t)f32_bias) & 15u) != 0) return EMK_ERR_ALIGN;
    g.epi = EMK_EPI_F32_INTERNAL;
    g.f32_bias = f32_bias;
  }
  g.qk_S = g.qk_Hq = g.qk_Hkv = 0;
  g.qk_eps = 0.f;
  if (qk) {  // fused q/k-norm + RoPE epilogue: 256-column CTA-pair tiles only (two whole heads per tile)
    g.epi = EMK_EPI_QKNORM_ROPE_INTERNAL;
    g.qk_qw = (const __nv_bfloat16*)qk->qw;
    g.qk_kw = (const __nv_bfloat16*)qk->kw;
    g.qk_rope = (const __nv_bfloat16*)qk->rope;
    g.qk_S = qk->S;
    g.qk_Hq = qk->Hq;
    g.qk_Hkv = qk->Hkv;
    g.qk_eps = qk->eps;
    g.qk_pos = qk->pos;
    if (args_only) {
      *args_only = g;
      return EMK_OK;
    }
    return emk_gemm2_launch(h, x, w, g, wlayout, s);
  }
  if (args_only) {
    *args_only = g;
    return EMK_OK;
  }
  // CTA-pair tiles (256x256) when the problem has at least one full pair tile; single-CTA tiles otherwise.
  const bool pair_ok = M > BM && N > 128 && !narrow;
  // The pair kernel's 128-wide tiles give each epilogue thread 64 columns, half of a row_sumsq_out slot: two threads
  // would write one slot. Such outputs (N <= 128) always take the single-CTA kernel, whose threads own whole slots.
  const bool pair_forced = h->gemm_impl == 2 && !(g.ss_out != nullptr && N <= 128);
  if (pair_forced || (h->gemm_impl == 0 && pair_ok)) return emk_gemm2_launch(h, x, w, g, wlayout, s);

  CUtensorMap ta, tb;
  int rc = emk_make_tmap_2d(h, &ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2,
                            BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != EMK_OK) return rc;
  if (wlayout == EMK_W_NK) {
    rc = emk_make_tmap_2d(h, &tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2,
                          BK, (uint32_t)BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != EMK_OK) return rc;
    return BN == 256 ? launch_gemm<256, 4, 0>(h, ta, tb, g, s) : launch_gemm<128, 6, 0>(h, ta, tb, g, s);
  }
  rc = emk_make_tmap_2d(h, &tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, (uint64_t)N, (uint64_t)K, (uint64_t)N * 2, 64,
                        BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != EMK_OK) return rc;
  return BN == 256 ? launch_gemm<256, 4, 1>(h, ta, tb, g, s) : launch_gemm<128, 6, 1>(h, ta, tb, g, s);
}

}  // namespace

// y = bf16(scale[n] * x·Wᵀ) with bf16 W [N,K]: the second step of the expand-then-multiply path of the e4m3 linear.
int emk_gemm_bf16_colscale_launch(emk_handle_t h, const void* x, const void* w, const float* scale, void* y, int64_t M,
                                  int64_t N, int64_t K, cudaStream_t s) {
  return gemm_dispatch(h, x, w, nullptr, scale, y, M, N, K, EMK_W_NK, EMK_EPI_NONE, s);
}


// y (fp32 [M,N]) = x·W (+ bias) with bf16 operands and the unrounded fp32 accumulator stored: the multiply step of
// the split-operand fp32 linear (emk_gemm_f32_split.cu).
int emk_gemm_bf16_f32out_launch(emk_handle_t h, const void* x, const void* w, const float* bias, float* y, int64_t M,
                                int64_t N, int64_t K, int wlayout, cudaStream_t s) {
  return gemm_dispatch(h, x, w, nullptr, nullptr, y, M, N, K, wlayout, EMK_EPI_NONE, s, nullptr, nullptr, true, bias);
}

extern "C" int emk_linear_bf16(emk_handle_t h, const void* x, const void* w, const void* residual, void* y, int64_t M,
                               int64_t N, int64_t K, int wlayout, int epilogue, emk_stream_t stream) {
  return gemm_dispatch(h, x, w, residual, nullptr, y, M, N, K, wlayout, epilogue, (cudaStream_t)stream);
}

extern "C" int emk_linear_bf16_qknorm_rope(emk_handle_t h, const void* x, const void* w, void* y, int64_t M, int64_t N,
                                           int64_t K, const void* qw, const void* kw, const void* rope_chunk_major,
                                           int64_t S, int64_t Hq, int64_t Hkv, float eps, emk_stream_t stream) {
  emk_gemm_desc_t d;
  memset(&d, 0, sizeof(d));
  d.x = x; d.w = w; d.y = y; d.M = M; d.N = N; d.K = K;
  d.wlayout = EMK_W_NK; d.epilogue = EMK_EPI_QKNORM_ROPE;
  d.q_norm_weight = qw; d.k_norm_weight = kw; d.rope_chunk_major = rope_chunk_major;
  d.seq_len = S; d.num_q_heads = Hq; d.num_kv_heads = Hkv; d.qk_eps = eps;
  return emk_gemm_bf16_fused(h, &d, stream);
}

namespace {
int gemm_fused_impl(emk_handle_t h, const emk_gemm_desc_t* d, cudaStream_t s, GemmArgs* args_only) {
  if (!h || !d) return EMK_ERR_ARG;
  if (d->row_sumsq_in && (d->norm_dim <= 0 || d->norm_dim % 128 != 0)) {
    EMK_SET_ERR(h, "row_sumsq_in needs norm_dim > 0 and a multiple of 128 (one partial slot per 128 columns)");
    return EMK_ERR_ARG;
  }
  RowStatArgs rs{d->row_sumsq_in, d->row_sumsq_in ? (int)(d->norm_dim / 128) : 0,
                 d->row_sumsq_in ? 1.0f / (float)d->norm_dim : 0.f, d->norm_eps, d->row_sumsq_out};
  const bool any_rs = d->row_sumsq_in || d->row_sumsq_out;
  if (d->row_sumsq_out && d->epilogue != EMK_EPI_RESIDUAL && d->epilogue != EMK_EPI_NONE && d->epilogue != EMK_EPI_BIAS) {
    EMK_SET_ERR(h, "row_sumsq_out is produced by the none / residual / bias epilogues only");
    return EMK_ERR_ARG;
  }
  if (d->epilogue == EMK_EPI_QKNORM_ROPE) {
    if (!d->x || !d->w || !d->y || !d->q_norm_weight || !d->k_norm_weight || !d->rope_chunk_major) return EMK_ERR_ARG;
    const int64_t S = d->seq_len, Hq = d->num_q_heads, Hkv = d->num_kv_heads;
    if (S <= 0 || Hq <= 0 || Hkv <= 0 || d->N != (Hq + 2 * Hkv) * 128 || (!d->positions && d->M % S != 0) ||
        d->wlayout != EMK_W_NK) {
      EMK_SET_ERR(h, "q/k-norm + RoPE epilogue: N must be (Hq + 2*Hkv)*128, M a multiple of seq_len (unless "
                  "positions are given), W [N,K]");
      return EMK_ERR_SHAPE;
    }
    if ((((uintptr_t)d->q_norm_weight | (uintptr_t)d->k_norm_weight) & 15u) != 0 ||
        (((uintptr_t)d->y | (uintptr_t)d->rope_chunk_major) & 31u) != 0)
      return EMK_ERR_ALIGN;
    QkRopeArgs qk{d->q_norm_weight, d->k_norm_weight, d->rope_chunk_major, (int)S, (int)Hq, (int)Hkv, d->qk_eps,
                  d->positions};
    return gemm_dispatch(h, d->x, d->w, nullptr, nullptr, d->y, d->M, d->N, d->K, EMK_W_NK, EMK_EPI_NONE, s, &qk,
                         any_rs ? &rs : nullptr, false, nullptr, args_only);
  }
  return gemm_dispatch(h, d->x, d->w, d->residual, nullptr, d->y, d->M, d->N, d->K, d->wlayout, d->epilogue, s, nullptr,
                       any_rs ? &rs : nullptr, false, nullptr, args_only);
}
}  // namespace

extern "C" int emk_gemm_bf16_fused(emk_handle_t h, const emk_gemm_desc_t* d, emk_stream_t stream) {
  return gemm_fused_impl(h, d, (cudaStream_t)stream, nullptr);
}

// The kernel arguments emk_gemm_bf16_fused would launch with (same validation), for callers that schedule the tiles
// themselves (the GEMM chain).
int emk_gemm_desc_to_args(emk_handle_t h, const emk_gemm_desc_t* d, emk::GemmArgs* out) {
  return gemm_fused_impl(h, d, nullptr, out);
}
