// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): two CTAs of a 2-CTA cluster compute one 256x256 output tile.
//
// Same contraction and epilogues as emk_gemm_sm100.cu (LinearOp / MatmulOp, emmy/compiler/ir/frontend/ir.py:202-237).
// Each CTA loads its own 128 rows of A and its own 128 columns (half) of the W tile, the leader CTA's single MMA thread
// issues 256x256x16 instructions that read A from each CTA's own shared memory and W halves from both, and each CTA's
// tensor memory receives the accumulator rows it owns. Per CTA and K-block that is 32 KB of operand traffic instead of
// 48 KB for the same math. A ring stage carries two 64-wide K slices (eight MMAs per barrier round trip): with one
// slice per stage the single MMA thread spent as long on waits and commits as the tensor core on the math.
//
//   warp 4      TMA producer (both CTAs; byte counts are credited to the LEADER's full barrier)
//   warp 5      MMA issuer (leader CTA only); tcgen05.commit arrives on the empty / tmem_full barriers of BOTH CTAs
//   warps 0..3, 6..9  epilogue (both CTAs, own accumulator rows; left / right half of the columns); arrive on the
//               leader's tmem_empty barrier
// No load uses cluster multicast. Every wait is bounded; the two cluster-wide barriers at start and end are reached by
// all threads of both CTAs on every path.
#include "emk_gemm_common.cuh"

#include <stdlib.h>

namespace {

using namespace emk;

constexpr int G2_THREADS = 320;  // warps 0-3 and 6-9: epilogue (left / right half of the tile's columns), 4: TMA, 5: MMA
constexpr int G2_GROUP_M = 8;  // row-tiles of 256 per raster group
constexpr int G2_MAX_STAGES = 8;

struct __align__(8) G2Barriers {
  uint64_t full[G2_MAX_STAGES];
  uint64_t empty[G2_MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// G2_BN: tile width (256 or 128 columns; each CTA loads half of them). A ring stage holds KSUB 64-wide K slices:
// KSUB x (16 KB of A + G2_BN/2 rows of W).
// EPI: the one epilogue this instantiation carries (EMK_EPI_*), or -1 for all of them chosen by the launch argument.
// FAST: whole tiles of 32-byte aligned rows only (no bounds tests, no narrow accesses in the epilogue).
template <int G2_BN, int G2_STAGES, int WL, int KSUB, int EPI, bool FAST>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                  const GemmArgs g) {
  constexpr int G2_HALF_N = G2_BN / 2;
  constexpr int G2_B_SUB_BYTES = G2_HALF_N * BK * 2;        // one 64-wide K slice of this CTA's W half
  constexpr int G2_A_STAGE = KSUB * A_STAGE_BYTES;          // a stage holds KSUB consecutive 64-wide K slices
  constexpr int G2_B_STAGE_BYTES = KSUB * G2_B_SUB_BYTES;
  constexpr uint32_t G2_STAGE_TX = 2u * (G2_A_STAGE + G2_B_STAGE_BYTES);  // both CTAs' bytes land on the leader barrier
  constexpr uint32_t G2_TMEM_COLS = (2 * G2_BN > 256) ? 512 : 256;
  constexpr uint32_t IDESC = make_idesc_bf16(2 * BM, G2_BN, 0, WL);
  static_assert(WL == 0 || G2_HALF_N % 64 == 0, "MN-major W needs whole 64-column chunks per CTA");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + G2_STAGES * G2_A_STAGE;
  G2Barriers* bars = reinterpret_cast<G2Barriers*>(sB + G2_STAGES * G2_B_STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const int ntiles = g.tiles_m * g.tiles_n;

  if (threadIdx.x == 0) {
    for (int i = 0; i < G2_STAGES; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 16);  // 8 epilogue warps of each CTA
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 0) {
    tmem_alloc_pair(&bars->tmem_base, G2_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  grid_dependency_wait();      // everything above overlaps the tail of the previous kernel in the stream
  grid_launch_dependents();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  const WaitCtx wc{&bars->abort_flag, g.status, g.limit_ns};

  if (warp == 4) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < ntiles && ok; tile += npairs) {
        int tm, tn;
        tile_coords(tile, g.tiles_m, g.tiles_n, G2_GROUP_M, tm, tn);
        const int m0 = tm * 2 * BM + (int)rank * BM;
        const int n0 = tn * G2_BN + (int)rank * G2_HALF_N;
        for (int kb = 0; kb < g.kblocks; kb += KSUB) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1u, wc, EMK_DEV_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = mapa_u32(smem_u32(&bars->full[stage]), 0);
          if (leader) mbar_arrive_expect_tx(&bars->full[stage], G2_STAGE_TX);
#pragma unroll
          for (int u = 0; u < KSUB; ++u) {  // slices past K are zero-filled by TMA and add nothing
            const int k0 = (kb + u) * BK;
            tma_load_2d_pair(sA + stage * G2_A_STAGE + u * A_STAGE_BYTES, &tma_a, full_leader, k0, m0);
            uint8_t* bdst = sB + stage * G2_B_STAGE_BYTES + u * G2_B_SUB_BYTES;
            if (WL == 0) {
              tma_load_2d_pair(bdst, &tma_b, full_leader, k0, n0);
            } else {
#pragma unroll
              for (int c = 0; c < G2_HALF_N / 64; ++c)
                tma_load_2d_pair(bdst + c * (BK * 128), &tma_b, full_leader, n0 + c * 64, k0);
            }
          }
          if (++stage == G2_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      // descriptor halves (see smem_desc_lo / smem_desc_hi): the low half advances by constants per K slice
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), 0);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), WL == 0 ? 0 : BK * 128);
      for (int tile = pair; tile < ntiles && ok; tile += npairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1u, wc, EMK_DEV_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * G2_BN);
        for (int kb = 0; kb < g.kblocks; kb += KSUB) {
          if (!mbar_wait(&bars->full[stage], phase, wc, EMK_DEV_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          // no tcgen05 fence here: the stage was written by TMA (async proxy) and the mbarrier wait orders it
          const uint32_t a_st = a_lo0 + (uint32_t)(stage * (G2_A_STAGE >> 4));
          const uint32_t b_st = b_lo0 + (uint32_t)(stage * (G2_B_STAGE_BYTES >> 4));
#pragma unroll
          for (int u = 0; u < KSUB; ++u) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint32_t a_lo = a_st + (uint32_t)((u * A_STAGE_BYTES + k * 32) >> 4);
              const uint32_t b_lo = b_st + (uint32_t)((u * G2_B_SUB_BYTES + (WL == 0 ? k * 32 : k * 16 * 128)) >> 4);
              umma_ss_pair_lohi(d_tmem, a_lo, b_lo, desc_hi, IDESC, (u | k) != 0 ? 1u : (uint32_t)(kb != 0));
            }
          }
          // release the stage in both CTAs (relaying the peer's release through the leader's producer thread was
          // measured 25 % slower: the peer's refills start late)
          const uint32_t e_local = smem_u32(&bars->empty[stage]);
          tc_commit_pair(e_local);
          tc_commit_pair(mapa_u32(e_local, 1));
          if (++stage == G2_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          const uint32_t f_local = smem_u32(&bars->tmem_full[acc]);
          tc_commit_pair(f_local);
          tc_commit_pair(mapa_u32(f_local, 1));
        }
      }
    }
  } else {
    // ---------------- epilogue: warps 0..3 drain the left half of the tile's columns, warps 6..9 the right half ------
    // (a warp may only touch the TMEM lanes of its quarter, warp_id % 4, so two warps share each quarter)
    const int quarter = warp & 3;
    const int half = warp >= 6 ? 1 : 0;
    int local = 0;
    for (int tile = pair; tile < ntiles; tile += npairs, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
      int tm, tn;
      tile_coords(tile, g.tiles_m, g.tiles_n, G2_GROUP_M, tm, tn);
      const int row = tm * 2 * BM + (int)rank * BM + quarter * 32 + lane;
      const int n0 = tn * G2_BN + half * (G2_BN / 2);
      epilogue_prefetch<EPI, FAST>(g, row, n0, G2_BN / 2);
      if (!mbar_wait_warp(&bars->tmem_full[acc], acc_phase, wc, EMK_DEV_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const uint32_t taddr =
          tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * G2_BN + half * (G2_BN / 2));
      epilogue_drain<G2_BN / 64, EPI, FAST>(g, taddr, row, n0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_relaxed(mapa_u32(smem_u32(&bars->tmem_empty[acc]), 0));
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (bars->abort_flag) abort_drain();
  cluster_sync_all();  // the peer's shared and tensor memory stay alive until the leader's MMAs are done
  if (warp == 0) tmem_dealloc_pair(tmem_base, G2_TMEM_COLS);
}

template <int G2_BN, int G2_STAGES, int WL, int KSUB, int EPI = -1, bool FAST = false>
int launch_gemm2(emk_handle_t h, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, cudaStream_t s) {
  constexpr int G2_SMEM = G2_STAGES * KSUB * (A_STAGE_BYTES + (G2_BN / 2) * BK * 2) + 1024 + (int)sizeof(G2Barriers);
  static emk_device_once once;
  static int max_pairs[EMK_MAX_DEVICES] = {0};
  auto kern = gemm2_bf16_kernel<G2_BN, G2_STAGES, WL, KSUB, EPI, FAST>;
  const int d = h->device;   // emk_create admits ordinals below EMK_MAX_DEVICES only
  std::unique_lock<std::mutex> lk(once.mu);
  if (!once.done[d]) {
    EMK_CUDA_TRY(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(h->sm_count & ~1), 1, 1);
    cfg.blockDim = dim3(G2_THREADS, 1, 1);
    cfg.dynamicSmemBytes = G2_SMEM;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int nclusters = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&nclusters, kern, &cfg);
    if (e != cudaSuccess || nclusters <= 0) {
      (void)cudaGetLastError();
      nclusters = h->sm_count / 2;
    }
    max_pairs[d] = nclusters < h->sm_count / 2 ? nclusters : h->sm_count / 2;
    once.done[d] = true;
  }
  const int pair_cap = max_pairs[d];
  lk.unlock();
  const int ntiles = g.tiles_m * g.tiles_n;
  const int pairs = ntiles < pair_cap ? ntiles : pair_cap;
  EMK_CUDA_TRY(h, launch_after_prologue(kern, 2u * (unsigned)pairs, G2_THREADS, G2_SMEM, s, h->overlap_launch != 0, ta, tb, g));
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

}  // namespace

// Called by the dispatcher in emk_gemm_sm100.cu. `g` arrives with tiles_m / tiles_n unset for this tiling.
int emk_gemm2_launch(emk_handle_t h, const void* x, const void* w, emk::GemmArgs g, int wlayout, cudaStream_t s) {
  // 256-column tiles whenever the output is wider than 128 columns: narrower tiles cost almost the same time per
  // K step (measured), so they only pay off when they avoid computing padding.
  const int bn = (g.N > 128 || g.epi == EMK_EPI_QKNORM_ROPE_INTERNAL) ? 256 : 128;
  g.tiles_m = (g.M + 2 * BM - 1) / (2 * BM);
  g.tiles_n = (g.N + bn - 1) / bn;
  CUtensorMap ta, tb;
  int rc = emk_make_tmap_2d(h, &ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)g.K, (uint64_t)g.M,
                            (uint64_t)g.K * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != EMK_OK) return rc;
  if (wlayout == EMK_W_NK) {
    rc = emk_make_tmap_2d(h, &tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, (uint64_t)g.K, (uint64_t)g.N,
                          (uint64_t)g.K * 2, BK, (uint32_t)(bn / 2), CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != EMK_OK) return rc;
    // two 64-wide K slices per ring stage: the per-stage barrier/commit work of the MMA thread is paid half as often
    if (bn == 256) {
      // the epilogues of the model path each have a kernel of their own (smaller code: see epi_of)
      const bool fast = (g.M % (2 * BM)) == 0 && (g.N % 256) == 0 && g.wide;
#define EMK_G2_CASE(E)                                                              \
  case E:                                                                           \
    return fast ? launch_gemm2<256, 3, 0, 2, E, true>(h, ta, tb, g, s)              \
                : launch_gemm2<256, 3, 0, 2, E, false>(h, ta, tb, g, s);
      switch (g.epi) {
        EMK_G2_CASE(EMK_EPI_NONE)
        EMK_G2_CASE(EMK_EPI_RESIDUAL)
        EMK_G2_CASE(EMK_EPI_SWIGLU)
        EMK_G2_CASE(EMK_EPI_QKNORM_ROPE_INTERNAL)
        default: return launch_gemm2<256, 3, 0, 2>(h, ta, tb, g, s);
      }
#undef EMK_G2_CASE
    }
    return launch_gemm2<128, 4, 0, 2>(h, ta, tb, g, s);
  }
  rc = emk_make_tmap_2d(h, &tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.N * 2,
                        64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != EMK_OK) return rc;
  if (bn == 256) return launch_gemm2<256, 3, 1, 2>(h, ta, tb, g, s);
  return launch_gemm2<128, 4, 1, 2>(h, ta, tb, g, s);
}
