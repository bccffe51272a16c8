// A chain of dependent bf16 GEMMs as ONE persistent launch on CTA pairs (tcgen05 cta_group::2, 256x256 tiles).
//
// A decoder layer is four projections in a row, each reading what the one before it wrote (o_proj -> gate/up -> down
// -> the next layer's QKV; LinearOp, emmy/compiler/ir/frontend/ir.py:202-217, with the epilogues the reference fuses
// around it). Launched one by one, each of them pays its own launch, pipeline fill, exposed last epilogue and partial
// last wave; with a few thousand rows per GPU (a batch sharded over eight GPUs) those fixed costs are a third of the
// time. Here the tiles of all phases form one list, walked round-robin by the CTA pairs:
//
//   * the list is phase after phase, and inside a phase the grouped raster of the single-GEMM kernel (groups of a few
//     256-row blocks by all column tiles), so the row blocks of a phase complete group by group and the next phase's
//     first tiles find their input ready;
//   * a tile of phase p > 0 reads, as its A operand, rows that phase p-1 wrote: its first A load waits until the
//     counter done[p-1][row block] has reached the number of CTA-level tile completions that make those rows final
//     (2 x column tiles of phase p-1); W loads do not wait. The gpu-scope acquire of that counter costs more than a
//     microsecond, so a watcher thread per CTA walks the CTA's tile list ahead of the TMA producer, does the acquire,
//     and publishes in shared memory how many tiles are clear; the producer only reads shared memory;
//   * a tile is complete when its epilogue warps have stored it: they arrive on a CTA-local barrier, and a separate
//     signalling thread then makes the stores visible (gpu-scope fence, cumulative over what it acquired from the
//     barrier) and bumps the counter — the epilogue warps themselves never wait for their stores;
//   * a pair that waits holds a tile whose inputs are earlier list entries, held by pairs that are running (the grid
//     never exceeds what the device holds at once): no cycle. Every wait is bounded like all others in this library.
//
// Residual and row-statistics reads of a phase may target rows another SM wrote earlier in the launch: they bypass L1
// (GemmArgs::coherent). The counters live in a caller-provided workspace that is zero before the first launch; the
// last CTA to leave the kernel zeroes them again, so launches (and CUDA-graph replays) can follow each other without
// host work. No load uses cluster multicast.
//
// Measured on the four projections of a Qwen3-0.6B layer (o_proj, gate/up, down, next QKV), chains launched back to
// back: 4096 rows 129 -> 120 us, 8192 rows 235 -> 208 us, 16384 rows 440 -> 425 us at the power-capped clock (at the
// burst clock 109 -> 105 us at 4096 rows); at 32768 rows the separate launches are 1-2 % faster (nothing left to hide,
// and the tracking costs a little). Inside the model, where an attention launch sits between two chains, the whole
// forward gains 1.5 % at 8192 rows, 1.8-3.3 % at 8192-16384 rows per rank in the multi-GPU bench, and LOSES 2-3 % at
// 4096 rows: the caller chains between 8192 and 16384 rows only. Asking every phase's weights into L2 at kernel start
// (cp.async.bulk.prefetch) changed nothing.
#include "emk_gemm_common.cuh"

int emk_gemm_desc_to_args(emk_handle_t h, const emk_gemm_desc_t* d, emk::GemmArgs* out);

namespace {

using namespace emk;

constexpr int CH_MAX = 4;
constexpr int CH_THREADS = 384;  // warps 0-3, 6-9: epilogue; 4: TMA; 5: MMA; 10: completion signalling; 11: dependency watcher
constexpr int CH_BN = 256;
constexpr int CH_STAGES = 3;
constexpr int CH_KSUB = 2;
constexpr int CH_HALF_N = CH_BN / 2;
constexpr int CH_B_SUB_BYTES = CH_HALF_N * BK * 2;
constexpr int CH_A_STAGE = CH_KSUB * A_STAGE_BYTES;
constexpr int CH_B_STAGE = CH_KSUB * CH_B_SUB_BYTES;
constexpr uint32_t CH_STAGE_TX = 2u * (CH_A_STAGE + CH_B_STAGE);
constexpr uint32_t CH_TMEM_COLS = 512;
constexpr uint32_t CH_IDESC = make_idesc_bf16(2 * BM, CH_BN, 0, 0);

struct __align__(64) ChainParams {
  CUtensorMap tma_a[CH_MAX];
  CUtensorMap tma_b[CH_MAX];
  GemmArgs g[CH_MAX];
  int tile_begin[CH_MAX + 1];  // first list index of each phase; tile_begin[n] = number of tiles
  int dep_target[CH_MAX];      // arrivals on done[p-1][row block] that make phase p's input rows final; 0: no wait
  int n;
  int row_blocks;              // 256-row blocks (the same for every phase)
  int group_m;                 // row blocks per raster group (tile_coords)
  int* done;                   // [CH_MAX][row_blocks], zero at launch
  int* exit_ticket;            // one counter, zero at launch
};

struct __align__(8) ChainBarriers {
  uint64_t full[CH_STAGES];
  uint64_t empty[CH_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t stored[2];    // this CTA's epilogue warps have stored the tile of accumulator slot acc
  uint64_t sig_done[2];  // the signalling thread has consumed stored[acc]
  uint32_t tmem_base;
  int abort_flag;
  int deps_ready;        // tiles of this CTA (in its list order) whose input rows the watcher has seen final
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until the shared-memory counter *c (written with release semantics by a thread of this CTA) >= target.
__device__ __forceinline__ bool smem_count_wait(const int* c, int target, const WaitCtx& w) {
  const uint32_t a = smem_u32(c);
  int v;
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  for (;;) {
    asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    if (v >= target) return true;
    if ((++spins & 0xffu) == 0) {
      if (*w.abort_flag) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > w.limit_ns) {
        *w.abort_flag = 1;
        *(volatile int*)w.status = EMK_DEV_TIMEOUT_DEPENDENCY;
        __threadfence_system();
        return false;
      }
    }
  }
}

// Bounded wait until *ctr >= target (same abort protocol as mbar_wait).
__device__ __forceinline__ bool dep_wait(const int* ctr, int target, const WaitCtx& w) {
  if (ld_acquire_gpu(ctr) >= target) return true;
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (ld_acquire_gpu(ctr) < target) {
    __nanosleep(64);
    if ((++spins & 0x3fu) == 0) {
      if (*w.abort_flag) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > w.limit_ns) {
        *w.abort_flag = 1;
        *(volatile int*)w.status = EMK_DEV_TIMEOUT_DEPENDENCY;
        __threadfence_system();
        return false;
      }
    }
  }
  return true;
}

// List index -> phase, row block, column tile.
__device__ __forceinline__ void chain_locate(const ChainParams& P, int t, int& p, int& tm, int& tn) {
  p = 0;
  while (p + 1 < P.n && t >= P.tile_begin[p + 1]) ++p;
  tile_coords(t - P.tile_begin[p], P.row_blocks, P.g[p].tiles_n, P.group_m, tm, tn);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(CH_THREADS, 1)
gemm2_chain_kernel(const __grid_constant__ ChainParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + CH_STAGES * CH_A_STAGE;
  ChainBarriers* bars = reinterpret_cast<ChainBarriers*>(sB + CH_STAGES * CH_B_STAGE);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const int total = P.tile_begin[P.n];

  if (threadIdx.x == 0) {
    for (int i = 0; i < CH_STAGES; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 16);  // 8 epilogue warps of each CTA
      mbar_init(&bars->stored[i], 8);       // this CTA's 8 epilogue warps
      mbar_init(&bars->sig_done[i], 1);
    }
    bars->abort_flag = 0;
    bars->deps_ready = 0;
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    for (int p = 0; p < P.n; ++p) {
      tma_prefetch_desc(&P.tma_a[p]);
      tma_prefetch_desc(&P.tma_b[p]);
    }
  }
  if (warp == 0) {
    tmem_alloc_pair(&bars->tmem_base, CH_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  grid_dependency_wait();
  grid_launch_dependents();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  const WaitCtx wc{&bars->abort_flag, P.g[0].status, P.g[0].limit_ns};

  if (warp == 4) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int t = pair; t < total && ok; t += npairs, ++local) {
        int p, tm, tn;
        chain_locate(P, t, p, tm, tn);
        const CUtensorMap* ta = &P.tma_a[p];
        const CUtensorMap* tb = &P.tma_b[p];
        const int kblocks = P.g[p].kblocks;
        const int m0 = tm * 2 * BM + (int)rank * BM;
        const int n0 = tn * CH_BN + (int)rank * CH_HALF_N;
        const int dep = P.dep_target[p];
        for (int kb = 0; kb < kblocks; kb += CH_KSUB) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1u, wc, EMK_DEV_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = mapa_u32(smem_u32(&bars->full[stage]), 0);
          if (leader) mbar_arrive_expect_tx(&bars->full[stage], CH_STAGE_TX);
          if (kb == 0 && dep > 0) {
            // The weights never depend on an earlier phase: they go first. The rows this tile reads were written by
            // phase p-1 of this launch, possibly by other SMs a moment ago.
#pragma unroll
            for (int u = 0; u < CH_KSUB; ++u)
              tma_load_2d_pair(sB + stage * CH_B_STAGE + u * CH_B_SUB_BYTES, tb, full_leader, (kb + u) * BK, n0);
            // The gpu-scope acquire of the counter costs more than a microsecond: the watcher thread (warp 11) does
            // it ahead of time and publishes, in shared memory, how many of this CTA's tiles have their input final.
            if (!smem_count_wait(&bars->deps_ready, local + 1, wc)) {
              ok = false;
              break;
            }
            // what the watcher acquired (generic proxy) before the TMA reads (async proxy). The global-only form:
            // the fence over all state spaces took a microsecond per tile (it waits for the copies in flight)
            fence_proxy_async_global();
#pragma unroll
            for (int u = 0; u < CH_KSUB; ++u)
              tma_load_2d_pair(sA + stage * CH_A_STAGE + u * A_STAGE_BYTES, ta, full_leader, (kb + u) * BK, m0);
          } else {
#pragma unroll
            for (int u = 0; u < CH_KSUB; ++u) {
              tma_load_2d_pair(sA + stage * CH_A_STAGE + u * A_STAGE_BYTES, ta, full_leader, (kb + u) * BK, m0);
              tma_load_2d_pair(sB + stage * CH_B_STAGE + u * CH_B_SUB_BYTES, tb, full_leader, (kb + u) * BK, n0);
            }
          }
          if (++stage == CH_STAGES) {
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
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), 0);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), 0);
      for (int t = pair; t < total && ok; t += npairs, ++local) {
        int p, tm, tn;
        chain_locate(P, t, p, tm, tn);
        const int kblocks = P.g[p].kblocks;
        const int acc = local & 1;
        const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1u, wc, EMK_DEV_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * CH_BN);
        for (int kb = 0; kb < kblocks; kb += CH_KSUB) {
          if (!mbar_wait(&bars->full[stage], phase, wc, EMK_DEV_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          const uint32_t a_st = a_lo0 + (uint32_t)(stage * (CH_A_STAGE >> 4));
          const uint32_t b_st = b_lo0 + (uint32_t)(stage * (CH_B_STAGE >> 4));
#pragma unroll
          for (int u = 0; u < CH_KSUB; ++u) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint32_t a_lo = a_st + (uint32_t)((u * A_STAGE_BYTES + k * 32) >> 4);
              const uint32_t b_lo = b_st + (uint32_t)((u * CH_B_SUB_BYTES + k * 32) >> 4);
              umma_ss_pair_lohi(d_tmem, a_lo, b_lo, desc_hi, CH_IDESC, (u | k) != 0 ? 1u : (uint32_t)(kb != 0));
            }
          }
          const uint32_t e_local = smem_u32(&bars->empty[stage]);
          tc_commit_pair(e_local);
          tc_commit_pair(mapa_u32(e_local, 1));
          if (++stage == CH_STAGES) {
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
  } else if (warp == 11) {
    // ---------------- dependency watcher (both CTAs, one thread) ----------------
    if (lane == 0 && P.n > 1) {
      int local = 0;
      for (int t = pair; t < total; t += npairs, ++local) {
        int p, tm, tn;
        chain_locate(P, t, p, tm, tn);
        const int dep = P.dep_target[p];
        if (dep > 0 && !dep_wait(P.done + (p - 1) * P.row_blocks + tm, dep, wc)) break;
        asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(smem_u32(&bars->deps_ready)), "r"(local + 1)
                     : "memory");
      }
    }
  } else if (warp == 10) {
    // ---------------- completion signalling (both CTAs, one thread) ----------------
    if (lane == 0 && P.n > 1) {
      int local = 0;
      for (int t = pair; t < total; t += npairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
        if (!mbar_wait(&bars->stored[acc], acc_phase, wc, EMK_DEV_TIMEOUT_EPILOGUE)) break;
        int p, tm, tn;
        chain_locate(P, t, p, tm, tn);
        if (p + 1 < P.n) {
          // The epilogue warps' stores were acquired through the barrier; the releasing reduction makes them visible
          // at gpu scope before the counter moves (release is cumulative), and it is this thread that waits for
          // them, not they. (A separate fence in front of it cost 1-2 % and adds nothing.)
          asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(P.done + p * P.row_blocks + tm) : "memory");
        }
        mbar_arrive(&bars->sig_done[acc]);
      }
    }
  } else {
    // ---------------- epilogue: warps 0..3 left half of the tile's columns, warps 6..9 right half ----------------
    const int quarter = warp & 3;
    const int half = warp >= 6 ? 1 : 0;
    int local = 0;
    for (int t = pair; t < total; t += npairs, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
      int p, tm, tn;
      chain_locate(P, t, p, tm, tn);
      const int row = tm * 2 * BM + (int)rank * BM + quarter * 32 + lane;
      const int n0 = tn * CH_BN + half * (CH_BN / 2);
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * CH_BN + half * (CH_BN / 2));
      bool ok = true;
      const GemmArgs g = P.g[p];  // a local copy: the fields the epilogue uses become registers
      epilogue_prefetch<EMK_EPI_SET_LAYER>(g, row, n0, CH_BN / 2);
      ok = mbar_wait_warp(&bars->tmem_full[acc], acc_phase, wc, EMK_DEV_TIMEOUT_EPILOGUE);
      if (ok) {
        tc_fence_after();
        epilogue_drain<CH_BN / 64, EMK_EPI_SET_LAYER>(g, taddr, row, n0);
      }
      if (!ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_relaxed(mapa_u32(smem_u32(&bars->tmem_empty[acc]), 0));
      // stored[acc] is reused every second tile: the signalling thread must have consumed its previous phase
      if (P.n > 1) {
        if (local >= 2 &&
            !mbar_wait_warp(&bars->sig_done[acc], ((uint32_t)(local >> 1) - 1u) & 1u, wc, EMK_DEV_TIMEOUT_EPILOGUE))
          break;
        if (lane == 0) mbar_arrive(&bars->stored[acc]);  // releasing, CTA scope: orders this warp's stores before it
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  const bool aborted = bars->abort_flag != 0;
  if (aborted) abort_drain();
  cluster_sync_all();
  if (warp == 0) tmem_dealloc_pair(tmem_base, CH_TMEM_COLS);
  // The last CTA to get here zeroes the counters for the next launch: every reader of them has finished.
  if (threadIdx.x == 0 && !aborted && P.n > 1) {
    __threadfence();
    const int old = atomicAdd(P.exit_ticket, 1);
    if (old == (int)gridDim.x - 1) {
      for (int i = 0; i < P.n * P.row_blocks; ++i) P.done[i] = 0;
      *P.exit_ticket = 0;
    }
  }
}

constexpr int CH_SMEM = CH_STAGES * (CH_A_STAGE + CH_B_STAGE) + 1024 + (int)sizeof(ChainBarriers);

int64_t chain_workspace_ints(int64_t M) { return CH_MAX * ((M + 2 * BM - 1) / (2 * BM)) + 16; }

}  // namespace

extern "C" int64_t emk_gemm_bf16_chain_workspace_bytes(int64_t M) {
  if (M <= 0) return 0;
  return chain_workspace_ints(M) * (int64_t)sizeof(int);
}

extern "C" int emk_gemm_bf16_chain(emk_handle_t h, const emk_gemm_desc_t* descs, int n, void* workspace,
                                   int64_t workspace_bytes, emk_stream_t stream) {
  if (!h || !descs || !workspace) return EMK_ERR_ARG;
  if (n < 1 || n > CH_MAX) {
    EMK_SET_ERR(h, "emk_gemm_bf16_chain: 1 to %d phases, got %d", CH_MAX, n);
    return EMK_ERR_ARG;
  }
  const int64_t M = descs[0].M;
  if (workspace_bytes < emk_gemm_bf16_chain_workspace_bytes(M) || ((uintptr_t)workspace & 15u) != 0) {
    EMK_SET_ERR(h, "emk_gemm_bf16_chain: workspace of %lld bytes (16-byte aligned), %lld needed",
                (long long)workspace_bytes, (long long)emk_gemm_bf16_chain_workspace_bytes(M));
    return EMK_ERR_WORKSPACE;
  }
  static ChainParams P;  // filled under the lock below, copied into the launch
  static std::mutex mu;
  static emk_device_once once;
  static int max_pairs[EMK_MAX_DEVICES] = {0};
  std::unique_lock<std::mutex> lk(mu);
  memset(&P, 0, sizeof(P));
  P.n = n;
  P.row_blocks = (int)((M + 2 * BM - 1) / (2 * BM));
  P.group_m = h->chain_group_m;
  P.done = (int*)workspace;
  P.exit_ticket = P.done + CH_MAX * P.row_blocks;
  int tiles = 0;
  for (int p = 0; p < n; ++p) {
    const emk_gemm_desc_t& d = descs[p];
    if (d.M != M || d.wlayout != EMK_W_NK || d.N <= 128) {
      EMK_SET_ERR(h, "emk_gemm_bf16_chain: phase %d: every phase needs the same M, W [N,K] and N > 128", p);
      return EMK_ERR_SHAPE;
    }
    if (p > 0) {
      const emk_gemm_desc_t& q = descs[p - 1];
      const int64_t prev_cols = q.epilogue == EMK_EPI_SWIGLU ? q.N / 2 : q.N;
      if (d.x != q.y || d.K != prev_cols) {
        EMK_SET_ERR(h, "emk_gemm_bf16_chain: phase %d must read the output of phase %d (x == y, K == its columns)", p,
                    p - 1);
        return EMK_ERR_ARG;
      }
    }
    GemmArgs& g = P.g[p];
    int rc = emk_gemm_desc_to_args(h, &d, &g);
    if (rc != EMK_OK) return rc;
    if (g.epi != EMK_EPI_RESIDUAL && g.epi != EMK_EPI_SWIGLU && g.epi != EMK_EPI_QKNORM_ROPE_INTERNAL) {
      EMK_SET_ERR(h, "emk_gemm_bf16_chain: phase %d: the chain kernel carries the residual, SwiGLU and q/k-norm + RoPE "
                  "epilogues only", p);
      return EMK_ERR_ARG;
    }
    g.coherent = 1;
    g.tiles_m = P.row_blocks;
    g.tiles_n = (int)((d.N + CH_BN - 1) / CH_BN);
    rc = emk_make_tmap_2d(h, &P.tma_a[p], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d.x, (uint64_t)d.K, (uint64_t)d.M,
                          (uint64_t)d.K * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != EMK_OK) return rc;
    rc = emk_make_tmap_2d(h, &P.tma_b[p], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d.w, (uint64_t)d.K, (uint64_t)d.N,
                          (uint64_t)d.K * 2, BK, (uint32_t)CH_HALF_N, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != EMK_OK) return rc;
    P.tile_begin[p] = tiles;
    tiles += g.tiles_m * g.tiles_n;
    P.dep_target[p] = p > 0 ? 2 * P.g[p - 1].tiles_n : 0;
  }
  for (int p = n; p <= CH_MAX; ++p) P.tile_begin[p] = tiles;

  auto kern = gemm2_chain_kernel;
  const int dv = h->device;
  if (!once.done[dv]) {
    EMK_CUDA_TRY(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CH_SMEM));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(h->sm_count & ~1), 1, 1);
    cfg.blockDim = dim3(CH_THREADS, 1, 1);
    cfg.dynamicSmemBytes = CH_SMEM;
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
    max_pairs[dv] = nclusters < h->sm_count / 2 ? nclusters : h->sm_count / 2;
    once.done[dv] = true;
  }
  // Every pair must be resident for the dependency waits to be safe: never more pairs than the device holds at once.
  const int pairs = tiles < max_pairs[dv] ? tiles : max_pairs[dv];
  // Launched WITHOUT programmatic dependent launch: with it the 16 x 512 forward measured 1.5-2 % slower (the chain's
  // CTAs that become resident early only spin until the attention kernel before them has drained).
  EMK_CUDA_TRY(h, launch_after_prologue(kern, 2u * (unsigned)pairs, CH_THREADS, CH_SMEM, (cudaStream_t)stream,
                                        false, P));
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}
