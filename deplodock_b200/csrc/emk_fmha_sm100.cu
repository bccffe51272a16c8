// Causal grouped-query flash attention on tcgen05 tensor cores, bf16 operands, head_dim 128, fp32 online softmax.
//
// Reference behaviour: SdpaOp (emmy/compiler/ir/frontend/ir.py:241-275) decomposed by
// emmy/compiler/pipeline/passes/frontend/decomposition/010_sdpa.py:52-141 (Kᵀ, GQA head h -> h / group, scale
// 1/sqrt(D), causal mask, softmax, PV) and lowered as a one-warp-per-16-rows mma.sync flash kernel
// (emmy/compiler/pipeline/passes/lowering/kernel/_twist.py:229) that re-reads Q and K fragments from global memory
// every 16 keys, never skips masked tiles and does not share K/V between the query heads of a group.
//
// Here one persistent CTA per SM walks a list of work items; an item is 128 query rows of TWO query heads that share
// a KV head (two 128x128 tiles, "ping-pong"). Four warpgroups, registers moved between them with setmaxnreg:
//   warps 0..3   softmax of tile 0 (thread = query row: no shuffles for row max / row sum), 192 registers
//   warps 4..7   softmax of tile 1
//   warps 8..11  epilogue of both tiles: O / row sum -> bf16 -> 128-byte-swizzled staging -> TMA store, so the
//                softmax warps go straight on to the next item
//   warp 12      TMA producer: one Q tile per head (own barriers, so a head's Q is replaced as soon as its last S is
//                done), then a 2-slot ring of K tiles and a 2-slot ring of V tiles with separate release: a K slot
//                comes free when its S products are done, so the next-but-one K block is on its way a whole block
//                before it is needed (with a joint release the load latency sat on the critical path whenever K/V
//                came from DRAM, as with many short sequences)
//   warp 13      MMA issuer: S = Q·Kᵀ (both operands from shared memory) and O += P·V (P from tensor memory,
//                V from shared memory as an MN-major operand); the first S of the next item is issued right behind
//                the last PV of the current one, so the pipeline does not drain between items
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; the bf16 probabilities P overwrite the
// first 64 columns of their S tile. While the tensor core works on one tile the softmax warps work on the other.
// Only KV blocks at or below the diagonal are visited; items are ordered so that the query blocks that read the same
// K/V run at about the same time (L2 reuse) and every CTA gets about the same number of KV blocks; O is rescaled
// lazily (only when the running max grows by more than 2^8), so most iterations never touch O.
// Measured dead ends, kept out: two threads per query row (the two warps share a scheduler, 2x slower); blocks of 64
// keys with two S buffers per tile (N=64 MMAs and the doubled per-block overheads, 1.6x slower); polynomial exp2 on
// the FMA pipe for part of the row (no gain: issue slots, not the MUFU pipe, bound the row pass).
// Every mbarrier wait is bounded; after an expiry all roles fall through to the common teardown.
#include "emk_common.cuh"

#include <math_constants.h>

namespace {

using namespace emk;

constexpr int FM = 128;   // query rows per tile
constexpr int FN = 128;   // keys per KV block
constexpr int HD = 128;   // head dim
constexpr int FMHA_THREADS = 512;  // four warpgroups: softmax tile 0, softmax tile 1, epilogue, {TMA, MMA, 2 idle}
constexpr int EPI_WARP0 = 8, TMA_WARP = 12, MMA_WARP = 13;
constexpr int TILE_BYTES = FM * HD * 2;   // 32 KB: two 64-column halves of 16 KB
constexpr int HALF_BYTES = FM * 64 * 2;   // 16 KB
constexpr int KV_STAGES = 2;
constexpr int OSTAGE_BYTES = 32 * 64 * 2;  // per softmax warp: 32 rows x 64 bf16 columns, 128-byte swizzled rows
constexpr uint32_t IDESC_S = make_idesc_bf16(FM, FN, 0, 0);
constexpr uint32_t IDESC_PV = make_idesc_bf16(FM, HD, 0, 1);
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

struct FmhaArgs {
  __nv_bfloat16* o;
  int B, Hq, Hkv, S, group, pairs;
  int nqblk;
  int n_items, n_rounds;
  int gp;  // (batch, KV head, head pair) triples per scheduling group
  // coordinates: x = h * cs + 64 * half, y = b * rb + h * rh + s  (q side indexed by query head, kv side by KV head)
  int q_cs, q_rb, q_rh;
  int kv_cs, kv_rb, kv_rh;
  int o_cs, o_rb, o_rh;
  int64_t ld_o;
  float scale_log2;
  int* status;
  unsigned long long limit_ns;
  // packed variable-length mode: one entry per 128-row query block of every sequence, heaviest first, written by
  // varlen_items_kernel into the caller's workspace: {first token row of the sequence, q0 within it, its length, 0};
  // n_entries[0] holds their number. Null in the fixed-length modes.
  const int4* vl_items;
  const int* vl_n_entries;
};

struct __align__(8) FmhaBarriers {
  uint64_t q_full[2], q_empty[2];   // one Q tile per query head of the item
  uint64_t k_full[KV_STAGES], v_full[KV_STAGES];
  uint64_t k_empty[KV_STAGES], v_empty[KV_STAGES];  // a K tile is free once its S products are done, a block earlier
                                                    // than the V tile of the same block (free after its PV products)
  uint64_t s_full[2], p_full[2], l_ready[2], o_done[2], o_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  float row_l[2][FM];   // row sums of the finished item, softmax warps -> epilogue warps
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Packed fp32 pairs (two lanes per instruction on the FMA pipe).
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b,
                                                        unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// One unit of work: 128 query rows of the (up to) two query heads `hq0`, `hq0 + 1` that share KV head `hkv`.
struct WorkItem {
  int b, hkv, hq0, q0, nblk;
  int row0;   // token-row offset of the item's sequence (packed mode; 0 otherwise)
  int slen;   // length of the item's sequence
  bool two;
};

// Number of work items and of rounds over the grid; fixed at launch, or read from the item table in packed mode.
struct Sched {
  int n_items, n_rounds;
};

// Items are numbered heaviest query block first and dealt to the CTAs in boustrophedon order (round r left to right,
// round r+1 right to left), which evens out the causal triangle: every CTA gets about the same number of KV blocks.
__device__ __forceinline__ int item_of_round(int round, int cta, int grid) {
  return round * grid + ((round & 1) ? (grid - 1 - cta) : cta);
}

__device__ __forceinline__ WorkItem decode_item(const FmhaArgs& a, int w) {
  WorkItem it;
  if (a.vl_items != nullptr) {
    // packed mode: entries are ordered heaviest query block first; the (KV head, head pair) combinations of an entry
    // are consecutive items, so they run at the same time on neighbouring SMs and share the sequence's K/V in L2
    const int per_entry = a.Hkv * a.pairs;
    const int e = w / per_entry;
    int rem = w - e * per_entry;
    const int4 ent = __ldg(a.vl_items + e);
    const int pair = rem % a.pairs;
    it.hkv = rem / a.pairs;
    it.b = 0;
    it.hq0 = it.hkv * a.group + 2 * pair;
    it.two = (2 * pair + 1) < a.group;
    it.row0 = ent.x;
    it.q0 = ent.y;
    it.slen = ent.z;
    it.nblk = ent.y / FM + 1;
    return it;
  }
  it.row0 = 0;
  it.slen = a.S;
  // (batch, KV head, head pair) triples are taken `a.gp` at a time; within such a group the query blocks go heaviest
  // first. Items that read the same K/V blocks then run at about the same time on different SMs, so all but the
  // first read hit in L2; with one group (small K/V) this is plain heaviest-first order.
  const int per_qblk = a.B * a.Hkv * a.pairs;
  const int g = w / (a.gp * a.nqblk);
  const int r = w - g * a.gp * a.nqblk;
  const int gl = min(a.gp, per_qblk - g * a.gp);
  const int qblk = a.nqblk - 1 - r / gl;
  int rem = g * a.gp + r % gl;
  const int pair = rem % a.pairs;
  rem /= a.pairs;
  it.hkv = rem % a.Hkv;
  it.b = rem / a.Hkv;
  it.hq0 = it.hkv * a.group + 2 * pair;
  it.two = (2 * pair + 1) < a.group;
  it.q0 = qblk * FM;
  it.nblk = qblk + 1;  // KV blocks 0..qblk (FM == FN)
  return it;
}

template <int N>
__device__ __forceinline__ void reg_grow() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_shrink() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// Work items of this CTA in order: the item of the first round >= `rnd` that exists; returns false past the end.
__device__ __forceinline__ bool next_item(const FmhaArgs& a, const Sched& sc, int& rnd, WorkItem& it) {
  for (; rnd < sc.n_rounds; ++rnd) {
    const int w = item_of_round(rnd, (int)blockIdx.x, (int)gridDim.x);
    if (w < sc.n_items) {
      it = decode_item(a, w);
      return true;
    }
  }
  return false;
}

__global__ void __launch_bounds__(FMHA_THREADS, 1)
fmha_causal_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                   const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_o,
                   const FmhaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                               // 2 tiles
  uint8_t* sK = sQ + 2 * TILE_BYTES;                // KV_STAGES tiles
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;        // KV_STAGES tiles
  uint8_t* sO = sV + KV_STAGES * TILE_BYTES;        // output staging: two 4 KB halves per epilogue warp
  FmhaBarriers* bars = reinterpret_cast<FmhaBarriers*>(sO + 8 * OSTAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->q_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_full[i], 4);   // one arrival per softmax warp of the tile
      mbar_init(&bars->l_ready[i], 4);  // one arrival per softmax warp of the tile
      mbar_init(&bars->o_done[i], 1);
      mbar_init(&bars->o_empty[i], 4);  // one arrival per epilogue warp
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == TMA_WARP && lane == 0) {
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
    tma_prefetch_desc(&tma_o);
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  const WaitCtx wc{&bars->abort_flag, a.status, a.limit_ns};
  grid_dependency_wait();      // everything above overlaps the tail of the previous kernel in the stream
  grid_launch_dependents();
  Sched sc{a.n_items, a.n_rounds};
  if (a.vl_items != nullptr) {   // the item table was written by the kernel before this one in the stream
    sc.n_items = *reinterpret_cast<const volatile int*>(a.vl_n_entries) * a.Hkv * a.pairs;
    sc.n_rounds = (sc.n_items + (int)gridDim.x - 1) / (int)gridDim.x;
  }

  // The CTA is persistent: every role walks the same list of work items with running counters for the barrier
  // phases. Nothing drains between items: the first S of the next item is issued right behind the last PV of the
  // current one, the softmax warps go straight on to it, and the epilogue warps write the finished O meanwhile.
  if (warp >= TMA_WARP) {
    reg_shrink<48>();
    if (warp == TMA_WARP && lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t kv_count = 0;
      uint32_t qn[2] = {0, 0};   // Q tiles loaded per tile slot
      bool ok = true;
      WorkItem it;
      for (int rnd = 0; ok && next_item(a, sc, rnd, it); ++rnd) {
        const int ntile = it.two ? 2 : 1;
        for (int t = 0; t < ntile && ok; ++t) {
          ok = mbar_wait(&bars->q_empty[t], (qn[t] & 1u) ^ 1u, wc, EMK_DEV_TIMEOUT_PRODUCER);
          if (!ok) break;
          ++qn[t];
          const int hq = it.hq0 + t;
          const int y = it.row0 + it.b * a.q_rb + hq * a.q_rh + it.q0;
          mbar_arrive_expect_tx(&bars->q_full[t], TILE_BYTES);
          tma_load_2d(sQ + t * TILE_BYTES, &tma_q, &bars->q_full[t], hq * a.q_cs, y);
          tma_load_2d(sQ + t * TILE_BYTES + HALF_BYTES, &tma_q, &bars->q_full[t], hq * a.q_cs + 64, y);
        }
        const int ykv = it.row0 + it.b * a.kv_rb + it.hkv * a.kv_rh;
        const int xkv = it.hkv * a.kv_cs;
        for (int j = 0; j < it.nblk && ok; ++j, ++kv_count) {
          const int st = (int)(kv_count % KV_STAGES);
          const uint32_t ph = (kv_count / KV_STAGES) & 1u;
          // K of this block goes out as soon as the S products of the block two back are done; its V follows when
          // that block's PV products are done too (the same moment at which the next block's K slot comes free)
          ok = mbar_wait(&bars->k_empty[st], ph ^ 1u, wc, EMK_DEV_TIMEOUT_PRODUCER);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars->k_full[st], TILE_BYTES);
          tma_load_2d(sK + st * TILE_BYTES, &tma_k, &bars->k_full[st], xkv, ykv + j * FN);
          tma_load_2d(sK + st * TILE_BYTES + HALF_BYTES, &tma_k, &bars->k_full[st], xkv + 64, ykv + j * FN);
          ok = mbar_wait(&bars->v_empty[st], ph ^ 1u, wc, EMK_DEV_TIMEOUT_PRODUCER);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars->v_full[st], TILE_BYTES);
          tma_load_2d(sV + st * TILE_BYTES, &tma_v, &bars->v_full[st], xkv, ykv + j * FN);
          tma_load_2d(sV + st * TILE_BYTES + HALF_BYTES, &tma_v, &bars->v_full[st], xkv + 64, ykv + j * FN);
        }
      }
    } else if (warp == MMA_WARP && lane == 0) {
      // ---------------- MMA issuer ----------------
      const uint32_t hi = smem_desc_hi(1024);
      const uint32_t q_lo = smem_desc_lo(smem_u32(sQ), 0);
      const uint32_t k_lo = smem_desc_lo(smem_u32(sK), 0);
      const uint32_t v_lo = smem_desc_lo(smem_u32(sV), HALF_BYTES);
      auto issue_s = [&](int t, int st) {
        const uint32_t qa = q_lo + (uint32_t)(t * (TILE_BYTES >> 4));
        const uint32_t ka = k_lo + (uint32_t)(st * (TILE_BYTES >> 4));
        const uint32_t d = tmem_base + (uint32_t)(t * FN);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = (uint32_t)(((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4);
          umma_ss_lohi(d, qa + off, ka + off, hi, IDESC_S, ks != 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int t, int st, bool accumulate) {
        const uint32_t va = v_lo + (uint32_t)(st * (TILE_BYTES >> 4));
        const uint32_t d = tmem_base + 256u + (uint32_t)(t * HD);
        const uint32_t pa = tmem_base + (uint32_t)(t * FN);
        umma_ts_lohi(d, pa, va, hi, IDESC_PV, accumulate ? 1u : 0u);
#pragma unroll
        for (int ks = 1; ks < FN / 16; ++ks)
          umma_ts_lohi(d, pa + (uint32_t)(ks * 8), va + (uint32_t)((ks * 16 * 128) >> 4), hi, IDESC_PV, 1u);
      };
      // A tcgen05.commit costs this thread about a hundred cycles, so only the commits another role cannot do without
      // are issued: one per S tile and one after the last PV of an item. "PV of block j-1 is done" is implied by the
      // S commit of block j (a commit covers every earlier MMA of this thread).
      uint32_t kv_count = 0;
      uint32_t iters[2] = {0, 0};   // softmax round trips per tile (parity of p_full)
      uint32_t items[2] = {0, 0};   // items per tile (parity of o_done / o_empty / q_full)
      bool ok = true;
      // first S of an item for tile t: its Q tile and the K block of stage `st` must have landed
      auto first_s = [&](int t, int st, uint32_t ph, bool wait_k) {
        ok = mbar_wait(&bars->q_full[t], items[t] & 1u, wc, EMK_DEV_TIMEOUT_MMA);
        if (ok && wait_k) ok = mbar_wait(&bars->k_full[st], ph, wc, EMK_DEV_TIMEOUT_MMA);
        if (!ok) return;
        tc_fence_after();
        issue_s(t, st);
        tc_commit(&bars->s_full[t]);
      };
      WorkItem it, nx;
      int rnd = 0;
      bool have = next_item(a, sc, rnd, it);
      if (have) {
        for (int t = 0; t < (it.two ? 2 : 1) && ok; ++t) first_s(t, 0, 0u, t == 0);
      }
      while (have && ok) {
        int rn = rnd + 1;
        const bool have_next = next_item(a, sc, rn, nx);
        const int ntile = it.two ? 2 : 1;
        const int ntile_next = have_next ? (nx.two ? 2 : 1) : 0;
        for (int j = 0; j < it.nblk && ok; ++j, ++kv_count) {
          const int st = (int)(kv_count % KV_STAGES);
          const uint32_t ph = (kv_count / KV_STAGES) & 1u;
          const int stn = (int)((kv_count + 1) % KV_STAGES);
          const uint32_t phn = ((kv_count + 1) / KV_STAGES) & 1u;
          const bool last = (j + 1) == it.nblk;
          for (int t = 0; t < ntile && ok; ++t) {
            ok = mbar_wait(&bars->p_full[t], iters[t] & 1u, wc, EMK_DEV_TIMEOUT_MMA);
            if (ok && t == 0) ok = mbar_wait(&bars->v_full[st], ph, wc, EMK_DEV_TIMEOUT_MMA);
            // the first PV of an item overwrites O: the epilogue of the previous item must have read it
            if (ok && j == 0) ok = mbar_wait(&bars->o_empty[t], (items[t] & 1u) ^ 1u, wc, EMK_DEV_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, st, j > 0);
            ++iters[t];
            if (!last) {
              if (t == 0) {
                ok = mbar_wait(&bars->k_full[stn], phn, wc, EMK_DEV_TIMEOUT_MMA);
                if (!ok) break;
              }
              issue_s(t, stn);
              tc_commit(&bars->s_full[t]);
            } else {
              tc_commit(&bars->o_done[t]);
              ++items[t];
              // the next item starts on this tile right away (its K block sits in the other stage of the ring)
              if (t < ntile_next) first_s(t, stn, phn, t == 0);
            }
          }
        }
        // a tile that sat the current item out but takes part in the next one
        for (int t = ntile; t < ntile_next && ok; ++t)
          first_s(t, (int)(kv_count % KV_STAGES), (kv_count / KV_STAGES) & 1u, false);
        have = have_next;
        it = nx;
        rnd = rn;
      }
    }
  } else if (warp >= EPI_WARP0) {
    // ---------------- epilogue: warp e owns rows 32e..32e+31 of both tiles ----------------
    reg_shrink<80>();
    const int quarter = warp & 3;
    const int r_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    uint8_t* stage = sO + quarter * 2 * OSTAGE_BYTES;   // two halves of 64 columns
    const uint32_t stage_row = smem_u32(stage) + (uint32_t)(lane * 128);
    uint32_t kv_base = 0;
    uint32_t items[2] = {0, 0};
    bool ok = true;
    WorkItem it;
    for (int rnd = 0; ok && next_item(a, sc, rnd, it); ++rnd) {
      const int ntile = it.two ? 2 : 1;
      for (int t = 0; t < ntile && ok; ++t) {
        const uint32_t tO = tmem_base + lane_base + 256u + (uint32_t)(t * HD);
        ok = mbar_wait_warp(&bars->o_done[t], items[t] & 1u, wc, EMK_DEV_TIMEOUT_SOFTMAX);
        if (ok) ok = mbar_wait_warp(&bars->l_ready[t], items[t] & 1u, wc, EMK_DEV_TIMEOUT_SOFTMAX);
        if (!ok) break;
        ++items[t];
        tc_fence_after();
        // every MMA of the item is done: the V slot of its last block goes back to the producer
        if (t == ntile - 1 && quarter == 0 && lane == 0)
          mbar_arrive(&bars->v_empty[(kv_base + (uint32_t)it.nblk - 1u) % KV_STAGES]);
        const float inv = __fdividef(1.0f, bars->row_l[t][r_in_tile]);
        const int hq = it.hq0 + t;
        const bool full = it.q0 + FM <= it.slen;
        const int q_row = it.q0 + r_in_tile;
        __nv_bfloat16* orow =
            a.o + ((int64_t)it.row0 + (int64_t)it.b * a.o_rb + (int64_t)hq * a.o_rh + q_row) * a.ld_o +
            (int64_t)hq * a.o_cs;
        // the stores of the previous tile out of the staging buffers must have read them
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
        uint32_t o[2][32];
        tmem_ld_x32(tO, o[0]);
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          tmem_ld_wait_regs(o[c & 1]);
          if (c + 1 < HD / 32) tmem_ld_x32(tO + (uint32_t)((c + 1) * 32), o[(c + 1) & 1]);
          if (c + 1 == HD / 32) {
            // O is in registers: the MMA thread may overwrite it with the next item's first PV
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->o_empty[t]);
          }
          uint32_t v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            v[i] = pack_bf16x2(__uint_as_float(o[c & 1][2 * i]) * inv, __uint_as_float(o[c & 1][2 * i + 1]) * inv);
          if (full) {
            // Full tile: 64 columns at a time leave through a 128-byte-swizzled staging buffer and one TMA store
            // (a direct store touches 32 different lines per instruction: one row per lane).
            const uint32_t half_base = stage_row + (uint32_t)((c >> 1) * OSTAGE_BYTES);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t addr = half_base + (uint32_t)((((c & 1) * 4 + q) ^ (lane & 7)) * 16);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v[4 * q]), "r"(v[4 * q + 1]),
                           "r"(v[4 * q + 2]), "r"(v[4 * q + 3])
                           : "memory");
            }
            if (c & 1) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tma_o, stage + (c >> 1) * OSTAGE_BYTES, hq * a.o_cs + (c >> 1) * 64,
                             it.row0 + it.b * a.o_rb + hq * a.o_rh + it.q0 + quarter * 32);
                tma_store_commit();
              }
            }
          } else if (q_row < it.slen) {
            // ragged last tile of a sequence: rows past the end are not stored
            st_global_v8(orow + c * 32, v);
            st_global_v8(orow + c * 32 + 16, v + 8);
          }
        }
      }
      kv_base += (uint32_t)it.nblk;
    }
    if (lane == 0) tma_store_wait_all();   // output tiles still in flight
  } else {
    // ---------------- softmax (and the rare rescale of O): warps 0..3 tile 0, warps 4..7 tile 1 ----------------
    reg_grow<192>();
    const int t = warp >> 2;
    const int quarter = warp & 3;
    const int r_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + (uint32_t)(t * FN);
    const uint32_t tO = tmem_base + lane_base + 256u + (uint32_t)(t * HD);
    const bool elected = quarter == 0 && lane == 0;
    uint32_t kv_base = 0;   // KV blocks consumed by the CTA before the current item
    uint32_t iter = 0;      // softmax round trips of this tile
    uint32_t item_n = 0;    // items this tile took part in
    bool ok = true;
    WorkItem it;
    for (int rnd = 0; ok && next_item(a, sc, rnd, it); ++rnd) {
      const int nblk = it.nblk;
      if (t == 1 && !it.two) {  // this tile sits the item out
        kv_base += (uint32_t)nblk;
        continue;
      }
      const bool last_tile = t == (it.two ? 1 : 0);  // its commits come last in the MMA thread's order
      float m_used = -CUDART_INF_F;
      float l = 0.f;
      for (int j = 0; j < nblk; ++j, ++iter) {
        if (!mbar_wait_warp(&bars->s_full[t], iter & 1u, wc, EMK_DEV_TIMEOUT_SOFTMAX)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (elected) {
          // the S commit of the last tile covers the S products of block j and the PV products of block j-1 of
          // both tiles: hand back this block's K slot and the previous block's V slot; after the last S of the item
          // this tile's Q buffer is free as well
          if (last_tile) {
            mbar_arrive(&bars->k_empty[(kv_base + (uint32_t)j) % KV_STAGES]);
            if (j > 0) mbar_arrive(&bars->v_empty[(kv_base + (uint32_t)j - 1u) % KV_STAGES]);
          }
          if (j == nblk - 1) mbar_arrive(&bars->q_empty[t]);
        }
        uint32_t s[FN];
#pragma unroll
        for (int c = 0; c < FN / 32; ++c) tmem_ld_x32(tS + (uint32_t)(c * 32), s + c * 32);
        tmem_ld_wait();
        if (j == nblk - 1) {
          // diagonal block: key index k0 + i is visible to query q_row iff k0 + i <= q_row, k0 == q0 here
#pragma unroll
          for (int i = 0; i < FN; ++i)
            if (i > r_in_tile) s[i] = __float_as_uint(-CUDART_INF_F);
        }
        // four independent 3-input max chains instead of one 128-long dependency chain
        float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F, mx2 = -CUDART_INF_F, mx3 = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < FN; i += 8) {
          mx0 = max3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
          mx1 = max3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
          mx2 = max3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
          mx3 = max3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        const float m_new = fmaxf(m_used, mx * a.scale_log2);
        // The decision to move a row's reference maximum is the row's own (true on the first block, m_used = -inf),
        // so a row's arithmetic does not depend on which rows share its warp; only the tensor-memory round trip that
        // rescales O is taken warp-wide, with factor 1 for the rows that keep their maximum.
        const bool need = (m_new - m_used) > RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, need)) {
          const float m_next = need ? m_new : m_used;
          if (j > 0) {  // PV of block j-1 has completed: implied by the S commit waited on above
            const float alpha = need ? ex2_approx(m_used - m_next) : 1.0f;
            l *= alpha;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
              uint32_t o[32];
              tmem_ld_x32(tO + (uint32_t)(c * 32), o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st_x32(tO + (uint32_t)(c * 32), o);
            }
            tmem_st_wait();
          }
          m_used = m_next;
        }
        const unsigned long long neg_m2 = pack_f32x2(-m_used, -m_used);
        const unsigned long long scale2 = pack_f32x2(a.scale_log2, a.scale_log2);
        unsigned long long sum_a = 0ull, sum_b = 0ull;  // two independent packed accumulators (4 partial sums)
        uint32_t p[FN / 2];
#pragma unroll
        for (int i = 0; i < FN / 2; i += 2) {
          float t0, t1, t2, t3;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), scale2, neg_m2),
                       t0, t1);
          unpack_f32x2(
              fma_f32x2(pack_f32x2(__uint_as_float(s[2 * i + 2]), __uint_as_float(s[2 * i + 3])), scale2, neg_m2), t2,
              t3);
          const float p0 = ex2_approx(t0), p1 = ex2_approx(t1), p2 = ex2_approx(t2), p3 = ex2_approx(t3);
          sum_a = add_f32x2(sum_a, pack_f32x2(p0, p1));
          sum_b = add_f32x2(sum_b, pack_f32x2(p2, p3));
          p[i] = pack_bf16x2(p0, p1);
          p[i + 1] = pack_bf16x2(p2, p3);
        }
        {
          float a0, a1, b0, b1;
          unpack_f32x2(sum_a, a0, a1);
          unpack_f32x2(sum_b, b0, b1);
          l += (a0 + a1) + (b0 + b1);
        }
        tmem_st_x32(tS, p);
        tmem_st_x32(tS + 32u, p + 32);
        tmem_st_wait();
        if (j == nblk - 1) {
          // The row sums go to the epilogue warps. They must have finished with the previous item of this tile
          // (its row sums and its l_ready phase), which their o_empty arrival says; it is almost always long past.
          if (item_n > 0 && !mbar_wait_warp(&bars->o_empty[t], (item_n - 1u) & 1u, wc, EMK_DEV_TIMEOUT_SOFTMAX)) {
            ok = false;
            break;
          }
          bars->row_l[t][r_in_tile] = l;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->p_full[t]);
          if (j == nblk - 1) mbar_arrive(&bars->l_ready[t]);
        }
      }
      ++item_n;
      kv_base += (uint32_t)nblk;
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (bars->abort_flag) abort_drain();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// Item table of the packed variable-length mode. One 1024-thread CTA: thread l owns query-block level l (query rows
// 128 l .. 128 l + 127) and walks the sequences twice — once to count how many are long enough to have that block,
// once to write their entries — so entries come out grouped by level, deepest (= most KV blocks) level first, in
// sequence order within a level. table[0].x receives the number of entries; entries start at table[1].
constexpr int VL_MAX_LEVELS = 1024;

// A sequence whose rows do not lie inside [0, total) or that is longer than max_seqlen is cut to the part that does
// (the attention kernel's row stores must never leave the output); the bounds-check build also reports it.
__device__ __forceinline__ void varlen_sequence(const int* __restrict__ cu_seqlens, int b, int total, int max_seqlen,
                                                int* status, int& r0, int& len) {
  const int a = cu_seqlens[b], e = cu_seqlens[b + 1];
  r0 = min(max(a, 0), total);
  len = min(min(max(e - r0, 0), total - r0), max_seqlen);
  if (a < 0 || e < a || e > total || e - a > max_seqlen) emk_record_bounds(status, EMK_DEV_BOUNDS_CU_SEQLENS);
}

__global__ void __launch_bounds__(VL_MAX_LEVELS) varlen_items_kernel(const int* __restrict__ cu_seqlens, int B,
                                                                     int levels, int4* __restrict__ table, int total,
                                                                     int max_seqlen, int* status) {
  __shared__ int count[VL_MAX_LEVELS];
  __shared__ int offset[VL_MAX_LEVELS];
  const int l = (int)threadIdx.x;
  grid_dependency_wait();
  grid_launch_dependents();
  int c = 0;
  if (l < levels) {
    for (int b = 0; b < B; ++b) {
      int r0, len;
      varlen_sequence(cu_seqlens, b, total, max_seqlen, l == 0 ? status : nullptr, r0, len);
      c += (len > l * FM) ? 1 : 0;
    }
  }
  count[l] = c;
  __syncthreads();
  if (l == 0) {
    int run = 0;
    for (int k = levels - 1; k >= 0; --k) {   // deepest level first
      offset[k] = run;
      run += count[k];
    }
    table[0] = make_int4(run, 0, 0, 0);
  }
  __syncthreads();
  if (l < levels && c > 0) {
    int4* out = table + 1 + offset[l];
    for (int b = 0; b < B; ++b) {
      int r0, len;
      varlen_sequence(cu_seqlens, b, total, max_seqlen, nullptr, r0, len);
      if (len > l * FM) *out++ = make_int4(r0, l * FM, len, 0);
    }
  }
}

constexpr int FMHA_SMEM = (2 + 2 * KV_STAGES) * TILE_BYTES + 8 * OSTAGE_BYTES + 1024 + (int)sizeof(FmhaBarriers);
static_assert(FMHA_SMEM <= 232448, "shared memory budget");

// Packed mode: `cu_seqlens` (device, B + 1 ints) is given, S is the longest sequence the caller admits and `total`
// the number of token rows; the operands are token-major.
struct VarlenArgs {
  const int* cu_seqlens;
  int64_t total;
  void* workspace;
  int64_t workspace_bytes;
};

int64_t varlen_max_entries(int64_t B, int64_t total) { return total / FM + B; }

int fmha_launch(emk_handle_t h, const void* q, const void* k, const void* v, void* o, int64_t B, int64_t Hq,
                int64_t Hkv, int64_t S, int64_t D, bool token_major, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                int64_t ld_o, float scale, cudaStream_t s, const VarlenArgs* vl = nullptr) {
  if (!h || !q || !k || !v || !o) return EMK_ERR_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0) return EMK_ERR_SHAPE;
  if (D != HD) {
    EMK_SET_ERR(h, "emk_sdpa_causal_gqa_bf16: head_dim must be 128, got %lld", (long long)D);
    return EMK_ERR_SHAPE;
  }
  if (Hq % Hkv != 0) {
    EMK_SET_ERR(h, "emk_sdpa_causal_gqa_bf16: Hq (%lld) must be a multiple of Hkv (%lld)", (long long)Hq,
                (long long)Hkv);
    return EMK_ERR_SHAPE;
  }
  if (!vl && (B * Hq * S > 0x7fffffffLL || B * S > 0x7fffffffLL)) return EMK_ERR_SHAPE;
  const int64_t rows = vl ? vl->total : B * S;   // token rows of the token-major operands
  if (vl) {
    if (!token_major || !vl->cu_seqlens || !vl->workspace || vl->total <= 0 || vl->total > 0x7fffffffLL)
      return EMK_ERR_ARG;
    if ((S + FM - 1) / FM > VL_MAX_LEVELS) {
      EMK_SET_ERR(h, "emk_sdpa_causal_gqa_bf16_varlen: max_seqlen %lld exceeds %d tokens", (long long)S,
                  VL_MAX_LEVELS * FM);
      return EMK_ERR_LIMIT;
    }
    if (vl->workspace_bytes < (1 + varlen_max_entries(B, vl->total)) * (int64_t)sizeof(int4) ||
        ((uintptr_t)vl->workspace & 15u) != 0) {
      EMK_SET_ERR(h, "emk_sdpa_causal_gqa_bf16_varlen: workspace of %lld bytes is too small or not 16-byte aligned "
                  "(see emk_sdpa_varlen_workspace_bytes)", (long long)vl->workspace_bytes);
      return EMK_ERR_WORKSPACE;
    }
  }
  if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15u) != 0) return EMK_ERR_ALIGN;
  if (token_major && ((ld_q | ld_k | ld_v | ld_o) % 8) != 0) return EMK_ERR_ALIGN;

  FmhaArgs a;
  a.o = (__nv_bfloat16*)o;
  a.B = (int)B;
  a.Hq = (int)Hq;
  a.Hkv = (int)Hkv;
  a.S = (int)S;
  a.group = (int)(Hq / Hkv);
  a.pairs = (a.group + 1) / 2;
  a.nqblk = (int)((S + FM - 1) / FM);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = h->status_dev;
  a.limit_ns = h->wait_limit_ns;
  a.vl_items = nullptr;
  a.vl_n_entries = nullptr;

  CUtensorMap tq, tk, tv, to;
  int rc;
  if (!token_major) {
    a.q_cs = 0; a.q_rb = (int)(Hq * S); a.q_rh = (int)S;
    a.kv_cs = 0; a.kv_rb = (int)(Hkv * S); a.kv_rh = (int)S;
    a.o_cs = 0; a.o_rb = (int)(Hq * S); a.o_rh = (int)S;
    a.ld_o = HD;
    rc = emk_make_tmap_2d(h, &tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, HD, (uint64_t)(B * Hq * S), HD * 2, 64, FM,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = emk_make_tmap_2d(h, &tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, HD, (uint64_t)(B * Hkv * S), HD * 2, 64, FN,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = emk_make_tmap_2d(h, &tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v, HD, (uint64_t)(B * Hkv * S), HD * 2, 64, FN,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = emk_make_tmap_2d(h, &to, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, o, HD, (uint64_t)(B * Hq * S), HD * 2, 64, 32,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  } else {
    a.q_cs = HD; a.q_rb = (int)S; a.q_rh = 0;
    a.kv_cs = HD; a.kv_rb = (int)S; a.kv_rh = 0;
    a.o_cs = HD; a.o_rb = (int)S; a.o_rh = 0;
    a.ld_o = ld_o;
    if (ld_q < Hq * HD || ld_k < Hkv * HD || ld_v < Hkv * HD || ld_o < Hq * HD) return EMK_ERR_SHAPE;
    rc = emk_make_tmap_2d(h, &tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, (uint64_t)(Hq * HD), (uint64_t)rows,
                          (uint64_t)ld_q * 2, 64, FM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = emk_make_tmap_2d(h, &tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, (uint64_t)(Hkv * HD), (uint64_t)rows,
                          (uint64_t)ld_k * 2, 64, FN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = emk_make_tmap_2d(h, &tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v, (uint64_t)(Hkv * HD), (uint64_t)rows,
                          (uint64_t)ld_v * 2, 64, FN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = emk_make_tmap_2d(h, &to, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, o, (uint64_t)(Hq * HD), (uint64_t)rows,
                          (uint64_t)ld_o * 2, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }

  static emk_device_once once;
  {
    std::lock_guard<std::mutex> lk(once.mu);
    if (!once.done[h->device]) {
      EMK_CUDA_TRY(h, cudaFuncSetAttribute(fmha_causal_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FMHA_SMEM));
      once.done[h->device] = true;
    }
  }
  // packed mode: the item count is known on the device only; the grid is sized for the upper bound
  const int64_t n_items = (vl ? varlen_max_entries(B, vl->total) : (int64_t)a.nqblk * B) * Hkv * a.pairs;
  if (n_items > 0x7fffffffLL) return EMK_ERR_SHAPE;
  a.n_items = (int)n_items;
  const int grid = a.n_items < h->sm_count ? a.n_items : h->sm_count;  // persistent: one CTA per SM
  a.n_rounds = (a.n_items + grid - 1) / grid;
  {
    // K/V that fits comfortably in L2 stays there whatever the order; otherwise about two rounds of items per group
    const int64_t per_qblk = B * Hkv * a.pairs;
    const int64_t kv_bytes = B * Hkv * S * HD * 2 * 2;
    int64_t gp = per_qblk;
    if (kv_bytes > (48ll << 20)) gp = (2ll * grid + a.nqblk - 1) / a.nqblk;
    if (gp < 1) gp = 1;
    if (gp > per_qblk) gp = per_qblk;
    a.gp = (int)gp;
  }
  if (vl) {
    int4* table = (int4*)vl->workspace;
    a.vl_n_entries = (const int*)table;
    a.vl_items = table + 1;
    a.B = 1;
    a.q_rb = a.kv_rb = a.o_rb = 0;
    EMK_CUDA_TRY(h, launch_after_prologue(varlen_items_kernel, 1u, (unsigned)VL_MAX_LEVELS, 0, s,
                                          h->overlap_launch != 0, vl->cu_seqlens, (int)B, (int)((S + FM - 1) / FM),
                                          table, (int)vl->total, (int)S, h->status_dev));
  }
  EMK_CUDA_TRY(h, launch_after_prologue(fmha_causal_kernel, (unsigned)grid, FMHA_THREADS, FMHA_SMEM, s,
                                        h->overlap_launch != 0, tq, tk, tv, to, a));
  EMK_LAUNCH_CHECK(h);
  return EMK_OK;
}

}  // namespace

extern "C" int emk_sdpa_causal_gqa_bf16(emk_handle_t h, const void* q, const void* k, const void* v, void* o,
                                        int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, float scale,
                                        emk_stream_t stream) {
  return fmha_launch(h, q, k, v, o, B, Hq, Hkv, S, D, false, 0, 0, 0, 0, scale, (cudaStream_t)stream);
}

extern "C" int emk_sdpa_causal_gqa_bf16_tok(emk_handle_t h, const void* q, const void* k, const void* v, void* o,
                                            int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, int64_t ld_q,
                                            int64_t ld_k, int64_t ld_v, int64_t ld_o, float scale,
                                            emk_stream_t stream) {
  return fmha_launch(h, q, k, v, o, B, Hq, Hkv, S, D, true, ld_q, ld_k, ld_v, ld_o, scale, (cudaStream_t)stream);
}

extern "C" int64_t emk_sdpa_varlen_workspace_bytes(int64_t B, int64_t total_tokens) {
  if (B <= 0 || total_tokens <= 0) return 0;
  return (1 + varlen_max_entries(B, total_tokens)) * (int64_t)sizeof(int4);
}

extern "C" int emk_sdpa_causal_gqa_bf16_varlen(emk_handle_t h, const void* q, const void* k, const void* v, void* o,
                                               const int32_t* cu_seqlens, int64_t B, int64_t total_tokens,
                                               int64_t max_seqlen, int64_t Hq, int64_t Hkv, int64_t D, int64_t ld_q,
                                               int64_t ld_k, int64_t ld_v, int64_t ld_o, float scale, void* workspace,
                                               int64_t workspace_bytes, emk_stream_t stream) {
  VarlenArgs vl{cu_seqlens, total_tokens, workspace, workspace_bytes};
  return fmha_launch(h, q, k, v, o, B, Hq, Hkv, max_seqlen, D, true, ld_q, ld_k, ld_v, ld_o, scale,
                     (cudaStream_t)stream, &vl);
}
