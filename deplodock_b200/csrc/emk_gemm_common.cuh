// Pieces shared by the bf16 and the e4m3-weight GEMM kernels: launch arguments and the fused epilogue that turns
// 32 fp32 accumulator columns of one output row (as read from tensor memory) into bf16 stores.
// The reference folds the same pointwise tails into its mma.sync fragment epilogue
// (RegEpilogue, emmy/compiler/ir/kernel/ir.py:1266-1288, built in lowering/kernel/_atom.py:114-153).
#pragma once
#include "emk_common.cuh"

namespace emk {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int A_STAGE_BYTES = BM * BK * 2;

struct GemmArgs {
  __nv_bfloat16* y;
  const __nv_bfloat16* residual;
  const float* scale;
  int M, N, K;
  int ldy;
  int tiles_m, tiles_n, kblocks;
  int epi;
  int wide;  // y (and residual) rows are 32-byte aligned: use 256-bit accesses
  // fused q/k-norm + RoPE epilogue (epi == EMK_EPI_QKNORM_ROPE_INTERNAL): output columns are heads of 128
  const __nv_bfloat16* qk_qw;
  const __nv_bfloat16* qk_kw;
  const __nv_bfloat16* qk_rope;  // chunk-major cos|sin table [8][S][16] bf16 (see emk.h)
  int qk_S, qk_Hq, qk_Hkv;
  float qk_eps;
  const int* qk_pos;             // rotary position of every row (packed sequences); null: position = row % qk_S
  const float* f32_bias;         // epi == EMK_EPI_F32_INTERNAL: optional fp32 bias [N]; y is then fp32 [M,N]
  // RMSNorm folded around the GEMM (the norm weight is folded into W by the caller):
  //   ss_in   partial sums of squares [M][ss_in_segs] of the un-normalised input rows (one slot per 128 columns):
  //           accumulator rows are scaled by rsqrt(sum_s ss_in[s][row] * ss_inv_dim + ss_eps) before the epilogue
  //   ss_out  partial sums of squares [M][N/128] of the bf16 values this GEMM stores: every epilogue thread writes the
  //           slot(s) of the columns it owns, so the buffer is fully overwritten, needs no clearing, and the sum the
  //           consumer forms is the same on every run (no atomics)
  const float* ss_in;
  int ss_in_segs;
  float ss_inv_dim, ss_eps;
  float* ss_out;
  // set by the GEMM chain: residual and ss_in may have been written by another SM earlier in the same launch, so
  // they are read past L1 and never prefetched into it
  int coherent;
  int* status;
  unsigned long long limit_ns;
};

constexpr int EMK_EPI_QKNORM_ROPE_INTERNAL = 100;
constexpr int EMK_EPI_F32_INTERNAL = 101;  // store the fp32 accumulator (+ fp32 bias) unrounded: y is float [M,N]

// Tile order of the persistent kernels: tiles are walked in groups of GROUP_M row-tiles by all column-tiles, rows
// fastest inside a group, so the CTAs running at one time share a few A row-blocks and a few W column-blocks and
// re-read them from L2 instead of HBM.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int gsize = min(tiles_m - first_m, group_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % gsize;
  tn = in_group / gsize;
}

// The epilogue kind of a kernel instantiation: a compile-time constant where the kernel was built for one epilogue
// (its code then holds only that epilogue), the launch argument where it was built for all of them (EPI < 0).
// A GEMM kernel that carries every epilogue is large enough to push the attention kernel out of the instruction
// cache and back at every switch between the two (measured: about 7 us per switch, two switches per decoder layer).
constexpr int EMK_EPI_SET_LAYER = -2;  // run-time choice among residual / SwiGLU / q-k-norm + RoPE only (GEMM chain)
template <int EPI>
__device__ __forceinline__ int epi_of(const GemmArgs& g) {
  if (EPI == EMK_EPI_SET_LAYER) {
    const int e = g.epi;   // any other value is refused by the host; the selects let the compiler drop the other paths
    return e == EMK_EPI_SWIGLU ? (int)EMK_EPI_SWIGLU
                               : (e == EMK_EPI_QKNORM_ROPE_INTERNAL ? EMK_EPI_QKNORM_ROPE_INTERNAL : (int)EMK_EPI_RESIDUAL);
  }
  return EPI < 0 ? g.epi : EPI;
}

// silu(g) = g / (1 + exp(-g)) with the approximate reciprocal (2 ulp): the result is rounded to bf16 right after, and
// the IEEE division's slow path made the SwiGLU epilogue longer than the main loop of a K = 1024 tile.
__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// Epilogue for 32 accumulator columns [col0, col0+32) of one output row held by this thread. `g.wide` says rows of
// y (and of the residual) are 32-byte aligned, so full 32-column groups move as 256-bit accesses.
template <int EPI, bool FAST = false>
__device__ __forceinline__ float epilogue_store32(const GemmArgs& g, const uint32_t* r, int row, int col0, float rs) {
  // FAST: the launch covers whole 256 x 256 tiles of 32-byte aligned rows, so no row / column test and no narrow
  // access path is compiled in (less code to fetch at every kernel switch)
  if (!FAST && (row >= g.M || col0 >= g.N)) return 0.f;
  if (epi_of<EPI>(g) == EMK_EPI_SWIGLU) {
    // columns are (gate, up) pairs; 16 outputs = 32 bytes
    __nv_bfloat16* out = g.y + (int64_t)row * g.ldy + (col0 >> 1);
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // roundings in pairs: one packed conversion does two (the scalar one runs at a quarter of the rate)
      const uint32_t gu0 = pack_bf16x2(__uint_as_float(r[j * 4]) * rs, __uint_as_float(r[j * 4 + 1]) * rs);
      const uint32_t gu1 = pack_bf16x2(__uint_as_float(r[j * 4 + 2]) * rs, __uint_as_float(r[j * 4 + 3]) * rs);
      const uint32_t sg = pack_bf16x2(silu_f(bf16_lo(gu0)), silu_f(bf16_lo(gu1)));
      o[j] = pack_bf16x2(bf16_lo(sg) * bf16_hi(gu0), bf16_hi(sg) * bf16_hi(gu1));
    }
    if (FAST || (g.wide && col0 + 32 <= g.N)) {
      st_global_v8(out, o);
    } else {
      if (col0 < g.N) *reinterpret_cast<uint4*>(out) = make_uint4(o[0], o[1], o[2], o[3]);
      if (col0 + 16 < g.N) *reinterpret_cast<uint4*>(out + 8) = make_uint4(o[4], o[5], o[6], o[7]);
    }
    return 0.f;
  }
  if (epi_of<EPI>(g) == EMK_EPI_F32_INTERNAL) {
    float* out = reinterpret_cast<float*>(g.y) + (int64_t)row * g.ldy + col0;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (col0 + q * 4 < g.N) {   // N is a multiple of 8: a quad is inside or outside as a whole
        float4 v4 = make_float4(__uint_as_float(r[q * 4]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]),
                                __uint_as_float(r[q * 4 + 3]));
        if (g.f32_bias != nullptr) {
          const float4 b4 = __ldg(reinterpret_cast<const float4*>(g.f32_bias + col0 + q * 4));
          v4.x += b4.x; v4.y += b4.y; v4.z += b4.z; v4.w += b4.w;
        }
        *reinterpret_cast<float4*>(out + q * 4) = v4;
      }
    }
    return 0.f;
  }
  const bool full = FAST || (g.wide && (col0 + 32 <= g.N));
  float v[32];
  if (g.ss_in != nullptr) {   // the row scale of a folded RMSNorm; without one rs is 1 and the multiplies are skipped
#pragma unroll
    for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]) * rs;
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
  }
  if (g.scale != nullptr) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (FAST || col0 + q * 4 < g.N) {
        const float4 s = __ldg(reinterpret_cast<const float4*>(g.scale + col0 + q * 4));
        v[q * 4 + 0] *= s.x; v[q * 4 + 1] *= s.y; v[q * 4 + 2] *= s.z; v[q * 4 + 3] *= s.w;
      }
    }
  }
  if (epi_of<EPI>(g) == EMK_EPI_RESIDUAL) {
    const __nv_bfloat16* res = g.residual + (int64_t)row * g.ldy + col0;
    uint32_t rr[16];
    if (full) {
      if (g.coherent) {
        ld_global_cg_v8(res, rr);
        ld_global_cg_v8(res + 16, rr + 8);
      } else {
        ld_global_v8(res, rr);
        ld_global_v8(res + 16, rr + 8);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 t = make_uint4(0, 0, 0, 0);
        if (col0 + q * 8 < g.N) t = __ldcg(reinterpret_cast<const uint4*>(res + q * 8));
        rr[q * 4 + 0] = t.x; rr[q * 4 + 1] = t.y; rr[q * 4 + 2] = t.z; rr[q * 4 + 3] = t.w;
      }
    }
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const uint32_t p = pack_bf16x2(v[2 * e], v[2 * e + 1]);   // both roundings in one packed conversion
      v[2 * e] = bf16_lo(p) + bf16_lo(rr[e]);
      v[2 * e + 1] = bf16_hi(p) + bf16_hi(rr[e]);
    }
  } else if (epi_of<EPI>(g) == EMK_EPI_BIAS) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (col0 + q * 8 < g.N) {
        const uint4 bv = __ldg(reinterpret_cast<const uint4*>(g.residual + col0 + q * 8));
        const uint32_t bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[q * 8 + 2 * e] += bf16_lo(bb[e]);
          v[q * 8 + 2 * e + 1] += bf16_hi(bb[e]);
        }
      }
    }
  }
  uint32_t o[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) o[e] = pack_bf16x2(v[2 * e], v[2 * e + 1]);
  float ss = 0.f;
  if (g.ss_out != nullptr) {  // sum of squares of what is stored (columns past N hold zeros: their weights are zero-filled)
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const float f0 = bf16_lo(o[e]), f1 = bf16_hi(o[e]);
      ss = fmaf(f0, f0, ss);
      ss = fmaf(f1, f1, ss);
    }
  }
  __nv_bfloat16* out = g.y + (int64_t)row * g.ldy + col0;
  if (full) {
    st_global_v8(out, o);
    st_global_v8(out + 16, o + 8);
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (col0 + q * 8 < g.N)
        *reinterpret_cast<uint4*>(out + q * 8) = make_uint4(o[q * 4], o[q * 4 + 1], o[q * 4 + 2], o[q * 4 + 3]);
  }
  return ss;
}


// Rotary position of output row `row`: given per row for packed sequences (clamped to the table), else the row's
// offset within its fixed-length sequence.
__device__ __forceinline__ int rope_position(const GemmArgs& g, int row) {
  if (g.qk_pos != nullptr) {
    const int p = __ldg(g.qk_pos + row);
    if (p < 0 || p >= g.qk_S) emk_record_bounds(g.status, EMK_DEV_BOUNDS_POSITION);
    return min(max(p, 0), g.qk_S - 1);
  }
  return row % g.qk_S;
}

// Issued by an epilogue thread BEFORE it waits for its accumulator: everything the epilogue will read from global
// memory for this row segment is pulled towards the SM while the tensor core is still working on the tile, so the
// epilogue (two warps per scheduler, little latency hiding of its own) finds it in L1 / L2.
template <int EPI = -1, bool FAST = false>
__device__ __forceinline__ void epilogue_prefetch(const GemmArgs& g, int row, int n0, int ncols) {
  if (!FAST && (row >= g.M || n0 >= g.N)) return;
  if (g.ss_in != nullptr && !g.coherent) {
    asm volatile("prefetch.global.L1 [%0];" ::"l"(g.ss_in + (int64_t)row * g.ss_in_segs));
  }
  if (epi_of<EPI>(g) == EMK_EPI_QKNORM_ROPE_INTERNAL) {
    if ((n0 >> 7) < g.qk_Hq + g.qk_Hkv) {
      const __nv_bfloat16* tp = g.qk_rope + (int64_t)rope_position(g, row) * 16;
#pragma unroll
      for (int q = 0; q < 8; ++q) asm volatile("prefetch.global.L1 [%0];" ::"l"(tp + (int64_t)q * g.qk_S * 16));
    }
  } else if (epi_of<EPI>(g) == EMK_EPI_RESIDUAL) {
    const __nv_bfloat16* res = g.residual + (int64_t)row * g.ldy + n0;
    for (int c = 0; c < ncols; c += 64) asm volatile("prefetch.global.L2 [%0];" ::"l"(res + c));
  }
}

// One head (128 accumulator columns of this thread's row) of the fused QKV projection: round to bf16 as the GEMM
// output would be, then for query/key heads the per-head RMSNorm and the rotate-half RoPE on packed bf16 pairs with
// the rounding steps of the eager bf16 module (normalised -> bf16, * weight -> bf16, each RoPE product -> bf16,
// sum -> bf16); value heads are stored as they are. Thread-local: the row's 128 columns live in this thread's TMEM lane.
//
// The accumulator is read TWICE: a first sweep forms the row's sum of squares (four independent partial sums) and
// keeps nothing; a second sweep takes 16 columns and their rotate-half partners (+64) at a time, normalises, rotates
// and stores them. Holding all 64 packed pairs in registers instead (one sweep) left no room to issue the rotary-table
// loads ahead of their use within the kernel's 168 registers, and the epilogue of a K = 1024 tile — about 10 000
// cycles for one head per warp, against 8 192 of tensor-core work — set the pace of the whole projection.
template <bool FAST = false>
__device__ __forceinline__ void epilogue_head_qknorm_rope(const GemmArgs& g, uint32_t taddr, int row, int col0,
                                                          float rs) {
  const int head = col0 >> 7;
  const bool rotate = head < g.qk_Hq + g.qk_Hkv;   // uniform over the warp (all lanes share the column range)
  const bool valid = FAST || (row < g.M && col0 < g.N);
  __nv_bfloat16* out = g.y + (int64_t)row * g.ldy + col0;
  if (!rotate) {
    // value head: bf16 of the (row-scaled) accumulator, 32 columns at a time
    uint32_t v[2][32];
    tmem_ld_x32(taddr, v[0]);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      tmem_ld_wait_regs(v[c & 1]);
      if (c + 1 < 4) tmem_ld_x32(taddr + (uint32_t)((c + 1) * 32), v[(c + 1) & 1]);
      uint32_t o[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        o[i] = pack_bf16x2(__uint_as_float(v[c & 1][2 * i]) * rs, __uint_as_float(v[c & 1][2 * i + 1]) * rs);
      if (valid) {
        st_global_v8(out + c * 32, o);
        st_global_v8(out + c * 32 + 16, o + 8);
      }
    }
    return;
  }
  // ---- sweep 1: sum of squares of the bf16-rounded row; the rounded pairs go back into tensor memory ----
  // Chunk c (32 fp32 columns) becomes 16 packed bf16 pairs, written over columns [16c, 16c+16) of the head's own
  // accumulator region: those columns were read by this or an earlier chunk, and the chunk in flight lies above them.
  // Sweep 2 then reads the packed pairs and does not round the accumulator a second time.
  float ss0 = 0.f, ss1 = 0.f, ss2 = 0.f, ss3 = 0.f;
  {
    uint32_t v[2][32];
    tmem_ld_x32(taddr, v[0]);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      tmem_ld_wait_regs(v[c & 1]);
      if (c + 1 < 4) tmem_ld_x32(taddr + (uint32_t)((c + 1) * 32), v[(c + 1) & 1]);
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        const uint32_t pa = pack_bf16x2(__uint_as_float(v[c & 1][2 * i]) * rs, __uint_as_float(v[c & 1][2 * i + 1]) * rs);
        const uint32_t pb = pack_bf16x2(__uint_as_float(v[c & 1][2 * i + 2]) * rs, __uint_as_float(v[c & 1][2 * i + 3]) * rs);
        pk[i] = pa;
        pk[i + 1] = pb;
        const float a0 = bf16_lo(pa), a1 = bf16_hi(pa), b0 = bf16_lo(pb), b1 = bf16_hi(pb);
        ss0 = fmaf(a0, a0, ss0);
        ss1 = fmaf(a1, a1, ss1);
        ss2 = fmaf(b0, b0, ss2);
        ss3 = fmaf(b1, b1, ss3);
      }
      tmem_st_x16(taddr + (uint32_t)(c * 16), pk);
    }
    tmem_st_wait();
  }
  const float r = 1.0f / sqrtf(((ss0 + ss1) + (ss2 + ss3)) * (1.0f / 128.0f) + g.qk_eps);
  const __nv_bfloat16* wp = head < g.qk_Hq ? g.qk_qw : g.qk_kw;
  // The table is chunk-major: chunk q of position s is 32 bytes (8 cos then 8 sin values of elements 8q..8q+7;
  // cos[i] == cos[i + 64] so the first 64 elements suffice). The lanes of a warp are consecutive rows, hence
  // consecutive positions, so each of these loads is one contiguous kilobyte per warp.
  const __nv_bfloat16* tp = g.qk_rope + (int64_t)(valid ? rope_position(g, row) : 0) * 16;
  // ---- sweep 2: 16 elements [16t, 16t+16) and their partners [64+16t, 64+16t+16) per step, as packed pairs:
  //      words [8t, 8t+8) and [32+8t, 32+8t+8) of the region written above ----
  uint32_t lo[2][8], hi[2][8];
  tmem_ld_x8(taddr, lo[0]);
  tmem_ld_x8(taddr + 32u, hi[0]);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint32_t cs[2][8];
    ld_global_nc_v8(tp + (int64_t)(2 * t) * g.qk_S * 16, cs[0]);
    ld_global_nc_v8(tp + (int64_t)(2 * t + 1) * g.qk_S * 16, cs[1]);
    const uint4 wl0 = __ldg(reinterpret_cast<const uint4*>(wp + 16 * t));
    const uint4 wl1 = __ldg(reinterpret_cast<const uint4*>(wp + 16 * t + 8));
    const uint4 wh0 = __ldg(reinterpret_cast<const uint4*>(wp + 64 + 16 * t));
    const uint4 wh1 = __ldg(reinterpret_cast<const uint4*>(wp + 64 + 16 * t + 8));
    const uint32_t wlo[8] = {wl0.x, wl0.y, wl0.z, wl0.w, wl1.x, wl1.y, wl1.z, wl1.w};
    const uint32_t whi[8] = {wh0.x, wh0.y, wh0.z, wh0.w, wh1.x, wh1.y, wh1.z, wh1.w};
    tmem_ld_wait_regs8x2(lo[t & 1], hi[t & 1]);
    if (t + 1 < 4) {
      tmem_ld_x8(taddr + (uint32_t)((t + 1) * 8), lo[(t + 1) & 1]);
      tmem_ld_x8(taddr + 32u + (uint32_t)((t + 1) * 8), hi[(t + 1) & 1]);
    }
    uint32_t olo[8], ohi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {   // pair j of this step: elements 16t + 2j, 16t + 2j + 1 and their partners
      const uint32_t pl = lo[t & 1][j];
      const uint32_t ph = hi[t & 1][j];
      const __nv_bfloat162 nl = __floats2bfloat162_rn(bf16_lo(pl) * r, bf16_hi(pl) * r);
      const __nv_bfloat162 nh = __floats2bfloat162_rn(bf16_lo(ph) * r, bf16_hi(ph) * r);
      const __nv_bfloat162 xl = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&wlo[j]), nl);
      const __nv_bfloat162 xh = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&whi[j]), nh);
      const uint32_t* cc = cs[j >> 2];          // cos of elements 8q..8q+7 in words 0..3, sin in words 4..7
      const __nv_bfloat162 c2 = *reinterpret_cast<const __nv_bfloat162*>(&cc[j & 3]);
      const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&cc[4 + (j & 3)]);
      const uint32_t xh_bits = *reinterpret_cast<const uint32_t*>(&xh) ^ 0x80008000u;
      const __nv_bfloat162 neg_xh = *reinterpret_cast<const __nv_bfloat162*>(&xh_bits);
      const __nv_bfloat162 yl = __hadd2_rn(__hmul2_rn(xl, c2), __hmul2_rn(neg_xh, s2));
      const __nv_bfloat162 yh = __hadd2_rn(__hmul2_rn(xh, c2), __hmul2_rn(xl, s2));
      olo[j] = *reinterpret_cast<const uint32_t*>(&yl);
      ohi[j] = *reinterpret_cast<const uint32_t*>(&yh);
    }
    if (valid) {
      st_global_v8(out + 16 * t, olo);
      st_global_v8(out + 64 + 16 * t, ohi);
    }
  }
}

// Drains one accumulator (NCHUNK x 32 columns of this thread's row) from tensor memory through the epilogue. The load
// of chunk c+1 is in flight while chunk c is converted and stored.
template <int NCHUNK, int EPI = -1, bool FAST = false>
__device__ __forceinline__ void epilogue_drain(const GemmArgs& g, uint32_t taddr, int row, int n0) {
  // row scale of a folded RMSNorm on the input side (1 when there is none)
  float rs = 1.0f;
  if (g.ss_in != nullptr && (FAST || row < g.M)) {
    const float* pr = g.ss_in + (int64_t)row * g.ss_in_segs;  // the row's partial sums are contiguous
    float tot = 0.f;
    if (g.ss_in_segs == 8) {
      uint32_t u[8];
      if (g.coherent) ld_global_cg_v8(pr, u);
      else ld_global_nc_v8(pr, u);
      tot = ((__uint_as_float(u[0]) + __uint_as_float(u[1])) + (__uint_as_float(u[2]) + __uint_as_float(u[3]))) +
            ((__uint_as_float(u[4]) + __uint_as_float(u[5])) + (__uint_as_float(u[6]) + __uint_as_float(u[7])));
    } else {
      for (int sg = 0; sg < g.ss_in_segs; ++sg) tot += g.coherent ? __ldcg(pr + sg) : __ldg(pr + sg);
    }
    rs = 1.0f / sqrtf(tot * g.ss_inv_dim + g.ss_eps);
  }
  if (epi_of<EPI>(g) == EMK_EPI_QKNORM_ROPE_INTERNAL) {
#pragma unroll 1
    for (int hd = 0; hd < NCHUNK / 4; ++hd)
      epilogue_head_qknorm_rope<FAST>(g, taddr + (uint32_t)(hd * 128), row, n0 + hd * 128, rs);
    return;
  }
  uint32_t r[2][32];
  float ss = 0.f;
  tmem_ld_x32(taddr, r[0]);
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c) {
    tmem_ld_wait_regs(r[c & 1]);
    if (c + 1 < NCHUNK) tmem_ld_x32(taddr + (uint32_t)((c + 1) * 32), r[(c + 1) & 1]);
    ss += epilogue_store32<EPI, FAST>(g, r[c & 1], row, n0 + c * 32, rs);
  }
  if (g.ss_out != nullptr && (FAST || row < g.M)) {
    // this thread owns columns [n0, n0 + 32*NCHUNK): its total goes to the first 128-column slot it covers, zeros to
    // the others
    const int slot0 = n0 >> 7;
    const int nslots = (g.N + 127) >> 7;
#pragma unroll
    for (int k = 0; k < (NCHUNK * 32 + 127) / 128; ++k)
      if (slot0 + k < nslots) g.ss_out[(int64_t)row * nslots + slot0 + k] = k == 0 ? ss : 0.f;
  }
}

}  // namespace emk
