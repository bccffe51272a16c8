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
  int* status;
  unsigned long long limit_ns;
};

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

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

// Epilogue for 32 accumulator columns [col0, col0+32) of one output row held by this thread.
__device__ __forceinline__ void epilogue_store32(const GemmArgs& g, const uint32_t* r, int row, int col0) {
  if (row >= g.M || col0 >= g.N) return;
  if (g.epi == EMK_EPI_SWIGLU) {
    // columns are (gate, up) pairs; 16 outputs
    __nv_bfloat16* out = g.y + (int64_t)row * g.ldy + (col0 >> 1);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      if (col0 + q * 16 < g.N) {
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int idx = q * 16 + j * 4 + e * 2;
            const float gate = bf16_round(__uint_as_float(r[idx]));
            const float up = bf16_round(__uint_as_float(r[idx + 1]));
            v[e] = bf16_round(silu_f(gate)) * up;
          }
          o[j] = pack_bf16x2(v[0], v[1]);
        }
        *reinterpret_cast<uint4*>(out + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    return;
  }
  __nv_bfloat16* out = g.y + (int64_t)row * g.ldy + col0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int col = col0 + q * 8;
    if (col < g.N) {
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[q * 8 + e]);
      if (g.scale != nullptr) {
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(g.scale + col));
        const float4 s1 = __ldg(reinterpret_cast<const float4*>(g.scale + col + 4));
        v[0] *= s0.x; v[1] *= s0.y; v[2] *= s0.z; v[3] *= s0.w;
        v[4] *= s1.x; v[5] *= s1.y; v[6] *= s1.z; v[7] *= s1.w;
      }
      if (g.epi == EMK_EPI_RESIDUAL) {
        const uint4 rv = *reinterpret_cast<const uint4*>(g.residual + (int64_t)row * g.ldy + col);
        const uint32_t rr[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[2 * e] = bf16_round(v[2 * e]) + bf16_lo(rr[e]);
          v[2 * e + 1] = bf16_round(v[2 * e + 1]) + bf16_hi(rr[e]);
        }
      } else if (g.epi == EMK_EPI_BIAS) {
        const uint4 bv = __ldg(reinterpret_cast<const uint4*>(g.residual + col));
        const uint32_t bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[2 * e] += bf16_lo(bb[e]);
          v[2 * e + 1] += bf16_hi(bb[e]);
        }
      }
      uint4 o;
      o.x = pack_bf16x2(v[0], v[1]);
      o.y = pack_bf16x2(v[2], v[3]);
      o.z = pack_bf16x2(v[4], v[5]);
      o.w = pack_bf16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(out + q * 8) = o;
    }
  }
}

}  // namespace emk
