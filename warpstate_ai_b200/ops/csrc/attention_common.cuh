// Shared pieces of the attention / memory kernels: tile geometry (128-token chunks, head_dim 64),
// the 128-byte-swizzled shared-memory tile layout that both TMA and tcgen05 descriptors use, and
// row-per-thread helpers (RoPE with interleaved pairs restarting every chunk, tanh).
#pragma once
#include "ws_ptx.cuh"
#include "ws_tma_host.h"

namespace ws {

constexpr int CHUNK = 128;
constexpr int HD = 64;
constexpr int TILE_BYTES = CHUNK * HD * 2;  // one [128 x 64] BF16 tile, 16 KiB

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}
__device__ __forceinline__ float sigmoid_f(float x) { return sigmoid_fast(x); }

// The arithmetic that two forms of a kernel must share bit for bit is written with explicitly rounded operations,
// so that the compiler's choice of which product to fuse into which addition cannot differ between them.
__device__ __forceinline__ float2 rope_rotate(float2 x, float2 cs) {  // (cos, sin) of the pair's angle
  return make_float2(__fmaf_rn(x.x, cs.x, -__fmul_rn(x.y, cs.y)), __fmaf_rn(x.y, cs.x, __fmul_rn(x.x, cs.y)));
}
// exp2((s - m) * k): the unnormalised softmax weight of a score
__device__ __forceinline__ float softmax_term(float s, float m, float k) { return exp2f(__fmul_rn(__fsub_rn(s, m), k)); }
// g * (o * inv_l) + (1 - g) * (mem / 8)
__device__ __forceinline__ float gate_blend(float g, float o, float inv_l, float mem) {
  return __fmaf_rn(g, __fmul_rn(o, inv_l), __fmul_rn(__fsub_rn(1.f, g), __fmul_rn(mem, 0.125f)));
}

// Address of the 16-byte chunk `j` (8 BF16 columns) of row `r` in a [rows x 64] swizzled tile.
__device__ __forceinline__ uint8_t* tile_chunk(uint8_t* tile, int r, int j) {
  return tile + r * 128 + ((j ^ (r & 7)) << 4);
}

// In place on row `r` of a tile: optional rotary embedding at in-chunk position r (pairs are
// adjacent elements; rope[p*128 + r] = (cos, sin) of pair p at position r -- pair-major, so that
// the 32 rows of a warp read 256 contiguous bytes instead of 32 cache lines), then optional tanh.
__device__ __forceinline__ void rope_tanh_row(uint8_t* tile, int r, const float2* __restrict__ rope,
                                              bool do_rope, bool do_tanh) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4* p = reinterpret_cast<uint4*>(tile_chunk(tile, r, j));
    uint4 v = *p;
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float2 x = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[t]));
      if (do_rope) x = rope_rotate(x, rope[(j * 4 + t) * CHUNK + r]);
      if (do_tanh) {
        x.x = tanh_fast(x.x);
        x.y = tanh_fast(x.y);
      }
      w[t] = pack_bf16x2(x.x, x.y);
    }
    *p = v;
  }
}

// Store 32 BF16 values (16 packed words) of row r, columns [c0, c0+32), into a [128 x 128]
// K-major operand made of two swizzled [128 x 64] tiles (columns 0-63 | 64-127).
__device__ __forceinline__ void store_row_chunk32(uint8_t* tiles, int r, int c0, const uint32_t (&pk)[16]) {
  uint8_t* tile = tiles + (c0 >> 6) * TILE_BYTES;
  const int j0 = (c0 & 63) >> 3;
#pragma unroll
  for (int q = 0; q < 4; ++q)
    *reinterpret_cast<uint4*>(tile_chunk(tile, r, j0 + q)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
}
__device__ __forceinline__ void load_row_chunk32(uint8_t* tiles, int r, int c0, uint32_t (&pk)[16]) {
  uint8_t* tile = tiles + (c0 >> 6) * TILE_BYTES;
  const int j0 = (c0 & 63) >> 3;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 v = *reinterpret_cast<const uint4*>(tile_chunk(tile, r, j0 + q));
    pk[4 * q] = v.x; pk[4 * q + 1] = v.y; pk[4 * q + 2] = v.z; pk[4 * q + 3] = v.w;
  }
}

// Host: 2-D map over a row-major BF16 matrix for [box_rows x box_cols] swizzled tiles.
inline int make_tile_map(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t ld,
                         uint32_t box_cols, uint32_t box_rows) {
  return make_map_bf16(map, base, cols, rows, ld, box_cols, box_rows);
}

}  // namespace ws
