// Bandwidth-bound row kernels: RMSNorm forward / backward (with the depth modulation of the
// residual stream folded in), casts, column sums and the embedding gather / scatter.
//
// One warp owns one row; a lane owns columns {lane*4 + 128*i}.  Row statistics are FP32
// (the reference norm, warpstate/model.py:22-28; its Triton twin ops/activation_execution.py:96-158).
// Weight-gradient column sums are accumulated per lane in registers, reduced across the warps
// of a block in shared memory and written as one partial row per block; a second kernel adds the
// partial rows in a fixed order, so the result does not depend on scheduling.
#include "ws_ptx.cuh"
#include "ws_api.h"
#include "ws_launch.h"

namespace ws {

extern "C" void ws_count_launch(void);

constexpr int ROW_WARPS = 8;
constexpr int ROW_THREADS = ROW_WARPS * 32;
constexpr int MAX_CHUNKS = 16;  // d <= 2048 for the register-accumulating backward

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  uint2 o;
  o.x = pack_bf16x2(v.x, v.y);
  o.y = pack_bf16x2(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = o;
}

// --------------------------------------------------------------------------- RMSNorm forward
// x_mod = x * (1 + col_scale) + col_bias (when given); z = bf16(x_mod * rstd * w).
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ col_scale,
                   const float* __restrict__ col_bias, const float* __restrict__ w, float eps, int rows,
                   int d, T* __restrict__ xmod_out, __nv_bfloat16* __restrict__ z,
                   float* __restrict__ rstd_out) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < rows; row += gridDim.x * ROW_WARPS) {
    const T* xr = x + static_cast<size_t>(row) * d;
    float ss = 0.f;
    for (int c = lane * 4; c < d; c += 128) {
      float4 v = ld4(xr + c);
      if (col_scale != nullptr) {
        const float4 s = ld4(col_scale + c), b = ld4(col_bias + c);
        v.x = v.x * (1.f + s.x) + b.x; v.y = v.y * (1.f + s.y) + b.y;
        v.z = v.z * (1.f + s.z) + b.z; v.w = v.w * (1.f + s.w) + b.w;
        if (sizeof(T) == 2) { v.x = bf16_round(v.x); v.y = bf16_round(v.y); v.z = bf16_round(v.z); v.w = bf16_round(v.w); }
      }
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / static_cast<float>(d) + eps);
    if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
    for (int c = lane * 4; c < d; c += 128) {
      float4 v = ld4(xr + c);
      if (col_scale != nullptr) {
        const float4 s = ld4(col_scale + c), b = ld4(col_bias + c);
        v.x = v.x * (1.f + s.x) + b.x; v.y = v.y * (1.f + s.y) + b.y;
        v.z = v.z * (1.f + s.z) + b.z; v.w = v.w * (1.f + s.w) + b.w;
        if (sizeof(T) == 2) { v.x = bf16_round(v.x); v.y = bf16_round(v.y); v.z = bf16_round(v.z); v.w = bf16_round(v.w); }
      }
      if (xmod_out != nullptr) st4(xmod_out + static_cast<size_t>(row) * d + c, v);
      const float4 ww = ld4(w + c);
      float4 o;
      if (sizeof(T) == 2) {  // BF16 stream: round x_hat and w first, as an eager BF16 norm does
        o.x = bf16_round(v.x * rstd) * bf16_round(ww.x); o.y = bf16_round(v.y * rstd) * bf16_round(ww.y);
        o.z = bf16_round(v.z * rstd) * bf16_round(ww.z); o.w = bf16_round(v.w * rstd) * bf16_round(ww.w);
      } else {
        o.x = v.x * rstd * ww.x; o.y = v.y * rstd * ww.y; o.z = v.z * rstd * ww.z; o.w = v.w * rstd * ww.w;
      }
      st4(z + static_cast<size_t>(row) * d + c, o);
    }
  }
}

// The same with the row held in registers between the two passes (d = 128 * CHUNKS known at compile time):
// x is read from memory once, and all CHUNKS loads of a lane are in flight together.
template <typename T, int CHUNKS>
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_fwd_rows_kernel(const T* __restrict__ x, const float* __restrict__ col_scale,
                        const float* __restrict__ col_bias, const float* __restrict__ w, float eps, int rows,
                        T* __restrict__ xmod_out, __nv_bfloat16* __restrict__ z, float* __restrict__ rstd_out) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int d = 128 * CHUNKS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < rows; row += gridDim.x * ROW_WARPS) {
    const T* xr = x + static_cast<size_t>(row) * d;
    float4 v[CHUNKS];
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) v[i] = ld4(xr + i * 128 + lane * 4);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      if (col_scale != nullptr) {
        const int c = i * 128 + lane * 4;
        const float4 s = ld4(col_scale + c), b = ld4(col_bias + c);
        v[i].x = v[i].x * (1.f + s.x) + b.x; v[i].y = v[i].y * (1.f + s.y) + b.y;
        v[i].z = v[i].z * (1.f + s.z) + b.z; v[i].w = v[i].w * (1.f + s.w) + b.w;
        if (sizeof(T) == 2) {
          v[i].x = bf16_round(v[i].x); v[i].y = bf16_round(v[i].y); v[i].z = bf16_round(v[i].z); v[i].w = bf16_round(v[i].w);
        }
      }
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / static_cast<float>(d) + eps);
    if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const int c = i * 128 + lane * 4;
      if (xmod_out != nullptr) st4(xmod_out + static_cast<size_t>(row) * d + c, v[i]);
      const float4 ww = ld4(w + c);
      float4 o;
      if (sizeof(T) == 2) {  // BF16 stream: round x_hat and w first, as an eager BF16 norm does
        o.x = bf16_round(v[i].x * rstd) * bf16_round(ww.x); o.y = bf16_round(v[i].y * rstd) * bf16_round(ww.y);
        o.z = bf16_round(v[i].z * rstd) * bf16_round(ww.z); o.w = bf16_round(v[i].w * rstd) * bf16_round(ww.w);
      } else {
        o.x = v[i].x * rstd * ww.x; o.y = v[i].y * rstd * ww.y; o.z = v[i].z * rstd * ww.z; o.w = v[i].w * rstd * ww.w;
      }
      st4(z + static_cast<size_t>(row) * d + c, o);
    }
  }
}

// --------------------------------------------------------------------------- RMSNorm backward
// dxn = rstd * (dz*w - x_hat * mean(dz*w*x_hat));  out = (dres + dxn) * (1 + out_scale)
// dw_partial[block] = sum over the block's rows of dz * x_hat.
//
// Column-owner layout: thread t owns columns 8t .. 8t+7 (256 threads cover d <= 2048) and the
// block walks over groups of RB_ROWS rows, so every operand is read from global memory exactly
// once with 16/32-byte coalesced accesses, the per-row mean needs one block reduction per group
// (double-buffered, one __syncthreads), and the weight-gradient column sums stay in 8 registers.
constexpr int RB_ROWS = 2;

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&v)[8]) {
  const float4 a = ld4(p), b = ld4(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&v)[8]) {
  st4(p, make_float4(v[0], v[1], v[2], v[3]));
  st4(p + 4, make_float4(v[4], v[5], v[6], v[7]));
}

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS, 3)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dz, const T* __restrict__ x,
                   const float* __restrict__ rstd_in, const float* __restrict__ w,
                   const T* __restrict__ dres, const float* __restrict__ out_scale, int rows, int d,
                   T* __restrict__ dx_out, __nv_bfloat16* __restrict__ dx_bf16,
                   float* __restrict__ dw_partial) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[2][RB_ROWS][ROW_WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = threadIdx.x * 8;
  const bool active = c < d;
  const float inv_d = 1.0f / static_cast<float>(d);
  float wv[8], sv[8], acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { wv[j] = 0.f; sv[j] = 1.f; acc[j] = 0.f; }
  if (active) {
    ld8(w + c, wv);
    if (out_scale != nullptr) {
      ld8(out_scale + c, sv);
#pragma unroll
      for (int j = 0; j < 8; ++j) sv[j] += 1.f;
    }
  }
  int it = 0;
  for (int row0 = blockIdx.x * RB_ROWS; row0 < rows; row0 += gridDim.x * RB_ROWS, ++it) {
    float g[RB_ROWS][8], xh[RB_ROWS][8], rs[RB_ROWS], part[RB_ROWS];
#pragma unroll
    for (int r = 0; r < RB_ROWS; ++r) {
      const int row = row0 + r;
      part[r] = 0.f;
      rs[r] = 0.f;
      if (row < rows && active) {
        const size_t base = static_cast<size_t>(row) * d + c;
        ld8(dz + base, g[r]);
        ld8(x + base, xh[r]);
        rs[r] = rstd_in[row];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) { g[r][j] = 0.f; xh[r][j] = 0.f; }
      }
    }
#pragma unroll
    for (int r = 0; r < RB_ROWS; ++r) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[r][j] *= rs[r];
        part[r] += g[r][j] * wv[j] * xh[r][j];
      }
      part[r] = warp_sum(part[r]);
      if (lane == 0) red[it & 1][r][warp] = part[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RB_ROWS; ++r) {
      const int row = row0 + r;
      if (row < rows && active) {
        float dot = 0.f;
#pragma unroll
        for (int wi = 0; wi < ROW_WARPS; ++wi) dot += red[it & 1][r][wi];
        dot *= inv_d;  // mean(dz * w * x_hat)
        const size_t base = static_cast<size_t>(row) * d + c;
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[j] += g[r][j] * xh[r][j];
          o[j] = rs[r] * (g[r][j] * wv[j] - xh[r][j] * dot);
        }
        if (dres != nullptr) {
          float rr[8];
          ld8(dres + base, rr);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rr[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= sv[j];
        st8(dx_out + base, o);
        if (dx_bf16 != nullptr) st8(dx_bf16 + base, o);
      }
    }
  }
  if (dw_partial != nullptr && active) st8(dw_partial + static_cast<size_t>(blockIdx.x) * d + c, acc);
}

// --------------------------------------------------------------------------- column sums
// partial_a[block] = sum_rows a ; partial_ab[block] = sum_rows a*b  (a, b: [rows, d])
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
colsum2_kernel(const T* __restrict__ a, const T* __restrict__ b, int rows, int d,
               float* __restrict__ partial_a, float* __restrict__ partial_ab) {
  pdl_launch_dependents();
  pdl_wait();
  // thread t owns columns t*4 .. t*4+3 of a 1024-wide panel; rows strided over blocks
  for (int c0 = 0; c0 < d; c0 += ROW_THREADS * 4) {
    const int c = c0 + threadIdx.x * 4;
    if (c >= d) continue;
    float4 sa = make_float4(0.f, 0.f, 0.f, 0.f), sab = sa;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      const float4 va = ld4(a + static_cast<size_t>(row) * d + c);
      sa.x += va.x; sa.y += va.y; sa.z += va.z; sa.w += va.w;
      if (b != nullptr) {
        const float4 vb = ld4(b + static_cast<size_t>(row) * d + c);
        sab.x += va.x * vb.x; sab.y += va.y * vb.y; sab.z += va.z * vb.z; sab.w += va.w * vb.w;
      }
    }
    st4(partial_a + static_cast<size_t>(blockIdx.x) * d + c, sa);
    if (b != nullptr) st4(partial_ab + static_cast<size_t>(blockIdx.x) * d + c, sab);
  }
}

// out[c] = beta*out[c] + scale(c) * sum_p partial[p][c];  scale(c) = 1/(1+inv_scale[c]) if given
// One block per 32 columns; warp w sums parts w, w+8, ... (independent 128-byte loads in
// flight), then the eight warp sums are combined in a fixed order: the result is deterministic.
constexpr int FIN_COLS = 32;
__global__ void __launch_bounds__(ROW_THREADS)
colsum_finalize_kernel(const float* __restrict__ partial, int parts, int d,
                       const float* __restrict__ inv_scale, float beta, float* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[ROW_WARPS][FIN_COLS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * FIN_COLS + lane;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < d) {
    int p = warp;
    for (; p + 3 * ROW_WARPS < parts; p += 4 * ROW_WARPS) {
      s0 += partial[static_cast<size_t>(p) * d + c];
      s1 += partial[static_cast<size_t>(p + ROW_WARPS) * d + c];
      s2 += partial[static_cast<size_t>(p + 2 * ROW_WARPS) * d + c];
      s3 += partial[static_cast<size_t>(p + 3 * ROW_WARPS) * d + c];
    }
    for (; p < parts; p += ROW_WARPS) s0 += partial[static_cast<size_t>(p) * d + c];
  }
  red[warp][lane] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (warp == 0 && c < d) {
    float s = 0.f;
#pragma unroll
    for (int wi = 0; wi < ROW_WARPS; ++wi) s += red[wi][lane];
    if (inv_scale != nullptr) {
      const float den = 1.f + inv_scale[c];
      s = den != 0.f ? s / den : 0.f;
    }
    out[c] = (beta != 0.f ? beta * out[c] : 0.f) + s;
  }
}

// --------------------------------------------------------------------------- casts
__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                     size_t n4) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    st4(out + i * 4, ld4(in + i * 4));
  }
}

// --------------------------------------------------------------------------- embedding
// out[row] = table[ids[row]] ; table FP32 (master) or BF16, out FP32 or BF16
template <typename TT, typename TO>
__global__ void __launch_bounds__(ROW_THREADS)
embed_fwd_kernel(const long long* __restrict__ ids, const TT* __restrict__ table, int rows, int d,
                 int vocab, TO* __restrict__ out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < rows; row += gridDim.x * ROW_WARPS) {
    long long id = ids[row];
    if (id < 0 || id >= vocab) id = 0;
    const TT* src = table + static_cast<size_t>(id) * d;
    for (int c = lane * 4; c < d; c += 128) st4(out + static_cast<size_t>(row) * d + c, ld4(src + c));
  }
}

// Deterministic embedding backward: rows were sorted by token id on the host side of the op
// (`order` = argsort of ids).  The unit of work is (position p of the sorted ids, 128-column chunk): a warp
// works only if a run of equal ids starts at p, and then adds that chunk of all gradient rows of the run, in
// order, into the FP32 gradient table - no atomics, run-to-run identical.  A run is therefore shared by d / 128
// warps, which keeps a run of thousands of equal ids (the padding of a fine-tuning batch) from being one
// warp's serial work.  The runs are found on the device, so the host needs no count of distinct tokens (which
// would cost a device-to-host read, and with it a drained launch queue, in every micro-batch).
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
embed_bwd_kernel(const T* __restrict__ dx, const long long* __restrict__ sorted_ids,
                 const long long* __restrict__ order, int rows, int d, int vocab, float* __restrict__ grad_table) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = d / 128;
  const long long units = static_cast<long long>(rows) * chunks;
  for (long long unit = blockIdx.x * ROW_WARPS + warp; unit < units; unit += static_cast<long long>(gridDim.x) * ROW_WARPS) {
    const int begin = static_cast<int>(unit / chunks);
    const int c = static_cast<int>(unit % chunks) * 128 + lane * 4;
    const long long id = sorted_ids[begin];
    if (begin > 0 && sorted_ids[begin - 1] == id) continue;  // not the head of a run
    if (id < 0 || id >= vocab) continue;
    // the end of the run, 32 positions per step
    int end = begin + 1;
    for (;;) {
      const int at = end + lane;
      const bool same = at < rows && sorted_ids[at] == id;
      const unsigned mask = __ballot_sync(0xffffffffu, same);
      if (mask == 0xffffffffu) {
        end += 32;
        continue;
      }
      end += __ffs(~mask) - 1;
      break;
    }
    float* dst = grad_table + static_cast<size_t>(id) * d + c;
    float4 s = ld4(dst);
    int j = begin;
    for (; j + 4 <= end; j += 4) {  // four independent loads in flight; the sum keeps the row order
      const float4 v0 = ld4(dx + static_cast<size_t>(order[j]) * d + c);
      const float4 v1 = ld4(dx + static_cast<size_t>(order[j + 1]) * d + c);
      const float4 v2 = ld4(dx + static_cast<size_t>(order[j + 2]) * d + c);
      const float4 v3 = ld4(dx + static_cast<size_t>(order[j + 3]) * d + c);
      s.x += v0.x; s.y += v0.y; s.z += v0.z; s.w += v0.w;
      s.x += v1.x; s.y += v1.y; s.z += v1.z; s.w += v1.w;
      s.x += v2.x; s.y += v2.y; s.z += v2.z; s.w += v2.w;
      s.x += v3.x; s.y += v3.y; s.z += v3.z; s.w += v3.w;
    }
    for (; j < end; ++j) {
      const float4 v = ld4(dx + static_cast<size_t>(order[j]) * d + c);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    st4(dst, s);
  }
}

static int row_grid(int rows) {
  int blocks = (rows + ROW_WARPS - 1) / ROW_WARPS;
  const int cap = 148 * 8;
  return blocks < cap ? (blocks > 0 ? blocks : 1) : cap;
}

}  // namespace ws

using namespace ws;

extern "C" int ws_rmsnorm_fwd(const void* x, int x_bf16, const float* col_scale, const float* col_bias,
                              const float* w, float eps, int rows, int d, void* xmod_out, void* z,
                              float* rstd, cudaStream_t stream) {
  if (d % 128 != 0 || rows <= 0) return -1;
  const int grid = row_grid(rows);
  if (d == 2048) {  // the model's width: the row stays in registers
    if (x_bf16)
      launch_dependent(rmsnorm_fwd_rows_kernel<__nv_bfloat16, 16>, dim3(grid), dim3(ROW_THREADS), 0, stream, (const __nv_bfloat16*)x,
                       col_scale, col_bias, w, eps, rows, (__nv_bfloat16*)xmod_out, (__nv_bfloat16*)z, rstd);
    else
      launch_dependent(rmsnorm_fwd_rows_kernel<float, 16>, dim3(grid), dim3(ROW_THREADS), 0, stream, (const float*)x, col_scale,
                       col_bias, w, eps, rows, (float*)xmod_out, (__nv_bfloat16*)z, rstd);
    ws_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  if (x_bf16)
    launch_dependent(rmsnorm_fwd_kernel<__nv_bfloat16>, dim3(grid), dim3(ROW_THREADS), 0, stream, (const __nv_bfloat16*)x, col_scale, col_bias, w, eps, rows, d, (__nv_bfloat16*)xmod_out,
        (__nv_bfloat16*)z, rstd);
  else
    launch_dependent(rmsnorm_fwd_kernel<float>, dim3(grid), dim3(ROW_THREADS), 0, stream, (const float*)x, col_scale, col_bias, w, eps, rows, d, (float*)xmod_out, (__nv_bfloat16*)z, rstd);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Number of partial rows ws_rmsnorm_bwd writes (the caller sizes dw_partial as parts*d floats).
constexpr int kRmsBwdMaxParts = 148 * 3;  // three resident blocks per SM
extern "C" int ws_rmsnorm_bwd_parts(int rows) {
  int blocks = (rows + RB_ROWS - 1) / RB_ROWS;
  return blocks < kRmsBwdMaxParts ? (blocks > 0 ? blocks : 1) : kRmsBwdMaxParts;
}

extern "C" int ws_rmsnorm_bwd(const void* dz, const void* x, int x_bf16, const float* rstd, const float* w,
                              const void* dres, const float* out_scale, int rows, int d, void* dx_out,
                              void* dx_bf16, float* dw_partial, cudaStream_t stream) {
  if (d % 128 != 0 || d > ROW_THREADS * 8 || rows <= 0) return -1;
  const int grid = ws_rmsnorm_bwd_parts(rows);
  if (x_bf16)
    launch_dependent(rmsnorm_bwd_kernel<__nv_bfloat16>, dim3(grid), dim3(ROW_THREADS), 0, stream, (const __nv_bfloat16*)dz, (const __nv_bfloat16*)x, rstd, w, (const __nv_bfloat16*)dres, out_scale,
        rows, d, (__nv_bfloat16*)dx_out, (__nv_bfloat16*)dx_bf16, dw_partial);
  else
    launch_dependent(rmsnorm_bwd_kernel<float>, dim3(grid), dim3(ROW_THREADS), 0, stream, (const __nv_bfloat16*)dz, (const float*)x, rstd, w, (const float*)dres, out_scale, rows, d,
        (float*)dx_out, (__nv_bfloat16*)dx_bf16, dw_partial);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int ws_colsum_parts(int rows) { return rows < 296 ? (rows > 0 ? rows : 1) : 296; }

extern "C" int ws_colsum2(const void* a, const void* b, int is_bf16, int rows, int d, float* partial_a,
                          float* partial_ab, cudaStream_t stream) {
  if (d % 4 != 0 || rows <= 0) return -1;
  const int grid = ws_colsum_parts(rows);
  if (is_bf16)
    launch_dependent(colsum2_kernel<__nv_bfloat16>, dim3(grid), dim3(ROW_THREADS), 0, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, rows, d, partial_a, partial_ab);
  else
    launch_dependent(colsum2_kernel<float>, dim3(grid), dim3(ROW_THREADS), 0, stream, (const float*)a, (const float*)b, rows, d,
                                                            partial_a, partial_ab);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int ws_colsum_finalize(const float* partial, int parts, int d, const float* inv_scale, float beta,
                                  float* out, cudaStream_t stream) {
  launch_dependent(colsum_finalize_kernel, dim3((d + FIN_COLS - 1) / FIN_COLS), dim3(ROW_THREADS), 0, stream, partial, parts, d, inv_scale, beta, out);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int ws_cast_f32_bf16(const float* in, void* out, size_t n, cudaStream_t stream) {
  if (n % 4 != 0) return -1;
  if (n == 0) return 0;
  const size_t n4 = n / 4;
  size_t blocks = (n4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_dependent(cast_f32_bf16_kernel, dim3((int)blocks), dim3(256), 0, stream, in, (__nv_bfloat16*)out, n4);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int ws_embed_fwd(const long long* ids, const void* table, int table_bf16, int rows, int d,
                            int vocab, void* out, int out_bf16, cudaStream_t stream) {
  if (d % 4 != 0 || rows <= 0) return -1;
  const int grid = row_grid(rows);
  if (table_bf16 && out_bf16)
    embed_fwd_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, ROW_THREADS, 0, stream>>>(
        ids, (const __nv_bfloat16*)table, rows, d, vocab, (__nv_bfloat16*)out);
  else if (!table_bf16 && out_bf16)
    embed_fwd_kernel<float, __nv_bfloat16><<<grid, ROW_THREADS, 0, stream>>>(
        ids, (const float*)table, rows, d, vocab, (__nv_bfloat16*)out);
  else if (!table_bf16 && !out_bf16)
    embed_fwd_kernel<float, float><<<grid, ROW_THREADS, 0, stream>>>(ids, (const float*)table, rows, d,
                                                                     vocab, (float*)out);
  else if (table_bf16 && !out_bf16)  // BF16 table of a frozen model feeding an FP32 residual stream
    embed_fwd_kernel<__nv_bfloat16, float><<<grid, ROW_THREADS, 0, stream>>>(ids, (const __nv_bfloat16*)table, rows,
                                                                              d, vocab, (float*)out);
  else
    return -3;
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int ws_embed_bwd(const void* dx, int dx_bf16, const long long* sorted_ids, const long long* order, int rows,
                            int d, int vocab, float* grad_table, cudaStream_t stream) {
  if (d % 128 != 0 || rows <= 0 || vocab <= 0) return -1;
  const int grid = 148 * 8;
  if (dx_bf16)
    embed_bwd_kernel<__nv_bfloat16><<<grid, ROW_THREADS, 0, stream>>>((const __nv_bfloat16*)dx, sorted_ids, order, rows,
                                                                      d, vocab, grad_table);
  else
    embed_bwd_kernel<float><<<grid, ROW_THREADS, 0, stream>>>((const float*)dx, sorted_ids, order, rows, d, vocab,
                                                              grad_table);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// =============================================================================== no-allocation entry
// RMSNorm backward whose partial-sum scratch is part of the library image (see
// ws_static_scratch.h for who needs this and for the sharing rules).
#include "ws_static_scratch.h"
#include <mutex>

// Lives in every GPU that loads this library until the process exits.  In host code this name is
// only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_static_scratch[WS_STATIC_SCRATCH_FLOATS];
// The array is exactly what the largest accepted problem writes: the most partial rows the kernel ever
// uses times the widest row it accepts.
static_assert(WS_STATIC_SCRATCH_FLOATS == kRmsBwdMaxParts * 128 * MAX_CHUNKS,
              "WS_STATIC_SCRATCH_FLOATS must equal the maximum number of partial rows times the maximum width");

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device, looked up once per device.
int static_scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return WS_STATIC_ERR_SYMBOL;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return WS_STATIC_ERR_SYMBOL;
    g_scratch_addr[dev] = static_cast<float*>(ptr);
  }
  *out = g_scratch_addr[dev];
  return 0;
}
}  // namespace

extern "C" const char* ws_static_scratch_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case WS_STATIC_ERR_BAD_SHAPE: return "rows must be positive and d a multiple of 128 not above 2048";
    case WS_STATIC_ERR_LAUNCH: return "kernel launch failed";
    case WS_STATIC_ERR_TOO_LARGE: return "problem needs more partial sums than the built-in scratch array holds "
                                         "(cannot happen while d <= 2048 is enforced; kept as a guard)";
    case WS_STATIC_ERR_SYMBOL: return "could not resolve the device address of the built-in scratch array";
    default: return "unknown error";
  }
}

extern "C" int ws_rmsnorm_bwd_static(const void* dz, const void* x, int x_bf16, const float* rstd, const float* w,
                                     const void* dres, const float* out_scale, int rows, int d, void* dx_out,
                                     void* dx_bf16, float* dw_out, cudaStream_t stream) {
  if (d % 128 != 0 || d > 128 * MAX_CHUNKS || rows <= 0) return WS_STATIC_ERR_BAD_SHAPE;
  const int parts = ws_rmsnorm_bwd_parts(rows);
  if (static_cast<long long>(parts) * d > static_cast<long long>(WS_STATIC_SCRATCH_FLOATS)) return WS_STATIC_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // Every partial row that the reduction reads below is written by the kernel first, so the
  // previous call's contents never leak into this result.
  if (x_bf16)
    launch_dependent(rmsnorm_bwd_kernel<__nv_bfloat16>, dim3(parts), dim3(ROW_THREADS), 0, stream, (const __nv_bfloat16*)dz, (const __nv_bfloat16*)x, rstd, w, (const __nv_bfloat16*)dres, out_scale,
        rows, d, (__nv_bfloat16*)dx_out, (__nv_bfloat16*)dx_bf16, scratch);
  else
    launch_dependent(rmsnorm_bwd_kernel<float>, dim3(parts), dim3(ROW_THREADS), 0, stream, (const __nv_bfloat16*)dz, (const float*)x, rstd, w, (const float*)dres, out_scale, rows, d,
        (float*)dx_out, (__nv_bfloat16*)dx_bf16, scratch);
  ws_count_launch();
  launch_dependent(colsum_finalize_kernel, dim3((d + FIN_COLS - 1) / FIN_COLS), dim3(ROW_THREADS), 0, stream, scratch, parts, d, nullptr, 0.f, dw_out);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : WS_STATIC_ERR_LAUNCH;
}
