// Forward kernels of the middle of a WarpState core (everything between in_proj and out_proj;
// reference math: warpstate/model.py:124-176), for chunk_size 128 and head_dim 64.
//
// The packed projection qkvgu [tokens, 5d] (Q,K,V,gate,U) is read in place with TMA: a tile of
// one (batch, chunk, head) is the box rows [b*T + n*128, +128) x cols [sel*d + h*64, +64) -- the
// reference's chunkify/permute/contiguous copies do not exist here.
//
//   chunk_writes_kernel : W[b,n,h] = tanh(rope(K))^T tanh(U) / 128            (tcgen05, 64x64 out)
//   memory_scan_kernel  : state seen by chunk n = mix*F_n + (1-mix)*S_n with
//                         F_n = d_f F_{n-1} + (1-d_f) W_{n-1}, F_0 = 0 (FP32, O(N) scan)
//   attn_fwd_kernel     : S = rope(Q) rope(K)^T (tcgen05 -> TMEM), causal softmax by one thread
//                         per row straight out of TMEM, O = P V and Mem = rope(Q) state (tcgen05),
//                         y = sigmoid(g) * O/l + (1 - sigmoid(g)) * Mem/8, stored token-major.
//
// One thread owns one token row (= one TMEM lane): no cross-thread reductions anywhere.
#include "ws_ptx.cuh"
#include "ws_api.h"
#include "ws_launch.h"
#include "attention_common.cuh"

#include <cstdlib>

namespace ws {

extern "C" void ws_count_launch(void);

// =============================================================================== writes
// smem: sK 16K | sU 16K | bars
constexpr int WR_SMEM = 2 * TILE_BYTES + 1024 + 128;

__global__ void __launch_bounds__(128, 6)
chunk_writes_kernel(const __grid_constant__ CUtensorMap tm_qkvgu, const __grid_constant__ CUtensorMap tm_out,
                    const float2* __restrict__ rope, int T, int H, int d, int* error_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sK = smem;
  uint8_t* sU = smem + TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * TILE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_chunks = T / CHUNK;
  const int tile = blockIdx.x;
  const int h = tile % H, n = (tile / H) % n_chunks, b = tile / (H * n_chunks);
  const int row0 = b * T + n * CHUNK;

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  if (tid == 0) {
    mbar_expect_tx(&bars[0], 2 * TILE_BYTES);
    tma_load_2d(sK, &tm_qkvgu, &bars[0], 1 * d + h * HD, row0);
    tma_load_2d(sU, &tm_qkvgu, &bars[0], 4 * d + h * HD, row0);
  }
  bool ok = mbar_wait(&bars[0], 0, abort_flag);
  if (ok) {
    rope_tanh_row(sK, tid, rope, true, true);    // K -> tanh(rope(K))
    rope_tanh_row(sU, tid, rope, false, true);   // U -> tanh(U)
  }
  fence_proxy_async_smem();
  __syncthreads();
  if (tid == 0 && ok) {
    // D[128 x 64]: rows 0..63 = tK^T tU.  A is read MN-major with a zero stride between its two
    // 64-wide atoms, so rows 64..127 repeat rows 0..63 and are ignored.
    constexpr uint32_t idesc = make_idesc_bf16(128, 64, true, true);
#pragma unroll
    for (int k = 0; k < CHUNK / 16; ++k) {
      const uint64_t da = make_smem_desc_sw128(smem_u32(sK) + k * 2048, 0, 1024);
      const uint64_t db = make_smem_desc_sw128(smem_u32(sU) + k * 2048, 0, 1024);
      umma_bf16(tmem, da, db, idesc, k > 0);
    }
    umma_commit(&bars[1]);
  }
  ok = ok && mbar_wait(&bars[1], 0, abort_flag);
  tc_fence_after_sync();
  if (warp < 2) {  // lanes 0..63 hold the result rows
    // Row `tid` goes to two swizzled [64 x 32] FP32 half tiles in the (consumed) K tile's space; each
    // warp then stores its 32 rows of both halves by TMA.
#pragma unroll
    for (int c = 0; c < HD; c += 16) {
      uint32_t r[16];
      tmem_ld_32x32b_x16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        const int col = c + j;
        uint8_t* dst = sK + (col >> 5) * 8192 + tid * 128 + ((((col & 31) >> 2) ^ (tid & 7)) << 4);
        *reinterpret_cast<float4*>(dst) =
            make_float4(__uint_as_float(r[j]) * (1.f / CHUNK), __uint_as_float(r[j + 1]) * (1.f / CHUNK),
                        __uint_as_float(r[j + 2]) * (1.f / CHUNK), __uint_as_float(r[j + 3]) * (1.f / CHUNK));
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if ((tid & 31) == 0) {
      if (ok) {
        tma_store_2d(&tm_out, sK + warp * 4096, 0, tile * HD + warp * 32);
        tma_store_2d(&tm_out, sK + 8192 + warp * 4096, 32, tile * HD + warp * 32);
        tma_store_commit();
      }
      tma_store_wait_read0();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag != 0 && error_flag != nullptr) atomicExch(error_flag, 2);
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 64);
  }
}

// =============================================================================== writes, streaming form
// The same product as chunk_writes_kernel, as one persistent CTA per SM with specialised warps:
//
//   warp 18      producer: TMA loads of the K and U tiles of tile i into stage i % 4 of a ring (4 x 32 KiB)
//   warps 0..15  workers (512 threads): thread (row r, quarter q) turns two of the eight 16-byte pieces of row r of K
//                into tanh(rope(K)) and of U into tanh(U), in place; its 8 (cos, sin) pairs are loaded once, since
//                they depend on the row and the column only.  (With 8 worker warps the kernel issued an instruction
//                in 33 % of the cycles, each warp waiting 8 cycles between two of its own: four warps per scheduler
//                instead of two hide that.)  Worker thread 0 then issues the tile's eight MMAs into
//                TMEM buffer i % 2; their completion frees the ring stage and hands the buffer to the epilogue.
//   warps 16, 17 epilogue (accumulator lanes 0..63): TMEM -> x 1/128 -> swizzled FP32 staging tile -> TMA store
//
// so the loads of the next three tiles, the element-wise work of the current one and the store of the previous
// one overlap; chunk_writes_kernel gets its overlap from six independent CTAs per SM instead, each of which walks
// the chain load -> element-wise -> MMA -> store alone.  Results are bit-identical (same arithmetic, same MMA order).
constexpr int WS_STAGES = 4;
constexpr int WS_THREADS = 19 * 32;
constexpr int WS_SMEM = WS_STAGES * 2 * TILE_BYTES + 2 * 16384 + 1024 + 256;

__global__ void __launch_bounds__(WS_THREADS, 1)
chunk_writes_stream_kernel(const __grid_constant__ CUtensorMap tm_qkvgu, const __grid_constant__ CUtensorMap tm_out,
                           const float2* __restrict__ rope, int T, int H, int d, int tiles, int* error_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* ring = smem;                                   // stage s: K at s * 32 KiB, U 16 KiB behind it
  uint8_t* staging = smem + WS_STAGES * 2 * TILE_BYTES;   // two FP32 [64 x 64] tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * 16384);
  uint64_t* full = bars;                    // [4] tile landed
  uint64_t* empty = bars + WS_STAGES;       // [4] MMAs have read the stage
  uint64_t* tfull = bars + 2 * WS_STAGES;   // [2] accumulator complete
  uint64_t* tempty = tfull + 2;             // [2] accumulator read by both epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_chunks = T / CHUNK;

  if (tid == 0) {
    for (int s = 0; s < WS_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 2);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_qkvgu);
    tma_prefetch_desc(&tm_out);
  }
  if (warp == 16) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  const int first = blockIdx.x, step = gridDim.x;
  if (warp == 18) {
    if (lane == 0) {
      int i = 0;
      for (int tile = first; tile < tiles; tile += step, ++i) {
        const int s = i % WS_STAGES;
        if (!mbar_wait(&empty[s], ((i / WS_STAGES) & 1) ^ 1, abort_flag)) break;
        const int h = tile % H, n = (tile / H) % n_chunks, b = tile / (H * n_chunks);
        const int row0 = b * T + n * CHUNK;
        mbar_expect_tx(&full[s], 2 * TILE_BYTES);
        tma_load_2d(ring + s * 2 * TILE_BYTES, &tm_qkvgu, &full[s], 1 * d + h * HD, row0);
        tma_load_2d(ring + s * 2 * TILE_BYTES + TILE_BYTES, &tm_qkvgu, &full[s], 4 * d + h * HD, row0);
      }
    }
  } else if (warp < 16) {
    const int r = tid & 127, q = tid >> 7;   // row, and which two of its eight pieces
    float2 cs[8];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int t = 0; t < 4; ++t) cs[j * 4 + t] = rope[((q * 2 + j) * 4 + t) * CHUNK + r];
    int i = 0;
    for (int tile = first; tile < tiles; tile += step, ++i) {
      const int s = i % WS_STAGES;
      uint8_t* sK = ring + s * 2 * TILE_BYTES;
      uint8_t* sU = sK + TILE_BYTES;
      const bool ok = mbar_wait(&full[s], (i / WS_STAGES) & 1, abort_flag);
      if (ok) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint4* pk = reinterpret_cast<uint4*>(tile_chunk(sK, r, q * 2 + j));
          uint4* pu = reinterpret_cast<uint4*>(tile_chunk(sU, r, q * 2 + j));
          uint4 kv = *pk, uv = *pu;
          uint32_t* kw = reinterpret_cast<uint32_t*>(&kv);
          uint32_t* uw = reinterpret_cast<uint32_t*>(&uv);
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 x = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&kw[t]));
            const float2 c = cs[j * 4 + t];
            const float2 kr = rope_rotate(x, c);
            kw[t] = pack_bf16x2(tanh_fast(kr.x), tanh_fast(kr.y));
            const float2 u = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&uw[t]));
            uw[t] = pack_bf16x2(tanh_fast(u.x), tanh_fast(u.y));
          }
          *pk = kv;
          *pu = uv;
        }
      }
      fence_proxy_async_smem();
      // the workers' barrier doubles as their vote: if any of them gave up on the tile, all leave together
      uint32_t any_bad;
      asm volatile(
          "{\n"
          ".reg .pred p, q;\n"
          "setp.ne.u32 q, %1, 0;\n"
          "bar.red.or.pred p, 2, 512, q;\n"
          "selp.u32 %0, 1, 0, p;\n"
          "}\n"
          : "=r"(any_bad)
          : "r"(ok ? 0u : 1u)
          : "memory");
      if (any_bad) break;
      if (tid == 0) {
        const int buf = i & 1;
        if (mbar_wait(&tempty[buf], ((i >> 1) & 1) ^ 1, abort_flag)) {
          tc_fence_after_sync();
          // D[128 x 64]: rows 0..63 = tK^T tU.  A is read MN-major with a zero stride between its two 64-wide
          // atoms, so rows 64..127 repeat rows 0..63 and are ignored.
          constexpr uint32_t idesc = make_idesc_bf16(128, 64, true, true);
#pragma unroll
          for (int k = 0; k < CHUNK / 16; ++k)
            umma_bf16(tmem + buf * 64, make_smem_desc_sw128(smem_u32(sK) + k * 2048, 0, 1024),
                      make_smem_desc_sw128(smem_u32(sU) + k * 2048, 0, 1024), idesc, k > 0);
          umma_commit(&empty[s]);
          umma_commit(&tfull[buf]);
        }
      }
    }
  } else {  // warps 16, 17: accumulator lanes 0..31 and 32..63
    const int ew = warp - 16, row = ew * 32 + lane;
    int i = 0;
    for (int tile = first; tile < tiles; tile += step, ++i) {
      const int buf = i & 1;
      uint32_t landed = 0;
      if (lane == 0) landed = mbar_wait(&tfull[buf], (i >> 1) & 1, abort_flag) ? 1u : 0u;
      if (__shfl_sync(0xffffffffu, landed, 0) == 0u) break;   // the whole warp leaves together
      tc_fence_after_sync();
      uint8_t* st = staging + buf * 16384;
      if (lane == 0) tma_store_wait_read0();   // the store issued two tiles ago from this buffer has read it
      __syncwarp();
#pragma unroll
      for (int c = 0; c < HD; c += 16) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(tmem + buf * 64 + (static_cast<uint32_t>(ew * 32) << 16) + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          const int col = c + j;
          uint8_t* dst = st + (col >> 5) * 8192 + row * 128 + ((((col & 31) >> 2) ^ (row & 7)) << 4);
          *reinterpret_cast<float4*>(dst) =
              make_float4(__uint_as_float(v[j]) * (1.f / CHUNK), __uint_as_float(v[j + 1]) * (1.f / CHUNK),
                          __uint_as_float(v[j + 2]) * (1.f / CHUNK), __uint_as_float(v[j + 3]) * (1.f / CHUNK));
        }
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tempty[buf]);   // this warp's 32 lanes of the accumulator have been read
        tma_store_2d(&tm_out, st + ew * 4096, 0, tile * HD + ew * 32);
        tma_store_2d(&tm_out, st + 8192 + ew * 4096, 32, tile * HD + ew * 32);
        tma_store_commit();
      }
    }
    if (lane == 0) tma_store_wait_all();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag != 0 && error_flag != nullptr) atomicExch(error_flag, 2);
  if (warp == 16) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 128);
  }
}

// =============================================================================== scan
// writes [B,N,H,4096] FP32 -> states [B,N,H,4096] BF16 (mixed state read by chunk n), and
// optionally the fast / slow states after the last chunk [B,H,4096] FP32 (prefill).
// One thread owns four consecutive state elements (16-byte loads, 8-byte stores) and requests the writes of
// SCAN_AHEAD chunks before it runs their recurrence, so a thread keeps 128 bytes in flight instead of 4.
constexpr int SCAN_AHEAD = 8;

__global__ void __launch_bounds__(128)
memory_scan_kernel(const float* __restrict__ writes, const float* __restrict__ fast_logit,
                   const float* __restrict__ slow_logit, const float* __restrict__ mix_logit,
                   __nv_bfloat16* __restrict__ states, float* __restrict__ final_fast,
                   float* __restrict__ final_slow, const float* __restrict__ init_fast,
                   const float* __restrict__ init_slow, int B, int N, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t quad = blockIdx.x * static_cast<size_t>(128) + threadIdx.x;  // over B*H*1024 groups of four
  const size_t total = static_cast<size_t>(B) * H * 1024;
  if (quad >= total) return;
  const int e = static_cast<int>(quad % 1024) * 4;
  const int h = (quad / 1024) % H;
  const int b = quad / (1024 * static_cast<size_t>(H));
  const float df = 1.f / (1.f + expf(-fast_logit[h]));
  const float ds = 1.f / (1.f + expf(-slow_logit[h]));
  const float mix = 1.f / (1.f + expf(-mix_logit[h]));
  const size_t flat = quad * 4;
  float4 f = init_fast != nullptr ? *reinterpret_cast<const float4*>(init_fast + flat) : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 s = init_slow != nullptr ? *reinterpret_cast<const float4*>(init_slow + flat) : make_float4(0.f, 0.f, 0.f, 0.f);
  const size_t chunk_stride = static_cast<size_t>(H) * 4096;
  const size_t base = (static_cast<size_t>(b) * N * H + h) * 4096 + e;
  for (int n0 = 0; n0 < N; n0 += SCAN_AHEAD) {
    float4 w[SCAN_AHEAD];
#pragma unroll
    for (int j = 0; j < SCAN_AHEAD; ++j)
      if (n0 + j < N) w[j] = *reinterpret_cast<const float4*>(writes + base + (n0 + j) * chunk_stride);
#pragma unroll
    for (int j = 0; j < SCAN_AHEAD; ++j) {
      if (n0 + j >= N) break;
      if (states != nullptr) {
        uint2 o;
        o.x = pack_bf16x2(mix * f.x + (1.f - mix) * s.x, mix * f.y + (1.f - mix) * s.y);
        o.y = pack_bf16x2(mix * f.z + (1.f - mix) * s.z, mix * f.w + (1.f - mix) * s.w);
        *reinterpret_cast<uint2*>(states + base + (n0 + j) * chunk_stride) = o;
      }
      f.x = df * f.x + (1.f - df) * w[j].x; f.y = df * f.y + (1.f - df) * w[j].y;
      f.z = df * f.z + (1.f - df) * w[j].z; f.w = df * f.w + (1.f - df) * w[j].w;
      s.x = ds * s.x + (1.f - ds) * w[j].x; s.y = ds * s.y + (1.f - ds) * w[j].y;
      s.z = ds * s.z + (1.f - ds) * w[j].z; s.w = ds * s.w + (1.f - ds) * w[j].w;
    }
  }
  if (final_fast != nullptr) {
    *reinterpret_cast<float4*>(final_fast + flat) = f;
    *reinterpret_cast<float4*>(final_slow + flat) = s;
  }
}

// =============================================================================== attention
// smem: sQ 16K | sK 16K | sX 16K | sV 16K | sSt 8K | bars  (73 KiB: three CTAs per SM)
// The gate tile arrives by TMA with the other operands (into sX; every thread moves its gate row to
// registers before the softmax) and the blended output leaves by TMA (staged in sQ, one 32-row
// store per warp): a thread that owns a token row would otherwise touch one 16-byte piece of 32
// different cache lines per warp instruction.  P (128 x 128 BF16) overlays sK | sX once S = Q K^T
// is complete.  TMEM: 128 columns; S occupies all of them, and after the softmax has read S, O takes
// columns 0-63 and Mem = Q State columns 64-127, so three CTAs fit the 512 columns of an SM too.
// The kernel is bound by the latency of its dependent chain, so tiles in flight are what counts.
constexpr int AF_SMEM = 4 * TILE_BYTES + 8192 + 1024 + 128;

__global__ void __launch_bounds__(128, 3)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkvgu, const __grid_constant__ CUtensorMap tm_state,
                const __grid_constant__ CUtensorMap tm_y, const float2* __restrict__ rope, int T, int H, int d,
                int* error_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE_BYTES;
  uint8_t* sG = smem + 2 * TILE_BYTES;   // gate tile, later the second half of P
  uint8_t* sV = smem + 3 * TILE_BYTES;
  uint8_t* sSt = smem + 4 * TILE_BYTES;
  uint8_t* sP = sK;                      // P overlays K | gate
  uint64_t* bars = reinterpret_cast<uint64_t*>(sSt + 8192);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_chunks = T / CHUNK;
  const int tile = blockIdx.x;
  const int h = tile % H, n = (tile / H) % n_chunks, b = tile / (H * n_chunks);
  const int row0 = b * T + n * CHUNK;

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t t_s = tmem, t_o = tmem, t_m = tmem + 64;  // O and Mem reuse S's columns after the softmax
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;

  if (tid == 0) {
    mbar_expect_tx(&bars[0], 4 * TILE_BYTES + 8192);
    tma_load_2d(sQ, &tm_qkvgu, &bars[0], 0 * d + h * HD, row0);
    tma_load_2d(sK, &tm_qkvgu, &bars[0], 1 * d + h * HD, row0);
    tma_load_2d(sV, &tm_qkvgu, &bars[0], 2 * d + h * HD, row0);
    tma_load_2d(sG, &tm_qkvgu, &bars[0], 3 * d + h * HD, row0);
    tma_load_2d(sSt, &tm_state, &bars[0], 0, tile * HD);
  }
  bool ok = mbar_wait(&bars[0], 0, abort_flag);
  uint4 gate_row[8];  // this thread's gate row: the tile's space becomes half of P
#pragma unroll
  for (int j = 0; j < 8; ++j) gate_row[j] = *reinterpret_cast<const uint4*>(tile_chunk(sG, tid, j));
  if (ok) {
    rope_tanh_row(sQ, tid, rope, true, false);
    rope_tanh_row(sK, tid, rope, true, false);
  }
  fence_proxy_async_smem();
  __syncthreads();
  if (tid == 0 && ok) {
    constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k)
      umma_bf16(t_s, make_smem_desc_sw128(smem_u32(sQ) + k * 32, 0, 1024),
                make_smem_desc_sw128(smem_u32(sK) + k * 32, 0, 1024), idesc_s, k > 0);
    umma_commit(&bars[1]);
  }
  ok = ok && mbar_wait(&bars[1], 0, abort_flag);
  tc_fence_after_sync();

  // ---- causal softmax of row `tid` (scores scaled by 1/8); P stays unnormalised
  const float kScale = 0.125f * 1.4426950408889634f;  // fold log2(e)
  float row_max = -INFINITY;
  const int last_chunk = warp;  // columns beyond 32*warp+31 are masked for the whole warp
  for (int cc = 0; cc <= last_chunk; ++cc) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_s + lane_base + cc * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (cc * 32 + j <= tid) row_max = fmaxf(row_max, __uint_as_float(r[j]));
  }
  float row_sum = 0.f;
  for (int cc = 0; cc < 4; ++cc) {
    uint32_t pk[16];
    if (cc <= last_chunk) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_s + lane_base + cc * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float p0 = (cc * 32 + j <= tid) ? softmax_term(__uint_as_float(r[j]), row_max, kScale) : 0.f;
        const float p1 = (cc * 32 + j + 1 <= tid) ? softmax_term(__uint_as_float(r[j + 1]), row_max, kScale) : 0.f;
        const __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
        const float2 back = __bfloat1622float2(v);
        row_sum += back.x + back.y;  // normalise by what the MMA will actually sum
        pk[j >> 1] = *reinterpret_cast<const uint32_t*>(&v);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) pk[j] = 0u;
    }
    store_row_chunk32(sP, tid, cc * 32, pk);
  }
  tc_fence_before_sync();  // every thread's reads of S precede the MMAs that overwrite its columns
  fence_proxy_async_smem();
  __syncthreads();
  if (tid == 0 && ok) {
    tc_fence_after_sync();
    constexpr uint32_t idesc_o = make_idesc_bf16(128, 64, false, true);
#pragma unroll
    for (int k = 0; k < CHUNK / 16; ++k)
      umma_bf16(t_o, make_smem_desc_sw128(smem_u32(sP) + (k >> 2) * TILE_BYTES + (k & 3) * 32, 0, 1024),
                make_smem_desc_sw128(smem_u32(sV) + k * 2048, 0, 1024), idesc_o, k > 0);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k)  // Mem = Q State
      umma_bf16(t_m, make_smem_desc_sw128(smem_u32(sQ) + k * 32, 0, 1024),
                make_smem_desc_sw128(smem_u32(sSt) + k * 2048, 0, 1024), idesc_o, k > 0);
    umma_commit(&bars[2]);
  }
  ok = ok && mbar_wait(&bars[2], 0, abort_flag);
  tc_fence_after_sync();

  // ---- gate blend into the (now idle) Q tile, then one TMA store of the warp's 32 rows
  const float inv_l = 1.f / row_sum;
#pragma unroll
  for (int c = 0; c < HD; c += 16) {
    uint32_t ro[16], rm[16];
    tmem_ld_32x32b_x16(t_o + lane_base + c, ro);
    tmem_ld_32x32b_x16(t_m + lane_base + c, rm);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; j += 8) {
      const int chunk = (c + j) >> 3;
      const uint4 gq = gate_row[chunk];
      const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gq);
      uint4 out;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 gf = __bfloat1622float2(gb[t]);
        const float g0 = sigmoid_f(gf.x), g1 = sigmoid_f(gf.y);
        ow[t] = pack_bf16x2(gate_blend(g0, __uint_as_float(ro[j + 2 * t]), inv_l, __uint_as_float(rm[j + 2 * t])),
                            gate_blend(g1, __uint_as_float(ro[j + 2 * t + 1]), inv_l, __uint_as_float(rm[j + 2 * t + 1])));
      }
      *reinterpret_cast<uint4*>(tile_chunk(sQ, tid, chunk)) = out;
    }
  }
  fence_proxy_async_smem();
  __syncwarp();
  if ((tid & 31) == 0) {
    if (ok) {
      tma_store_2d(&tm_y, sQ + warp * 4096, h * HD, row0 + warp * 32);
      tma_store_commit();
    }
    tma_store_wait_read0();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag != 0 && error_flag != nullptr) atomicExch(error_flag, 3);
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 128);
  }
}

// =============================================================================== attention, streaming form
// attn_fwd_kernel as one persistent CTA per SM with specialised warps (17 warps):
//
//   warp 16        producer: TMA loads of tile i (Q, K, gate, V, state: 72 KiB) into stage i % 3 of a ring
//   warps 0..7     RoPE workers: thread (row r, half q) rotates four of the eight 16-byte pieces of row r of Q and of
//                  K in place (its 16 (cos, sin) pairs live in registers); worker 0 then issues S = Qr Kr^T and
//                  Mem = Qr State into TMEM set i % 2 -- Mem does not depend on the softmax, so it rides with S
//   warps 8..11    softmax group 0 (tiles 0, 2, 4, ...), warps 12..15 softmax group 1 (tiles 1, 3, ...): one thread per
//                  token row, as in attn_fwd_kernel: causal softmax straight out of TMEM, unnormalised P (BF16) into
//                  the tile's K and Q space (both dead once S and Mem are complete; the gate tile stays where it is),
//                  O = P V issued by the group's first thread into the first 64 columns of S, gate blend from O, Mem
//                  and the gate tile into the Q space, one TMA store per warp; the store's read of the tile releases
//                  the ring stage, the group's last TMEM read releases the TMEM set.
//
// Two tiles are in their softmax / blend phase at any time while a third is being rotated and a fourth loaded;
// attn_fwd_kernel gets its overlap from three independent CTAs per SM, each walking the whole chain alone.
// TMEM: set g = columns [192 g, 192 g + 192): S 128 (O reuses its first 64), Mem 64.  Bit-identical results.
constexpr int AS_STAGES = 3;
constexpr int AS_THREADS = 17 * 32;
constexpr int AS_STAGE_BYTES = 4 * TILE_BYTES + 8192;
constexpr int AS_SMEM = AS_STAGES * AS_STAGE_BYTES + 1024 + 256;

__global__ void __launch_bounds__(AS_THREADS, 1)
attn_fwd_stream_kernel(const __grid_constant__ CUtensorMap tm_qkvgu, const __grid_constant__ CUtensorMap tm_state,
                       const __grid_constant__ CUtensorMap tm_y, const float2* __restrict__ rope, int T, int H, int d,
                       int tiles, int* error_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AS_STAGES * AS_STAGE_BYTES);
  uint64_t* full = bars;                     // [3] stage loaded
  uint64_t* empty = bars + AS_STAGES;        // [3] stage released (4 warps of the owning group)
  uint64_t* sfull = bars + 2 * AS_STAGES;    // [2] S and Mem complete
  uint64_t* ofull = sfull + 2;               // [2] O complete
  uint64_t* setfree = ofull + 2;             // [2] TMEM set read out (4 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(setfree + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_chunks = T / CHUNK;

  if (tid == 0) {
    for (int s = 0; s < AS_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 4);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&sfull[g], 1);
      mbar_init(&ofull[g], 1);
      mbar_init(&setfree[g], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_qkvgu);
    tma_prefetch_desc(&tm_state);
    tma_prefetch_desc(&tm_y);
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  const int first = blockIdx.x, step = gridDim.x;
  auto stage_ptr = [&](int s) { return smem + s * AS_STAGE_BYTES; };  // Q | K | gate | V | state

  if (warp == 16) {
    if (lane == 0) {
      int i = 0;
      for (int tile = first; tile < tiles; tile += step, ++i) {
        const int s = i % AS_STAGES;
        if (!mbar_wait(&empty[s], ((i / AS_STAGES) & 1) ^ 1, abort_flag)) break;
        const int h = tile % H, n = (tile / H) % n_chunks, b = tile / (H * n_chunks);
        const int row0 = b * T + n * CHUNK;
        uint8_t* st = stage_ptr(s);
        mbar_expect_tx(&full[s], AS_STAGE_BYTES);
        tma_load_2d(st, &tm_qkvgu, &full[s], 0 * d + h * HD, row0);
        tma_load_2d(st + TILE_BYTES, &tm_qkvgu, &full[s], 1 * d + h * HD, row0);
        tma_load_2d(st + 2 * TILE_BYTES, &tm_qkvgu, &full[s], 3 * d + h * HD, row0);
        tma_load_2d(st + 3 * TILE_BYTES, &tm_qkvgu, &full[s], 2 * d + h * HD, row0);
        tma_load_2d(st + 4 * TILE_BYTES, &tm_state, &full[s], 0, tile * HD);
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ RoPE workers + S / Mem issue
    const int r = tid & 127, q = tid >> 7;
    float2 cs[16];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int t = 0; t < 4; ++t) cs[j * 4 + t] = rope[((q * 4 + j) * 4 + t) * CHUNK + r];
    int i = 0;
    for (int tile = first; tile < tiles; tile += step, ++i) {
      const int s = i % AS_STAGES, g = i & 1;
      uint8_t* sQ = stage_ptr(s);
      uint8_t* sK = sQ + TILE_BYTES;
      uint8_t* sSt = sQ + 4 * TILE_BYTES;
      const bool ok = mbar_wait(&full[s], (i / AS_STAGES) & 1, abort_flag);
      if (ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4* pq = reinterpret_cast<uint4*>(tile_chunk(sQ, r, q * 4 + j));
          uint4* pk = reinterpret_cast<uint4*>(tile_chunk(sK, r, q * 4 + j));
          uint4 qv = *pq, kv = *pk;
          uint32_t* qw = reinterpret_cast<uint32_t*>(&qv);
          uint32_t* kw = reinterpret_cast<uint32_t*>(&kv);
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 c = cs[j * 4 + t];
            const float2 x = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&qw[t]));
            const float2 qr = rope_rotate(x, c);
            qw[t] = pack_bf16x2(qr.x, qr.y);
            const float2 kr = rope_rotate(__bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&kw[t])), c);
            kw[t] = pack_bf16x2(kr.x, kr.y);
          }
          *pq = qv;
          *pk = kv;
        }
      }
      fence_proxy_async_smem();
      uint32_t any_bad;
      asm volatile(
          "{\n"
          ".reg .pred p, q;\n"
          "setp.ne.u32 q, %1, 0;\n"
          "bar.red.or.pred p, 2, 256, q;\n"
          "selp.u32 %0, 1, 0, p;\n"
          "}\n"
          : "=r"(any_bad)
          : "r"(ok ? 0u : 1u)
          : "memory");
      if (any_bad) break;
      if (tid == 0 && mbar_wait(&setfree[g], ((i >> 1) & 1) ^ 1, abort_flag)) {
        tc_fence_after_sync();
        const uint32_t t_s = tmem + g * 192, t_m = t_s + 128;
        constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
        constexpr uint32_t idesc_m = make_idesc_bf16(128, 64, false, true);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_bf16(t_s, make_smem_desc_sw128(smem_u32(sQ) + k * 32, 0, 1024),
                    make_smem_desc_sw128(smem_u32(sK) + k * 32, 0, 1024), idesc_s, k > 0);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)  // Mem = Qr State
          umma_bf16(t_m, make_smem_desc_sw128(smem_u32(sQ) + k * 32, 0, 1024),
                    make_smem_desc_sw128(smem_u32(sSt) + k * 2048, 0, 1024), idesc_m, k > 0);
        umma_commit(&sfull[g]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax groups
    const int g = (warp - 8) >> 2;
    const int gt = tid - (256 + g * 128);       // row of the tile = TMEM lane
    const int wq = gt >> 5;                     // lane quarter of this warp
    const uint32_t t_s = tmem + g * 192, t_o = t_s, t_m = t_s + 128;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const float kScale = 0.125f * 1.4426950408889634f;  // fold log2(e)
    const int last_chunk = wq;  // columns beyond 32*wq+31 are masked for the whole warp
    int i = g;
    for (int tile = first + g * step; tile < tiles; tile += 2 * step, i += 2) {
      const int s = i % AS_STAGES, k2 = i >> 1;
      uint8_t* sQ = stage_ptr(s);
      uint8_t* sK = sQ + TILE_BYTES;
      uint8_t* sG = sQ + 2 * TILE_BYTES;
      uint8_t* sV = sQ + 3 * TILE_BYTES;
      const int h = tile % H, n = (tile / H) % n_chunks, b = tile / (H * n_chunks);
      const int row0 = b * T + n * CHUNK;
      uint32_t landed = 0;
      if (lane == 0) landed = mbar_wait(&sfull[g], k2 & 1, abort_flag) ? 1u : 0u;
      bool ok = __shfl_sync(0xffffffffu, landed, 0) != 0u;
      tc_fence_after_sync();
      float row_sum = 0.f;
      if (ok) {
        float row_max = -INFINITY;
        for (int cc = 0; cc <= last_chunk; ++cc) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_s + lane_base + cc * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (cc * 32 + j <= gt) row_max = fmaxf(row_max, __uint_as_float(v[j]));
        }
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t pk[16];
          if (cc <= last_chunk) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_s + lane_base + cc * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float p0 = (cc * 32 + j <= gt) ? softmax_term(__uint_as_float(v[j]), row_max, kScale) : 0.f;
              const float p1 = (cc * 32 + j + 1 <= gt) ? softmax_term(__uint_as_float(v[j + 1]), row_max, kScale) : 0.f;
              const __nv_bfloat162 pv = __floats2bfloat162_rn(p0, p1);
              const float2 back = __bfloat1622float2(pv);
              row_sum += back.x + back.y;  // normalise by what the MMA will actually sum
              pk[j >> 1] = *reinterpret_cast<const uint32_t*>(&pv);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) pk[j] = 0u;
          }
          // columns 0..63 of P go to the K tile's space, columns 64..127 to the Q tile's
          uint8_t* half = (cc < 2) ? sK : sQ;
          const int j0 = (cc & 1) * 4;
#pragma unroll
          for (int w4 = 0; w4 < 4; ++w4)
            *reinterpret_cast<uint4*>(tile_chunk(half, gt, j0 + w4)) =
                make_uint4(pk[4 * w4], pk[4 * w4 + 1], pk[4 * w4 + 2], pk[4 * w4 + 3]);
        }
      }
      tc_fence_before_sync();  // every thread's reads of S precede the MMA that overwrites its first columns
      fence_proxy_async_smem();
      uint32_t any_bad;
      if (g == 0)
        asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.or.pred p, 3, 128, q;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(any_bad) : "r"(ok ? 0u : 1u) : "memory");
      else
        asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.or.pred p, 4, 128, q;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(any_bad) : "r"(ok ? 0u : 1u) : "memory");
      if (any_bad) break;
      if (gt == 0) {
        tc_fence_after_sync();
        constexpr uint32_t idesc_o = make_idesc_bf16(128, 64, false, true);
#pragma unroll
        for (int k = 0; k < CHUNK / 16; ++k)
          umma_bf16(t_o, make_smem_desc_sw128(smem_u32((k >> 2) ? sQ : sK) + (k & 3) * 32, 0, 1024),
                    make_smem_desc_sw128(smem_u32(sV) + k * 2048, 0, 1024), idesc_o, k > 0);
        umma_commit(&ofull[g]);
      }
      landed = 0;
      if (lane == 0) landed = mbar_wait(&ofull[g], k2 & 1, abort_flag) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, landed, 0) != 0u;
      tc_fence_after_sync();
      if (ok) {
        // ---- gate blend into the (now idle) Q tile, then one TMA store of the warp's 32 rows
        const float inv_l = 1.f / row_sum;
#pragma unroll
        for (int c = 0; c < HD; c += 16) {
          uint32_t ro[16], rm[16];
          tmem_ld_32x32b_x16(t_o + lane_base + c, ro);
          tmem_ld_32x32b_x16(t_m + lane_base + c, rm);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; j += 8) {
            const int chunk = (c + j) >> 3;
            const uint4 gq = *reinterpret_cast<const uint4*>(tile_chunk(sG, gt, chunk));
            const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gq);
            uint4 out;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float2 gf = __bfloat1622float2(gb[t]);
              const float g0 = sigmoid_f(gf.x), g1 = sigmoid_f(gf.y);
              ow[t] = pack_bf16x2(gate_blend(g0, __uint_as_float(ro[j + 2 * t]), inv_l, __uint_as_float(rm[j + 2 * t])),
                                  gate_blend(g1, __uint_as_float(ro[j + 2 * t + 1]), inv_l, __uint_as_float(rm[j + 2 * t + 1])));
            }
            *reinterpret_cast<uint4*>(tile_chunk(sQ, gt, chunk)) = out;
          }
        }
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&setfree[g]);   // this warp's lanes of S / O / Mem have been read
        if (ok) {
          tma_store_2d(&tm_y, sQ + wq * 4096, h * HD, row0 + wq * 32);
          tma_store_commit();
        }
        tma_store_wait_read0();
        mbar_arrive(&empty[s]);     // this warp no longer touches the stage
      }
      __syncwarp();
      // a warp that gave up does not leave alone: its next wait fails at once (the abort flag is up), and the
      // group's vote at the next barrier takes all four warps out together
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag != 0 && error_flag != nullptr) atomicExch(error_flag, 3);
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace ws

using namespace ws;

// Which form the tile kernels of the attention block take: 1 = persistent streaming CTAs, 0 = one tile per CTA,
// -1 = the process default (streaming unless WS_ATTN_STREAM=0 is in the environment).
static int g_attn_stream_mode = -1;
extern "C" void ws_attn_set_stream_mode(int mode) { g_attn_stream_mode = mode; }
extern "C" int ws_attn_stream_form(void) {
  if (g_attn_stream_mode >= 0) return g_attn_stream_mode != 0;
  static const bool from_env = [] {
    const char* e = std::getenv("WS_ATTN_STREAM");
    return e == nullptr || e[0] != '0';
  }();
  return from_env ? 1 : 0;
}

extern "C" int ws_chunk_writes(const void* qkvgu, const float* rope, float* writes, int B, int T, int H, int d,
                               int* error_flag, cudaStream_t stream) {
  if (T % CHUNK != 0 || d != H * HD) return -1;
  CUtensorMap tm;
  int rc = make_tile_map(&tm, qkvgu, 5 * (uint64_t)d, (uint64_t)B * T, 5 * (uint64_t)d, HD, CHUNK);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(chunk_writes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WR_SMEM) != cudaSuccess)
      return -20;
    configured = true;
  }
  const int tiles = B * (T / CHUNK) * H;
  CUtensorMap to;
  rc = make_map_f32(&to, writes, HD, (uint64_t)tiles * HD, HD, 32, 32);
  if (rc) return rc;
  const bool stream_form = ws_attn_stream_form() != 0;
  static int sms = 0;
  if (stream_form && sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaFuncSetAttribute(chunk_writes_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WS_SMEM) != cudaSuccess)
      return -20;
  }
  if (stream_form)
    launch_dependent(chunk_writes_stream_kernel, dim3(tiles < sms ? tiles : sms), dim3(WS_THREADS), WS_SMEM, stream, tm, to,
                     reinterpret_cast<const float2*>(rope), T, H, d, tiles, error_flag);
  else
    launch_dependent(chunk_writes_kernel, dim3(tiles), dim3(128), WR_SMEM, stream, tm, to, reinterpret_cast<const float2*>(rope), T, H, d,
                     error_flag);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ws_memory_scan(const float* writes, const float* fast_logit, const float* slow_logit,
                              const float* mix_logit, void* states, float* final_fast, float* final_slow,
                              const float* init_fast, const float* init_slow, int B, int N, int H,
                              cudaStream_t stream) {
  const size_t total = (size_t)B * H * 4096;
  launch_dependent(memory_scan_kernel, dim3((unsigned)((total / 4 + 127) / 128)), dim3(128), 0, stream, writes, fast_logit, slow_logit, mix_logit, (__nv_bfloat16*)states, final_fast, final_slow, init_fast,
      init_slow, B, N, H);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ws_attn_fwd(const void* qkvgu, const void* states, const float* rope, void* y, int B, int T, int H,
                           int d, int* error_flag, cudaStream_t stream) {
  if (T % CHUNK != 0 || d != H * HD) return -1;
  const int tiles = B * (T / CHUNK) * H;
  CUtensorMap tm, ts, ty;
  int rc = make_tile_map(&tm, qkvgu, 5 * (uint64_t)d, (uint64_t)B * T, 5 * (uint64_t)d, HD, CHUNK);
  if (rc) return rc;
  rc = make_tile_map(&ts, states, HD, (uint64_t)tiles * HD, HD, HD, HD);
  if (rc) return rc;
  rc = make_tile_map(&ty, y, (uint64_t)d, (uint64_t)B * T, (uint64_t)d, HD, 32);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AF_SMEM) != cudaSuccess)
      return -20;
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaFuncSetAttribute(attn_fwd_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AS_SMEM) != cudaSuccess)
      return -20;
  }
  if (ws_attn_stream_form() != 0)
    launch_dependent(attn_fwd_stream_kernel, dim3(tiles < sms ? tiles : sms), dim3(AS_THREADS), AS_SMEM, stream, tm, ts, ty,
                     reinterpret_cast<const float2*>(rope), T, H, d, tiles, error_flag);
  else
    launch_dependent(attn_fwd_kernel, dim3(tiles), dim3(128), AF_SMEM, stream, tm, ts, ty, reinterpret_cast<const float2*>(rope), T, H, d,
                     error_flag);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
