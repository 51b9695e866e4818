// Backward kernels of the middle of a WarpState core (chunk 128, head_dim 64).
//
//   dstate_kernel       : dState[b,n,h] = rope(Q)^T (dy * (1 - sigmoid(g)) / 8)           (64x64)
//   memory_scan_bwd     : reverse scan over chunks: dState -> dWrites (BF16) and the partial
//                         gradients of the three per-head scalars (decays, mix); FP32, fixed order
//   attn_bwd_kernel     : per (batch, chunk, head) tile recomputes S / P / O / Mem, then
//                            dP = dlocal V^T, dV = P^T dlocal, dS = P*(dP - D)/8,
//                            dQr = dS Kr + dmem State^T, dKr = dS^T Qr,
//                            dtK = tU dW^T, dtU = tK dW   (write path),
//                         and writes the packed gradient [tokens, 5d] = (dQ, dK, dV, dGate, dU)
//                         with the RoPE transpose and the tanh / sigmoid derivatives applied --
//                         the region the reference handles with flash-attention backward plus
//                         its "paired backward layout" kernels (ops/backward_layout.py:114-210).
//
// All ten matrix products of the tile run on tcgen05 with accumulators in TMEM; one thread owns
// one token row in every element-wise stage.
#include "ws_ptx.cuh"
#include "ws_api.h"
#include "ws_launch.h"
#include "attention_common.cuh"

namespace ws {

extern "C" void ws_count_launch(void);

// =============================================================================== dState
// smem: Qr 16K | dy -> dmem/8 16K | gate, then the FP32 result 16K | bars
constexpr int DS_SMEM = 3 * TILE_BYTES + 1024 + 128;

__global__ void __launch_bounds__(128, 4)
dstate_kernel(const __grid_constant__ CUtensorMap tm_qkvgu, const __grid_constant__ CUtensorMap tm_dy,
              const __grid_constant__ CUtensorMap tm_out, const float2* __restrict__ rope, int T, int H, int d,
              int* error_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sQ = smem;
  uint8_t* sD = smem + TILE_BYTES;
  uint8_t* sG = smem + 2 * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * TILE_BYTES);
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
    mbar_expect_tx(&bars[0], 3 * TILE_BYTES);
    tma_load_2d(sQ, &tm_qkvgu, &bars[0], h * HD, row0);
    tma_load_2d(sD, &tm_dy, &bars[0], h * HD, row0);
    tma_load_2d(sG, &tm_qkvgu, &bars[0], 3 * d + h * HD, row0);
  }
  bool ok = mbar_wait(&bars[0], 0, abort_flag);
  if (ok) {
    rope_tanh_row(sQ, tid, rope, true, false);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint4* p = reinterpret_cast<uint4*>(tile_chunk(sD, tid, j));
      uint4 v = *p;
      const uint4 gq = *reinterpret_cast<const uint4*>(tile_chunk(sG, tid, j));
      uint32_t* w = reinterpret_cast<uint32_t*>(&v);
      const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gq);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 dyv = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[t]));
        const float2 gf = __bfloat1622float2(gb[t]);
        w[t] = pack_bf16x2(dyv.x * (1.f - sigmoid_f(gf.x)) * 0.125f, dyv.y * (1.f - sigmoid_f(gf.y)) * 0.125f);
      }
      *p = v;
    }
  }
  fence_proxy_async_smem();
  __syncthreads();
  if (tid == 0 && ok) {
    constexpr uint32_t idesc = make_idesc_bf16(128, 64, true, true);
#pragma unroll
    for (int k = 0; k < CHUNK / 16; ++k)
      umma_bf16(tmem, make_smem_desc_sw128(smem_u32(sQ) + k * 2048, 0, 1024),
                make_smem_desc_sw128(smem_u32(sD) + k * 2048, 0, 1024), idesc, k > 0);
    umma_commit(&bars[1]);
  }
  ok = ok && mbar_wait(&bars[1], 0, abort_flag);
  tc_fence_after_sync();
  if (warp < 2) {
    // Row `tid` of the [64 x 64] FP32 result goes to two swizzled [64 x 32] half tiles (the gate tile's
    // space), and each warp stores its 32 rows of both halves by TMA.
#pragma unroll
    for (int c = 0; c < HD; c += 16) {
      uint32_t r[16];
      tmem_ld_32x32b_x16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        const int col = c + j;
        uint8_t* dst = sG + (col >> 5) * 8192 + tid * 128 + ((((col & 31) >> 2) ^ (tid & 7)) << 4);
        *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                      __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if ((tid & 31) == 0) {
      if (ok) {
        tma_store_2d(&tm_out, sG + warp * 4096, 0, tile * HD + warp * 32);
        tma_store_2d(&tm_out, sG + 8192 + warp * 4096, 32, tile * HD + warp * 32);
        tma_store_commit();
      }
      tma_store_wait_read0();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag != 0 && error_flag != nullptr) atomicExch(error_flag, 4);
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 64);
  }
}

// =============================================================================== dState, streaming form
// dstate_kernel as one persistent CTA per SM with specialised warps, exactly as chunk_writes_stream_kernel
// (attention_fwd.cu): producer warp with a 3-stage ring of (Q, dy, gate) tiles, 512 workers that turn Q into rope(Q)
// and dy into dy (1 - sigmoid(gate)) / 8 in place, MMA issue into a double-buffered accumulator, two epilogue warps
// that store the FP32 [64 x 64] result by TMA.  Bit-identical to dstate_kernel.
constexpr int DSS_STAGES = 3;
constexpr int DSS_THREADS = 19 * 32;
constexpr int DSS_SMEM = DSS_STAGES * 3 * TILE_BYTES + 2 * 16384 + 1024 + 256;

__global__ void __launch_bounds__(DSS_THREADS, 1)
dstate_stream_kernel(const __grid_constant__ CUtensorMap tm_qkvgu, const __grid_constant__ CUtensorMap tm_dy,
                     const __grid_constant__ CUtensorMap tm_out, const float2* __restrict__ rope, int T, int H, int d,
                     int tiles, int* error_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* ring = smem;                                   // stage s: Q, dy, gate at s * 48 KiB
  uint8_t* staging = smem + DSS_STAGES * 3 * TILE_BYTES;  // two FP32 [64 x 64] tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * 16384);
  uint64_t* full = bars;                    // [4] tile landed
  uint64_t* empty = bars + DSS_STAGES;       // [4] MMAs have read the stage
  uint64_t* tfull = bars + 2 * DSS_STAGES;   // [2] accumulator complete
  uint64_t* tempty = tfull + 2;             // [2] accumulator read by both epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_chunks = T / CHUNK;

  if (tid == 0) {
    for (int s = 0; s < DSS_STAGES; ++s) {
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
    tma_prefetch_desc(&tm_dy);
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
        const int s = i % DSS_STAGES;
        if (!mbar_wait(&empty[s], ((i / DSS_STAGES) & 1) ^ 1, abort_flag)) break;
        const int h = tile % H, n = (tile / H) % n_chunks, b = tile / (H * n_chunks);
        const int row0 = b * T + n * CHUNK;
        mbar_expect_tx(&full[s], 3 * TILE_BYTES);
        tma_load_2d(ring + s * 3 * TILE_BYTES, &tm_qkvgu, &full[s], h * HD, row0);
        tma_load_2d(ring + s * 3 * TILE_BYTES + TILE_BYTES, &tm_dy, &full[s], h * HD, row0);
        tma_load_2d(ring + s * 3 * TILE_BYTES + 2 * TILE_BYTES, &tm_qkvgu, &full[s], 3 * d + h * HD, row0);
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
      const int s = i % DSS_STAGES;
      uint8_t* sQ = ring + s * 3 * TILE_BYTES;
      uint8_t* sD = sQ + TILE_BYTES;
      uint8_t* sGate = sD + TILE_BYTES;
      const bool ok = mbar_wait(&full[s], (i / DSS_STAGES) & 1, abort_flag);
      if (ok) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint4* pq = reinterpret_cast<uint4*>(tile_chunk(sQ, r, q * 2 + j));
          uint4* pd = reinterpret_cast<uint4*>(tile_chunk(sD, r, q * 2 + j));
          uint4 qv = *pq, dv = *pd;
          const uint4 gv = *reinterpret_cast<const uint4*>(tile_chunk(sGate, r, q * 2 + j));
          uint32_t* qw = reinterpret_cast<uint32_t*>(&qv);
          uint32_t* dw = reinterpret_cast<uint32_t*>(&dv);
          const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 x = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&qw[t]));
            const float2 c = cs[j * 4 + t];
            const float2 qr = rope_rotate(x, c);
            qw[t] = pack_bf16x2(qr.x, qr.y);
            const float2 dyv = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&dw[t]));
            const float2 gf = __bfloat1622float2(gb[t]);
            dw[t] = pack_bf16x2(dyv.x * (1.f - sigmoid_f(gf.x)) * 0.125f, dyv.y * (1.f - sigmoid_f(gf.y)) * 0.125f);
          }
          *pq = qv;
          *pd = dv;
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
          // D[128 x 64]: rows 0..63 = Qr^T (dmem / 8); rows 64..127 repeat them (zero stride between A's atoms)
          constexpr uint32_t idesc = make_idesc_bf16(128, 64, true, true);
#pragma unroll
          for (int k = 0; k < CHUNK / 16; ++k)
            umma_bf16(tmem + buf * 64, make_smem_desc_sw128(smem_u32(sQ) + k * 2048, 0, 1024),
                      make_smem_desc_sw128(smem_u32(sD) + k * 2048, 0, 1024), idesc, k > 0);
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
              make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
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
  if (tid == 0 && *abort_flag != 0 && error_flag != nullptr) atomicExch(error_flag, 4);
  if (warp == 16) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 128);
  }
}

// =============================================================================== reverse scan
// The reverse scan needs the state every chunk saw.  Those are recomputed from the writes in groups of
// SCAN_GROUP chunks: a first pass keeps the state at every group boundary, then the groups are walked
// from the last to the first, each re-running its forward recurrence into registers before its reverse
// part.  One group (sequences up to 2048 tokens) skips the first pass.
constexpr int SCAN_GROUP = 16;
constexpr int SCAN_MAX_GROUPS = 16;
constexpr int SCAN_MAX_CHUNKS = SCAN_GROUP * SCAN_MAX_GROUPS;  // 32768 tokens per sequence

// dstate [B,N,H,4096] FP32 (gradient of the mixed state read by chunk n), writes [B,N,H,4096] FP32
// -> dwrites [B,N,H,4096] BF16 and partial sums [B*H*16][3] of d(fast decay), d(slow decay), d(mix).
__global__ void __launch_bounds__(256)
memory_scan_bwd_kernel(const float* __restrict__ dstate, const float* __restrict__ writes,
                       const float* __restrict__ fast_logit, const float* __restrict__ slow_logit,
                       const float* __restrict__ mix_logit, __nv_bfloat16* __restrict__ dwrites,
                       float* __restrict__ partials, int B, int N, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[3][8];
  const size_t idx = blockIdx.x * static_cast<size_t>(256) + threadIdx.x;  // over B*H*4096 (exact multiple)
  const int e = idx % 4096;
  const int h = (idx / 4096) % H;
  const int b = idx / (4096 * static_cast<size_t>(H));
  const float df = 1.f / (1.f + expf(-fast_logit[h]));
  const float ds = 1.f / (1.f + expf(-slow_logit[h]));
  const float mix = 1.f / (1.f + expf(-mix_logit[h]));
  const size_t chunk_stride = static_cast<size_t>(H) * 4096;
  const size_t base = (static_cast<size_t>(b) * N * H + h) * 4096 + e;  // chunk 0 of this element
  const int groups = (N + SCAN_GROUP - 1) / SCAN_GROUP;
  float start_f[SCAN_MAX_GROUPS], start_s[SCAN_MAX_GROUPS];
  {
    float f = 0.f, s = 0.f;
#pragma unroll 1
    for (int g = 0; g < groups; ++g) {
      start_f[g] = f;
      start_s[g] = s;
      if (g + 1 < groups) {
#pragma unroll
        for (int i = 0; i < SCAN_GROUP; ++i) {
          const float w = writes[base + (g * SCAN_GROUP + i) * chunk_stride];
          f = df * f + (1.f - df) * w;
          s = ds * s + (1.f - ds) * w;
        }
      }
    }
  }
  // a, bb: gradients of the fast and slow state AFTER the chunk being visited (F_{n+1}, S_{n+1})
  float a = 0.f, bb = 0.f, g_df = 0.f, g_ds = 0.f, g_mix = 0.f;
#pragma unroll 1
  for (int g = groups - 1; g >= 0; --g) {
    const int n0 = g * SCAN_GROUP;
    const int count = min(SCAN_GROUP, N - n0);
    // every load of the group is requested before its recurrences run: 2 x SCAN_GROUP independent loads in flight
    float F[SCAN_GROUP], S[SCAN_GROUP], W[SCAN_GROUP], G[SCAN_GROUP];
#pragma unroll
    for (int i = 0; i < SCAN_GROUP; ++i) {
      if (i < count) {
        W[i] = writes[base + (n0 + i) * chunk_stride];
        G[i] = dstate[base + (n0 + i) * chunk_stride];
      }
    }
    float f = start_f[g], s = start_s[g];
#pragma unroll
    for (int i = 0; i < SCAN_GROUP; ++i) {  // forward: state seen by chunk n0 + i
      if (i < count) {
        F[i] = f;
        S[i] = s;
        f = df * f + (1.f - df) * W[i];
        s = ds * s + (1.f - ds) * W[i];
      }
    }
#pragma unroll
    for (int i = SCAN_GROUP - 1; i >= 0; --i) {
      if (i < count) {
        dwrites[base + (n0 + i) * chunk_stride] = __float2bfloat16_rn((1.f - df) * a + (1.f - ds) * bb);
        g_df += a * (F[i] - W[i]);    // F_{n+1} = df F_n + (1 - df) w_n
        g_ds += bb * (S[i] - W[i]);
        g_mix += G[i] * (F[i] - S[i]);
        a = mix * G[i] + df * a;      // gradient of F_n
        bb = (1.f - mix) * G[i] + ds * bb;
      }
    }
  }
  // block reduction (fixed order)
  float vals[3] = {g_df, g_ds, g_mix};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int q = 0; q < 3; ++q) {
    float v = vals[q];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[q][warp] = v;
  }
  __syncthreads();
  if (threadIdx.x < 3) {
    float v = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; ++wi) v += red[threadIdx.x][wi];
    partials[static_cast<size_t>(blockIdx.x) * 3 + threadIdx.x] = v;
  }
}

// =============================================================================== attention bwd
// One CTA of 128 threads per (batch, chunk, head) tile; thread t owns row t of the chunk.
// The kernel is a chain of four MMA phases with element-wise work between them, so a single
// tile cannot keep an SM busy; what matters is how many tiles an SM holds at once.  Shared
// memory is therefore kept to 112 KiB and TMEM to 256 columns, so that TWO CTAs fit per SM:
//
//   smem: B0 Qr | B1 Kr | B2 dy -> dlocal -> tanh(U) | B3 dmem/8 -> V -> tanh(Kr) | sP (32K: P -> dS)
//         | sSt (8K) | sDW (8K) | barriers
//   TMEM: [0,128) S -> O (first 64) -> dP -> dKr (first 64) + dtK (last 64)
//         [128,192) Mem -> dV -> dtU        [192,256) dQr (memory part, later += attention part)
//
// V and U are fetched late (into buffers that earlier operands have left), each behind work that
// hides most of the load latency.  P is stored normalised, so O and dV need no row scaling.
constexpr int AB_THREADS = 128;
// No alignment slack: 2 x (114816 + 1024 reserved) = 231680 <= 233472 bytes of an SM.  The dynamic
// segment is declared 1024-byte aligned (the 128-byte swizzle needs it); the kernel checks.
constexpr int AB_SMEM = 4 * TILE_BYTES + 2 * TILE_BYTES + 2 * 8192 + 128;

__global__ void __launch_bounds__(AB_THREADS, 2)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkvgu, const __grid_constant__ CUtensorMap tm_state,
                const __grid_constant__ CUtensorMap tm_dy, const __grid_constant__ CUtensorMap tm_dw,
                const __grid_constant__ CUtensorMap tm_dout, const float2* __restrict__ rope, int T, int H, int d,
                int* error_flag) {
  extern __shared__ __align__(1024) uint8_t smem_ab[];
  uint8_t* smem = smem_ab;
  if ((smem_u32(smem) & 1023u) != 0u) {  // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0 && error_flag != nullptr) atomicExch(error_flag, 7);
    return;
  }
  uint8_t* sQ = smem;                    // B0
  uint8_t* sK = sQ + TILE_BYTES;         // B1
  uint8_t* sB2 = sK + TILE_BYTES;        // dy -> dlocal -> tanh(U)
  uint8_t* sB3 = sB2 + TILE_BYTES;       // dmem/8 -> V -> tanh(Kr)
  uint8_t* sP = sB3 + TILE_BYTES;
  uint8_t* sSt = sP + 2 * TILE_BYTES;
  uint8_t* sDW = sSt + 8192;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDW + 8192);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_chunks = T / CHUNK;
  const int tile = blockIdx.x;
  const int h = tile % H, n = (tile / H) % n_chunks, b = tile / (H * n_chunks);
  const int row0 = b * T + n * CHUNK;

  if (tid == 0) {
    for (int i = 0; i < 7; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t t_lo = tmem;          // S / O / dP / dKr+dtK
  const uint32_t t_mid = tmem + 128;   // Mem / dV / dtU
  const uint32_t t_dq = tmem + 192;    // dQr
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;

  if (tid == 0) {
    mbar_expect_tx(&bars[0], 4 * TILE_BYTES + 2 * 8192);
    tma_load_2d(sQ, &tm_qkvgu, &bars[0], 0 * d + h * HD, row0);
    tma_load_2d(sK, &tm_qkvgu, &bars[0], 1 * d + h * HD, row0);
    tma_load_2d(sB2, &tm_dy, &bars[0], h * HD, row0);
    tma_load_2d(sP, &tm_qkvgu, &bars[0], 3 * d + h * HD, row0);  // gate: kept in registers after the first stage
    tma_load_2d(sSt, &tm_state, &bars[0], 0, tile * HD);
    tma_load_2d(sDW, &tm_dw, &bars[0], 0, tile * HD);
  }
  // The thread's gate row, its dGate row and its dV row stay in registers (8 x 16 bytes each) until
  // the last stage, where all five gradient tiles leave through shared memory and TMA stores.
  uint4 gate_row[8], dgate_row[8], dv_row[8];

  bool ok = mbar_wait(&bars[0], 0, abort_flag);
#pragma unroll
  for (int j = 0; j < 8; ++j) gate_row[j] = *reinterpret_cast<const uint4*>(tile_chunk(sP, tid, j));
  if (ok) {
    rope_tanh_row(sQ, tid, rope, true, false);
    rope_tanh_row(sK, tid, rope, true, false);
    // dmem/8 = dy * (1 - sigmoid(gate)) / 8  -> B3
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint4 dyq = *reinterpret_cast<const uint4*>(tile_chunk(sB2, tid, j));
      const uint4 gq = gate_row[j];
      const __nv_bfloat162* dyb = reinterpret_cast<const __nv_bfloat162*>(&dyq);
      const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gq);
      uint4 o;
      uint32_t* wo = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 dyv = __bfloat1622float2(dyb[t]);
        const float2 gf = __bfloat1622float2(gb[t]);
        wo[t] = pack_bf16x2(dyv.x * (1.f - sigmoid_f(gf.x)) * 0.125f, dyv.y * (1.f - sigmoid_f(gf.y)) * 0.125f);
      }
      *reinterpret_cast<uint4*>(tile_chunk(sB3, tid, j)) = o;
    }
  }
  fence_proxy_async_smem();
  __syncthreads();
  // ---- MMA A: S = Qr Kr^T, Mem = Qr State, dQr = (dmem/8) State^T
  if (tid == 0 && ok) {
    constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
    constexpr uint32_t idesc_m = make_idesc_bf16(128, 64, false, true);
    constexpr uint32_t idesc_kk64 = make_idesc_bf16(128, 64, false, false);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k)
      umma_bf16(t_lo, make_smem_desc_sw128(smem_u32(sQ) + k * 32, 0, 1024),
                make_smem_desc_sw128(smem_u32(sK) + k * 32, 0, 1024), idesc_s, k > 0);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k)
      umma_bf16(t_mid, make_smem_desc_sw128(smem_u32(sQ) + k * 32, 0, 1024),
                make_smem_desc_sw128(smem_u32(sSt) + k * 2048, 0, 1024), idesc_m, k > 0);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k)
      umma_bf16(t_dq, make_smem_desc_sw128(smem_u32(sB3) + k * 32, 0, 1024),
                make_smem_desc_sw128(smem_u32(sSt) + k * 32, 0, 1024), idesc_kk64, k > 0);
    umma_commit(&bars[1]);
  }
  ok = ok && mbar_wait(&bars[1], 0, abort_flag);
  tc_fence_after_sync();
  if (tid == 0 && ok) {  // B3 (dmem) has been consumed: fetch V into it behind the softmax
    mbar_expect_tx(&bars[2], TILE_BYTES);
    tma_load_2d(sB3, &tm_qkvgu, &bars[2], 2 * d + h * HD, row0);
  }

  // ---- softmax: max, sum, then normalised P (BF16) to smem
  const float kScale = 0.125f * 1.4426950408889634f;
  const int last_chunk = warp;
  float row_max = -INFINITY;
  for (int cc = 0; cc <= last_chunk; ++cc) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_lo + lane_base + cc * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (cc * 32 + j <= tid) row_max = fmaxf(row_max, __uint_as_float(r[j]));
  }
  float row_sum = 0.f;
  for (int cc = 0; cc <= last_chunk; ++cc) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_lo + lane_base + cc * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (cc * 32 + j <= tid) row_sum += exp2f((__uint_as_float(r[j]) - row_max) * kScale);
  }
  const float inv_l = 1.f / row_sum;
  for (int cc = 0; cc < 4; ++cc) {
    uint32_t pk[16];
    if (cc <= last_chunk) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_lo + lane_base + cc * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float p0 = (cc * 32 + j <= tid) ? exp2f((__uint_as_float(r[j]) - row_max) * kScale) * inv_l : 0.f;
        const float p1 = (cc * 32 + j + 1 <= tid) ? exp2f((__uint_as_float(r[j + 1]) - row_max) * kScale) * inv_l : 0.f;
        pk[j >> 1] = pack_bf16x2(p0, p1);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) pk[j] = 0u;
    }
    store_row_chunk32(sP, tid, cc * 32, pk);
  }
  tc_fence_before_sync();
  fence_proxy_async_smem();
  __syncthreads();
  // ---- MMA B: O = P V
  if (tid == 0 && ok) {
    ok = mbar_wait(&bars[2], 0, abort_flag);  // V has landed
    if (ok) {
      tc_fence_after_sync();
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 64, false, true);
#pragma unroll
      for (int k = 0; k < CHUNK / 16; ++k)
        umma_bf16(t_lo, make_smem_desc_sw128(smem_u32(sP) + (k >> 2) * TILE_BYTES + (k & 3) * 32, 0, 1024),
                  make_smem_desc_sw128(smem_u32(sB3) + k * 2048, 0, 1024), idesc_o, k > 0);
      umma_commit(&bars[3]);
    }
  }
  ok = mbar_wait(&bars[3], 0, abort_flag) && ok;
  tc_fence_after_sync();

  // ---- element-wise stage 1: dlocal = dy * g (in place in B2), dGate, D = sum(dlocal * local)
  float Drow = 0.f;
#pragma unroll
  for (int c = 0; c < HD; c += 16) {
    uint32_t ro[16], rm[16];
    tmem_ld_32x32b_x16(t_lo + lane_base + c, ro);
    tmem_ld_32x32b_x16(t_mid + lane_base + c, rm);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; j += 8) {
      const int chunk = (c + j) >> 3;
      uint4* pdl = reinterpret_cast<uint4*>(tile_chunk(sB2, tid, chunk));
      const uint4 dyq = *pdl;
      const uint4 gq = gate_row[chunk];
      const __nv_bfloat162* dyb = reinterpret_cast<const __nv_bfloat162*>(&dyq);
      const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gq);
      uint4 o_dl, o_dg;
      uint32_t* w_dl = reinterpret_cast<uint32_t*>(&o_dl);
      uint32_t* w_dg = reinterpret_cast<uint32_t*>(&o_dg);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 dyv = __bfloat1622float2(dyb[t]);
        const float2 gf = __bfloat1622float2(gb[t]);
        const float g0 = sigmoid_f(gf.x), g1 = sigmoid_f(gf.y);
        const float l0 = __uint_as_float(ro[j + 2 * t]), l1 = __uint_as_float(ro[j + 2 * t + 1]);
        const float m0 = __uint_as_float(rm[j + 2 * t]) * 0.125f, m1 = __uint_as_float(rm[j + 2 * t + 1]) * 0.125f;
        const float dl0 = dyv.x * g0, dl1 = dyv.y * g1;
        Drow += dl0 * l0 + dl1 * l1;
        w_dl[t] = pack_bf16x2(dl0, dl1);
        w_dg[t] = pack_bf16x2(dyv.x * (l0 - m0) * g0 * (1.f - g0), dyv.y * (l1 - m1) * g1 * (1.f - g1));
      }
      *pdl = o_dl;
      dgate_row[chunk] = o_dg;
    }
  }
  tc_fence_before_sync();
  fence_proxy_async_smem();
  __syncthreads();
  // ---- MMA C: dP = dlocal V^T, dV = P^T dlocal
  if (tid == 0 && ok) {
    tc_fence_after_sync();
    constexpr uint32_t idesc_kk128 = make_idesc_bf16(128, 128, false, false);
    constexpr uint32_t idesc_mnmn64 = make_idesc_bf16(128, 64, true, true);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k)
      umma_bf16(t_lo, make_smem_desc_sw128(smem_u32(sB2) + k * 32, 0, 1024),
                make_smem_desc_sw128(smem_u32(sB3) + k * 32, 0, 1024), idesc_kk128, k > 0);
#pragma unroll
    for (int k = 0; k < CHUNK / 16; ++k)
      umma_bf16(t_mid, make_smem_desc_sw128(smem_u32(sP) + k * 2048, TILE_BYTES, 1024),
                make_smem_desc_sw128(smem_u32(sB2) + k * 2048, 0, 1024), idesc_mnmn64, k > 0);
    umma_commit(&bars[4]);
  }
  ok = mbar_wait(&bars[4], 0, abort_flag) && ok;
  tc_fence_after_sync();
  if (tid == 0 && ok) {  // B2 (dlocal) has been consumed: fetch U into it behind the dS phase
    mbar_expect_tx(&bars[5], TILE_BYTES);
    tma_load_2d(sB2, &tm_qkvgu, &bars[5], 4 * d + h * HD, row0);
  }

  // ---- dS = P * (dP - D) / 8 over P; dV out; tanh(Kr) -> B3
  for (int cc = 0; cc <= last_chunk; ++cc) {
    uint32_t r[32], pk[16];
    tmem_ld_32x32b_x32(t_lo + lane_base + cc * 32, r);
    load_row_chunk32(sP, tid, cc * 32, pk);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 pv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[j]));
      const float s0 = pv.x * (__uint_as_float(r[2 * j]) - Drow) * 0.125f;
      const float s1 = pv.y * (__uint_as_float(r[2 * j + 1]) - Drow) * 0.125f;
      pk[j] = pack_bf16x2(s0, s1);
    }
    store_row_chunk32(sP, tid, cc * 32, pk);
  }
#pragma unroll
  for (int c = 0; c < HD; c += 16) {
    uint32_t rv[16];
    tmem_ld_32x32b_x16(t_mid + lane_base + c, rv);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; j += 8) {
      dv_row[(c + j) >> 3] = make_uint4(pack_bf16x2(__uint_as_float(rv[j]), __uint_as_float(rv[j + 1])),
                                        pack_bf16x2(__uint_as_float(rv[j + 2]), __uint_as_float(rv[j + 3])),
                                        pack_bf16x2(__uint_as_float(rv[j + 4]), __uint_as_float(rv[j + 5])),
                                        pack_bf16x2(__uint_as_float(rv[j + 6]), __uint_as_float(rv[j + 7])));
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {  // tanh(Kr) -> B3 (V is no longer needed)
    const uint4 kq = *reinterpret_cast<const uint4*>(tile_chunk(sK, tid, j));
    const __nv_bfloat162* kb = reinterpret_cast<const __nv_bfloat162*>(&kq);
    uint4 o;
    uint32_t* wo = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 kv = __bfloat1622float2(kb[t]);
      wo[t] = pack_bf16x2(tanh_fast(kv.x), tanh_fast(kv.y));
    }
    *reinterpret_cast<uint4*>(tile_chunk(sB3, tid, j)) = o;
  }
  ok = mbar_wait(&bars[5], 0, abort_flag) && ok;  // U has landed
  if (ok) rope_tanh_row(sB2, tid, rope, false, true);
  tc_fence_before_sync();
  fence_proxy_async_smem();
  __syncthreads();
  // ---- MMA D: dQr += dS Kr, dKr = dS^T Qr, dtK = tU dW^T, dtU = tK dW
  if (tid == 0 && ok) {
    tc_fence_after_sync();
    constexpr uint32_t idesc_kmn64 = make_idesc_bf16(128, 64, false, true);
    constexpr uint32_t idesc_mnmn64 = make_idesc_bf16(128, 64, true, true);
    constexpr uint32_t idesc_kk64 = make_idesc_bf16(128, 64, false, false);
#pragma unroll
    for (int k = 0; k < CHUNK / 16; ++k)
      umma_bf16(t_dq, make_smem_desc_sw128(smem_u32(sP) + (k >> 2) * TILE_BYTES + (k & 3) * 32, 0, 1024),
                make_smem_desc_sw128(smem_u32(sK) + k * 2048, 0, 1024), idesc_kmn64, 1u);
#pragma unroll
    for (int k = 0; k < CHUNK / 16; ++k)
      umma_bf16(t_lo, make_smem_desc_sw128(smem_u32(sP) + k * 2048, TILE_BYTES, 1024),
                make_smem_desc_sw128(smem_u32(sQ) + k * 2048, 0, 1024), idesc_mnmn64, k > 0);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k)  // dtK = tU dW^T
      umma_bf16(t_lo + 64, make_smem_desc_sw128(smem_u32(sB2) + k * 32, 0, 1024),
                make_smem_desc_sw128(smem_u32(sDW) + k * 32, 0, 1024), idesc_kk64, k > 0);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k)  // dtU = tK dW
      umma_bf16(t_mid, make_smem_desc_sw128(smem_u32(sB3) + k * 32, 0, 1024),
                make_smem_desc_sw128(smem_u32(sDW) + k * 2048, 0, 1024), idesc_kmn64, k > 0);
    umma_commit(&bars[6]);
  }
  ok = mbar_wait(&bars[6], 0, abort_flag) && ok;
  tc_fence_after_sync();

  // ---- final: dQ, dK (RoPE transpose), dU
#pragma unroll
  for (int c = 0; c < HD; c += 16) {
    uint32_t rq[16], rk[16], rtk[16], rtu[16];
    tmem_ld_32x32b_x16(t_dq + lane_base + c, rq);
    tmem_ld_32x32b_x16(t_lo + lane_base + c, rk);
    tmem_ld_32x32b_x16(t_lo + 64 + lane_base + c, rtk);
    tmem_ld_32x32b_x16(t_mid + lane_base + c, rtu);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; j += 8) {
      const int chunk = (c + j) >> 3;
      const uint4 tkq = *reinterpret_cast<const uint4*>(tile_chunk(sB3, tid, chunk));
      const uint4 tuq = *reinterpret_cast<const uint4*>(tile_chunk(sB2, tid, chunk));
      const __nv_bfloat162* tkb = reinterpret_cast<const __nv_bfloat162*>(&tkq);
      const __nv_bfloat162* tub = reinterpret_cast<const __nv_bfloat162*>(&tuq);
      uint4 o_q, o_k, o_u;
      uint32_t* w_q = reinterpret_cast<uint32_t*>(&o_q);
      uint32_t* w_k = reinterpret_cast<uint32_t*>(&o_k);
      uint32_t* w_u = reinterpret_cast<uint32_t*>(&o_u);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int e0 = j + 2 * t, e1 = e0 + 1;
        const float2 cs = rope[((c + e0) >> 1) * CHUNK + tid];
        const float2 tk = __bfloat1622float2(tkb[t]);
        const float2 tu = __bfloat1622float2(tub[t]);
        // y0 = x0 c - x1 s ; y1 = x1 c + x0 s   =>   dx0 = dy0 c + dy1 s ; dx1 = dy1 c - dy0 s
        const float q0 = __uint_as_float(rq[e0]), q1 = __uint_as_float(rq[e1]);
        w_q[t] = pack_bf16x2(q0 * cs.x + q1 * cs.y, q1 * cs.x - q0 * cs.y);
        const float k0 = __uint_as_float(rk[e0]) + __uint_as_float(rtk[e0]) * (1.f / CHUNK) * (1.f - tk.x * tk.x);
        const float k1 = __uint_as_float(rk[e1]) + __uint_as_float(rtk[e1]) * (1.f / CHUNK) * (1.f - tk.y * tk.y);
        w_k[t] = pack_bf16x2(k0 * cs.x + k1 * cs.y, k1 * cs.x - k0 * cs.y);
        w_u[t] = pack_bf16x2(__uint_as_float(rtu[e0]) * (1.f / CHUNK) * (1.f - tu.x * tu.x),
                             __uint_as_float(rtu[e1]) * (1.f / CHUNK) * (1.f - tu.y * tu.y));
      }
      // every operand of the last MMA group has been consumed: Q, K, P, State and dW tiles are free
      *reinterpret_cast<uint4*>(tile_chunk(sQ, tid, chunk)) = o_q;
      *reinterpret_cast<uint4*>(tile_chunk(sK, tid, chunk)) = o_k;
      *reinterpret_cast<uint4*>(tile_chunk(sP, tid, chunk)) = o_u;
      *reinterpret_cast<uint4*>(tile_chunk(sP + TILE_BYTES, tid, chunk)) = dgate_row[chunk];
      *reinterpret_cast<uint4*>(tile_chunk(sSt, tid, chunk)) = dv_row[chunk];
    }
  }
  fence_proxy_async_smem();
  __syncwarp();
  if ((tid & 31) == 0) {  // one store per gradient tile for the warp's 32 token rows
    if (ok) {
      const int r = row0 + warp * 32, off = warp * 4096;
      tma_store_2d(&tm_dout, sQ + off, 0 * d + h * HD, r);
      tma_store_2d(&tm_dout, sK + off, 1 * d + h * HD, r);
      tma_store_2d(&tm_dout, sSt + off, 2 * d + h * HD, r);
      tma_store_2d(&tm_dout, sP + TILE_BYTES + off, 3 * d + h * HD, r);
      tma_store_2d(&tm_dout, sP + off, 4 * d + h * HD, r);
      tma_store_commit();
    }
    tma_store_wait_read0();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag != 0 && error_flag != nullptr) atomicExch(error_flag, 5);
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 256);
  }
}

}  // namespace ws

using namespace ws;

extern "C" int ws_attn_dstate(const void* qkvgu, const void* dy, const float* rope, float* dstate, int B, int T,
                              int H, int d, int* error_flag, cudaStream_t stream) {
  if (T % CHUNK != 0 || d != H * HD) return -1;
  CUtensorMap tm, td, to;
  int rc = make_tile_map(&tm, qkvgu, 5 * (uint64_t)d, (uint64_t)B * T, 5 * (uint64_t)d, HD, CHUNK);
  if (rc) return rc;
  rc = make_tile_map(&td, dy, (uint64_t)d, (uint64_t)B * T, (uint64_t)d, HD, CHUNK);
  if (rc) return rc;
  rc = make_map_f32(&to, dstate, HD, (uint64_t)B * (T / CHUNK) * H * HD, HD, 32, 32);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(dstate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DS_SMEM) != cudaSuccess)
      return -20;
    configured = true;
  }
  const int tiles = B * (T / CHUNK) * H;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaFuncSetAttribute(dstate_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DSS_SMEM) != cudaSuccess)
      return -20;
  }
  if (ws_attn_stream_form() != 0)
    launch_dependent(dstate_stream_kernel, dim3(tiles < sms ? tiles : sms), dim3(DSS_THREADS), DSS_SMEM, stream, tm, td, to,
                     reinterpret_cast<const float2*>(rope), T, H, d, tiles, error_flag);
  else
    launch_dependent(dstate_kernel, dim3(tiles), dim3(128), DS_SMEM, stream, tm, td, to, reinterpret_cast<const float2*>(rope), T, H, d,
                     error_flag);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ws_memory_scan_bwd(const float* dstate, const float* writes, const float* fast_logit,
                                  const float* slow_logit, const float* mix_logit, void* dwrites, float* partials,
                                  int B, int N, int H, cudaStream_t stream) {
  if (N > SCAN_MAX_CHUNKS) return -1;
  const size_t total = (size_t)B * H * 4096;
  launch_dependent(memory_scan_bwd_kernel, dim3((unsigned)(total / 256)), dim3(256), 0, stream, dstate, writes, fast_logit, slow_logit,
                                                                      mix_logit, (__nv_bfloat16*)dwrites, partials,
                                                                      B, N, H);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ws_attn_bwd(const void* qkvgu, const void* states, const void* dy, const void* dwrites,
                           const float* rope, void* dqkvgu, int B, int T, int H, int d, int* error_flag,
                           cudaStream_t stream) {
  if (T % CHUNK != 0 || d != H * HD) return -1;
  const int tiles = B * (T / CHUNK) * H;
  CUtensorMap tm, ts, td, tw, to;
  int rc = make_tile_map(&tm, qkvgu, 5 * (uint64_t)d, (uint64_t)B * T, 5 * (uint64_t)d, HD, CHUNK);
  if (rc) return rc;
  rc = make_tile_map(&to, dqkvgu, 5 * (uint64_t)d, (uint64_t)B * T, 5 * (uint64_t)d, HD, 32);
  if (rc) return rc;
  rc = make_tile_map(&ts, states, HD, (uint64_t)tiles * HD, HD, HD, HD);
  if (rc) return rc;
  rc = make_tile_map(&td, dy, (uint64_t)d, (uint64_t)B * T, (uint64_t)d, HD, CHUNK);
  if (rc) return rc;
  rc = make_tile_map(&tw, dwrites, HD, (uint64_t)tiles * HD, HD, HD, HD);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AB_SMEM) != cudaSuccess)
      return -20;
    configured = true;
  }
  launch_dependent(attn_bwd_kernel, dim3(tiles), dim3(AB_THREADS), AB_SMEM, stream, tm, ts, td, tw, to, reinterpret_cast<const float2*>(rope),
                                                          T, H, d, error_flag);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
