// Decode-step kernels: one new token for every sequence of a batch (batch <= 64).
//
// A decode step is bound by streaming the weights once (4.0 GB for the 2.005 B model) and the
// current chunk's K/V cache, so the GEMMs here are weight-streaming kernels, not tile kernels:
//
//   decode_gemm_kernel     out[b, n] = sum_k x[b, k] W[n, k].  The roles of the MMA operands are
//                          swapped with respect to training: 128 weight rows are the M dimension of
//                          tcgen05.mma, the (padded) batch is its N dimension, so one CTA streams a
//                          128-row slab of W exactly once through an 8-stage TMA ring while the
//                          tiny activation block comes from L2.  Slabs x K-splits give >= 128 CTAs
//                          for every projection of the model; split partials are FP32.
//                          Epilogues: BF16, FP32 (logits), FP32 split-K partial, SwiGLU (64 up rows
//                          and their 64 gate rows share a slab).
//   decode_reduce_norm_kernel  x += sum of split partials (or x = embedding row), optional depth
//                          modulation of the next layer, RMSNorm -> BF16: everything between two
//                          GEMMs of the residual stream in one pass, one CTA per sequence.
//   decode_attn_kernel     one CTA per (sequence, head): RoPE of q/k at the in-chunk position,
//                          append k/v/u to the chunk cache, causal attention over the cache rows
//                          <= position, memory read q.M, gate blend.
//
// The ~200 launches of a step form one chain of programmatic dependent launches: every kernel lets
// its successor start at once, and a GEMM fills its whole TMA ring with weight tiles (which no
// kernel of the step writes) before it waits for its predecessor, so the weight stream of the
// next projection runs under the small kernels and the tail of the previous GEMM.
//
// Reference semantics: WarpStateCore.step (reference warpstate/model.py:222-274) in the
// training-consistent form of ops/posttrain_chat.py:94-142.  The reference runs these as
// ~40 eager PyTorch ops per layer at batch 1.
#include "ws_ptx.cuh"
#include "ws_api.h"
#include "ws_tma_host.h"

#include <cuda_bf16.h>

#include <cstdlib>

namespace ws {

extern "C" void ws_count_launch(void);

namespace dec {
constexpr int TM = 128;  // weight rows per slab
constexpr int BK = 64;
constexpr int THREADS = 192;  // warp 0 TMA, warp 1 MMA + TMEM, warps 2..5 epilogue
constexpr int W_BYTES = TM * BK * 2;
}  // namespace dec

struct DecodeGemmParams {
  int n;        // output features (SwiGLU: hidden size h; W has 2h rows)
  int k;
  int batch;
  int kb_per_split;
  int packed;   // W is stored tile by tile: [slab][k block][128 rows][64 columns], each tile contiguous
  void* out;    // BF16 [batch, ldo] | FP32 [batch, ldo] | FP32 partial [splits, batch, n]
  int ldo;
  int* error_flag;
};

// DEPTH = stages of the TMA ring.  8: one CTA per SM with 192 KiB of tiles in flight.  4: half the ring, so that
// two CTAs fit on an SM -- the successor of a launch in the dependent chain can then become resident, set up and
// request its first ring of weights while its predecessor still occupies every SM.  The SwiGLU exchange buffer
// overlays the first ring stages (the ring is idle once the last MMA has completed).
template <int BPAD, int DEPTH>
struct DecodeCfg {
  static constexpr int STAGES = DEPTH;
  static constexpr int X_BYTES = BPAD * dec::BK * 2;
  static constexpr int STAGE_BYTES = dec::W_BYTES + X_BYTES;
  static constexpr int EXCHANGE_BYTES = 64 * BPAD * 4;
  static_assert(EXCHANGE_BYTES <= STAGES * dec::W_BYTES, "the exchange buffer overlays the weight stages");
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = BPAD < 32 ? 32 : BPAD;
  static constexpr int CTAS_PER_SM = 2 * (SMEM + 1024) <= 233472 ? 2 : 1;
};

// EPI: 0 = BF16 out, 1 = FP32 split-K partial, 2 = SwiGLU (BF16 activation), 3 = FP32 out
template <int BPAD, int EPI, int DEPTH>
__global__ void __launch_bounds__(dec::THREADS, DecodeCfg<BPAD, DEPTH>::CTAS_PER_SM)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const DecodeGemmParams p) {
  using namespace dec;
  using Cfg = DecodeCfg<BPAD, DEPTH>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sW = smem;
  uint8_t* sX = smem + Cfg::STAGES * W_BYTES;
  float* sG = reinterpret_cast<float*>(sW);  // written only after the last MMA has read the ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::STAGES;
  uint64_t* tfull = bars + 2 * Cfg::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tfull, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();

  const int slab = blockIdx.x;
  const int total_kb = (p.k + BK - 1) / BK;
  const int kb0 = blockIdx.y * p.kb_per_split;
  const int kb1 = min(total_kb, kb0 + p.kb_per_split);
  const int rows_per_slab = EPI == 2 ? 64 : TM;
  const int n0 = slab * rows_per_slab;

  if (warp == 0) {
    if (lane == 0) {
      auto load_w = [&](int s, int kb) {
        mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
        if (p.packed) {  // one contiguous 16 KiB tile (SwiGLU: the up and gate rows are already paired)
          tma_load_2d(sW + s * W_BYTES, &tm_w, &full[s], 0, (slab * total_kb + kb) * TM);
          return;
        }
        tma_load_2d(sW + s * W_BYTES, &tm_w, &full[s], kb * BK, n0);
        if (EPI == 2)  // 64 up rows + the 64 matching gate rows
          tma_load_2d(sW + s * W_BYTES + 64 * 128, &tm_w, &full[s], kb * BK, p.n + n0);
      };
      // Every CTA walks its k blocks from a different starting block (wrapping around): all CTAs of a
      // launch read the same activation tiles, and in lock step they would queue on the few L2
      // slices that hold the current one.
      const int nkb = kb1 - kb0;
      const int rot = nkb > 0 ? static_cast<int>((blockIdx.x * 5u + blockIdx.y * 3u) % static_cast<unsigned>(nkb)) : 0;
      auto block_of = [&](int it) {
        const int r = it + rot;
        return kb0 + (r >= nkb ? r - nkb : r);
      };
      // The weights are constant during a step: the first ring of weight tiles is requested before
      // the wait for the previous kernel, whose output is this kernel's activation block.
      const int pre = min(nkb, Cfg::STAGES);
      for (int it = 0; it < pre; ++it) load_w(it, block_of(it));
      pdl_wait();
      for (int it = 0; it < pre; ++it) tma_load_2d(sX + it * Cfg::X_BYTES, &tm_x, &full[it], block_of(it) * BK, 0);
      for (int it = pre; it < nkb; ++it) {
        const int s = it % Cfg::STAGES;
        const uint32_t ph = (it / Cfg::STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) break;
        const int kb = block_of(it);
        load_w(s, kb);
        tma_load_2d(sX + s * Cfg::X_BYTES, &tm_x, &full[s], kb * BK, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TM, BPAD, false, false);
      bool ok = true;
      for (int kb = kb0, it = 0; kb < kb1; ++kb, ++it) {
        const int s = it % Cfg::STAGES;
        const uint32_t ph = (it / Cfg::STAGES) & 1;
        if (!mbar_wait(&full[s], ph, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t a = smem_u32(sW + s * W_BYTES), b = smem_u32(sX + s * Cfg::X_BYTES);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_bf16(tmem, make_smem_desc_sw128(a + k * 32, 0, 1024), make_smem_desc_sw128(b + k * 32, 0, 1024), idesc,
                    (it | k) != 0 ? 1u : 0u);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(tfull);
    }
  } else {
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    const int row = quarter * 32 + lane;
    const bool ok = kb1 > kb0 && mbar_wait(tfull, 0, abort_flag);
    tc_fence_after_sync();
    const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    if (EPI == 2) {
      // rows 0..63 = up, 64..127 = gate: the gate warps hand silu-ready values over through smem
      if (row >= 64 && ok) {
#pragma unroll
        for (int c0 = 0; c0 < BPAD; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g = __uint_as_float(r[j]);
            sG[(c0 + j) * 64 + (row - 64)] = g * sigmoid_fast(g);
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (row < 64 && ok) {
        const int hcol = n0 + row;
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
        for (int c0 = 0; c0 < BPAD; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int b = c0 + j;
            if (b < p.batch && hcol < p.n)
              out[static_cast<size_t>(b) * p.ldo + hcol] = __float2bfloat16(__uint_as_float(r[j]) * sG[b * 64 + row]);
          }
        }
      }
    } else if (ok) {
      const int n = n0 + row;
#pragma unroll
      for (int c0 = 0; c0 < BPAD; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int b = c0 + j;
          if (b >= p.batch || n >= p.n) continue;
          const float v = __uint_as_float(r[j]);
          if (EPI == 0) {
            static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(b) * p.ldo + n] = __float2bfloat16(v);
          } else if (EPI == 3) {
            static_cast<float*>(p.out)[static_cast<size_t>(b) * p.ldo + n] = v;
          } else {
            static_cast<float*>(p.out)[(static_cast<size_t>(blockIdx.y) * p.batch + b) * p.n + n] = v;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && p.error_flag != nullptr) atomicExch(p.error_flag, 8);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// --------------------------------------------------------------------------- residual + norm
// One CTA per sequence.  x (FP32 residual stream, [batch, d]) is updated in place:
//   token != null : x = table[token[b]]           (embedding gather)
//   partial != null: x += sum_s partial[s][b]     (split-K partials of the previous projection)
//   scale != null : x = x * (1 + scale) + bias    (depth modulation of the layer that follows)
// then out = BF16(x * rsqrt(mean(x^2) + eps) * w).
__global__ void __launch_bounds__(256)
decode_reduce_norm_kernel(float* __restrict__ x, const float* __restrict__ partial, int splits,
                          const long long* __restrict__ token, const float* __restrict__ table, int vocab,
                          const float* __restrict__ scale, const float* __restrict__ bias, const float* __restrict__ w,
                          float eps, int d, int batch, __nv_bfloat16* __restrict__ out) {
  __shared__ float red[8];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  float* xr = x + static_cast<size_t>(b) * d;
  const float* src = xr;
  if (token != nullptr) {
    long long id = token[b];
    if (id < 0) id = 0;
    if (id >= vocab) id = vocab - 1;
    src = table + static_cast<size_t>(id) * d;
  }
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < d; c += 256 * 4) {
    float4 v = *reinterpret_cast<const float4*>(src + c);
    for (int s = 0; s < splits; ++s) {
      const float4 q = *reinterpret_cast<const float4*>(partial + (static_cast<size_t>(s) * batch + b) * d + c);
      v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
    }
    if (scale != nullptr) {
      const float4 sc = *reinterpret_cast<const float4*>(scale + c), bi = *reinterpret_cast<const float4*>(bias + c);
      v.x = v.x * (1.f + sc.x) + bi.x; v.y = v.y * (1.f + sc.y) + bi.y;
      v.z = v.z * (1.f + sc.z) + bi.z; v.w = v.w * (1.f + sc.w) + bi.w;
    }
    *reinterpret_cast<float4*>(xr + c) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += red[i];
  const float rstd = rsqrtf(total / static_cast<float>(d) + eps);
  if (out == nullptr) return;
  for (int c = threadIdx.x * 4; c < d; c += 256 * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + c);  // this thread's own stores
    const float4 ww = *reinterpret_cast<const float4*>(w + c);
    uint2 o;
    o.x = pack_bf16x2(v.x * rstd * ww.x, v.y * rstd * ww.y);
    o.y = pack_bf16x2(v.z * rstd * ww.z, v.w * rstd * ww.w);
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(b) * d + c) = o;
  }
}

// --------------------------------------------------------------------------- attention step
// One CTA of 128 threads per (sequence, head); head_dim 64, chunk 128.
// qkvgu: [batch, 5*d] BF16 (q | k | v | gate | u); caches kc/vc/uc: [batch, H, 128, 64] BF16;
// mixed: [batch, H, 64, 64] BF16 (mix*fast + (1-mix)*slow); rope: [128, 32] (cos, sin);
// y: [batch, d] BF16.  `pos_ptr` is the in-chunk position (device scalar, so that one captured
// graph serves every position).
__global__ void __launch_bounds__(128)
decode_attn_kernel(const __nv_bfloat16* __restrict__ qkvgu, __nv_bfloat16* __restrict__ kc,
                   __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ uc,
                   const __nv_bfloat16* __restrict__ mixed, const float2* __restrict__ rope,
                   const long long* __restrict__ pos_ptr, int H, int d, __nv_bfloat16* __restrict__ y) {
  constexpr int HD = 64, C = 128;
  __shared__ float sq[HD], sk[HD], sp[C], sl[16][HD + 1], sm[16][HD + 1], sred[4];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x % H, b = blockIdx.x / H;
  pdl_launch_dependents();
  pdl_wait();
  int pos = static_cast<int>(*pos_ptr);
  pos = pos < 0 ? 0 : (pos >= C ? C - 1 : pos);
  const __nv_bfloat16* row = qkvgu + static_cast<size_t>(b) * 5 * d + h * HD;
  const size_t cache = (static_cast<size_t>(b) * H + h) * C * HD;
  // Thread (rg, jg) owns columns 8*jg .. 8*jg+7 of the rows rg, rg+16, ... of the K and V caches and of M: a warp
  // instruction reads four whole 128-byte rows.  Every load the step needs from the caches is issued here, before
  // the RoPE of the new token, so that the three dependent phases below (scores, softmax, P.V) wait for memory once.
  const int jg = tid & 7, rg = tid >> 3;
  uint4 kreg[C / 16], vreg[C / 16], mreg[HD / 16];
#pragma unroll
  for (int it = 0; it < C / 16; ++it) {
    const int c = rg + it * 16;
    if (c < pos) {
      kreg[it] = *reinterpret_cast<const uint4*>(kc + cache + static_cast<size_t>(c) * HD + jg * 8);
      vreg[it] = *reinterpret_cast<const uint4*>(vc + cache + static_cast<size_t>(c) * HD + jg * 8);
    } else if (c == pos) {
      vreg[it] = *reinterpret_cast<const uint4*>(row + 2 * d + jg * 8);  // the new token's own value row
    }
  }
  const __nv_bfloat16* mbase = mixed + (static_cast<size_t>(b) * H + h) * HD * HD;
#pragma unroll
  for (int it = 0; it < HD / 16; ++it) mreg[it] = *reinterpret_cast<const uint4*>(mbase + (rg + it * 16) * HD + jg * 8);
  // RoPE (adjacent pairs) of q and k; append k, v, u at `pos`
  if (tid < 32) {
    const float2 cs = rope[pos * 32 + tid];
    const float2 q = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + 2 * tid));
    const float2 k = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + d + 2 * tid));
    // round through BF16 as the cached / batched path does
    const __nv_bfloat162 qr = __floats2bfloat162_rn(q.x * cs.x - q.y * cs.y, q.y * cs.x + q.x * cs.y);
    const __nv_bfloat162 kr = __floats2bfloat162_rn(k.x * cs.x - k.y * cs.y, k.y * cs.x + k.x * cs.y);
    const float2 qf = __bfloat1622float2(qr), kf = __bfloat1622float2(kr);
    sq[2 * tid] = qf.x; sq[2 * tid + 1] = qf.y;
    sk[2 * tid] = kf.x; sk[2 * tid + 1] = kf.y;
    *reinterpret_cast<__nv_bfloat162*>(kc + cache + static_cast<size_t>(pos) * HD + 2 * tid) = kr;
  } else if (tid < 64) {
    const int t = tid - 32;
    *reinterpret_cast<__nv_bfloat162*>(vc + cache + static_cast<size_t>(pos) * HD + 2 * t) =
        *reinterpret_cast<const __nv_bfloat162*>(row + 2 * d + 2 * t);
  } else if (tid < 96) {
    const int t = tid - 64;
    *reinterpret_cast<__nv_bfloat162*>(uc + cache + static_cast<size_t>(pos) * HD + 2 * t) =
        *reinterpret_cast<const __nv_bfloat162*>(row + 4 * d + 2 * t);
  }
  __syncthreads();
  // scores: the eight lanes of a row group each hold an eighth of q . k[c]; key `pos` is the new token's own
  {
    float qv[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) qv[t] = sq[jg * 8 + t];
#pragma unroll
    for (int it = 0; it < C / 16; ++it) {
      const int c = rg + it * 16;
      float acc = 0.f;
      if (c < pos) {
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&kreg[it]);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = __bfloat1622float2(pb[t]);
          acc += qv[2 * t] * f.x + qv[2 * t + 1] * f.y;
        }
      } else if (c == pos) {
#pragma unroll
        for (int t = 0; t < 8; ++t) acc += qv[t] * sk[jg * 8 + t];
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (jg == 0) sp[c] = acc * 0.125f;
    }
  }
  __syncthreads();
  const float score = tid <= pos ? sp[tid] : -INFINITY;
  float m = score;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) sred[warp] = m;
  __syncthreads();
  m = fmaxf(fmaxf(sred[0], sred[1]), fmaxf(sred[2], sred[3]));
  const float e = tid <= pos ? __expf(score - m) : 0.f;
  float s = e;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __syncthreads();
  if (lane == 0) sred[warp] = s;
  sp[tid] = e;
  __syncthreads();
  const float inv = 1.f / (sred[0] + sred[1] + sred[2] + sred[3]);
  // local = sum_c p[c] V[c] and memory = q . M from the rows already in registers; the 16 row groups are then
  // summed through shared memory.
  {
    float accl[8], accm[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) { accl[t] = 0.f; accm[t] = 0.f; }
#pragma unroll
    for (int it = 0; it < C / 16; ++it) {
      const int c = rg + it * 16;
      if (c <= pos) {
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&vreg[it]);
        const float pc = sp[c];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = __bfloat1622float2(pb[t]);
          accl[2 * t] += pc * f.x;
          accl[2 * t + 1] += pc * f.y;
        }
      }
    }
#pragma unroll
    for (int it = 0; it < HD / 16; ++it) {
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&mreg[it]);
      const float qi = sq[rg + it * 16];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = __bfloat1622float2(pb[t]);
        accm[2 * t] += qi * f.x;
        accm[2 * t + 1] += qi * f.y;
      }
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      sl[rg][jg * 8 + t] = accl[t];
      sm[rg][jg * 8 + t] = accm[t];
    }
  }
  __syncthreads();
  if (tid < HD) {
    float local = 0.f, mem = 0.f;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      local += sl[r][tid];
      mem += sm[r][tid];
    }
    local *= inv;
    mem *= 0.125f;
    const float g = sigmoid_fast(__bfloat162float(row[3 * d + tid]));
    y[static_cast<size_t>(b) * d + h * HD + tid] = __float2bfloat16(g * local + (1.f - g) * mem);
  }
}

// --------------------------------------------------------------------------- attention step, row-per-thread scores
// The earlier form of decode_attn_kernel (WS_DECODE_ATTN=rows): thread c computes the score of key c from its own
// 128-byte cache row, and the value / memory rows are read after the softmax.  Fewer registers (more CTAs per SM),
// three dependent memory phases.  One CTA of 128 threads per (sequence, head); head_dim 64, chunk 128.
// qkvgu: [batch, 5*d] BF16 (q | k | v | gate | u); caches kc/vc/uc: [batch, H, 128, 64] BF16;
// mixed: [batch, H, 64, 64] BF16 (mix*fast + (1-mix)*slow); rope: [128, 32] (cos, sin);
// y: [batch, d] BF16.  `pos_ptr` is the in-chunk position (device scalar, so that one captured
// graph serves every position).
__global__ void __launch_bounds__(128)
decode_attn_rows_kernel(const __nv_bfloat16* __restrict__ qkvgu, __nv_bfloat16* __restrict__ kc,
                   __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ uc,
                   const __nv_bfloat16* __restrict__ mixed, const float2* __restrict__ rope,
                   const long long* __restrict__ pos_ptr, int H, int d, __nv_bfloat16* __restrict__ y) {
  constexpr int HD = 64, C = 128;
  __shared__ float sq[HD], sk[HD], sp[C], sl[16][HD + 1], sm[16][HD + 1], sred[4];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x % H, b = blockIdx.x / H;
  pdl_launch_dependents();
  pdl_wait();
  int pos = static_cast<int>(*pos_ptr);
  pos = pos < 0 ? 0 : (pos >= C ? C - 1 : pos);
  const __nv_bfloat16* row = qkvgu + static_cast<size_t>(b) * 5 * d + h * HD;
  const size_t cache = (static_cast<size_t>(b) * H + h) * C * HD;
  // RoPE (adjacent pairs) of q and k; append k, v, u at `pos`
  if (tid < 32) {
    const float2 cs = rope[pos * 32 + tid];
    const float2 q = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + 2 * tid));
    const float2 k = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + d + 2 * tid));
    // round through BF16 as the cached / batched path does
    const __nv_bfloat162 qr = __floats2bfloat162_rn(q.x * cs.x - q.y * cs.y, q.y * cs.x + q.x * cs.y);
    const __nv_bfloat162 kr = __floats2bfloat162_rn(k.x * cs.x - k.y * cs.y, k.y * cs.x + k.x * cs.y);
    const float2 qf = __bfloat1622float2(qr), kf = __bfloat1622float2(kr);
    sq[2 * tid] = qf.x; sq[2 * tid + 1] = qf.y;
    sk[2 * tid] = kf.x; sk[2 * tid + 1] = kf.y;
    *reinterpret_cast<__nv_bfloat162*>(kc + cache + static_cast<size_t>(pos) * HD + 2 * tid) = kr;
  } else if (tid < 64) {
    const int t = tid - 32;
    *reinterpret_cast<__nv_bfloat162*>(vc + cache + static_cast<size_t>(pos) * HD + 2 * t) =
        *reinterpret_cast<const __nv_bfloat162*>(row + 2 * d + 2 * t);
  } else if (tid < 96) {
    const int t = tid - 64;
    *reinterpret_cast<__nv_bfloat162*>(uc + cache + static_cast<size_t>(pos) * HD + 2 * t) =
        *reinterpret_cast<const __nv_bfloat162*>(row + 4 * d + 2 * t);
  }
  __syncthreads();
  // scores: thread c owns key c
  float score = -INFINITY;
  if (tid <= pos) {
    float acc = 0.f;
    if (tid == pos) {
#pragma unroll
      for (int i = 0; i < HD; ++i) acc += sq[i] * sk[i];
    } else {
      const uint4* kr = reinterpret_cast<const uint4*>(kc + cache + static_cast<size_t>(tid) * HD);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 v = kr[j];
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = __bfloat1622float2(pb[t]);
          acc += sq[j * 8 + 2 * t] * f.x + sq[j * 8 + 2 * t + 1] * f.y;
        }
      }
    }
    score = acc * 0.125f;
  }
  float m = score;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) sred[warp] = m;
  __syncthreads();
  m = fmaxf(fmaxf(sred[0], sred[1]), fmaxf(sred[2], sred[3]));
  const float e = tid <= pos ? __expf(score - m) : 0.f;
  float s = e;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __syncthreads();
  if (lane == 0) sred[warp] = s;
  sp[tid] = e;
  __syncthreads();
  const float inv = 1.f / (sred[0] + sred[1] + sred[2] + sred[3]);
  // local = sum_c p[c] V[c] and memory = q . M in one pass of wide loads: thread (rg, jg) owns
  // columns 8*jg .. 8*jg+7 and the rows rg, rg+16, ... of V (keys) and of M; the 16 row groups
  // are then summed through shared memory.
  {
    const int jg = tid & 7, rg = tid >> 3;
    float accl[8], accm[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) { accl[t] = 0.f; accm[t] = 0.f; }
#pragma unroll
    for (int it = 0; it < C / 16; ++it) {
      const int c = rg + it * 16;
      if (c <= pos) {
        const uint4 v = (c == pos) ? *reinterpret_cast<const uint4*>(row + 2 * d + jg * 8)
                                   : *reinterpret_cast<const uint4*>(vc + cache + static_cast<size_t>(c) * HD + jg * 8);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&v);
        const float pc = sp[c];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = __bfloat1622float2(pb[t]);
          accl[2 * t] += pc * f.x;
          accl[2 * t + 1] += pc * f.y;
        }
      }
    }
    const __nv_bfloat16* mbase = mixed + (static_cast<size_t>(b) * H + h) * HD * HD;
#pragma unroll
    for (int it = 0; it < HD / 16; ++it) {
      const int i = rg + it * 16;
      const uint4 v = *reinterpret_cast<const uint4*>(mbase + i * HD + jg * 8);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&v);
      const float qi = sq[i];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = __bfloat1622float2(pb[t]);
        accm[2 * t] += qi * f.x;
        accm[2 * t + 1] += qi * f.y;
      }
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      sl[rg][jg * 8 + t] = accl[t];
      sm[rg][jg * 8 + t] = accm[t];
    }
  }
  __syncthreads();
  if (tid < HD) {
    float local = 0.f, mem = 0.f;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      local += sl[r][tid];
      mem += sm[r][tid];
    }
    local *= inv;
    mem *= 0.125f;
    const float g = sigmoid_fast(__bfloat162float(row[3 * d + tid]));
    y[static_cast<size_t>(b) * d + h * HD + tid] = __float2bfloat16(g * local + (1.f - g) * mem);
  }
}

// --------------------------------------------------------------------------- greedy pick
// One CTA per sequence: token[b] = argmax of logits[b, :] (the lowest index among equal maxima, as torch.argmax
// picks), written where the next step's embedding gather reads it and into column `*cursor` of the history
// [batch, capacity]; CTA 0 then advances the in-chunk position and the cursor.  With this kernel as the last node of
// the step graph a greedy decode needs nothing from the host between steps.
__global__ void __launch_bounds__(256)
decode_pick_kernel(const float* __restrict__ logits, int vocab, long long* __restrict__ token,
                   long long* __restrict__ history, int capacity, long long* __restrict__ cursor,
                   long long* __restrict__ pos) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float best_v[8];
  __shared__ int best_i[8];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* row = logits + static_cast<size_t>(b) * vocab;
  float v = -INFINITY;
  int at = 0x7fffffff;
  for (int c = threadIdx.x * 4; c < vocab; c += 256 * 4) {  // vocab % 4 == 0 (checked by the caller)
    const float4 q = *reinterpret_cast<const float4*>(row + c);
    const float e[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (e[j] > v || (e[j] == v && c + j < at)) {
        v = e[j];
        at = c + j;
      }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, at, o);
    if (ov > v || (ov == v && oi < at)) {
      v = ov;
      at = oi;
    }
  }
  if (lane == 0) {
    best_v[warp] = v;
    best_i[warp] = at;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (best_v[w] > v || (best_v[w] == v && best_i[w] < at)) {
        v = best_v[w];
        at = best_i[w];
      }
    if (at == 0x7fffffff) at = 0;  // a row of NaNs: any token, as long as it is a valid one
    const long long column = *cursor;
    token[b] = at;
    if (history != nullptr && column < capacity) history[static_cast<size_t>(b) * capacity + column] = at;
  }
  // every CTA has read the cursor before CTA 0 may advance it: CTA 0 waits for the others' arrival count
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned arrived = atomicAdd(reinterpret_cast<unsigned*>(cursor + 1), 1u) + 1u;
    if (arrived == gridDim.x) {
      *reinterpret_cast<unsigned*>(cursor + 1) = 0u;
      *cursor += 1;
      *pos += 1;
    }
  }
}

// Launch with the programmatic-stream-serialization attribute (WS_DECODE_PDL=0 launches normally).
template <typename... KArgs, typename... Args>
static cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args... args) {
  static const bool chained = [] {
    const char* e = std::getenv("WS_DECODE_PDL");
    return e == nullptr || e[0] != '0';
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

template <int BPAD, int EPI, int DEPTH>
static int launch_decode_gemm_depth(const CUtensorMap& tw, const CUtensorMap& tx, const DecodeGemmParams& p, dim3 grid,
                                    cudaStream_t stream) {
  static bool configured = false;
  auto kern = decode_gemm_kernel<BPAD, EPI, DEPTH>;
  using Cfg = DecodeCfg<BPAD, DEPTH>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) return -20;
    configured = true;
  }
  const cudaError_t err = launch_chained(kern, grid, dim3(dec::THREADS), Cfg::SMEM, stream, tw, tx, p);
  ws_count_launch();
  return err == cudaSuccess ? 0 : -21;
}

// WS_DECODE_STAGES=9 is the deepest ring that fits (217 KiB at batch 64).  WS_DECODE_STAGES=4 selects the shallow ring (two CTAs per SM); the default is 8 (one CTA per SM): measured at
// batch 64, 2.14 ms per token with 8 stages against 2.42 with 4 (2.21 with twice the K splits) -- the bytes a CTA
// keeps in flight matter more than letting the next launch become resident early.
static int decode_ring_depth() {
  static const int depth = [] {
    const char* e = std::getenv("WS_DECODE_STAGES");
    return e != nullptr && e[0] == '4' ? 4 : e != nullptr && e[0] == '9' ? 9 : 8;
  }();
  return depth;
}

template <int BPAD, int EPI>
static int launch_decode_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const DecodeGemmParams& p, dim3 grid,
                              cudaStream_t stream) {
  switch (decode_ring_depth()) {
    case 4: return launch_decode_gemm_depth<BPAD, EPI, 4>(tw, tx, p, grid, stream);
    case 9: return launch_decode_gemm_depth<BPAD, EPI, 9>(tw, tx, p, grid, stream);
    default: return launch_decode_gemm_depth<BPAD, EPI, 8>(tw, tx, p, grid, stream);
  }
}

}  // namespace ws

using namespace ws;

// Number of K splits ws_decode_gemm uses for an [n x k] weight (the caller sizes the FP32 partial
// buffer as splits * batch * n floats when the result is > 1).
extern "C" int ws_decode_gemm_splits(int n, int k) {
  // CTAs a split-K launch aims for: one per SM by default; WS_DECODE_SPLIT_CTAS overrides (two CTAs fit per SM
  // with the 4-stage ring)
  static const int target = [] {
    const char* e = std::getenv("WS_DECODE_SPLIT_CTAS");
    const int v = e != nullptr ? std::atoi(e) : 0;
    return v >= 16 && v <= 1184 ? v : 148;
  }();
  const int slabs = (n + dec::TM - 1) / dec::TM;
  const int total_kb = (k + dec::BK - 1) / dec::BK;
  int splits = target / (slabs > 0 ? slabs : 1);
  if (splits < 1) splits = 1;
  while (splits > 1 && total_kb / splits < 4) --splits;
  const int per = (total_kb + splits - 1) / splits;
  return (total_kb + per - 1) / per;  // no split is empty
}

// epilogue: 0 BF16 out [batch, ldo]; 1 FP32 split-K partials [splits, batch, n] (splits from
// ws_decode_gemm_splits); 2 SwiGLU, W is [2n, k] (up rows then gate rows), BF16 out [batch, ldo];
// 3 FP32 out [batch, ldo].  batch <= 64; k % 8 == 0.
// packed != 0: W is the tile-by-tile copy [slabs][ceil(k/64)][128][64] (zero padded; for SwiGLU a tile
// holds 64 up rows followed by their 64 gate rows), so that every TMA load reads 16 contiguous KiB
// instead of 128 row pieces of 128 bytes that lie a full weight row apart.
extern "C" int ws_decode_gemm(const void* w, const void* x, int n, int k, int batch, int epilogue, void* out, int ldo,
                              int* error_flag, int packed, cudaStream_t stream) {
  if (n <= 0 || k <= 0 || batch <= 0 || batch > 64 || k % 8 != 0 || epilogue < 0 || epilogue > 3) return -1;
  if (epilogue == 2 && n % 64 != 0) return -2;
  CUtensorMap tw, tx;
  const int w_rows = epilogue == 2 ? 2 * n : n;
  int rc;
  if (packed) {
    const uint64_t tiles = (uint64_t)(epilogue == 2 ? n / 64 : (n + dec::TM - 1) / dec::TM) * ((k + dec::BK - 1) / dec::BK);
    rc = make_map_bf16(&tw, w, dec::BK, tiles * dec::TM, dec::BK, dec::BK, dec::TM);
  } else {
    rc = make_map_bf16(&tw, w, k, w_rows, k, dec::BK, epilogue == 2 ? 64 : dec::TM);
  }
  if (rc) return rc;
  const int bpad = batch <= 16 ? 16 : 64;
  rc = make_map_bf16(&tx, x, k, batch, k, dec::BK, bpad);
  if (rc) return rc;
  DecodeGemmParams p;
  p.n = n; p.k = k; p.batch = batch; p.packed = packed; p.out = out; p.ldo = ldo; p.error_flag = error_flag;
  const int total_kb = (k + dec::BK - 1) / dec::BK;
  int splits = 1;
  if (epilogue == 1) splits = ws_decode_gemm_splits(n, k);
  p.kb_per_split = (total_kb + splits - 1) / splits;
  const int slabs = epilogue == 2 ? n / 64 : (n + dec::TM - 1) / dec::TM;
  const dim3 grid(slabs, splits);
  const int key = (bpad == 16 ? 0 : 4) + epilogue;
  switch (key) {
    case 0: return launch_decode_gemm<16, 0>(tw, tx, p, grid, stream);
    case 1: return launch_decode_gemm<16, 1>(tw, tx, p, grid, stream);
    case 2: return launch_decode_gemm<16, 2>(tw, tx, p, grid, stream);
    case 3: return launch_decode_gemm<16, 3>(tw, tx, p, grid, stream);
    case 4: return launch_decode_gemm<64, 0>(tw, tx, p, grid, stream);
    case 5: return launch_decode_gemm<64, 1>(tw, tx, p, grid, stream);
    case 6: return launch_decode_gemm<64, 2>(tw, tx, p, grid, stream);
    default: return launch_decode_gemm<64, 3>(tw, tx, p, grid, stream);
  }
}

extern "C" int ws_decode_reduce_norm(float* x, const float* partial, int splits, const long long* token,
                                     const float* table, int vocab, const float* scale, const float* bias,
                                     const float* w, float eps, int d, int batch, void* out, cudaStream_t stream) {
  if (d % 4 != 0 || batch <= 0 || (splits > 0 && partial == nullptr)) return -1;
  const cudaError_t err = launch_chained(decode_reduce_norm_kernel, dim3(batch), dim3(256), 0, stream, x, partial, splits,
                                         token, table, vocab, scale, bias, w, eps, d, batch,
                                         static_cast<__nv_bfloat16*>(out));
  ws_count_launch();
  return err == cudaSuccess ? 0 : -21;
}

extern "C" int ws_decode_attn(const void* qkvgu, void* kc, void* vc, void* uc, const void* mixed, const float* rope,
                              const long long* pos, int batch, int H, int d, void* y, cudaStream_t stream) {
  if (d != H * 64 || batch <= 0) return -1;
  // WS_DECODE_ATTN=rows selects the row-per-thread form of the kernel
  static const bool rows_form = [] {
    const char* e = std::getenv("WS_DECODE_ATTN");
    return e != nullptr && e[0] == 'r';
  }();
  const cudaError_t err = launch_chained(
      rows_form ? decode_attn_rows_kernel : decode_attn_kernel, dim3(batch * H), dim3(128), 0, stream,
      static_cast<const __nv_bfloat16*>(qkvgu),
      static_cast<__nv_bfloat16*>(kc), static_cast<__nv_bfloat16*>(vc), static_cast<__nv_bfloat16*>(uc),
      static_cast<const __nv_bfloat16*>(mixed), reinterpret_cast<const float2*>(rope), pos, H, d,
      static_cast<__nv_bfloat16*>(y));
  ws_count_launch();
  return err == cudaSuccess ? 0 : -21;
}

// token [batch] int64 = argmax(logits [batch, vocab] FP32); also stored in history[:, cursor[0]] (history may be
// NULL); then pos[0] += 1 and cursor[0] += 1.  cursor is two int64 words: the column, and a word of scratch (zero).
extern "C" int ws_decode_pick(const float* logits, int batch, int vocab, long long* token, long long* history,
                              int capacity, long long* cursor, long long* pos, cudaStream_t stream) {
  if (batch <= 0 || vocab <= 0 || vocab % 4 != 0) return -1;
  const cudaError_t err = launch_chained(decode_pick_kernel, dim3(batch), dim3(256), 0, stream, logits, vocab, token, history,
                                         capacity, cursor, pos);
  ws_count_launch();
  return err == cudaSuccess ? 0 : -21;
}
