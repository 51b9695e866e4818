// Decode step, the part of a layer that follows its attention: ONE persistent launch runs
//
//   out_proj (split-K partials) | residual + RMSNorm | up/gate + SwiGLU | down (split-K partials) |
//   residual + depth modulation of the next layer + RMSNorm | in_proj of the next layer
//
// on one CTA per SM, with a grid-wide barrier where a kernel boundary used to be.  What the five boundaries cost
// as separate launches of a dependent chain -- launch and drain, barrier initialisation, TMEM allocation, the
// first DRAM round trip of every projection -- is paid once: the TMEM accumulator and the TMA ring live for the
// whole launch, and because no phase writes weights, the producer warp requests the next projection's first ring
// of weight tiles while the current phase is still computing or waiting at its barrier; only the small activation
// tiles wait for the barrier.
//
// Roles per CTA (192 threads): warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2-5 epilogue, norm
// phases and the grid barrier.  A GEMM phase gives every CTA at most one work item (slab x K split): the grid must
// be at least as large as the largest phase (144 items for the 2.005 B shapes; the host refuses otherwise).
//
// Grid barrier: arrival counter in global memory (atomicAdd after a device-scope fence), a bounded spin on it, and
// a CTA-local word that tells the producer warp how many barriers have been passed.  The launch is cooperative, so
// every CTA is resident; should the spin run out of its time budget all the same, the CTA records it in the error
// word, raises its abort flag (every wait of the CTA then falls through) and the launch drains.
//
// Semantics and operand layouts are those of decode_gemm_kernel / decode_reduce_norm_kernel (decode.cu); k blocks
// are walked in the same rotated order, so the results are bit-identical to the launch-per-projection path.
#include "ws_ptx.cuh"
#include "ws_api.h"
#include "ws_tma_host.h"

#include <cuda_bf16.h>

namespace ws {

extern "C" void ws_count_launch(void);

namespace tail {
constexpr int TM = 128, BK = 64, BPAD = 64, STAGES = 8, THREADS = 192;
constexpr int W_BYTES = TM * BK * 2, X_BYTES = BPAD * BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
constexpr int EXCHANGE_BYTES = 64 * BPAD * 4;
constexpr int SMEM = STAGES * STAGE_BYTES + EXCHANGE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 64;
constexpr uint64_t kBarrierBudgetNs = 2000000000ull;
}  // namespace tail

struct LayerTailParams {
  int batch, d, ffn;
  int splits_out, kb_per_split_out;     // out_proj: [d x d]
  int splits_down, kb_per_split_down;   // down: [d x ffn]
  int has_in;                           // 0 for the last layer: the launch ends after the final norm
  float eps;
  float* x;                             // residual stream [batch, d] FP32, updated in place
  float* part_out;                      // [splits_out, batch, d]
  float* part_down;                     // [splits_down, batch, d]
  __nv_bfloat16* n;                     // [batch, d]: RMSNorm output (operand of up/gate, then of in_proj)
  __nv_bfloat16* act;                   // [batch, ffn]
  __nv_bfloat16* qkvgu;                 // [batch, 5 d] (next layer's projections)
  const float* w_norm2;                 // this layer's second norm
  const float* next_scale;              // depth modulation of the next layer (NULL after the last layer)
  const float* next_bias;
  const float* w_norm_next;             // next layer's first norm, or the final norm
  unsigned* barrier;                    // [0] arrivals, [1] exits; both zero between launches
  int* error_flag;
  long long* trace;                     // optional [grid, 16]: %globaltimer of every CTA at its phase boundaries
};

struct TailCta {
  uint8_t* sW;
  uint8_t* sX;
  float* sG;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* tfull;
  volatile unsigned* passed;   // barriers this CTA has passed (written by the epilogue leader)
  volatile int* abort_flag;
  uint32_t tmem;
};

// One GEMM work item: 128 weight rows (SwiGLU: 64 up + 64 gate) x the k blocks [kb0, kb1).
struct TailItem {
  bool valid;
  int slab, split, kb0, kb1, n0;
};

template <int EPI>
__device__ __forceinline__ TailItem tail_item(int index, int n, int k, int splits, int kb_per_split) {
  TailItem it;
  const int slabs = EPI == 2 ? n / 64 : (n + tail::TM - 1) / tail::TM;
  it.valid = index < slabs * splits;
  it.slab = index % slabs;
  it.split = index / slabs;
  const int total_kb = (k + tail::BK - 1) / tail::BK;
  it.kb0 = it.split * kb_per_split;
  it.kb1 = min(total_kb, it.kb0 + kb_per_split);
  it.n0 = it.slab * (EPI == 2 ? 64 : tail::TM);
  if (it.kb1 <= it.kb0) it.valid = false;
  return it;
}

__device__ __forceinline__ int tail_block_of(const TailItem& w, int i) {
  const int nkb = w.kb1 - w.kb0;
  const int rot = static_cast<int>((static_cast<unsigned>(w.slab) * 5u + static_cast<unsigned>(w.split) * 3u) %
                                   static_cast<unsigned>(nkb));
  const int r = i + rot;
  return w.kb0 + (r >= nkb ? r - nkb : r);
}

// Producer side of one GEMM phase.  `need` = barriers that must have been passed before the activation tiles may be
// read (0: they were written before the launch).  `pit` counts ring slots over the whole launch.
template <int EPI>
__device__ __forceinline__ void tail_produce(const TailCta& c, const CUtensorMap* tm_w, const CUtensorMap* tm_x,
                                             const TailItem& w, int n_total, unsigned need, uint32_t& pit) {
  using namespace tail;
  if (!w.valid) return;
  const int nkb = w.kb1 - w.kb0;
  auto load_w = [&](int s, int kb) {
    mbar_expect_tx(&c.full[s], STAGE_BYTES);
    tma_load_2d(c.sW + s * W_BYTES, tm_w, &c.full[s], kb * BK, w.n0);
    if (EPI == 2) tma_load_2d(c.sW + s * W_BYTES + 64 * 128, tm_w, &c.full[s], kb * BK, n_total + w.n0);
  };
  const int pre = min(nkb, STAGES);
  const uint32_t first = pit;
  for (int i = 0; i < pre; ++i, ++pit) {  // weights first: nothing in the step writes them
    const int s = pit % STAGES;
    if (!mbar_wait(&c.empty[s], ((pit / STAGES) & 1) ^ 1, c.abort_flag)) return;
    load_w(s, tail_block_of(w, i));
  }
  if (need > 0) {  // the activations of this phase exist once barrier `need` has been passed
    const uint64_t t0 = globaltimer_ns();
    while (*c.passed < need) {
      if (*c.abort_flag) return;
      if (globaltimer_ns() - t0 > kBarrierBudgetNs) {
        *c.abort_flag = 1;
        return;
      }
      __nanosleep(40);
    }
    asm volatile("fence.proxy.async;" ::: "memory");
  }
  for (int i = 0; i < pre; ++i) {
    const int s = (first + i) % STAGES;
    tma_load_2d(c.sX + s * X_BYTES, tm_x, &c.full[s], tail_block_of(w, i) * BK, 0);
  }
  for (int i = pre; i < nkb; ++i, ++pit) {
    const int s = pit % STAGES;
    if (!mbar_wait(&c.empty[s], ((pit / STAGES) & 1) ^ 1, c.abort_flag)) return;
    const int kb = tail_block_of(w, i);
    load_w(s, kb);
    tma_load_2d(c.sX + s * X_BYTES, tm_x, &c.full[s], kb * BK, 0);
  }
}

// MMA side.  `cit` mirrors the producer's slot counter.
__device__ __forceinline__ void tail_mma(const TailCta& c, const TailItem& w, uint32_t& cit) {
  using namespace tail;
  if (!w.valid) return;
  constexpr uint32_t idesc = make_idesc_bf16(TM, BPAD, false, false);
  const int nkb = w.kb1 - w.kb0;
  for (int i = 0; i < nkb; ++i, ++cit) {
    const int s = cit % STAGES;
    if (!mbar_wait(&c.full[s], (cit / STAGES) & 1, c.abort_flag)) return;
    tc_fence_after_sync();
    const uint32_t a = smem_u32(c.sW + s * W_BYTES), b = smem_u32(c.sX + s * X_BYTES);
#pragma unroll
    for (int k = 0; k < BK / 16; ++k)
      umma_bf16(c.tmem, make_smem_desc_sw128(a + k * 32, 0, 1024), make_smem_desc_sw128(b + k * 32, 0, 1024), idesc,
                (i | k) != 0 ? 1u : 0u);
    umma_commit(&c.empty[s]);
  }
  umma_commit(c.tfull);
}

// Epilogue of one item (warps 2..5, `et` = thread index within them).  EPI 0: BF16 [batch, ldo]; 1: FP32 partial
// [split, batch, n]; 2: SwiGLU, BF16 [batch, ldo].
template <int EPI>
__device__ __forceinline__ void tail_epilogue(const TailCta& c, const TailItem& w, int n, int batch, void* out, int ldo,
                                              uint32_t tparity, int warp, int lane) {
  using namespace tail;
  const int quarter = warp & 3;
  const int row = quarter * 32 + lane;
  const bool ok = w.valid && mbar_wait(c.tfull, tparity, c.abort_flag);
  tc_fence_after_sync();
  const uint32_t taddr = c.tmem + (static_cast<uint32_t>(quarter * 32) << 16);
  if (EPI == 2) {
    if (row >= 64 && ok) {
#pragma unroll
      for (int c0 = 0; c0 < BPAD; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float g = __uint_as_float(r[j]);
          c.sG[(c0 + j) * 64 + (row - 64)] = g * sigmoid_fast(g);
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (row < 64 && ok) {
      const int hcol = w.n0 + row;
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
#pragma unroll
      for (int c0 = 0; c0 < BPAD; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int b = c0 + j;
          if (b < batch && hcol < n)
            o[static_cast<size_t>(b) * ldo + hcol] = __float2bfloat16(__uint_as_float(r[j]) * c.sG[b * 64 + row]);
        }
      }
    }
  } else if (ok) {
    const int col = w.n0 + row;
#pragma unroll
    for (int c0 = 0; c0 < BPAD; c0 += 16) {
      uint32_t r[16];
      tmem_ld_32x32b_x16(taddr + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int b = c0 + j;
        if (b >= batch || col >= n) continue;
        const float v = __uint_as_float(r[j]);
        if (EPI == 0)
          static_cast<__nv_bfloat16*>(out)[static_cast<size_t>(b) * ldo + col] = __float2bfloat16(v);
        else
          static_cast<float*>(out)[(static_cast<size_t>(w.split) * batch + b) * n + col] = v;
      }
    }
  }
  tc_fence_before_sync();
}

// x[b] += sum of split partials; optional depth modulation; out[b] = BF16(RMSNorm(x[b]) * w).  128 threads, one row.
// The sum of squares is formed exactly as decode_reduce_norm_kernel forms it with 256 threads: thread t here plays
// that kernel's threads t (column blocks 0, 2, ...) and t + 128 (column blocks 1, 3, ...), the two sums are reduced
// per warp separately and the eight warp sums are added in the same order, so rstd is bit-identical.
__device__ __forceinline__ void tail_norm_row(float* x, const float* partial, int splits, int batch, int b, int d,
                                              const float* __restrict__ scale, const float* __restrict__ bias,
                                              const float* __restrict__ w, float eps, __nv_bfloat16* out, float* red,
                                              int et) {
  float* xr = x + static_cast<size_t>(b) * d;
  float ss[2] = {0.f, 0.f};
  int block = 0;
  for (int col = et * 4; col < d; col += 128 * 4, ++block) {
    float4 v = *reinterpret_cast<const float4*>(xr + col);
    for (int s = 0; s < splits; ++s) {  // written by other CTAs in this launch: read through L2
      const float4 q = __ldcg(reinterpret_cast<const float4*>(partial + (static_cast<size_t>(s) * batch + b) * d + col));
      v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
    }
    if (scale != nullptr) {
      const float4 sc = *reinterpret_cast<const float4*>(scale + col), bi = *reinterpret_cast<const float4*>(bias + col);
      v.x = v.x * (1.f + sc.x) + bi.x; v.y = v.y * (1.f + sc.y) + bi.y;
      v.z = v.z * (1.f + sc.z) + bi.z; v.w = v.w * (1.f + sc.w) + bi.w;
    }
    *reinterpret_cast<float4*>(xr + col) = v;
    ss[block & 1] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ss[0] += __shfl_xor_sync(0xffffffffu, ss[0], o);
    ss[1] += __shfl_xor_sync(0xffffffffu, ss[1], o);
  }
  if ((et & 31) == 0) {
    red[et >> 5] = ss[0];
    red[4 + (et >> 5)] = ss[1];
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += red[i];
  const float rstd = rsqrtf(total / static_cast<float>(d) + eps);
  for (int col = et * 4; col < d; col += 128 * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + col);  // this thread's own stores
    const float4 ww = *reinterpret_cast<const float4*>(w + col);
    uint2 o;
    o.x = pack_bf16x2(v.x * rstd * ww.x, v.y * rstd * ww.y);
    o.y = pack_bf16x2(v.z * rstd * ww.z, v.w * rstd * ww.w);
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(b) * d + col) = o;
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");  // `red` is reused by the next norm phase
}

// Grid barrier number `index` (1-based), executed by the 128 epilogue threads of every CTA.
__device__ __forceinline__ void tail_grid_barrier(const TailCta& c, unsigned* counter, unsigned index, int* error_flag,
                                                  int et) {
  asm volatile("bar.sync 1, 128;" ::: "memory");  // every epilogue thread's global stores are issued
  if (et == 0) {
    asm volatile("fence.proxy.async;" ::: "memory");  // those stores are read by other CTAs' TMA loads
    __threadfence();
    atomicAdd(counter, 1u);
    const unsigned target = index * gridDim.x;
    const uint64_t t0 = globaltimer_ns();
    unsigned seen;
    while (true) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
      if (seen >= target || *c.abort_flag) break;
      if (globaltimer_ns() - t0 > tail::kBarrierBudgetNs) {
        *c.abort_flag = 1;
        if (error_flag != nullptr) atomicExch(error_flag, 9);
        break;
      }
      __nanosleep(20);
    }
    *c.passed = index;
    __threadfence_block();
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

__global__ void __launch_bounds__(tail::THREADS, 1)
decode_layer_tail_kernel(const __grid_constant__ CUtensorMap tm_wout, const __grid_constant__ CUtensorMap tm_wug,
                         const __grid_constant__ CUtensorMap tm_wdown, const __grid_constant__ CUtensorMap tm_win,
                         const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ CUtensorMap tm_n,
                         const __grid_constant__ CUtensorMap tm_act, const LayerTailParams p) {
  using namespace tail;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ float red[8];
  TailCta c;
  c.sW = smem;
  c.sX = smem + STAGES * W_BYTES;
  c.sG = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + EXCHANGE_BYTES);
  c.full = bars;
  c.empty = bars + STAGES;
  c.tfull = bars + 2 * STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  c.abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  c.passed = reinterpret_cast<volatile unsigned*>(tmem_slot + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&c.full[s], 1);
      mbar_init(&c.empty[s], 1);
    }
    mbar_init(c.tfull, 1);
    *c.abort_flag = 0;
    *c.passed = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tm_wout);
    tma_prefetch_desc(&tm_wug);
    tma_prefetch_desc(&tm_wdown);
    tma_prefetch_desc(&tm_win);
    tma_prefetch_desc(&tm_y);
    tma_prefetch_desc(&tm_n);
    tma_prefetch_desc(&tm_act);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  c.tmem = *tmem_slot;

  const int me = blockIdx.x;
  const TailItem w_out = tail_item<1>(me, p.d, p.d, p.splits_out, p.kb_per_split_out);
  const TailItem w_ug = tail_item<2>(me, p.ffn, p.d, 1, (p.d + BK - 1) / BK);
  const TailItem w_down = tail_item<1>(me, p.d, p.ffn, p.splits_down, p.kb_per_split_down);
  TailItem w_in = tail_item<0>(me, 5 * p.d, p.d, 1, (p.d + BK - 1) / BK);
  if (!p.has_in) w_in.valid = false;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t pit = 0;
      tail_produce<1>(c, &tm_wout, &tm_y, w_out, p.d, 0u, pit);
      tail_produce<2>(c, &tm_wug, &tm_n, w_ug, p.ffn, 2u, pit);
      tail_produce<1>(c, &tm_wdown, &tm_act, w_down, p.d, 3u, pit);
      tail_produce<0>(c, &tm_win, &tm_n, w_in, 5 * p.d, 5u, pit);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t cit = 0;
      tail_mma(c, w_out, cit);
      tail_mma(c, w_ug, cit);
      tail_mma(c, w_down, cit);
      tail_mma(c, w_in, cit);
    }
  } else {
    const int et = threadIdx.x - 64;
    int stamp_index = 0;
    auto stamp = [&]() {
      if (p.trace != nullptr && et == 0) p.trace[static_cast<size_t>(me) * 16 + stamp_index] = static_cast<long long>(globaltimer_ns());
      ++stamp_index;
    };
    stamp();                                                                                   // 0 start
    uint32_t worked = 0;  // GEMM phases in which this CTA had an item: the parity of its accumulator barrier
    tail_epilogue<1>(c, w_out, p.d, p.batch, p.part_out, 0, worked & 1, warp, lane);
    worked += w_out.valid ? 1u : 0u;
    stamp();                                                                                   // 1 out_proj stored
    tail_grid_barrier(c, p.barrier, 1u, p.error_flag, et);
    stamp();                                                                                   // 2 barrier 1
    if (me < p.batch)
      tail_norm_row(p.x, p.part_out, p.splits_out, p.batch, me, p.d, nullptr, nullptr, p.w_norm2, p.eps, p.n, red, et);
    stamp();                                                                                   // 3 norm 1
    tail_grid_barrier(c, p.barrier, 2u, p.error_flag, et);
    stamp();                                                                                   // 4 barrier 2
    tail_epilogue<2>(c, w_ug, p.ffn, p.batch, p.act, p.ffn, worked & 1, warp, lane);
    worked += w_ug.valid ? 1u : 0u;
    stamp();                                                                                   // 5 up/gate stored
    tail_grid_barrier(c, p.barrier, 3u, p.error_flag, et);
    stamp();                                                                                   // 6 barrier 3
    tail_epilogue<1>(c, w_down, p.d, p.batch, p.part_down, 0, worked & 1, warp, lane);
    worked += w_down.valid ? 1u : 0u;
    stamp();                                                                                   // 7 down stored
    tail_grid_barrier(c, p.barrier, 4u, p.error_flag, et);
    stamp();                                                                                   // 8 barrier 4
    if (me < p.batch)
      tail_norm_row(p.x, p.part_down, p.splits_down, p.batch, me, p.d, p.next_scale, p.next_bias, p.w_norm_next, p.eps,
                    p.n, red, et);
    stamp();                                                                                   // 9 norm 2
    if (p.has_in) {
      tail_grid_barrier(c, p.barrier, 5u, p.error_flag, et);
      stamp();                                                                                 // 10 barrier 5
      tail_epilogue<0>(c, w_in, 5 * p.d, p.batch, p.qkvgu, 5 * p.d, worked & 1, warp, lane);
      stamp();                                                                                 // 11 in_proj stored
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (*c.abort_flag != 0 && p.error_flag != nullptr) atomicCAS(p.error_flag, 0, 8);
    // the last CTA to leave zeroes both counters for the next launch (stream order keeps that launch behind this one)
    __threadfence();
    if (atomicAdd(p.barrier + 1, 1u) + 1u == gridDim.x) {
      p.barrier[0] = 0u;
      p.barrier[1] = 0u;
      __threadfence();
    }
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(c.tmem, TMEM_COLS);
  }
}

}  // namespace ws

using namespace ws;

// The part of a decode layer after its attention, as one persistent cooperative launch (see the head of this file).
// w_out [d, d], w_ug [2 ffn, d] (up rows, then gate rows), w_down [d, ffn], w_in_next [5 d, d] (NULL after the last
// layer): row-major BF16.  y [batch, d] BF16 is the attention output.  x, part_out, part_down, n, act, qkvgu as in
// LayerTailParams; part_* are sized with ws_decode_gemm_splits.  barrier: two zeroed 32-bit words, shared by all
// launches of a stream.  trace (optional): [SMs, 16] int64, receives %globaltimer at every CTA's phase boundaries
// (start, out stored, barrier 1, norm 1, barrier 2, up/gate stored, barrier 3, down stored, barrier 4, norm 2,
// barrier 5, in_proj stored).  Returns -30 when the device has fewer SMs than the largest phase has work items.
extern "C" int ws_decode_layer_tail(const void* w_out, const void* w_ug, const void* w_down, const void* w_in_next,
                                    const void* y, float* x, float* part_out, float* part_down, void* n, void* act,
                                    void* qkvgu, const float* w_norm2, const float* next_scale, const float* next_bias,
                                    const float* w_norm_next, float eps, int batch, int d, int ffn, unsigned* barrier,
                                    int* error_flag, long long* trace, cudaStream_t stream) {
  using namespace tail;
  if (batch <= 0 || batch > BPAD || d % 128 != 0 || ffn % 64 != 0 || d % 8 != 0 || ffn % 8 != 0) return -1;
  static int sms = 0;
  static bool configured = false;
  if (!configured) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -20;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -20;
    if (cudaFuncSetAttribute(decode_layer_tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return -20;
    configured = true;
  }
  LayerTailParams p;
  p.batch = batch; p.d = d; p.ffn = ffn; p.eps = eps; p.has_in = w_in_next != nullptr ? 1 : 0;
  p.splits_out = ws_decode_gemm_splits(d, d);
  p.kb_per_split_out = ((d + BK - 1) / BK + p.splits_out - 1) / p.splits_out;
  p.splits_down = ws_decode_gemm_splits(d, ffn);
  p.kb_per_split_down = ((ffn + BK - 1) / BK + p.splits_down - 1) / p.splits_down;
  const int slabs_d = (d + TM - 1) / TM;
  int items = slabs_d * p.splits_out;
  if (slabs_d * p.splits_down > items) items = slabs_d * p.splits_down;
  if (ffn / 64 > items) items = ffn / 64;
  if (p.has_in && (5 * d + TM - 1) / TM > items) items = (5 * d + TM - 1) / TM;
  if (batch > items) items = batch;
  if (items > sms) return -30;
  p.x = x; p.part_out = part_out; p.part_down = part_down;
  p.n = static_cast<__nv_bfloat16*>(n); p.act = static_cast<__nv_bfloat16*>(act);
  p.qkvgu = static_cast<__nv_bfloat16*>(qkvgu);
  p.w_norm2 = w_norm2; p.next_scale = next_scale; p.next_bias = next_bias; p.w_norm_next = w_norm_next;
  p.barrier = barrier; p.error_flag = error_flag; p.trace = trace;
  CUtensorMap t_wout, t_wug, t_wdown, t_win, t_y, t_n, t_act;
  int rc;
  if ((rc = make_map_bf16(&t_wout, w_out, d, d, d, BK, TM))) return rc;
  if ((rc = make_map_bf16(&t_wug, w_ug, d, 2 * (uint64_t)ffn, d, BK, 64))) return rc;
  if ((rc = make_map_bf16(&t_wdown, w_down, ffn, d, ffn, BK, TM))) return rc;
  if ((rc = make_map_bf16(&t_win, p.has_in ? w_in_next : w_out, d, p.has_in ? 5 * (uint64_t)d : (uint64_t)d, d, BK, TM))) return rc;
  if ((rc = make_map_bf16(&t_y, y, d, batch, d, BK, BPAD))) return rc;
  if ((rc = make_map_bf16(&t_n, n, d, batch, d, BK, BPAD))) return rc;
  if ((rc = make_map_bf16(&t_act, act, ffn, batch, ffn, BK, BPAD))) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sms);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t err = cudaLaunchKernelEx(&cfg, decode_layer_tail_kernel, t_wout, t_wug, t_wdown, t_win, t_y, t_n, t_act, p);
  ws_count_launch();
  return err == cudaSuccess ? 0 : -21;
}
