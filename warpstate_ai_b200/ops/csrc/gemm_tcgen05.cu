// Persistent warp-specialised BF16 GEMM for sm_100a.
//
//   warp 0      : TMA producer (one lane) - streams 128x64 A tiles and 256x64 B tiles into a
//                 4-stage shared-memory ring (128-byte swizzle), one mbarrier per stage.
//   warp 1      : TMEM owner + MMA issuer (one lane) - tcgen05.mma 128x256x16, FP32 accumulators
//                 in TMEM, two accumulator buffers (2 x 256 columns) so that the epilogue of
//                 tile i overlaps the main loop of tile i+1.
//   warps 2..9  : epilogue (two groups of four, each group drains half of the tile columns) -
//                 tcgen05.ld of the warp's 32-lane quarter, fused epilogue math,
//                 vectorised global stores.
//
// Operand layouts: each operand is either K-major (contraction contiguous, the nn.Linear
// layout) or MN-major (output dimension contiguous); MN-major lets dX = dY*W and
// dW = dY^T*X read the tensors exactly as the forward pass left them, with no transposes.
// One CTA per SM; tiles are visited in a grouped order so that concurrently running CTAs
// share A row-panels and B column-panels in L2.
//
// Role of this file in the model: every projection of a WarpState core (in_proj, out_proj,
// up_gate, down; reference call sites warpstate/model.py:109,177,59,60) and their dX / dW
// products, plus the epilogues the reference runs as separate kernels (SwiGLU forward
// ops/matmul_epilogue.py:30-83 and backward ops/activation_execution.py:36-55, residual adds,
// the BF16->FP32 gradient accumulation of autograd's AccumulateGrad).
#include "ws_ptx.cuh"
#include "ws_api.h"
#include "ws_tma_host.h"
#include "gemm_epilogue.cuh"
#include "ws_launch.h"

#include <atomic>
#include <mutex>
#include <unordered_map>
#include <cstdio>
#include <cstring>
#include <cstdlib>

namespace ws {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int GEMM_THREADS = 320;  // producer warp, MMA warp, 2 groups of 4 epilogue warps
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;


__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& mb, int& nb) {
  const int group_size = GROUP_M * num_n;
  const int group = tile / group_size;
  const int first_m = group * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int r = tile - group * group_size;
  mb = first_m + (r % gsz);
  nb = r / gsz;
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  constexpr bool kSwiglu = (EPI == WS_EPI_SWIGLU);
  const int n_tile = kSwiglu ? 128 : BN;  // logical output columns per tile
  const int num_m = (p.m + BM - 1) / BM;
  const int num_n = (p.n + n_tile - 1) / n_tile;
  const int tiles = num_m * num_n;
  const int num_k = (p.k + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, num_m, num_n, mb, nb);
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          if (!A_MN) {
            tma_load_2d(a_dst, &tma_a, &full[s], kb * BK, mb * BM);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d(a_dst + i * (BK * 128), &tma_a, &full[s], mb * BM + i * 64, kb * BK);
          }
          if (!B_MN) {
            const int r0 = kSwiglu ? nb * 128 : nb * BN;
            const int r1 = kSwiglu ? p.h + nb * 128 : nb * BN + 128;
            tma_load_2d(b_dst, &tma_b, &full[s], kb * BK, r0);
            tma_load_2d(b_dst + 128 * 128, &tma_b, &full[s], kb * BK, r1);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(b_dst + i * (BK * 128), &tma_b, &full[s], nb * BN + i * 64, kb * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int it = 0;
      int tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++tcount) {
        const int buf = tcount & 1;
        const uint32_t tph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty[buf], tph ^ 1, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_base = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 8-row groups are 1024 B apart (SBO); a K step of 16 elements is 32 B
            // inside the 128-byte swizzle row.  MN-major: 64-element column groups are
            // BK*128 B apart (LBO), 8-row K groups 1024 B apart (SBO); a K step is 16 rows.
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_base + k * UMMA_K * 128, BK * 128, 1024)
                                     : make_smem_desc_sw128(a_base + k * UMMA_K * 2, 0, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_base + k * UMMA_K * 128, BK * 128, 1024)
                                     : make_smem_desc_sw128(b_base + k * UMMA_K * 2, 0, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&tfull[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;
    const int egroup = (warp - 2) >> 2;  // which half of the tile columns this warp drains
    int tcount = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++tcount) {
      int mb, nb;
      tile_coords(tile, num_m, num_n, mb, nb);
      const int buf = tcount & 1;
      const uint32_t tph = (tcount >> 1) & 1;
      if (!mbar_wait(&tfull[buf], tph, abort_flag)) break;
      tc_fence_after_sync();
      const int row = mb * BM + quarter * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
      const float rs = (p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.0f;

      gemm_epilogue<EPI>(p, taddr, row, row_ok, rs, nb, egroup);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && p.error_flag != nullptr) atomicExch(p.error_flag, 1);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// =============================================================================== host side
static std::atomic<long long> g_launches{0};
static std::atomic<int> g_sm_limit{0};

template <bool A_MN, bool B_MN, int EPI>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                  cudaStream_t stream) {
  static bool configured = false;  // per-instantiation; the attribute is per function
  auto kern = gemm_kernel<A_MN, B_MN, EPI>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return -20;
    configured = true;
  }
  launch_dependent(kern, dim3(grid), dim3(GEMM_THREADS), SMEM_BYTES, stream, ta, tb, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

static int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

}  // namespace ws

extern "C" long long ws_launch_count(void) { return ws::g_launches.load(); }
extern "C" void ws_count_launch(void) { ws::g_launches.fetch_add(1, std::memory_order_relaxed); }
extern "C" void ws_gemm_set_sm_limit(int sms) { ws::g_sm_limit.store(sms); }

// CTA-pair kernel (gemm2_tcgen05.cu): the default for problems with at least 256 rows;
// WS_GEMM_PAIR=0 in the environment keeps every GEMM on the single-CTA kernel.
extern "C" int ws_gemm_pair(const WsGemm* g, int sms, cudaStream_t stream);
static std::atomic<int> g_pair_override{-1};
extern "C" void ws_gemm_set_pair_mode(int mode) { g_pair_override.store(mode); }
static bool pair_mode() {
  static const bool on = [] {
    const char* e = getenv("WS_GEMM_PAIR");
    return e == nullptr || atoi(e) != 0;
  }();
  const int forced = g_pair_override.load(std::memory_order_relaxed);
  return forced < 0 ? on : forced != 0;
}

// Argument checks shared by every entry point (0 = acceptable).
static int validate_gemm(const WsGemm* g) {
  using namespace ws;
  if (g->m <= 0 || g->n <= 0 || g->k <= 0) return -1;
  const bool swiglu = g->epilogue == WS_EPI_SWIGLU;
  // Vector-store alignment of the epilogues (8 BF16 or 4 FP32 per store).
  const bool f32_out = g->epilogue == WS_EPI_RESID_F32 || g->epilogue == WS_EPI_ACC_F32 ||
                       g->epilogue == WS_EPI_F32;
  const int vec = f32_out ? 4 : 8;
  if (g->epilogue == WS_EPI_CE_FWD) {
    if (g->aux == nullptr || g->out2 == nullptr || g->ldo < 2 * ((g->n + BN - 1) / BN)) return -7;
  } else if (g->n % vec != 0 || g->ldo % vec != 0) {
    return -2;
  }
  if (g->epilogue == WS_EPI_CE_BWD && (g->aux == nullptr || g->row_vec == nullptr || g->row_scale == nullptr)) return -8;
  if ((g->epilogue == WS_EPI_RESID_F32 || g->epilogue == WS_EPI_RESID_BF16) &&
      (g->aux == nullptr || g->ldaux % vec != 0)) return -3;
  if (swiglu && (g->out2 == nullptr || g->ldo2 % 8 != 0)) return -4;
  if (g->epilogue == WS_EPI_SWIGLU_BWD && (g->aux == nullptr || g->ldaux % 8 != 0)) return -5;

  return 0;
}

static int usable_sms() {
  int sms = ws::sm_count();
  const int lim = ws::g_sm_limit.load();
  if (lim > 0 && lim < sms) sms = lim;
  return sms;
}

extern "C" int ws_gemm_pair_group(const WsGemm* items, int count, int sms, cudaStream_t stream);

// Several problems of one kind in one persistent launch when the CTA-pair kernel can take them
// (all with >= 256 rows, at most 4); otherwise one launch each, in order.
extern "C" int ws_gemm_group(const WsGemm* items, int count, cudaStream_t stream) {
  if (count <= 0) return 0;
  bool groupable = pair_mode() && count <= 4 && usable_sms() >= 2;
  for (int i = 0; i < count; ++i) {
    const int rc = validate_gemm(&items[i]);
    if (rc) return rc;
    groupable = groupable && items[i].m >= 256 && items[i].a_mn == items[0].a_mn &&
                items[i].b_mn == items[0].b_mn && items[i].epilogue == items[0].epilogue;
  }
  if (groupable) return ws_gemm_pair_group(items, count, usable_sms(), stream);
  for (int i = 0; i < count; ++i) {
    const int rc = ws_gemm(&items[i], stream);
    if (rc) return rc;
  }
  return 0;
}

extern "C" int ws_gemm(const WsGemm* g, cudaStream_t stream) {
  {
    const int vrc = validate_gemm(g);
    if (vrc) return vrc;
  }
  using namespace ws;
  const int sms = usable_sms();
  if (pair_mode() && g->m >= 256 && sms >= 2) return ws_gemm_pair(g, sms, stream);
  const bool swiglu = g->epilogue == WS_EPI_SWIGLU;
  const int b_rows = swiglu ? 2 * g->n : g->n;  // output features held by B
  CUtensorMap ta, tb;
  int rc;
  if (!g->a_mn)
    rc = make_map_bf16(&ta, g->a, g->k, g->m, g->lda, BK, BM);
  else
    rc = make_map_bf16(&ta, g->a, g->m, g->k, g->lda, 64, BK);
  if (rc) return rc;
  if (!g->b_mn)
    rc = make_map_bf16(&tb, g->b, g->k, b_rows, g->ldb, BK, 128);
  else
    rc = make_map_bf16(&tb, g->b, b_rows, g->k, g->ldb, 64, BK);
  if (rc) return rc;

  GemmParams p;
  p.m = g->m; p.n = g->n; p.k = g->k;
  p.h = g->n;
  p.epi_n = swiglu ? 128 : BN;
  p.out = g->out; p.ldo = g->ldo;
  p.out2 = g->out2; p.ldo2 = g->ldo2;
  p.aux = g->aux; p.ldaux = g->ldaux;
  p.row_scale = g->row_scale;
  p.row_vec = g->row_vec;
  p.alpha = g->alpha; p.beta = g->beta;
  p.error_flag = g->error_flag;
  p.debug = 0;

  const int n_tile = swiglu ? 128 : BN;
  const int tiles = ((g->m + BM - 1) / BM) * ((g->n + n_tile - 1) / n_tile);
  const int grid = tiles < sms ? tiles : sms;

  const int key = (g->a_mn ? 1 : 0) | (g->b_mn ? 2 : 0) | (g->epilogue << 2);
  switch (key) {
    case (0 | (WS_EPI_BF16 << 2)): return launch<false, false, WS_EPI_BF16>(ta, tb, p, grid, stream);
    case (2 | (WS_EPI_BF16 << 2)): return launch<false, true, WS_EPI_BF16>(ta, tb, p, grid, stream);
    case (0 | (WS_EPI_RESID_F32 << 2)): return launch<false, false, WS_EPI_RESID_F32>(ta, tb, p, grid, stream);
    case (0 | (WS_EPI_RESID_BF16 << 2)): return launch<false, false, WS_EPI_RESID_BF16>(ta, tb, p, grid, stream);
    case (0 | (WS_EPI_SWIGLU << 2)): return launch<false, false, WS_EPI_SWIGLU>(ta, tb, p, grid, stream);
    case (0 | (WS_EPI_F32 << 2)): return launch<false, false, WS_EPI_F32>(ta, tb, p, grid, stream);
    case (3 | (WS_EPI_ACC_F32 << 2)): return launch<true, true, WS_EPI_ACC_F32>(ta, tb, p, grid, stream);
    case (3 | (WS_EPI_BF16 << 2)): return launch<true, true, WS_EPI_BF16>(ta, tb, p, grid, stream);
    case (2 | (WS_EPI_SWIGLU_BWD << 2)): return launch<false, true, WS_EPI_SWIGLU_BWD>(ta, tb, p, grid, stream);
    case (0 | (WS_EPI_CE_FWD << 2)): return launch<false, false, WS_EPI_CE_FWD>(ta, tb, p, grid, stream);
    case (0 | (WS_EPI_CE_BWD << 2)): return launch<false, false, WS_EPI_CE_BWD>(ta, tb, p, grid, stream);
    default: return -6;
  }
}
