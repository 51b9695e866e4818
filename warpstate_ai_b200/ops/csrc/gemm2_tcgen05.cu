// CTA-pair BF16 GEMM for sm_100a: two CTAs of a cluster compute one 256x256 tile with
// tcgen05.mma.cta_group::2.
//
// Why pairs: with one CTA per 128x256 tile every k-block moves 48 KiB into shared memory by TMA
// and 48 KiB out of it into the tensor core, which exceeds what one SM's shared memory can
// stream at the tensor core's rate (the single-CTA kernel saturates near 70 % tensor-pipe
// activity).  In a pair each CTA stages only its own 128 rows of A and its own 128 of the 256
// B rows (32 KiB per k-block) and the hardware feeds both tensor cores from both shared
// memories, so the same tile costs two thirds of the shared-memory traffic and the ring holds
// six stages instead of four.
//
// Roles per CTA (320 threads): warp 0 = TMA producer (its own halves; plain per-CTA loads whose
// completion is counted on the LEADER CTA's `full` barrier, on which the leader alone announces
// the bytes of both CTAs), warp 1 = TMEM owner and, in the leader CTA only, MMA issuer;
// warps 2..9 = epilogue of the CTA's own 128 rows.  `empty` / `tmem_full` barriers exist in
// both CTAs and are signalled together by one tcgen05.commit with a CTA mask; `tmem_empty`
// lives in the leader and counts the epilogue warps of both CTAs.
//
// Cross-CTA signals avoid release semantics: a `release.cluster` arrival first drains the
// issuing thread's outstanding global stores, and having the peer's producer announce its own
// bytes that way halved the throughput of the whole kernel (0.69 vs 1.5 PFLOP/s on
// 16384x10240x2048).  Every wait is bounded; both CTAs always reach the closing cluster barrier.
#include "ws_ptx.cuh"
#include "ws_api.h"
#include "ws_tma_host.h"
#include "gemm_epilogue.cuh"
#include "ws_launch.h"

#include <cuda_bf16.h>
#include <cstdlib>
#include <cstring>

namespace ws {

extern "C" void ws_count_launch(void);

namespace pair {
constexpr int BM = 128;        // rows per CTA (256 per pair)
constexpr int BN = 256;        // accumulator columns (128 B rows staged per CTA)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;          // staged-epilogue instantiations use one fewer (see pair_stages)
constexpr int ESTAGE_BYTES = 8 * 8192;  // staged epilogue: 8 warps x 2 buffers x 2 tiles of 32 x 32 BF16
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_BYTES = (BN / 2) * BK * 2;  // 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;
}  // namespace pair

__device__ __forceinline__ void pair_tile_coords(int tile, int num_m, int num_n, int& mb, int& nb) {
  const int group_size = pair::GROUP_M * num_n;
  const int group = tile / group_size;
  const int first_m = group * pair::GROUP_M;
  const int gsz = min(num_m - first_m, pair::GROUP_M);
  const int r = tile - group * group_size;
  mb = first_m + (r % gsz);
  nb = r / gsz;
}

// The weight-gather variant (GATHER): B is a weight whose FP32 master rows are sharded over the GPUs
// of a node.  Four extra warps per CTA pull the shards (plain peer loads over NVLink for the rows other
// ranks own), cast them to BF16 into a local [n, k] buffer and count finished 8-row chunks per
// 256-row block in a flag word; the TMA producer takes a B tile only once its block is complete.
// Tiles are walked N-block by N-block, so block j is needed about j * 12 us into the kernel while
// the whole gather of in_proj takes ~0.1 ms of link time: all-gather, cast and GEMM are one launch and
// after the first block the transfer hides under the tensor-core work.  Nothing is multicast.
struct GatherJob {
  const float* shard[8];   // rank r owns rows [r * rows_per_shard, (r + 1) * rows_per_shard) of W
  int world;
  int rows_per_shard;      // a multiple of 8 (so a chunk never straddles two shards)
  int n, k;                // k % 8 == 0
  __nv_bfloat16* dst;      // local BF16 [n, k]
  unsigned* flags;         // one word per 128-row block of W, zero at launch
  unsigned* counter;       // next unclaimed chunk, zero at launch
  unsigned target;         // chunks per complete block
  int interleave_h;        // SwiGLU: h (n = 2h rows: up, then gate; h % 128 == 0); otherwise 0
  unsigned long long wait_ns;
};
constexpr int GATHER_ROWS = 2;   // rows per chunk: small, so that the first block is spread over 128 CTAs
constexpr int GATHER_THREADS = 128;
constexpr int GATHER_BLOCK = 128;  // weight rows per ready flag (the rows one CTA of a pair stages)

// Up to MAX_GROUP independent problems of the same kind share one persistent launch: their
// tiles form one list, so the last partial wave is paid once per group instead of once per
// problem (the four weight-gradient GEMMs of a layer: 17 waves of 74 pairs separately, 15 grouped).
constexpr int MAX_GROUP = 4;
struct alignas(64) PairGroup {
  CUtensorMap a[MAX_GROUP];
  CUtensorMap b[MAX_GROUP];
  GemmParams p[MAX_GROUP];
  CUtensorMap epi[4];  // staged epilogue of problem 0, 32 x 32 boxes.  SwiGLU backward: aux up, aux gate,
                       // out up, out gate; SwiGLU forward: packed up, packed gate, activation
  int tile_start[MAX_GROUP + 1];
  int count;
};

// The SwiGLU-backward epilogue reads and writes 4 bytes of global memory per accumulator element.
// Done with one thread per row, that is 32 L1 wavefronts per warp instruction and the epilogue
// takes twice as long as the main loop; staged through shared memory with TMA loads and stores,
// global memory never goes through L1 and each thread touches only swizzled shared memory.
template <int EPI>
constexpr bool staged_epilogue() {
  return EPI == WS_EPI_SWIGLU_BWD || EPI == WS_EPI_SWIGLU || EPI == WS_EPI_RESID_F32;
}
template <int EPI>
constexpr int pair_stages() {
  return staged_epilogue<EPI>() ? pair::STAGES - 1 : pair::STAGES;
}
template <int EPI>
constexpr int pair_smem() {
  return pair_stages<EPI>() * pair::STAGE_BYTES + (staged_epilogue<EPI>() ? pair::ESTAGE_BYTES : 0) + 1024 + 512;
}

// 16-byte chunk j of row r in a 32-row x 64-byte tile written by TMA with the 64-byte swizzle
__device__ __forceinline__ uint8_t* tile_chunk64(uint8_t* tile, int r, int j) {
  return tile + r * 64 + ((j ^ ((r >> 1) & 3)) << 4);
}
// the same for 128-byte rows and the 128-byte swizzle (32 x 32 FP32 tiles)
__device__ __forceinline__ uint8_t* tile_chunk128(uint8_t* tile, int r, int j) {
  return tile + r * 128 + ((j ^ (r & 7)) << 4);
}

struct PairTile {
  int prob, mb, nb, num_k;
};
__device__ __forceinline__ PairTile resolve_tile(const PairGroup& g, int tile, int n_tile, bool n_major = false) {
  PairTile t;
  t.prob = 0;
  while (t.prob + 1 < g.count && tile >= g.tile_start[t.prob + 1]) ++t.prob;
  const GemmParams& p = g.p[t.prob];
  const int num_m = (p.m + 2 * pair::BM - 1) / (2 * pair::BM);
  const int num_n = (p.n + n_tile - 1) / n_tile;
  if (n_major) {  // every M tile of one N block before the next block (weight-gather variant)
    const int local = tile - g.tile_start[t.prob];
    t.mb = local % num_m;
    t.nb = local / num_m;
  } else {
    pair_tile_coords(tile - g.tile_start[t.prob], num_m, num_n, t.mb, t.nb);
  }
  t.num_k = (p.k + pair::BK - 1) / pair::BK;
  return t;
}

template <int EPI>
constexpr int pair_threads() {
  return 64 + 128 * epilogue_groups<EPI>();  // TMA warp, MMA warp, GROUPS x 4 epilogue warps
}

template <bool A_MN, bool B_MN, int EPI, bool GATHER = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair_threads<EPI>() + (GATHER ? GATHER_THREADS : 0), 1)
gemm2_kernel(const __grid_constant__ PairGroup g, const __grid_constant__ GatherJob gj) {
  using namespace pair;
  static_assert(!GATHER || (!A_MN && !B_MN && (EPI == WS_EPI_BF16 || EPI == WS_EPI_SWIGLU)),
                "the gather variant is the NT forward GEMM (plain or SwiGLU)");
  constexpr int GROUPS = epilogue_groups<EPI>();
  constexpr int STAGES = pair_stages<EPI>();
  constexpr bool STAGED = staged_epilogue<EPI>();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint8_t* eStage = smem + STAGES * STAGE_BYTES;  // staged epilogue buffers (STAGED only)
  uint64_t* bars = reinterpret_cast<uint64_t*>(eStage + (STAGED ? ESTAGE_BYTES : 0));
  uint64_t* full = bars;                    // used in the leader CTA
  uint64_t* empty = bars + STAGES;          // per CTA
  uint64_t* tfull = bars + 2 * STAGES;      // per CTA
  uint64_t* tempty = bars + 2 * STAGES + 2; // used in the leader CTA
  uint64_t* ebar = bars + 2 * STAGES + 4;   // 16: per epilogue warp, per buffer (STAGED only)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);   // the leader's expect-tx arrival; both CTAs' loads complete on it
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 8 * GROUPS);  // epilogue warps of both CTAs
    }
    if (STAGED) {
      for (int i = 0; i < 16; ++i) mbar_init(&ebar[i], 1);
      for (int i = 0; i < (EPI == WS_EPI_SWIGLU ? 3 : EPI == WS_EPI_RESID_F32 ? 2 : 4); ++i) tma_prefetch_desc(&g.epi[i]);
    }
    *abort_flag = 0;
    mbar_fence_init();
    for (int i = 0; i < g.count; ++i) {
      tma_prefetch_desc(&g.a[i]);
      tma_prefetch_desc(&g.b[i]);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // peer barriers are initialised before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // set-up is done: let the next kernel of the stream be scheduled, then wait for the previous one's results
  pdl_launch_dependents();
  pdl_wait();

  constexpr bool kSwiglu = (EPI == WS_EPI_SWIGLU);
  const int n_tile = kSwiglu ? 128 : BN;
  const int tiles = g.tile_start[g.count];
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      [[maybe_unused]] int ready_nb = -1;
      for (int tile = pair_id; tile < tiles && ok; tile += num_pairs) {
        const PairTile t = resolve_tile(g, tile, n_tile, GATHER);
        const GemmParams& p = g.p[t.prob];
        const CUtensorMap* tma_a = &g.a[t.prob];
        const CUtensorMap* tma_b = &g.b[t.prob];
        const int nb = t.nb;
        const int m0 = t.mb * 2 * BM + rank * BM;  // this CTA's rows
        if constexpr (GATHER) {
          if (nb != ready_nb) {  // the 256 weight rows of this N block must have landed in the local buffer
            // this CTA's 128 weight rows: plain [nb*256 + rank*128, +128); SwiGLU up rows nb*128.. (rank 0)
            // or gate rows h + nb*128.. (rank 1).  One flag word per 128-row block of W.
            const int block = kSwiglu ? (rank ? gj.interleave_h / GATHER_BLOCK + nb : nb) : 2 * nb + static_cast<int>(rank);
            const unsigned* flag = gj.flags + block;
            const int block_rows = min(GATHER_BLOCK, gj.n - block * GATHER_BLOCK);
            const unsigned want = block_rows <= 0 ? 0u : static_cast<unsigned>((block_rows + GATHER_ROWS - 1) / GATHER_ROWS);
            unsigned seen = want;  // a block past the last weight row has nothing to wait for (and no flag word)
            if (want > 0) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
            if (seen < want) {
              const uint64_t t0 = globaltimer_ns();
              uint32_t spins = 0;
              while (true) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
                if (seen >= want) break;
                if ((++spins & 63u) == 0 && (*abort_flag || globaltimer_ns() - t0 > gj.wait_ns)) {
                  *abort_flag = 1;
                  ok = false;
                  break;
                }
              }
              if (!ok) break;
            }
            asm volatile("fence.proxy.async.global;" ::: "memory");
            ready_nb = nb;
          }
        }
        for (int kb = 0; kb < t.num_k; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = mapa_shared(smem_u32(&full[s]), 0);
          const uint32_t bar = full_leader;
          // The leader alone announces the bytes of both CTAs (a remote expect-tx arrival with
          // release semantics from the peer measured 2x slower for the whole kernel).
          if (leader) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_BYTES;
          uint8_t* b_dst = sB + s * B_BYTES;
          if (!A_MN) {
            tma_load_2d_pair(a_dst, tma_a, bar, kb * BK, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d_pair(a_dst + i * (BK * 128), tma_a, bar, m0 + i * 64, kb * BK);
          }
          if (!B_MN) {
            const int r0 = kSwiglu ? (rank ? p.h + nb * 128 : nb * 128) : nb * BN + rank * 128;
            tma_load_2d_pair(b_dst, tma_b, bar, kb * BK, r0);
          } else {
#pragma unroll
            for (int i = 0; i < 2; ++i)
              tma_load_2d_pair(b_dst + i * (BK * 128), tma_b, bar, nb * BN + rank * 128 + i * 64, kb * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      int it = 0;
      int tcount = 0;
      bool ok = true;
      for (int tile = pair_id; tile < tiles && ok; tile += num_pairs, ++tcount) {
        const int buf = tcount & 1;
        const uint32_t tph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty[buf], tph ^ 1, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        const int num_k = resolve_tile(g, tile, n_tile, GATHER).num_k;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(sA + s * A_BYTES);
          const uint32_t b_base = smem_u32(sB + s * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_base + k * UMMA_K * 128, BK * 128, 1024)
                                     : make_smem_desc_sw128(a_base + k * UMMA_K * 2, 0, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_base + k * UMMA_K * 128, BK * 128, 1024)
                                     : make_smem_desc_sw128(b_base + k * UMMA_K * 2, 0, 1024);
            umma_bf16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // free the stage in both CTAs once these MMAs have consumed it
          umma_commit_pair_mask(smem_u32(&empty[s]), 3);
        }
        if (ok) {
          umma_commit_pair_mask(smem_u32(&tfull[buf]), 3);
        }
      }
    }
  } else if (warp < 2 + 4 * GROUPS) {
    // ------------------------------------------------------------------ epilogue warps (both CTAs)
    const int quarter = warp & 3;
    const int egroup = (warp - 2) >> 2;
    int tcount = 0;
    if constexpr (EPI == WS_EPI_SWIGLU) {
      // SwiGLU forward through shared memory: per warp 32 rows, per step 32 features; the three
      // output tiles (up, gate, activation) are written to swizzled shared memory and leave by TMA.
      uint8_t* ebuf = eStage + (warp - 2) * 8192;  // 3 tiles of 2 KiB used
      constexpr int STEPS = (128 / GROUPS) / 32;
      const GemmParams& p = g.p[0];
      for (int tile = pair_id; tile < tiles; tile += num_pairs, ++tcount) {
        const PairTile t = resolve_tile(g, tile, n_tile, GATHER);
        const int buf_t = tcount & 1;
        const uint32_t tph = (tcount >> 1) & 1;
        if (!mbar_wait(&tfull[buf_t], tph, abort_flag)) break;
        tc_fence_after_sync();
        const int y = t.mb * 2 * BM + rank * BM + quarter * 32;
        const int row = y + lane;
        const float rs = (p.row_scale != nullptr && row < p.m) ? p.row_scale[row] : 1.0f;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf_t * BN;
#pragma unroll 1
        for (int step = 0; step < STEPS; ++step) {
          const int c = egroup * (128 / GROUPS) + step * 32;
          const int x = t.nb * 128 + c;
          uint32_t ru[32], rg[32];
          tmem_ld_32x32b_x32(taddr + c, ru);
          tmem_ld_32x32b_x32(taddr + 128 + c, rg);
          tmem_ld_wait();
          uint32_t wu[16], wg[16], wa[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float u0 = bf16_round(__uint_as_float(ru[2 * i]) * rs), u1 = bf16_round(__uint_as_float(ru[2 * i + 1]) * rs);
            const float g0 = bf16_round(__uint_as_float(rg[2 * i]) * rs), g1 = bf16_round(__uint_as_float(rg[2 * i + 1]) * rs);
            wu[i] = pack_bf16x2(u0, u1);
            wg[i] = pack_bf16x2(g0, g1);
            wa[i] = pack_bf16x2(g0 * sigmoidf_(g0) * u0, g1 * sigmoidf_(g1) * u1);
          }
          if (lane == 0) tma_store_wait_read0();  // the previous step's stores have read the tiles
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<uint4*>(tile_chunk64(ebuf, lane, j)) = make_uint4(wu[4 * j], wu[4 * j + 1], wu[4 * j + 2], wu[4 * j + 3]);
            *reinterpret_cast<uint4*>(tile_chunk64(ebuf + 2048, lane, j)) = make_uint4(wg[4 * j], wg[4 * j + 1], wg[4 * j + 2], wg[4 * j + 3]);
            *reinterpret_cast<uint4*>(tile_chunk64(ebuf + 4096, lane, j)) = make_uint4(wa[4 * j], wa[4 * j + 1], wa[4 * j + 2], wa[4 * j + 3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (x < p.h && y < p.m) {
              if (p.out != nullptr) {
                tma_store_2d(&g.epi[0], ebuf, x, y);
                tma_store_2d(&g.epi[1], ebuf + 2048, x, y);
              }
              tma_store_2d(&g.epi[2], ebuf + 4096, x, y);
            }
            tma_store_commit();
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(mapa_shared(smem_u32(&tempty[buf_t]), 0));
      }
      if (lane == 0) tma_store_wait_all();
    } else if constexpr (EPI == WS_EPI_RESID_F32) {
      // out = residual + acc through shared memory: per warp 32 rows, per step 32 FP32 columns;
      // the residual tile is TMA-loaded (double-buffered), updated in place and TMA-stored.
      uint8_t* ebuf = eStage + (warp - 2) * 8192;  // two buffers of one 4 KiB tile
      uint64_t* mybar = ebar + (warp - 2) * 2;
      constexpr int STEPS = (BN / GROUPS) / 32;
      const GemmParams& p = g.p[0];
      auto coords = [&](int tile, int step, int& x, int& y) {
        const PairTile t = resolve_tile(g, tile, n_tile, GATHER);
        x = t.nb * BN + egroup * (BN / GROUPS) + step * 32;
        y = t.mb * 2 * BM + rank * BM + quarter * 32;
      };
      auto issue_load = [&](int tile, int step, int buf) {
        if (lane == 0) {
          int x, y;
          coords(tile, step, x, y);
          mbar_expect_tx(&mybar[buf], 4096);
          tma_load_2d(ebuf + buf * 4096, &g.epi[0], &mybar[buf], x, y);
        }
      };
      int q = 0;
      if (pair_id < tiles) issue_load(pair_id, 0, 0);
      bool ok = true;
      for (int tile = pair_id; tile < tiles && ok; tile += num_pairs, ++tcount) {
        const int buf_t = tcount & 1;
        const uint32_t tph = (tcount >> 1) & 1;
        if (!mbar_wait(&tfull[buf_t], tph, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf_t * BN + egroup * (BN / GROUPS);
#pragma unroll 1
        for (int step = 0; step < STEPS; ++step, ++q) {
          const int buf = q & 1;
          if (lane == 0) tma_store_wait_read0();
          if (step + 1 < STEPS) {
            issue_load(tile, step + 1, buf ^ 1);
          } else if (tile + num_pairs < tiles) {
            issue_load(tile + num_pairs, 0, buf ^ 1);
          }
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + step * 32, r);
          if (!mbar_wait(&mybar[buf], (q >> 1) & 1, abort_flag)) {
            ok = false;
            tmem_ld_wait();
            break;
          }
          tmem_ld_wait();
          uint8_t* tr = ebuf + buf * 4096;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4* pv = reinterpret_cast<float4*>(tile_chunk128(tr, lane, j));
            float4 v = *pv;
            v.x += __uint_as_float(r[4 * j]);
            v.y += __uint_as_float(r[4 * j + 1]);
            v.z += __uint_as_float(r[4 * j + 2]);
            v.w += __uint_as_float(r[4 * j + 3]);
            *pv = v;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            int x, y;
            coords(tile, step, x, y);
            if (x < p.n && y < p.m) tma_store_2d(&g.epi[1], tr, x, y);
            tma_store_commit();
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(mapa_shared(smem_u32(&tempty[buf_t]), 0));
      }
      if (lane == 0) tma_store_wait_all();
    } else if constexpr (STAGED) {
      // SwiGLU backward through shared memory.  Per warp: 32 rows; per step: 32 columns; two
      // buffers, each holding the (up, gate) tiles that become (dUp, dGate) in place.
      uint8_t* ebuf = eStage + (warp - 2) * 8192;
      uint64_t* mybar = ebar + (warp - 2) * 2;
      constexpr int STEPS = (BN / GROUPS) / 32;
      const GemmParams& p = g.p[0];
      auto coords = [&](int tile, int step, int& x, int& y) {
        const PairTile t = resolve_tile(g, tile, n_tile, GATHER);
        x = t.nb * BN + egroup * (BN / GROUPS) + step * 32;
        y = t.mb * 2 * BM + rank * BM + quarter * 32;
      };
      auto issue_load = [&](int tile, int step, int buf) {
        if (lane == 0) {
          int x, y;
          coords(tile, step, x, y);
          mbar_expect_tx(&mybar[buf], 4096);
          tma_load_2d(ebuf + buf * 4096, &g.epi[0], &mybar[buf], x, y);
          tma_load_2d(ebuf + buf * 4096 + 2048, &g.epi[1], &mybar[buf], x, y);
        }
      };
      int q = 0;  // steps done by this warp (buffer = q & 1, barrier phase = (q >> 1) & 1)
      if (pair_id < tiles) issue_load(pair_id, 0, 0);
      bool ok = true;
      for (int tile = pair_id; tile < tiles && ok; tile += num_pairs, ++tcount) {
        const int buf_t = tcount & 1;
        const uint32_t tph = (tcount >> 1) & 1;
        if (!mbar_wait(&tfull[buf_t], tph, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf_t * BN + egroup * (BN / GROUPS);
#pragma unroll 1
        for (int step = 0; step < STEPS; ++step, ++q) {
          const int buf = q & 1;
          // the store issued from the other buffer one step ago must have read it before it is refilled
          if (lane == 0) tma_store_wait_read0();
          if (step + 1 < STEPS) {
            issue_load(tile, step + 1, buf ^ 1);
          } else if (tile + num_pairs < tiles) {
            issue_load(tile + num_pairs, 0, buf ^ 1);
          }
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + step * 32, r);
          if (!mbar_wait(&mybar[buf], (q >> 1) & 1, abort_flag)) {
            ok = false;
            tmem_ld_wait();
            break;
          }
          tmem_ld_wait();
          uint8_t* tu = ebuf + buf * 4096;
          uint8_t* tg = tu + 2048;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4* pu = reinterpret_cast<uint4*>(tile_chunk64(tu, lane, j));
            uint4* pg = reinterpret_cast<uint4*>(tile_chunk64(tg, lane, j));
            const uint4 qu = *pu, qg = *pg;
            const __nv_bfloat162* bu = reinterpret_cast<const __nv_bfloat162*>(&qu);
            const __nv_bfloat162* bg = reinterpret_cast<const __nv_bfloat162*>(&qg);
            uint4 vu, vg;
            uint32_t* wu = reinterpret_cast<uint32_t*>(&vu);
            uint32_t* wg = reinterpret_cast<uint32_t*>(&vg);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float2 u = __bfloat1622float2(bu[t]);
              const float2 gg = __bfloat1622float2(bg[t]);
              const float d0 = bf16_round(__uint_as_float(r[j * 8 + 2 * t]));
              const float d1 = bf16_round(__uint_as_float(r[j * 8 + 2 * t + 1]));
              const float s0 = sigmoidf_(gg.x), s1 = sigmoidf_(gg.y);
              wu[t] = pack_bf16x2(d0 * gg.x * s0, d1 * gg.y * s1);
              wg[t] = pack_bf16x2(d0 * u.x * s0 * (1.0f + gg.x * (1.0f - s0)),
                                  d1 * u.y * s1 * (1.0f + gg.y * (1.0f - s1)));
            }
            *pu = vu;
            *pg = vg;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            int x, y;
            coords(tile, step, x, y);
            if (x < p.n && y < p.m) {  // a box that lies entirely outside is skipped
              tma_store_2d(&g.epi[2], tu, x, y);
              tma_store_2d(&g.epi[3], tg, x, y);
            }
            tma_store_commit();
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(mapa_shared(smem_u32(&tempty[buf_t]), 0));
      }
      if (lane == 0) tma_store_wait_all();
    } else {
      for (int tile = pair_id; tile < tiles; tile += num_pairs, ++tcount) {
        const PairTile t = resolve_tile(g, tile, n_tile, GATHER);
        const GemmParams& p = g.p[t.prob];
        const int nb = t.nb;
        const int buf = tcount & 1;
        const uint32_t tph = (tcount >> 1) & 1;
        if (!mbar_wait(&tfull[buf], tph, abort_flag)) break;
        tc_fence_after_sync();
        const int row = t.mb * 2 * BM + rank * BM + quarter * 32 + lane;
        const bool row_ok = row < p.m;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
        const float rs = (p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.0f;
        gemm_epilogue<EPI, GROUPS>(p, taddr, row, row_ok, rs, nb, egroup);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(mapa_shared(smem_u32(&tempty[buf]), 0));
      }
    }
  }

  if constexpr (GATHER) {
    if (warp >= 2 + 4 * GROUPS) {
      // ---------------------------------------------------------------- weight gather (both CTAs)
      // Chunk c = GATHER_ROWS rows of W.  A thread converts 8 consecutive floats (two 16-byte loads,
      // local or peer) into one 16-byte BF16 store.
      // Chunks are claimed from a counter in global memory, in order, by whichever CTAs are running: the
      // tile loop of a CTA never depends on a CTA that is not resident yet (another kernel may hold SMs),
      // and the blocks still complete in the order in which the tile loop needs them.
      const int gt = threadIdx.x - (2 + 4 * GROUPS) * 32;
      const int vec_per_row = gj.k / 8;
      const int chunks = (gj.n + GATHER_ROWS - 1) / GATHER_ROWS;
      volatile int* chunk_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);
      while (true) {
        if (gt == 0) *chunk_slot = static_cast<int>(atomicAdd(gj.counter, 1u));
        asm volatile("bar.sync 3, %0;" ::"n"(GATHER_THREADS) : "memory");
        const int c = *chunk_slot;
        asm volatile("bar.sync 3, %0;" ::"n"(GATHER_THREADS) : "memory");
        if (c >= chunks) break;
        // SwiGLU (W = h up rows, then h gate rows): even chunks walk the up rows, odd chunks the gate
        // rows, so that the two 128-row blocks of an N tile complete together
        const int row0 = gj.interleave_h > 0 ? (c & 1) * gj.interleave_h + (c >> 1) * GATHER_ROWS : c * GATHER_ROWS;
        const int rows = min(GATHER_ROWS, gj.n - row0);
        const int owner = row0 / gj.rows_per_shard;
        const float* src = gj.shard[owner] + static_cast<size_t>(row0 - owner * gj.rows_per_shard) * gj.k;
        __nv_bfloat16* dst = gj.dst + static_cast<size_t>(row0) * gj.k;
        const int vecs = rows * vec_per_row;  // rows are contiguous in both buffers
        // four 32-byte pieces per thread are requested before the first is converted: a peer load takes
        // a few microseconds, and a chunk is one such round trip
        for (int v0 = 0; v0 < vecs; v0 += 4 * GATHER_THREADS) {
          float4 lo[4], hi[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * GATHER_THREADS + gt;
            if (v < vecs) {
              lo[u] = __ldg(reinterpret_cast<const float4*>(src) + 2 * v);
              hi[u] = __ldg(reinterpret_cast<const float4*>(src) + 2 * v + 1);
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * GATHER_THREADS + gt;
            if (v < vecs) {
              uint4 o;
              o.x = pack_bf16x2(lo[u].x, lo[u].y);
              o.y = pack_bf16x2(lo[u].z, lo[u].w);
              o.z = pack_bf16x2(hi[u].x, hi[u].y);
              o.w = pack_bf16x2(hi[u].z, hi[u].w);
              reinterpret_cast<uint4*>(dst)[v] = o;
            }
          }
        }
        __threadfence();
        asm volatile("fence.proxy.async.global;" ::: "memory");
        asm volatile("bar.sync 3, %0;" ::"n"(GATHER_THREADS) : "memory");
        if (gt == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(gj.flags + row0 / GATHER_BLOCK) : "memory");
      }
    }
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && g.p[0].error_flag != nullptr) atomicExch(g.p[0].error_flag, 6);
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while the peer may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_pair(const PairGroup& g, int pairs, cudaStream_t stream) {
  static bool configured = false;
  auto kern = gemm2_kernel<A_MN, B_MN, EPI>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem<EPI>()) != cudaSuccess)
      return -20;
    configured = true;
  }
  launch_dependent(kern, dim3(2 * pairs), dim3(pair_threads<EPI>()), pair_smem<EPI>(), stream, g, GatherJob{});
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

template <int EPI>
static int launch_pair_gather(const PairGroup& g, const GatherJob& job, int pairs, cudaStream_t stream) {
  static bool configured = false;
  auto kern = gemm2_kernel<false, false, EPI, true>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem<EPI>()) != cudaSuccess)
      return -20;
    configured = true;
  }
  launch_dependent(kern, dim3(2 * pairs), dim3(pair_threads<EPI>() + GATHER_THREADS), pair_smem<EPI>(), stream, g, job);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

// Tensor maps, kernel parameters and tile count of one problem.
static int fill_problem(const WsGemm* g, PairGroup& grp, int i, int* tiles_out) {
  if (g->m <= 0 || g->n <= 0 || g->k <= 0) return -1;
  const bool swiglu = g->epilogue == WS_EPI_SWIGLU;
  const int b_rows = swiglu ? 2 * g->n : g->n;
  int rc;
  if (!g->a_mn)
    rc = make_map_bf16(&grp.a[i], g->a, g->k, g->m, g->lda, pair::BK, pair::BM);
  else
    rc = make_map_bf16(&grp.a[i], g->a, g->m, g->k, g->lda, 64, pair::BK);
  if (rc) return rc;
  if (!g->b_mn)
    rc = make_map_bf16(&grp.b[i], g->b, g->k, b_rows, g->ldb, pair::BK, 128);
  else
    rc = make_map_bf16(&grp.b[i], g->b, b_rows, g->k, g->ldb, 64, pair::BK);
  if (rc) return rc;
  GemmParams& p = grp.p[i];
  p.m = g->m; p.n = g->n; p.k = g->k;
  p.h = g->n;
  p.epi_n = swiglu ? 128 : pair::BN;
  p.out = g->out; p.ldo = g->ldo;
  p.out2 = g->out2; p.ldo2 = g->ldo2;
  p.aux = g->aux; p.ldaux = g->ldaux;
  p.row_scale = g->row_scale;
  p.row_vec = g->row_vec;
  p.alpha = g->alpha; p.beta = g->beta;
  p.error_flag = g->error_flag;
  p.debug = 0;
  const int n_tile = swiglu ? 128 : pair::BN;
  *tiles_out = ((g->m + 2 * pair::BM - 1) / (2 * pair::BM)) * ((g->n + n_tile - 1) / n_tile);
  return 0;
}

// Staged SwiGLU-forward epilogue: 32 x 32 store boxes over the packed (up | gate) matrix and the activation.
static int fill_swiglu_maps(const WsGemm* g0, PairGroup& grp) {
  __nv_bfloat16* packed = static_cast<__nv_bfloat16*>(g0->out);
  __nv_bfloat16* act = static_cast<__nv_bfloat16*>(g0->out2);
  const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_64B;
  int rc = 0;
  if (packed != nullptr) {
    rc = make_map_bf16_swz(&grp.epi[0], packed, g0->n, g0->m, g0->ldo, 32, 32, sw);
    if (!rc) rc = make_map_bf16_swz(&grp.epi[1], packed + g0->n, g0->n, g0->m, g0->ldo, 32, 32, sw);
  }
  if (!rc) rc = make_map_bf16_swz(&grp.epi[2], act, g0->n, g0->m, g0->ldo2, 32, 32, sw);
  if (rc) return rc;
  if (packed == nullptr) {
    grp.epi[0] = grp.epi[2];  // never used for a store; keeps the descriptor prefetch valid
    grp.epi[1] = grp.epi[2];
  }
  return 0;
}

}  // namespace ws

// `count` problems (1..4) of one kind (same operand majors and epilogue) in one launch.  The
// argument checks of ws_gemm have already run on every item; `sms` bounds the SMs used.
// Returns -6 for a combination this kernel does not build.
extern "C" int ws_gemm_pair_group(const WsGemm* items, int count, int sms, cudaStream_t stream) {
  using namespace ws;
  if (count < 1 || count > MAX_GROUP) return -9;
  PairGroup grp;
  memset(&grp, 0, sizeof(grp));
  grp.count = count;
  int total = 0;
  for (int i = 0; i < count; ++i) {
    if (items[i].a_mn != items[0].a_mn || items[i].b_mn != items[0].b_mn || items[i].epilogue != items[0].epilogue)
      return -9;
    int tiles = 0;
    const int rc = fill_problem(&items[i], grp, i, &tiles);
    if (rc) return rc;
    grp.tile_start[i] = total;
    total += tiles;
  }
  for (int i = count; i <= MAX_GROUP; ++i) grp.tile_start[i] = total;
  if (items[0].epilogue == WS_EPI_RESID_F32) {
    if (count != 1) return -9;
    const WsGemm* g0 = &items[0];
    int rc = make_map_f32(&grp.epi[0], g0->aux, g0->n, g0->m, g0->ldaux, 32, 32);
    if (!rc) rc = make_map_f32(&grp.epi[1], g0->out, g0->n, g0->m, g0->ldo, 32, 32);
    if (rc) return rc;
  }
  if (items[0].epilogue == WS_EPI_SWIGLU) {
    if (count != 1) return -9;
    const int rc = fill_swiglu_maps(&items[0], grp);
    if (rc) return rc;
  }
  if (items[0].epilogue == WS_EPI_SWIGLU_BWD) {
    if (count != 1) return -9;
    const WsGemm* g0 = &items[0];
    const __nv_bfloat16* aux = static_cast<const __nv_bfloat16*>(g0->aux);
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(g0->out);
    const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_64B;
    int rc = make_map_bf16_swz(&grp.epi[0], aux, g0->n, g0->m, g0->ldaux, 32, 32, sw);
    if (!rc) rc = make_map_bf16_swz(&grp.epi[1], aux + g0->n, g0->n, g0->m, g0->ldaux, 32, 32, sw);
    if (!rc) rc = make_map_bf16_swz(&grp.epi[2], out, g0->n, g0->m, g0->ldo, 32, 32, sw);
    if (!rc) rc = make_map_bf16_swz(&grp.epi[3], out + g0->n, g0->n, g0->m, g0->ldo, 32, 32, sw);
    if (rc) return rc;
  }
  int pairs = sms / 2;
  if (pairs < 1) pairs = 1;
  if (total < pairs) pairs = total;
  const WsGemm* g = &items[0];
  const int key = (g->a_mn ? 1 : 0) | (g->b_mn ? 2 : 0) | (g->epilogue << 2);
  switch (key) {
    case (0 | (WS_EPI_BF16 << 2)): return launch_pair<false, false, WS_EPI_BF16>(grp, pairs, stream);
    case (2 | (WS_EPI_BF16 << 2)): return launch_pair<false, true, WS_EPI_BF16>(grp, pairs, stream);
    case (0 | (WS_EPI_RESID_F32 << 2)): return launch_pair<false, false, WS_EPI_RESID_F32>(grp, pairs, stream);
    case (0 | (WS_EPI_RESID_BF16 << 2)): return launch_pair<false, false, WS_EPI_RESID_BF16>(grp, pairs, stream);
    case (0 | (WS_EPI_SWIGLU << 2)): return launch_pair<false, false, WS_EPI_SWIGLU>(grp, pairs, stream);
    case (0 | (WS_EPI_F32 << 2)): return launch_pair<false, false, WS_EPI_F32>(grp, pairs, stream);
    case (3 | (WS_EPI_ACC_F32 << 2)): return launch_pair<true, true, WS_EPI_ACC_F32>(grp, pairs, stream);
    case (3 | (WS_EPI_BF16 << 2)): return launch_pair<true, true, WS_EPI_BF16>(grp, pairs, stream);
    case (2 | (WS_EPI_SWIGLU_BWD << 2)): return launch_pair<false, true, WS_EPI_SWIGLU_BWD>(grp, pairs, stream);
    case (0 | (WS_EPI_CE_FWD << 2)): return launch_pair<false, false, WS_EPI_CE_FWD>(grp, pairs, stream);
    case (0 | (WS_EPI_CE_BWD << 2)): return launch_pair<false, false, WS_EPI_CE_BWD>(grp, pairs, stream);
    default: return -6;
  }
}

extern "C" int ws_gemm_pair(const WsGemm* g, int sms, cudaStream_t stream) {
  return ws_gemm_pair_group(g, 1, sms, stream);
}

// y[m, n] = x[m, k] . W[n, k]^T where W is the row-sharded FP32 master weight of `world` ranks
// (shards[r] = address, in this process, of rank r's [rows_per_shard, k] FP32 block; peers' blocks are
// symmetric-memory mappings).  `wb` is this rank's BF16 landing buffer for the whole weight, `flags` a
// device array of one word per 128 weight rows plus one more (zeroed here).  epilogue WS_EPI_BF16: W has n rows, out is
// BF16 [m, n].  WS_EPI_SWIGLU: W has 2n rows (n up rows, then n gate rows; n % 128 == 0), out is the packed
// (up | gate) [m, 2n] (may be NULL), out2 the activation silu(gate) * up [m, n].  The caller guarantees that
// no rank changes its shard while the kernel runs.  A bounded wait that runs out sets *error_flag to 6 and
// the launch still terminates.
extern "C" int ws_gather_gemm(const void* x, int m, int n, int k, const void* const* shards, int world,
                              int rows_per_shard, void* wb, void* flags, int epilogue, void* out, int ldo,
                              void* out2, int ldo2, int* error_flag, float budget_seconds, int sms,
                              cudaStream_t stream) {
  using namespace ws;
  const bool swiglu = epilogue == WS_EPI_SWIGLU;
  if (epilogue != WS_EPI_BF16 && !swiglu) return -6;
  if (m <= 0 || n <= 0 || k <= 0 || k % 8 != 0 || world < 1 || world > 8) return -1;
  const int w_rows = swiglu ? 2 * n : n;
  if (swiglu && (n % GATHER_BLOCK != 0 || out2 == nullptr || ldo2 < n || ldo2 % 8 != 0)) return -1;
  if (rows_per_shard <= 0 || rows_per_shard % 8 != 0 || (long long)rows_per_shard * world < w_rows) return -1;
  if (out != nullptr && (ldo < w_rows || ldo % 8 != 0)) return -1;
  if (!swiglu && out == nullptr) return -1;
  if (((uintptr_t)x | (uintptr_t)wb | (uintptr_t)out | (uintptr_t)out2) & 15) return -5;
  for (int r = 0; r < world; ++r)
    if (shards[r] == nullptr || ((uintptr_t)shards[r] & 15)) return -5;
  WsGemm item;
  memset(&item, 0, sizeof(item));
  item.a = x; item.b = wb; item.m = m; item.n = n; item.k = k; item.lda = k; item.ldb = k;
  item.epilogue = epilogue; item.out = out; item.ldo = ldo; item.out2 = out2; item.ldo2 = ldo2;
  item.alpha = 1.f; item.error_flag = error_flag;
  PairGroup grp;
  memset(&grp, 0, sizeof(grp));
  grp.count = 1;
  int tiles = 0;
  int rc = fill_problem(&item, grp, 0, &tiles);
  if (rc) return rc;
  for (int i = 1; i <= MAX_GROUP; ++i) grp.tile_start[i] = tiles;
  if (swiglu) {
    rc = fill_swiglu_maps(&item, grp);
    if (rc) return rc;
  }
  GatherJob job;
  memset(&job, 0, sizeof(job));
  for (int r = 0; r < world; ++r) job.shard[r] = static_cast<const float*>(shards[r]);
  job.world = world;
  job.rows_per_shard = rows_per_shard;
  job.n = w_rows; job.k = k;
  job.dst = static_cast<__nv_bfloat16*>(wb);
  job.flags = static_cast<unsigned*>(flags);
  job.target = GATHER_BLOCK / GATHER_ROWS;
  job.interleave_h = swiglu ? n : 0;
  job.wait_ns = static_cast<unsigned long long>((budget_seconds > 0.f ? budget_seconds : 2.0f) * 1e9);
  const int blocks = (w_rows + GATHER_BLOCK - 1) / GATHER_BLOCK;
  job.counter = job.flags + blocks;  // the word after the block flags
  if (cudaMemsetAsync(flags, 0, sizeof(unsigned) * (blocks + 1), stream) != cudaSuccess) return -21;
  // Gather chunks are claimed dynamically by running CTAs, so no CTA waits for one that is not resident;
  // with fewer tiles than pairs the spare pairs still take gather chunks.
  int dev = 0, sm_count = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  int pairs = (sms > 0 ? sms : sm_count) / 2;
  if (pairs < 1) pairs = 1;
  if (pairs > sm_count / 2) pairs = sm_count / 2;
  return swiglu ? launch_pair_gather<WS_EPI_SWIGLU>(grp, job, pairs, stream)
                : launch_pair_gather<WS_EPI_BF16>(grp, job, pairs, stream);
}
