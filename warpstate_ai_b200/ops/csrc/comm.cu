// Data-parallel communication kernels over NVLink peer memory (one process per GPU; every
// rank maps every other rank's buffers: "symmetric memory").
//
//   bucket_ready_kernel + grad_reduce_kernel : two-shot all-reduce of one gradient bucket, in place, fused with
//                           the 1/world scaling and a sum-of-squares partial for the global norm.
//                           Rank r reduces slice r of the bucket by pulling it from all ranks
//                           (plain peer loads, summed in rank order -> every rank ends with
//                           bit-identical gradients), or with one in-switch reduction
//                           (multimem.ld_reduce) when a multimem address is given; then pushes the
//                           reduced slice to all ranks (peer stores or multimem.st).
//                           `push == 0` gives the reduce-scatter used by the sharded optimizer.
//   adamw_shard_push      : AdamW on the shard a rank owns, fused with the clip scale and the
//                           FP32->BF16 re-cast, storing the updated FP32 master and BF16 weights
//                           straight into every rank's replicas (the all-gather of the update).
//
// This replaces the reference's DDP bucket all-reduce through NCCL (57 FP32 buckets per update,
// reference ops/OPTIMIZATION_20260912.md:228-229; DDP wrap run_40b.py:601-603) and, in sharded
// mode, the parameter all-gather a ZeRO-style design needs.
//
// Cross-rank signalling: per bucket, per source rank, a `ready` word (value = update sequence
// number) and a `done` counter (value = sequence number * CTAs) live in each rank's flag
// buffer.  Writers use st.release.sys / red.release.sys, readers ld.acquire.sys.  Every wait is
// bounded by a caller-given time budget; on expiry the kernel records
// {code, bucket, waiting-for rank, expected, seen} in its status words and returns.
// No TMA is used here and nothing in this file reads another GPU's memory through a tensor map.
#include "ws_ptx.cuh"
#include "ws_api.h"

#include <cstring>

namespace ws {

extern "C" void ws_count_launch(void);

constexpr int MAX_RANKS = 8;
constexpr int COMM_THREADS = 512;

struct PeerTable {
  float* grad[MAX_RANKS];      // each rank's gradient arena (same layout everywhere)
  unsigned* flags[MAX_RANKS];  // each rank's flag buffer
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_f4(float* p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f4(float* p, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

// Flag layout inside one rank's flag buffer.
__device__ __host__ __forceinline__ int ready_index(int bucket, int src) { return (bucket * 2 + 0) * MAX_RANKS + src; }
__device__ __host__ __forceinline__ int done_index(int bucket, int src) { return (bucket * 2 + 1) * MAX_RANKS + src; }

// Bounded wait until *p >= expected.  Returns false on expiry (and fills the status words).
__device__ __forceinline__ bool wait_at_least(const unsigned* p, unsigned expected, unsigned long long budget_ns,
                                              int* status, int code, int bucket, int src) {
  unsigned seen = ld_acquire_sys(p);
  if (seen >= expected) return true;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    seen = ld_acquire_sys(p);
    if (seen >= expected) return true;
    __nanosleep(200);
    if (globaltimer_ns() - t0 > budget_ns) {
      if (status != nullptr && atomicCAS(status, 0, code) == 0) {
        status[1] = bucket;
        status[2] = src;
        status[3] = static_cast<int>(expected);
        status[4] = static_cast<int>(seen);
      }
      return false;
    }
  }
}

// Up to MAX_SEGMENTS ranges of the arena handled by one launch: a core's projection matrices as
// reduce-scatter segments (each rank keeps the rows it owns) and its small parameters as an
// all-reduce segment, or one range for a whole replicated bucket.
constexpr int MAX_SEGMENTS = 6;
struct Segments {
  size_t start[MAX_SEGMENTS];
  size_t count[MAX_SEGMENTS];
  int push[MAX_SEGMENTS];
  int n;
};

// Step 1 of a bucket: announce that this rank's bucket is final (its producers ran earlier on this
// stream) and wait for every rank's announcement.  One warp: while ranks are out of step nothing
// but this warp is resident, and the data kernel that follows on the stream starts only when
// every rank's gradients are there.
__global__ void bucket_ready_kernel(PeerTable peers, int rank, int world, int bucket, unsigned seq, int* status,
                                    unsigned long long budget_ns) {
  const int tid = threadIdx.x;
  if (tid < world) {
    __threadfence_system();
    st_release_sys(peers.flags[tid] + ready_index(bucket, rank), seq);
    wait_at_least(peers.flags[rank] + ready_index(bucket, tid), seq, budget_ns, status, 1, bucket, tid);
  }
}

// Step 2: reduce my slice of every segment, scale, push (or keep), count completions.
__global__ void __launch_bounds__(COMM_THREADS)
grad_reduce_kernel(PeerTable peers, float* mc_grad, int rank, int world, Segments segs, int bucket, unsigned seq,
                   float scale, float* sumsq_out, int* status, unsigned long long budget_ns) {
  __shared__ float s_red[COMM_THREADS / 32];
  const int tid = threadIdx.x;
  // a wait that ran out earlier in this update (this bucket's or another's): move nothing more
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  float ss = 0.f;
  // Four independent 16-byte pieces per thread and pass: a peer or multimem load takes microseconds, and
  // with one piece in flight per thread the kernel's bandwidth is set by its CTA count (6.7 GB/s per CTA
  // measured).  The element-to-thread mapping and the order in which a thread adds its pieces (to the
  // reduction and to the sum of squares) are those of a one-piece loop.
  constexpr int U = 4;
  const size_t stride = static_cast<size_t>(gridDim.x) * COMM_THREADS;
  for (int sg = 0; sg < segs.n; ++sg) {
    const size_t start = segs.start[sg];
    const int push = segs.push[sg];
    const size_t n4 = segs.count[sg] / 4;
    const size_t per = (n4 + world - 1) / world;
    const size_t lo = per * rank < n4 ? per * rank : n4;
    size_t hi = lo + per;
    if (hi > n4) hi = n4;
    auto finish = [&](size_t off, float4 acc) {
      acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
      ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
      if (!push) {
        *reinterpret_cast<float4*>(peers.grad[rank] + off) = acc;
      } else if (mc_grad != nullptr) {
        multimem_st_f4(mc_grad + off, acc);
      } else {
        for (int r = 0; r < world; ++r) st_sys_f4(peers.grad[r] + off, acc);
      }
    };
    size_t i = lo + blockIdx.x * static_cast<size_t>(COMM_THREADS) + tid;
    for (; i + (U - 1) * stride < hi; i += U * stride) {
      float4 acc[U];
      if (mc_grad != nullptr) {
#pragma unroll
        for (int u = 0; u < U; ++u) acc[u] = multimem_ld_reduce_f4(mc_grad + start + (i + u * stride) * 4);
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) acc[u] = ld_sys_f4(peers.grad[0] + start + (i + u * stride) * 4);
        for (int r = 1; r < world; ++r) {
          float4 v[U];
#pragma unroll
          for (int u = 0; u < U; ++u) v[u] = ld_sys_f4(peers.grad[r] + start + (i + u * stride) * 4);
#pragma unroll
          for (int u = 0; u < U; ++u) {
            acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) finish(start + (i + u * stride) * 4, acc[u]);
    }
    for (; i < hi; i += stride) {
      const size_t off = start + i * 4;
      float4 acc;
      if (mc_grad != nullptr) {
        acc = multimem_ld_reduce_f4(mc_grad + off);
      } else {
        acc = ld_sys_f4(peers.grad[0] + off);
        for (int r = 1; r < world; ++r) {
          const float4 v = ld_sys_f4(peers.grad[r] + off);
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
      }
      finish(off, acc);
    }
  }
  // sum-of-squares partial of this CTA (fixed order inside the CTA; CTAs and buckets are combined in index
  // order by norm_exchange_kernel).  Every element of the bucket is reduced by exactly one rank, so the
  // partials of all ranks together cover the whole averaged gradient once.
  if (sumsq_out != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) s_red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
      for (int wi = 0; wi < COMM_THREADS / 32; ++wi) t += s_red[wi];
      sumsq_out[blockIdx.x] = t;
    }
  }
  // tell every rank that this CTA's share of slice `rank` has landed
  __threadfence_system();
  __syncthreads();
  if (tid < world) red_release_sys_add(peers.flags[tid] + done_index(bucket, rank), 1u);
  // one CTA waits until every rank has finished reading from and writing to this rank's buffer
  if (blockIdx.x == 0 && tid < world)
    wait_at_least(peers.flags[rank] + done_index(bucket, tid), seq * gridDim.x, budget_ns, status, 2, bucket, tid);
}

// Global gradient norm, clip coefficient and loss sum in one launch, with no library collective: every
// rank sums its own partial sums of squares in index order, stores that sum (and its local loss sum) into
// slot `rank` of every rank's exchange words, waits (bounded) for all slots, and adds the slots in rank
// order -- so all ranks compute bit-identical statistics.
//   stats[0] norm, [1] clip coefficient, [2] norm^2, [3] skip flag (non-finite norm or *status != 0),
//   [4] sum over ranks of *local_loss (when given).
// Exchange words (in each rank's flag buffer, from word `base`): MAX_RANKS ready words, then
// MAX_RANKS x 2 value words.
__global__ void norm_exchange_kernel(PeerTable peers, int rank, int world, int base, unsigned seq,
                                     const float* __restrict__ partial, int parts, const float* local_loss,
                                     float max_norm, int* status, float* __restrict__ stats,
                                     unsigned long long budget_ns) {
  __shared__ float red[32];
  __shared__ float s_local;
  float s = 0.f;
  for (int i = threadIdx.x; i < parts; i += blockDim.x) s += partial[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    s_local = t;
  }
  __syncthreads();
  const int tid = threadIdx.x;
  if (tid < world) {
    unsigned* words = peers.flags[tid] + base;
    float* vals = reinterpret_cast<float*>(words + MAX_RANKS);
    vals[2 * rank + 0] = s_local;
    vals[2 * rank + 1] = local_loss != nullptr ? *local_loss : 0.f;
    __threadfence_system();
    st_release_sys(words + rank, seq);
    wait_at_least(peers.flags[rank] + base + tid, seq, budget_ns, status, 3, -2, tid);
  }
  __syncthreads();
  if (tid == 0) {
    const float* vals = reinterpret_cast<const float*>(peers.flags[rank] + base + MAX_RANKS);
    float total = 0.f, loss = 0.f;
    for (int r = 0; r < world; ++r) {
      total += *reinterpret_cast<const volatile float*>(vals + 2 * r);
      loss += *reinterpret_cast<const volatile float*>(vals + 2 * r + 1);
    }
    const float norm = __fsqrt_rn(total);
    float coef = max_norm > 0.f ? __fdiv_rn(max_norm, norm + 1e-6f) : 1.0f;
    if (coef > 1.0f) coef = 1.0f;
    const bool bad = (__float_as_uint(norm) & 0x7f800000u) == 0x7f800000u || *reinterpret_cast<volatile int*>(status) != 0;
    stats[0] = norm;
    stats[1] = bad ? 0.0f : coef;
    stats[2] = total;
    stats[3] = bad ? 1.0f : 0.0f;
    stats[4] = loss;
  }
}

// Copy-and-cast of a row-sharded FP32 weight into a local BF16 [n, k] buffer: rank r owns rows
// [r * rows_per_shard, ...); rows of other ranks are plain peer loads over NVLink.  A thread converts 8
// consecutive floats (two 16-byte loads) into one 16-byte store, four such pieces in flight.
struct GatherTable {
  const float* shard[MAX_RANKS];
};
__global__ void __launch_bounds__(256)
gather_cast_kernel(GatherTable t, int rows_per_shard, int n, int k, __nv_bfloat16* __restrict__ dst) {
  const size_t vec_per_row = static_cast<size_t>(k) / 8;
  const size_t vecs = static_cast<size_t>(n) * vec_per_row;
  const size_t stride = static_cast<size_t>(gridDim.x) * 256;
  constexpr int U = 4;
  for (size_t v0 = blockIdx.x * static_cast<size_t>(256) + threadIdx.x; v0 < vecs; v0 += U * stride) {
    float4 lo[U], hi[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = v0 + u * stride;
      if (v < vecs) {
        const size_t row = v / vec_per_row;
        const int owner = static_cast<int>(row / rows_per_shard);
        const float* src = t.shard[owner] + (row - static_cast<size_t>(owner) * rows_per_shard) * k + (v - row * vec_per_row) * 8;
        lo[u] = ld_sys_f4(src);
        hi[u] = ld_sys_f4(src + 4);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = v0 + u * stride;
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
}

// Node barrier on the device: every rank stores `seq` into slot `rank` of every rank's barrier words and
// waits (bounded) for all slots.  Orders "my shard is updated" before "a peer gathers it".
__global__ void node_barrier_kernel(PeerTable peers, int rank, int world, int base, unsigned seq, int* status,
                                    unsigned long long budget_ns) {
  const int tid = threadIdx.x;
  if (tid < world) {
    __threadfence_system();
    st_release_sys(peers.flags[tid] + base + rank, seq);
    wait_at_least(peers.flags[rank] + base + tid, seq, budget_ns, status, 4, -3, tid);
  }
}

// A wait that nothing satisfies: used to check on a GPU that an expired wait returns an error
// status and leaves the context usable.  It reads only this rank's own flag buffer.
__global__ void wait_probe_kernel(const unsigned* flag, unsigned expected, int* status, unsigned long long budget_ns) {
  if (threadIdx.x == 0 && blockIdx.x == 0) wait_at_least(flag, expected, budget_ns, status, 9, -1, -1);
}

struct ParamPeers {
  float* master[MAX_RANKS];
  __nv_bfloat16* bf16[MAX_RANKS];
};

// AdamW on [lo, lo+n) of the arena (this rank's shard) with the result stored to every rank.
__global__ void __launch_bounds__(256)
adamw_shard_push_kernel(ParamPeers peers, int world, const float* __restrict__ g, float* __restrict__ m,
                        float* __restrict__ v, size_t lo, size_t n4, float lr, float beta1, float beta2, float eps,
                        float wd, float bias1, float bias2_sqrt, const float* __restrict__ grad_scale_ptr,
                        int rank, int push_master, const float* __restrict__ skip_ptr) {
  if (skip_ptr != nullptr && *skip_ptr != 0.0f) return;  // non-finite norm or failed gradient exchange
  const float gs = grad_scale_ptr != nullptr ? *grad_scale_ptr : 1.0f;
  const float decay = 1.0f - lr * wd;
  const float step_size = lr / bias1;
  for (size_t i = blockIdx.x * static_cast<size_t>(256) + threadIdx.x; i < n4;
       i += static_cast<size_t>(gridDim.x) * 256) {
    const size_t off = lo + i * 4;
    float4 pp = *reinterpret_cast<const float4*>(peers.master[rank] + off);
    const float4 gg = *reinterpret_cast<const float4*>(g + off);
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* pa = reinterpret_cast<float*>(&pp);
    const float* ga = reinterpret_cast<const float*>(&gg);
    float* ma = reinterpret_cast<float*>(&mm);
    float* va = reinterpret_cast<float*>(&vv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float grad = ga[k] * gs;
      float param = pa[k] * decay;
      const float mom = ma[k] + (grad - ma[k]) * (1.0f - beta1);
      const float var = beta2 * va[k] + (1.0f - beta2) * grad * grad;
      const float denom = __fdiv_rn(__fsqrt_rn(var), bias2_sqrt) + eps;
      param -= step_size * __fdiv_rn(mom, denom);
      pa[k] = param; ma[k] = mom; va[k] = var;
    }
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    uint2 o;
    o.x = pack_bf16x2(pa[0], pa[1]);
    o.y = pack_bf16x2(pa[2], pa[3]);
    for (int r = 0; r < world; ++r) {
      if (r == rank || push_master) st_sys_f4(peers.master[r] + off, pp);
      asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(peers.bf16[r] + off), "r"(o.x), "r"(o.y)
                   : "memory");
    }
  }
}

}  // namespace ws

using namespace ws;

extern "C" int ws_comm_flag_words(int buckets) { return buckets * 2 * MAX_RANKS; }
extern "C" int ws_comm_max_ctas(void) { return 64; }

static void fill_peers(PeerTable& t, const unsigned long long* grad_ptrs, const unsigned long long* flag_ptrs, int world) {
  for (int r = 0; r < MAX_RANKS; ++r) {
    t.grad[r] = (grad_ptrs != nullptr && r < world) ? reinterpret_cast<float*>(grad_ptrs[r]) : nullptr;
    t.flags[r] = r < world ? reinterpret_cast<unsigned*>(flag_ptrs[r]) : nullptr;
  }
}

// grad_ptrs / flag_ptrs: `world` device addresses (this process's mappings of every rank's
// buffers, own rank included).  mc_grad: multimem address of the gradient arena or NULL.
// `nseg` ranges [starts[i], starts[i] + counts[i]) of the arena; push[i] = 1 all-reduce, 0 reduce-scatter.
// sumsq_out: `ctas` floats (may be NULL).  status: 8 ints on the device.
// Two launches: a one-warp kernel that announces this rank's bucket and waits for the others', then the data
// kernel.  `seq` counts the calls on this bucket from 1, on every rank alike, and `ctas` must be the same in
// every call on a bucket: its completion counter advances by `ctas` per call and a rank waits for seq * ctas.
// (A different CTA count needs a bucket of its own; a mismatch ends in a reported time-out, code 2.)
extern "C" int ws_grad_reduce_segments(const unsigned long long* grad_ptrs, const unsigned long long* flag_ptrs,
                                       unsigned long long mc_grad, int rank, int world, const size_t* starts,
                                       const size_t* counts, const int* push, int nseg, int bucket, unsigned seq,
                                       float scale, int ctas, float* sumsq_out, int* status, double budget_seconds,
                                       cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || nseg < 1 || nseg > MAX_SEGMENTS) return -1;
  if (ctas < 1 || ctas > ws_comm_max_ctas()) return -2;
  Segments segs;
  memset(&segs, 0, sizeof(segs));
  segs.n = nseg;
  for (int i = 0; i < nseg; ++i) {
    if (counts[i] % 4 != 0 || starts[i] % 4 != 0) return -1;
    segs.start[i] = starts[i];
    segs.count[i] = counts[i];
    segs.push[i] = push[i];
  }
  PeerTable t;
  fill_peers(t, grad_ptrs, flag_ptrs, world);
  const unsigned long long budget = static_cast<unsigned long long>(budget_seconds * 1e9);
  bucket_ready_kernel<<<1, 32, 0, stream>>>(t, rank, world, bucket, seq, status, budget);
  ws_count_launch();
  grad_reduce_kernel<<<ctas, COMM_THREADS, 0, stream>>>(t, reinterpret_cast<float*>(mc_grad), rank, world, segs, bucket,
                                                        seq, scale, sumsq_out, status, budget);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ws_grad_allreduce(const unsigned long long* grad_ptrs, const unsigned long long* flag_ptrs,
                                 unsigned long long mc_grad, int rank, int world, size_t start, size_t count,
                                 int bucket, unsigned seq, float scale, int push, int ctas, float* sumsq_out,
                                 int* status, double budget_seconds, cudaStream_t stream) {
  return ws_grad_reduce_segments(grad_ptrs, flag_ptrs, mc_grad, rank, world, &start, &count, &push, 1, bucket, seq,
                                 scale, ctas, sumsq_out, status, budget_seconds, stream);
}

// Words a rank's flag buffer needs beyond the bucket flags: norm exchange (ready + 2 values per rank) and
// the node barrier.
extern "C" int ws_comm_extra_words(void) { return 4 * MAX_RANKS; }

extern "C" int ws_norm_exchange(const unsigned long long* flag_ptrs, int rank, int world, int base_word, unsigned seq,
                                const float* partial, int parts, const float* local_loss, float max_norm, int* status,
                                float* stats, double budget_seconds, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || parts < 1 || base_word < 0) return -1;
  PeerTable t;
  fill_peers(t, nullptr, flag_ptrs, world);
  norm_exchange_kernel<<<1, 256, 0, stream>>>(t, rank, world, base_word, seq, partial, parts, local_loss, max_norm,
                                              status, stats, static_cast<unsigned long long>(budget_seconds * 1e9));
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ws_node_barrier(const unsigned long long* flag_ptrs, int rank, int world, int base_word, unsigned seq,
                               int* status, double budget_seconds, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || base_word < 0) return -1;
  PeerTable t;
  fill_peers(t, nullptr, flag_ptrs, world);
  node_barrier_kernel<<<1, 32, 0, stream>>>(t, rank, world, base_word, seq, status,
                                            static_cast<unsigned long long>(budget_seconds * 1e9));
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

// dst[n, k] (BF16, local) = cast of the FP32 weight whose rows are sharded over `world` ranks in blocks of
// rows_per_shard; shards[r] is rank r's block as mapped in this process.  `ctas` bounds the SMs used.
extern "C" int ws_gather_cast(const void* const* shards, int world, int rows_per_shard, int n, int k, void* dst,
                              int ctas, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || n <= 0 || k <= 0 || k % 8 != 0 || rows_per_shard <= 0) return -1;
  if ((long long)rows_per_shard * world < n) return -1;
  if ((uintptr_t)dst & 15) return -5;
  GatherTable t;
  for (int r = 0; r < MAX_RANKS; ++r) {
    t.shard[r] = r < world ? static_cast<const float*>(shards[r]) : nullptr;
    if (r < world && (shards[r] == nullptr || ((uintptr_t)shards[r] & 15))) return -5;
  }
  if (ctas < 1) ctas = 1;
  if (ctas > 148 * 4) ctas = 148 * 4;
  gather_cast_kernel<<<ctas, 256, 0, stream>>>(t, rows_per_shard, n, k, static_cast<__nv_bfloat16*>(dst));
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ws_wait_probe(const unsigned* flag, unsigned expected, int* status, double budget_seconds,
                             cudaStream_t stream) {
  wait_probe_kernel<<<1, 32, 0, stream>>>(flag, expected, status, static_cast<unsigned long long>(budget_seconds * 1e9));
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ws_adamw_shard_push(const unsigned long long* master_ptrs, const unsigned long long* bf16_ptrs,
                                   int rank, int world, const float* g, float* m, float* v, size_t lo, size_t n,
                                   float lr, float beta1, float beta2, float eps, float wd, int step,
                                   const float* grad_scale_ptr, int push_master, const float* skip_ptr,
                                   cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || n % 4 != 0 || lo % 4 != 0 || step < 1) return -1;
  if (n == 0) return 0;
  ParamPeers t;
  for (int r = 0; r < MAX_RANKS; ++r) {
    t.master[r] = r < world ? reinterpret_cast<float*>(master_ptrs[r]) : nullptr;
    t.bf16[r] = r < world ? reinterpret_cast<__nv_bfloat16*>(bf16_ptrs[r]) : nullptr;
  }
  const double bias1 = 1.0 - pow((double)beta1, (double)step);
  const double bias2 = 1.0 - pow((double)beta2, (double)step);
  size_t blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  adamw_shard_push_kernel<<<(int)blocks, 256, 0, stream>>>(t, world, g, m, v, lo, n / 4, lr, beta1, beta2, eps, wd,
                                                          (float)bias1, (float)sqrt(bias2), grad_scale_ptr, rank,
                                                          push_master, skip_ptr);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
