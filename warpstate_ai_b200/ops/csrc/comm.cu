// Data-parallel communication kernels over NVLink peer memory (one process per GPU; every
// rank maps every other rank's buffers: "symmetric memory").
//
//   grad_allreduce_kernel : two-shot all-reduce of one gradient bucket, in place, fused with
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

__global__ void __launch_bounds__(COMM_THREADS)
grad_allreduce_kernel(PeerTable peers, float* mc_grad, int rank, int world, size_t start, size_t count, int bucket,
                      unsigned seq, float scale, int push, float* sumsq_out, int* status,
                      unsigned long long budget_ns) {
  __shared__ int s_ok;
  __shared__ float s_red[COMM_THREADS / 32];
  const int tid = threadIdx.x;
  if (tid == 0) s_ok = 1;
  __syncthreads();
  // 1. announce that this rank's bucket is final (its producers ran earlier on this stream)
  if (blockIdx.x == 0 && tid < world) {
    __threadfence_system();
    st_release_sys(peers.flags[tid] + ready_index(bucket, rank), seq);
  }
  // 2. wait for every rank's announcement
  if (tid < world) {
    if (!wait_at_least(peers.flags[rank] + ready_index(bucket, tid), seq, budget_ns, status, 1, bucket, tid))
      s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;

  // 3. reduce my slice, scale, push
  const size_t n4 = count / 4;
  const size_t per = (n4 + world - 1) / world;
  const size_t lo = per * rank;
  size_t hi = lo + per;
  if (hi > n4) hi = n4;
  float ss = 0.f;
  // Four independent 16-byte pieces per thread and pass: a peer or multimem load takes microseconds, and
  // with one piece in flight per thread the kernel's bandwidth is set by its CTA count (6.7 GB/s per CTA
  // measured).  The element-to-thread mapping and the order in which a thread adds its pieces (to the
  // reduction and to the sum of squares) are those of the one-piece loop, so results are unchanged.
  constexpr int U = 4;
  const size_t stride = static_cast<size_t>(gridDim.x) * COMM_THREADS;
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
  // sum-of-squares partial of this CTA (fixed order inside the CTA; CTAs are combined by the host op)
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
  // 4. tell every rank that this CTA's share of slice `rank` has landed
  __threadfence_system();
  __syncthreads();
  if (tid < world) red_release_sys_add(peers.flags[tid] + done_index(bucket, rank), 1u);
  // 5. one CTA waits until every rank has finished reading from and writing to this rank's buffer
  if (blockIdx.x == 0 && tid < world)
    wait_at_least(peers.flags[rank] + done_index(bucket, tid), seq * gridDim.x, budget_ns, status, 2, bucket, tid);
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
                        int rank, int push_master) {
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

// grad_ptrs / flag_ptrs: `world` device addresses (this process's mappings of every rank's
// buffers, own rank included).  mc_grad: multimem address of the gradient arena or NULL.
// sumsq_out: `ctas` floats (may be NULL).  status: 8 ints on the device.
// `seq` counts the calls on this bucket from 1, on every rank alike, and `ctas` must be the same in every
// call on a bucket: its completion counter advances by `ctas` per call and a rank waits for seq * ctas.
// (A different CTA count needs a bucket of its own; a mismatch ends in a reported time-out, code 2.)
extern "C" int ws_grad_allreduce(const unsigned long long* grad_ptrs, const unsigned long long* flag_ptrs,
                                 unsigned long long mc_grad, int rank, int world, size_t start, size_t count,
                                 int bucket, unsigned seq, float scale, int push, int ctas, float* sumsq_out,
                                 int* status, double budget_seconds, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || count % 4 != 0 || start % 4 != 0) return -1;
  if (ctas < 1 || ctas > ws_comm_max_ctas()) return -2;
  PeerTable t;
  for (int r = 0; r < MAX_RANKS; ++r) {
    t.grad[r] = r < world ? reinterpret_cast<float*>(grad_ptrs[r]) : nullptr;
    t.flags[r] = r < world ? reinterpret_cast<unsigned*>(flag_ptrs[r]) : nullptr;
  }
  grad_allreduce_kernel<<<ctas, COMM_THREADS, 0, stream>>>(
      t, reinterpret_cast<float*>(mc_grad), rank, world, start, count, bucket, seq, scale, push, sumsq_out, status,
      static_cast<unsigned long long>(budget_seconds * 1e9));
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
                                   const float* grad_scale_ptr, int push_master, cudaStream_t stream) {
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
                                                          push_master);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
