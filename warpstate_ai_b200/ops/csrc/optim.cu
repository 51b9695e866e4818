// Flat-buffer optimizer kernels: global gradient norm (two deterministic stages), the clip
// coefficient kept on the device, and AdamW over FP32 master / gradient / moment arenas with the
// BF16 compute copy of the weights refreshed in the same pass.
//
// Replaces, for the whole model in three launches per step: torch's clip_grad_norm_ (foreach
// norms + scale), AdamW(fused=True) (reference run_40b.py:534-535,751-752) and the FP32->BF16
// weight casts that autocast repeats every micro-batch (run_40b.py:744).
#include "ws_ptx.cuh"
#include "ws_api.h"

namespace ws {

extern "C" void ws_count_launch(void);

constexpr int OPT_THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float s = 0.f;
  if (warp == 0) {
    s = lane < (blockDim.x >> 5) ? smem[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  }
  __syncthreads();
  return s;  // valid in warp 0
}

// partial[block] = sum of squares of a fixed, contiguous slice of g (slice size is a function
// of n and gridDim only, so the summation order is reproducible).
__global__ void __launch_bounds__(OPT_THREADS)
sumsq_kernel(const float* __restrict__ g, size_t n4, float* __restrict__ partial) {
  __shared__ float red[32];
  const size_t per_block = (n4 + gridDim.x - 1) / gridDim.x;
  const size_t begin = per_block * blockIdx.x;
  size_t end = begin + per_block;
  if (end > n4) end = n4;
  float s = 0.f;
  for (size_t i = begin + threadIdx.x; i < end; i += OPT_THREADS) {
    const float4 v = reinterpret_cast<const float4*>(g)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__device__ __forceinline__ bool not_finite(float x) { return (__float_as_uint(x) & 0x7f800000u) == 0x7f800000u; }

// stats[0] = ||g||, stats[1] = clip coefficient min(1, max_norm/(||g||+1e-6)), stats[2] = ||g||^2,
// stats[3] = skip flag: 1 when the norm is not finite or `status` (optional device word of a
// communication kernel, 0 = no error) is non-zero.  The update kernels return without touching
// parameters or moments when the flag is set, so a caller that raises on the host afterwards
// still holds the state of the previous update.
// `extra_sumsq` (optional) is added first: other ranks' shares when the gradient is sharded.
__global__ void clip_coef_kernel(const float* __restrict__ partial, int parts, const float* extra_sumsq,
                                 float max_norm, const int* __restrict__ status, float* __restrict__ stats) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < parts; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    if (extra_sumsq != nullptr) s += *extra_sumsq;
    const float norm = __fsqrt_rn(s);
    float coef = max_norm > 0.f ? __fdiv_rn(max_norm, norm + 1e-6f) : 1.0f;
    if (coef > 1.0f) coef = 1.0f;
    const bool bad = not_finite(norm) || (status != nullptr && *status != 0);
    stats[0] = norm;
    stats[1] = bad ? 0.0f : coef;
    stats[2] = s;
    stats[3] = bad ? 1.0f : 0.0f;
  }
}

// AdamW with decoupled weight decay, bias correction and gradient pre-scaling (clip coefficient
// read from the device).  Operation order matches torch.optim.AdamW:
//   p *= 1 - lr*wd ; m = lerp(m, g, 1-b1) ; v = b2*v + (1-b2) g^2 ;
//   p -= (lr/bias1) * m / (sqrt(v)/sqrt(bias2) + eps)
__global__ void __launch_bounds__(OPT_THREADS)
adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
             float* __restrict__ v, __nv_bfloat16* __restrict__ p_bf16, size_t n4, float lr, float beta1,
             float beta2, float eps, float wd, float bias1, float bias2_sqrt,
             const float* __restrict__ grad_scale_ptr, float grad_scale_const,
             const float* __restrict__ skip_ptr) {
  if (skip_ptr != nullptr && *skip_ptr != 0.0f) return;  // non-finite norm or failed gradient exchange
  const float gs = (grad_scale_ptr != nullptr ? *grad_scale_ptr : 1.0f) * grad_scale_const;
  const float decay = 1.0f - lr * wd;
  const float step_size = lr / bias1;
  for (size_t i = blockIdx.x * static_cast<size_t>(OPT_THREADS) + threadIdx.x; i < n4;
       i += static_cast<size_t>(gridDim.x) * OPT_THREADS) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 gg = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* pa = reinterpret_cast<float*>(&pp);
    float* ga = reinterpret_cast<float*>(&gg);
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
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (p_bf16 != nullptr) {
      uint2 o;
      o.x = pack_bf16x2(pa[0], pa[1]);
      o.y = pack_bf16x2(pa[2], pa[3]);
      reinterpret_cast<uint2*>(p_bf16)[i] = o;
    }
  }
}

}  // namespace ws

using namespace ws;

extern "C" int ws_sumsq_parts(void) { return 148 * 8; }

// stats: 4 floats on the device.  partial: ws_sumsq_parts() floats of scratch.
extern "C" int ws_grad_norm_clip(const float* g, size_t n, float* partial, const float* extra_sumsq,
                                 float max_norm, const int* status, float* stats, cudaStream_t stream) {
  if (n % 4 != 0) return -1;
  const int parts = ws_sumsq_parts();
  sumsq_kernel<<<parts, OPT_THREADS, 0, stream>>>(g, n / 4, partial);
  ws_count_launch();
  clip_coef_kernel<<<1, 256, 0, stream>>>(partial, parts, extra_sumsq, max_norm, status, stats);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// The same statistics from `parts` partial sums of squares that other kernels produced.
extern "C" int ws_clip_from_partials(const float* partial, int parts, const float* extra_sumsq, float max_norm,
                                     const int* status, float* stats, cudaStream_t stream) {
  if (parts < 1) return -1;
  clip_coef_kernel<<<1, 256, 0, stream>>>(partial, parts, extra_sumsq, max_norm, status, stats);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int ws_adamw(float* p, const float* g, float* m, float* v, void* p_bf16, size_t n, float lr,
                        float beta1, float beta2, float eps, float wd, int step, const float* grad_scale_ptr,
                        float grad_scale_const, const float* skip_ptr, cudaStream_t stream) {
  if (n % 4 != 0 || step < 1) return -1;
  if (n == 0) return 0;
  const double bias1 = 1.0 - pow((double)beta1, (double)step);
  const double bias2 = 1.0 - pow((double)beta2, (double)step);
  size_t blocks = (n / 4 + OPT_THREADS - 1) / OPT_THREADS;
  if (blocks > 148 * 16) blocks = 148 * 16;
  adamw_kernel<<<(int)blocks, OPT_THREADS, 0, stream>>>(p, g, m, v, (__nv_bfloat16*)p_bf16, n / 4, lr, beta1,
                                                       beta2, eps, wd, (float)bias1, (float)sqrt(bias2),
                                                       grad_scale_ptr, grad_scale_const, skip_ptr);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
