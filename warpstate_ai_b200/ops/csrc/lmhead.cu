// LM-head cross-entropy helpers.  The vocabulary projection itself runs in the tcgen05 GEMM with
// the WS_EPI_CE_FWD / WS_EPI_CE_BWD epilogues (gemm_tcgen05.cu), so the [tokens, vocab] logits
// never reach HBM in the forward pass; this file combines the per-128-column (max, sum exp)
// partials of a row into its log-sum-exp and label log-probability.
//
// Replaces the reference's chunked / full LM-head losses (warpstate/model.py:316-334,
// ops/loss_experiment.py:14-19: BF16 head GEMM, FP32 cast of the logits, log-softmax, NLL) and
// the per-sequence log-probability head of DPO (dpo.py:150-161).
#include "ws_ptx.cuh"
#include "ws_api.h"
#include "ws_launch.h"

namespace ws {

extern "C" void ws_count_launch(void);

// One warp per row.  parts: float2 [rows, ld] with `nparts` valid entries per row.
// lse[row] = log sum_j exp(logit_j);  logp[row] = label_logit - lse (0 where label == ignore).
__global__ void __launch_bounds__(256)
ce_combine_kernel(const float2* __restrict__ parts, int ld, int nparts, const float* __restrict__ label_logit,
                  const long long* __restrict__ labels, long long ignore_index, int rows,
                  float* __restrict__ lse_out, float* __restrict__ logp_out) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const float2* pr = parts + static_cast<size_t>(row) * ld;
  float mx = -INFINITY;
  for (int i = lane; i < nparts; i += 32) mx = fmaxf(mx, pr[i].x);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float s = 0.f;
  for (int i = lane; i < nparts; i += 32) {
    const float2 v = pr[i];
    s += v.y * expf(v.x - mx);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    const float lse = mx + logf(s);
    lse_out[row] = lse;
    const long long lab = labels[row];
    logp_out[row] = (lab == ignore_index) ? 0.f : label_logit[row] - lse;
  }
}

}  // namespace ws

using namespace ws;

extern "C" int ws_ce_combine(const void* parts, int ld, int nparts, const float* label_logit,
                             const long long* labels, long long ignore_index, int rows, float* lse,
                             float* logp, cudaStream_t stream) {
  if (rows <= 0 || nparts <= 0) return -1;
  launch_dependent(ce_combine_kernel, dim3((rows + 7) / 8), dim3(256), 0, stream, reinterpret_cast<const float2*>(parts), ld, nparts,
                                                         label_logit, labels, ignore_index, rows, lse, logp);
  ws_count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
