// C ABI of the sm_100a kernel library.  Every function takes raw device pointers and a CUDA
// stream, launches on that stream and returns 0 on success or a negative error code; none of
// them allocates unless stated.  The torch bindings (bindings.cpp) are a thin layer over these.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ----------------------------------------------------------------------------- GEMM
// C[M,N] = op(A)[M,K] * op(B)[N,K]^T with BF16 operands and FP32 accumulation in TMEM.
//   a_mn == 0: A is stored [M, K] row-major (K contiguous), leading dimension lda.
//   a_mn == 1: A is stored [K, M] row-major (M contiguous), leading dimension lda.
//   b_mn == 0: B is stored [N, K] row-major (the nn.Linear weight layout), ldb.
//   b_mn == 1: B is stored [K, N] row-major (N contiguous), ldb.
enum WsEpilogue {
  WS_EPI_BF16 = 0,        // out_bf16[M,N] = rowscale[m] * acc
  WS_EPI_RESID_F32 = 1,   // out_f32[M,N]  = resid_f32[M,N] + acc
  WS_EPI_SWIGLU = 2,      // B holds [2h, K]; out_bf16[M,2h] = (up|gate), out2_bf16[M,h] = silu(gate)*up
  WS_EPI_ACC_F32 = 3,     // out_f32[M,N]  = beta * out_f32 + alpha * acc
  WS_EPI_SWIGLU_BWD = 4,  // acc = dAct[M,h]; aux_bf16[M,2h] = (up|gate); out_bf16[M,2h] = (dUp|dGate)
  WS_EPI_F32 = 5,         // out_f32[M,N]  = acc
  WS_EPI_RESID_BF16 = 6,  // out_bf16[M,N] = resid_bf16[M,N] + acc   (BF16 residual stream)
};

typedef struct WsGemm {
  const void* a;
  const void* b;
  int m, n, k;  // for SWIGLU: n = h (the activation width); B has 2h rows
  int lda, ldb;
  int a_mn, b_mn;
  int epilogue;
  void* out;
  int ldo;
  void* out2;  // SWIGLU: activation [M,h]
  int ldo2;
  const void* aux;  // RESID: residual; SWIGLU_BWD: packed (up|gate)
  int ldaux;
  const float* row_scale;  // optional per-row multiplier applied to acc (may be NULL)
  float alpha;
  float beta;
  int* error_flag;  // device int; set non-zero if a bounded wait ran out (may be NULL)
} WsGemm;

int ws_gemm(const WsGemm* g, cudaStream_t stream);
// Number of SMs the GEMM may use on this stream's device (0 = all).  Lets a communication
// kernel keep a few SMs for itself while persistent GEMM CTAs fill the rest.
void ws_gemm_set_sm_limit(int sms);

// Number of kernels this library has launched in this process.
long long ws_launch_count(void);

#ifdef __cplusplus
}
#endif
