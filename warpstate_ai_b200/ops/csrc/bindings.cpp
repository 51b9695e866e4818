// torch.ops.ws_b200.* registrations: argument checking and pointer extraction only; all
// device work is in the .cu files behind the C ABI of ws_api.h.
#include <torch/library.h>
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "ws_api.h"

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "ws_b200::", what, " failed with code ", rc);
}

const void* opt_ptr(const c10::optional<at::Tensor>& t) {
  return t.has_value() && t->defined() ? t->data_ptr() : nullptr;
}
int64_t opt_ld(const c10::optional<at::Tensor>& t) {
  return t.has_value() && t->defined() && t->dim() >= 2 ? t->stride(0) : 0;
}

// Generic GEMM entry.  `a`/`b` are 2-D BF16 tensors whose last dimension is contiguous; the
// caller states how they are to be read (a_mn/b_mn) and the problem size.
void gemm(const at::Tensor& a, const at::Tensor& b, bool a_mn, bool b_mn, int64_t epilogue,
          int64_t m, int64_t n, int64_t k, at::Tensor out, c10::optional<at::Tensor> out2,
          c10::optional<at::Tensor> aux, c10::optional<at::Tensor> row_scale, double alpha,
          double beta, c10::optional<at::Tensor> error_flag) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16,
              "gemm: BF16 operands required");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1,
              "gemm: operands must be 2-D with a contiguous last dimension");
  TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1, "gemm: out must be 2-D row-major");
  const int64_t b_rows = epilogue == WS_EPI_SWIGLU ? 2 * n : n;
  if (!a_mn) { TORCH_CHECK(a.size(0) == m && a.size(1) == k, "gemm: A must be [m,k]"); }
  else { TORCH_CHECK(a.size(0) == k && a.size(1) == m, "gemm: A must be [k,m]"); }
  if (!b_mn) { TORCH_CHECK(b.size(0) == b_rows && b.size(1) == k, "gemm: B must be [n,k]"); }
  else { TORCH_CHECK(b.size(0) == k && b.size(1) == b_rows, "gemm: B must be [k,n]"); }
  const bool f32_out = epilogue == WS_EPI_RESID_F32 || epilogue == WS_EPI_ACC_F32 || epilogue == WS_EPI_F32;
  TORCH_CHECK(out.scalar_type() == (f32_out ? at::kFloat : at::kBFloat16), "gemm: wrong out dtype");
  const int64_t out_cols = (epilogue == WS_EPI_SWIGLU || epilogue == WS_EPI_SWIGLU_BWD) ? 2 * n : n;
  TORCH_CHECK(out.size(0) == m && out.size(1) == out_cols, "gemm: wrong out shape");
  if (row_scale.has_value() && row_scale->defined()) {
    TORCH_CHECK(row_scale->scalar_type() == at::kFloat && row_scale->numel() == m && row_scale->is_contiguous(),
                "gemm: row_scale must be float32 [m]");
  }
  if (epilogue == WS_EPI_RESID_F32) {
    TORCH_CHECK(aux.has_value() && aux->scalar_type() == at::kFloat && aux->size(0) == m && aux->size(1) == n,
                "gemm: residual must be float32 [m,n]");
  }
  if (epilogue == WS_EPI_RESID_BF16) {
    TORCH_CHECK(aux.has_value() && aux->scalar_type() == at::kBFloat16 && aux->size(0) == m && aux->size(1) == n,
                "gemm: residual must be bfloat16 [m,n]");
  }
  if (epilogue == WS_EPI_SWIGLU_BWD) {
    TORCH_CHECK(aux.has_value() && aux->scalar_type() == at::kBFloat16 && aux->size(0) == m && aux->size(1) == 2 * n,
                "gemm: packed (up|gate) must be bfloat16 [m,2n]");
  }
  if (epilogue == WS_EPI_SWIGLU) {
    TORCH_CHECK(out2.has_value() && out2->scalar_type() == at::kBFloat16 && out2->size(0) == m && out2->size(1) == n,
                "gemm: activation output must be bfloat16 [m,n]");
  }

  c10::cuda::CUDAGuard guard(a.device());
  WsGemm g;
  g.a = a.data_ptr(); g.b = b.data_ptr();
  g.m = (int)m; g.n = (int)n; g.k = (int)k;
  g.lda = (int)a.stride(0); g.ldb = (int)b.stride(0);
  g.a_mn = a_mn; g.b_mn = b_mn; g.epilogue = (int)epilogue;
  g.out = out.data_ptr(); g.ldo = (int)out.stride(0);
  g.out2 = const_cast<void*>(opt_ptr(out2)); g.ldo2 = (int)opt_ld(out2);
  g.aux = opt_ptr(aux); g.ldaux = (int)opt_ld(aux);
  g.row_scale = reinterpret_cast<const float*>(opt_ptr(row_scale));
  g.alpha = (float)alpha; g.beta = (float)beta;
  g.error_flag = reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag)));
  check_rc(ws_gemm(&g, cur_stream()), "gemm");
}

}  // namespace

TORCH_LIBRARY(ws_b200, m) {
  m.def("gemm(Tensor a, Tensor b, bool a_mn, bool b_mn, int epilogue, int m, int n, int k, "
        "Tensor(a!) out, Tensor(b!)? out2, Tensor? aux, Tensor? row_scale, float alpha, float beta, "
        "Tensor(c!)? error_flag) -> ()");
}

TORCH_LIBRARY_IMPL(ws_b200, CUDA, m) {
  m.impl("gemm", &gemm);
}
