// torch.ops.ws_b200.* registrations: argument checking and pointer extraction only; all
// device work is in the .cu files behind the C ABI of ws_api.h.
#include <cstdio>
#include <torch/library.h>
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <string>
#include <vector>

#include "ws_api.h"

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// The message is built as a std::string first: passing the `const char*` and the int straight
// to TORCH_CHECK's variadic formatter crashed the process (SIGSEGV) instead of throwing.
void check_rc(int rc, const char* what) {
  if (rc != 0) {
    const std::string message = std::string("ws_b200::") + what + " failed with code " + std::to_string(rc);
    TORCH_CHECK(false, message);
  }
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
  // TMA needs 16-byte aligned bases and row pitches (8 BF16 elements).
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0 &&
              reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0,
              "gemm: operand row pitches must be multiples of 8 elements and bases 16-byte aligned");
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
  g.row_vec = nullptr;
  g.alpha = (float)alpha; g.beta = (float)beta;
  g.error_flag = reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag)));
  const int rc = ws_gemm(&g, cur_stream());
  if (rc != 0) {  // name the problem: a bare code is of little use for a tensor-map or shape refusal
    char what[256];
    snprintf(what, sizeof(what), "gemm (m=%lld n=%lld k=%lld a_mn=%d b_mn=%d epilogue=%lld lda=%d ldb=%d ldo=%d)",
             (long long)m, (long long)n, (long long)k, (int)a_mn, (int)b_mn, (long long)epilogue, g.lda, g.ldb, g.ldo);
    check_rc(rc, what);
  }
}

// grads[i] = beta[i] * grads[i] + dy[i]^T x[i]  (FP32), all problems in one persistent launch
// when the CTA-pair kernel can take them (up to four with >= 256 output rows each).
void grad_weight_group(at::TensorList dys, at::TensorList xs, at::TensorList grads,
                       at::ArrayRef<double> betas, c10::optional<at::Tensor> error_flag) {
  const size_t count = dys.size();
  TORCH_CHECK(count > 0 && xs.size() == count && grads.size() == count && betas.size() == count,
              "grad_weight_group: list lengths differ");
  std::vector<WsGemm> items(count);
  for (size_t i = 0; i < count; ++i) {
    const at::Tensor& dy = dys[i];
    const at::Tensor& x = xs[i];
    const at::Tensor& grad = grads[i];
    TORCH_CHECK(dy.is_cuda() && x.is_cuda() && grad.is_cuda() && dy.device() == dys[0].device(),
                "grad_weight_group: CUDA tensors on one device required");
    TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && x.scalar_type() == at::kBFloat16 && grad.scalar_type() == at::kFloat,
                "grad_weight_group: BF16 operands and FP32 gradients required");
    TORCH_CHECK(dy.dim() == 2 && x.dim() == 2 && grad.dim() == 2 && dy.stride(1) == 1 && x.stride(1) == 1 &&
                grad.stride(1) == 1, "grad_weight_group: 2-D tensors with a contiguous last dimension required");
    TORCH_CHECK(dy.size(0) == x.size(0) && grad.size(0) == dy.size(1) && grad.size(1) == x.size(1),
                "grad_weight_group: shapes must be dy [T,N], x [T,K], grad [N,K]");
    TORCH_CHECK(dy.stride(0) % 8 == 0 && x.stride(0) % 8 == 0 &&
                reinterpret_cast<uintptr_t>(dy.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0,
                "grad_weight_group: operand row pitches must be multiples of 8 elements and bases 16-byte aligned");
    WsGemm& g = items[i];
    g.a = dy.data_ptr(); g.b = x.data_ptr();
    g.m = (int)dy.size(1); g.n = (int)x.size(1); g.k = (int)dy.size(0);
    g.lda = (int)dy.stride(0); g.ldb = (int)x.stride(0);
    g.a_mn = true; g.b_mn = true; g.epilogue = WS_EPI_ACC_F32;
    g.out = grad.data_ptr(); g.ldo = (int)grad.stride(0);
    g.out2 = nullptr; g.ldo2 = 0;
    g.aux = nullptr; g.ldaux = 0;
    g.row_scale = nullptr; g.row_vec = nullptr;
    g.alpha = 1.0f; g.beta = (float)betas[i];
    g.error_flag = reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag)));
  }
  c10::cuda::CUDAGuard guard(dys[0].device());
  check_rc(ws_gemm_group(items.data(), (int)count, cur_stream()), "grad_weight_group");
}

// ----------------------------------------------------------------------------- row kernels
std::tuple<at::Tensor, at::Tensor, at::Tensor> rmsnorm_fwd(const at::Tensor& x,
                                                           const c10::optional<at::Tensor>& col_scale,
                                                           const c10::optional<at::Tensor>& col_bias,
                                                           const at::Tensor& w, double eps, bool want_xmod) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous(), "rmsnorm_fwd: x must be contiguous [rows,d]");
  TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16, "rmsnorm_fwd: x dtype");
  TORCH_CHECK(w.scalar_type() == at::kFloat && w.is_contiguous() && w.numel() == x.size(1), "rmsnorm_fwd: w");
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = (int)x.size(0), d = (int)x.size(1);
  const bool mod = col_scale.has_value() && col_scale->defined();
  if (mod) {
    TORCH_CHECK(col_scale->scalar_type() == at::kFloat && col_scale->is_contiguous() && col_scale->numel() == d &&
                col_bias.has_value() && col_bias->scalar_type() == at::kFloat && col_bias->is_contiguous() &&
                col_bias->numel() == d, "rmsnorm_fwd: depth modulation vectors must be float32 [d]");
  }
  at::Tensor z = at::empty({rows, d}, x.options().dtype(at::kBFloat16));
  at::Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  at::Tensor xmod = (mod && want_xmod) ? at::empty_like(x) : at::Tensor();
  check_rc(ws_rmsnorm_fwd(x.data_ptr(), x.scalar_type() == at::kBFloat16,
                          mod ? col_scale->data_ptr<float>() : nullptr,
                          mod ? col_bias->data_ptr<float>() : nullptr, w.data_ptr<float>(), (float)eps, rows, d,
                          xmod.defined() ? xmod.data_ptr() : nullptr, z.data_ptr(), rstd.data_ptr<float>(),
                          cur_stream()), "rmsnorm_fwd");
  return {z, rstd, xmod.defined() ? xmod : x};
}

// returns (dx, dx_bf16, dw) ; dw is the finished column sum [d]
std::tuple<at::Tensor, at::Tensor, at::Tensor> rmsnorm_bwd(const at::Tensor& dz, const at::Tensor& x,
                                                           const at::Tensor& rstd, const at::Tensor& w,
                                                           const c10::optional<at::Tensor>& dres,
                                                           const c10::optional<at::Tensor>& out_scale,
                                                           bool want_bf16) {
  TORCH_CHECK(dz.is_cuda() && dz.scalar_type() == at::kBFloat16 && dz.is_contiguous(), "rmsnorm_bwd: dz");
  TORCH_CHECK(x.is_contiguous() && x.sizes() == dz.sizes(), "rmsnorm_bwd: x");
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = (int)x.size(0), d = (int)x.size(1);
  const bool has_res = dres.has_value() && dres->defined();
  if (has_res) { TORCH_CHECK(dres->scalar_type() == x.scalar_type() && dres->is_contiguous() && dres->sizes() == x.sizes(), "rmsnorm_bwd: dres"); }
  const bool has_scale = out_scale.has_value() && out_scale->defined();
  at::Tensor dx = at::empty_like(x);
  at::Tensor dxb = want_bf16 ? at::empty({rows, d}, x.options().dtype(at::kBFloat16)) : at::Tensor();
  const int parts = ws_rmsnorm_bwd_parts(rows);
  at::Tensor partial = at::empty({parts, d}, x.options().dtype(at::kFloat));
  check_rc(ws_rmsnorm_bwd(dz.data_ptr(), x.data_ptr(), x.scalar_type() == at::kBFloat16, rstd.data_ptr<float>(),
                          w.data_ptr<float>(), has_res ? dres->data_ptr() : nullptr,
                          has_scale ? out_scale->data_ptr<float>() : nullptr, rows, d, dx.data_ptr(),
                          want_bf16 ? dxb.data_ptr() : nullptr, partial.data_ptr<float>(), cur_stream()),
           "rmsnorm_bwd");
  at::Tensor dw = at::empty({d}, x.options().dtype(at::kFloat));
  check_rc(ws_colsum_finalize(partial.data_ptr<float>(), parts, d, nullptr, 0.f, dw.data_ptr<float>(), cur_stream()),
           "colsum_finalize");
  return {dx, dxb, dw};
}

// (sum_rows a / (1+inv_scale), sum_rows a*b / (1+inv_scale))
std::tuple<at::Tensor, at::Tensor> colsum2(const at::Tensor& a, const at::Tensor& b,
                                           const c10::optional<at::Tensor>& inv_scale) {
  TORCH_CHECK(a.is_cuda() && a.is_contiguous() && b.is_contiguous() && a.sizes() == b.sizes() &&
              a.scalar_type() == b.scalar_type(), "colsum2: a, b");
  c10::cuda::CUDAGuard guard(a.device());
  const int rows = (int)a.size(0), d = (int)a.size(1);
  const int parts = ws_colsum_parts(rows);
  at::Tensor pa = at::empty({parts, d}, a.options().dtype(at::kFloat));
  at::Tensor pab = at::empty({parts, d}, a.options().dtype(at::kFloat));
  check_rc(ws_colsum2(a.data_ptr(), b.data_ptr(), a.scalar_type() == at::kBFloat16, rows, d, pa.data_ptr<float>(),
                      pab.data_ptr<float>(), cur_stream()), "colsum2");
  at::Tensor sa = at::empty({d}, a.options().dtype(at::kFloat));
  at::Tensor sab = at::empty({d}, a.options().dtype(at::kFloat));
  const float* inv = inv_scale.has_value() && inv_scale->defined() ? inv_scale->data_ptr<float>() : nullptr;
  check_rc(ws_colsum_finalize(pa.data_ptr<float>(), parts, d, inv, 0.f, sa.data_ptr<float>(), cur_stream()), "colsum_finalize");
  check_rc(ws_colsum_finalize(pab.data_ptr<float>(), parts, d, inv, 0.f, sab.data_ptr<float>(), cur_stream()), "colsum_finalize");
  return {sa, sab};
}

at::Tensor cast_bf16(const at::Tensor& x, c10::optional<at::Tensor> out) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous(), "cast_bf16: x");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor o = out.has_value() && out->defined() ? *out : at::empty(x.sizes(), x.options().dtype(at::kBFloat16));
  TORCH_CHECK(o.scalar_type() == at::kBFloat16 && o.is_contiguous() && o.numel() == x.numel(), "cast_bf16: out");
  if (x.numel() % 4 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0) &&
      (reinterpret_cast<uintptr_t>(o.data_ptr()) % 8 == 0)) {
    check_rc(ws_cast_f32_bf16(x.data_ptr<float>(), o.data_ptr(), (size_t)x.numel(), cur_stream()), "cast_bf16");
  } else {
    o.copy_(x);
  }
  return o;
}

at::Tensor embed_fwd(const at::Tensor& ids, const at::Tensor& table, bool out_bf16) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "embed_fwd: ids");
  TORCH_CHECK(table.dim() == 2 && table.is_contiguous(), "embed_fwd: table");
  c10::cuda::CUDAGuard guard(table.device());
  const int rows = (int)ids.numel(), d = (int)table.size(1);
  at::Tensor out = at::empty({rows, d}, table.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
  check_rc(ws_embed_fwd(ids.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()) : nullptr,
                        table.data_ptr(), table.scalar_type() == at::kBFloat16, rows, d, (int)table.size(0),
                        out.data_ptr(), out_bf16, cur_stream()), "embed_fwd");
  return out;
}

// grad_table [V,d] FP32 += scatter of dx rows by token id, deterministic (sorted segments).
void embed_bwd(const at::Tensor& dx, const at::Tensor& ids, at::Tensor grad_table) {
  TORCH_CHECK(dx.is_cuda() && dx.dim() == 2 && dx.is_contiguous(), "embed_bwd: dx");
  TORCH_CHECK(grad_table.scalar_type() == at::kFloat && grad_table.is_contiguous(), "embed_bwd: grad_table");
  c10::cuda::CUDAGuard guard(dx.device());
  const int rows = (int)dx.size(0), d = (int)dx.size(1);
  at::Tensor flat = ids.reshape({-1});
  auto sorted = flat.sort(/*stable=*/true, /*dim=*/0, /*descending=*/false);
  at::Tensor sorted_ids = std::get<0>(sorted).contiguous();
  at::Tensor order = std::get<1>(sorted).contiguous();
  TORCH_CHECK(grad_table.dim() == 2 && grad_table.size(1) == d && flat.numel() == rows, "embed_bwd: shapes");
  // the runs of equal ids are found by the kernel: no host-side count, no device-to-host read
  check_rc(ws_embed_bwd(dx.data_ptr(), dx.scalar_type() == at::kBFloat16,
                        reinterpret_cast<const long long*>(sorted_ids.data_ptr<int64_t>()),
                        reinterpret_cast<const long long*>(order.data_ptr<int64_t>()), rows, d,
                        (int)grad_table.size(0), grad_table.data_ptr<float>(), cur_stream()), "embed_bwd");
}

// ----------------------------------------------------------------------------- attention / memory
void check_qkvgu(const at::Tensor& qkvgu, int64_t B, int64_t T, int64_t H) {
  TORCH_CHECK(qkvgu.is_cuda() && qkvgu.scalar_type() == at::kBFloat16 && qkvgu.is_contiguous() && qkvgu.dim() == 2,
              "attention: qkvgu must be contiguous BF16 [B*T, 5d]");
  TORCH_CHECK(qkvgu.size(0) == B * T && qkvgu.size(1) == 5 * H * 64 && T % 128 == 0,
              "attention: shape mismatch (chunk 128, head_dim 64)");
}

at::Tensor chunk_writes(const at::Tensor& qkvgu, const at::Tensor& rope, int64_t B, int64_t T, int64_t H,
                        const c10::optional<at::Tensor>& error_flag) {
  check_qkvgu(qkvgu, B, T, H);
  TORCH_CHECK(rope.scalar_type() == at::kFloat && rope.is_contiguous() && rope.numel() == 128 * 64, "rope table");
  c10::cuda::CUDAGuard guard(qkvgu.device());
  at::Tensor writes = at::empty({B, T / 128, H, 64, 64}, qkvgu.options().dtype(at::kFloat));
  check_rc(ws_chunk_writes(qkvgu.data_ptr(), rope.data_ptr<float>(), writes.data_ptr<float>(), (int)B, (int)T,
                           (int)H, (int)(H * 64), reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag))),
                           cur_stream()), "chunk_writes");
  return writes;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> memory_scan(const at::Tensor& writes, const at::Tensor& fast_logit,
                                                           const at::Tensor& slow_logit, const at::Tensor& mix_logit,
                                                           bool want_states, bool want_final,
                                                           const c10::optional<at::Tensor>& init_fast,
                                                           const c10::optional<at::Tensor>& init_slow) {
  TORCH_CHECK(writes.is_cuda() && writes.scalar_type() == at::kFloat && writes.is_contiguous() && writes.dim() == 5,
              "memory_scan: writes must be FP32 [B,N,H,64,64]");
  const int B = (int)writes.size(0), N = (int)writes.size(1), H = (int)writes.size(2);
  for (const at::Tensor* t : {&fast_logit, &slow_logit, &mix_logit})
    TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == H, "memory_scan: logits");
  c10::cuda::CUDAGuard guard(writes.device());
  at::Tensor states = want_states ? at::empty(writes.sizes(), writes.options().dtype(at::kBFloat16)) : at::Tensor();
  at::Tensor ff = want_final ? at::empty({B, H, 64, 64}, writes.options()) : at::Tensor();
  at::Tensor fs = want_final ? at::empty({B, H, 64, 64}, writes.options()) : at::Tensor();
  const float* i_f = init_fast.has_value() && init_fast->defined() ? init_fast->data_ptr<float>() : nullptr;
  const float* i_s = init_slow.has_value() && init_slow->defined() ? init_slow->data_ptr<float>() : nullptr;
  check_rc(ws_memory_scan(writes.data_ptr<float>(), fast_logit.data_ptr<float>(), slow_logit.data_ptr<float>(),
                          mix_logit.data_ptr<float>(), want_states ? states.data_ptr() : nullptr,
                          want_final ? ff.data_ptr<float>() : nullptr, want_final ? fs.data_ptr<float>() : nullptr,
                          i_f, i_s, B, N, H, cur_stream()), "memory_scan");
  return {states, ff, fs};
}

at::Tensor attn_fwd(const at::Tensor& qkvgu, const at::Tensor& states, const at::Tensor& rope, int64_t B, int64_t T,
                    int64_t H, const c10::optional<at::Tensor>& error_flag) {
  check_qkvgu(qkvgu, B, T, H);
  TORCH_CHECK(states.scalar_type() == at::kBFloat16 && states.is_contiguous() &&
              states.numel() == B * (T / 128) * H * 4096, "attn_fwd: states");
  c10::cuda::CUDAGuard guard(qkvgu.device());
  at::Tensor y = at::empty({B * T, H * 64}, qkvgu.options());
  check_rc(ws_attn_fwd(qkvgu.data_ptr(), states.data_ptr(), rope.data_ptr<float>(), y.data_ptr(), (int)B, (int)T,
                       (int)H, (int)(H * 64), reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag))),
                       cur_stream()), "attn_fwd");
  return y;
}

// returns (dqkvgu [M,5d] BF16, partials [B*H*16,3] FP32)
std::tuple<at::Tensor, at::Tensor> attn_bwd(const at::Tensor& qkvgu, const at::Tensor& dy, const at::Tensor& states,
                                            const at::Tensor& writes, const at::Tensor& rope,
                                            const at::Tensor& fast_logit, const at::Tensor& slow_logit,
                                            const at::Tensor& mix_logit, int64_t B, int64_t T, int64_t H,
                                            const c10::optional<at::Tensor>& error_flag) {
  check_qkvgu(qkvgu, B, T, H);
  const int64_t d = H * 64, N = T / 128;
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && dy.numel() == B * T * d,
              "attn_bwd: dy must be contiguous BF16 [B*T, d]");
  TORCH_CHECK(states.scalar_type() == at::kBFloat16 && states.is_contiguous() && states.numel() == B * N * H * 4096,
              "attn_bwd: states");
  TORCH_CHECK(writes.scalar_type() == at::kFloat && writes.is_contiguous() && writes.numel() == B * N * H * 4096,
              "attn_bwd: writes");
  TORCH_CHECK(N <= 256, "attn_bwd: at most 256 chunks (32768 tokens) per sequence");
  c10::cuda::CUDAGuard guard(qkvgu.device());
  int* err = reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag)));
  at::Tensor dstate = at::empty({B, N, H, 64, 64}, qkvgu.options().dtype(at::kFloat));
  check_rc(ws_attn_dstate(qkvgu.data_ptr(), dy.data_ptr(), rope.data_ptr<float>(), dstate.data_ptr<float>(), (int)B,
                          (int)T, (int)H, (int)d, err, cur_stream()), "attn_dstate");
  at::Tensor dwrites = at::empty({B, N, H, 64, 64}, qkvgu.options());
  at::Tensor partials = at::empty({B * H * 16, 3}, qkvgu.options().dtype(at::kFloat));
  check_rc(ws_memory_scan_bwd(dstate.data_ptr<float>(), writes.data_ptr<float>(), fast_logit.data_ptr<float>(),
                              slow_logit.data_ptr<float>(), mix_logit.data_ptr<float>(), dwrites.data_ptr(),
                              partials.data_ptr<float>(), (int)B, (int)N, (int)H, cur_stream()), "memory_scan_bwd");
  at::Tensor dqkvgu = at::empty_like(qkvgu);
  check_rc(ws_attn_bwd(qkvgu.data_ptr(), states.data_ptr(), dy.data_ptr(), dwrites.data_ptr(), rope.data_ptr<float>(),
                       dqkvgu.data_ptr(), (int)B, (int)T, (int)H, (int)d, err, cur_stream()), "attn_bwd");
  return {dqkvgu, partials};
}

// ----------------------------------------------------------------------------- optimizer
static const int* opt_status(const c10::optional<at::Tensor>& status) {
  if (!status.has_value() || !status->defined()) return nullptr;
  TORCH_CHECK(status->is_cuda() && status->scalar_type() == at::kInt && status->numel() >= 1, "status: int32 CUDA tensor");
  return status->data_ptr<int>();
}
static const float* opt_f32(const c10::optional<at::Tensor>& t, const char* what) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->numel() >= 1, what);
  return t->data_ptr<float>();
}

// -> stats [8] FP32: norm, clip coefficient, norm^2, skip flag (the rest is zero)
at::Tensor grad_norm_clip(const at::Tensor& g, double max_norm, const c10::optional<at::Tensor>& extra_sumsq,
                          const c10::optional<at::Tensor>& status) {
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == at::kFloat && g.is_contiguous() && g.numel() % 4 == 0,
              "grad_norm_clip: flat float32 buffer with numel % 4 == 0 required");
  c10::cuda::CUDAGuard guard(g.device());
  at::Tensor partial = at::empty({ws_sumsq_parts()}, g.options());
  at::Tensor stats = at::zeros({8}, g.options());
  check_rc(ws_grad_norm_clip(g.data_ptr<float>(), (size_t)g.numel(), partial.data_ptr<float>(),
                             opt_f32(extra_sumsq, "grad_norm_clip: extra_sumsq"), (float)max_norm, opt_status(status),
                             stats.data_ptr<float>(), cur_stream()), "grad_norm_clip");
  return stats;
}

at::Tensor clip_from_partials(const at::Tensor& partial, double max_norm, const c10::optional<at::Tensor>& extra_sumsq,
                              const c10::optional<at::Tensor>& status) {
  TORCH_CHECK(partial.is_cuda() && partial.scalar_type() == at::kFloat && partial.is_contiguous() && partial.numel() >= 1,
              "clip_from_partials: float32 CUDA partial sums required");
  c10::cuda::CUDAGuard guard(partial.device());
  at::Tensor stats = at::zeros({8}, partial.options());
  check_rc(ws_clip_from_partials(partial.data_ptr<float>(), (int)partial.numel(),
                                 opt_f32(extra_sumsq, "clip_from_partials: extra_sumsq"), (float)max_norm,
                                 opt_status(status), stats.data_ptr<float>(), cur_stream()), "clip_from_partials");
  return stats;
}

void adamw_step(at::Tensor p, const at::Tensor& g, at::Tensor m, at::Tensor v, c10::optional<at::Tensor> p_bf16,
                double lr, double beta1, double beta2, double eps, double wd, int64_t step,
                const c10::optional<at::Tensor>& grad_scale, double grad_scale_const,
                const c10::optional<at::Tensor>& skip) {
  TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kFloat && p.is_contiguous(), "adamw_step: p");
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel(), "adamw_step: sizes");
  TORCH_CHECK(g.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat &&
              g.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adamw_step: float32 contiguous");
  c10::cuda::CUDAGuard guard(p.device());
  void* pb = nullptr;
  if (p_bf16.has_value() && p_bf16->defined()) {
    TORCH_CHECK(p_bf16->scalar_type() == at::kBFloat16 && p_bf16->numel() == p.numel() && p_bf16->is_contiguous(),
                "adamw_step: p_bf16");
    pb = p_bf16->data_ptr();
  }
  const float* gs = grad_scale.has_value() && grad_scale->defined() ? grad_scale->data_ptr<float>() : nullptr;
  check_rc(ws_adamw(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), pb,
                    (size_t)p.numel(), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd, (int)step, gs,
                    (float)grad_scale_const, opt_f32(skip, "adamw_step: skip"), cur_stream()), "adamw_step");
}

int64_t launch_count() { return (int64_t)ws_launch_count(); }

// ----------------------------------------------------------------------------- LM head
// (lse [rows], logp [rows]) of hidden @ weight.T against labels; logits stay on chip.
std::tuple<at::Tensor, at::Tensor> lm_head_fwd(const at::Tensor& hidden, const at::Tensor& weight,
                                               const at::Tensor& labels, int64_t ignore_index,
                                               const c10::optional<at::Tensor>& error_flag) {
  TORCH_CHECK(hidden.is_cuda() && hidden.scalar_type() == at::kBFloat16 && hidden.dim() == 2 && hidden.stride(1) == 1,
              "lm_head_fwd: hidden must be BF16 [rows, d]");
  TORCH_CHECK(weight.scalar_type() == at::kBFloat16 && weight.dim() == 2 && weight.is_contiguous() &&
              weight.size(1) == hidden.size(1), "lm_head_fwd: weight must be BF16 [vocab, d]");
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == hidden.size(0),
              "lm_head_fwd: labels must be int64 [rows]");
  c10::cuda::CUDAGuard guard(hidden.device());
  const int rows = (int)hidden.size(0), d = (int)hidden.size(1), vocab = (int)weight.size(0);
  const int nparts = 2 * ((vocab + 255) / 256) - (((vocab % 256) != 0 && (vocab % 256) <= 128) ? 1 : 0);
  const int ld = 2 * ((vocab + 255) / 256);
  at::Tensor parts = at::empty({rows, ld, 2}, hidden.options().dtype(at::kFloat));
  at::Tensor label_logit = at::zeros({rows}, hidden.options().dtype(at::kFloat));
  WsGemm g;
  g.a = hidden.data_ptr(); g.b = weight.data_ptr();
  g.m = rows; g.n = vocab; g.k = d;
  g.lda = (int)hidden.stride(0); g.ldb = (int)weight.stride(0);
  g.a_mn = 0; g.b_mn = 0; g.epilogue = WS_EPI_CE_FWD;
  g.out = parts.data_ptr(); g.ldo = ld;
  g.out2 = label_logit.data_ptr(); g.ldo2 = 0;
  g.aux = labels.data_ptr(); g.ldaux = 0;
  g.row_scale = nullptr; g.row_vec = nullptr; g.alpha = 1.f; g.beta = 0.f;
  g.error_flag = reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag)));
  check_rc(ws_gemm(&g, cur_stream()), "lm_head_fwd gemm");
  at::Tensor lse = at::empty({rows}, hidden.options().dtype(at::kFloat));
  at::Tensor logp = at::empty({rows}, hidden.options().dtype(at::kFloat));
  check_rc(ws_ce_combine(parts.data_ptr(), ld, nparts, label_logit.data_ptr<float>(),
                         reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), (long long)ignore_index, rows,
                         lse.data_ptr<float>(), logp.data_ptr<float>(), cur_stream()), "ce_combine");
  return {lse, logp};
}

// dlogits [rows, vocab] BF16 = (softmax(hidden @ weight.T) - onehot(labels)) * row_weight
at::Tensor lm_head_dlogits(const at::Tensor& hidden, const at::Tensor& weight, const at::Tensor& labels,
                           const at::Tensor& lse, const at::Tensor& row_weight,
                           const c10::optional<at::Tensor>& error_flag) {
  TORCH_CHECK(hidden.is_cuda() && hidden.scalar_type() == at::kBFloat16 && hidden.dim() == 2 && hidden.stride(1) == 1,
              "lm_head_dlogits: hidden");
  TORCH_CHECK(weight.scalar_type() == at::kBFloat16 && weight.is_contiguous() && weight.size(1) == hidden.size(1) &&
              weight.size(0) % 8 == 0, "lm_head_dlogits: weight must be BF16 [vocab, d] with vocab % 8 == 0");
  const int rows = (int)hidden.size(0), d = (int)hidden.size(1), vocab = (int)weight.size(0);
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == rows &&
              lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == rows &&
              row_weight.scalar_type() == at::kFloat && row_weight.is_contiguous() && row_weight.numel() == rows,
              "lm_head_dlogits: per-row vectors");
  c10::cuda::CUDAGuard guard(hidden.device());
  at::Tensor out = at::empty({rows, vocab}, hidden.options());
  WsGemm g;
  g.a = hidden.data_ptr(); g.b = weight.data_ptr();
  g.m = rows; g.n = vocab; g.k = d;
  g.lda = (int)hidden.stride(0); g.ldb = (int)weight.stride(0);
  g.a_mn = 0; g.b_mn = 0; g.epilogue = WS_EPI_CE_BWD;
  g.out = out.data_ptr(); g.ldo = vocab;
  g.out2 = nullptr; g.ldo2 = 0;
  g.aux = labels.data_ptr(); g.ldaux = 0;
  g.row_scale = row_weight.data_ptr<float>(); g.row_vec = lse.data_ptr<float>(); g.alpha = 1.f; g.beta = 0.f;
  g.error_flag = reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag)));
  check_rc(ws_gemm(&g, cur_stream()), "lm_head_dlogits gemm");
  return out;
}

// ----------------------------------------------------------------------------- communication
std::vector<unsigned long long> ptr_table(at::IntArrayRef v) {
  std::vector<unsigned long long> out;
  for (int64_t p : v) out.push_back(static_cast<unsigned long long>(p));
  return out;
}

void grad_allreduce(at::IntArrayRef grad_ptrs, at::IntArrayRef flag_ptrs, int64_t mc_grad, int64_t rank,
                    int64_t world, int64_t start, int64_t count, int64_t bucket, int64_t seq, double scale, bool push,
                    int64_t ctas, c10::optional<at::Tensor> sumsq_out, at::Tensor status, double budget_seconds) {
  TORCH_CHECK((int64_t)grad_ptrs.size() == world && (int64_t)flag_ptrs.size() == world, "grad_allreduce: peer tables");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 8, "grad_allreduce: status");
  c10::cuda::CUDAGuard guard(status.device());
  float* ss = nullptr;
  if (sumsq_out.has_value() && sumsq_out->defined()) {
    TORCH_CHECK(sumsq_out->scalar_type() == at::kFloat && sumsq_out->numel() >= ctas, "grad_allreduce: sumsq_out");
    ss = sumsq_out->data_ptr<float>();
  }
  auto g = ptr_table(grad_ptrs), f = ptr_table(flag_ptrs);
  check_rc(ws_grad_allreduce(g.data(), f.data(), (unsigned long long)mc_grad, (int)rank, (int)world, (size_t)start,
                             (size_t)count, (int)bucket, (unsigned)seq, (float)scale, push ? 1 : 0, (int)ctas, ss,
                             status.data_ptr<int>(), budget_seconds, cur_stream()), "grad_allreduce");
}

void wait_probe(const at::Tensor& flag, int64_t expected, at::Tensor status, double budget_seconds) {
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == at::kInt && status.scalar_type() == at::kInt &&
              status.numel() >= 8, "wait_probe: int32 CUDA tensors required");
  c10::cuda::CUDAGuard guard(flag.device());
  check_rc(ws_wait_probe(reinterpret_cast<const unsigned*>(flag.data_ptr<int>()), (unsigned)expected,
                         status.data_ptr<int>(), budget_seconds, cur_stream()), "wait_probe");
}

void grad_reduce_segments(at::IntArrayRef grad_ptrs, at::IntArrayRef flag_ptrs, int64_t mc_grad, int64_t rank,
                          int64_t world, at::IntArrayRef starts, at::IntArrayRef counts, at::IntArrayRef push,
                          int64_t bucket, int64_t seq, double scale, int64_t ctas, c10::optional<at::Tensor> sumsq_out,
                          at::Tensor status, double budget_seconds) {
  TORCH_CHECK((int64_t)grad_ptrs.size() == world && (int64_t)flag_ptrs.size() == world, "grad_reduce_segments: peer tables");
  TORCH_CHECK(starts.size() == counts.size() && starts.size() == push.size() && !starts.empty() && starts.size() <= 6,
              "grad_reduce_segments: 1..6 segments with start, count and push each");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 8, "grad_reduce_segments: status");
  c10::cuda::CUDAGuard guard(status.device());
  float* ss = nullptr;
  if (sumsq_out.has_value() && sumsq_out->defined()) {
    TORCH_CHECK(sumsq_out->scalar_type() == at::kFloat && sumsq_out->numel() >= ctas && sumsq_out->is_contiguous(),
                "grad_reduce_segments: sumsq_out");
    ss = sumsq_out->data_ptr<float>();
  }
  size_t st[6], ct[6];
  int pu[6];
  for (size_t i = 0; i < starts.size(); ++i) {
    TORCH_CHECK(starts[i] >= 0 && counts[i] >= 0, "grad_reduce_segments: negative range");
    st[i] = (size_t)starts[i]; ct[i] = (size_t)counts[i]; pu[i] = push[i] ? 1 : 0;
  }
  auto g = ptr_table(grad_ptrs), f = ptr_table(flag_ptrs);
  check_rc(ws_grad_reduce_segments(g.data(), f.data(), (unsigned long long)mc_grad, (int)rank, (int)world, st, ct, pu,
                                   (int)starts.size(), (int)bucket, (unsigned)seq, (float)scale, (int)ctas, ss,
                                   status.data_ptr<int>(), budget_seconds, cur_stream()), "grad_reduce_segments");
}

// -> stats [8] FP32: global norm, clip coefficient, norm^2, skip flag, loss summed over ranks
at::Tensor norm_exchange(at::IntArrayRef flag_ptrs, int64_t rank, int64_t world, int64_t base_word, int64_t seq,
                         const at::Tensor& partial, const c10::optional<at::Tensor>& local_loss, double max_norm,
                         at::Tensor status, double budget_seconds) {
  TORCH_CHECK((int64_t)flag_ptrs.size() == world, "norm_exchange: peer table");
  TORCH_CHECK(partial.is_cuda() && partial.scalar_type() == at::kFloat && partial.is_contiguous() && partial.numel() >= 1,
              "norm_exchange: partial");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 8, "norm_exchange: status");
  c10::cuda::CUDAGuard guard(partial.device());
  at::Tensor stats = at::zeros({8}, partial.options());
  auto f = ptr_table(flag_ptrs);
  check_rc(ws_norm_exchange(f.data(), (int)rank, (int)world, (int)base_word, (unsigned)seq, partial.data_ptr<float>(),
                            (int)partial.numel(), opt_f32(local_loss, "norm_exchange: local_loss"), (float)max_norm,
                            status.data_ptr<int>(), stats.data_ptr<float>(), budget_seconds, cur_stream()),
           "norm_exchange");
  return stats;
}

void node_barrier(at::IntArrayRef flag_ptrs, int64_t rank, int64_t world, int64_t base_word, int64_t seq,
                  at::Tensor status, double budget_seconds) {
  TORCH_CHECK((int64_t)flag_ptrs.size() == world, "node_barrier: peer table");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 8, "node_barrier: status");
  c10::cuda::CUDAGuard guard(status.device());
  auto f = ptr_table(flag_ptrs);
  check_rc(ws_node_barrier(f.data(), (int)rank, (int)world, (int)base_word, (unsigned)seq, status.data_ptr<int>(),
                           budget_seconds, cur_stream()), "node_barrier");
}

// wb [n, k] BF16 (local) = cast of the row-sharded FP32 weight (shard addresses as mapped in this process)
void gather_cast(std::vector<int64_t> shard_ptrs, int64_t rows_per_shard, at::Tensor wb, int64_t ctas) {
  TORCH_CHECK(wb.is_cuda() && wb.scalar_type() == at::kBFloat16 && wb.is_contiguous() && wb.dim() == 2,
              "gather_cast: wb must be contiguous BF16 [n, k]");
  const int64_t world = (int64_t)shard_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8, "gather_cast: 1..8 shards");
  const void* shards[8] = {};
  for (int64_t r = 0; r < world; ++r) shards[r] = reinterpret_cast<const void*>(static_cast<uintptr_t>(shard_ptrs[r]));
  c10::cuda::CUDAGuard guard(wb.device());
  check_rc(ws_gather_cast(shards, (int)world, (int)rows_per_shard, (int)wb.size(0), (int)wb.size(1), wb.data_ptr(),
                          (int)ctas, cur_stream()), "gather_cast");
}

void adamw_shard_push(at::IntArrayRef master_ptrs, at::IntArrayRef bf16_ptrs, int64_t rank, int64_t world,
                      const at::Tensor& g, at::Tensor m, at::Tensor v, int64_t lo, int64_t n, double lr, double beta1,
                      double beta2, double eps, double wd, int64_t step, const c10::optional<at::Tensor>& grad_scale,
                      bool push_master, const c10::optional<at::Tensor>& skip) {
  TORCH_CHECK((int64_t)master_ptrs.size() == world && (int64_t)bf16_ptrs.size() == world, "adamw_shard_push: tables");
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == at::kFloat && g.is_contiguous() && g.numel() >= lo + n, "adamw_shard_push: g");
  TORCH_CHECK(m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat && m.numel() == n && v.numel() == n &&
              m.is_contiguous() && v.is_contiguous(), "adamw_shard_push: moments");
  c10::cuda::CUDAGuard guard(g.device());
  auto mp = ptr_table(master_ptrs), bp = ptr_table(bf16_ptrs);
  const float* gs = grad_scale.has_value() && grad_scale->defined() ? grad_scale->data_ptr<float>() : nullptr;
  check_rc(ws_adamw_shard_push(mp.data(), bp.data(), (int)rank, (int)world, g.data_ptr<float>(), m.data_ptr<float>(),
                               v.data_ptr<float>(), (size_t)lo, (size_t)n, (float)lr, (float)beta1, (float)beta2,
                               (float)eps, (float)wd, (int)step, gs, push_master ? 1 : 0,
                               opt_f32(skip, "adamw_shard_push: skip"), cur_stream()),
           "adamw_shard_push");
}

// ----------------------------------------------------------------------------- sharded-weight linear
// y = x @ W^T where W [n, k] is FP32 and row-sharded over `shard_ptrs.size()` ranks (addresses as mapped in
// this process: the local shard and the peers' symmetric-memory shards).  One launch gathers, casts and
// multiplies; `wb` receives the BF16 copy of the whole weight as a by-product.
std::tuple<at::Tensor, at::Tensor> gather_cast_linear(const at::Tensor& x, std::vector<int64_t> shard_ptrs, int64_t n,
                                                      int64_t rows_per_shard, at::Tensor wb, at::Tensor flags,
                                                      c10::optional<at::Tensor> error_flag, double budget_seconds,
                                                      bool swiglu, bool want_packed) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous(),
              "gather_cast_linear: x must be contiguous BF16 [m, k]");
  const int64_t m = x.size(0), k = x.size(1);
  const int64_t world = (int64_t)shard_ptrs.size();
  const int64_t w_rows = swiglu ? 2 * n : n;
  TORCH_CHECK(world >= 1 && world <= 8, "gather_cast_linear: 1..8 shards");
  TORCH_CHECK(k % 8 == 0 && n > 0 && n % 8 == 0 && rows_per_shard > 0 && rows_per_shard % 8 == 0 &&
              rows_per_shard * world >= w_rows,
              "gather_cast_linear: k, n and rows_per_shard must be multiples of 8 and the shards must cover the weight");
  TORCH_CHECK(!swiglu || n % 128 == 0, "gather_cast_linear: the SwiGLU form needs a hidden width that is a multiple of 128");
  TORCH_CHECK(wb.is_cuda() && wb.scalar_type() == at::kBFloat16 && wb.is_contiguous() && wb.numel() == w_rows * k,
              "gather_cast_linear: wb must be contiguous BF16 with the weight's shape");
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && flags.is_contiguous() && flags.numel() >= (w_rows + 127) / 128 + 1,
              "gather_cast_linear: flags must be int32 with one word per 128 weight rows and one more");
  const void* shards[8] = {};
  for (int64_t r = 0; r < world; ++r) {
    TORCH_CHECK(shard_ptrs[r] != 0 && shard_ptrs[r] % 16 == 0, "gather_cast_linear: null or misaligned shard address");
    shards[r] = reinterpret_cast<const void*>(static_cast<uintptr_t>(shard_ptrs[r]));
  }
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out, act;
  if (swiglu) {
    act = at::empty({m, n}, x.options());
    if (want_packed) out = at::empty({m, 2 * n}, x.options());
  } else {
    out = at::empty({m, n}, x.options());
  }
  check_rc(ws_gather_gemm(x.data_ptr(), (int)m, (int)n, (int)k, shards, (int)world, (int)rows_per_shard, wb.data_ptr(),
                          flags.data_ptr(), swiglu ? WS_EPI_SWIGLU : WS_EPI_BF16, out.defined() ? out.data_ptr() : nullptr,
                          (int)w_rows, swiglu ? act.data_ptr() : nullptr, (int)n,
                          reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag))), (float)budget_seconds, 0,
                          cur_stream()), "gather_cast_linear");
  if (!out.defined()) out = at::empty({0}, x.options());
  if (!act.defined()) act = at::empty({0}, x.options());
  return std::make_tuple(out, act);
}

// ----------------------------------------------------------------------------- decode step
int64_t decode_gemm_splits(int64_t n, int64_t k) { return ws_decode_gemm_splits((int)n, (int)k); }
// Raises the library's error for a non-zero status of a C entry point (what every binding does
// with the codes it gets back); callable without a GPU, so the error path itself is testable.
int64_t raise_for_status(int64_t code) {
  check_rc((int)code, "status");
  return code;
}

void decode_gemm(const at::Tensor& w, const at::Tensor& x, int64_t n, int64_t epilogue, at::Tensor out,
                 c10::optional<at::Tensor> error_flag, bool packed) {
  TORCH_CHECK(w.is_cuda() && x.is_cuda() && out.is_cuda(), "decode_gemm: CUDA tensors required");
  TORCH_CHECK(w.scalar_type() == at::kBFloat16 && x.scalar_type() == at::kBFloat16 && w.is_contiguous() &&
              x.is_contiguous() && x.dim() == 2, "decode_gemm: contiguous BF16 W and x [batch, k] required");
  const int64_t k = x.size(1), batch = x.size(0);
  TORCH_CHECK(batch >= 1 && batch <= 64 && k % 8 == 0, "decode_gemm: batch must be 1..64 and k a multiple of 8");
  TORCH_CHECK(epilogue >= 0 && epilogue <= 3 && n > 0, "decode_gemm: epilogue 0..3 and n > 0 required");
  if (packed) {
    const int64_t slabs = epilogue == 2 ? n / 64 : (n + 127) / 128;
    TORCH_CHECK(w.dim() == 4 && w.size(0) == slabs && w.size(1) == (k + 63) / 64 && w.size(2) == 128 && w.size(3) == 64,
                "decode_gemm: a packed W must be [slabs, ceil(k/64), 128, 64]");
  } else {
    TORCH_CHECK(w.dim() == 2 && w.size(1) == k && w.size(0) == (epilogue == 2 ? 2 * n : n),
                "decode_gemm: W must be [rows, k] with rows matching n");
  }
  TORCH_CHECK(reinterpret_cast<uintptr_t>(w.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0,
              "decode_gemm: 16-byte aligned operands required");
  TORCH_CHECK(out.is_contiguous(), "decode_gemm: contiguous out required");
  if (epilogue == 1) {
    TORCH_CHECK(out.scalar_type() == at::kFloat && out.numel() == decode_gemm_splits(n, k) * batch * n,
                "decode_gemm: partial buffer must be FP32 [splits, batch, n]");
  } else {
    TORCH_CHECK(out.scalar_type() == (epilogue == 3 ? at::kFloat : at::kBFloat16) && out.dim() == 2 &&
                out.size(0) == batch && out.size(1) == n, "decode_gemm: out must be [batch, n] of the epilogue's dtype");
  }
  c10::cuda::CUDAGuard guard(w.device());
  check_rc(ws_decode_gemm(w.data_ptr(), x.data_ptr(), (int)n, (int)k, (int)batch, (int)epilogue, out.data_ptr(), (int)n,
                          reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag))), packed ? 1 : 0, cur_stream()),
           "decode_gemm");
}

void decode_reduce_norm(at::Tensor x, const c10::optional<at::Tensor>& partial, const c10::optional<at::Tensor>& token,
                        const c10::optional<at::Tensor>& table, const c10::optional<at::Tensor>& scale,
                        const c10::optional<at::Tensor>& bias, const at::Tensor& w, double eps,
                        c10::optional<at::Tensor> out) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.dim() == 2 && x.is_contiguous(), "decode_reduce_norm: x");
  const int64_t batch = x.size(0), d = x.size(1);
  TORCH_CHECK(d % 4 == 0 && w.scalar_type() == at::kFloat && w.numel() == d && w.is_contiguous(), "decode_reduce_norm: w");
  int splits = 0;
  const float* pp = nullptr;
  if (partial.has_value() && partial->defined()) {
    TORCH_CHECK(partial->scalar_type() == at::kFloat && partial->is_contiguous() && partial->numel() % (batch * d) == 0,
                "decode_reduce_norm: partial must be FP32 [splits, batch, d]");
    splits = (int)(partial->numel() / (batch * d));
    pp = partial->data_ptr<float>();
  }
  const long long* tok = nullptr;
  const float* tab = nullptr;
  int vocab = 0;
  if (token.has_value() && token->defined()) {
    TORCH_CHECK(table.has_value() && token->scalar_type() == at::kLong && token->numel() == batch && token->is_contiguous() &&
                table->scalar_type() == at::kFloat && table->is_contiguous() && table->size(1) == d && splits == 0,
                "decode_reduce_norm: token [batch] int64 with an FP32 table [vocab, d], and no partials");
    tok = reinterpret_cast<const long long*>(token->data_ptr<int64_t>());
    tab = table->data_ptr<float>();
    vocab = (int)table->size(0);
  }
  const bool mod = scale.has_value() && scale->defined();
  if (mod) {
    TORCH_CHECK(bias.has_value() && scale->scalar_type() == at::kFloat && bias->scalar_type() == at::kFloat &&
                scale->numel() == d && bias->numel() == d && scale->is_contiguous() && bias->is_contiguous(),
                "decode_reduce_norm: modulation vectors must be FP32 [d]");
  }
  void* op = nullptr;
  if (out.has_value() && out->defined()) {
    TORCH_CHECK(out->scalar_type() == at::kBFloat16 && out->is_contiguous() && out->numel() == batch * d, "decode_reduce_norm: out");
    op = out->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(ws_decode_reduce_norm(x.data_ptr<float>(), pp, splits, tok, tab, vocab, mod ? scale->data_ptr<float>() : nullptr,
                                 mod ? bias->data_ptr<float>() : nullptr, w.data_ptr<float>(), (float)eps, (int)d,
                                 (int)batch, op, cur_stream()), "decode_reduce_norm");
}

void decode_attn(const at::Tensor& qkvgu, at::Tensor kc, at::Tensor vc, at::Tensor uc, const at::Tensor& mixed,
                 const at::Tensor& rope, const at::Tensor& pos, int64_t H, at::Tensor y) {
  TORCH_CHECK(qkvgu.is_cuda() && qkvgu.scalar_type() == at::kBFloat16 && qkvgu.dim() == 2 && qkvgu.is_contiguous(),
              "decode_attn: qkvgu must be contiguous BF16 [batch, 5d]");
  const int64_t batch = qkvgu.size(0), d = qkvgu.size(1) / 5;
  TORCH_CHECK(d == H * 64, "decode_attn: head_dim must be 64");
  for (const at::Tensor* t : {&kc, &vc, &uc}) {
    TORCH_CHECK(t->scalar_type() == at::kBFloat16 && t->is_contiguous() && t->numel() == batch * H * 128 * 64,
                "decode_attn: caches must be contiguous BF16 [batch, H, 128, 64]");
  }
  TORCH_CHECK(mixed.scalar_type() == at::kBFloat16 && mixed.is_contiguous() && mixed.numel() == batch * H * 64 * 64,
              "decode_attn: mixed state must be contiguous BF16 [batch, H, 64, 64]");
  TORCH_CHECK(rope.scalar_type() == at::kFloat && rope.is_contiguous() && rope.numel() == 128 * 32 * 2, "decode_attn: rope table");
  TORCH_CHECK(pos.scalar_type() == at::kLong && pos.numel() == 1 && pos.is_cuda(), "decode_attn: pos must be a CUDA int64 scalar");
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.is_contiguous() && y.numel() == batch * d, "decode_attn: y");
  c10::cuda::CUDAGuard guard(qkvgu.device());
  check_rc(ws_decode_attn(qkvgu.data_ptr(), kc.data_ptr(), vc.data_ptr(), uc.data_ptr(), mixed.data_ptr(),
                          rope.data_ptr<float>(), reinterpret_cast<const long long*>(pos.data_ptr<int64_t>()), (int)batch,
                          (int)H, (int)d, y.data_ptr(), cur_stream()), "decode_attn");
}

void decode_layer_tail(const at::Tensor& w_out, const at::Tensor& w_ug, const at::Tensor& w_down,
                       const c10::optional<at::Tensor>& w_in_next, const at::Tensor& y, at::Tensor x, at::Tensor part_out,
                       at::Tensor part_down, at::Tensor n, at::Tensor act, at::Tensor qkvgu, const at::Tensor& w_norm2,
                       const c10::optional<at::Tensor>& next_scale, const c10::optional<at::Tensor>& next_bias,
                       const at::Tensor& w_norm_next, double eps, at::Tensor barrier, const c10::optional<at::Tensor>& error_flag,
                       const c10::optional<at::Tensor>& trace) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.dim() == 2 && x.is_contiguous(), "decode_layer_tail: x");
  const int64_t batch = x.size(0), d = x.size(1);
  TORCH_CHECK(w_down.dim() == 2 && w_down.size(0) == d, "decode_layer_tail: w_down must be [d, ffn]");
  const int64_t ffn = w_down.size(1);
  auto bf16 = [](const at::Tensor& t, int64_t rows, int64_t cols, const char* what) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.dim() == 2 && t.size(0) == rows &&
                t.size(1) == cols && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, what);
  };
  bf16(w_out, d, d, "decode_layer_tail: w_out must be contiguous BF16 [d, d]");
  bf16(w_ug, 2 * ffn, d, "decode_layer_tail: w_ug must be contiguous BF16 [2 ffn, d]");
  bf16(w_down, d, ffn, "decode_layer_tail: w_down must be contiguous BF16 [d, ffn]");
  if (w_in_next.has_value()) bf16(*w_in_next, 5 * d, d, "decode_layer_tail: w_in_next must be contiguous BF16 [5 d, d]");
  bf16(y, batch, d, "decode_layer_tail: y must be contiguous BF16 [batch, d]");
  bf16(n, batch, d, "decode_layer_tail: n must be contiguous BF16 [batch, d]");
  bf16(act, batch, ffn, "decode_layer_tail: act must be contiguous BF16 [batch, ffn]");
  bf16(qkvgu, batch, 5 * d, "decode_layer_tail: qkvgu must be contiguous BF16 [batch, 5 d]");
  TORCH_CHECK(part_out.scalar_type() == at::kFloat && part_out.is_contiguous() &&
              part_out.numel() == decode_gemm_splits(d, d) * batch * d, "decode_layer_tail: part_out [splits, batch, d] FP32");
  TORCH_CHECK(part_down.scalar_type() == at::kFloat && part_down.is_contiguous() &&
              part_down.numel() == decode_gemm_splits(d, ffn) * batch * d, "decode_layer_tail: part_down [splits, batch, d] FP32");
  for (const at::Tensor* t : {&w_norm2, &w_norm_next}) {
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == d,
                "decode_layer_tail: norm weights must be FP32 [d]");
  }
  TORCH_CHECK(next_scale.has_value() == next_bias.has_value(), "decode_layer_tail: modulation needs scale and bias");
  if (next_scale.has_value()) {
    TORCH_CHECK(next_scale->scalar_type() == at::kFloat && next_scale->numel() == d && next_scale->is_contiguous() &&
                next_bias->scalar_type() == at::kFloat && next_bias->numel() == d && next_bias->is_contiguous(),
                "decode_layer_tail: modulation vectors must be FP32 [d]");
  }
  TORCH_CHECK(barrier.is_cuda() && barrier.scalar_type() == at::kInt && barrier.is_contiguous() && barrier.numel() >= 2,
              "decode_layer_tail: barrier must hold two int32 words");
  long long* stamps = nullptr;
  if (trace.has_value()) {
    const int sms = at::cuda::getDeviceProperties(x.device().index())->multiProcessorCount;
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == at::kLong && trace->is_contiguous() && trace->numel() >= 16 * sms,
                "decode_layer_tail: trace must be int64 [SMs, 16]");
    stamps = reinterpret_cast<long long*>(trace->data_ptr<int64_t>());
  }
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(ws_decode_layer_tail(w_out.data_ptr(), w_ug.data_ptr(), w_down.data_ptr(),
                                w_in_next.has_value() ? w_in_next->data_ptr() : nullptr, y.data_ptr(), x.data_ptr<float>(),
                                part_out.data_ptr<float>(), part_down.data_ptr<float>(), n.data_ptr(), act.data_ptr(),
                                qkvgu.data_ptr(), w_norm2.data_ptr<float>(),
                                next_scale.has_value() ? next_scale->data_ptr<float>() : nullptr,
                                next_bias.has_value() ? next_bias->data_ptr<float>() : nullptr, w_norm_next.data_ptr<float>(),
                                (float)eps, (int)batch, (int)d, (int)ffn, reinterpret_cast<unsigned*>(barrier.data_ptr<int>()),
                                reinterpret_cast<int*>(const_cast<void*>(opt_ptr(error_flag))), stamps, cur_stream()), "decode_layer_tail");
}

void decode_pick(const at::Tensor& logits, at::Tensor token, const c10::optional<at::Tensor>& history, at::Tensor cursor,
                 at::Tensor pos) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.is_contiguous() &&
              logits.size(1) % 4 == 0, "decode_pick: logits must be contiguous FP32 [batch, vocab], vocab a multiple of 4");
  const int64_t batch = logits.size(0);
  TORCH_CHECK(token.is_cuda() && token.scalar_type() == at::kLong && token.is_contiguous() && token.numel() == batch,
              "decode_pick: token must be int64 [batch]");
  TORCH_CHECK(cursor.is_cuda() && cursor.scalar_type() == at::kLong && cursor.is_contiguous() && cursor.numel() == 2,
              "decode_pick: cursor must be two int64 words");
  TORCH_CHECK(pos.is_cuda() && pos.scalar_type() == at::kLong && pos.numel() == 1, "decode_pick: pos must be an int64 scalar");
  long long* hist = nullptr;
  int capacity = 0;
  if (history.has_value()) {
    TORCH_CHECK(history->is_cuda() && history->scalar_type() == at::kLong && history->is_contiguous() && history->dim() == 2 &&
                history->size(0) == batch, "decode_pick: history must be contiguous int64 [batch, capacity]");
    hist = reinterpret_cast<long long*>(history->data_ptr<int64_t>());
    capacity = (int)history->size(1);
  }
  c10::cuda::CUDAGuard guard(logits.device());
  check_rc(ws_decode_pick(logits.data_ptr<float>(), (int)batch, (int)logits.size(1),
                          reinterpret_cast<long long*>(token.data_ptr<int64_t>()), hist, capacity,
                          reinterpret_cast<long long*>(cursor.data_ptr<int64_t>()),
                          reinterpret_cast<long long*>(pos.data_ptr<int64_t>()), cur_stream()), "decode_pick");
}

}  // namespace

TORCH_LIBRARY(ws_b200, m) {
  m.def("decode_gemm_splits(int n, int k) -> int");
  m.def("gather_cast_linear(Tensor x, int[] shard_ptrs, int n, int rows_per_shard, Tensor(a!) wb, Tensor(b!) flags, "
        "Tensor(c!)? error_flag, float budget_seconds, bool swiglu=False, bool want_packed=True) -> (Tensor, Tensor)");
  m.def("raise_for_status(int code) -> int");
  m.def("decode_gemm(Tensor w, Tensor x, int n, int epilogue, Tensor(a!) out, Tensor(b!)? error_flag, bool packed=False) -> ()");
  m.def("decode_reduce_norm(Tensor(a!) x, Tensor? partial, Tensor? token, Tensor? table, Tensor? scale, Tensor? bias, "
        "Tensor w, float eps, Tensor(b!)? out) -> ()");
  m.def("decode_layer_tail(Tensor w_out, Tensor w_ug, Tensor w_down, Tensor? w_in_next, Tensor y, Tensor(a!) x, "
        "Tensor(b!) part_out, Tensor(c!) part_down, Tensor(d!) n, Tensor(e!) act, Tensor(f!) qkvgu, Tensor w_norm2, "
        "Tensor? next_scale, Tensor? next_bias, Tensor w_norm_next, float eps, Tensor(g!) barrier, Tensor(h!)? error_flag, "
        "Tensor(i!)? trace=None) -> ()");
  m.def("decode_pick(Tensor logits, Tensor(a!) token, Tensor(b!)? history, Tensor(c!) cursor, Tensor(d!) pos) -> ()");
  m.def("decode_attn(Tensor qkvgu, Tensor(a!) kc, Tensor(b!) vc, Tensor(c!) uc, Tensor mixed, Tensor rope, Tensor pos, "
        "int H, Tensor(d!) y) -> ()");
  m.def("rmsnorm_fwd(Tensor x, Tensor? col_scale, Tensor? col_bias, Tensor w, float eps, bool want_xmod) -> (Tensor, Tensor, Tensor)");
  m.def("rmsnorm_bwd(Tensor dz, Tensor x, Tensor rstd, Tensor w, Tensor? dres, Tensor? out_scale, bool want_bf16) -> (Tensor, Tensor, Tensor)");
  m.def("colsum2(Tensor a, Tensor b, Tensor? inv_scale) -> (Tensor, Tensor)");
  m.def("cast_bf16(Tensor x, Tensor(a!)? out) -> Tensor");
  m.def("embed_fwd(Tensor ids, Tensor table, bool out_bf16) -> Tensor");
  m.def("embed_bwd(Tensor dx, Tensor ids, Tensor(a!) grad_table) -> ()");
  m.def("launch_count() -> int");
  m.def("lm_head_fwd(Tensor hidden, Tensor weight, Tensor labels, int ignore_index, Tensor(a!)? error_flag) -> (Tensor, Tensor)");
  m.def("lm_head_dlogits(Tensor hidden, Tensor weight, Tensor labels, Tensor lse, Tensor row_weight, Tensor(a!)? error_flag) -> Tensor");
  m.def("grad_allreduce(int[] grad_ptrs, int[] flag_ptrs, int mc_grad, int rank, int world, int start, int count, "
        "int bucket, int seq, float scale, bool push, int ctas, Tensor(a!)? sumsq_out, Tensor(b!) status, "
        "float budget_seconds) -> ()");
  m.def("wait_probe(Tensor flag, int expected, Tensor(a!) status, float budget_seconds) -> ()");
  m.def("adamw_shard_push(int[] master_ptrs, int[] bf16_ptrs, int rank, int world, Tensor g, Tensor(a!) m, "
        "Tensor(b!) v, int lo, int n, float lr, float beta1, float beta2, float eps, float wd, int step, "
        "Tensor? grad_scale, bool push_master, Tensor? skip=None) -> ()");
  m.def("attn_bwd(Tensor qkvgu, Tensor dy, Tensor states, Tensor writes, Tensor rope, Tensor fast_logit, "
        "Tensor slow_logit, Tensor mix_logit, int B, int T, int H, Tensor(a!)? error_flag) -> (Tensor, Tensor)");
  m.def("chunk_writes(Tensor qkvgu, Tensor rope, int B, int T, int H, Tensor(a!)? error_flag) -> Tensor");
  m.def("memory_scan(Tensor writes, Tensor fast_logit, Tensor slow_logit, Tensor mix_logit, bool want_states, "
        "bool want_final, Tensor? init_fast, Tensor? init_slow) -> (Tensor, Tensor, Tensor)");
  m.def("attn_fwd(Tensor qkvgu, Tensor states, Tensor rope, int B, int T, int H, Tensor(a!)? error_flag) -> Tensor");
  m.def("grad_norm_clip(Tensor g, float max_norm, Tensor? extra_sumsq, Tensor? status=None) -> Tensor");
  m.def("clip_from_partials(Tensor partial, float max_norm, Tensor? extra_sumsq=None, Tensor? status=None) -> Tensor");
  m.def("grad_reduce_segments(int[] grad_ptrs, int[] flag_ptrs, int mc_grad, int rank, int world, int[] starts, "
        "int[] counts, int[] push, int bucket, int seq, float scale, int ctas, Tensor(a!)? sumsq_out, "
        "Tensor(b!) status, float budget_seconds) -> ()");
  m.def("norm_exchange(int[] flag_ptrs, int rank, int world, int base_word, int seq, Tensor partial, "
        "Tensor? local_loss, float max_norm, Tensor(a!) status, float budget_seconds) -> Tensor");
  m.def("node_barrier(int[] flag_ptrs, int rank, int world, int base_word, int seq, Tensor(a!) status, "
        "float budget_seconds) -> ()");
  m.def("gather_cast(int[] shard_ptrs, int rows_per_shard, Tensor(a!) wb, int ctas) -> ()");
  m.def("adamw_step(Tensor(a!) p, Tensor g, Tensor(b!) m, Tensor(c!) v, Tensor(d!)? p_bf16, float lr, float beta1, "
        "float beta2, float eps, float wd, int step, Tensor? grad_scale, float grad_scale_const, "
        "Tensor? skip=None) -> ()");
  m.def("gemm(Tensor a, Tensor b, bool a_mn, bool b_mn, int epilogue, int m, int n, int k, "
        "Tensor(a!) out, Tensor(b!)? out2, Tensor? aux, Tensor? row_scale, float alpha, float beta, "
        "Tensor(c!)? error_flag) -> ()");
  m.def("grad_weight_group(Tensor[] dys, Tensor[] xs, Tensor(a!)[] grads, float[] betas, Tensor(b!)? error_flag) -> ()");
}

TORCH_LIBRARY_IMPL(ws_b200, CompositeExplicitAutograd, m) {
  m.impl("launch_count", &launch_count);
  m.impl("decode_gemm_splits", &decode_gemm_splits);
  m.impl("raise_for_status", &raise_for_status);
}

TORCH_LIBRARY_IMPL(ws_b200, CUDA, m) {
  m.impl("gemm", &gemm);
  m.impl("decode_gemm", &decode_gemm);
  m.impl("gather_cast_linear", &gather_cast_linear);
  m.impl("decode_reduce_norm", &decode_reduce_norm);
  m.impl("decode_attn", &decode_attn);
  m.impl("decode_pick", &decode_pick);
  m.impl("decode_layer_tail", &decode_layer_tail);
  m.impl("grad_weight_group", &grad_weight_group);
  m.impl("rmsnorm_fwd", &rmsnorm_fwd);
  m.impl("rmsnorm_bwd", &rmsnorm_bwd);
  m.impl("colsum2", &colsum2);
  m.impl("cast_bf16", &cast_bf16);
  m.impl("embed_fwd", &embed_fwd);
  m.impl("embed_bwd", &embed_bwd);
  m.impl("grad_norm_clip", &grad_norm_clip);
  m.impl("clip_from_partials", &clip_from_partials);
  m.impl("grad_reduce_segments", &grad_reduce_segments);
  m.impl("norm_exchange", &norm_exchange);
  m.impl("node_barrier", &node_barrier);
  m.impl("gather_cast", &gather_cast);
  m.impl("attn_bwd", &attn_bwd);
  m.impl("chunk_writes", &chunk_writes);
  m.impl("memory_scan", &memory_scan);
  m.impl("attn_fwd", &attn_fwd);
  m.impl("adamw_step", &adamw_step);
  m.impl("lm_head_fwd", &lm_head_fwd);
  m.impl("lm_head_dlogits", &lm_head_dlogits);
  m.impl("grad_allreduce", &grad_allreduce);
  m.impl("wait_probe", &wait_probe);
  m.impl("adamw_shard_push", &adamw_shard_push);
}
