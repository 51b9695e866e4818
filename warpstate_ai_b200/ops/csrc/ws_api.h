// C ABI of the sm_100a kernel library.  Every function takes raw device pointers and a CUDA
// stream, launches on that stream and returns 0 on success or a negative error code; none of
// them allocates unless stated.  The torch bindings (bindings.cpp) are a thin layer over these.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

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
  WS_EPI_CE_FWD = 7,      // LM head: out = float2 parts[M, ldo] of (max, sum exp) per 128 columns, out2 = label logit[M]; aux = labels (int64)
  WS_EPI_CE_BWD = 8,      // LM head: out_bf16[M,N] = (exp(logit - row_vec[m]) - onehot(label)) * row_scale[m]; aux = labels
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
  const float* row_vec;    // CE_BWD: per-row log-sum-exp (otherwise NULL)
  float alpha;
  float beta;
  int* error_flag;  // device int; set non-zero if a bounded wait ran out (may be NULL)
} WsGemm;

int ws_gemm(const WsGemm* g, cudaStream_t stream);
// Number of SMs the GEMM may use on this stream's device (0 = all).  Lets a communication
// kernel keep a few SMs for itself while persistent GEMM CTAs fill the rest.
// `count` problems in one persistent launch where possible (same operand majors and epilogue, each
// with >= 256 rows, count <= 4); otherwise equivalent to calling ws_gemm on each item in order.
int ws_gemm_group(const WsGemm* items, int count, cudaStream_t stream);
void ws_gemm_set_sm_limit(int sms);
// Fused all-gather + FP32->BF16 cast + GEMM for a row-sharded weight (ops/csrc/gemm2_tcgen05.cu):
// out[m, n] = x[m, k] . W[n, k]^T with W's FP32 rows owned by `world` ranks in blocks of rows_per_shard;
// shards[r] is rank r's block as mapped in this process.  wb: local BF16 copy of W; flags: one word per 128
// weight rows.  epilogue WS_EPI_BF16 (W [n, k]) or WS_EPI_SWIGLU (W [2n, k]; out packed or NULL, out2 activation).
int ws_gather_gemm(const void* x, int m, int n, int k, const void* const* shards, int world, int rows_per_shard,
                   void* wb, void* flags, int epilogue, void* out, int ldo, void* out2, int ldo2, int* error_flag,
                   float budget_seconds, int sms, cudaStream_t stream);
// ---- decode step (ops/csrc/decode.cu); batch <= 64
// out[b, n] = sum_k x[b, k] W[n, k] as a weight-streaming kernel.  epilogue: 0 BF16 [batch, ldo];
// 1 FP32 split-K partials [ws_decode_gemm_splits(n, k), batch, n]; 2 SwiGLU with W = [2n, k]
// (up rows, then gate rows), BF16 [batch, ldo]; 3 FP32 [batch, ldo].
int ws_decode_gemm_splits(int n, int k);
int ws_decode_gemm(const void* w, const void* x, int n, int k, int batch, int epilogue, void* out, int ldo,
                   int* error_flag, int packed, cudaStream_t stream);
// x (FP32 [batch, d], in place) = table[token] if token else x + sum of split partials; optional
// depth modulation x*(1+scale)+bias; out (BF16 [batch, d], may be NULL) = RMSNorm(x) * w.
int ws_decode_reduce_norm(float* x, const float* partial, int splits, const long long* token, const float* table,
                          int vocab, const float* scale, const float* bias, const float* w, float eps, int d,
                          int batch, void* out, cudaStream_t stream);
// One decode step of the attention block for every (sequence, head); see decode_attn_kernel.
int ws_decode_attn(const void* qkvgu, void* kc, void* vc, void* uc, const void* mixed, const float* rope,
                   const long long* pos, int batch, int H, int d, void* y, cudaStream_t stream);

// The part of a decode layer after its attention as ONE persistent cooperative launch (ops/csrc/decode_layer.cu):
// out_proj, residual + norm, up/gate + SwiGLU, down, residual + next layer's modulation + norm, next layer's in_proj.
// Weights row-major BF16: w_out [d, d], w_ug [2 ffn, d], w_down [d, ffn], w_in_next [5 d, d] or NULL after the last
// layer.  y [batch, d] BF16 attention output; x [batch, d] FP32 residual (in place); part_out / part_down FP32
// [ws_decode_gemm_splits(d, d) | (d, ffn), batch, d]; n [batch, d], act [batch, ffn], qkvgu [batch, 5 d] BF16.
// barrier: two zeroed 32-bit words.  trace: NULL, or [SMs, 16] int64 receiving %globaltimer at phase boundaries.
// batch <= 64.  -30: fewer SMs than the largest phase has work items.
int ws_decode_layer_tail(const void* w_out, const void* w_ug, const void* w_down, const void* w_in_next,
                         const void* y, float* x, float* part_out, float* part_down, void* n, void* act, void* qkvgu,
                         const float* w_norm2, const float* next_scale, const float* next_bias,
                         const float* w_norm_next, float eps, int batch, int d, int ffn, unsigned* barrier,
                         int* error_flag, long long* trace, cudaStream_t stream);

// Greedy pick at the end of a decode step: token[b] = argmax(logits[b, :]), also written to history[b, cursor[0]]
// (history [batch, capacity] int64, may be NULL); then pos[0] += 1 and cursor[0] += 1.  cursor: two int64 words
// (column, zeroed scratch).  vocab % 4 == 0.
int ws_decode_pick(const float* logits, int batch, int vocab, long long* token, long long* history, int capacity,
                   long long* cursor, long long* pos, cudaStream_t stream);

// Kernel choice for problems with >= 256 rows: 1 = CTA-pair (cta_group::2) kernel, 0 = single-CTA
// kernel, -1 = the process default (pair unless WS_GEMM_PAIR=0 is in the environment).
void ws_gemm_set_pair_mode(int mode);

// Number of kernels this library has launched in this process.
long long ws_launch_count(void);
void ws_count_launch(void);

// ----------------------------------------------------------------------------- row kernels
// RMSNorm forward over `rows` rows of width d (d % 128 == 0).  The residual stream `x` is FP32
// (x_bf16 = 0) or BF16.  When col_scale/col_bias are given the depth modulation
// x*(1+scale)+bias is applied first and (optionally) written to xmod_out.  z is BF16.
int ws_rmsnorm_fwd(const void* x, int x_bf16, const float* col_scale, const float* col_bias,
                   const float* w, float eps, int rows, int d, void* xmod_out, void* z, float* rstd,
                   cudaStream_t stream);
// RMSNorm backward: dx_out = (dres + norm_bwd(dz)) * (1 + out_scale); optional BF16 copy;
// dw_partial holds ws_rmsnorm_bwd_parts(rows) partial rows of d floats (d <= 2048).
int ws_rmsnorm_bwd_parts(int rows);
int ws_rmsnorm_bwd(const void* dz, const void* x, int x_bf16, const float* rstd, const float* w,
                   const void* dres, const float* out_scale, int rows, int d, void* dx_out,
                   void* dx_bf16, float* dw_partial, cudaStream_t stream);
// Column sums of a and a*b over rows, as ws_colsum_parts(rows) partial rows.
int ws_colsum_parts(int rows);
int ws_colsum2(const void* a, const void* b, int is_bf16, int rows, int d, float* partial_a,
               float* partial_ab, cudaStream_t stream);
// out[c] = beta*out[c] + (sum_p partial[p][c]) / (1 + inv_scale[c])   (inv_scale may be NULL)
int ws_colsum_finalize(const float* partial, int parts, int d, const float* inv_scale, float beta,
                       float* out, cudaStream_t stream);
int ws_cast_f32_bf16(const float* in, void* out, size_t n, cudaStream_t stream);
int ws_embed_fwd(const long long* ids, const void* table, int table_bf16, int rows, int d, int vocab,
                 void* out, int out_bf16, cudaStream_t stream);
int ws_embed_bwd(const void* dx, int dx_bf16, const long long* sorted_ids, const long long* order, int rows,
                 int d, int vocab, float* grad_table, cudaStream_t stream);

// ----------------------------------------------------------------------------- attention / memory
// qkvgu: BF16 [B*T, 5d] (Q,K,V,gate,U); chunk 128, head_dim 64, d = H*64.  rope: float2 [128][32].
// writes: FP32 [B, T/128, H, 64, 64] = tanh(rope(K))^T tanh(U) / 128.
// Form of the attention block's tile kernels: 1 persistent streaming CTAs, 0 one tile per CTA, -1 process default
// (streaming unless WS_ATTN_STREAM=0).
void ws_attn_set_stream_mode(int mode);
int ws_attn_stream_form(void);   // the resolved choice: 1 streaming, 0 one tile per CTA
int ws_chunk_writes(const void* qkvgu, const float* rope, float* writes, int B, int T, int H, int d,
                    int* error_flag, cudaStream_t stream);
// states (BF16, may be NULL): mixed state read by each chunk; final_* (FP32 [B,H,64,64], may be NULL);
// init_* (may be NULL) start the scan from given states.
int ws_memory_scan(const float* writes, const float* fast_logit, const float* slow_logit,
                   const float* mix_logit, void* states, float* final_fast, float* final_slow,
                   const float* init_fast, const float* init_slow, int B, int N, int H,
                   cudaStream_t stream);
// y: BF16 [B*T, d] token-major.
int ws_attn_fwd(const void* qkvgu, const void* states, const float* rope, void* y, int B, int T, int H,
                int d, int* error_flag, cudaStream_t stream);

// Backward of the same block.  dy: BF16 [B*T, d].  dstate: FP32 [B,N,H,64,64].
int ws_attn_dstate(const void* qkvgu, const void* dy, const float* rope, float* dstate, int B, int T, int H,
                   int d, int* error_flag, cudaStream_t stream);
// dwrites: BF16 [B,N,H,64,64]; partials: FP32 [B*H*16][3] (d fast decay, d slow decay, d mix); N <= 64.
int ws_memory_scan_bwd(const float* dstate, const float* writes, const float* fast_logit,
                       const float* slow_logit, const float* mix_logit, void* dwrites, float* partials,
                       int B, int N, int H, cudaStream_t stream);
// dqkvgu: BF16 [B*T, 5d], fully written.
int ws_attn_bwd(const void* qkvgu, const void* states, const void* dy, const void* dwrites,
                const float* rope, void* dqkvgu, int B, int T, int H, int d, int* error_flag,
                cudaStream_t stream);

// ----------------------------------------------------------------------------- optimizer
int ws_sumsq_parts(void);
// stats (4 floats): [0] = ||g||_2, [1] = min(1, max_norm / (||g|| + 1e-6)), [2] = ||g||^2 (+ *extra_sumsq),
// [3] = skip flag, 1 when the norm is not finite or *status (device int of a communication kernel, may be
// NULL) is non-zero; the coefficient is 0 then.
int ws_grad_norm_clip(const float* g, size_t n, float* partial, const float* extra_sumsq, float max_norm,
                      const int* status, float* stats, cudaStream_t stream);
// The same from `parts` partial sums of squares produced elsewhere (summed in index order).
int ws_clip_from_partials(const float* partial, int parts, const float* extra_sumsq, float max_norm,
                          const int* status, float* stats, cudaStream_t stream);
// AdamW over flat FP32 arenas (n % 4 == 0); gradients are multiplied by *grad_scale_ptr (device,
// may be NULL) times grad_scale_const first; p_bf16 (may be NULL) receives the BF16 copy of p.
// When *skip_ptr (device, may be NULL) is non-zero the kernel changes nothing.
int ws_adamw(float* p, const float* g, float* m, float* v, void* p_bf16, size_t n, float lr, float beta1,
             float beta2, float eps, float wd, int step, const float* grad_scale_ptr,
             float grad_scale_const, const float* skip_ptr, cudaStream_t stream);

// ----------------------------------------------------------------------------- LM head
// parts: float2 [rows, ld] of (max, sum exp) per 128 vocabulary columns (nparts valid per row),
// written by the WS_EPI_CE_FWD epilogue.  lse[rows], logp[rows] (0 where label == ignore_index).
int ws_ce_combine(const void* parts, int ld, int nparts, const float* label_logit, const long long* labels,
                  long long ignore_index, int rows, float* lse, float* logp, cudaStream_t stream);

// ----------------------------------------------------------------------------- communication
// Peer tables are arrays of `world` (<= 8) device addresses valid in THIS process: its mappings
// of every rank's buffer, own rank included.  Flag buffers hold ws_comm_flag_words(buckets)
// zero-initialised 32-bit words per rank.  status: 8 ints on the device, 0 = no error.
int ws_comm_flag_words(int buckets);
int ws_comm_max_ctas(void);
// In-place all-reduce (push = 1) or reduce-scatter (push = 0) of grad[start, start+count) with
// the result scaled by `scale`; mc_grad is the multimem address of the arena or 0.
// sumsq_out (may be NULL) receives `ctas` partial sums of squares of this rank's reduced slice.
// Two launches: a one-warp kernel that announces the bucket and waits (bounded) for the peers', then
// the data kernel, which moves nothing when *status is already non-zero.
int ws_grad_allreduce(const unsigned long long* grad_ptrs, const unsigned long long* flag_ptrs,
                      unsigned long long mc_grad, int rank, int world, size_t start, size_t count, int bucket,
                      unsigned seq, float scale, int push, int ctas, float* sumsq_out, int* status,
                      double budget_seconds, cudaStream_t stream);
// The same over up to 6 ranges of the arena with their own push flags, under one bucket's flags.
int ws_grad_reduce_segments(const unsigned long long* grad_ptrs, const unsigned long long* flag_ptrs,
                            unsigned long long mc_grad, int rank, int world, const size_t* starts,
                            const size_t* counts, const int* push, int nseg, int bucket, unsigned seq, float scale,
                            int ctas, float* sumsq_out, int* status, double budget_seconds, cudaStream_t stream);
// Words a flag buffer needs after the bucket flags for ws_norm_exchange (3 * 8 words from its base) and
// ws_node_barrier (8 words from its base).
int ws_comm_extra_words(void);
// stats[0..4] = global gradient norm, clip coefficient, norm^2, skip flag, sum over ranks of *local_loss,
// bit-identical on every rank: each rank sums its `parts` partials, the sums are exchanged through the flag
// buffers (words [base_word, base_word + 24)) and added in rank order.  `seq` as for the buckets.
int ws_norm_exchange(const unsigned long long* flag_ptrs, int rank, int world, int base_word, unsigned seq,
                     const float* partial, int parts, const float* local_loss, float max_norm, int* status,
                     float* stats, double budget_seconds, cudaStream_t stream);
// Device-side barrier over the ranks of the node through words [base_word, base_word + 8) of the flag buffers.
int ws_node_barrier(const unsigned long long* flag_ptrs, int rank, int world, int base_word, unsigned seq,
                    int* status, double budget_seconds, cudaStream_t stream);
// dst[n, k] (BF16, local) = the FP32 weight whose rows are sharded over `world` ranks in blocks of
// rows_per_shard (shards[r]: rank r's block as mapped in this process; plain peer loads).
int ws_gather_cast(const void* const* shards, int world, int rows_per_shard, int n, int k, void* dst, int ctas,
                   cudaStream_t stream);
// Waits (bounded) for *flag >= expected and reports expiry through `status` like the kernels do.
int ws_wait_probe(const unsigned* flag, unsigned expected, int* status, double budget_seconds,
                  cudaStream_t stream);
// AdamW on arena elements [lo, lo+n) owned by this rank; m, v are the rank's shard-local moments;
// updated BF16 weights (and FP32 masters when push_master) are stored to every rank.
int ws_adamw_shard_push(const unsigned long long* master_ptrs, const unsigned long long* bf16_ptrs, int rank,
                        int world, const float* g, float* m, float* v, size_t lo, size_t n, float lr,
                        float beta1, float beta2, float eps, float wd, int step, const float* grad_scale_ptr,
                        int push_master, const float* skip_ptr, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
