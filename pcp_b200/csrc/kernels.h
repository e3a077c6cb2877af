// Host-callable launchers of the training-step kernels.  Every launcher enqueues on `st` and
// returns the CUDA error of the launch; none allocates or synchronises.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace pcpb {

// ---- GEMM ----------------------------------------------------------------------------------
// C[M,N] (+epilogue) = sum_k A(m,k) * B(k,n), A(m,k) = A[m*sam + k*sak], B(k,n) = B[k*sbk + n*sbn],
// f32 accumulation, operands of model dtype `dt` (DT_F32 | DT_BF16).
enum GemmEpilogue : int {
  EPI_STORE = 0,    // C = T(acc)
  EPI_RESID = 1,    // C = T(R + T(acc))                  (residual add in model dtype)
  EPI_RELU2 = 2,    // C = T(acc); C2 = T(max(C,0)^2)     (MLP activation, two outputs)
  EPI_DRELU2 = 3,   // C = backward of max(.,0)^2 at U given dA = T(acc)
  EPI_WGRAD = 4,    // Cf32 = clamp(finite(T(acc)), +-clip)   (weight gradient, f32 out)
  EPI_RELU = 5,     // C = T(acc); C2 = max(C, 0)         (nanoGPT MLP activation, two outputs)
  EPI_DRELU = 6,    // C = U > 0 ? T(acc) : 0             (backward of max(., 0), U in R)
  EPI_BIAS = 7,     // C = T(acc + bias[n])               (lm_head with bias; bias of model dtype in R, length N)
  EPI_GELU = 8,     // C = T(acc); C2 = gelu_tanh(C), every op of the activation rounded to T (two outputs)
  EPI_DGELU = 9,    // C = T(T(acc) * gelu_tanh'(U))      (backward of the tanh GELU, U in R)
  EPI_RAWF32 = 10,  // tensor-core kernels only: Cf32 = acc, nothing else (the f32 models' split-operand path)
};
struct GemmArgs {
  const void* A; long long sam, sak;
  const void* B; long long sbk, sbn;
  void* C; long long ldc;
  const void* R;        // EPI_RESID: residual [M,ldc];  EPI_DRELU2 / EPI_DRELU / EPI_DGELU: U [M,ldc];  EPI_BIAS: bias [N]
  void* C2;             // EPI_RELU2 / EPI_RELU / EPI_GELU: second output [M,ldc]
  int M, N, K;
  int epi;
  float clip;           // EPI_WGRAD
  int adj = 0;          // EPI_STORE only: 1 = the output is an activation gradient, finite-guarded and clamped to +-100
                        // like every adjoint edge of the reference's engine (src/autodiff/engine.zig:622-682); the
                        // backward epilogues (EPI_D*) always do so
  // tensor-core path only: split-K scratch of the caller (f32 slabs) and its device error word
  void* scratch = nullptr; size_t scratch_bytes = 0; int* err_word = nullptr;
};
cudaError_t launch_gemm_generic(cudaStream_t st, int dt, const GemmArgs& g);
// f32 models on the bf16 tensor cores.  An f32 value is the sum of three bf16 values to 24 bits (x1 = bf16(x),
// x2 = bf16(x - x1), x3 = bf16(x - x1 - x2)); a product a*b is then a1 b1 + a1 b2 + a2 b1 + a1 b3 + a2 b2 + a3 b1 up to
// 2^-24 relative, every bf16 product exact in the f32 accumulator.  launch_split3_pack writes the operand src(row, k) =
// src[row * s_row + k * s_k] as bf16 [rows, 6 K], the six K-long segments being (x3 x2 x1 x2 x1 x1) for the A operand
// (b_pattern 0) and (x1 x2 x3 x1 x2 x1) for the B operand (b_pattern 1), so that ONE bf16 GEMM over 6 K sums the six
// products — the 2^-16 terms first, then the 2^-8 terms, a1 b1 last.  The order matters: the tensor core adds into its
// f32 accumulator with truncation, an error of up to 2^-24 of the accumulator's magnitude per MMA step; with the large
// term last only K / 16 of the 6 K / 16 steps run at full magnitude (measured at K = 2048, unit-variance operands:
// largest error 4.2e-3 with a1 b1 first, against 2.7e-4 for an f32 FMA chain).  launch_gemm_epilogue_f32 then applies g's epilogue (the generic kernel's, element by element) to the f32
// result acc [M, N].  Non-finite inputs do not survive the split (Inf - Inf): the caller keeps such cases on the
// generic kernel only in so far as its shapes are small; a non-finite operand gives NaN here.
cudaError_t launch_split3_pack(cudaStream_t st, const float* src, long long s_row, long long s_k, int rows, int K, int b_pattern,
                               void* dst_bf16);
cudaError_t launch_gemm_epilogue_f32(cudaStream_t st, const GemmArgs& g, const float* acc);

// ---- elementwise / normalisation -------------------------------------------------------------
cudaError_t launch_convert_f32(cudaStream_t st, int dt, const float* in, void* out, size_t n);
cudaError_t launch_widen_to_f32(cudaStream_t st, int dt, const void* in, float* out, size_t n);
cudaError_t launch_fifo_batch(cudaStream_t st, const uint16_t* tokens, long long cursor, long long bt,
                              long long* inputs, long long* targets);
// tokens: device pointer to uint16_t (token_bytes 2) or uint32_t (4) tokens; starts: device array of `batch` offsets
cudaError_t launch_window_batch(cudaStream_t st, const void* tokens, int token_bytes, const unsigned long long* starts,
                                int batch, long long block, long long* inputs, long long* targets);
cudaError_t launch_embed_norm_fwd(cudaStream_t st, int dt, const void* wte, const long long* idx, int M, int d,
                                  int V, void* x, float* tsave);
// Embedding gradient without atomics: dwte[token] = sum of the rows of `rows` ([M, d], model dtype) whose token it is,
// added in ascending position order, so the result does not depend on timing (the reference's scatter has no such
// freedom either).  Tokens are sorted by a stable radix sort of (token, position); one block per distinct token walks its
// positions.  dwte must be zero where a token does not occur (the caller clears it).  scratch: embed_scatter_scratch_bytes.
size_t embed_scatter_scratch_bytes(int M, int d);
cudaError_t launch_embed_scatter_sorted(cudaStream_t st, int dt, const long long* idx, int M, int d, int V, const void* rows,
                                        void* scratch, size_t scratch_bytes, float* dwte);
// rows != nullptr: write the per-position gradient rows there instead of adding them into dwte
cudaError_t launch_embed_norm_bwd_rows(cudaStream_t st, int dt, const void* wte, const long long* idx, int M, int d, int V,
                                       const void* dy, const float* tsave, void* rows);
cudaError_t launch_embed_norm_bwd(cudaStream_t st, int dt, const void* wte, const long long* idx, int M, int d,
                                  int V, const void* dy, const float* tsave, float* dwte);
cudaError_t launch_rmsnorm_fwd(cudaStream_t st, int dt, const void* x, int M, int d, void* y, float* tsave);
// dx = dres + backward(dy) ; dres may be null, may alias dx
cudaError_t launch_rmsnorm_bwd(cudaStream_t st, int dt, const void* x, const float* tsave, const void* dy,
                               const void* dres, int M, int d, void* dx);
// RoPE (half split) + per-head RMSNorm of q and k.  qkv: [M, d + 2*dkv] raw projections.
// qkn: [M, d + dkv] normalised roped q then k.  tq: [M, H + Hkv] saved (mean square + eps).
cudaError_t launch_rope_qknorm_fwd(cudaStream_t st, int dt, const void* qkv, const uint16_t* cos_bf16,
                                   const uint16_t* sin_bf16, int M, int T, int H, int Hkv, int hd, void* qkn,
                                   float* tq);
// dqkn: [M, d + dkv] gradient wrt qkn -> writes q and k parts of dqkv [M, d + 2*dkv]
cudaError_t launch_rope_qknorm_bwd(cudaStream_t st, int dt, const void* qkv, const void* dqkn, const float* tq,
                                   const uint16_t* cos_bf16, const uint16_t* sin_bf16, int M, int T, int H,
                                   int Hkv, int hd, void* dqkv);

// ---- attention (generic path) -------------------------------------------------------------------
struct AttnArgs {
  const void* qkn;      // [M, d + dkv]
  const void* qkv;      // [M, d + 2 dkv]  (v part is read)
  void* o;              // [M, d]
  float* mrow;          // [B*H*T] row max of scaled masked scores
  float* lrow;          // [B*H*T] row sum of exp
  int B, T, H, Hkv, hd;
  float scale;          // 1/sqrt(hd) rounded to the model dtype
  // backward only
  const void* dout;     // [M, d]
  void* dqkn;           // [M, d + dkv]  (q part written; k part written by the finish pass)
  void* dqkv;           // [M, d + 2 dkv] (v part written by the finish pass)
  float* dkv_acc;       // [M, 2*dkv] f32 scratch: dk then dv, zeroed by the launcher
};
cudaError_t launch_attn_fwd_generic(cudaStream_t st, int dt, const AttnArgs& a);
// f32 models with 16-, 32-, 64- or 128-wide heads and T a multiple of 64: tiled SIMT kernels, backward without atomics
// (attn_f32.cu).
// drow: f32 scratch of at least B * H * T elements (the callers pass dkv_acc, which these kernels do not need).
bool attn_f32_supported(int dt, const AttnArgs& a);
cudaError_t launch_attn_f32_fwd(cudaStream_t st, const AttnArgs& a);
cudaError_t launch_attn_f32_bwd(cudaStream_t st, const AttnArgs& a, float* drow);     // 3 kernels
cudaError_t launch_attn_bwd_generic(cudaStream_t st, int dt, const AttnArgs& a);

// ---- nanoGPT family ---------------------------------------------------------------------------------
cudaError_t launch_embed_pos_fwd(cudaStream_t st, int dt, const void* wte, const void* wpe, const long long* idx, int M,
                                 int Tlen, int d, int V, void* x);
// dwte must be zeroed by the caller (atomic accumulation); dwpe is overwritten
cudaError_t launch_embed_pos_bwd(cudaStream_t st, int dt, const long long* idx, int B, int Tlen, int d, int V, const void* dx,
                                 float* dwte, float* dwpe);
cudaError_t launch_layernorm_fwd(cudaStream_t st, int dt, const void* x, const void* gamma, const void* beta, int M, int d,
                                 void* y, float* mean, float* tsave, double* mean64);
size_t layernorm_bwd_scratch_floats(int M, int d);
// dx = dres + backward(dy); dgamma / dbeta: f32, rounded to the model dtype, guarded and clamped
cudaError_t launch_layernorm_bwd(cudaStream_t st, int dt, const void* x, const void* gamma, const float* mean,
                                 const float* tsave, const double* mean64, const void* dy, const void* dres, int M, int d,
                                 void* dx, float* partial, float* dgamma, float* dbeta);
size_t colsum_scratch_floats(int M, int V);
cudaError_t launch_colsum(cudaStream_t st, int dt, const void* z, int M, int V, float* partial, float* out);
cudaError_t launch_copy_cols(cudaStream_t st, int dt, const void* src, long long src_pitch, void* dst, long long dst_pitch,
                             int M, int ncols);

// ---- soft-capped cross entropy -------------------------------------------------------------------
// logits [M,V] of model dtype are overwritten with d(loss)/d(logits).  rowloss[M]: per-row NLL (0 if
// ignored).  count: number of targets != ignore (device scalar, written by launch_count_valid).
// cap == 0 selects the plain cross entropy of the nanoGPT family (no soft-cap).
cudaError_t launch_count_valid(cudaStream_t st, const long long* targets, int M, long long ignore, float* count);
cudaError_t launch_softcap_ce(cudaStream_t st, int dt, void* logits, const long long* targets, int M, int V,
                              float cap, long long ignore, const float* count, float* rowloss, int write_grad,
                              float seed = 1.f);       // seed: d(loss) of model_forward_pass_grad
// Adjoint-edge status of the kernels in kernels.cu / kernels_gpt.cu / gemm_tc.cu / attn_tc.cu / attn_flash.cu on the
// current device (bits ADJ_CLAMPED, ADJ_INTERNAL of common.cuh), optionally cleared.  Blocks on `st`.
cudaError_t adj_status_fetch_kernels(cudaStream_t st, int* out, bool clear);
cudaError_t adj_status_fetch_kernels_gpt(cudaStream_t st, int* out, bool clear);
cudaError_t adj_status_fetch_gemm_tc(cudaStream_t st, int* out, bool clear);
cudaError_t adj_status_fetch_attn_tc(cudaStream_t st, int* out, bool clear);
cudaError_t adj_status_fetch_attn_flash(cudaStream_t st, int* out, bool clear);
cudaError_t adj_status_fetch_attn_f32(cudaStream_t st, int* out, bool clear);
cudaError_t launch_loss_finalize(cudaStream_t st, const float* rowloss, int M, const float* count, float* loss);

// ---- optimiser -----------------------------------------------------------------------------------
struct TensorSeg {          // one parameter tensor of a multi-tensor launch
  const float* p; const float* g; const float* m; const float* v;
  float* p_out; float* m_out; float* v_out;
  void* shadow;             // model-dtype copy of p_out, may be null
  long long n;
  int first_chunk;          // index of this tensor's first chunk
  int num_chunks;
};
struct AdamHyper {
  float lr, beta1, beta2, eps, wd, max_norm;
  float m_corr, v_corr;     // max(1 - beta^t, eps), computed on the host with powf
};
static const int ADAM_CHUNK = 8192;
// segs: device array of `nseg` TensorSeg; chunk2seg: device array mapping chunk -> segment;
// partial: device scratch of `nchunks` floats; normsq: device scratch of `nseg` floats.
cudaError_t launch_adamw(cudaStream_t st, int shadow_dt, const TensorSeg* segs, int nseg, const int* chunk2seg,
                         int nchunks, float* partial, float* normsq, AdamHyper h);
cudaError_t launch_axpy_f32(cudaStream_t st, float* acc, const float* g, float alpha, size_t n);   // acc += alpha*g
cudaError_t launch_scale_f32(cudaStream_t st, float* x, float alpha, size_t n);
// x = clamp(finite(round_to_dt(x)))   (gradient edge guard, src/autodiff/engine.zig:622-682)
cudaError_t launch_round_guard_f32(cudaStream_t st, int dt, float* x, size_t n, float clip);
// nonfinite m/v detection per segment (src/nodes/workers/worker.zig:1346-1369): flags[seg] = 1 if corrupt
cudaError_t launch_check_finite(cudaStream_t st, const float* x, size_t n, int* flag);

// ---- DiLoCo outer step ---------------------------------------------------------------------------
// delta = theta0 - theta (f32), truncated to bf16 precision if trunc != 0
cudaError_t launch_delta(cudaStream_t st, const float* theta0, const float* theta, float* delta, size_t n, int trunc);
// Shard update over [0,n): acc = sum_w deltas[w][i] (in order), /ncontrib, nonfinite -> 0,
// vel = mu*vel + acc, master = master - lr*(acc + mu*vel), master truncated to bf16 if trunc.
// Up to 8 delta pointers (peer or local memory).  outs: up to 8 destinations that receive the new master.
struct OuterArgs {
  const float* deltas[8]; int ncontrib;
  float* vel; float* master;
  float* outs[8]; int nouts;
  long long n; float lr, mu; int trunc;
  int keep_nonfinite;          // 0: a non-finite mean becomes 0 (DiLoCo outer step); 1: passed on (streaming path)
};
cudaError_t launch_nesterov_shard(cudaStream_t st, const OuterArgs& a);
// Streaming DiLoCo, worker side: delta = snapshot - theta, snapshot <- theta;  theta <- alpha*theta + (1-alpha)*global,
// snapshot <- theta.
cudaError_t launch_stream_delta(cudaStream_t st, float* snapshot, const float* theta, float* delta, size_t n);
cudaError_t launch_stream_merge(cudaStream_t st, float* theta, const float* global, float* snapshot, float alpha, size_t n);

}  // namespace pcpb
