// C ABI of the necklace_b200 native library (loaded from Python with ctypes).
//
// Conventions: every function returns 0 on success, a positive cudaError_t or a
// negative library error.  Pointers are device pointers unless named host_*.
// `stream` is a cudaStream_t passed as void*.  Nothing here allocates device
// memory: callers own inputs, outputs and scratch.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// GEMM epilogue selectors
#define NKB_EPI_NONE 0
#define NKB_EPI_GELU_FWD 1  // aux <- (acc+bias) ; C <- gelu(acc+bias)
#define NKB_EPI_GELU_BWD 2  // C <- acc * gelu'(aux)
#define NKB_EPI_RELU 3

// ---- gemm_sm100.cu ---------------------------------------------------------
// C[M,N] = epi(alpha * A[M,K] * B[N,K]^T + bias) + res.  a_mn / b_mn = 1 when the
// operand is stored with its M / N index contiguous ([K][ld] in memory).
int nkb_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
                  void* C, long long ldc, int c_fp32, int accumulate, int M, int N, int K,
                  float alpha, const void* bias, const void* res, long long ldres, int epi,
                  void* aux, long long ldaux, int* status, const int* ready_flags,
                  int rows_per_flag, int ready_target, int max_ctas, int bn_hint,
                  const float* alpha_dev, void* stream);

// ---- norm.cu ---------------------------------------------------------------
// rms = 1: RMSNorm (no mean, no bias).  stats: [rows,2] fp32 (mean, rstd).
int nkb_norm_fwd(const void* x, const void* w, const void* b, void* y, float* stats, int rows,
                 int C, float eps, int rms, void* stream);
int nkb_norm_bwd_dx(const void* dy, const void* x, const void* w, const float* stats, void* dx,
                    int rows, int C, int rms, void* stream);
// same, plus dres [rows, C] (bf16): the gradient that reaches x along a residual connection
int nkb_norm_bwd_dx_res(const void* dy, const void* x, const void* w, const float* stats, void* dx,
                        int rows, int C, int rms, const void* dres, void* stream);
// Column sums over rows: acc[0][c] += sum_r dy[r,c]*xhat[r,c] (if x) ; acc[1][c] += sum_r dy[r,c].
// `acc` is fp32 [2][C] scratch that must be zero on entry.
int nkb_colsum(const void* dy, const void* x, const float* stats, float* acc, int rows, int C,
               long long ld, int rms, void* stream);
// Column sums straight to bf16 outputs in one launch (the last CTA of a column strip converts
// and re-zeroes).  acc (fp32 [2][C]) and tickets (int [ceil(C/256)]) are caller-owned, zero
// before the first call and left zero; calls sharing them must be ordered on one stream.
int nkb_colsum_fused(const void* dy, const void* x, const float* stats, float* acc, int* tickets,
                     void* out_a, void* out_b, int accum_a, int accum_b, int rows, int C,
                     long long ld, int rms, void* stream);
// out_bf16[i] = (accumulate ? out[i] : 0) + acc[i]
int nkb_f32_to_bf16(const float* src, void* dst, long long n, int accumulate, void* stream);

// ---- loss_embed.cu ---------------------------------------------------------
// logits [T, ld] bf16 (first V columns valid) are overwritten with
// dlogits = (softmax - onehot) * grad_scale ; columns >= V get 0 ; losses[t] = -log p[target].
// Rows with target < 0 are ignored (loss 0, grad 0).
int nkb_ce_fwd_bwd(void* logits, const long long* targets, float* losses, int T, int V,
                   long long ld, float grad_scale, void* stream);
// Two-phase form for a vocabulary split over ranks: local stats [T,3] = (max, sumexp, target logit or 0)
int nkb_ce_stats(const void* logits, const long long* targets, float* stats, int T, int V,
                 long long ld, int vocab_start, void* stream);
// grads from global (max, sumexp) per row: stats_g [T,2]
int nkb_ce_grad(void* logits, const long long* targets, const float* stats_g, int T, int V,
                long long ld, int vocab_start, float grad_scale, void* stream);
int nkb_embed_fwd(const long long* idx, const void* wte, const void* wpe, void* out, int T, int S,
                  int C, int vocab_start, int vocab_rows, void* stream);
int nkb_embed_bwd(const long long* idx, const void* dout, void* dwte, void* dwpe, int T, int S,
                  int C, int vocab_start, int vocab_rows, void* stream);

// ---- conv.cu ----------------------------------------------------------------
// NHWC bf16.  col [N*Ho*Wo, Kpad], K index = (kh*KW + kw)*C + c, Kpad >= KH*KW*C, Kpad % 8 == 0.
int nkb_im2col_nhwc(const void* x, void* col, int N, int H, int W, int C, int KH, int KW,
                    int stride, int pad, int Kpad, void* stream);
int nkb_col2im_nhwc(const void* dcol, void* dx, int N, int H, int W, int C, int KH, int KW,
                    int stride, int pad, int Kpad, void* stream);
// Training-mode batch norm over the rows of x [M, C] (+ residual, + ReLU).  acc: fp32 [2][C]
// scratch, zero on entry and on exit; stats: fp32 [2][C] = (mean, rstd).
int nkb_bn_fwd(const void* x, const void* gamma, const void* beta, const void* res, void* y,
               float* stats, float* acc, float* run_mean, float* run_var, long long M, int C,
               float eps, float momentum, int relu, void* stream);
int nkb_bn_apply(const void* x, const float* stats, const void* gamma, const void* beta,
                 const void* res, void* y, long long M, int C, int relu, void* stream);
int nkb_bn_bwd(const void* dy, const void* x, const void* y, const float* stats, const void* gamma,
               void* dx, void* dres, void* dgamma, void* dbeta, int acc_g, int acc_b, float* acc,
               long long M, int C, int relu, void* stream);
int nkb_maxpool3x3s2_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C,
                         void* stream);
int nkb_maxpool3x3s2_bwd(const void* dy, const void* idx, void* dx, int N, int H, int W, int C,
                         void* stream);
int nkb_avgpool_fwd(const void* x, void* y, int N, int HW, int C, void* stream);
int nkb_avgpool_bwd(const void* dy, void* dx, int N, int HW, int C, void* stream);

// ---- optim_quant.cu --------------------------------------------------------
// Adam / AdamW on flat buffers; master fp32, optional bf16 copy out. grad dtype: 0 bf16, 1 fp32.
int nkb_adam_flat(float* master, float* m, float* v, const void* grad, int grad_fp32,
                  void* param_bf16, long long n, float lr, float beta1, float beta2, float eps,
                  float weight_decay, float bias_c1, float bias_c2, float grad_scale,
                  const float* hyper_dev /* optional device {lr, c1, c2, t, gmul} */, void* stream);
// hyper = device floats {lr, c1, c2, t}: t += 1 and the Adam bias corrections follow from t.
int nkb_hyper_advance(float* hyper, float beta1, float beta2, void* stream);
// SGD with momentum on flat buffers (torch.optim.SGD semantics, dampening 0).
int nkb_sgd_flat(float* master, float* mom, const void* grad, int grad_fp32, void* param_bf16,
                 long long n, float lr, float momentum, float weight_decay, float grad_scale,
                 int first_step, const float* hyper_dev /* optional {lr, .., .., .., gmul} */,
                 void* stream);
// hyper[4] = min(1, max_norm / (sqrt(*sumsq) * gscale)); hyper[5] = the norm.
int nkb_clip_coef(float* hyper, const float* sumsq, float max_norm, float gscale, void* stream);
// 2-bit threshold codec with error feedback over a flat fp32/bf16 vector:
//   a = g[i] + residual[i]; code 01 if a >= thr, 10 if a <= -thr, else 00;
//   residual[i] = a - decode(code); 16 codes per uint32, element i in bits [2(i%16), 2(i%16)+2).
int nkb_quant2_flat(const void* g, int g_fp32, float* residual, uint32_t* codes, long long n,
                    float thr, void* stream);
int nkb_dequant2_flat(const uint32_t* codes, void* out, int out_fp32, long long n, float thr,
                      float scale, int accumulate, void* stream);
// Matrix form with the packing of the reference kernels (16 rows -> one word):
// codes[x, y] packs A[16x+i, y], i = 0..15.  A, R: fp32 [n, ncol]; codes: [ceil(n/16), ncol].
int nkb_quant2_matrix(const float* A, uint32_t* codes, float* R, int n, int ncol, float thr,
                      void* stream);
int nkb_dequant2_matrix(float* A, const uint32_t* codes, int n, int ncol, float thr, void* stream);
// flat helpers
int nkb_scale_cast(const void* src, int src_fp32, void* dst, int dst_fp32, long long n,
                   float scale, int accumulate, void* stream);
int nkb_sumsq(const void* src, int src_fp32, long long n, float* out_accum, void* stream);

// ---- attention_sm100.cu ------------------------------------------------------
// Causal (or full) multi-head attention, head dim 64 or 128.  q,k,v,o: bf16 with
// element strides (batch, head, seq); the head dim is contiguous.  lse: [B,H,S] fp32.
int nkb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H,
                 int S, int D, long long sb, long long sh, long long ss, long long ob,
                 long long oh, long long os, float scale, int causal, int* status, void* stream);
// delta: [B,H,S] fp32 scratch; dq_acc: [B,H,S,D] fp32 scratch (both written by the call itself).
int nkb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                 const float* lse, void* dq, void* dk, void* dv, float* delta, float* dq_acc,
                 int B, int H, int S, int D, long long sb, long long sh, long long ss,
                 long long ob, long long oh, long long os, float scale, int causal, int* status,
                 void* stream);

// ---- comm.cu -----------------------------------------------------------------
// Peer-memory collectives over a symmetric heap.  `heap` is a device array of
// `world` base pointers (index = rank within the group); buffers are byte offsets
// into every member's heap.  The flag region (nkb_comm_flag_bytes() bytes, zeroed
// once) sits at `flag_off`.  `epoch` is a device int[2] (zeroed once) owned by the
// group: the kernels advance it, so calls can be replayed from a CUDA graph.
int nkb_comm_flag_bytes(void);
int nkb_comm_barrier(void** heap, long long flag_off, int rank, int world, int* epoch, int* status,
                     void* stream);
// in-place sum (times scale) of n elements at data_off; fp32 = 1 float, 0 bf16
int nkb_comm_allreduce(void** heap, long long flag_off, long long data_off, long long n, int fp32,
                       float scale, int rank, int world, int* epoch, int* status, int max_ctas,
                       void* stream);
// member r's shard is at data_off + r*shard_bytes; afterwards every member has all shards
int nkb_comm_reduce_scatter(void** heap, long long flag_off, long long data_off, long long n,
                            int fp32, float scale, void* out, int rank, int world, int* epoch,
                            int* status, int max_ctas, void* stream);
int nkb_comm_bcast(void** heap, long long flag_off, long long data_off, long long nbytes, int root,
                   int rank, int world, int* epoch, int* status, int max_ctas, void* stream);
int nkb_comm_allgather(void** heap, long long flag_off, long long data_off, long long shard_bytes,
                       int rank, int world, int* epoch, int* status, int max_ctas, void* stream);
// 2-bit compressed gradient all-reduce with error feedback, one kernel:
// out = scale * thr * sum_ranks sign-code(g + residual); residual updated in place.
// codes_off: uint32[ceil(n/16)], counts_off: int8[16*ceil(n/16)] in the heap.
int nkb_comm_dp_quant_allreduce(void** heap, long long flag_off, const void* g, int g_fp32,
                                float* residual, long long codes_off, long long counts_off,
                                void* out, int out_fp32, long long n, float thr, float scale,
                                int rank, int world, int* epoch, int* status, int max_ctas,
                                void* stream);
// ZeRO step in one kernel: reduce-scatter of bf16 grads (grad_off) + Adam/SGD on this
// rank's fp32 shard + all-gather of the new bf16 params (param_off) into every heap.
// n_total % (8*world) == 0; master/s1/s2 hold n_total/world floats.
int nkb_comm_rs_opt_ag(void** heap, long long flag_off, long long grad_off, long long param_off,
                       long long n_total, float* master, float* s1, float* s2, int adam, float lr,
                       float beta1, float beta2, float eps, float wd, float c1, float c2,
                       float gscale, int first_step, const float* hyper_dev, int rank, int world,
                       int* epoch, int* status, int max_ctas, void* stream);

// ---- elementwise.cu ----------------------------------------------------------
// Rotary embedding in place on q and k of a packed [T, 3*H*D] bf16 buffer
// (pairs (i, i + D/2), angle = (t % S + pos_offset) * base^(-2i/D)); backward = inverse.
int nkb_rope(void* qkv, int T, int S, int H, int D, float base, int backward, int pos_offset,
             void* stream);
// gu = [T, 2F] (gate | up) ; h = silu(gate) * up ; dgu from dh
int nkb_swiglu_fwd(const void* gu, void* h, long long T, int F, void* stream);
int nkb_swiglu_bwd(const void* gu, const void* dh, void* dgu, long long T, int F, void* stream);

int nkb_num_sms(void);
const char* nkb_build_info(void);

#ifdef __cplusplus
}
#endif
