// C ABI of libaeris_b200.so. Every function returns 0 on success and a negative code on a host-side argument or
// launch error. Kernels report device-side problems (bounded waits that ran out, failed bounds checks) through
// the `status` word, which the caller owns and reads after synchronising.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

int aeris_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                    int a_mn, int b_mn, int epi, const void* resid, int ldr, const float* gate,
                    int rows_per_gate, void* aux, int ld_aux, int swiglu_f, int k_splits, int bn, int* status,
                    void* stream);

int aeris_gemm_bf16_2cta(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                         int a_mn, int b_mn, int epi, const void* resid, int ldr, const float* gate,
                         int rows_per_gate, void* aux, int ld_aux, int swiglu_f, int k_splits, int* status,
                         void* stream);

int aeris_attn_fwd(const void* q, int ldq, int q_col0, const void* k, int ldk, int k_col0, const void* v, int ldv,
                   int v_col0, void* o, int ldo, float* lse, int n_win, int N, int H, int head_dim, float scale,
                   int* status, void* stream);

int aeris_attn_bwd(const void* qkv, int ldq, int q_col0, int k_col0, int v_col0, const void* o, const void* d_o,
                   int ldo, const float* lse, float* delta, void* dqkv, int ldg, int n_win, int N, int H,
                   int head_dim, float scale, int* status, void* stream);

int aeris_gemm_scatter_heads(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int b_mn,
                             const void* const* peers, int sp, int sp_rank, int n_local, int L, int sec_w, int* status,
                             void* stream);
// Variant of the attention forward kernel: poly = softmax arithmetic at head_dim 64 (-1 scalar; 0 two-wide; 2 two-wide
// with two of every eight score pairs on the polynomial exp2); p_in_tmem = probabilities kept in tensor memory as the
// A operand of P V. Returns non-zero for an unknown variant.
int aeris_attn_set_fwd_variant(int poly, int p_in_tmem);
// Checking build (-DAERIS_BOUNDS_CHECK) only: status word and source rows for the gathers launched next; returns 1 when
// the library validates gather codes, 0 when it was built without the checks.
int aeris_debug_set_gather_bounds(int* status, unsigned src_rows);
int aeris_attn_fwd_push(const void* qkv, int ld, int H_local, void* o, int ldo, float* lse, int n_win, int N,
                        int head_dim, float scale, const void* const* o_peers, int sp, int n_local, int push_ld,
                        int push_col0, int* status, void* stream);
int aeris_attn_bwd_push(const void* qkv, int ld, int H_local, const void* o, const void* d_o, int ldo, const float* lse,
                        float* delta, int n_win, int N, int head_dim, float scale, const void* const* dq_peers, int sp,
                        int n_local, int push_ld, int push_sec_w, int push_col0, int* status, void* stream);

// `w` is the bf16 norm weight, or null with the fp32 weight in `w_f32`; `h_lo` (optional) receives the bf16 rounding
// residual of `h`, so that h + h_lo carries the fp32 result (used by the fp32 output head).
int aeris_modnorm_fwd(const void* x, const void* gidx, const void* const* peer_ptrs, int n_peers, void* x_out,
                      const float* scale, const float* shift, const void* w, void* h, int rows, int D, int mode,
                      float eps, const float* w_f32, void* h_lo, void* stream);
int aeris_modnorm_bwd(const void* x, const void* dh, const void* dres, const float* scale, const float* shift,
                      const void* w, void* dx, float* dscale, float* dshift, float* dw, int rows, int D, int mode,
                      float eps, const float* w_f32, void* stream);
int aeris_gather_rows(const void* gidx, const void* const* peer_ptrs, int n_peers, void* out, long long rows, int D,
                      void* stream);
int aeris_swiglu_fwd(const void* u, void* act, long long rows, int F, void* stream);
int aeris_swiglu_bwd(const void* u, const void* dact, void* du, long long rows, int F, void* stream);
int aeris_scale_rows(const void* W, const float* g, void* Wg, int R, int C, void* stream);
// In-place 2-D rotary embedding of the q and k sections of qkv [rows, 3 * heads * d] (bf16); cos / sin: [L, d / 2] fp32.
int aeris_rope_qk(void* qkv, const float* cos_t, const float* sin_t, long long rows, int L, int heads, int d, int inverse,
                  void* stream);
int aeris_gate_grad_finalize(float* G, const void* W, const float* g, float* dW, float* dg, int R, int C,
                             void* stream);
int aeris_sumsq(const float* x, long long n, double* out, void* stream);
int aeris_adamw(float* master, float* grad, float* m, float* v, void* wbf16, float* ema, const double* norm_sq,
                long long n, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                float grad_scale, float max_norm, float ema_beta, void* stream);

int aeris_signal_barrier(const void* const* flag_ptrs, int rank, int world, unsigned epoch, int* status,
                         double timeout_s, void* stream);
int aeris_wait_flag(const void* flag, unsigned expected, int* status, double timeout_s, void* stream);
int aeris_grad_reduce_scatter(const void* const* grad_ptrs, const void* mc_grad, int world, long long lo, long long n,
                              float scale, float* out, double* sumsq, void* stream);
int aeris_shard_adamw_allgather(float* master, const float* grad, float* m, float* v, float* ema,
                                const void* const* param_ptrs, void* mc_params, int world, long long lo, long long n,
                                const double* norm_sq, float lr, float beta1, float beta2, float eps,
                                float weight_decay, int step, float max_norm, float ema_beta, void* stream);

int aeris_gemm_allgather_a(void* A, const void* const* peers, const void* const* counter_peers, int world, int rank,
                           int rows_per_rank, unsigned call_index, const void* B, void* C, int N, int K, int ldb,
                           int ldc, int b_mn, int epi, const void* resid, int ldr, void* aux, int ld_aux, int swiglu_f,
                           int* status, void* stream);
int aeris_gemm_rs_push(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int b_mn,
                       const void* const* peers, int world, int rank, int rows_per_rank, int ld_dst, int* status,
                       void* stream);
int aeris_rs_finalize(const void* slots, int world, long long rows, int D, const void* resid, const float* gate,
                      void* out, void* stream);

// Geometry of one rank's token stream and image block (see csrc/diffusion.cu).
typedef struct TokGeom {
  int B, nwy_loc, nwx_loc, ws_y, ws_x, n_local, sp_rank;
  int y0, x0, H, W;
  long long sample0;
} TokGeom;
int aeris_embed_pack(const float* x_img, const float* c_img, const float* cs, const TokGeom* g, int Cx, int Cc,
                     const float* ape_y, const float* ape_x, int ape_ch, unsigned long long seed, float sd, int noise,
                     void* out, int KP, long long row0, long long rows, void* stream);
int aeris_trigflow_loss(const float* pred, int ldp, const float* x_img, const float* cs, const TokGeom* g, int Cx,
                        unsigned long long seed, float sd, const float* w_var, const float* w_lat, float inv_rows,
                        float gscale, void* dpred, int ldd, double* loss, long long row0, long long rows, void* stream);
int aeris_sampler_update(float* x_out, const float* x_base, const float* pa, const float* pb, int ldp, float ca,
                         float cb, const TokGeom* g, int Cx, void* stream);
int aeris_noise_mix(float* x, float a, float b, unsigned long long seed, const TokGeom* g, int Cx, void* stream);
int aeris_affine_channels(float* out, const float* in, const float* a, const float* b, const float* add, long long n,
                          int C, void* stream);
int aeris_gemv_bias_act(const void* W, int w_f32, const float* bias, const float* x, float* y, int N, int K, int B,
                        int act, int silu_in, void* stream);

#ifdef __cplusplus
}
#endif
