// C launch interface of the kernels (no torch headers here: the .cu files compile in seconds).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// rows of the RMSNorm/RoPE backward that one warp reduces before it writes a weight-gradient partial (a CTA has 8 warps). The
// torch operator and the allocation-free entry point both pass this value, which is what makes their results bit-identical.
#define CB200_RMSNORM_BWD_ROWS_PER_WARP 64

extern "C" {
// elementwise.cu
int cb200_ln_groups_per_frame(int L, int rows_per_cta);
void cb200_ln_modulate_fwd(const void* x, const float* shift, const float* scale, void* y, float* mean, float* rstd,
                           long rows, int D, int L, float eps, cudaStream_t st);
void cb200_ln_modulate_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const float* scale,
                           void* dx, float* dshift, float* dscale, float* partials, long frames, int D, int L,
                           int rows_per_cta, cudaStream_t st);
void cb200_gate_residual_fwd(const void* x, const float* gate, const void* y, void* out, long rows, int D, int L,
                             cudaStream_t st);
void cb200_gate_residual_bwd(const void* dout, const float* gate, const void* y, void* dy, float* dgate, float* partials,
                             long frames, int D, int L, int rows_per_cta, cudaStream_t st);
void cb200_rmsnorm_rope_fwd(const void* x, const float* w, const float* cosv, const float* sinv, void* y, float* rstd,
                            long n_rows, int S, int H, int HD, float eps, cudaStream_t st);
long cb200_rmsnorm_bwd_blocks(long n_rows, int rows_per_warp);
void cb200_rmsnorm_rope_bwd(const void* dy, const void* x, const float* w, const float* rstd, const float* cosv,
                            const float* sinv, void* dx, float* dw, float* partials, long n_rows, int S, int H, int HD,
                            int rows_per_warp, cudaStream_t st);
void cb200_gelu_fwd(const void* x, void* y, long n, cudaStream_t st);
void cb200_gelu_bwd(const void* dy, const void* x, void* dx, long n, cudaStream_t st);
void cb200_cfg_combine(const float* c, const float* u, float* o, float g, long n, cudaStream_t st);
// sampler_ops.cu (return 0, or 1 when the shape is not served: the caller falls back)
int cb200_lincomb(const float* const* xs, const float* cs, int count, float* out, long n, cudaStream_t st);
int cb200_frame_blend(const float* x, const float* gt, const float* noise, const float* mask, const float* flag, void* out,
                      int out_bf16, long B, long C, long S, cudaStream_t st);
int cb200_grad_cast_norm_blocks(long n);
void cb200_grad_cast_norm(const void* g16, float* g32, float* sumsq, float* partials, float scale, long n, cudaStream_t st);
void cb200_adamw_ema_shard(float* master, const float* grad, float* m, float* v, float* ema, void* out16,
                           const float* clip_coef, float lr, float beta1, float beta2, float eps, float wd, long step,
                           float ema_beta, long n, cudaStream_t st);
void cb200_cast_f32_bf16(const float* src, void* dst, long n, cudaStream_t st);

// tangent.cu: value and directional derivative in one pass (forward-mode variants)
void cb200_ln_modulate_jvp(const void* x, const void* tx, const float* shift, const float* scale, const float* tshift,
                           const float* tscale, void* y, void* ty, long rows, int D, int L, float eps, cudaStream_t st);
void cb200_rmsnorm_rope_jvp(const void* x, const void* tx, const float* w, const float* cosv, const float* sinv, void* y, void* ty,
                            long n_rows, int S, int H, int HD, float eps, cudaStream_t st);

// skinny.cu: Z small fp32 GEMMs C[z][r,n] = sum_k fa(A[z][r,k]) fb(B[z][n,k]) (+ add[r,n], n < add_cols) with element strides;
// ksplit > 1: C is [Z * ksplit, R, N] partial sums over ranges of k (the caller adds them)
int cb200_skinny_bgemm(const float* a, long a_z, long a_r, long a_k, const long long* b_ptrs, const void* b_base, long b_z, long b_n,
                       long b_k, int b_is_bf16, void* c, long c_z, int ldc, int c_is_bf16, const float* add, int ld_add, int add_cols,
                       int Z, int R, int N, int K, int silu_a, int silu_b, int ksplit, cudaStream_t st);

// gemm_tcgen05.cu
int cb200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int a_mn, int b_mn, const void* bias,
                    int act, void* pre, const void* resid, const float* gate, int L, int* err, int sms, cudaStream_t st);
int cb200_gemm_pair_mode(int mode);   // 0 / 1 sets, -1 reads; returns the previous mode (1 = CTA-pair tiles where the shape allows)
int cb200_gemm_bf16_gather(const void* A, void* ws, void* C, int M, int rows, int ld, int b_mn, const int64_t* shard_ptrs, int P,
                           int chunk_rows, int* counters, const void* bias, int act, void* pre, int* err, int sms, cudaStream_t st);
int cb200_gemm_bf16_scatter_heads(const void* A, const void* W, int M, int N, int K, const int64_t* ptrs, int P, int rank, int S,
                                  const float* norm_w, const float* cosv, const float* sinv, float eps, void* raw, float* rstd_out, int* err, int sms,
                                  cudaStream_t st);
}

extern "C" {
// fa_fwd.cu
int cb200_fa_fwd_scatter_seq(const void* q, const void* k, const void* v, const int64_t* out_ptrs, int P, int rank, float* lse,
                             int B, int Sq, int Skv, int H, float scale, int* err, cudaStream_t st);
int cb200_fa_fwd_na(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int H, float scale,
                    const int* kv_idx, const int* kv_cnt, int max_n, const uint8_t* bt, const uint8_t* bh, const uint8_t* bw, int nT,
                    int nH, int nW, int* err, cudaStream_t st);
// neighbourhood attention backward; every tensor in tile order (128-row tile = one 4 x 4 x 8 token box); q_list [S/128][max_n]
// (top bit: whole tile pair visible), q_cnt [S/128]; transposed visibility tables bt [4 nT][nT], bh [4 nH][nH], bw [8 nW][nW]
long cb200_fa_bwd_na_scratch_floats(int B, int S, int H);
int cb200_fa_bwd_na(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* lse, void* dq, void* dk,
                    void* dv, float* scratch, int B, int S, int H, float scale, const int* q_list, const int* q_cnt, int max_n,
                    const uint8_t* bt, const uint8_t* bh, const uint8_t* bw, int nT, int nH, int nW, int* err, cudaStream_t st);
int cb200_fa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Skv, int H, float scale,
                 int variant, int* err, cudaStream_t st);
}

extern "C" {
// peer.cu
void cb200_peer_barrier(const int64_t* flag_ptrs, int rank, int P, unsigned epoch, unsigned max_spins, int* err, cudaStream_t st);
int cb200_rs_blocks_x(void);
void cb200_rs_cast_norm_peer(const int64_t* grad_ptrs, const void* segs, int nseg, float* g32, float* partials, float* unit_sumsq,
                             float* total_sumsq, int rank, int P, float scale, cudaStream_t st);
void cb200_adamw_push_peer(const int64_t* full_ptrs, const int64_t* sumsq_ptrs, const void* segs, int nseg, float* master,
                           const float* grad, float* m, float* v, float* ema, int rank, int P, float max_norm, float lr,
                           float beta1, float beta2, float eps, float wd, long step, float ema_beta, float* norm_out,
                           cudaStream_t st);
void cb200_a2a_scatter_heads_peer(const void* x, const int64_t* out_ptrs, const float* w, const float* cosv, const float* sinv,
                                  float* rstd, long n_rows, int S, int H, int HD, int rank, int P, int norm, float eps,
                                  cudaStream_t st);
void cb200_a2a_gather_seq_peer(const int64_t* src_ptrs, void* out, long B, int S, int H, int HD, int rank, int P, cudaStream_t st);
void cb200_gather_slots_peer(const int64_t* shard_ptrs, const void* segs, int nseg, void* full, int P, cudaStream_t st);
}

extern "C" {
// fa_jvp.cu
int cb200_fa_jvp(const void* q, const void* k, const void* v, const void* tq, const void* tk, const void* tv, const void* o,
                 const float* lse, void* to, int B, int Sq, int Skv, int H, float scale, int* err, cudaStream_t st);

// fa_bwd.cu
int cb200_fa_bwd_scratch_floats(int B, int Sq, int H);
long cb200_fa_bwd_scratch_floats_v(int B, int Sq, int Skv, int H, int variant);
int cb200_fa_bwd_v(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* lse, void* dq, void* dk,
                   void* dv, float* scratch, int B, int Sq, int Skv, int H, float scale, int variant, int* err, cudaStream_t st);
int cb200_fa_bwd(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* lse, void* dq, void* dk,
                 void* dv, float* scratch, int B, int Sq, int Skv, int H, float scale, int* err, cudaStream_t st);
}

extern "C" {
// conv3d_cl.cu
int cb200_conv_cl(const void* x, int T_in, int H_in, int W_in, int Cin, const void* w, int n_rows, int n_tile, int Cout,
                  const int* taps, int ntaps, int T_out, int H_out, int W_out, const int* out_map, void* y, const void* resid,
                  const float* bias, int* err, int sms, cudaStream_t st);
int cb200_rmsnorm_silu_cl(const void* x, const float* gamma, void* y, long n_vox, int C, int silu, cudaStream_t st);
}
