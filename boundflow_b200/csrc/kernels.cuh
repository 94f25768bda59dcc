// Internal launchers shared between the C-ABI wrappers and the chain drivers.
#pragma once
#include "common.cuh"

namespace bf {

// crown_linear.cu
int launch_crown_bwd_linear(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                            const float* add, const float* W, const float* kbias, float* A_prev, float* delta,
                            int accumulate, const float* mid, const float* rad, float* partial, int side, int M, int S,
                            int K, int N, cudaStream_t stream);
int crown_bwd_partial_tiles(int N, int M = 0);  // M <= 0: the largest count any M gives (workspace sizing)
// true when the 64 x 64 tiles of the FFMA contraction kernels cover an [M,N] result in one wave (two CTAs per SM)
bool ffma_fits_one_wave(int M, int N);
int launch_crown_adjoint_linear(const float* Hprev, int first_layer, const float* mid, const float* rad, const float* W,
                                const float* nbias, const float* Ahat, const float* dpos, const float* dneg,
                                const float* epos, const float* eneg, const float* pre_l, const float* pre_u,
                                float* hout, float* grad, float* gsum, int M, int S, int K, int N, cudaStream_t stream,
                                const float* gw = nullptr);

// crown_tc.cu (tcgen05 3xTF32 path; weights pre-packed by tc_pack_weights)
size_t tc_packed_bytes(int N, int K, int tile_rows = 0);
int tc_pack_weights(const float* W, int rows, int cols, int transposed, unsigned char* out, cudaStream_t stream, int tile_rows = 0);
int launch_crown_bwd_linear_tc(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                               const float* add, const unsigned char* Wpk, const float* kbias, float* A_prev, float* delta,
                               int accumulate, const float* mid, const float* rad, float* partial, int side, int M, int S, int K,
                               int N, int* status, cudaStream_t stream, bool cta_pairs = false);
int launch_crown_adjoint_linear_tc(const float* Hprev, int first_layer, const float* mid, const float* rad,
                                   const unsigned char* Wpk, const float* nbias, const float* Ahat, const float* dpos,
                                   const float* dneg, const float* epos, const float* eneg, const float* pre_l,
                                   const float* pre_u, float* hout, float* grad, float* gsum, int M, int S, int K, int N,
                                   int* status, cudaStream_t stream, const float* gw = nullptr);
int crown_tc_partial_tiles(int N, int K);
void tc_tile_shape(int N, int K, int* BN, int* ntiles, int* nkb);

// crown_tc_persist.cu (persistent, warp-specialised backward contraction; same packed weights as crown_tc.cu)
int launch_crown_bwd_linear_tc_persistent(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                                          const float* add, const unsigned char* Wpk, const float* kbias, float* A_prev,
                                          float* delta, int accumulate, const float* mid, const float* rad, float* partial,
                                          int side, int M, int S, int K, int N, int* status, cudaStream_t stream);
bool crown_tc_persistent_supports(const float* epos, const float* eneg, const float* add);  // else: the classic kernel
int crown_tc_persist_partial_tiles(int M, int N, int K);  // column tiles (= partial sums per row) for this problem
int crown_tc_persist_max_partial_tiles(int N);            // upper bound over every M (workspace sizing)

// crown_tc_adj.cu (feature-major adjoint step; weights packed with tile_rows = tc_adjoint_tile_rows())
int tc_adjoint_tile_rows();
int launch_crown_adjoint_linear_tc_fm(const float* Hprev, int first_layer, const float* mid, const float* rad,
                                      const unsigned char* Wpk, const float* nbias, const float* Ahat, const float* dpos,
                                      const float* dneg, const float* epos, const float* eneg, const float* pre_l,
                                      const float* pre_u, float* hout, float* grad, float* gsum, int M, int S, int K, int N,
                                      int* status, cudaStream_t stream);

// ibp.cu
int launch_ibp_linear(const float* in_a, const float* in_b, int in_mode, int relu_in, const float* W, const float* bias,
                      const int8_t* split, int split_stride, const float* cons_l, const float* cons_u, float* out_l,
                      float* out_u, int* infeasible, int B, int K, int N, const float* row_dev, cudaStream_t stream);
int launch_row_dual_norm(const float* rows, int n_rows, int n, int p, float scale, float* out, cudaStream_t stream);
int launch_h0_lp(float* A, const float* center, float eps, int p, int B, int S, int n0, cudaStream_t stream);
int launch_concretize_lp(const float* A, const float* center, const float* bias_in, float* out, int side, float eps, int p, int B,
                         int S, int n0, cudaStream_t stream);

// elementwise.cu
int launch_relu_relax(const float* l, const float* u, const float* alpha, int alpha_stride, float* alpha_u,
                      float* beta_u, float* alpha_l, int B, int n, cudaStream_t stream);
int launch_concretize(const float* A, const float* mid, const float* rad, const float* bias_in, float* out, int side,
                      int B, int S, int n0, cudaStream_t stream);
// lower[m] = c[m] + sum_t partial[m,t]; out may alias nothing else
int launch_sum_partials(const float* c, const float* partial, int ntiles, float* out, int M, cudaStream_t stream);
// per-domain objective + strict best-of tracking (first != 0 initialises)
int launch_select_best(const float* cur, float* best_lower, float* best_metric, int* improve, int first,
                       int spec_reduce, float soft_tau, float* row_weight, int B, int S, cudaStream_t stream);
// the same for paired spec rows (S rows followed by their negations) and the gap / both objectives
int launch_select_best_paired(const float* cur, float* best_rows, float* best_metric, int* improve, int first, int objective,
                              int spec_reduce, float soft_tau, float lb_weight, float ub_weight, float* row_weight, int B, int S,
                              cudaStream_t stream);
int launch_scale_rows(float* A, const float* w, long long M, int n, cudaStream_t stream);
struct AdamScalars {
  float lr_step;      // lr / (1 - beta1^t)
  float bc2_sqrt;     // sqrt(1 - beta2^t)
  float beta1, beta2, eps;
  float one_minus_beta1, one_minus_beta2;
  float grad_scale;   // -1/S (mean) or -1 (sum): d loss / d lower
};
// Snapshot of the best alpha (where improve[b]), Adam update + projection to [0,1], and the
// lower slope for the next evaluation.  grad is scaled by grad_scale before use and zeroed.
int launch_adam_step(float* alpha, float* m, float* v, float* grad, const int* improve, float* best_alpha,
                     const float* pre_l, const float* pre_u, float* slope_l, AdamScalars sc, int do_update, int B, int n,
                     cudaStream_t stream);
int launch_scale_copy(const float* src, float scale, float* dst, long long n, cudaStream_t stream);
int launch_colmax_abs(const float* A, float* out, int B, int S, int n, cudaStream_t stream);
int launch_relu_adjoint_rows(float* G, const float* Ahat, const float* dpos, const float* dneg, const float* eneg,
                             const float* pre_l, const float* pre_u, float* grad, float* gsum, int B, int S, int n,
                             cudaStream_t stream, const float* gw = nullptr);
int launch_interval_intersect(float* l, float* u, const float* cl, const float* cu, int* infeasible, int B, int n, cudaStream_t stream);
int launch_h0_box(float* A0, const float* mid, const float* rad, int B, int S, int n0, cudaStream_t stream);
// windowed coefficient rows of identity-row sweeps on conv layers (conv.cu)
struct WindowGeom {
  int M;                 // coefficient rows
  int first, S;          // spec row m is identity row first + m % S of the bounded value
  int HoB, WoB;          // spatial size of the bounded value (row j -> channel j / (HoB*WoB), pixel (ho, wo))
  int C, WH, WW;         // window of the current value
  int H, W;              // feature-map size of the current value
  int sy, ty, sx, tx;    // window origin: (ho*sy + ty, wo*sx + tx)
};
int launch_onehot_conv_window(const float* W, const float* bias, float* out, float* delta, const WindowGeom& w, int M, int Ci, int kk,
                              cudaStream_t stream);
int launch_relu_bwd_window(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                           const float* bias, float* Lam, float* delta, const WindowGeom& w, int M, cudaStream_t stream);
int launch_window_to_dense(const float* Awin, float* dense, const WindowGeom& w, int M, cudaStream_t stream);
int launch_concretize_window(const float* Awin, const float* mid, const float* rad, const float* delta, float* out, int side,
                             const WindowGeom& w, int M, cudaStream_t stream);
// shared-alpha mode (one alpha per neuron for the whole batch)
int launch_shared_metric(const float* cur, long long M, float* best_metric, int* improve, int first, cudaStream_t stream);
int launch_copy_if(const float* src, float* dst, long long n, const int* flag, cudaStream_t stream);
int shared_alpha_chunks(int B);
int launch_shared_adam(float* param, float* m, float* v, float* grad, const int8_t* split, int split_stride, float* part,
                       const int* improve, float* best, AdamScalars sc, int do_update, int is_beta, int B, int n,
                       cudaStream_t stream);
int launch_shared_beta_add(const float* beta, const int8_t* split, int split_stride, float* add, int B, int n, cudaStream_t stream);
// beta parameters: snapshot, Adam step with gradient -split * gsum * grad_scale, projection to >= 0,
// and the next split term add = -beta * split (split in {-1,0,+1}; entries with split == 0 never move)
int launch_beta_step(float* beta, float* m, float* v, float* gsum, const int8_t* split, int split_stride, const int* improve,
                     float* best_beta, float* add, AdamScalars sc, int do_update, int B, int n, cudaStream_t stream);
int launch_verdict(const float* lower, float threshold, float tol, const int* infeasible, int8_t* verdict, float* min_lower,
                   int B, int S, cudaStream_t stream);
int launch_poison_on_status(const int* status, float* a, long long na, float* b, long long nb, cudaStream_t stream);
// building blocks for graphs that are not chains
int launch_relu_split_apply(float* l, float* u, const int8_t* split, int split_stride, int* infeasible, int B, int n,
                            cudaStream_t stream);
int launch_rows_add_broadcast(float* A, const float* v, int v_stride, int B, int S, int n, cudaStream_t stream);

}  // namespace bf
