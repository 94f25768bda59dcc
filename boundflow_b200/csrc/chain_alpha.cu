// alpha-CROWN / alpha-beta-CROWN driver for linear (relu linear)* chains: steps+1 lower-bound
// sweeps, analytic gradients by an adjoint sweep, Adam, projections and per-domain best-of
// tracking, all queued on one stream without host synchronisation.
#include <math.h>

#include <algorithm>

#include "chain_internal.cuh"

namespace bf {

int launch_crown_bwd_conv2d(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                            const float* W, const float* bias, float* A_prev, float* delta, int accumulate, int M, int S,
                            const bf_layer_desc& L, void* scratch, cudaStream_t stream, const float* add = nullptr);
size_t crown_bwd_conv2d_scratch_bytes(int M, const bf_layer_desc& L);
int launch_conv_forward_rows(const float* in, const float* W, const float* bias, float* out, int M, const bf_layer_desc& L,
                             cudaStream_t stream);

struct AlphaWs {
  std::vector<float*> au, bu, sl, grad, m, v, Ahat;
  std::vector<float*> gsum, mb, vb, addv;  // beta: gradient sums, Adam moments, split term -beta*s
  float* A0;
  float* H[2];
  float* cacc;
  float* partial;
  float* cur;
  float* row_weight;  // [M] d objective / d lower per spec row (min / softmin objectives)
  float* metric;
  int* improve;
  void* conv_scratch;  // ReLU-scaled coefficients of a conv layer's backward step
  size_t state_begin, state_bytes;  // grad/m/v (+ beta state) region, zero-initialised per call
  size_t bytes;
};

static size_t alpha_ws_layout(const bf_chain* c, int B, int S, bool with_beta, void* base, AlphaWs* ws) {
  const size_t M = (size_t)B * S;
  const int R = (int)c->relu_layers.size();
  Carver cv(base);
  AlphaWs w;
  int maxw = 1;
  const size_t z0 = cv.off;
  for (int r = 0; r < R; ++r) {
    const size_t n = (size_t)c->layers[c->relu_layers[r]].n_in;
    w.grad.push_back(cv.take<float>((size_t)B * n));
    w.m.push_back(cv.take<float>((size_t)B * n));
    w.v.push_back(cv.take<float>((size_t)B * n));
    if (with_beta) {
      w.gsum.push_back(cv.take<float>((size_t)B * n));
      w.mb.push_back(cv.take<float>((size_t)B * n));
      w.vb.push_back(cv.take<float>((size_t)B * n));
      w.addv.push_back(cv.take<float>((size_t)B * n));
    }
  }
  w.state_begin = z0;
  w.state_bytes = cv.off - z0;
  for (int r = 0; r < R; ++r) {
    const size_t n = (size_t)c->layers[c->relu_layers[r]].n_in;
    if ((int)n > maxw) maxw = (int)n;
    w.au.push_back(cv.take<float>((size_t)B * n));
    w.bu.push_back(cv.take<float>((size_t)B * n));
    w.sl.push_back(cv.take<float>((size_t)B * n));
    w.Ahat.push_back(cv.take<float>(M * n));
  }
  w.A0 = cv.take<float>(M * (size_t)c->n0);
  w.H[0] = cv.take<float>(M * (size_t)maxw);
  w.H[1] = cv.take<float>(M * (size_t)maxw);
  w.cacc = cv.take<float>(M);
  w.partial = cv.take<float>(M * (size_t)std::max(std::max(crown_bwd_partial_tiles(c->n0), crown_tc_partial_tiles(c->n0, 32)), crown_tc_persist_max_partial_tiles(c->n0)));
  w.cur = cv.take<float>(M);
  w.row_weight = cv.take<float>(M);
  w.metric = cv.take<float>((size_t)B);
  w.improve = cv.take<int>((size_t)B);
  size_t conv_scratch = 0;
  for (const bf_layer_desc& L : c->layers)
    if (L.op == BF_OP_CONV2D) conv_scratch = std::max(conv_scratch, crown_bwd_conv2d_scratch_bytes((int)M, L));
  w.conv_scratch = cv.take<char>(conv_scratch);
  w.bytes = cv.off;
  if (ws) *ws = w;
  return cv.off;
}

// The input set of a query: a box (mid, rad) or an Lp ball (mid = centre, eps, norm_p).
struct InputSetArg {
  const float* mid;
  const float* rad;
  int norm_p;
  float eps;
  bool box() const { return norm_p == BF_NORM_BOX; }
};

// One lower- or upper-side sweep with the relaxations in ws; `use_add` adds the split term of
// every ReLU to the lower coefficients (beta-CROWN).
// Backward step of affine layer `layer` (Linear: tensor-core / FFMA GEMM with optional fused box concretisation;
// Conv2d: ReLU scaling pass + transposed convolution, never fused with the concretisation).
static int alpha_bwd_layer(const bf_chain* c, const AlphaWs& ws, int layer, const float* A, const float* dpos, const float* dneg,
                           const float* epos, const float* eneg, const float* add, float* dst, int accumulate, const float* mid,
                           const float* rad, float* partial, int side, int M, int S, int* ptiles, cudaStream_t stream) {
  const bf_layer_desc& L = c->layers[layer];
  if (L.op == BF_OP_LINEAR)
    return dispatch_bwd(c, layer, A, dpos, dneg, epos, eneg, add, dst, ws.cacc, accumulate, mid, rad, partial, side, M, S, ptiles, stream);
  return launch_crown_bwd_conv2d(A, dpos, dneg, epos, eneg, L.W, L.bias, dst, ws.cacc, accumulate, M, S, L, ws.conv_scratch, stream, add);
}

static int alpha_sweep(const bf_chain* c, const AlphaWs& ws, const float* C, int side, bool keep_A0, bool use_add,
                       const InputSetArg& in, float* out, int B, int S, cudaStream_t stream) {
  const int M = B * S;
  const int R = (int)c->relu_layers.size();
  // a box is concretised inside the last Linear layer's epilogue; an Lp ball or a conv first layer needs the final
  // coefficient rows and a separate concretisation
  const bool fused = in.box() && c->layers[c->affine_layers[0]].op == BF_OP_LINEAR;
  const float* mid = fused ? in.mid : nullptr;
  const float* rad = fused ? in.rad : nullptr;
  if (!fused) keep_A0 = true;
  int rc;
  int ptiles = 1;
  if (R == 0) {
    rc = alpha_bwd_layer(c, ws, c->affine_layers[0], C, nullptr, nullptr, nullptr, nullptr, nullptr, keep_A0 ? ws.A0 : nullptr, 0, mid,
                         rad, fused ? ws.partial : nullptr, side, M, S, &ptiles, stream);
    if (rc != BF_OK) return rc;
  } else {
    rc = alpha_bwd_layer(c, ws, c->affine_layers[R], C, nullptr, nullptr, nullptr, nullptr, nullptr, ws.Ahat[R - 1], 0, nullptr,
                         nullptr, nullptr, side, M, S, nullptr, stream);
    if (rc != BF_OK) return rc;
    for (int r = R - 1; r >= 0; --r) {
      const float *dpos, *dneg, *epos = nullptr, *eneg = nullptr;
      if (side == BF_SIDE_LOWER) { dpos = ws.sl[r]; dneg = ws.au[r]; eneg = ws.bu[r]; }
      else { dpos = ws.au[r]; dneg = ws.sl[r]; epos = ws.bu[r]; }
      const float* add = (use_add && side == BF_SIDE_LOWER) ? ws.addv[r] : nullptr;
      const bool last = (r == 0);
      float* dst = last ? (keep_A0 ? ws.A0 : nullptr) : ws.Ahat[r - 1];
      rc = alpha_bwd_layer(c, ws, c->affine_layers[r], ws.Ahat[r], dpos, dneg, epos, eneg, add, dst, 1, last ? mid : nullptr,
                           last ? rad : nullptr, (last && fused) ? ws.partial : nullptr, side, M, S, last ? &ptiles : nullptr, stream);
      if (rc != BF_OK) return rc;
    }
  }
  if (fused) return launch_sum_partials(ws.cacc, ws.partial, ptiles, out, M, stream);
  if (in.box()) return launch_concretize(ws.A0, in.mid, in.rad, ws.cacc, out, side, B, S, c->n0, stream);
  return launch_concretize_lp(ws.A0, in.mid, ws.cacc, out, side, in.eps, in.norm_p, B, S, c->n0, stream);
}

// Adjoint sweep: accumulates d(sum_s lower[b,s])/d(alpha_r[b,j]) into ws.grad[r] and, with beta,
// sum_s gw[b,s] * g_r[b,s,j] (gw null: weight 1) into ws.gsum[r].
static int alpha_adjoint(const bf_chain* c, const AlphaWs& ws, const float* const* pre_l, const float* const* pre_u,
                         bool with_beta, const InputSetArg& in, int B, int S, cudaStream_t stream, const float* gw = nullptr) {
  const int M = B * S;
  const int R = (int)c->relu_layers.size();
  // the first Linear layer on a box forms h_0 = mid - sgn(A_0) * rad in its prologue; every other case writes the
  // start vector over the final coefficient rows first
  const bool h0_fused = in.box() && c->layers[c->affine_layers[0]].op == BF_OP_LINEAR;
  if (!h0_fused) {
    int rc = in.box() ? launch_h0_box(ws.A0, in.mid, in.rad, B, S, c->n0, stream)
                      : launch_h0_lp(ws.A0, in.mid, in.eps, in.norm_p, B, S, c->n0, stream);
    if (rc != BF_OK) return rc;
  }
  for (int r = 0; r < R; ++r) {
    const int layer = c->affine_layers[r];
    const bf_layer_desc& L = c->layers[layer];
    const float* hprev = (r == 0) ? ws.A0 : ws.H[(r - 1) & 1];
    int rc;
    if (L.op == BF_OP_LINEAR) {
      float* hout = (r < R - 1) ? ws.H[r & 1] : nullptr;
      const bool from_box = (r == 0) && h0_fused;
      rc = dispatch_adjoint(c, layer, hprev, from_box ? 1 : 0, from_box ? in.mid : nullptr, from_box ? in.rad : nullptr, ws.Ahat[r],
                            ws.sl[r], ws.au[r], nullptr, ws.bu[r], pre_l[r], pre_u[r], hout, ws.grad[r],
                            with_beta ? ws.gsum[r] : nullptr, M, S, stream, with_beta ? gw : nullptr);
    } else {
      float* g = ws.H[r & 1];
      rc = launch_conv_forward_rows(hprev, L.W, L.bias, g, M, L, stream);
      if (rc != BF_OK) return rc;
      rc = launch_relu_adjoint_rows(g, ws.Ahat[r], ws.sl[r], ws.au[r], ws.bu[r], pre_l[r], pre_u[r], ws.grad[r],
                                    with_beta ? ws.gsum[r] : nullptr, B, S, L.n_out, stream, with_beta ? gw : nullptr);
    }
    if (rc != BF_OK) return rc;
  }
  return BF_OK;
}

static AdamScalars adam_scalars(int t, float lr, int spec_reduce, int S) {
  const double beta1 = 0.9, beta2 = 0.999;
  AdamScalars sc{};
  const double bc1 = 1.0 - pow(beta1, t + 1), bc2 = 1.0 - pow(beta2, t + 1);
  sc.lr_step = (float)((double)lr / bc1);
  sc.bc2_sqrt = (float)sqrt(bc2);
  sc.beta1 = (float)beta1;
  sc.beta2 = (float)beta2;
  sc.eps = 1e-8f;
  sc.one_minus_beta1 = (float)(1.0 - beta1);
  sc.one_minus_beta2 = (float)(1.0 - beta2);
  // mean: loss = -sum_b mean_s lower; sum: -sum_b sum_s lower; min / softmin: the row weights carry d metric / d lower
  sc.grad_scale = (spec_reduce == BF_REDUCE_MEAN) ? (-1.0f / (float)S) : -1.0f;
  return sc;
}

}  // namespace bf

extern "C" size_t bf_chain_alpha_workspace_bytes(const bf_chain* chain, int B, int S) {
  if (!chain || B <= 0 || S <= 0) return 0;
  return bf::alpha_ws_layout(chain, B, S, false, nullptr, nullptr);
}

extern "C" size_t bf_chain_alpha_beta_workspace_bytes(const bf_chain* chain, int B, int S) {
  if (!chain || B <= 0 || S <= 0) return 0;
  return bf::alpha_ws_layout(chain, B, S, true, nullptr, nullptr);
}

static int alpha_common_checks(const char* who, const bf_chain* chain, const void* C, const void* pre_l, const void* pre_u,
                               const void* alpha, const void* mid, const void* rad, int norm_p, float eps, void* workspace,
                               size_t workspace_bytes, int B, int S, bool with_beta, bf::AlphaWs* ws) {
  BF_REQUIRE(chain && C && pre_l && pre_u && alpha && mid && workspace, BF_E_INVALID, "%s: null argument", who);
  BF_REQUIRE(norm_p == BF_NORM_BOX || norm_p == BF_NORM_INF || norm_p == BF_NORM_L2 || norm_p == BF_NORM_L1, BF_E_INVALID,
             "%s: bad norm", who);
  BF_REQUIRE(norm_p != BF_NORM_BOX || rad != nullptr, BF_E_INVALID, "%s: a box needs its radius tensor", who);
  BF_REQUIRE(norm_p == BF_NORM_BOX || eps >= 0.f, BF_E_INVALID, "%s: negative eps", who);
  BF_REQUIRE(B > 0 && S > 0 && (long long)B * S < 2147483647LL, BF_E_INVALID, "%s: bad B/S", who);
  BF_REQUIRE(chain->affine_relu_alternating, BF_E_UNSUPPORTED, "%s: only affine (relu affine)* chains are supported", who);
  const size_t need = bf::alpha_ws_layout(chain, B, S, with_beta, workspace, ws);
  BF_REQUIRE(workspace_bytes >= need, BF_E_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who, need, workspace_bytes);
  return BF_OK;
}

extern "C" int bf_chain_alpha_beta_crown(const bf_chain* chain, const float* C, const float* const* pre_l,
                                         const float* const* pre_u, float* const* alpha, float* const* best_alpha,
                                         float* const* beta, float* const* best_beta, const int8_t* const* splits,
                                         const int* split_strides, const float* mid, const float* rad, int norm_p, float eps,
                                         float* best_lower, float* best_upper, float* best_metric, int steps, float lr,
                                         int spec_reduce, void* workspace, size_t workspace_bytes, int B, int S,
                                         bf_stream_t stream_) {
  return bf_chain_alpha_beta_crown_reduce(chain, C, pre_l, pre_u, alpha, best_alpha, beta, best_beta, splits, split_strides, mid, rad,
                                          norm_p, eps, best_lower, best_upper, best_metric, steps, lr, spec_reduce, 1.0f, workspace,
                                          workspace_bytes, B, S, stream_);
}

// The per-domain loop behind every entry point.  objective 0: maximise reduce(lower) over the S rows as given;
// BF_OBJECTIVE_GAP / _BOTH: the S rows are S/2 spec rows followed by their negations (see bf_chain_alpha_crown_objective).
static int alpha_loop(const char* who, const bf_chain* chain, const float* C, const float* const* pre_l,
                      const float* const* pre_u, float* const* alpha, float* const* best_alpha, float* const* beta,
                      float* const* best_beta, const int8_t* const* splits, const int* split_strides, const float* mid,
                      const float* rad, int norm_p, float eps, float* best_lower, float* best_upper, float* best_metric, int steps,
                      float lr, int objective, float lb_weight, float ub_weight, int spec_reduce, float soft_tau, void* workspace,
                      size_t workspace_bytes, int B, int S, bf_stream_t stream_) {
  const bool with_beta = beta != nullptr;
  const bool paired = objective != 0;
  const bf::InputSetArg in{mid, rad, norm_p, eps};
  bf::AlphaWs ws;
  int rc = alpha_common_checks(who, chain, C, pre_l, pre_u, alpha, mid, rad, norm_p, eps, workspace, workspace_bytes, B, S, with_beta, &ws);
  if (rc != BF_OK) return rc;
  BF_REQUIRE(best_alpha && best_lower && steps >= 0, BF_E_INVALID, "%s: null output or negative steps", who);
  BF_REQUIRE(spec_reduce >= BF_REDUCE_MEAN && spec_reduce <= BF_REDUCE_SOFTMIN, BF_E_INVALID, "%s: bad spec_reduce", who);
  const bool weighted = paired || (spec_reduce == BF_REDUCE_MIN || spec_reduce == BF_REDUCE_SOFTMIN);
  BF_REQUIRE(!paired || (S % 2 == 0 && spec_reduce != BF_REDUCE_SUM && !best_upper), BF_E_INVALID,
             "%s: paired rows need an even row count, no separate upper output and a mean / min / softmin reduction", who);
  BF_REQUIRE(!paired || !with_beta, BF_E_UNSUPPORTED, "%s: the gap / both objectives carry no beta term", who);
  BF_REQUIRE(spec_reduce != BF_REDUCE_SOFTMIN || soft_tau > 0.f, BF_E_INVALID, "%s: soft_tau must be positive", who);
  BF_REQUIRE(!with_beta || (best_beta && splits), BF_E_INVALID, "%s: beta needs best_beta and the split assignment", who);
  cudaStream_t stream = bf::as_stream(stream_);
  const int R = (int)chain->relu_layers.size();
  float* metric = best_metric ? best_metric : ws.metric;
  bf::refresh_switches(chain);

  if (cudaMemsetAsync(static_cast<char*>(workspace) + ws.state_begin, 0, ws.state_bytes, stream) != cudaSuccess) {
    bf::set_error("%s: cudaMemsetAsync failed", who);
    return BF_E_CUDA;
  }
  for (int r = 0; r < R; ++r) {
    const int n = chain->layers[chain->relu_layers[r]].n_in;
    rc = bf::launch_relu_relax(pre_l[r], pre_u[r], alpha[r], n, ws.au[r], ws.bu[r], ws.sl[r], B, n, stream);
    if (rc != BF_OK) return rc;
    if (with_beta) {  // split term of the start beta (no update, no snapshot: improve flags are not set yet)
      bf::AdamScalars none{};
      rc = bf::launch_beta_step(beta[r], ws.mb[r], ws.vb[r], ws.gsum[r], splits[r], split_strides ? split_strides[r] : n, nullptr,
                                nullptr, ws.addv[r], none, 0, B, n, stream);
      if (rc != BF_OK) return rc;
    }
  }
  for (int t = 0; t <= steps; ++t) {
    const bool last = (t == steps);
    rc = bf::alpha_sweep(chain, ws, C, BF_SIDE_LOWER, !last, with_beta, in, ws.cur, B, S, stream);
    if (rc != BF_OK) return rc;
    float* row_weight = (weighted && !last) ? ws.row_weight : nullptr;
    rc = paired ? bf::launch_select_best_paired(ws.cur, best_lower, metric, ws.improve, t == 0, objective, spec_reduce, soft_tau,
                                                lb_weight, ub_weight, row_weight, B, S / 2, stream)
                : bf::launch_select_best(ws.cur, best_lower, metric, ws.improve, t == 0, spec_reduce, soft_tau, row_weight, B, S, stream);
    if (rc != BF_OK) return rc;
    bf::AdamScalars sc{};
    if (!last) {
      if (weighted) {  // the gradient of min_s / softmin_s lower: every spec row enters with its weight
        for (int r = 0; r < R; ++r) {
          rc = bf::launch_scale_rows(ws.Ahat[r], ws.row_weight, (long long)B * S, chain->layers[chain->relu_layers[r]].n_in, stream);
          if (rc != BF_OK) return rc;
        }
      }
      rc = bf::alpha_adjoint(chain, ws, pre_l, pre_u, with_beta, in, B, S, stream, weighted ? ws.row_weight : nullptr);
      if (rc != BF_OK) return rc;
      sc = bf::adam_scalars(t, lr, paired ? BF_REDUCE_SUM : spec_reduce, S);  // row weights already carry 1/S of a paired mean
    }
    for (int r = 0; r < R; ++r) {
      const int n = chain->layers[chain->relu_layers[r]].n_in;
      rc = bf::launch_adam_step(alpha[r], ws.m[r], ws.v[r], ws.grad[r], ws.improve, best_alpha[r], pre_l[r], pre_u[r], ws.sl[r],
                                sc, last ? 0 : 1, B, n, stream);
      if (rc != BF_OK) return rc;
      if (with_beta) {
        rc = bf::launch_beta_step(beta[r], ws.mb[r], ws.vb[r], ws.gsum[r], splits[r], split_strides ? split_strides[r] : n,
                                  ws.improve, best_beta[r], ws.addv[r], sc, last ? 0 : 1, B, n, stream);
        if (rc != BF_OK) return rc;
      }
    }
  }
  if (best_upper) {
    // the upper bound of each domain's best iteration = the upper sweep at its best alpha (beta acts on the lower side only)
    for (int r = 0; r < R; ++r) {
      const int n = chain->layers[chain->relu_layers[r]].n_in;
      rc = bf::launch_relu_relax(pre_l[r], pre_u[r], best_alpha[r], n, ws.au[r], ws.bu[r], ws.sl[r], B, n, stream);
      if (rc != BF_OK) return rc;
    }
    rc = bf::alpha_sweep(chain, ws, C, BF_SIDE_UPPER, false, false, in, best_upper, B, S, stream);
    if (rc != BF_OK) return rc;
  }
  if (bf::tc_may_run(chain, B * S)) {  // a tensor-core wait that expired invalidates every bound of this call
    rc = bf::launch_poison_on_status(chain->status, best_lower, (long long)B * S, best_upper, best_upper ? (long long)B * S : 0, stream);
    if (rc != BF_OK) return rc;
    rc = bf::launch_poison_on_status(chain->status, metric, B, nullptr, 0, stream);
    if (rc != BF_OK) return rc;
  }
  return BF_OK;
}

extern "C" int bf_chain_alpha_beta_crown_reduce(const bf_chain* chain, const float* C, const float* const* pre_l,
                                                const float* const* pre_u, float* const* alpha, float* const* best_alpha,
                                                float* const* beta, float* const* best_beta, const int8_t* const* splits,
                                                const int* split_strides, const float* mid, const float* rad, int norm_p,
                                                float eps, float* best_lower, float* best_upper, float* best_metric, int steps,
                                                float lr, int spec_reduce, float soft_tau, void* workspace,
                                                size_t workspace_bytes, int B, int S, bf_stream_t stream) {
  return alpha_loop(beta ? "bf_chain_alpha_beta_crown" : "bf_chain_alpha_crown", chain, C, pre_l, pre_u, alpha, best_alpha, beta,
                    best_beta, splits, split_strides, mid, rad, norm_p, eps, best_lower, best_upper, best_metric, steps, lr, 0, 1.f,
                    1.f, spec_reduce, soft_tau, workspace, workspace_bytes, B, S, stream);
}

extern "C" int bf_chain_alpha_crown_objective(const bf_chain* chain, const float* C_paired, const float* const* pre_l,
                                              const float* const* pre_u, float* const* alpha, float* const* best_alpha,
                                              const float* mid, const float* rad, int norm_p, float eps, float* best_rows,
                                              float* best_metric, int steps, float lr, int objective, int spec_reduce,
                                              float soft_tau, float lb_weight, float ub_weight, void* workspace,
                                              size_t workspace_bytes, int B, int S, bf_stream_t stream) {
  BF_REQUIRE(objective == BF_OBJECTIVE_GAP || objective == BF_OBJECTIVE_BOTH, BF_E_INVALID,
             "bf_chain_alpha_crown_objective: objective must be BF_OBJECTIVE_GAP or BF_OBJECTIVE_BOTH");
  BF_REQUIRE(S > 0, BF_E_INVALID, "bf_chain_alpha_crown_objective: S must be positive");
  return alpha_loop("bf_chain_alpha_crown_objective", chain, C_paired, pre_l, pre_u, alpha, best_alpha, nullptr, nullptr, nullptr,
                    nullptr, mid, rad, norm_p, eps, best_rows, nullptr, best_metric, steps, lr, objective, lb_weight, ub_weight,
                    spec_reduce, soft_tau, workspace, workspace_bytes, B, 2 * S, stream);
}

extern "C" int bf_chain_alpha_crown(const bf_chain* chain, const float* C, const float* const* pre_l,
                                    const float* const* pre_u, float* const* alpha, float* const* best_alpha,
                                    const float* mid, const float* rad, int norm_p, float eps, float* best_lower,
                                    float* best_upper, float* best_metric, int steps, float lr, int spec_reduce, void* workspace,
                                    size_t workspace_bytes, int B, int S, bf_stream_t stream) {
  return bf_chain_alpha_beta_crown(chain, C, pre_l, pre_u, alpha, best_alpha, nullptr, nullptr, nullptr, nullptr, mid, rad, norm_p,
                                   eps, best_lower, best_upper, best_metric, steps, lr, spec_reduce, workspace, workspace_bytes, B, S,
                                   stream);
}

extern "C" int bf_chain_alpha_grad(const bf_chain* chain, const float* C, const float* const* pre_l,
                                   const float* const* pre_u, const float* const* alpha, const float* mid,
                                   const float* rad, int norm_p, float eps, float* const* grad, float* lower, int spec_reduce,
                                   void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream_) {
  bf::AlphaWs ws;
  const bf::InputSetArg in{mid, rad, norm_p, eps};
  int rc = alpha_common_checks("bf_chain_alpha_grad", chain, C, pre_l, pre_u, alpha, mid, rad, norm_p, eps, workspace, workspace_bytes,
                               B, S, false, &ws);
  if (rc != BF_OK) return rc;
  BF_REQUIRE(grad && lower, BF_E_INVALID, "bf_chain_alpha_grad: null output");
  bf::refresh_switches(chain);
  cudaStream_t stream = bf::as_stream(stream_);
  const int R = (int)chain->relu_layers.size();
  if (cudaMemsetAsync(static_cast<char*>(workspace) + ws.state_begin, 0, ws.state_bytes, stream) != cudaSuccess) {
    bf::set_error("bf_chain_alpha_grad: cudaMemsetAsync failed");
    return BF_E_CUDA;
  }
  for (int r = 0; r < R; ++r) {
    const int n = chain->layers[chain->relu_layers[r]].n_in;
    rc = bf::launch_relu_relax(pre_l[r], pre_u[r], alpha[r], n, ws.au[r], ws.bu[r], ws.sl[r], B, n, stream);
    if (rc != BF_OK) return rc;
  }
  rc = bf::alpha_sweep(chain, ws, C, BF_SIDE_LOWER, true, false, in, lower, B, S, stream);
  if (rc != BF_OK) return rc;
  rc = bf::alpha_adjoint(chain, ws, pre_l, pre_u, false, in, B, S, stream);
  if (rc != BF_OK) return rc;
  const float scale = (spec_reduce == BF_REDUCE_MEAN) ? (-1.0f / (float)S) : -1.0f;
  for (int r = 0; r < R; ++r) {
    const int n = chain->layers[chain->relu_layers[r]].n_in;
    rc = bf::launch_scale_copy(ws.grad[r], scale, grad[r], (long long)B * n, stream);
    if (rc != BF_OK) return rc;
    if (bf::tc_may_run(chain, B * S)) {
      rc = bf::launch_poison_on_status(chain->status, grad[r], (long long)B * n, r == 0 ? lower : nullptr, (long long)B * S, stream);
      if (rc != BF_OK) return rc;
    }
  }
  return BF_OK;
}

// ---------------------------------------------------------------------------
// shared-parameter mode: one alpha (and one beta) per neuron for every domain and spec row
// ---------------------------------------------------------------------------
namespace bf {

struct SharedWs {
  std::vector<float*> m, v, mb, vb, part;
  // per-domain objective values and scratch of the reductions / objectives other than the plain mean
  float* dom_metric;
  float* dom_rows;
  int* dom_improve;
  size_t begin, bytes;  // extra region (after the per-domain layout), zero-initialised per call
};

static size_t shared_ws_layout(const bf_chain* c, int B, int S, bool with_beta, void* base, AlphaWs* ws, SharedWs* sw) {
  const size_t base_bytes = alpha_ws_layout(c, B, S, with_beta, base, ws);
  Carver cv(base);
  cv.off = base_bytes;
  SharedWs w;
  w.begin = base_bytes;
  const int chunks = shared_alpha_chunks(B);
  for (size_t r = 0; r < c->relu_layers.size(); ++r) {
    const size_t n = (size_t)c->layers[c->relu_layers[r]].n_in;
    w.m.push_back(cv.take<float>(n));
    w.v.push_back(cv.take<float>(n));
    if (with_beta) {
      w.mb.push_back(cv.take<float>(n));
      w.vb.push_back(cv.take<float>(n));
    }
    w.part.push_back(cv.take<float>((size_t)chunks * n));
  }
  w.dom_metric = cv.take<float>((size_t)B);
  w.dom_rows = cv.take<float>((size_t)B * S);
  w.dom_improve = cv.take<int>((size_t)B);
  w.bytes = cv.off - base_bytes;
  if (sw) *sw = w;
  return cv.off;
}

}  // namespace bf

extern "C" size_t bf_chain_alpha_shared_workspace_bytes(const bf_chain* chain, int B, int S, int with_beta) {
  if (!chain || B <= 0 || S <= 0) return 0;
  return bf::shared_ws_layout(chain, B, S, with_beta != 0, nullptr, nullptr, nullptr);
}

// objective 0: reduce(lower) over the S rows as given; BF_OBJECTIVE_GAP / _BOTH: the S rows are S/2 spec rows followed by
// their negations.  The whole-batch metric is the mean over the domains of the per-domain objective.
static int shared_loop(const char* who, const bf_chain* chain, const float* C, const float* const* pre_l,
                       const float* const* pre_u, float* const* alpha, float* const* best_alpha, float* const* beta,
                       float* const* best_beta, const int8_t* const* splits, const int* split_strides, const float* mid,
                       const float* rad, int norm_p, float eps, float* best_lower, float* best_upper, float* best_metric, int steps,
                       float lr, int objective, float lb_weight, float ub_weight, int spec_reduce, float soft_tau, void* workspace,
                       size_t workspace_bytes, int B, int S, bf_stream_t stream_) {
  BF_REQUIRE(chain && C && pre_l && pre_u && alpha && best_alpha && mid && best_lower && workspace, BF_E_INVALID,
             "%s: null argument", who);
  BF_REQUIRE(norm_p == BF_NORM_BOX || norm_p == BF_NORM_INF || norm_p == BF_NORM_L2 || norm_p == BF_NORM_L1, BF_E_INVALID,
             "%s: bad norm", who);
  BF_REQUIRE(norm_p != BF_NORM_BOX || rad != nullptr, BF_E_INVALID, "%s: a box needs its radius tensor", who);
  const bf::InputSetArg in{mid, rad, norm_p, eps};
  BF_REQUIRE(B > 0 && S > 0 && (long long)B * S < 2147483647LL && steps >= 0, BF_E_INVALID, "%s: bad B/S/steps", who);
  BF_REQUIRE(chain->affine_relu_alternating, BF_E_UNSUPPORTED, "%s: only affine (relu affine)* chains are supported", who);
  const bool with_beta = beta != nullptr;
  BF_REQUIRE(!with_beta || (best_beta && splits), BF_E_INVALID, "%s: beta needs best_beta and the split assignment", who);
  const bool paired = objective != 0;
  const bool weighted = paired || spec_reduce == BF_REDUCE_MIN || spec_reduce == BF_REDUCE_SOFTMIN;
  BF_REQUIRE(spec_reduce == BF_REDUCE_MEAN || spec_reduce == BF_REDUCE_MIN || spec_reduce == BF_REDUCE_SOFTMIN, BF_E_INVALID,
             "%s: spec_reduce must be mean, min or softmin", who);
  BF_REQUIRE(spec_reduce != BF_REDUCE_SOFTMIN || soft_tau > 0.f, BF_E_INVALID, "%s: soft_tau must be positive", who);
  BF_REQUIRE(!paired || (S % 2 == 0 && !best_upper), BF_E_INVALID, "%s: paired rows need an even row count and no separate upper output", who);
  BF_REQUIRE(!paired || !with_beta, BF_E_UNSUPPORTED, "%s: the gap / both objectives carry no beta term", who);
  bf::AlphaWs ws;
  bf::SharedWs sw;
  const size_t need = bf::shared_ws_layout(chain, B, S, with_beta, workspace, &ws, &sw);
  BF_REQUIRE(workspace_bytes >= need, BF_E_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who, need, workspace_bytes);
  cudaStream_t stream = bf::as_stream(stream_);
  const int R = (int)chain->relu_layers.size();
  const long long M = (long long)B * S;
  float* metric = best_metric ? best_metric : ws.metric;
  bf::refresh_switches(chain);
  char* wsb = static_cast<char*>(workspace);
  // also clears the split term of ReLUs without a split (ws.addv lies inside the state region)
  if (cudaMemsetAsync(wsb + ws.state_begin, 0, ws.state_bytes, stream) != cudaSuccess ||
      (sw.bytes && cudaMemsetAsync(wsb + sw.begin, 0, sw.bytes, stream) != cudaSuccess)) {
    bf::set_error("%s: cudaMemsetAsync failed", who);
    return BF_E_CUDA;
  }
  int rc;
  auto width = [&](int r) { return chain->layers[chain->relu_layers[r]].n_in; };
  auto stride = [&](int r) { return split_strides ? split_strides[r] : width(r); };
  auto relax_all = [&](float* const* a) -> int {
    for (int r = 0; r < R; ++r) {
      int e = bf::launch_relu_relax(pre_l[r], pre_u[r], a[r], /*alpha_stride=*/0, ws.au[r], ws.bu[r], ws.sl[r], B, width(r), stream);
      if (e != BF_OK) return e;
    }
    return BF_OK;
  };
  for (int t = 0; t <= steps; ++t) {
    const bool last = (t == steps);
    if ((rc = relax_all(alpha)) != BF_OK) return rc;
    if (with_beta)
      for (int r = 0; r < R; ++r)
        if (splits[r] && (rc = bf::launch_shared_beta_add(beta[r], splits[r], stride(r), ws.addv[r], B, width(r), stream)) != BF_OK)
          return rc;
    rc = bf::alpha_sweep(chain, ws, C, BF_SIDE_LOWER, !last, with_beta, in, ws.cur, B, S, stream);
    if (rc != BF_OK) return rc;
    if (!weighted) {
      if ((rc = bf::launch_shared_metric(ws.cur, M, metric, ws.improve, t == 0, stream)) != BF_OK) return rc;
    } else {
      // per-domain objective and d objective / d row (first = 1: no per-domain best-of here), then the batch mean
      float* row_weight = last ? nullptr : ws.row_weight;
      rc = paired ? bf::launch_select_best_paired(ws.cur, sw.dom_rows, sw.dom_metric, sw.dom_improve, 1, objective, spec_reduce, soft_tau,
                                                  lb_weight, ub_weight, row_weight, B, S / 2, stream)
                  : bf::launch_select_best(ws.cur, sw.dom_rows, sw.dom_metric, sw.dom_improve, 1, spec_reduce, soft_tau, row_weight, B, S, stream);
      if (rc != BF_OK) return rc;
      if ((rc = bf::launch_shared_metric(sw.dom_metric, B, metric, ws.improve, t == 0, stream)) != BF_OK) return rc;
    }
    if ((rc = bf::launch_copy_if(ws.cur, best_lower, M, ws.improve, stream)) != BF_OK) return rc;
    bf::AdamScalars sc{};
    if (!last) {
      if (weighted) {
        for (int r = 0; r < R; ++r)
          if ((rc = bf::launch_scale_rows(ws.Ahat[r], ws.row_weight, M, width(r), stream)) != BF_OK) return rc;
      }
      rc = bf::alpha_adjoint(chain, ws, pre_l, pre_u, with_beta, in, B, S, stream, weighted ? ws.row_weight : nullptr);
      if (rc != BF_OK) return rc;
      sc = bf::adam_scalars(t, lr, BF_REDUCE_SUM, S);
      // loss = -mean over every domain and spec row; with row weights (which sum to the objective's weight per domain): -mean over domains
      sc.grad_scale = weighted ? (-1.0f / (float)B) : (-1.0f / (float)M);
    }
    for (int r = 0; r < R; ++r) {
      rc = bf::launch_shared_adam(alpha[r], sw.m[r], sw.v[r], ws.grad[r], nullptr, 0, sw.part[r], ws.improve, best_alpha[r], sc,
                                  last ? 0 : 1, 0, B, width(r), stream);
      if (rc != BF_OK) return rc;
      if (with_beta) {
        // without a split on this ReLU the beta gradient is identically zero: snapshot only
        const bool upd = !last && splits[r] != nullptr;
        rc = bf::launch_shared_adam(beta[r], sw.mb[r], sw.vb[r], ws.gsum[r], splits[r], splits[r] ? stride(r) : 0, sw.part[r],
                                    ws.improve, best_beta[r], sc, upd ? 1 : 0, 1, B, width(r), stream);
        if (rc != BF_OK) return rc;
      }
    }
  }
  if (best_upper) {  // beta acts on the lower side only
    if ((rc = relax_all(best_alpha)) != BF_OK) return rc;
    rc = bf::alpha_sweep(chain, ws, C, BF_SIDE_UPPER, false, false, in, best_upper, B, S, stream);
    if (rc != BF_OK) return rc;
  }
  if (bf::tc_may_run(chain, B * S)) {  // a tensor-core wait that expired invalidates every bound of this call
    rc = bf::launch_poison_on_status(chain->status, best_lower, (long long)B * S, best_upper, best_upper ? (long long)B * S : 0, stream);
    if (rc != BF_OK) return rc;
    rc = bf::launch_poison_on_status(chain->status, metric, B, nullptr, 0, stream);
    if (rc != BF_OK) return rc;
  }
  return BF_OK;
}

extern "C" int bf_chain_alpha_crown_shared(const bf_chain* chain, const float* C, const float* const* pre_l,
                                           const float* const* pre_u, float* const* alpha, float* const* best_alpha,
                                           float* const* beta, float* const* best_beta, const int8_t* const* splits,
                                           const int* split_strides, const float* mid, const float* rad, int norm_p, float eps,
                                           float* best_lower, float* best_upper, float* best_metric, int steps, float lr,
                                           void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream) {
  return shared_loop("bf_chain_alpha_crown_shared", chain, C, pre_l, pre_u, alpha, best_alpha, beta, best_beta, splits, split_strides,
                     mid, rad, norm_p, eps, best_lower, best_upper, best_metric, steps, lr, 0, 1.f, 1.f, BF_REDUCE_MEAN, 1.f, workspace,
                     workspace_bytes, B, S, stream);
}

extern "C" int bf_chain_alpha_beta_crown_shared_reduce(const bf_chain* chain, const float* C, const float* const* pre_l,
                                                       const float* const* pre_u, float* const* alpha, float* const* best_alpha,
                                                       float* const* beta, float* const* best_beta, const int8_t* const* splits,
                                                       const int* split_strides, const float* mid, const float* rad, int norm_p,
                                                       float eps, float* best_lower, float* best_upper, float* best_metric, int steps,
                                                       float lr, int spec_reduce, float soft_tau, void* workspace,
                                                       size_t workspace_bytes, int B, int S, bf_stream_t stream) {
  return shared_loop("bf_chain_alpha_beta_crown_shared_reduce", chain, C, pre_l, pre_u, alpha, best_alpha, beta, best_beta, splits,
                     split_strides, mid, rad, norm_p, eps, best_lower, best_upper, best_metric, steps, lr, 0, 1.f, 1.f, spec_reduce,
                     soft_tau, workspace, workspace_bytes, B, S, stream);
}

extern "C" int bf_chain_alpha_crown_shared_objective(const bf_chain* chain, const float* C, const float* const* pre_l,
                                                     const float* const* pre_u, float* const* alpha, float* const* best_alpha,
                                                     const float* mid, const float* rad, int norm_p, float eps, float* best_rows,
                                                     float* best_upper, float* best_metric, int steps, float lr, int objective,
                                                     int spec_reduce, float soft_tau, float lb_weight, float ub_weight,
                                                     void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream) {
  const char* who = "bf_chain_alpha_crown_shared_objective";
  BF_REQUIRE(objective == 0 || objective == BF_OBJECTIVE_GAP || objective == BF_OBJECTIVE_BOTH, BF_E_INVALID,
             "%s: objective must be 0 (lower), BF_OBJECTIVE_GAP or BF_OBJECTIVE_BOTH", who);
  BF_REQUIRE(S > 0, BF_E_INVALID, "%s: S must be positive", who);
  return shared_loop(who, chain, C, pre_l, pre_u, alpha, best_alpha, nullptr, nullptr, nullptr, nullptr, mid, rad, norm_p, eps, best_rows,
                     objective == 0 ? best_upper : nullptr, best_metric, steps, lr, objective, lb_weight, ub_weight, spec_reduce,
                     soft_tau, workspace, workspace_bytes, B, objective == 0 ? S : 2 * S, stream);
}

// ---------------------------------------------------------------------------
// The pieces of the per-domain alpha / beta loop as separate entry points, for graphs that are not chains: the
// caller walks its graph and calls these per value (ReLU split, adjoint start vector, forward convolution of rows,
// ReLU adjoint step, objective / best-of, Adam steps).
// ---------------------------------------------------------------------------
extern "C" int bf_relu_split_apply(float* l, float* u, const int8_t* split, int split_stride, int* infeasible, int B, int n,
                                   bf_stream_t stream) {
  BF_REQUIRE(l && u && split, BF_E_INVALID, "bf_relu_split_apply: null tensor");
  BF_REQUIRE(B > 0 && n > 0 && (split_stride == 0 || split_stride == n), BF_E_INVALID, "bf_relu_split_apply: bad sizes");
  return bf::launch_relu_split_apply(l, u, split, split_stride, infeasible, B, n, bf::as_stream(stream));
}

extern "C" int bf_interval_intersect(float* l, float* u, const float* cons_l, const float* cons_u, int* infeasible, int B, int n,
                                     bf_stream_t stream) {
  BF_REQUIRE(l && u && cons_l && cons_u, BF_E_INVALID, "bf_interval_intersect: null tensor");
  BF_REQUIRE(B > 0 && n > 0, BF_E_INVALID, "bf_interval_intersect: bad sizes");
  return bf::launch_interval_intersect(l, u, cons_l, cons_u, infeasible, B, n, bf::as_stream(stream));
}

extern "C" int bf_rows_add_broadcast(float* A, const float* v, int v_stride, int B, int S, int n, bf_stream_t stream) {
  BF_REQUIRE(A && v, BF_E_INVALID, "bf_rows_add_broadcast: null tensor");
  BF_REQUIRE(B > 0 && S > 0 && n > 0 && (v_stride == 0 || v_stride == n), BF_E_INVALID, "bf_rows_add_broadcast: bad sizes");
  return bf::launch_rows_add_broadcast(A, v, v_stride, B, S, n, bf::as_stream(stream));
}

extern "C" int bf_adjoint_start_box(float* A0, const float* mid, const float* rad, int B, int S, int n0, bf_stream_t stream) {
  BF_REQUIRE(A0 && mid && rad, BF_E_INVALID, "bf_adjoint_start_box: null tensor");
  BF_REQUIRE(B > 0 && S > 0 && n0 > 0, BF_E_INVALID, "bf_adjoint_start_box: bad sizes");
  return bf::launch_h0_box(A0, mid, rad, B, S, n0, bf::as_stream(stream));
}

extern "C" int bf_adjoint_start_lp(float* A0, const float* center, float eps, int p, int B, int S, int n0, bf_stream_t stream) {
  BF_REQUIRE(A0 && center, BF_E_INVALID, "bf_adjoint_start_lp: null tensor");
  BF_REQUIRE(B > 0 && S > 0 && n0 > 0 && eps >= 0.f && (p == BF_NORM_L1 || p == BF_NORM_L2 || p == BF_NORM_INF), BF_E_INVALID,
             "bf_adjoint_start_lp: bad sizes, eps or norm");
  return bf::launch_h0_lp(A0, center, eps, p, B, S, n0, bf::as_stream(stream));
}

extern "C" int bf_rows_conv2d_fwd(const float* in, const float* W, const float* bias, float* out, int M, int Ci, int Hi, int Wi,
                                  int Co, int Ho, int Wo, int kh, int kw, int sh, int sw, int ph, int pw, bf_stream_t stream) {
  BF_REQUIRE(in && W && out, BF_E_INVALID, "bf_rows_conv2d_fwd: null tensor");
  BF_REQUIRE(M > 0 && Ci > 0 && Hi > 0 && Wi > 0 && Co > 0 && Ho > 0 && Wo > 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0 && ph >= 0 && pw >= 0,
             BF_E_INVALID, "bf_rows_conv2d_fwd: bad sizes");
  bf_layer_desc L{};
  L.op = BF_OP_CONV2D; L.W = W; L.bias = bias;
  L.Ci = Ci; L.Hi = Hi; L.Wi = Wi; L.Co = Co; L.Ho = Ho; L.Wo = Wo; L.kh = kh; L.kw = kw; L.sh = sh; L.sw = sw; L.ph = ph; L.pw = pw;
  L.n_in = Ci * Hi * Wi; L.n_out = Co * Ho * Wo;
  return bf::launch_conv_forward_rows(in, W, bias, out, M, L, bf::as_stream(stream));
}

extern "C" int bf_relu_adjoint_rows(float* G, const float* Ahat, const float* alpha_u, const float* alpha_l, const float* beta_u,
                                    const float* pre_l, const float* pre_u, float* grad, float* gsum, const float* row_weight, int B,
                                    int S, int n,
                                    bf_stream_t stream) {
  BF_REQUIRE(G && Ahat && alpha_u && alpha_l && pre_l && pre_u && grad, BF_E_INVALID, "bf_relu_adjoint_rows: null tensor");
  BF_REQUIRE(B > 0 && S > 0 && n > 0, BF_E_INVALID, "bf_relu_adjoint_rows: bad sizes");
  return bf::launch_relu_adjoint_rows(G, Ahat, alpha_l, alpha_u, beta_u, pre_l, pre_u, grad, gsum, B, S, n, bf::as_stream(stream),
                                      gsum ? row_weight : nullptr);
}

extern "C" int bf_alpha_select_best(const float* cur, float* best_lower, float* best_metric, int* improve, int first, int spec_reduce,
                                    float soft_tau, float* row_weight, int B, int S, bf_stream_t stream) {
  BF_REQUIRE(cur && best_lower && best_metric && improve, BF_E_INVALID, "bf_alpha_select_best: null tensor");
  BF_REQUIRE(B > 0 && S > 0 && spec_reduce >= BF_REDUCE_MEAN && spec_reduce <= BF_REDUCE_SOFTMIN, BF_E_INVALID,
             "bf_alpha_select_best: bad sizes or reduction");
  BF_REQUIRE(spec_reduce != BF_REDUCE_SOFTMIN || soft_tau > 0.f, BF_E_INVALID, "bf_alpha_select_best: soft_tau must be positive");
  return bf::launch_select_best(cur, best_lower, best_metric, improve, first, spec_reduce, soft_tau, row_weight, B, S, bf::as_stream(stream));
}

extern "C" int bf_alpha_adam_step(float* alpha, float* m, float* v, float* grad, const int* improve, float* best_alpha,
                                  const float* pre_l, const float* pre_u, float* slope_l, int t, float lr, int spec_reduce, int S,
                                  int do_update, int B, int n, bf_stream_t stream) {
  BF_REQUIRE(alpha && m && v && grad && improve && best_alpha && pre_l && pre_u && slope_l, BF_E_INVALID,
             "bf_alpha_adam_step: null tensor");
  BF_REQUIRE(B > 0 && n > 0 && S > 0 && t >= 0 && lr > 0.f, BF_E_INVALID, "bf_alpha_adam_step: bad sizes or options");
  return bf::launch_adam_step(alpha, m, v, grad, improve, best_alpha, pre_l, pre_u, slope_l, bf::adam_scalars(t, lr, spec_reduce, S),
                              do_update, B, n, bf::as_stream(stream));
}

extern "C" int bf_beta_adam_step(float* beta, float* m, float* v, float* gsum, const int8_t* split, int split_stride,
                                 const int* improve, float* best_beta, float* add, int t, float lr, int spec_reduce, int S,
                                 int do_update, int B, int n, bf_stream_t stream) {
  BF_REQUIRE(beta && m && v && gsum && split && add, BF_E_INVALID, "bf_beta_adam_step: null tensor");
  BF_REQUIRE(B > 0 && n > 0 && S > 0 && t >= 0 && lr > 0.f && (split_stride == 0 || split_stride == n), BF_E_INVALID,
             "bf_beta_adam_step: bad sizes or options");
  return bf::launch_beta_step(beta, m, v, gsum, split, split_stride, improve, best_beta, add, bf::adam_scalars(t, lr, spec_reduce, S),
                              do_update, B, n, bf::as_stream(stream));
}

extern "C" int bf_alpha_select_best_paired(const float* cur, float* best_rows, float* best_metric, int* improve, int first,
                                           int objective, int spec_reduce, float soft_tau, float lb_weight, float ub_weight,
                                           float* row_weight, int B, int S, bf_stream_t stream) {
  BF_REQUIRE(cur && best_rows && best_metric && improve, BF_E_INVALID, "bf_alpha_select_best_paired: null tensor");
  BF_REQUIRE(objective == BF_OBJECTIVE_GAP || objective == BF_OBJECTIVE_BOTH, BF_E_INVALID,
             "bf_alpha_select_best_paired: objective must be BF_OBJECTIVE_GAP or BF_OBJECTIVE_BOTH");
  BF_REQUIRE(B > 0 && S > 0 && (spec_reduce == BF_REDUCE_MEAN || spec_reduce == BF_REDUCE_MIN || spec_reduce == BF_REDUCE_SOFTMIN),
             BF_E_INVALID, "bf_alpha_select_best_paired: bad sizes or reduction");
  BF_REQUIRE(spec_reduce != BF_REDUCE_SOFTMIN || soft_tau > 0.f, BF_E_INVALID, "bf_alpha_select_best_paired: soft_tau must be positive");
  BF_REQUIRE(lb_weight >= 0.f && ub_weight >= 0.f, BF_E_UNSUPPORTED, "bf_alpha_select_best_paired: negative objective weight");
  return bf::launch_select_best_paired(cur, best_rows, best_metric, improve, first, objective, spec_reduce, soft_tau, lb_weight, ub_weight,
                                       row_weight, B, S, bf::as_stream(stream));
}

extern "C" int bf_rows_scale(float* A, const float* w, long long M, int n, bf_stream_t stream) {
  BF_REQUIRE(A && w, BF_E_INVALID, "bf_rows_scale: null tensor");
  BF_REQUIRE(M > 0 && n > 0, BF_E_INVALID, "bf_rows_scale: bad sizes");
  return bf::launch_scale_rows(A, w, M, n, bf::as_stream(stream));
}

extern "C" int bf_rows_colmax_abs(const float* A, float* out, int B, int S, int n, bf_stream_t stream) {
  BF_REQUIRE(A && out, BF_E_INVALID, "bf_rows_colmax_abs: null tensor");
  BF_REQUIRE(B > 0 && S > 0 && n > 0, BF_E_INVALID, "bf_rows_colmax_abs: bad sizes");
  return bf::launch_colmax_abs(A, out, B, S, n, bf::as_stream(stream));
}

extern "C" int bf_shared_metric(const float* values, long long M, float* best_metric, int* improve, int first, bf_stream_t stream) {
  BF_REQUIRE(values && best_metric && improve, BF_E_INVALID, "bf_shared_metric: null tensor");
  BF_REQUIRE(M > 0, BF_E_INVALID, "bf_shared_metric: bad size");
  return bf::launch_shared_metric(values, M, best_metric, improve, first, bf::as_stream(stream));
}

extern "C" int bf_copy_if(const float* src, float* dst, long long n, const int* flag, bf_stream_t stream) {
  BF_REQUIRE(src && dst && flag, BF_E_INVALID, "bf_copy_if: null tensor");
  BF_REQUIRE(n > 0, BF_E_INVALID, "bf_copy_if: bad size");
  return bf::launch_copy_if(src, dst, n, flag, bf::as_stream(stream));
}

extern "C" size_t bf_shared_adam_scratch_floats(int B, int n) {
  if (B <= 0 || n <= 0) return 0;
  return (size_t)bf::shared_alpha_chunks(B) * (size_t)n;
}

extern "C" int bf_shared_adam_step(float* param, float* m, float* v, float* grad, const int8_t* split, int split_stride, float* scratch,
                                   const int* improve, float* best, int t, float lr, float grad_scale, int do_update, int is_beta,
                                   int B, int n, bf_stream_t stream) {
  BF_REQUIRE(param && m && v && grad && scratch && improve && best, BF_E_INVALID, "bf_shared_adam_step: null tensor");
  BF_REQUIRE(B > 0 && n > 0 && t >= 0 && lr > 0.f && (split == nullptr || split_stride == 0 || split_stride == n), BF_E_INVALID,
             "bf_shared_adam_step: bad sizes or options");
  bf::AdamScalars sc = bf::adam_scalars(t, lr, BF_REDUCE_SUM, 1);
  sc.grad_scale = grad_scale;
  return bf::launch_shared_adam(param, m, v, grad, split, split_stride, scratch, improve, best, sc, do_update, is_beta, B, n,
                                bf::as_stream(stream));
}

extern "C" int bf_shared_beta_add(const float* beta, const int8_t* split, int split_stride, float* add, int B, int n, bf_stream_t stream) {
  BF_REQUIRE(beta && split && add, BF_E_INVALID, "bf_shared_beta_add: null tensor");
  BF_REQUIRE(B > 0 && n > 0 && (split_stride == 0 || split_stride == n), BF_E_INVALID, "bf_shared_beta_add: bad sizes");
  return bf::launch_shared_beta_add(beta, split, split_stride, add, B, n, bf::as_stream(stream));
}
