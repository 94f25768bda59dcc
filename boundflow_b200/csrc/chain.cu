// Whole-chain drivers: host loops that string the layer kernels together on one
// stream without any host synchronisation (IBP trace, CROWN sweep, the
// alpha-CROWN optimisation loop and its analytic gradient).
#include <math.h>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "kernels.cuh"

namespace bf {

static thread_local char g_err[512] = "ok";
std::atomic<unsigned long long> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

// ---- optional kernel timing ----------------------------------------------------
struct TimingSlot {
  std::vector<cudaEvent_t> start, stop;
  size_t used = 0;
};
static TimingSlot g_timing[2];
static bool g_timing_on = false;

void timing_begin(int slot, cudaStream_t stream) {
  if (!g_timing_on) return;
  TimingSlot& t = g_timing[slot];
  if (t.used == t.start.size()) {
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
    t.start.push_back(a);
    t.stop.push_back(b);
  }
  cudaEventRecord(t.start[t.used], stream);
}

void timing_end(int slot, cudaStream_t stream) {
  if (!g_timing_on) return;
  TimingSlot& t = g_timing[slot];
  if (t.used < t.stop.size()) {
    cudaEventRecord(t.stop[t.used], stream);
    ++t.used;
  }
}

}  // namespace bf

extern "C" void bf_kernel_timing_enable(int on) {
  bf::g_timing_on = on != 0;
  for (auto& t : bf::g_timing) t.used = 0;
}

extern "C" int bf_kernel_timing_read(int slot, int* launches, float* total_ms) {
  BF_REQUIRE(slot >= 0 && slot < 2 && launches && total_ms, BF_E_INVALID, "bf_kernel_timing_read: bad argument");
  bf::TimingSlot& t = bf::g_timing[slot];
  float sum = 0.f;
  for (size_t i = 0; i < t.used; ++i) {
    if (cudaEventSynchronize(t.stop[i]) != cudaSuccess) {
      bf::set_error("bf_kernel_timing_read: cudaEventSynchronize failed");
      return BF_E_CUDA;
    }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, t.start[i], t.stop[i]);
    sum += ms;
  }
  *launches = (int)t.used;
  *total_ms = sum;
  return BF_OK;
}

struct bf_chain {
  std::vector<bf_layer_desc> layers;
  std::vector<int> relu_layers;  // layer index of every ReLU, chain order
  int n0 = 0;
  int max_width = 0;
  bool linear_relu_alternating = false;  // linear (relu linear)*
  // tensor-core path: per layer, packed hi/lo weight images for the backward (W^T as B) and
  // adjoint (W as B) orientation inside a caller-owned buffer, plus a device status word
  std::vector<const unsigned char*> pk_bwd, pk_adj;
  int* status = nullptr;
};

extern "C" int bf_version(void) { return 100; }
extern "C" const char* bf_last_error_string(void) { return bf::g_err; }
extern "C" unsigned long long bf_launch_count(void) { return bf::g_launches.load(); }

extern "C" int bf_chain_create(const bf_layer_desc* layers, int n_layers, bf_chain** out) {
  BF_REQUIRE(layers && out && n_layers > 0, BF_E_INVALID, "bf_chain_create: null/empty layer list");
  bf_chain* c = new bf_chain();
  int width = layers[0].n_in;
  c->n0 = width;
  c->max_width = width;
  bool alternating = true;
  for (int i = 0; i < n_layers; ++i) {
    const bf_layer_desc& L = layers[i];
    bool ok = (L.n_in == width) && L.n_in > 0 && L.n_out > 0;
    switch (L.op) {
      case BF_OP_LINEAR:
        ok = ok && L.W != nullptr;
        if (i % 2 != 0) alternating = false;
        break;
      case BF_OP_CONV2D:
        ok = ok && L.W != nullptr && L.n_in == L.Ci * L.Hi * L.Wi && L.n_out == L.Co * L.Ho * L.Wo && L.sh > 0 && L.sw > 0 &&
             L.Ho == (L.Hi + 2 * L.ph - L.kh) / L.sh + 1 && L.Wo == (L.Wi + 2 * L.pw - L.kw) / L.sw + 1;
        alternating = false;
        break;
      case BF_OP_RELU:
        ok = ok && L.n_in == L.n_out;
        c->relu_layers.push_back(i);
        if (i % 2 != 1) alternating = false;
        break;
      case BF_OP_FLATTEN:
        ok = ok && L.n_in == L.n_out;
        alternating = false;
        break;
      default:
        ok = false;
    }
    if (!ok) {
      bf::set_error("bf_chain_create: layer %d (op %d, n_in %d, n_out %d) is inconsistent with the chain (width %d)", i, L.op,
                    L.n_in, L.n_out, width);
      delete c;
      return BF_E_INVALID;
    }
    width = L.n_out;
    if (width > c->max_width) c->max_width = width;
    c->layers.push_back(L);
  }
  c->linear_relu_alternating = alternating && (n_layers % 2 == 1);
  *out = c;
  return BF_OK;
}

extern "C" void bf_chain_destroy(bf_chain* chain) { delete chain; }
extern "C" int bf_chain_num_relu(const bf_chain* chain) { return chain ? (int)chain->relu_layers.size() : BF_E_INVALID; }

namespace bf {

static inline size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  template <typename T>
  T* take(size_t n) {
    T* p = reinterpret_cast<T*>(base + off);
    off += align_up(n * sizeof(T));
    return p;
  }
};

static int relu_index_of(const bf_chain* c, int layer) {
  for (size_t r = 0; r < c->relu_layers.size(); ++r)
    if (c->relu_layers[r] == layer) return (int)r;
  return -1;
}

static int lowest_affine(const bf_chain* c) {
  for (size_t i = 0; i < c->layers.size(); ++i)
    if (c->layers[i].op == BF_OP_LINEAR || c->layers[i].op == BF_OP_CONV2D) return (int)i;
  return -1;
}

}  // namespace bf

// conv kernels (conv.cu)
namespace bf {
int launch_ibp_conv2d(const float* in_a, const float* in_b, int in_mode, int relu_in, const float* W, const float* bias,
                      const int8_t* split, int split_stride, const float* cons_l, const float* cons_u, float* out_l,
                      float* out_u, int* infeasible, int B, const bf_layer_desc& L, cudaStream_t stream);
int launch_crown_bwd_conv2d(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                            const float* W, const float* bias, float* A_prev, float* delta, int accumulate, int M, int S,
                            const bf_layer_desc& L, void* scratch, cudaStream_t stream);
size_t crown_bwd_conv2d_scratch_bytes(int M, const bf_layer_desc& L);
}  // namespace bf

// ---------------------------------------------------------------------------
// tensor-core path set-up and dispatch
// ---------------------------------------------------------------------------
namespace bf {

static bool tc_allowed() {
  const char* e = getenv("BF_B200_FORCE_FFMA");
  return !(e && e[0] == '1');
}

static const unsigned char* tc_weights(const bf_chain* c, int layer, bool adjoint, int M, int K, int N) {
  if (c->pk_bwd.empty() || !tc_allowed()) return nullptr;
  if (M < 256 || K < 32 || N < 32) return nullptr;  // tiny problems stay on the FFMA tiles
  return adjoint ? c->pk_adj[layer] : c->pk_bwd[layer];
}

// Backward contraction of linear layer `layer`; *ptiles receives the number of column tiles
// (the second dimension of the concretisation partial-sum buffer).
static int dispatch_bwd(const bf_chain* c, int layer, const float* A, const float* dpos, const float* dneg,
                        const float* epos, const float* eneg, const float* add, float* A_prev, float* delta, int accumulate,
                        const float* mid, const float* rad, float* partial, int side, int M, int S, int* ptiles,
                        cudaStream_t stream) {
  const bf_layer_desc& L = c->layers[layer];
  const int K = L.n_out, N = L.n_in;
  const unsigned char* pk = tc_weights(c, layer, false, M, K, N);
  if (pk) {
    if (ptiles) *ptiles = crown_tc_partial_tiles(N, K);
    return launch_crown_bwd_linear_tc(A, dpos, dneg, epos, eneg, add, pk, L.bias, A_prev, delta, accumulate, mid, rad, partial,
                                      side, M, S, K, N, c->status, stream);
  }
  if (ptiles) *ptiles = crown_bwd_partial_tiles(N);
  return launch_crown_bwd_linear(A, dpos, dneg, epos, eneg, add, L.W, L.bias, A_prev, delta, accumulate, mid, rad, partial, side,
                                 M, S, K, N, stream);
}

static int dispatch_adjoint(const bf_chain* c, int layer, const float* Hprev, int first_layer, const float* mid,
                            const float* rad, const float* Ahat, const float* dpos, const float* dneg, const float* epos,
                            const float* eneg, const float* pre_l, const float* pre_u, float* hout, float* grad, int M, int S,
                            cudaStream_t stream) {
  const bf_layer_desc& L = c->layers[layer];
  const int K = L.n_in, N = L.n_out;
  const unsigned char* pk = tc_weights(c, layer, true, M, K, N);
  if (pk)
    return launch_crown_adjoint_linear_tc(Hprev, first_layer, mid, rad, pk, L.bias, Ahat, dpos, dneg, epos, eneg, pre_l, pre_u,
                                          hout, grad, M, S, K, N, c->status, stream);
  return launch_crown_adjoint_linear(Hprev, first_layer, mid, rad, L.W, L.bias, Ahat, dpos, dneg, epos, eneg, pre_l, pre_u, hout,
                                     grad, M, S, K, N, stream);
}

}  // namespace bf

extern "C" size_t bf_chain_tc_bytes(const bf_chain* chain) {
  if (!chain) return 0;
  size_t total = 256;  // status word
  for (const bf_layer_desc& L : chain->layers)
    if (L.op == BF_OP_LINEAR)
      total += bf::align_up(bf::tc_packed_bytes(L.n_in, L.n_out)) + bf::align_up(bf::tc_packed_bytes(L.n_out, L.n_in));
  return total;
}

extern "C" int bf_chain_tc_prepare(bf_chain* chain, void* buffer, size_t bytes, bf_stream_t stream_) {
  BF_REQUIRE(chain && buffer, BF_E_INVALID, "bf_chain_tc_prepare: null argument");
  BF_REQUIRE((reinterpret_cast<uintptr_t>(buffer) & 255u) == 0, BF_E_INVALID, "bf_chain_tc_prepare: buffer must be 256-byte aligned");
  BF_REQUIRE(bytes >= bf_chain_tc_bytes(chain), BF_E_WORKSPACE, "bf_chain_tc_prepare: %zu bytes needed", bf_chain_tc_bytes(chain));
  cudaStream_t stream = bf::as_stream(stream_);
  unsigned char* base = static_cast<unsigned char*>(buffer);
  if (cudaMemsetAsync(base, 0, 256, stream) != cudaSuccess) {
    bf::set_error("bf_chain_tc_prepare: cudaMemsetAsync failed");
    return BF_E_CUDA;
  }
  chain->status = reinterpret_cast<int*>(base);
  size_t off = 256;
  chain->pk_bwd.assign(chain->layers.size(), nullptr);
  chain->pk_adj.assign(chain->layers.size(), nullptr);
  for (size_t i = 0; i < chain->layers.size(); ++i) {
    const bf_layer_desc& L = chain->layers[i];
    if (L.op != BF_OP_LINEAR) continue;
    // backward: C = Lambda[M, n_out] * W[n_out, n_in]  ->  B[n][k] = W[k][n]  (transposed read)
    unsigned char* pb = base + off;
    off += bf::align_up(bf::tc_packed_bytes(L.n_in, L.n_out));
    int rc = bf::tc_pack_weights(L.W, L.n_out, L.n_in, 1, pb, stream);
    if (rc != BF_OK) return rc;
    // adjoint: g = h[M, n_in] * W[n_out, n_in]^T  ->  B[n][k] = W[n][k]
    unsigned char* pa = base + off;
    off += bf::align_up(bf::tc_packed_bytes(L.n_out, L.n_in));
    rc = bf::tc_pack_weights(L.W, L.n_out, L.n_in, 0, pa, stream);
    if (rc != BF_OK) return rc;
    chain->pk_bwd[i] = pb;
    chain->pk_adj[i] = pa;
  }
  return BF_OK;
}

extern "C" int bf_chain_tc_status(const bf_chain* chain, int* status_out) {
  BF_REQUIRE(chain && status_out, BF_E_INVALID, "bf_chain_tc_status: null argument");
  *status_out = 0;
  if (!chain->status) return BF_OK;
  if (cudaMemcpy(status_out, chain->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
    bf::set_error("bf_chain_tc_status: cudaMemcpy failed");
    return BF_E_CUDA;
  }
  return BF_OK;
}

// ---------------------------------------------------------------------------
// IBP trace
// ---------------------------------------------------------------------------
extern "C" int bf_chain_ibp(const bf_chain* chain, const float* in_a, const float* in_b, int in_mode,
                            const int8_t* const* splits, const int* split_strides, const float* const* cons_l,
                            const float* const* cons_u, float* const* pre_l, float* const* pre_u, float* out_l,
                            float* out_u, int* infeasible, float* scratch, size_t scratch_bytes, int B,
                            bf_stream_t stream_) {
  BF_REQUIRE(chain && in_a && in_b && out_l && out_u, BF_E_INVALID, "bf_chain_ibp: null argument");
  BF_REQUIRE(B > 0, BF_E_INVALID, "bf_chain_ibp: B must be positive");
  cudaStream_t stream = bf::as_stream(stream_);
  const int nl = (int)chain->layers.size();
  const size_t need = 4 * bf::align_up((size_t)B * chain->max_width * sizeof(float));
  const float* cur_a = in_a;
  const float* cur_b = in_b;
  int mode = in_mode;
  int relu_pending = 0;
  int toggle = 0;
  int last_affine = -1;
  for (int i = 0; i < nl; ++i)
    if (chain->layers[i].op == BF_OP_LINEAR || chain->layers[i].op == BF_OP_CONV2D) last_affine = i;
  BF_REQUIRE(last_affine >= 0, BF_E_UNSUPPORTED, "bf_chain_ibp: chain has no affine layer");
  for (int i = last_affine + 1; i < nl; ++i)
    BF_REQUIRE(chain->layers[i].op == BF_OP_FLATTEN, BF_E_UNSUPPORTED, "bf_chain_ibp: the chain must end with an affine layer");

  for (int i = 0; i < nl; ++i) {
    const bf_layer_desc& L = chain->layers[i];
    if (L.op == BF_OP_FLATTEN) continue;
    if (L.op == BF_OP_RELU) {
      BF_REQUIRE(!relu_pending && i > 0, BF_E_UNSUPPORTED, "bf_chain_ibp: ReLU must follow an affine layer");
      relu_pending = 1;
      continue;
    }
    // affine layer: where does its output go?
    int j = i + 1;
    while (j < nl && chain->layers[j].op == BF_OP_FLATTEN) ++j;
    float *dst_l, *dst_u;
    const int8_t* sp = nullptr;
    int sp_stride = 0;
    const float *cl = nullptr, *cu = nullptr;
    if (i == last_affine) {
      dst_l = out_l;
      dst_u = out_u;
    } else if (j < nl && chain->layers[j].op == BF_OP_RELU) {
      const int r = bf::relu_index_of(chain, j);
      BF_REQUIRE(pre_l && pre_u && pre_l[r] && pre_u[r], BF_E_INVALID, "bf_chain_ibp: missing pre-activation output %d", r);
      dst_l = pre_l[r];
      dst_u = pre_u[r];
      if (splits && splits[r]) {
        sp = splits[r];
        sp_stride = split_strides ? split_strides[r] : L.n_out;
      }
      if (cons_l && cons_u && cons_l[r] && cons_u[r]) {
        cl = cons_l[r];
        cu = cons_u[r];
      }
    } else {
      BF_REQUIRE(scratch && scratch_bytes >= need, BF_E_WORKSPACE, "bf_chain_ibp: scratch of %zu bytes needed", need);
      dst_l = scratch + (size_t)(2 * toggle) * (bf::align_up((size_t)B * chain->max_width * sizeof(float)) / sizeof(float));
      dst_u = scratch + (size_t)(2 * toggle + 1) * (bf::align_up((size_t)B * chain->max_width * sizeof(float)) / sizeof(float));
      toggle ^= 1;
    }
    int rc;
    if (L.op == BF_OP_LINEAR) {
      rc = bf::launch_ibp_linear(cur_a, cur_b, mode, relu_pending, L.W, L.bias, sp, sp_stride, cl, cu, dst_l, dst_u,
                                 infeasible, B, L.n_in, L.n_out, stream);
    } else {
      rc = bf::launch_ibp_conv2d(cur_a, cur_b, mode, relu_pending, L.W, L.bias, sp, sp_stride, cl, cu, dst_l, dst_u,
                                 infeasible, B, L, stream);
    }
    if (rc != BF_OK) return rc;
    cur_a = dst_l;
    cur_b = dst_u;
    mode = BF_IN_LOWER_UPPER;
    relu_pending = 0;
  }
  return BF_OK;
}

// ---------------------------------------------------------------------------
// CROWN sweep
// ---------------------------------------------------------------------------
namespace bf {

struct CrownWs {
  float* buf[2];
  float* cacc;
  float* partial;
  void* conv_scratch;
  size_t bytes;
};

static size_t crown_ws_layout(const bf_chain* c, int B, int S, int upto, void* base, CrownWs* ws) {
  const size_t M = (size_t)B * S;
  int maxw = c->n0;
  size_t conv_scratch = 0;
  for (int i = 0; i < upto; ++i) {
    if (c->layers[i].n_in > maxw) maxw = c->layers[i].n_in;
    if (c->layers[i].op == BF_OP_CONV2D) {
      size_t s = crown_bwd_conv2d_scratch_bytes((int)M, c->layers[i]);
      if (s > conv_scratch) conv_scratch = s;
    }
  }
  Carver cv(base);
  float* b0 = cv.take<float>(M * maxw);
  float* b1 = cv.take<float>(M * maxw);
  float* cacc = cv.take<float>(M);
  float* partial = cv.take<float>(M * (size_t)std::max(crown_bwd_partial_tiles(c->n0), crown_tc_partial_tiles(c->n0, 32)));
  char* cs = cv.take<char>(conv_scratch);
  if (ws) {
    ws->buf[0] = b0; ws->buf[1] = b1; ws->cacc = cacc; ws->partial = partial; ws->conv_scratch = cs; ws->bytes = cv.off;
  }
  return cv.off;
}

}  // namespace bf

extern "C" size_t bf_chain_crown_workspace_bytes(const bf_chain* chain, int B, int S, int upto_layer) {
  if (!chain || B <= 0 || S <= 0) return 0;
  if (upto_layer <= 0 || upto_layer > (int)chain->layers.size()) upto_layer = (int)chain->layers.size();
  return bf::crown_ws_layout(chain, B, S, upto_layer, nullptr, nullptr);
}

extern "C" int bf_chain_crown(const bf_chain* chain, int upto_layer, int side, const float* C,
                              const float* const* alpha_u, const float* const* beta_u, const float* const* alpha_l,
                              const float* const* add, const float* mid, const float* rad, float* out, void* workspace,
                              size_t workspace_bytes, int B, int S, bf_stream_t stream_) {
  BF_REQUIRE(chain && C && mid && rad && out && workspace, BF_E_INVALID, "bf_chain_crown: null argument");
  BF_REQUIRE(B > 0 && S > 0 && (long long)B * S < 2147483647LL, BF_E_INVALID, "bf_chain_crown: bad B/S");
  BF_REQUIRE(side == BF_SIDE_LOWER || side == BF_SIDE_UPPER, BF_E_INVALID, "bf_chain_crown: bad side");
  const int nl = (int)chain->layers.size();
  if (upto_layer <= 0 || upto_layer > nl) upto_layer = nl;
  cudaStream_t stream = bf::as_stream(stream_);
  bf::CrownWs ws;
  const size_t need = bf::crown_ws_layout(chain, B, S, upto_layer, workspace, &ws);
  BF_REQUIRE(workspace_bytes >= need, BF_E_WORKSPACE, "bf_chain_crown: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  const int M = B * S;
  const int low = bf::lowest_affine(chain);
  BF_REQUIRE(low >= 0 && low < upto_layer, BF_E_UNSUPPORTED, "bf_chain_crown: no affine layer below the bounded value");

  const float* curA = C;
  int pending = -1;
  int have_c = 0;
  int toggle = 0;
  bool fused_concretize = false;
  int ptiles = 1;
  for (int i = upto_layer - 1; i >= 0; --i) {
    const bf_layer_desc& L = chain->layers[i];
    if (L.op == BF_OP_FLATTEN) continue;
    if (L.op == BF_OP_RELU) {
      BF_REQUIRE(pending < 0, BF_E_UNSUPPORTED, "bf_chain_crown: two ReLUs without an affine layer between them");
      pending = bf::relu_index_of(chain, i);
      BF_REQUIRE(alpha_u && beta_u && alpha_l && alpha_u[pending] && beta_u[pending] && alpha_l[pending], BF_E_INVALID,
                 "bf_chain_crown: missing relaxation of ReLU %d", pending);
      continue;
    }
    const float *dpos = nullptr, *dneg = nullptr, *epos = nullptr, *eneg = nullptr, *ad = nullptr;
    if (pending >= 0) {
      if (side == BF_SIDE_LOWER) { dpos = alpha_l[pending]; dneg = alpha_u[pending]; eneg = beta_u[pending]; }
      else { dpos = alpha_u[pending]; dneg = alpha_l[pending]; epos = beta_u[pending]; }
      if (add && add[pending] && side == BF_SIDE_LOWER) ad = add[pending];
    }
    int rc;
    if (L.op == BF_OP_LINEAR) {
      const bool last = (i == low);
      float* dst = last ? nullptr : ws.buf[toggle];
      rc = bf::dispatch_bwd(chain, i, curA, dpos, dneg, epos, eneg, ad, dst, ws.cacc, have_c, last ? mid : nullptr,
                            last ? rad : nullptr, last ? ws.partial : nullptr, side, M, S, &ptiles, stream);
      if (last) fused_concretize = true;
      curA = dst;
    } else {
      BF_REQUIRE(ad == nullptr, BF_E_UNSUPPORTED, "bf_chain_crown: beta terms on conv layers are not supported");
      float* dst = ws.buf[toggle];
      rc = bf::launch_crown_bwd_conv2d(curA, dpos, dneg, epos, eneg, L.W, L.bias, dst, ws.cacc, have_c, M, S, L,
                                       ws.conv_scratch, stream);
      curA = dst;
    }
    if (rc != BF_OK) return rc;
    toggle ^= 1;
    have_c = 1;
    pending = -1;
  }
  BF_REQUIRE(pending < 0, BF_E_UNSUPPORTED, "bf_chain_crown: a ReLU directly on the input is not supported");
  if (fused_concretize) return bf::launch_sum_partials(ws.cacc, ws.partial, ptiles, out, M, stream);
  return bf::launch_concretize(curA, mid, rad, have_c ? ws.cacc : nullptr, out, side, B, S, chain->n0, stream);
}

// ---------------------------------------------------------------------------
// alpha-CROWN
// ---------------------------------------------------------------------------
namespace bf {

struct AlphaWs {
  std::vector<float*> au, bu, sl, grad, m, v, Ahat;
  float* A0;
  float* H[2];
  float* cacc;
  float* partial;
  float* cur;
  float* metric;
  int* improve;
  size_t state_floats_begin, state_bytes;  // grad/m/v region (zero-initialised)
  size_t bytes;
};

static size_t alpha_ws_layout(const bf_chain* c, int B, int S, void* base, AlphaWs* ws) {
  const size_t M = (size_t)B * S;
  const int R = (int)c->relu_layers.size();
  Carver cv(base);
  AlphaWs w;
  int maxw = 1;
  // zero-initialised optimiser state first, as one contiguous region
  const size_t z0 = cv.off;
  for (int r = 0; r < R; ++r) {
    const size_t n = (size_t)c->layers[c->relu_layers[r]].n_in;
    w.grad.push_back(cv.take<float>((size_t)B * n));
    w.m.push_back(cv.take<float>((size_t)B * n));
    w.v.push_back(cv.take<float>((size_t)B * n));
  }
  w.state_floats_begin = z0;
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
  w.partial = cv.take<float>(M * (size_t)std::max(crown_bwd_partial_tiles(c->n0), crown_tc_partial_tiles(c->n0, 32)));
  w.cur = cv.take<float>(M);
  w.metric = cv.take<float>((size_t)B);
  w.improve = cv.take<int>((size_t)B);
  w.bytes = cv.off;
  if (ws) *ws = w;
  return cv.off;
}

// One lower- or upper-side sweep of a linear/ReLU chain with the relaxations in ws.
static int alpha_sweep(const bf_chain* c, const AlphaWs& ws, const float* C, int side, bool keep_A0, const float* mid,
                       const float* rad, float* out, int B, int S, cudaStream_t stream) {
  const int M = B * S;
  const int R = (int)c->relu_layers.size();
  const bf_layer_desc& top = c->layers[2 * R];
  int rc;
  int ptiles = 1;
  (void)top;
  if (R == 0) {
    rc = dispatch_bwd(c, 2 * R, C, nullptr, nullptr, nullptr, nullptr, nullptr, keep_A0 ? ws.A0 : nullptr, ws.cacc, 0, mid, rad,
                      ws.partial, side, M, S, &ptiles, stream);
    if (rc != BF_OK) return rc;
  } else {
    rc = dispatch_bwd(c, 2 * R, C, nullptr, nullptr, nullptr, nullptr, nullptr, ws.Ahat[R - 1], ws.cacc, 0, nullptr, nullptr,
                      nullptr, side, M, S, nullptr, stream);
    if (rc != BF_OK) return rc;
    for (int r = R - 1; r >= 0; --r) {
      const bf_layer_desc& L = c->layers[2 * r];
      const float *dpos, *dneg, *epos = nullptr, *eneg = nullptr;
      if (side == BF_SIDE_LOWER) { dpos = ws.sl[r]; dneg = ws.au[r]; eneg = ws.bu[r]; }
      else { dpos = ws.au[r]; dneg = ws.sl[r]; epos = ws.bu[r]; }
      const bool last = (r == 0);
      float* dst = last ? (keep_A0 ? ws.A0 : nullptr) : ws.Ahat[r - 1];
      rc = dispatch_bwd(c, 2 * r, ws.Ahat[r], dpos, dneg, epos, eneg, nullptr, dst, ws.cacc, 1, last ? mid : nullptr,
                        last ? rad : nullptr, last ? ws.partial : nullptr, side, M, S, last ? &ptiles : nullptr, stream);
      if (rc != BF_OK) return rc;
    }
  }
  return launch_sum_partials(ws.cacc, ws.partial, ptiles, out, M, stream);
}

// Adjoint sweep: accumulates d(sum_s lower[b,s])/d(alpha_r[b,j]) into ws.grad[r].
static int alpha_adjoint(const bf_chain* c, const AlphaWs& ws, const float* const* pre_l, const float* const* pre_u,
                         const float* mid, const float* rad, int B, int S, cudaStream_t stream) {
  const int M = B * S;
  const int R = (int)c->relu_layers.size();
  for (int r = 0; r < R; ++r) {
    const bf_layer_desc& L = c->layers[2 * r];
    const float* hprev = (r == 0) ? ws.A0 : ws.H[(r - 1) & 1];
    float* hout = (r < R - 1) ? ws.H[r & 1] : nullptr;
    int rc = dispatch_adjoint(c, 2 * r, hprev, r == 0, mid, rad, ws.Ahat[r], ws.sl[r], ws.au[r], nullptr, ws.bu[r], pre_l[r],
                              pre_u[r], hout, ws.grad[r], M, S, stream);
    if (rc != BF_OK) return rc;
  }
  return BF_OK;
}

}  // namespace bf

extern "C" size_t bf_chain_alpha_workspace_bytes(const bf_chain* chain, int B, int S) {
  if (!chain || B <= 0 || S <= 0) return 0;
  return bf::alpha_ws_layout(chain, B, S, nullptr, nullptr);
}

static int alpha_common_checks(const char* who, const bf_chain* chain, const void* C, const void* pre_l, const void* pre_u,
                               const void* alpha, const void* mid, const void* rad, void* workspace, size_t workspace_bytes,
                               int B, int S, bf::AlphaWs* ws) {
  BF_REQUIRE(chain && C && pre_l && pre_u && alpha && mid && rad && workspace, BF_E_INVALID, "%s: null argument", who);
  BF_REQUIRE(B > 0 && S > 0 && (long long)B * S < 2147483647LL, BF_E_INVALID, "%s: bad B/S", who);
  BF_REQUIRE(chain->linear_relu_alternating, BF_E_UNSUPPORTED, "%s: only linear (relu linear)* chains are supported", who);
  const size_t need = bf::alpha_ws_layout(chain, B, S, workspace, ws);
  BF_REQUIRE(workspace_bytes >= need, BF_E_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who, need, workspace_bytes);
  return BF_OK;
}

extern "C" int bf_chain_alpha_crown(const bf_chain* chain, const float* C, const float* const* pre_l,
                                    const float* const* pre_u, float* const* alpha, float* const* best_alpha,
                                    const float* mid, const float* rad, float* best_lower, float* best_upper,
                                    float* best_metric, int steps, float lr, int spec_reduce, void* workspace,
                                    size_t workspace_bytes, int B, int S, bf_stream_t stream_) {
  bf::AlphaWs ws;
  int rc = alpha_common_checks("bf_chain_alpha_crown", chain, C, pre_l, pre_u, alpha, mid, rad, workspace, workspace_bytes, B, S, &ws);
  if (rc != BF_OK) return rc;
  BF_REQUIRE(best_alpha && best_lower && steps >= 0, BF_E_INVALID, "bf_chain_alpha_crown: null output or negative steps");
  BF_REQUIRE(spec_reduce == BF_REDUCE_MEAN || spec_reduce == BF_REDUCE_SUM, BF_E_INVALID, "bf_chain_alpha_crown: bad spec_reduce");
  cudaStream_t stream = bf::as_stream(stream_);
  const int R = (int)chain->relu_layers.size();
  float* metric = best_metric ? best_metric : ws.metric;

  if (cudaMemsetAsync(static_cast<char*>(workspace) + ws.state_floats_begin, 0, ws.state_bytes, stream) != cudaSuccess) {
    bf::set_error("bf_chain_alpha_crown: cudaMemsetAsync failed");
    return BF_E_CUDA;
  }
  for (int r = 0; r < R; ++r) {
    const int n = chain->layers[chain->relu_layers[r]].n_in;
    rc = bf::launch_relu_relax(pre_l[r], pre_u[r], alpha[r], n, ws.au[r], ws.bu[r], ws.sl[r], B, n, stream);
    if (rc != BF_OK) return rc;
  }
  const double beta1 = 0.9, beta2 = 0.999;
  for (int t = 0; t <= steps; ++t) {
    const bool last = (t == steps);
    rc = bf::alpha_sweep(chain, ws, C, BF_SIDE_LOWER, !last, mid, rad, ws.cur, B, S, stream);
    if (rc != BF_OK) return rc;
    rc = bf::launch_select_best(ws.cur, best_lower, metric, ws.improve, t == 0, spec_reduce, B, S, stream);
    if (rc != BF_OK) return rc;
    bf::AdamScalars sc{};
    if (!last) {
      rc = bf::alpha_adjoint(chain, ws, pre_l, pre_u, mid, rad, B, S, stream);
      if (rc != BF_OK) return rc;
      const double bc1 = 1.0 - pow(beta1, t + 1), bc2 = 1.0 - pow(beta2, t + 1);
      sc.lr_step = (float)((double)lr / bc1);
      sc.bc2_sqrt = (float)sqrt(bc2);
      sc.beta1 = (float)beta1;
      sc.beta2 = (float)beta2;
      sc.eps = 1e-8f;
      sc.one_minus_beta1 = (float)(1.0 - beta1);
      sc.one_minus_beta2 = (float)(1.0 - beta2);
      sc.grad_scale = (spec_reduce == BF_REDUCE_MEAN) ? (-1.0f / (float)S) : -1.0f;
    }
    for (int r = 0; r < R; ++r) {
      const int n = chain->layers[chain->relu_layers[r]].n_in;
      rc = bf::launch_adam_step(alpha[r], ws.m[r], ws.v[r], ws.grad[r], ws.improve, best_alpha[r], pre_l[r], pre_u[r],
                                ws.sl[r], sc, last ? 0 : 1, B, n, stream);
      if (rc != BF_OK) return rc;
    }
  }
  if (best_upper) {
    for (int r = 0; r < R; ++r) {
      const int n = chain->layers[chain->relu_layers[r]].n_in;
      rc = bf::launch_relu_relax(pre_l[r], pre_u[r], best_alpha[r], n, ws.au[r], ws.bu[r], ws.sl[r], B, n, stream);
      if (rc != BF_OK) return rc;
    }
    rc = bf::alpha_sweep(chain, ws, C, BF_SIDE_UPPER, false, mid, rad, best_upper, B, S, stream);
    if (rc != BF_OK) return rc;
  }
  return BF_OK;
}

extern "C" int bf_chain_alpha_grad(const bf_chain* chain, const float* C, const float* const* pre_l,
                                   const float* const* pre_u, const float* const* alpha, const float* mid,
                                   const float* rad, float* const* grad, float* lower, int spec_reduce, void* workspace,
                                   size_t workspace_bytes, int B, int S, bf_stream_t stream_) {
  bf::AlphaWs ws;
  int rc = alpha_common_checks("bf_chain_alpha_grad", chain, C, pre_l, pre_u, alpha, mid, rad, workspace, workspace_bytes, B, S, &ws);
  if (rc != BF_OK) return rc;
  BF_REQUIRE(grad && lower, BF_E_INVALID, "bf_chain_alpha_grad: null output");
  cudaStream_t stream = bf::as_stream(stream_);
  const int R = (int)chain->relu_layers.size();
  if (cudaMemsetAsync(static_cast<char*>(workspace) + ws.state_floats_begin, 0, ws.state_bytes, stream) != cudaSuccess) {
    bf::set_error("bf_chain_alpha_grad: cudaMemsetAsync failed");
    return BF_E_CUDA;
  }
  for (int r = 0; r < R; ++r) {
    const int n = chain->layers[chain->relu_layers[r]].n_in;
    rc = bf::launch_relu_relax(pre_l[r], pre_u[r], alpha[r], n, ws.au[r], ws.bu[r], ws.sl[r], B, n, stream);
    if (rc != BF_OK) return rc;
  }
  rc = bf::alpha_sweep(chain, ws, C, BF_SIDE_LOWER, true, mid, rad, lower, B, S, stream);
  if (rc != BF_OK) return rc;
  rc = bf::alpha_adjoint(chain, ws, pre_l, pre_u, mid, rad, B, S, stream);
  if (rc != BF_OK) return rc;
  const float scale = (spec_reduce == BF_REDUCE_MEAN) ? (-1.0f / (float)S) : -1.0f;
  for (int r = 0; r < R; ++r) {
    const int n = chain->layers[chain->relu_layers[r]].n_in;
    rc = bf::launch_scale_copy(ws.grad[r], scale, grad[r], (long long)B * n, stream);
    if (rc != BF_OK) return rc;
  }
  return BF_OK;
}
