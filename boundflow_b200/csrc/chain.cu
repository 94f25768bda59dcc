// Whole-chain drivers: host loops that string the layer kernels together on one
// stream without any host synchronisation (IBP trace, CROWN sweep, the
// alpha-CROWN optimisation loop and its analytic gradient).
#include <math.h>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <vector>

#include "chain_internal.cuh"

namespace bf {

static thread_local char g_err[512] = "ok";
std::atomic<unsigned long long> g_launches{0};
std::atomic<unsigned long long> g_tc_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

// ---- optional kernel timing ----------------------------------------------------
// One mutex guards the slots: launches from several host threads interleave their event pairs safely
// (a begin/end pair is matched by slot and thread: the open event index is kept per thread).
struct TimingSlot {
  std::vector<cudaEvent_t> start, stop;
  size_t used = 0;
  double bytes = 0.0, flops = 0.0;
};
static TimingSlot g_timing[T_SLOTS];
static std::atomic<bool> g_timing_on{false};
static std::mutex g_timing_mutex;
static thread_local long long g_timing_open[T_SLOTS];  // index + 1 of this thread's open event pair per slot

void timing_begin(int slot, cudaStream_t stream) {
  if (!g_timing_on.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  TimingSlot& t = g_timing[slot];
  g_timing_open[slot] = 0;
  if (t.used == t.start.size()) {
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess) return;
    if (cudaEventCreate(&b) != cudaSuccess) {
      cudaEventDestroy(a);
      return;
    }
    t.start.push_back(a);
    t.stop.push_back(b);
  }
  cudaEventRecord(t.start[t.used], stream);
  g_timing_open[slot] = (long long)(++t.used);
}

void timing_end(int slot, cudaStream_t stream, double bytes, double flops) {
  if (g_timing_open[slot] == 0) return;
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  TimingSlot& t = g_timing[slot];
  const size_t idx = (size_t)(g_timing_open[slot] - 1);
  g_timing_open[slot] = 0;
  if (idx >= t.used) return;  // the slots were reset between begin and end
  cudaEventRecord(t.stop[idx], stream);
  t.bytes += bytes;
  t.flops += flops;
}

static const char* const g_timing_names[T_SLOTS] = {
    "crown_bwd_contraction", "crown_adjoint_contraction", "crown_bwd_thin_kernel", "ibp_linear_kernel", "ibp_conv2d_kernel",
    "adam_step_kernel", "concretize_kernel", "relu_bwd_window_kernel", "conv_transpose_kernel", "relu_bwd_rows_kernel"};

}  // namespace bf

extern "C" void bf_kernel_timing_enable(int on) {
  std::lock_guard<std::mutex> lock(bf::g_timing_mutex);
  bf::g_timing_on.store(on != 0);
  for (auto& t : bf::g_timing) {
    t.used = 0;
    t.bytes = 0.0;
    t.flops = 0.0;
  }
}

extern "C" int bf_kernel_timing_slots(void) { return bf::T_SLOTS; }

extern "C" const char* bf_kernel_timing_slot_name(int slot) {
  return (slot >= 0 && slot < bf::T_SLOTS) ? bf::g_timing_names[slot] : "";
}

extern "C" int bf_kernel_timing_read_work(int slot, int* launches, float* total_ms, double* bytes, double* flops) {
  BF_REQUIRE(slot >= 0 && slot < bf::T_SLOTS && launches && total_ms, BF_E_INVALID, "bf_kernel_timing_read: bad argument");
  std::lock_guard<std::mutex> lock(bf::g_timing_mutex);
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
  if (bytes) *bytes = t.bytes;
  if (flops) *flops = t.flops;
  return BF_OK;
}

extern "C" int bf_kernel_timing_read(int slot, int* launches, float* total_ms) {
  return bf_kernel_timing_read_work(slot, launches, total_ms, nullptr, nullptr);
}


extern "C" int bf_version(void) { return 100; }
extern "C" const char* bf_last_error_string(void) { return bf::g_err; }
extern "C" unsigned long long bf_launch_count(void) { return bf::g_launches.load(); }
extern "C" unsigned long long bf_tc_launch_count(void) { return bf::g_tc_launches.load(); }

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
  {
    // affine (relu affine)* with flatten layers anywhere in between
    bool ok = true, want_affine = true;
    for (int i = 0; i < n_layers; ++i) {
      const int op = c->layers[i].op;
      if (op == BF_OP_FLATTEN) continue;
      const bool is_affine = (op == BF_OP_LINEAR || op == BF_OP_CONV2D);
      if (is_affine != want_affine) ok = false;
      if (is_affine) c->affine_layers.push_back(i);
      if (op == BF_OP_CONV2D) c->has_conv = true;
      want_affine = !want_affine;
    }
    c->affine_relu_alternating = ok && !want_affine && c->affine_layers.size() == c->relu_layers.size() + 1;
  }
  *out = c;
  return BF_OK;
}

extern "C" void bf_chain_destroy(bf_chain* chain) { delete chain; }
extern "C" int bf_chain_num_relu(const bf_chain* chain) { return chain ? (int)chain->relu_layers.size() : BF_E_INVALID; }

namespace bf {

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
                            const bf_layer_desc& L, void* scratch, cudaStream_t stream, const float* add = nullptr);
size_t crown_bwd_conv2d_scratch_bytes(int M, const bf_layer_desc& L);
int launch_onehot_conv_rows(int first, const float* W, const float* bias, float* A_prev, float* delta, int M, int S,
                            const bf_layer_desc& L, cudaStream_t stream);
int launch_onehot_linear_rows(int first, const float* W, const float* bias, float* A_prev, float* delta, int M, int S, int n_in,
                              cudaStream_t stream);
}  // namespace bf

// ---------------------------------------------------------------------------
// tensor-core path set-up and dispatch
// ---------------------------------------------------------------------------
namespace bf {

// The feature-major adjoint kernel works on 256-row x 256-feature CTAs: it pays off once those fill the GPU;
// smaller problems keep the row-major kernel (128-row CTAs, twice as many of them).
static bool env_is_one(const char* name) {
  const char* e = getenv(name);
  return e && e[0] == '1';
}

void refresh_switches(const bf_chain* c) {
  c->sw.force_ffma = env_is_one("BF_B200_FORCE_FFMA");
  c->sw.adjoint_kernel = env_is_one("BF_B200_ADJ_ROWMAJOR") ? 1 : (env_is_one("BF_B200_ADJ_FEATURE_MAJOR") ? 2 : 0);
  c->sw.no_windows = getenv("BF_B200_NO_WINDOWS") != nullptr;
  c->sw.persistent_bwd = env_is_one("BF_B200_BWD_PERSISTENT");
  c->sw.pair_bwd = env_is_one("BF_B200_BWD_PAIRS");
  const char* rows = getenv("BF_B200_TC_MIN_ROWS");
  c->sw.tc_min_rows = (rows && atoi(rows) > 0) ? atoi(rows) : 256;
  c->sw.tc_auto = !(rows && atoi(rows) > 0);
}

bool tc_may_run(const bf_chain* c, int M) { return c->status != nullptr && !c->pk_bwd.empty() && !c->sw.force_ffma && M >= c->sw.tc_min_rows; }

static bool adjoint_feature_major(const bf_chain* c, int M, int N) {
  if (c->sw.adjoint_kernel == 1) return false;
  if (c->sw.adjoint_kernel == 2) return true;
  const long long ctas = (long long)((M + 255) / 256) * ((((N + tc_adjoint_tile_rows() - 1) / tc_adjoint_tile_rows()) + 1) / 2);
  // measured: with the GPU filled the feature-major kernel wins; below that it still wins on layers of 512 and more features
  // (two feature CTAs per row block: c4 with 384-1024 subdomains 5.95-6.23 against 6.64-6.90 ms per call), the row-major
  // kernel on narrower ones (256 features, 9216-18432 rows: 4.7 against 5.2 ms)
  return ctas >= 128 || N >= 512;
}

static const unsigned char* tc_weights(const bf_chain* c, int layer, bool adjoint, int M, int K, int N) {
  if (c->pk_bwd.empty() || c->sw.force_ffma) return nullptr;
  if (M < c->sw.tc_min_rows || K < 32 || N < 32) return nullptr;  // tiny problems stay on the FFMA tiles
  if (c->sw.tc_auto && ffma_fits_one_wave(M, N)) return nullptr;   // so do layers whose 64 x 64 tiles fit one wave
  return adjoint ? c->pk_adj[layer] : c->pk_bwd[layer];
}

// Backward contraction of linear layer `layer`; *ptiles receives the number of column tiles
// (the second dimension of the concretisation partial-sum buffer).
int dispatch_bwd(const bf_chain* c, int layer, const float* A, const float* dpos, const float* dneg,
                        const float* epos, const float* eneg, const float* add, float* A_prev, float* delta, int accumulate,
                        const float* mid, const float* rad, float* partial, int side, int M, int S, int* ptiles,
                        cudaStream_t stream) {
  const bf_layer_desc& L = c->layers[layer];
  const int K = L.n_out, N = L.n_in;
  const unsigned char* pk = tc_weights(c, layer, false, M, K, N);
  if (pk && c->sw.persistent_bwd && crown_tc_persistent_supports(epos, eneg, add)) {
    if (ptiles) *ptiles = crown_tc_persist_partial_tiles(M, N, K);
    return launch_crown_bwd_linear_tc_persistent(A, dpos, dneg, epos, eneg, add, pk, L.bias, A_prev, delta, accumulate, mid, rad,
                                                 partial, side, M, S, K, N, c->status, stream);
  }
  if (pk) {
    if (ptiles) *ptiles = crown_tc_partial_tiles(N, K);
    return launch_crown_bwd_linear_tc(A, dpos, dneg, epos, eneg, add, pk, L.bias, A_prev, delta, accumulate, mid, rad, partial,
                                      side, M, S, K, N, c->status, stream, c->sw.pair_bwd);
  }
  if (ptiles) *ptiles = crown_bwd_partial_tiles(N, M);
  return launch_crown_bwd_linear(A, dpos, dneg, epos, eneg, add, L.W, L.bias, A_prev, delta, accumulate, mid, rad, partial, side,
                                 M, S, K, N, stream);
}

int dispatch_adjoint(const bf_chain* c, int layer, const float* Hprev, int first_layer, const float* mid,
                            const float* rad, const float* Ahat, const float* dpos, const float* dneg, const float* epos,
                            const float* eneg, const float* pre_l, const float* pre_u, float* hout, float* grad, float* gsum,
                            int M, int S, cudaStream_t stream, const float* gw) {
  const bf_layer_desc& L = c->layers[layer];
  const int K = L.n_in, N = L.n_out;
  const unsigned char* pk = tc_weights(c, layer, true, M, K, N);
  // gw (row weights of the beta sums, min / softmin with beta parameters) is implemented by the row-major and FFMA kernels
  if (pk && gw == nullptr && adjoint_feature_major(c, M, N))
    return launch_crown_adjoint_linear_tc_fm(Hprev, first_layer, mid, rad, c->pk_adj_fm[layer], L.bias, Ahat, dpos, dneg, epos, eneg, pre_l, pre_u,
                                             hout, grad, gsum, M, S, K, N, c->status, stream);
  if (pk)
    return launch_crown_adjoint_linear_tc(Hprev, first_layer, mid, rad, pk, L.bias, Ahat, dpos, dneg, epos, eneg, pre_l, pre_u,
                                          hout, grad, gsum, M, S, K, N, c->status, stream, gw);
  return launch_crown_adjoint_linear(Hprev, first_layer, mid, rad, L.W, L.bias, Ahat, dpos, dneg, epos, eneg, pre_l, pre_u, hout,
                                     grad, gsum, M, S, K, N, stream, gw);
}

}  // namespace bf

extern "C" size_t bf_chain_tc_bytes(const bf_chain* chain) {
  if (!chain) return 0;
  size_t total = 256;  // status word
  for (const bf_layer_desc& L : chain->layers)
    if (L.op == BF_OP_LINEAR)
      total += bf::align_up(bf::tc_packed_bytes(L.n_in, L.n_out)) + bf::align_up(bf::tc_packed_bytes(L.n_out, L.n_in)) +
               bf::align_up(bf::tc_packed_bytes(L.n_out, L.n_in, bf::tc_adjoint_tile_rows()));
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
  chain->pk_adj_fm.assign(chain->layers.size(), nullptr);
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
    // the same orientation as 128-row images (features on the MMA's M side)
    unsigned char* pf = base + off;
    off += bf::align_up(bf::tc_packed_bytes(L.n_out, L.n_in, bf::tc_adjoint_tile_rows()));
    rc = bf::tc_pack_weights(L.W, L.n_out, L.n_in, 0, pf, stream, bf::tc_adjoint_tile_rows());
    if (rc != BF_OK) return rc;
    chain->pk_adj_fm[i] = pf;
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
      if (mode == BF_IN_CENTER_DEV)  // Lp ball on the input: in_b holds eps * dual norm of this layer's weight rows
        rc = bf::launch_ibp_linear(cur_a, nullptr, BF_IN_MID_RAD, 0, L.W, L.bias, sp, sp_stride, cl, cu, dst_l, dst_u, infeasible, B,
                                   L.n_in, L.n_out, cur_b, stream);
      else
        rc = bf::launch_ibp_linear(cur_a, cur_b, mode, relu_pending, L.W, L.bias, sp, sp_stride, cl, cu, dst_l, dst_u,
                                   infeasible, B, L.n_in, L.n_out, nullptr, stream);
    } else {
      BF_REQUIRE(mode != BF_IN_CENTER_DEV, BF_E_UNSUPPORTED, "bf_chain_ibp: an Lp-ball input needs a Linear first layer (give a box otherwise)");
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
  float* partial = cv.take<float>(M * (size_t)std::max(std::max(crown_bwd_partial_tiles(c->n0), crown_tc_partial_tiles(c->n0, 32)), crown_tc_persist_max_partial_tiles(c->n0)));
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

// One sweep; `C` dense [B,S,width of the bounded value], or NULL with onehot_first >= 0: the spec rows are rows
// onehot_first .. onehot_first+S-1 of the identity for every domain.
static int crown_sweep(const bf_chain* chain, int upto_layer, int side, const float* C, int onehot_first,
                       const float* const* alpha_u, const float* const* beta_u, const float* const* alpha_l,
                       const float* const* add, const float* mid, const float* rad, int norm_p, float eps, float* out,
                       void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream_,
                       float* const* influence = nullptr) {
  BF_REQUIRE(chain && (C || onehot_first >= 0) && mid && out && workspace, BF_E_INVALID, "bf_chain_crown: null argument");
  BF_REQUIRE(norm_p == BF_NORM_BOX || norm_p == BF_NORM_INF || norm_p == BF_NORM_L2 || norm_p == BF_NORM_L1, BF_E_INVALID,
             "bf_chain_crown: bad norm");
  BF_REQUIRE(norm_p != BF_NORM_BOX || rad != nullptr, BF_E_INVALID, "bf_chain_crown: a box needs its radius tensor");
  const bool box = (norm_p == BF_NORM_BOX);
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
  // identity-row sweeps on conv layers keep only the window of each row that can be non-zero (see conv.cu)
  bf::WindowGeom win{};
  bool windowed = false;
  bf::refresh_switches(chain);
  const bool windows_allowed = box && influence == nullptr && !chain->sw.no_windows;
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
      if (add && add[pending]) ad = add[pending];  // the caller passes the add terms of the side it asks for
    }
    int rc;
    if (windowed && !(L.op == BF_OP_CONV2D && pending >= 0 && ad == nullptr && win.C == L.Co && win.H == L.Ho && win.W == L.Wo &&
                      (win.WH - 1) * L.sh + L.kh < L.Hi && (win.WW - 1) * L.sw + L.kw < L.Wi)) {
      // the window has grown to the feature map (or the next layer is not a ReLU + conv pair): back to full rows
      float* dense = ws.buf[toggle];
      rc = bf::launch_window_to_dense(curA, dense, win, M, stream);
      if (rc != BF_OK) return rc;
      curA = dense;
      toggle ^= 1;
      windowed = false;
    }
    if (influence && pending >= 0 && influence[pending]) {
      BF_REQUIRE(curA != nullptr, BF_E_UNSUPPORTED, "bf_chain_crown_influence: no coefficients reach this ReLU");
      rc = bf::launch_colmax_abs(curA, influence[pending], B, S, chain->layers[chain->relu_layers[pending]].n_in, stream);
      if (rc != BF_OK) return rc;
    }
    if (curA == nullptr) {
      // identity spec rows: the first backward step copies weights instead of multiplying by them
      BF_REQUIRE(pending < 0, BF_E_UNSUPPORTED, "bf_chain_crown_onehot: the bounded value must be the output of an affine layer");
      BF_REQUIRE(onehot_first + S <= L.n_out, BF_E_INVALID, "bf_chain_crown_onehot: rows %d..%d exceed the value's width %d",
                 onehot_first, onehot_first + S - 1, L.n_out);
      float* dst = ws.buf[toggle];
      if (L.op == BF_OP_LINEAR) {
        rc = bf::launch_onehot_linear_rows(onehot_first, L.W, L.bias, dst, ws.cacc, M, S, L.n_in, stream);
      } else if (windows_allowed && L.kh < L.Hi && L.kw < L.Wi) {
        win = bf::WindowGeom{M, onehot_first, S, L.Ho, L.Wo, L.Ci, L.kh, L.kw, L.Hi, L.Wi, L.sh, -L.ph, L.sw, -L.pw};
        windowed = true;
        rc = bf::launch_onehot_conv_window(L.W, L.bias, dst, ws.cacc, win, M, L.Ci, L.kh * L.kw, stream);
      } else {
        rc = bf::launch_onehot_conv_rows(onehot_first, L.W, L.bias, dst, ws.cacc, M, S, L, stream);
      }
      curA = dst;
    } else if (windowed && L.op == BF_OP_CONV2D && pending >= 0 && ad == nullptr && win.C == L.Co && win.H == L.Ho && win.W == L.Wo &&
               (win.WH - 1) * L.sh + L.kh < L.Hi && (win.WW - 1) * L.sw + L.kw < L.Wi) {
      // ReLU pass and transposed convolution in window coordinates (zero padding: the window grows by the kernel)
      float* lam = static_cast<float*>(ws.conv_scratch);
      rc = bf::launch_relu_bwd_window(curA, dpos, dneg, epos, eneg, L.bias, lam, ws.cacc, win, M, stream);
      if (rc != BF_OK) return rc;
      bf_layer_desc Lw = L;
      Lw.Ho = win.WH; Lw.Wo = win.WW;
      Lw.Hi = (win.WH - 1) * L.sh + L.kh; Lw.Wi = (win.WW - 1) * L.sw + L.kw;
      Lw.ph = 0; Lw.pw = 0;
      Lw.n_out = L.Co * Lw.Ho * Lw.Wo; Lw.n_in = L.Ci * Lw.Hi * Lw.Wi;
      float* dst = ws.buf[toggle];
      rc = bf::launch_crown_bwd_conv2d(lam, nullptr, nullptr, nullptr, nullptr, L.W, nullptr, dst, nullptr, 1, M, S, Lw, nullptr, stream);
      win.C = L.Ci; win.WH = Lw.Hi; win.WW = Lw.Wi; win.H = L.Hi; win.W = L.Wi;
      win.ty = win.ty * L.sh - L.ph; win.sy *= L.sh;
      win.tx = win.tx * L.sw - L.pw; win.sx *= L.sw;
      curA = dst;
    } else if (L.op == BF_OP_LINEAR) {
      const bool last = box && (i == low);  // the fused concretisation handles boxes; Lp balls concretise separately
      float* dst = last ? nullptr : ws.buf[toggle];
      rc = bf::dispatch_bwd(chain, i, curA, dpos, dneg, epos, eneg, ad, dst, ws.cacc, have_c, last ? mid : nullptr,
                            last ? rad : nullptr, last ? ws.partial : nullptr, side, M, S, &ptiles, stream);
      if (last) fused_concretize = true;
      curA = dst;
    } else {
      float* dst = ws.buf[toggle];
      rc = bf::launch_crown_bwd_conv2d(curA, dpos, dneg, epos, eneg, L.W, L.bias, dst, ws.cacc, have_c, M, S, L,
                                       ws.conv_scratch, stream, ad);
      curA = dst;
    }
    if (rc != BF_OK) return rc;
    toggle ^= 1;
    have_c = 1;
    pending = -1;
  }
  BF_REQUIRE(pending < 0, BF_E_UNSUPPORTED, "bf_chain_crown: a ReLU directly on the input is not supported");
  int rc;
  if (windowed) rc = bf::launch_concretize_window(curA, mid, rad, ws.cacc, out, side, win, M, stream);
  else if (fused_concretize) rc = bf::launch_sum_partials(ws.cacc, ws.partial, ptiles, out, M, stream);
  else if (!box) rc = bf::launch_concretize_lp(curA, mid, have_c ? ws.cacc : nullptr, out, side, eps, norm_p, B, S, chain->n0, stream);
  else rc = bf::launch_concretize(curA, mid, rad, have_c ? ws.cacc : nullptr, out, side, B, S, chain->n0, stream);
  if (rc == BF_OK && bf::tc_may_run(chain, M)) rc = bf::launch_poison_on_status(chain->status, out, M, nullptr, 0, stream);
  return rc;
}

extern "C" int bf_chain_crown(const bf_chain* chain, int upto_layer, int side, const float* C,
                              const float* const* alpha_u, const float* const* beta_u, const float* const* alpha_l,
                              const float* const* add, const float* mid, const float* rad, int norm_p, float eps, float* out,
                              void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream) {
  BF_REQUIRE(C, BF_E_INVALID, "bf_chain_crown: null argument");
  return crown_sweep(chain, upto_layer, side, C, -1, alpha_u, beta_u, alpha_l, add, mid, rad, norm_p, eps, out, workspace,
                     workspace_bytes, B, S, stream);
}

extern "C" int bf_chain_crown_influence(const bf_chain* chain, int upto_layer, int side, const float* C,
                                        const float* const* alpha_u, const float* const* beta_u, const float* const* alpha_l,
                                        const float* const* add, const float* mid, const float* rad, int norm_p, float eps,
                                        float* out, float* const* influence, void* workspace, size_t workspace_bytes, int B, int S,
                                        bf_stream_t stream) {
  BF_REQUIRE(C && influence, BF_E_INVALID, "bf_chain_crown_influence: null argument");
  return crown_sweep(chain, upto_layer, side, C, -1, alpha_u, beta_u, alpha_l, add, mid, rad, norm_p, eps, out, workspace,
                     workspace_bytes, B, S, stream, influence);
}

extern "C" int bf_chain_crown_onehot(const bf_chain* chain, int upto_layer, int side, int first_row,
                                     const float* const* alpha_u, const float* const* beta_u, const float* const* alpha_l,
                                     const float* const* add, const float* mid, const float* rad, int norm_p, float eps,
                                     float* out, void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream) {
  BF_REQUIRE(first_row >= 0, BF_E_INVALID, "bf_chain_crown_onehot: negative first row");
  return crown_sweep(chain, upto_layer, side, nullptr, first_row, alpha_u, beta_u, alpha_l, add, mid, rad, norm_p, eps, out,
                     workspace, workspace_bytes, B, S, stream);
}

