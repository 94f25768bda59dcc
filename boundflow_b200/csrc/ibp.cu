// Interval bound propagation through a Linear layer in centre/radius form:
//   c = (relu(l)+relu(u))/2, r = (relu(u)-relu(l))/2
//   y_l = W c - |W| r + b,  y_u = W c + |W| r + b
// fused with the preceding interval ReLU, the pre-activation constraint
// intersection and the ReLU split clamp.  One CTA owns a 64x64 output tile and
// keeps two accumulators per output (centre and radius); |W| costs nothing
// (absolute value is an operand modifier of FFMA).
#include "kernels.cuh"

namespace bf {

constexpr int IBM = 64, IBN = 64, IBK = 16, ILD = 68, ISLAB = IBK * ILD;

struct IbpArgs {
  const float* in_a; const float* in_b; int in_mode; int relu_in;
  const float* W; const float* bias;
  const int8_t* split; int split_stride;
  const float* cons_l; const float* cons_u;
  float* out_l; float* out_u; int* infeasible;
  int B, K, N; int vecK, vecN;
  const float* row_dev;  // [N] or null: per-output deviation (eps * dual norm of the weight row), Lp-ball first layer
};

// Two CTAs per SM (95 registers).  Forcing three (80 registers) was measured at +2 % on 8192 x 512 x 512, +10 % on the
// 784-wide first layer and -7 % on 1024 rows and fewer; four CTAs spill and lose everywhere: occupancy is not the limit.  A 64 x 128 tile (4 x 8 outputs per thread, 1.0 instead of
// 1.5 shared-memory bytes per FFMA, 128 registers) was measured at 233 against 226 us on 8192 x 512 x 512 (512 CTAs are 1.7
// waves of 296), 364 against 391 us on the 784-wide layer and 137 against 105 us on a ragged 260-wide one: not kept.
__global__ void __launch_bounds__(256) ibp_linear_kernel(IbpArgs g) {
  __shared__ __align__(16) float smem[2 * 3 * ISLAB];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.x * IBM, n0 = blockIdx.y * IBN;
  const int lrow = tid >> 2, lkc = (tid & 3) * 4;
  const bool vK = g.vecK != 0, vN = g.vecN != 0;

  float accC[4][4], accR[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) accC[i][j] = accR[i][j] = 0.f;

  float4 creg, rreg, wreg;
  auto load_slab = [&](int kt) {
    const int k = kt * IBK + lkc;
    const int m = m0 + lrow, n = n0 + lrow;
    creg = rreg = wreg = make_float4(0.f, 0.f, 0.f, 0.f);
    if (m < g.B && k < g.K) {
      float4 a = load4_guard(g.in_a + (size_t)m * g.K, k, g.K, vK);
      float4 b = g.in_b ? load4_guard(g.in_b + (size_t)m * g.K, k, g.K, vK) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (g.in_mode == BF_IN_LOWER_UPPER) {
        if (g.relu_in) {
          a.x = fmaxf(a.x, 0.f); a.y = fmaxf(a.y, 0.f); a.z = fmaxf(a.z, 0.f); a.w = fmaxf(a.w, 0.f);
          b.x = fmaxf(b.x, 0.f); b.y = fmaxf(b.y, 0.f); b.z = fmaxf(b.z, 0.f); b.w = fmaxf(b.w, 0.f);
        }
        creg = make_float4((a.x + b.x) * 0.5f, (a.y + b.y) * 0.5f, (a.z + b.z) * 0.5f, (a.w + b.w) * 0.5f);
        rreg = make_float4((b.x - a.x) * 0.5f, (b.y - a.y) * 0.5f, (b.z - a.z) * 0.5f, (b.w - a.w) * 0.5f);
      } else {
        creg = a;
        rreg = b;
      }
    }
    if (n < g.N && k < g.K) wreg = load4_guard(g.W + (size_t)n * g.K, k, g.K, vK);
  };
  auto store_slab = [&](int stage) {
    float* cs = smem + stage * 3 * ISLAB;
    float* rs = cs + ISLAB;
    float* ws = rs + ISLAB;
    cs[(lkc + 0) * ILD + lrow] = creg.x; cs[(lkc + 1) * ILD + lrow] = creg.y;
    cs[(lkc + 2) * ILD + lrow] = creg.z; cs[(lkc + 3) * ILD + lrow] = creg.w;
    rs[(lkc + 0) * ILD + lrow] = rreg.x; rs[(lkc + 1) * ILD + lrow] = rreg.y;
    rs[(lkc + 2) * ILD + lrow] = rreg.z; rs[(lkc + 3) * ILD + lrow] = rreg.w;
    ws[(lkc + 0) * ILD + lrow] = wreg.x; ws[(lkc + 1) * ILD + lrow] = wreg.y;
    ws[(lkc + 2) * ILD + lrow] = wreg.z; ws[(lkc + 3) * ILD + lrow] = wreg.w;
  };

  const int nk = (g.K + IBK - 1) / IBK;
  load_slab(0);
  store_slab(0);
  __syncthreads();
  for (int kt = 0; kt < nk; ++kt) {
    const int stage = kt & 1;
    if (kt + 1 < nk) load_slab(kt + 1);
    const float* cs = smem + stage * 3 * ISLAB;
    const float* rs = cs + ISLAB;
    const float* ws = rs + ISLAB;
#pragma unroll
    for (int kk = 0; kk < IBK; ++kk) {
      const float4 c4 = *reinterpret_cast<const float4*>(&cs[kk * ILD + ty * 4]);
      const float4 r4 = *reinterpret_cast<const float4*>(&rs[kk * ILD + ty * 4]);
      const float4 w4 = *reinterpret_cast<const float4*>(&ws[kk * ILD + tx * 4]);
      const float c[4] = {c4.x, c4.y, c4.z, c4.w};
      const float r[4] = {r4.x, r4.y, r4.z, r4.w};
      const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          accC[i][j] = fmaf(c[i], w[j], accC[i][j]);
          accR[i][j] = fmaf(r[i], fabsf(w[j]), accR[i][j]);
        }
    }
    if (kt + 1 < nk) store_slab(stage ^ 1);
    __syncthreads();
  }

  const int col = n0 + tx * 4;
  if (col >= g.N) return;
  float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (g.bias) bv = load4_guard(g.bias, col, g.N, vN);
  const float bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + ty * 4 + i;
    if (row >= g.B) continue;
    float lo[4], up[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo[j] = (accC[i][j] - accR[i][j]) + bb[j];
      up[j] = (accC[i][j] + accR[i][j]) + bb[j];
    }
    if (g.row_dev) {  // Lp-ball first layer: deviation eps * ||W_row||_q instead of |W| * radius
      const float4 dv = load4_guard(g.row_dev, col, g.N, vN);
      const float d4[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo[j] -= d4[j];
        up[j] += d4[j];
      }
    }
    bool bad = false;
    if (g.cons_l) {
      const float4 cl = load4_guard(g.cons_l + (size_t)row * g.N, col, g.N, vN);
      const float4 cu = load4_guard(g.cons_u + (size_t)row * g.N, col, g.N, vN);
      const float cl4[4] = {cl.x, cl.y, cl.z, cl.w}, cu4[4] = {cu.x, cu.y, cu.z, cu.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (col + j < g.N) {
          lo[j] = fmaxf(lo[j], cl4[j]);
          up[j] = fminf(up[j], cu4[j]);
          bad |= lo[j] > up[j];
        }
      }
    }
    if (g.split) {
      const int8_t* sp = g.split + (size_t)row * g.split_stride;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (col + j < g.N) {
          const int s = sp[col + j];
          if (s > 0) lo[j] = fmaxf(lo[j], 0.f);
          if (s < 0) up[j] = fminf(up[j], 0.f);
          bad |= lo[j] > up[j];
        }
      }
    }
    store4_guard(g.out_l + (size_t)row * g.N, col, g.N, vN, make_float4(lo[0], lo[1], lo[2], lo[3]));
    store4_guard(g.out_u + (size_t)row * g.N, col, g.N, vN, make_float4(up[0], up[1], up[2], up[3]));
    if (bad && g.infeasible) g.infeasible[row] = 1;
  }
}

int launch_ibp_linear(const float* in_a, const float* in_b, int in_mode, int relu_in, const float* W, const float* bias,
                      const int8_t* split, int split_stride, const float* cons_l, const float* cons_u, float* out_l,
                      float* out_u, int* infeasible, int B, int K, int N, const float* row_dev, cudaStream_t stream) {
  IbpArgs g{in_a, in_b, in_mode, relu_in, W, bias, split, split_stride, cons_l, cons_u, out_l, out_u, infeasible, B, K, N, 0, 0, row_dev};
  g.vecK = (K % 4 == 0);
  const void* kptrs[] = {in_a, in_b, W};
  for (const void* p : kptrs) if (p && (reinterpret_cast<uintptr_t>(p) & 15u)) g.vecK = 0;
  g.vecN = (N % 4 == 0);
  const void* nptrs[] = {bias, cons_l, cons_u, out_l, out_u, row_dev};
  for (const void* p : nptrs) if (p && (reinterpret_cast<uintptr_t>(p) & 15u)) g.vecN = 0;
  dim3 grid(ceil_div(B, IBM), ceil_div(N, IBN));
  timing_begin(T_IBP_LINEAR, stream);
  ibp_linear_kernel<<<grid, 256, 0, stream>>>(g);
  // weights and bias once, the input interval once, both output bounds once (+ the split bytes)
  timing_end(T_IBP_LINEAR, stream, 4.0 * ((double)K * N + N) + 8.0 * (double)B * (K + N) + (split ? (double)B * N : 0.0),
             4.0 * (double)B * K * N);
  BF_CHECK_LAUNCH("ibp_linear_kernel");
  return BF_OK;
}

}  // namespace bf

extern "C" int bf_ibp_linear(const float* in_a, const float* in_b, int in_mode, int relu_in, const float* W,
                             const float* bias, const int8_t* split, int split_stride, const float* cons_l,
                             const float* cons_u, float* out_l, float* out_u, int* infeasible, int B, int n_in,
                             int n_out, bf_stream_t stream) {
  BF_REQUIRE(in_a && in_b && W && out_l && out_u, BF_E_INVALID, "bf_ibp_linear: null tensor");
  BF_REQUIRE(B > 0 && n_in > 0 && n_out > 0, BF_E_INVALID, "bf_ibp_linear: sizes must be positive");
  BF_REQUIRE(in_mode == BF_IN_LOWER_UPPER || in_mode == BF_IN_MID_RAD, BF_E_INVALID, "bf_ibp_linear: bad in_mode");
  BF_REQUIRE(!(relu_in && in_mode == BF_IN_MID_RAD), BF_E_INVALID, "bf_ibp_linear: relu_in needs lower/upper inputs");
  BF_REQUIRE((cons_l == nullptr) == (cons_u == nullptr), BF_E_INVALID, "bf_ibp_linear: give both constraint tensors or none");
  BF_REQUIRE(!split || split_stride == 0 || split_stride == n_out, BF_E_INVALID, "bf_ibp_linear: split_stride must be 0 or n_out");
  return bf::launch_ibp_linear(in_a, in_b, in_mode, relu_in, W, bias, split, split_stride, cons_l, cons_u, out_l, out_u,
                               infeasible, B, n_in, n_out, nullptr, bf::as_stream(stream));
}

// ---------------------------------------------------------------------------
// Lp-ball (p = 1, 2, inf) support: dual-norm row reductions
// ---------------------------------------------------------------------------
namespace bf {

// out[r] = scale * ||rows[r, :]||_q with q the dual of p: p=inf -> sum |x|, p=2 -> sqrt(sum x^2), p=1 -> max |x|.
// One warp per row.
__global__ void __launch_bounds__(256) row_dual_norm_kernel(const float* __restrict__ rows, int n_rows, int n, int p, float scale,
                                                            float* __restrict__ out) {
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  float acc = 0.f;
  for (int k = lane; k < n; k += 32) {
    const float x = rows[(size_t)r * n + k];
    if (p == 2) acc = fmaf(x, x, acc);
    else if (p == 1) acc = fmaxf(acc, fabsf(x));
    else acc += fabsf(x);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = (p == 1) ? fmaxf(acc, other) : (acc + other);
  }
  if (lane == 0) out[r] = scale * ((p == 2) ? sqrtf(acc) : acc);
}

int launch_row_dual_norm(const float* rows, int n_rows, int n, int p, float scale, float* out, cudaStream_t stream) {
  row_dual_norm_kernel<<<ceil_div((long long)n_rows * 32, 256), 256, 0, stream>>>(rows, n_rows, n, p, scale, out);
  BF_CHECK_LAUNCH("row_dual_norm_kernel");
  return BF_OK;
}

// out[m] = A[m,:].center[d,:] -/+ eps * ||A[m,:]||_q + bias_in[m]
__global__ void __launch_bounds__(256) concretize_lp_kernel(const float* __restrict__ A, const float* __restrict__ center,
                                                            const float* __restrict__ bias_in, float* __restrict__ out, float sgn,
                                                            float eps, int p, int M, int S, int n0) {
  const int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (m >= M) return;
  const float* a = A + (size_t)m * n0;
  const float* c = center + (size_t)(m / S) * n0;
  float dot = 0.f, acc = 0.f;
  for (int k = lane; k < n0; k += 32) {
    const float x = a[k];
    dot = fmaf(x, c[k], dot);
    if (p == 2) acc = fmaf(x, x, acc);
    else if (p == 1) acc = fmaxf(acc, fabsf(x));
    else acc += fabsf(x);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float other = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = (p == 1) ? fmaxf(acc, other) : (acc + other);
  }
  if (lane == 0) out[m] = dot + sgn * eps * ((p == 2) ? sqrtf(acc) : acc) + (bias_in ? bias_in[m] : 0.f);
}

int launch_concretize_lp(const float* A, const float* center, const float* bias_in, float* out, int side, float eps, int p, int B,
                         int S, int n0, cudaStream_t stream) {
  const int M = B * S;
  concretize_lp_kernel<<<ceil_div((long long)M * 32, 256), 256, 0, stream>>>(A, center, bias_in, out, side == BF_SIDE_LOWER ? -1.f : 1.f,
                                                                           eps, p, M, S, n0);
  BF_CHECK_LAUNCH("concretize_lp_kernel");
  return BF_OK;
}

// Derivative of the Lp-ball lower bound  A.center - eps * ||A||_q  with respect to the coefficient row,
// written over the row itself:  H[m,k] = center[d,k] - eps * d||A[m,:]||_q / dA[m,k]
//   q = 2: A_k / ||A||_2 (0 for a zero row);  q = inf (p = 1): sign(A_k) / #maxima at the maxima of |A|, else 0;
//   q = 1 (p = inf): sign(A_k).   This is the start vector of the adjoint (gradient) sweep.
__global__ void __launch_bounds__(256) h0_lp_kernel(float* __restrict__ A, const float* __restrict__ center, float eps, int p, int M,
                                                    int S, int n0) {
  const int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (m >= M) return;
  float* a = A + (size_t)m * n0;
  const float* c = center + (size_t)(m / S) * n0;
  float acc = 0.f;
  for (int k = lane; k < n0; k += 32) {
    const float x = a[k];
    if (p == 2) acc = fmaf(x, x, acc);
    else if (p == 1) acc = fmaxf(acc, fabsf(x));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = (p == 1) ? fmaxf(acc, other) : (acc + other);
  }
  float cnt = 0.f;
  if (p == 1) {
    for (int k = lane; k < n0; k += 32) cnt += (fabsf(a[k]) == acc) ? 1.f : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  }
  const float nrm = (p == 2) ? sqrtf(acc) : acc;
  for (int k = lane; k < n0; k += 32) {
    const float x = a[k];
    const float sg = (x > 0.f) ? 1.f : ((x < 0.f) ? -1.f : 0.f);
    float g;
    if (p == 2) g = (nrm > 0.f) ? x / nrm : 0.f;
    else if (p == 1) g = (fabsf(x) == nrm && nrm > 0.f) ? sg / cnt : 0.f;
    else g = sg;
    a[k] = c[k] - eps * g;
  }
}

int launch_h0_lp(float* A, const float* center, float eps, int p, int B, int S, int n0, cudaStream_t stream) {
  const int M = B * S;
  h0_lp_kernel<<<ceil_div((long long)M * 32, 256), 256, 0, stream>>>(A, center, eps, p, M, S, n0);
  BF_CHECK_LAUNCH("h0_lp_kernel");
  return BF_OK;
}

}  // namespace bf

static bool lp_ok(int p) { return p == BF_NORM_INF || p == BF_NORM_L2 || p == BF_NORM_L1; }

extern "C" int bf_row_dual_norms(const float* W, int n_rows, int n_cols, int p, float scale, float* out, bf_stream_t stream) {
  BF_REQUIRE(W && out && n_rows > 0 && n_cols > 0, BF_E_INVALID, "bf_row_dual_norms: bad argument");
  BF_REQUIRE(lp_ok(p), BF_E_INVALID, "bf_row_dual_norms: p must be BF_NORM_INF, BF_NORM_L2 or BF_NORM_L1");
  return bf::launch_row_dual_norm(W, n_rows, n_cols, p, scale, out, bf::as_stream(stream));
}

extern "C" int bf_ibp_linear_lp(const float* center, const float* row_dev, const float* W, const float* bias, const int8_t* split,
                                int split_stride, const float* cons_l, const float* cons_u, float* out_l, float* out_u,
                                int* infeasible, int B, int n_in, int n_out, bf_stream_t stream) {
  BF_REQUIRE(center && row_dev && W && out_l && out_u, BF_E_INVALID, "bf_ibp_linear_lp: null tensor");
  BF_REQUIRE(B > 0 && n_in > 0 && n_out > 0, BF_E_INVALID, "bf_ibp_linear_lp: sizes must be positive");
  BF_REQUIRE((cons_l == nullptr) == (cons_u == nullptr), BF_E_INVALID, "bf_ibp_linear_lp: give both constraint tensors or none");
  return bf::launch_ibp_linear(center, nullptr, BF_IN_MID_RAD, 0, W, bias, split, split_stride, cons_l, cons_u, out_l, out_u,
                               infeasible, B, n_in, n_out, row_dev, bf::as_stream(stream));
}

// ---------------------------------------------------------------------------
// IBP linear layer whose weight differs per batch element (the output spec merged into the last
// layer: W' = C @ W, b' = C @ b): one warp per (batch element, output row), midpoint/radius form.
// HBM-bound: every weight is read once.
// ---------------------------------------------------------------------------
namespace bf {
__global__ void __launch_bounds__(256) ibp_linear_batched_kernel(const float* __restrict__ in_l, const float* __restrict__ in_u,
                                                                 int relu_in, const float* __restrict__ W,
                                                                 const float* __restrict__ bias, float* __restrict__ out_l,
                                                                 float* __restrict__ out_u, int B, int S, int n_in) {
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= (long long)B * S) return;
  const int b = (int)(row / S);
  const float* w = W + (size_t)row * n_in;
  const float* xl = in_l + (size_t)b * n_in;
  const float* xu = in_u + (size_t)b * n_in;
  float c = 0.f, d = 0.f;
  for (int i = lane; i < n_in; i += 32) {
    float lo = xl[i], up = xu[i];
    if (relu_in) { lo = fmaxf(lo, 0.f); up = fmaxf(up, 0.f); }
    const float wv = w[i];
    c = fmaf(0.5f * (lo + up), wv, c);
    d = fmaf(0.5f * (up - lo), fabsf(wv), d);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    c += __shfl_xor_sync(0xffffffffu, c, o);
    d += __shfl_xor_sync(0xffffffffu, d, o);
  }
  if (lane == 0) {
    const float bb = bias ? bias[row] : 0.f;
    out_l[row] = c - d + bb;
    out_u[row] = c + d + bb;
  }
}
}  // namespace bf

extern "C" int bf_ibp_linear_batched(const float* in_l, const float* in_u, int relu_in, const float* W, const float* bias,
                                     float* out_l, float* out_u, int B, int S, int n_in, bf_stream_t stream) {
  BF_REQUIRE(in_l && in_u && W && out_l && out_u, BF_E_INVALID, "bf_ibp_linear_batched: null tensor");
  BF_REQUIRE(B > 0 && S > 0 && n_in > 0 && (long long)B * S < 2147483647LL, BF_E_INVALID, "bf_ibp_linear_batched: bad sizes");
  const long long warps = (long long)B * S;
  bf::ibp_linear_batched_kernel<<<(int)((warps + 7) / 8), 256, 0, bf::as_stream(stream)>>>(in_l, in_u, relu_in, W, bias, out_l, out_u,
                                                                                          B, S, n_in);
  BF_CHECK_LAUNCH("ibp_linear_batched_kernel");
  return BF_OK;
}

extern "C" int bf_concretize_lp(const float* A, const float* center, float eps, int p, const float* bias_in, float* out, int side,
                                int B, int S, int n0, bf_stream_t stream) {
  BF_REQUIRE(A && center && out, BF_E_INVALID, "bf_concretize_lp: null tensor");
  BF_REQUIRE(B > 0 && S > 0 && n0 > 0 && (long long)B * S < 2147483647LL, BF_E_INVALID, "bf_concretize_lp: bad sizes");
  BF_REQUIRE(lp_ok(p) && eps >= 0.f, BF_E_INVALID, "bf_concretize_lp: bad norm or eps");
  BF_REQUIRE(side == BF_SIDE_LOWER || side == BF_SIDE_UPPER, BF_E_INVALID, "bf_concretize_lp: bad side");
  return bf::launch_concretize_lp(A, center, bias_in, out, side, eps, p, B, S, n0, bf::as_stream(stream));
}
