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
};

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
      float4 b = load4_guard(g.in_b + (size_t)m * g.K, k, g.K, vK);
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
                      float* out_u, int* infeasible, int B, int K, int N, cudaStream_t stream) {
  IbpArgs g{in_a, in_b, in_mode, relu_in, W, bias, split, split_stride, cons_l, cons_u, out_l, out_u, infeasible, B, K, N, 0, 0};
  g.vecK = (K % 4 == 0);
  const void* kptrs[] = {in_a, in_b, W};
  for (const void* p : kptrs) if (p && (reinterpret_cast<uintptr_t>(p) & 15u)) g.vecK = 0;
  g.vecN = (N % 4 == 0);
  const void* nptrs[] = {bias, cons_l, cons_u, out_l, out_u};
  for (const void* p : nptrs) if (p && (reinterpret_cast<uintptr_t>(p) & 15u)) g.vecN = 0;
  dim3 grid(ceil_div(B, IBM), ceil_div(N, IBN));
  ibp_linear_kernel<<<grid, 256, 0, stream>>>(g);
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
                               infeasible, B, n_in, n_out, bf::as_stream(stream));
}
