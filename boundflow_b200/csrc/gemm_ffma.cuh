// FP32 (FFMA) tiled contraction shared by the CROWN backward sweep and the
// adjoint (gradient) sweep.  One CTA computes a 128x128 tile of
//   C[M,N] = f(A)[M,K] * B[K,N]
// with a 16-deep k-slab double-buffered through shared memory; every thread owns
// an 8x8 micro-tile (two 4-row groups x two 4-column groups).  The template parameters
// MH / NH (1 or 2) give the number of 64-row / 64-column halves a CTA computes: 64x64,
// 64x128 or 128x64 tiles (4x4 ... 4x8 micro-tiles, same thread mapping, the unused half
// simply absent) put four times as many CTAs on problems whose 128x128 tiles would leave
// most SMs idle; MH == 0 stands for 32 rows (2x4 micro-tiles, 32x64 tiles) for problems that
// still do not give every SM a CTA.  `f` is the
// per-element prologue applied while the A slab moves global -> shared:
//   PRO_PLAIN : identity                    (top linear layer, adjoint hidden layers)
//   PRO_RELU  : ReLU backward transformer   (sign-select slope, intercept and bias row sums)
//   PRO_H0    : mid - sign(a)*rad           (adjoint point at the network input)
// B is either [K,N] row-major (backward sweep: A' = Lambda * W) or [N,K]
// row-major (adjoint sweep: g = h * W^T).
#pragma once
#include "common.cuh"

namespace bf {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 16;
constexpr int GEMM_THREADS = 256;
constexpr int LDS = BM + 4;  // padded leading dimension of both shared slabs
constexpr int SLAB = BK * LDS;
constexpr int MAINLOOP_SMEM_FLOATS = 4 * SLAB;  // 2 stages x (A slab + B slab)

enum { PRO_PLAIN = 0, PRO_RELU = 1, PRO_H0 = 2 };

struct GemmArgs {
  const float* A;   // [M,K]
  const float* Bm;  // [K,N] (B_NT == false) or [N,K] (B_NT == true)
  int M, N, K;
  int S;            // coefficient rows per domain: domain(m) = m / S
  int vecK, vecN;   // 1 when 128-bit accesses along K / N are legal for every operand
  // PRO_RELU (all [D,K]; dpos == nullptr means "no ReLU": lam = a)
  const float* dpos;   // slope applied where a >= 0
  const float* dneg;   // slope applied where a <  0
  const float* epos;   // intercept where a >= 0 (nullable = 0)
  const float* eneg;   // intercept where a <  0 (nullable = 0)
  const float* add;    // added to the scaled coefficient (nullable)
  const float* kbias;  // [K] bias of the affine layer being transposed (nullable)
  // PRO_H0 ([D,K])
  const float* mid;
  const float* rad;
  // row sums of the prologue: delta[m] (+)= sum_k a*e_sel + lam*kbias
  float* delta;
  int accumulate;
};

__device__ __forceinline__ float sgnf(float a) { return (a > 0.f) ? 1.f : ((a < 0.f) ? -1.f : 0.f); }

template <int PRO, bool B_NT, int MH = 2, int NH = 2>
__device__ __forceinline__ void gemm_mainloop(const GemmArgs& g, const int m0, const int n0, float (&acc)[8][8],
                                              float* __restrict__ smem) {
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int lrow = tid >> 2;       // rows lrow and lrow + 64 of the slab
  const int lkc = (tid & 3) * 4;   // k offset of this thread's float4 inside the slab
  const int bkr = tid >> 5;        // B_NN: k rows bkr and bkr + 8
  const int bnc = (tid & 31) * 4;  // B_NN: column offset
  const bool vK = g.vecK != 0, vN = g.vecN != 0;
  float* As = smem;
  float* Bs = smem + 2 * SLAB;

#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  constexpr int LROWS = (MH == 0) ? 1 : MH;   // tile rows a loader thread owns (rows lrow, lrow + 64)
  constexpr int MR = (MH == 0) ? 2 : 4 * MH;  // micro-tile rows of a thread
  const bool a_loader = (MH != 0) || lrow < 32;  // 32-row tiles: half of the threads load coefficient rows
  float rowacc[2] = {0.f, 0.f};
  int dom[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < LROWS; ++i) {
    int m = m0 + lrow + i * 64;
    dom[i] = (m < g.M) ? (m / g.S) : 0;
  }

  float4 areg[2], breg[2];
  // Small tiles (MH == 1) run with one CTA of 8 warps on an SM, so nothing hides a load's latency: there the slab that is
  // loaded while the current one is multiplied stays RAW in registers (coefficients and the slope / intercept vectors of
  // the row's domain) and the prologue is applied right before the slab goes to shared memory, after the multiply loop.
  // The large tiles (several CTAs per SM, 128 registers in use) apply the prologue at load time as before.
  constexpr bool DEFER = (MH <= 1);
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 kbr = z4, dpr[LROWS], dnr[LROWS], epr[LROWS], enr[LROWS], adr[LROWS];  // PRO_H0 keeps mid / rad in dpr / dnr
  bool live[LROWS];

  // the per-element prologue of row slot i; same operations in the same order wherever it runs
  auto prologue = [&](int i, float4 a, const float4& kb, const float4& dp, const float4& dn, const float4& ep, const float4& en,
                      const float4& ad) -> float4 {
    if (PRO == PRO_RELU) {
      if (g.dpos) {
        float r = rowacc[i];
#define BF_RELU_SEL(c)                                   \
  {                                                      \
    const bool sel = a.c >= 0.f;                         \
    const float lam = a.c * (sel ? dp.c : dn.c) + ad.c;  \
    r += a.c * (sel ? ep.c : en.c);                      \
    r = fmaf(lam, kb.c, r);                              \
    a.c = lam;                                           \
  }
        BF_RELU_SEL(x) BF_RELU_SEL(y) BF_RELU_SEL(z) BF_RELU_SEL(w)
#undef BF_RELU_SEL
        rowacc[i] = r;
      } else {
        rowacc[i] += a.x * kb.x + a.y * kb.y + a.z * kb.z + a.w * kb.w;
      }
    } else if (PRO == PRO_H0) {
      a.x = dp.x - sgnf(a.x) * dn.x;
      a.y = dp.y - sgnf(a.y) * dn.y;
      a.z = dp.z - sgnf(a.z) * dn.z;
      a.w = dp.w - sgnf(a.w) * dn.w;
    }
    return a;
  };

  auto load_slab = [&](int kt) {
    const int k = kt * BK + lkc;
#pragma unroll
    for (int i = 0; i < LROWS; ++i) {
      const int m = m0 + lrow + i * 64;
      const bool ok = a_loader && m < g.M && k < g.K;
      float4 a = z4, kb = z4, dp = z4, dn = z4, ep = z4, en = z4, ad = z4;
      if (ok) {
        a = load4_guard(g.A + (size_t)m * g.K, k, g.K, vK);
        const size_t off = (size_t)dom[i] * g.K;
        if (PRO == PRO_RELU) {
          if (g.kbias) kb = load4_guard(g.kbias, k, g.K, vK);
          if (g.dpos) {
            dp = load4_guard(g.dpos + off, k, g.K, vK);
            dn = load4_guard(g.dneg + off, k, g.K, vK);
            if (g.epos) ep = load4_guard(g.epos + off, k, g.K, vK);
            if (g.eneg) en = load4_guard(g.eneg + off, k, g.K, vK);
            if (g.add) ad = load4_guard(g.add + off, k, g.K, vK);
          }
        } else if (PRO == PRO_H0) {
          dp = load4_guard(g.mid + off, k, g.K, vK);
          dn = load4_guard(g.rad + off, k, g.K, vK);
        }
      }
      if (DEFER) {
        areg[i] = a; kbr = kb; dpr[i] = dp; dnr[i] = dn; epr[i] = ep; enr[i] = en; adr[i] = ad; live[i] = ok;
      } else {
        areg[i] = ok ? prologue(i, a, kb, dp, dn, ep, en, ad) : a;
      }
    }
    if (B_NT) {
#pragma unroll
      for (int i = 0; i < NH; ++i) {
        const int n = n0 + lrow + i * 64;
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n < g.N && k < g.K) b = load4_guard(g.Bm + (size_t)n * g.K, k, g.K, vK);
        breg[i] = b;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int kk = kt * BK + bkr + i * 8;
        const int n = n0 + bnc;
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (kk < g.K && n < g.N && bnc < 64 * NH) b = load4_guard(g.Bm + (size_t)kk * g.N, n, g.N, vN);
        breg[i] = b;
      }
    }
  };

  // applies the deferred prologue to the slab held in registers (small tiles)
  auto finish_slab = [&]() {
    if (DEFER) {
#pragma unroll
      for (int i = 0; i < LROWS; ++i)
        if (live[i]) areg[i] = prologue(i, areg[i], kbr, dpr[i], dnr[i], epr[i], enr[i], adr[i]);
    }
  };

  auto store_slab = [&](int stage) {
    float* as = As + stage * SLAB;
    float* bs = Bs + stage * SLAB;
#pragma unroll
    for (int i = 0; i < LROWS; ++i) {
      const int r = lrow + i * 64;
      if (!a_loader) continue;
      as[(lkc + 0) * LDS + r] = areg[i].x;
      as[(lkc + 1) * LDS + r] = areg[i].y;
      as[(lkc + 2) * LDS + r] = areg[i].z;
      as[(lkc + 3) * LDS + r] = areg[i].w;
    }
    if (B_NT) {
#pragma unroll
      for (int i = 0; i < NH; ++i) {
        const int r = lrow + i * 64;
        bs[(lkc + 0) * LDS + r] = breg[i].x;
        bs[(lkc + 1) * LDS + r] = breg[i].y;
        bs[(lkc + 2) * LDS + r] = breg[i].z;
        bs[(lkc + 3) * LDS + r] = breg[i].w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 2; ++i) *reinterpret_cast<float4*>(&bs[(bkr + i * 8) * LDS + bnc]) = breg[i];
    }
  };

  const int nk = (g.K + BK - 1) / BK;
  load_slab(0);
  finish_slab();
  store_slab(0);
  __syncthreads();
  for (int kt = 0; kt < nk; ++kt) {
    const int stage = kt & 1;
    if (kt + 1 < nk) load_slab(kt + 1);
    const float* as = As + stage * SLAB;
    const float* bs = Bs + stage * SLAB;
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float4 a0;
      if (MH == 0) {
        const float2 a2 = *reinterpret_cast<const float2*>(&as[kk * LDS + ty * 2]);
        a0 = make_float4(a2.x, a2.y, 0.f, 0.f);
      } else {
        a0 = *reinterpret_cast<const float4*>(&as[kk * LDS + ty * 4]);
      }
      const float4 b0 = *reinterpret_cast<const float4*>(&bs[kk * LDS + tx * 4]);
      float4 a1 = a0, b1 = b0;
      if (MH == 2) a1 = *reinterpret_cast<const float4*>(&as[kk * LDS + 64 + ty * 4]);
      if (NH == 2) b1 = *reinterpret_cast<const float4*>(&bs[kk * LDS + 64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < MR; ++i)
#pragma unroll
        for (int j = 0; j < 4 * NH; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kt + 1 < nk) {
      finish_slab();
      store_slab(stage ^ 1);
    }
    __syncthreads();
  }

  // Row sums of the prologue: the 4 threads that loaded one row are adjacent lanes.
  if (PRO == PRO_RELU) {
#pragma unroll
    for (int i = 0; i < LROWS; ++i) {
      float v = rowacc[i];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      const int m = m0 + lrow + i * 64;
      if (g.delta != nullptr && blockIdx.y == 0 && (tid & 3) == 0 && a_loader && m < g.M) {
        g.delta[m] = g.accumulate ? (g.delta[m] + v) : v;
      }
    }
  }
}

// Row / column of micro-tile element (i, j) inside the CTA tile (MH == 0: 32-row tiles, two rows per thread).
template <int MH = 2>
__device__ __forceinline__ int tile_row(int ty, int i) {
  if (MH == 0) return ty * 2 + i;
  return (i < 4) ? (ty * 4 + i) : (64 + ty * 4 + (i - 4));
}
__device__ __forceinline__ int tile_col(int tx, int jb) { return jb * 64 + tx * 4; }

}  // namespace bf
