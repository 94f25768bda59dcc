// CROWN backward sweep through Linear layers (fused with the ReLU backward
// transformer and, on the first layer, with the concretisation) and the adjoint
// (alpha-gradient) sweep, as FP32 FFMA tiles.
#include "gemm_ffma.cuh"
#include <stdlib.h>

#include "kernels.cuh"

namespace bf {

// ---------------------------------------------------------------------------
// Backward: A_prev[M,N] = relu_bwd(A)[M,K] * W[K,N]
// ---------------------------------------------------------------------------
struct BwdEpilogue {
  float* out;            // [M,N] or nullptr
  const float* mid;      // [D,N] (only with `partial`)
  const float* rad;      // [D,N]
  float* partial;        // [M, gridDim.y] concretisation partial sums or nullptr
  int side;              // BF_SIDE_LOWER: a*mid - |a|*rad ; BF_SIDE_UPPER: a*mid + |a|*rad
};

template <int PRO, int MH, int NH>
__global__ void __launch_bounds__(GEMM_THREADS, 2) crown_bwd_linear_kernel(GemmArgs g, BwdEpilogue e) {
  __shared__ __align__(16) float smem[MAINLOOP_SMEM_FLOATS];
  constexpr int TM = (MH == 0) ? 32 : 64 * MH, MR = (MH == 0) ? 2 : 4 * MH;
  const int m0 = blockIdx.x * TM, n0 = blockIdx.y * (64 * NH);
  float acc[8][8];
  gemm_mainloop<PRO, false, MH, NH>(g, m0, n0, acc, smem);

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const bool vN = g.vecN != 0;
  const float sgn = (e.side == BF_SIDE_LOWER) ? -1.f : 1.f;
#pragma unroll
  for (int i = 0; i < MR; ++i) {
    const int row = m0 + tile_row<MH>(ty, i);
    const bool row_ok = row < g.M;
    float p = 0.f;
#pragma unroll
    for (int jb = 0; jb < NH; ++jb) {
      const int col = n0 + tile_col(tx, jb);
      const float4 v = make_float4(acc[i][jb * 4 + 0], acc[i][jb * 4 + 1], acc[i][jb * 4 + 2], acc[i][jb * 4 + 3]);
      if (row_ok && col < g.N) {
        if (e.out) store4_guard(e.out + (size_t)row * g.N, col, g.N, vN, v);
        if (e.partial) {
          const size_t off = (size_t)(row / g.S) * g.N;
          const float4 md = load4_guard(e.mid + off, col, g.N, vN);
          const float4 rd = load4_guard(e.rad + off, col, g.N, vN);
          p += v.x * md.x + sgn * fabsf(v.x) * rd.x;
          p += v.y * md.y + sgn * fabsf(v.y) * rd.y;
          p += v.z * md.z + sgn * fabsf(v.z) * rd.z;
          p += v.w * md.w + sgn * fabsf(v.w) * rd.w;
        }
      }
    }
    if (e.partial) {  // uniform across the CTA
      p += __shfl_xor_sync(0xffffffffu, p, 1);
      p += __shfl_xor_sync(0xffffffffu, p, 2);
      p += __shfl_xor_sync(0xffffffffu, p, 4);
      p += __shfl_xor_sync(0xffffffffu, p, 8);
      if (tx == 0 && row_ok) e.partial[(size_t)row * gridDim.y + blockIdx.y] = p;
    }
  }
}

// Top layer of a sweep (no ReLU in front, K = spec width <= 16): A_prev[M,N] = A[M,K] * W[K,N] and
// delta[m] (+)= sum_k A[m,k] * kbias[k].  A store-bound pass, so no tiles: a thread keeps its four
// columns of W in registers and walks the block's rows, whose K values sit in shared memory.
constexpr int THIN_KMAX = 16;
constexpr int THIN_ROWS = 64;
__global__ void __launch_bounds__(128) crown_bwd_thin_kernel(const float* __restrict__ A, const float* __restrict__ W,
                                                             const float* __restrict__ kbias, float* __restrict__ out,
                                                             float* __restrict__ delta, int accumulate, int M, int K, int N) {
  __shared__ float a_s[THIN_ROWS * THIN_KMAX];
  const int m0 = blockIdx.x * THIN_ROWS;
  const int rows = min(THIN_ROWS, M - m0);
  for (int i = threadIdx.x; i < rows * K; i += blockDim.x) a_s[i] = A[(size_t)m0 * K + i];
  __syncthreads();
  const int cg = blockIdx.y * blockDim.x + threadIdx.x;  // group of four columns
  if (cg * 4 < N) {
    float4 w[THIN_KMAX];
#pragma unroll
    for (int k = 0; k < THIN_KMAX; ++k)
      w[k] = (k < K) ? *reinterpret_cast<const float4*>(W + (size_t)k * N + cg * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < rows; ++r) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k = 0; k < THIN_KMAX; ++k) {
        if (k < K) {
          const float a = a_s[r * K + k];
          acc.x = fmaf(a, w[k].x, acc.x); acc.y = fmaf(a, w[k].y, acc.y);
          acc.z = fmaf(a, w[k].z, acc.z); acc.w = fmaf(a, w[k].w, acc.w);
        }
      }
      *reinterpret_cast<float4*>(out + (size_t)(m0 + r) * N + cg * 4) = acc;
    }
  }
  if (delta && blockIdx.y == 0) {
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
      float sum = 0.f;
      if (kbias)
        for (int k = 0; k < K; ++k) sum = fmaf(a_s[r * K + k], __ldg(kbias + k), sum);
      delta[m0 + r] = accumulate ? delta[m0 + r] + sum : sum;
    }
  }
}

// 128 x 128 tiles leave most of the 148 SMs idle on small problems: below one CTA per SM the kernels switch to 64 x 64 tiles
bool ffma_small_tiles(int M, int N) { return (long long)ceil_div(M, BM) * ceil_div(N, BN) < 148; }
// ... and 32 x 64 tiles when even the 64 x 64 tiles give fewer CTAs than SMs
static bool ffma_quarter_tiles(int M, int N) { return ffma_small_tiles(M, N) && M > 32 && (long long)ceil_div(M, 64) * ceil_div(N, 64) < 148; }

// Measured on B200 (c3: 1152 x 256 x 256 layers, 20 Adam steps): 8.9 ms on these tiles against 9.7 ms on the tcgen05
// kernels, whose per-launch time of 23-36 us is a serial k-loop on 9-36 CTAs; at 144 rows 6.3 against 7.3 ms.  Beyond one
// wave the tensor-core kernels win.
bool ffma_fits_one_wave(int M, int N) { return (long long)ceil_div(M, 64) * ceil_div(N, 64) <= 2 * 148; }

int launch_crown_bwd_linear(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                            const float* add, const float* W, const float* kbias, float* A_prev, float* delta,
                            int accumulate, const float* mid, const float* rad, float* partial, int side, int M, int S,
                            int K, int N, cudaStream_t stream) {
  if (!dpos && !add && !partial && A_prev && K <= THIN_KMAX && N % 4 == 0 &&
      ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(A_prev)) & 15u) == 0) {
    dim3 grid(ceil_div(M, THIN_ROWS), ceil_div(N / 4, 128));
    timing_begin(T_THIN, stream);
    crown_bwd_thin_kernel<<<grid, 128, 0, stream>>>(A, W, kbias, A_prev, delta, accumulate, M, K, N);
    timing_end(T_THIN, stream, 4.0 * (double)M * N + 4.0 * (double)M * K + 4.0 * (double)K * N, 2.0 * (double)M * K * N);
    BF_CHECK_LAUNCH("crown_bwd_thin_kernel");
    return BF_OK;
  }
  GemmArgs g{};
  g.A = A; g.Bm = W; g.M = M; g.N = N; g.K = K; g.S = S;
  const void* kptrs[] = {A, dpos, dneg, epos, eneg, add, kbias};
  g.vecK = (K % 4 == 0);
  for (const void* p : kptrs) if (p && (reinterpret_cast<uintptr_t>(p) & 15u)) g.vecK = 0;
  const void* nptrs[] = {W, A_prev, mid, rad};
  g.vecN = (N % 4 == 0);
  for (const void* p : nptrs) if (p && (reinterpret_cast<uintptr_t>(p) & 15u)) g.vecN = 0;
  g.dpos = dpos; g.dneg = dneg; g.epos = epos; g.eneg = eneg; g.add = add; g.kbias = kbias;
  g.delta = delta; g.accumulate = accumulate;
  BwdEpilogue e{A_prev, mid, rad, partial, side};
  timing_begin(T_BWD, stream);
  if (ffma_quarter_tiles(M, N)) {  // 32 x 64 tiles
    dim3 grid(ceil_div(M, 32), ceil_div(N, 64));
    crown_bwd_linear_kernel<PRO_RELU, 0, 1><<<grid, GEMM_THREADS, 0, stream>>>(g, e);
  } else if (ffma_small_tiles(M, N)) {  // 64 x 64 tiles: four times as many CTAs
    dim3 grid(ceil_div(M, 64), ceil_div(N, 64));
    crown_bwd_linear_kernel<PRO_RELU, 1, 1><<<grid, GEMM_THREADS, 0, stream>>>(g, e);
  } else {
    dim3 grid(ceil_div(M, BM), ceil_div(N, BN));
    crown_bwd_linear_kernel<PRO_RELU, 2, 2><<<grid, GEMM_THREADS, 0, stream>>>(g, e);
  }
  timing_end(T_BWD, stream, 4.0 * (double)M * K + (A_prev ? 4.0 * (double)M * N : 0.0), 2.0 * (double)M * K * N);
  BF_CHECK_LAUNCH("crown_bwd_linear_kernel");
  return BF_OK;
}

// column tiles (= concretisation partial sums per row) of the backward kernel for this problem; M <= 0: the largest count
int crown_bwd_partial_tiles(int N, int M) { return (M <= 0 || ffma_small_tiles(M, N)) ? ceil_div(N, 64) : ceil_div(N, BN); }

// ---------------------------------------------------------------------------
// Adjoint (gradient) sweep: g[M,N] = h_prev[M,K] * W[N,K]^T + b[N]
// epilogue: h = d_sel*g + e_sel ; grad[d,n] += sum_s [amb][A>=0] * A * g
// ---------------------------------------------------------------------------
struct AdjEpilogue {
  const float* nbias;  // [N] bias of this layer (nullable)
  const float* Ahat;   // [M,N] coefficients w.r.t. this layer's ReLU output, saved by the backward sweep
  const float* dpos;   // [D,N]
  const float* dneg;   // [D,N]
  const float* epos;   // [D,N] nullable
  const float* eneg;   // [D,N] nullable
  const float* pre_l;  // [D,N]
  const float* pre_u;  // [D,N]
  float* hout;         // [M,N] or nullptr (last ReLU layer needs no adjoint point)
  float* grad;         // [D,N], accumulated with atomicAdd (at most two row tiles touch one entry when S <= the tile height: 32, 64 or 128)
  float* gsum;         // [D,N] or nullptr: sum over the domain's rows of g (beta gradient), same accumulation
  const float* gw;     // [M] or nullptr: weight of each row in gsum (d objective / d row for min / softmin)
};

constexpr int STAGE_LD = BN + 1;
constexpr int ADJ_SMEM_BYTES = BM * STAGE_LD * (int)sizeof(float);
static_assert(ADJ_SMEM_BYTES >= MAINLOOP_SMEM_FLOATS * (int)sizeof(float), "stage buffer must cover the main loop slabs");

template <int PRO, int MH, int NH>
__global__ void __launch_bounds__(GEMM_THREADS, 2) crown_adjoint_linear_kernel(GemmArgs g, AdjEpilogue e) {
  extern __shared__ __align__(16) float dsmem[];
  constexpr int TM = (MH == 0) ? 32 : 64 * MH, TN = 64 * NH, MR = (MH == 0) ? 2 : 4 * MH;
  const int m0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
  float acc[8][8];
  gemm_mainloop<PRO, true, MH, NH>(g, m0, n0, acc, dsmem);
  // the main loop ends with __syncthreads(): the slabs may now be overwritten by the stage tile

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const bool vN = g.vecN != 0;
#pragma unroll
  for (int i = 0; i < MR; ++i) {
    const int rl = tile_row<MH>(ty, i);
    const int row = m0 + rl;
#pragma unroll
    for (int jb = 0; jb < NH; ++jb) {
      const int cl = tile_col(tx, jb);
      const int col = n0 + cl;
      float c4[4] = {0.f, 0.f, 0.f, 0.f};
      if (row < g.M && col < g.N) {
        const size_t off = (size_t)(row / g.S) * g.N;
        float4 nb = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e.nbias) nb = load4_guard(e.nbias, col, g.N, vN);
        const float4 ah = load4_guard(e.Ahat + (size_t)row * g.N, col, g.N, vN);
        const float4 dp = load4_guard(e.dpos + off, col, g.N, vN);
        const float4 dn = load4_guard(e.dneg + off, col, g.N, vN);
        float4 ep = make_float4(0.f, 0.f, 0.f, 0.f), en = ep;
        if (e.epos) ep = load4_guard(e.epos + off, col, g.N, vN);
        if (e.eneg) en = load4_guard(e.eneg + off, col, g.N, vN);
        const float4 pl = load4_guard(e.pre_l + off, col, g.N, vN);
        const float4 pu = load4_guard(e.pre_u + off, col, g.N, vN);
        float4 h;
#define BF_ADJ(c, idx)                                               \
  {                                                                  \
    const float gg = acc[i][jb * 4 + idx] + nb.c;                    \
    const bool sel = ah.c >= 0.f;                                    \
    h.c = (sel ? dp.c : dn.c) * gg + (sel ? ep.c : en.c);            \
    c4[idx] = (sel && pl.c < 0.f && pu.c > 0.f) ? ah.c * gg : 0.f;   \
  }
        BF_ADJ(x, 0) BF_ADJ(y, 1) BF_ADJ(z, 2) BF_ADJ(w, 3)
#undef BF_ADJ
        if (e.hout) store4_guard(e.hout + (size_t)row * g.N, col, g.N, vN, h);
        // columns beyond N inside this float4 carry zeros from the guarded loads
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) dsmem[rl * STAGE_LD + cl + q] = c4[q];
    }
  }
  __syncthreads();

  // Deterministic per-domain reduction over the spec rows that fall inside this tile.
  const int c = tid % TN;                 // column of this thread in the reductions
  const int half = tid / TN;              // domains are dealt round-robin to the GEMM_THREADS / TN thread groups
  constexpr int GROUPS = GEMM_THREADS / TN;
  const int m_end = min(m0 + TM, g.M);
  const int d_first = m0 / g.S;
  const int d_last = (m_end - 1) / g.S;
  const int col = n0 + c;
  for (int d = d_first + half; d <= d_last; d += GROUPS) {
    const int r_lo = max(d * g.S, m0) - m0;
    const int r_hi = min((d + 1) * g.S, m_end) - m0;
    float s = 0.f;
    for (int r = r_lo; r < r_hi; ++r) s += dsmem[r * STAGE_LD + c];
    if (col < g.N) atomicAdd(&e.grad[(size_t)d * g.N + col], s);
  }

  // Second reduction for the beta gradient: sum over the domain's spec rows of g itself.
  if (e.gsum != nullptr) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < MR; ++i) {
      const int rl = tile_row<MH>(ty, i);
      const int row = m0 + rl;
#pragma unroll
      for (int jb = 0; jb < NH; ++jb) {
        const int cl = tile_col(tx, jb);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int cc = n0 + cl + q;
          float gg = 0.f;
          if (row < g.M && cc < g.N) gg = acc[i][jb * 4 + q] + (e.nbias ? __ldg(e.nbias + cc) : 0.f);
          if (e.gw != nullptr && row < g.M) gg *= __ldg(e.gw + row);
          dsmem[rl * STAGE_LD + cl + q] = gg;
        }
      }
    }
    __syncthreads();
    for (int d = d_first + half; d <= d_last; d += GROUPS) {
      const int r_lo = max(d * g.S, m0) - m0;
      const int r_hi = min((d + 1) * g.S, m_end) - m0;
      float s = 0.f;
      for (int r = r_lo; r < r_hi; ++r) s += dsmem[r * STAGE_LD + c];
      if (col < g.N) atomicAdd(&e.gsum[(size_t)d * g.N + col], s);
    }
  }
}

int launch_crown_adjoint_linear(const float* Hprev, int first_layer, const float* mid, const float* rad, const float* W,
                                const float* nbias, const float* Ahat, const float* dpos, const float* dneg,
                                const float* epos, const float* eneg, const float* pre_l, const float* pre_u,
                                float* hout, float* grad, float* gsum, int M, int S, int K, int N, cudaStream_t stream,
                                const float* gw) {
  static SmemOptIn opt_in[6];
  GemmArgs g{};
  g.A = Hprev; g.Bm = W; g.M = M; g.N = N; g.K = K; g.S = S;
  const void* kptrs[] = {Hprev, W, mid, rad};
  g.vecK = (K % 4 == 0);
  for (const void* p : kptrs) if (p && (reinterpret_cast<uintptr_t>(p) & 15u)) g.vecK = 0;
  const void* nptrs[] = {nbias, Ahat, dpos, dneg, epos, eneg, pre_l, pre_u, hout};
  g.vecN = (N % 4 == 0);
  for (const void* p : nptrs) if (p && (reinterpret_cast<uintptr_t>(p) & 15u)) g.vecN = 0;
  g.mid = mid; g.rad = rad;
  AdjEpilogue e{nbias, Ahat, dpos, dneg, epos, eneg, pre_l, pre_u, hout, grad, gsum, gw};
  // 32-row tiles only while a domain's S rows still touch at most two row tiles (two atomic addends commute: deterministic sums)
  const bool small = ffma_small_tiles(M, N), quarter = ffma_quarter_tiles(M, N) && S <= 32;
  dim3 grid(ceil_div(M, quarter ? 32 : (small ? 64 : BM)), ceil_div(N, small ? 64 : BN));
  timing_begin(T_ADJ, stream);
#define BF_ADJ_LAUNCH(PRO_, MH_, NH_, slot)                                                                                     \
  {                                                                                                                             \
    if (int rc = ensure_dynamic_smem(crown_adjoint_linear_kernel<PRO_, MH_, NH_>, ADJ_SMEM_BYTES, opt_in[slot],                 \
                                     "crown_adjoint_linear_kernel"))                                                            \
      return rc;                                                                                                                \
    crown_adjoint_linear_kernel<PRO_, MH_, NH_><<<grid, GEMM_THREADS, ADJ_SMEM_BYTES, stream>>>(g, e);                          \
  }
  if (first_layer) {
    if (quarter) BF_ADJ_LAUNCH(PRO_H0, 0, 1, 4) else if (small) BF_ADJ_LAUNCH(PRO_H0, 1, 1, 0) else BF_ADJ_LAUNCH(PRO_H0, 2, 2, 1)
  } else {
    if (quarter) BF_ADJ_LAUNCH(PRO_PLAIN, 0, 1, 5) else if (small) BF_ADJ_LAUNCH(PRO_PLAIN, 1, 1, 2) else BF_ADJ_LAUNCH(PRO_PLAIN, 2, 2, 3)
  }
#undef BF_ADJ_LAUNCH
  timing_end(T_ADJ, stream, 4.0 * (double)M * K + 8.0 * (double)M * N, 2.0 * (double)M * K * N);
  BF_CHECK_LAUNCH("crown_adjoint_linear_kernel");
  return BF_OK;
}

}  // namespace bf

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
extern "C" int bf_crown_relu_linear_bwd(const float* A, int side, const float* alpha_u, const float* alpha_l,
                                        const float* beta_u, const float* beta_l, const float* add, const float* W,
                                        const float* bias, float* A_prev, float* delta, int accumulate, int B, int S,
                                        int n_cur, int n_prev, bf_stream_t stream) {
  BF_REQUIRE(A && W, BF_E_INVALID, "bf_crown_relu_linear_bwd: A and W must be non-null");
  BF_REQUIRE(B > 0 && S > 0 && n_cur > 0 && n_prev > 0, BF_E_INVALID, "bf_crown_relu_linear_bwd: sizes must be positive");
  BF_REQUIRE(side == BF_SIDE_LOWER || side == BF_SIDE_UPPER, BF_E_INVALID, "bf_crown_relu_linear_bwd: bad side");
  BF_REQUIRE(A_prev || delta, BF_E_INVALID, "bf_crown_relu_linear_bwd: nothing to compute");
  const bool relu = alpha_u || alpha_l || beta_u || beta_l;
  BF_REQUIRE(!relu || (alpha_u && alpha_l), BF_E_INVALID, "bf_crown_relu_linear_bwd: alpha_u and alpha_l must both be given");
  BF_REQUIRE((long long)B * S < 2147483647LL, BF_E_INVALID, "bf_crown_relu_linear_bwd: B*S overflows int");
  const float *dpos = nullptr, *dneg = nullptr, *epos = nullptr, *eneg = nullptr;
  if (relu) {
    if (side == BF_SIDE_LOWER) { dpos = alpha_l; dneg = alpha_u; epos = beta_l; eneg = beta_u; }
    else { dpos = alpha_u; dneg = alpha_l; epos = beta_u; eneg = beta_l; }
  }
  return bf::launch_crown_bwd_linear(A, dpos, dneg, epos, eneg, relu ? add : nullptr, W, bias, A_prev, delta, accumulate,
                                     nullptr, nullptr, nullptr, side, B * S, S, n_cur, n_prev, bf::as_stream(stream));
}

// ---------------------------------------------------------------------------
// Layer-level tensor-core path: the caller packs a layer's weight once (hi/lo TF32 images in the shared-memory
// layout of the tcgen05 kernel, preceded by a status word) and passes the pack with every call.
// ---------------------------------------------------------------------------
static const size_t kPackHeader = 256;  // status word + padding in front of the packed images

extern "C" size_t bf_linear_pack_bytes(int n_cur, int n_prev) {
  if (n_cur <= 0 || n_prev <= 0) return 0;
  return kPackHeader + ((bf::tc_packed_bytes(n_prev, n_cur) + 255) & ~(size_t)255);
}

extern "C" int bf_linear_pack(const float* W, int n_cur, int n_prev, void* pack, size_t pack_bytes, bf_stream_t stream_) {
  BF_REQUIRE(W && pack && n_cur > 0 && n_prev > 0, BF_E_INVALID, "bf_linear_pack: bad argument");
  BF_REQUIRE((reinterpret_cast<uintptr_t>(pack) & 255u) == 0, BF_E_INVALID, "bf_linear_pack: the pack buffer must be 256-byte aligned");
  BF_REQUIRE(pack_bytes >= bf_linear_pack_bytes(n_cur, n_prev), BF_E_WORKSPACE, "bf_linear_pack: %zu bytes needed",
             bf_linear_pack_bytes(n_cur, n_prev));
  cudaStream_t stream = bf::as_stream(stream_);
  if (cudaMemsetAsync(pack, 0, kPackHeader, stream) != cudaSuccess) {
    bf::set_error("bf_linear_pack: cudaMemsetAsync failed");
    return BF_E_CUDA;
  }
  // backward: A_prev = Lambda[M, n_cur] * W[n_cur, n_prev]  ->  B[n][k] = W[k][n] (transposed read)
  return bf::tc_pack_weights(W, n_cur, n_prev, 1, static_cast<unsigned char*>(pack) + kPackHeader, stream);
}

extern "C" int bf_linear_pack_status(const void* pack, int* status_out) {
  BF_REQUIRE(pack && status_out, BF_E_INVALID, "bf_linear_pack_status: null argument");
  if (cudaMemcpy(status_out, pack, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
    bf::set_error("bf_linear_pack_status: cudaMemcpy failed");
    return BF_E_CUDA;
  }
  return BF_OK;
}

extern "C" int bf_crown_relu_linear_bwd_packed(const float* A, int side, const float* alpha_u, const float* alpha_l,
                                               const float* beta_u, const float* beta_l, const float* add, const float* W,
                                               const float* bias, const void* pack, float* A_prev, float* delta, int accumulate,
                                               int B, int S, int n_cur, int n_prev, bf_stream_t stream_) {
  const long long M = (long long)B * S;
  // small problems, delta-only calls and calls without a pack take the FP32 FFMA tiles; so does (unless BF_B200_TC_MIN_ROWS
  // pins a plain row threshold) a problem whose 64 x 64 FFMA tiles fit one wave
  const char* rows_env = getenv("BF_B200_TC_MIN_ROWS");
  const int min_rows = (rows_env && atoi(rows_env) > 0) ? atoi(rows_env) : 256;
  const bool one_wave = !(rows_env && atoi(rows_env) > 0) && M < 2147483647LL && bf::ffma_fits_one_wave((int)M, n_prev);
  if (!pack || !A_prev || M < min_rows || one_wave || n_cur < 32 || n_prev < 32)
    return bf_crown_relu_linear_bwd(A, side, alpha_u, alpha_l, beta_u, beta_l, add, W, bias, A_prev, delta, accumulate, B, S, n_cur,
                                    n_prev, stream_);
  BF_REQUIRE(A && W, BF_E_INVALID, "bf_crown_relu_linear_bwd_packed: A and W must be non-null");
  BF_REQUIRE(B > 0 && S > 0 && M < 2147483647LL, BF_E_INVALID, "bf_crown_relu_linear_bwd_packed: bad sizes");
  BF_REQUIRE(side == BF_SIDE_LOWER || side == BF_SIDE_UPPER, BF_E_INVALID, "bf_crown_relu_linear_bwd_packed: bad side");
  BF_REQUIRE((reinterpret_cast<uintptr_t>(pack) & 255u) == 0, BF_E_INVALID, "bf_crown_relu_linear_bwd_packed: misaligned pack");
  const bool relu = alpha_u || alpha_l || beta_u || beta_l;
  BF_REQUIRE(!relu || (alpha_u && alpha_l), BF_E_INVALID, "bf_crown_relu_linear_bwd_packed: alpha_u and alpha_l must both be given");
  const float *dpos = nullptr, *dneg = nullptr, *epos = nullptr, *eneg = nullptr;
  if (relu) {
    if (side == BF_SIDE_LOWER) { dpos = alpha_l; dneg = alpha_u; epos = beta_l; eneg = beta_u; }
    else { dpos = alpha_u; dneg = alpha_l; epos = beta_u; eneg = beta_l; }
  }
  cudaStream_t stream = bf::as_stream(stream_);
  int* status = reinterpret_cast<int*>(const_cast<void*>(pack));
  const unsigned char* images = static_cast<const unsigned char*>(pack) + kPackHeader;
  const char* persistent = getenv("BF_B200_BWD_PERSISTENT");
  const char* pairs_env = getenv("BF_B200_BWD_PAIRS");
  int rc = (!(persistent && persistent[0] == '1') || !bf::crown_tc_persistent_supports(epos, eneg, relu ? add : nullptr))
               ? bf::launch_crown_bwd_linear_tc(A, dpos, dneg, epos, eneg, relu ? add : nullptr, images, bias, A_prev, delta, accumulate,
                                                nullptr, nullptr, nullptr, side, (int)M, S, n_cur, n_prev, status, stream, pairs_env && pairs_env[0] == '1')
               : bf::launch_crown_bwd_linear_tc_persistent(A, dpos, dneg, epos, eneg, relu ? add : nullptr, images, bias, A_prev, delta,
                                                           accumulate, nullptr, nullptr, nullptr, side, (int)M, S, n_cur, n_prev, status,
                                                           stream);
  if (rc != BF_OK) return rc;
  // a wait that expired inside the kernel invalidates the result: hand on NaN, never stale memory
  return bf::launch_poison_on_status(status, A_prev, M * n_prev, delta, delta ? M : 0, stream);
}
