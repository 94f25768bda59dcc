// First-layer infeasibility certificate for ReLU-split subdomains, one block per domain.
//
// Every split on the first ReLU is a half-space of the INPUT: s_j * (W1[j] . x + b1[j]) >= 0.
// If some convex combination of those half-spaces has a negative maximum over the input box,
//     max_{x in box} (sum_i w_i a_i) . x + sum_i w_i c_i  <  0,     w on the simplex,
// no input satisfies all of them and the domain is empty.  The weights are softmax(logits); the
// logits take `steps` Adam steps on that maximum (value = a.mid + |a|.rad + c), stopping at the
// first negative value.  A single half-space is tested directly.  On an L1 / L2 ball the maximum of a combination is
// a.centre + eps * ||a||_q (q dual to p), attained at centre + eps * (the unit-ball point aligned with a).
#include <math.h>

#include "kernels.cuh"

namespace bf {

constexpr int CERT_MAX_M = 16;     // half-spaces per domain handled by the kernel
constexpr int CERT_THREADS = 256;

// Sum over the block in a fixed order; result valid in every thread.
__device__ __forceinline__ float cert_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < CERT_THREADS / 32; ++w) t += red[w];
  return t;
}

__global__ void __launch_bounds__(CERT_THREADS) first_layer_cert_kernel(const int8_t* __restrict__ split, int split_stride,
                                                                        const float* __restrict__ W1, const float* __restrict__ b1,
                                                                        const float* __restrict__ mid, const float* __restrict__ rad,
                                                                        int norm_p, float eps, int n1, int n0, int steps, float lr,
                                                                        float tol, int* __restrict__ infeasible,
                                                                        float* __restrict__ best_value, int* __restrict__ n_halfspaces) {
  extern __shared__ __align__(16) float cert_smem[];
  float* A = cert_smem;                      // [CERT_MAX_M][n0]  s_i * W1[j_i]
  float* smid = A + (size_t)CERT_MAX_M * n0;  // [n0]
  float* srad = smid + n0;                   // [n0] box radius; on an Lp ball: the combination a of the current iteration
  __shared__ int idx[CERT_MAX_M];
  __shared__ float sgn[CERT_MAX_M], cvec[CERT_MAX_M], logit[CERT_MAX_M], wgt[CERT_MAX_M], am[CERT_MAX_M], av[CERT_MAX_M];
  __shared__ float red[CERT_THREADS / 32];
  __shared__ int m_sh;
  const int d = blockIdx.x;
  const int8_t* sp = split + (size_t)d * split_stride;

  // half-spaces in ascending neuron order (warp 0, ballot compaction)
  if (threadIdx.x < 32) {
    int count = 0;
    for (int base = 0; base < n1; base += 32) {
      const int j = base + threadIdx.x;
      const int s = (j < n1) ? (int)sp[j] : 0;
      const unsigned mask = __ballot_sync(0xffffffffu, s != 0);
      if (s != 0) {
        const int pos = count + __popc(mask & ((1u << threadIdx.x) - 1u));
        if (pos < CERT_MAX_M) { idx[pos] = j; sgn[pos] = (float)s; }
      }
      count += __popc(mask);
    }
    if (threadIdx.x == 0) m_sh = count;
  }
  __syncthreads();
  const int m = m_sh;
  if (threadIdx.x == 0 && n_halfspaces) n_halfspaces[d] = m;
  if (m == 0 || m > CERT_MAX_M) {  // nothing to test / more half-spaces than the kernel holds: no verdict
    if (threadIdx.x == 0) {
      infeasible[d] = (m == 0) ? 0 : -1;
      if (best_value) best_value[d] = INFINITY;
    }
    return;
  }
  for (int k = threadIdx.x; k < n0; k += CERT_THREADS) {
    smid[k] = mid[(size_t)d * n0 + k];
    srad[k] = (norm_p == BF_NORM_BOX) ? rad[(size_t)d * n0 + k] : 0.f;
  }
  for (int i = 0; i < m; ++i)
    for (int k = threadIdx.x; k < n0; k += CERT_THREADS) A[(size_t)i * n0 + k] = sgn[i] * __ldg(W1 + (size_t)idx[i] * n0 + k);
  if (threadIdx.x < m) {
    cvec[threadIdx.x] = sgn[threadIdx.x] * (b1 ? b1[idx[threadIdx.x]] : 0.f);
    logit[threadIdx.x] = 0.f;
    am[threadIdx.x] = 0.f;
    av[threadIdx.x] = 0.f;
  }
  __syncthreads();

  float best = INFINITY;
  int found = 0;
  const int iters = (m == 1) ? 1 : steps;
  for (int t = 0; t < iters; ++t) {
    // weights on the simplex
    if (threadIdx.x == 0) {
      float mx = logit[0];
      for (int i = 1; i < m; ++i) mx = fmaxf(mx, logit[i]);
      float s = 0.f;
      for (int i = 0; i < m; ++i) { wgt[i] = expf(logit[i] - mx); s += wgt[i]; }
      for (int i = 0; i < m; ++i) wgt[i] /= s;
    }
    __syncthreads();
    // value of the combination and d value / d w_i
    float val_p = 0.f, g_p[CERT_MAX_M];
#pragma unroll
    for (int i = 0; i < CERT_MAX_M; ++i) g_p[i] = 0.f;
    float val;
    if (norm_p == BF_NORM_BOX) {
      for (int k = threadIdx.x; k < n0; k += CERT_THREADS) {
        float a = 0.f;
        for (int i = 0; i < m; ++i) a = fmaf(wgt[i], A[(size_t)i * n0 + k], a);
        const float sg = (a > 0.f) ? 1.f : ((a < 0.f) ? -1.f : 0.f);
        const float x = fmaf(sg, srad[k], smid[k]);  // maximiser of a . x over the box (sub-gradient 0 at a == 0)
        val_p = fmaf(a, smid[k], val_p);
        val_p = fmaf(fabsf(a), srad[k], val_p);
#pragma unroll
        for (int i = 0; i < CERT_MAX_M; ++i)
          if (i < m) g_p[i] = fmaf(A[(size_t)i * n0 + k], x, g_p[i]);
      }
      val = cert_block_sum(val_p, red);
    } else {
      // L2 ball: dual norm ||a||_2, maximiser centre + eps * a / ||a||_2; L1 ball: dual norm max |a_k|, maximiser
      // centre + eps * sign(a_k) / (number of maxima) at the maxima (the sub-gradient torch's amax backward takes)
      float nrm_p = 0.f;
      for (int k = threadIdx.x; k < n0; k += CERT_THREADS) {
        float a = 0.f;
        for (int i = 0; i < m; ++i) a = fmaf(wgt[i], A[(size_t)i * n0 + k], a);
        srad[k] = a;
        val_p = fmaf(a, smid[k], val_p);
        nrm_p = (norm_p == BF_NORM_L2) ? fmaf(a, a, nrm_p) : fmaxf(nrm_p, fabsf(a));
      }
      float nrm, cnt = 1.f;
      if (norm_p == BF_NORM_L2) {
        nrm = sqrtf(cert_block_sum(nrm_p, red));
      } else {
        // block maximum through the sum helper: every thread contributes its maximum once per candidate round
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) nrm_p = fmaxf(nrm_p, __shfl_xor_sync(0xffffffffu, nrm_p, o));
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = nrm_p;
        __syncthreads();
        nrm = red[0];
#pragma unroll
        for (int w = 1; w < CERT_THREADS / 32; ++w) nrm = fmaxf(nrm, red[w]);
        __syncthreads();
        float c_p = 0.f;
        for (int k = threadIdx.x; k < n0; k += CERT_THREADS) c_p += (fabsf(srad[k]) == nrm) ? 1.f : 0.f;
        cnt = fmaxf(cert_block_sum(c_p, red), 1.f);
      }
      for (int k = threadIdx.x; k < n0; k += CERT_THREADS) {
        const float a = srad[k];
        float dir;
        if (norm_p == BF_NORM_L2) dir = (nrm > 0.f) ? a / nrm : 0.f;
        else dir = (fabsf(a) == nrm && nrm > 0.f) ? ((a > 0.f) ? 1.f : -1.f) / cnt : 0.f;
        const float x = fmaf(eps, dir, smid[k]);
#pragma unroll
        for (int i = 0; i < CERT_MAX_M; ++i)
          if (i < m) g_p[i] = fmaf(A[(size_t)i * n0 + k], x, g_p[i]);
      }
      val = cert_block_sum(val_p, red) + eps * nrm;
    }
    float g[CERT_MAX_M];
#pragma unroll
    for (int i = 0; i < CERT_MAX_M; ++i) g[i] = (i < m) ? cert_block_sum(g_p[i], red) + cvec[i] : 0.f;
    for (int i = 0; i < m; ++i) val = fmaf(wgt[i], cvec[i], val);
    best = fminf(best, val);
    if (val < -tol) { found = 1; break; }   // uniform across the block: every thread holds the same sums
    if (m == 1) break;
    // Adam on the logits (torch.optim.Adam defaults), gradient through the softmax
    __syncthreads();
    if (threadIdx.x == 0) {
      float dot = 0.f;
      for (int i = 0; i < m; ++i) dot = fmaf(wgt[i], g[i], dot);
      const float bc1 = 1.f - powf(0.9f, (float)(t + 1)), bc2 = 1.f - powf(0.999f, (float)(t + 1));
      for (int i = 0; i < m; ++i) {
        const float gi = wgt[i] * (g[i] - dot);
        am[i] = am[i] + 0.1f * (gi - am[i]);
        av[i] = av[i] * 0.999f + 0.001f * gi * gi;
        const float denom = sqrtf(av[i]) / sqrtf(bc2) + 1e-8f;
        logit[i] -= (lr / bc1) * (am[i] / denom);
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    infeasible[d] = (found || best < -tol) ? 1 : 0;
    if (best_value) best_value[d] = best;
  }
}

}  // namespace bf

extern "C" int bf_first_layer_certificate_max_halfspaces(void) { return bf::CERT_MAX_M; }

static int first_layer_certificate(const char* who, const int8_t* split, int split_stride, const float* W1, const float* b1,
                                   const float* mid, const float* rad, int norm_p, float eps, int* infeasible, float* best_value,
                                   int* n_halfspaces, int steps, float lr, float tol, int B, int n1, int n0, bf_stream_t stream);

extern "C" int bf_first_layer_certificate(const int8_t* split, int split_stride, const float* W1, const float* b1,
                                          const float* mid, const float* rad, int* infeasible, float* best_value,
                                          int* n_halfspaces, int steps, float lr, float tol, int B, int n1, int n0,
                                          bf_stream_t stream) {
  BF_REQUIRE(rad, BF_E_INVALID, "bf_first_layer_certificate: null tensor");
  return first_layer_certificate("bf_first_layer_certificate", split, split_stride, W1, b1, mid, rad, BF_NORM_BOX, 0.f, infeasible,
                                 best_value, n_halfspaces, steps, lr, tol, B, n1, n0, stream);
}

extern "C" int bf_first_layer_certificate_lp(const int8_t* split, int split_stride, const float* W1, const float* b1,
                                             const float* center, float eps, int p, int* infeasible, float* best_value,
                                             int* n_halfspaces, int steps, float lr, float tol, int B, int n1, int n0,
                                             bf_stream_t stream) {
  BF_REQUIRE((p == BF_NORM_L1 || p == BF_NORM_L2) && eps >= 0.f, BF_E_INVALID, "bf_first_layer_certificate_lp: p must be BF_NORM_L1 or BF_NORM_L2, eps >= 0");
  return first_layer_certificate("bf_first_layer_certificate_lp", split, split_stride, W1, b1, center, nullptr, p, eps, infeasible,
                                 best_value, n_halfspaces, steps, lr, tol, B, n1, n0, stream);
}

static int first_layer_certificate(const char* who, const int8_t* split, int split_stride, const float* W1, const float* b1,
                                   const float* mid, const float* rad, int norm_p, float eps, int* infeasible, float* best_value,
                                   int* n_halfspaces, int steps, float lr, float tol, int B, int n1, int n0, bf_stream_t stream) {
  BF_REQUIRE(split && W1 && mid && infeasible, BF_E_INVALID, "%s: null tensor", who);
  BF_REQUIRE(B > 0 && n1 > 0 && n0 > 0 && steps > 0 && lr > 0.f && tol >= 0.f, BF_E_INVALID, "%s: bad sizes or options", who);
  BF_REQUIRE(split_stride == 0 || split_stride == n1, BF_E_INVALID, "%s: split_stride must be 0 or n1", who);
  const size_t smem = ((size_t)bf::CERT_MAX_M + 2) * n0 * sizeof(float);
  BF_REQUIRE(smem <= 200 * 1024, BF_E_UNSUPPORTED, "%s: input dimension %d too large for one block", who, n0);
  static bf::SmemOptIn opt_in;
  if (int rc = bf::ensure_dynamic_smem(bf::first_layer_cert_kernel, 200 * 1024, opt_in, "first_layer_cert_kernel")) return rc;
  bf::first_layer_cert_kernel<<<B, bf::CERT_THREADS, smem, bf::as_stream(stream)>>>(split, split_stride, W1, b1, mid, rad, norm_p, eps, n1, n0,
                                                                                  steps, lr, tol, infeasible, best_value, n_halfspaces);
  BF_CHECK_LAUNCH("first_layer_cert_kernel");
  return BF_OK;
}

// ---------------------------------------------------------------------------
// Half-space rows of a Conv2d first layer: out[r, :] = the row of the layer's dense matrix that produces output
// neuron rows[r] = (co, ho, wo), i.e. the filter W[co] placed at (ho*sh - ph, wo*sw - pw) in the [Ci,Hi,Wi] input
// (zero elsewhere, taps outside the image dropped), and out_b[r] = bias[co].  One block per requested row.
// ---------------------------------------------------------------------------
namespace bf {

__global__ void __launch_bounds__(256) conv_dense_rows_kernel(const float* __restrict__ W, const float* __restrict__ bias,
                                                              const int* __restrict__ rows, float* __restrict__ out,
                                                              float* __restrict__ out_b, int Ci, int Hi, int Wi, int Co, int Ho,
                                                              int Wo, int kh, int kw, int sh, int sw, int ph, int pw) {
  const int r = blockIdx.x;
  const int j = rows[r];
  const int n0 = Ci * Hi * Wi;
  float* o = out + (size_t)r * n0;
  const bool valid = j >= 0 && j < Co * Ho * Wo;  // an index outside the layer gives a zero row
  const int co = valid ? j / (Ho * Wo) : 0;
  const int rem = valid ? j - co * (Ho * Wo) : 0;
  const int y0 = (rem / Wo) * sh - ph, x0 = (rem % Wo) * sw - pw;
  for (int i = threadIdx.x; i < n0; i += blockDim.x) {
    const int ci = i / (Hi * Wi);
    const int p = i - ci * (Hi * Wi);
    const int ky = p / Wi - y0, kx = p % Wi - x0;
    float v = 0.f;
    if (valid && ky >= 0 && ky < kh && kx >= 0 && kx < kw) v = W[(((size_t)co * Ci + ci) * kh + ky) * kw + kx];
    o[i] = v;
  }
  if (threadIdx.x == 0 && out_b) out_b[r] = (valid && bias) ? bias[co] : 0.f;
}

}  // namespace bf

extern "C" int bf_conv2d_dense_rows(const float* W, const float* bias, const int* rows, int n_rows, float* out_W, float* out_b,
                                    int Ci, int Hi, int Wi, int Co, int Ho, int Wo, int kh, int kw, int sh, int sw, int ph, int pw,
                                    bf_stream_t stream) {
  BF_REQUIRE(W && rows && out_W, BF_E_INVALID, "bf_conv2d_dense_rows: null tensor");
  BF_REQUIRE(n_rows > 0 && Ci > 0 && Hi > 0 && Wi > 0 && Co > 0 && Ho > 0 && Wo > 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0 && ph >= 0 && pw >= 0,
             BF_E_INVALID, "bf_conv2d_dense_rows: bad sizes");
  BF_REQUIRE((long long)Ci * Hi * Wi < 2147483647LL && (long long)Co * Ho * Wo < 2147483647LL, BF_E_UNSUPPORTED,
             "bf_conv2d_dense_rows: layer too large");
  bf::conv_dense_rows_kernel<<<n_rows, 256, 0, bf::as_stream(stream)>>>(W, bias, rows, out_W, out_b, Ci, Hi, Wi, Co, Ho, Wo, kh, kw, sh, sw,
                                                                         ph, pw);
  BF_CHECK_LAUNCH("conv_dense_rows_kernel");
  return BF_OK;
}
