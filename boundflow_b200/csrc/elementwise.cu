// HBM-bound pieces: ReLU relaxation, concretisation, partial-sum finalisation,
// per-domain best tracking, the fused Adam/projection/slope kernel and verdicts.
#include <float.h>

#include "kernels.cuh"

namespace bf {

// ---- ReLU relaxation ---------------------------------------------------------
__device__ __forceinline__ void relax_one(float l, float u, float& au, float& bu, float& al_plain) {
  // pos = l >= 0 -> slope 1; neg = u <= 0 -> slope 0 and wins when both hold.
  if (u <= 0.f) { au = 0.f; bu = 0.f; al_plain = 0.f; }
  else if (l >= 0.f) { au = 1.f; bu = 0.f; al_plain = 1.f; }
  else {
    const float denom = fmaxf(u - l, FLT_EPSILON);
    au = u / denom;
    bu = -l * au;
    al_plain = 0.f;
  }
}

__global__ void relu_relax_kernel(const float* __restrict__ l, const float* __restrict__ u, const float* __restrict__ alpha,
                                  int alpha_stride, float* __restrict__ alpha_u, float* __restrict__ beta_u,
                                  float* __restrict__ alpha_l, int n, long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const float lo = l[i], up = u[i];
    float au, bu, al;
    relax_one(lo, up, au, bu, al);
    if (alpha != nullptr && lo < 0.f && up > 0.f) {
      // alpha_stride is n (per-domain rows, same flat index) or 0 (one shared row)
      const float a = (alpha_stride != 0) ? alpha[i] : alpha[i % n];
      al = fminf(fmaxf(a, 0.f), 1.f);
    }
    alpha_u[i] = au;
    beta_u[i] = bu;
    alpha_l[i] = al;
  }
}

static int ew_grid(long long total, int threads) {
  long long blocks = (total + threads - 1) / threads;
  const long long cap = 148LL * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

int launch_relu_relax(const float* l, const float* u, const float* alpha, int alpha_stride, float* alpha_u,
                      float* beta_u, float* alpha_l, int B, int n, cudaStream_t stream) {
  const long long total = (long long)B * n;
  relu_relax_kernel<<<ew_grid(total, 256), 256, 0, stream>>>(l, u, alpha, alpha_stride, alpha_u, beta_u, alpha_l, n, total);
  BF_CHECK_LAUNCH("relu_relax_kernel");
  return BF_OK;
}

// ---- concretisation: one warp per coefficient row -----------------------------
__global__ void __launch_bounds__(256) concretize_kernel(const float* __restrict__ A, const float* __restrict__ mid,
                                                         const float* __restrict__ rad, const float* __restrict__ bias_in,
                                                         float* __restrict__ out, float sgn, int M, int S, int n0, int vec) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int m = warp; m < M; m += nwarps) {
    const float* a = A + (size_t)m * n0;
    const size_t off = (size_t)(m / S) * n0;
    float center = 0.f, dev = 0.f;
    for (int k = lane * 4; k < n0; k += 128) {
      const float4 av = load4_guard(a, k, n0, vec != 0);
      const float4 md = load4_guard(mid + off, k, n0, vec != 0);
      const float4 rd = load4_guard(rad + off, k, n0, vec != 0);
      center = fmaf(av.x, md.x, center); center = fmaf(av.y, md.y, center);
      center = fmaf(av.z, md.z, center); center = fmaf(av.w, md.w, center);
      dev = fmaf(fabsf(av.x), rd.x, dev); dev = fmaf(fabsf(av.y), rd.y, dev);
      dev = fmaf(fabsf(av.z), rd.z, dev); dev = fmaf(fabsf(av.w), rd.w, dev);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      center += __shfl_xor_sync(0xffffffffu, center, o);
      dev += __shfl_xor_sync(0xffffffffu, dev, o);
    }
    if (lane == 0) out[m] = center + sgn * dev + (bias_in ? bias_in[m] : 0.f);
  }
}

int launch_concretize(const float* A, const float* mid, const float* rad, const float* bias_in, float* out, int side,
                      int B, int S, int n0, cudaStream_t stream) {
  const int M = B * S;
  int vec = (n0 % 4 == 0);
  const void* ptrs[] = {A, mid, rad};
  for (const void* p : ptrs) if (reinterpret_cast<uintptr_t>(p) & 15u) vec = 0;
  int blocks = ceil_div(M, 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  timing_begin(T_CONCRETIZE, stream);
  concretize_kernel<<<blocks, 256, 0, stream>>>(A, mid, rad, bias_in, out, side == BF_SIDE_LOWER ? -1.f : 1.f, M, S, n0, vec);
  // every coefficient row once, the box of every domain once, one result per row
  timing_end(T_CONCRETIZE, stream, 4.0 * (double)M * n0 + 8.0 * (double)B * n0 + 4.0 * M, 4.0 * (double)M * n0);
  BF_CHECK_LAUNCH("concretize_kernel");
  return BF_OK;
}

// ---- finalisation of the fused first-layer concretisation ---------------------
__global__ void sum_partials_kernel(const float* __restrict__ c, const float* __restrict__ partial, int ntiles,
                                    float* __restrict__ out, int M) {
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  float s = 0.f;
  for (int t = 0; t < ntiles; ++t) s += partial[(size_t)m * ntiles + t];
  out[m] = s + (c ? c[m] : 0.f);
}

int launch_sum_partials(const float* c, const float* partial, int ntiles, float* out, int M, cudaStream_t stream) {
  sum_partials_kernel<<<ceil_div(M, 256), 256, 0, stream>>>(c, partial, ntiles, out, M);
  BF_CHECK_LAUNCH("sum_partials_kernel");
  return BF_OK;
}

// ---- per-domain objective and strict best-of ----------------------------------
__global__ void select_best_kernel(const float* __restrict__ cur, float* __restrict__ best_lower,
                                   float* __restrict__ best_metric, int* __restrict__ improve, int first, int spec_reduce,
                                   float soft_tau, float* __restrict__ row_weight, int B, int S) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const float* row = cur + (size_t)b * S;
  float metric;
  if (spec_reduce == BF_REDUCE_MEAN || spec_reduce == BF_REDUCE_SUM) {
    float s = 0.f;
    for (int k = 0; k < S; ++k) s += row[k];
    metric = (spec_reduce == BF_REDUCE_MEAN) ? (s / (float)S) : s;
  } else {
    // min: the smallest spec row; softmin: -tau * logsumexp(-x / tau).  row_weight receives d metric / d row[k]
    // (one-hot at the first minimum, or softmax(-x / tau)): the gradient sweep weights the spec rows with it.
    float mn = row[0];
    int arg = 0;
    for (int k = 1; k < S; ++k)
      if (row[k] < mn) { mn = row[k]; arg = k; }
    if (spec_reduce == BF_REDUCE_MIN) {
      metric = mn;
      if (row_weight)
        for (int k = 0; k < S; ++k) row_weight[(size_t)b * S + k] = (k == arg) ? 1.f : 0.f;
    } else {
      float z = 0.f;
      for (int k = 0; k < S; ++k) z += expf(-(row[k] - mn) / soft_tau);
      metric = mn - soft_tau * logf(z);
      if (row_weight)
        for (int k = 0; k < S; ++k) row_weight[(size_t)b * S + k] = expf(-(row[k] - mn) / soft_tau) / z;
    }
  }
  const bool imp = first || (metric > best_metric[b]);
  if (imp) {
    best_metric[b] = metric;
    for (int k = 0; k < S; ++k) best_lower[(size_t)b * S + k] = row[k];
  }
  improve[b] = imp ? 1 : 0;
}

int launch_select_best(const float* cur, float* best_lower, float* best_metric, int* improve, int first,
                       int spec_reduce, float soft_tau, float* row_weight, int B, int S, cudaStream_t stream) {
  select_best_kernel<<<ceil_div(B, 128), 128, 0, stream>>>(cur, best_lower, best_metric, improve, first, spec_reduce, soft_tau,
                                                           row_weight, B, S);
  BF_CHECK_LAUNCH("select_best_kernel");
  return BF_OK;
}

// Objectives that also involve the upper bound.  The caller evaluates 2S spec rows per domain, the S rows c_s followed
// by their negations, so cur[b, s] is the lower bound of row s and cur[b, S + s] is minus its upper bound; with
// reduce() = mean | min | softmin over s (upper-side max / softmax are min / softmin of the negated values):
//   both:  metric = lb_weight * reduce(cur[b, :S]) + ub_weight * reduce(cur[b, S:])
//   gap:   metric = reduce(cur[b, :S] + cur[b, S:])                    (= -reduce_max(upper - lower))
// row_weight receives d metric / d cur[b, j] for all 2S rows (the gradient sweep weights the saved rows with it).
__device__ __forceinline__ float reduce_pass(const float* x, const float* y, int S, int spec_reduce, float tau, float* w, float scale) {
  // value of reduce(x + y) (y may be null); w (if given) receives scale * d value / d x[k]
  auto at = [&](int k) { return y ? x[k] + y[k] : x[k]; };
  if (spec_reduce == BF_REDUCE_MEAN) {
    float s = 0.f;
    for (int k = 0; k < S; ++k) s += at(k);
    if (w) for (int k = 0; k < S; ++k) w[k] = scale / (float)S;
    return s / (float)S;
  }
  float mn = at(0);
  int arg = 0;
  for (int k = 1; k < S; ++k) {
    const float v = at(k);
    if (v < mn) { mn = v; arg = k; }
  }
  if (spec_reduce == BF_REDUCE_MIN) {
    if (w) for (int k = 0; k < S; ++k) w[k] = (k == arg) ? scale : 0.f;
    return mn;
  }
  float z = 0.f;
  for (int k = 0; k < S; ++k) z += expf(-(at(k) - mn) / tau);
  if (w) for (int k = 0; k < S; ++k) w[k] = scale * expf(-(at(k) - mn) / tau) / z;
  return mn - tau * logf(z);
}

__global__ void select_best_paired_kernel(const float* __restrict__ cur, float* __restrict__ best_rows, float* __restrict__ best_metric,
                                          int* __restrict__ improve, int first, int objective, int spec_reduce, float soft_tau,
                                          float lb_weight, float ub_weight, float* __restrict__ row_weight, int B, int S) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const float* lo = cur + (size_t)b * 2 * S;
  const float* nu = lo + S;
  float* w = row_weight ? row_weight + (size_t)b * 2 * S : nullptr;
  float metric;
  if (objective == BF_OBJECTIVE_BOTH) {
    metric = lb_weight * reduce_pass(lo, nullptr, S, spec_reduce, soft_tau, w, lb_weight);
    metric += ub_weight * reduce_pass(nu, nullptr, S, spec_reduce, soft_tau, w ? w + S : nullptr, ub_weight);
  } else {  // gap
    metric = reduce_pass(lo, nu, S, spec_reduce, soft_tau, w, 1.f);
    if (w) for (int k = 0; k < S; ++k) w[S + k] = w[k];
  }
  const bool imp = first || (metric > best_metric[b]);
  if (imp) {
    best_metric[b] = metric;
    for (int k = 0; k < 2 * S; ++k) best_rows[(size_t)b * 2 * S + k] = lo[k];
  }
  improve[b] = imp ? 1 : 0;
}

int launch_select_best_paired(const float* cur, float* best_rows, float* best_metric, int* improve, int first, int objective,
                              int spec_reduce, float soft_tau, float lb_weight, float ub_weight, float* row_weight, int B, int S,
                              cudaStream_t stream) {
  select_best_paired_kernel<<<ceil_div(B, 128), 128, 0, stream>>>(cur, best_rows, best_metric, improve, first, objective, spec_reduce,
                                                                  soft_tau, lb_weight, ub_weight, row_weight, B, S);
  BF_CHECK_LAUNCH("select_best_paired_kernel");
  return BF_OK;
}

// A[m, :] *= w[m]: weights the saved coefficient rows of a layer by d objective / d lower[m] before the gradient sweep
// (min / softmin objectives; a positive factor keeps every sign decision of the sweep, a zero factor removes the row).
__global__ void scale_rows_kernel(float* __restrict__ A, const float* __restrict__ w, long long total, int n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    A[i] *= w[i / n];
}

int launch_scale_rows(float* A, const float* w, long long M, int n, cudaStream_t stream) {
  scale_rows_kernel<<<ew_grid(M * n, 256), 256, 0, stream>>>(A, w, M * n, n);
  BF_CHECK_LAUNCH("scale_rows_kernel");
  return BF_OK;
}

// ---- Adam + projection + best-alpha snapshot + next lower slope ---------------
// One element: torch.optim.Adam (no amsgrad / weight decay): lerp for the first moment,
// mul+addcmul for the second, sqrt(v)/sqrt(bc2)+eps as denominator, then clamp to [0,1].
__device__ __forceinline__ void adam_one(float& a, float& mi, float& vi, float g, float lo, float up, float& sl,
                                         const AdamScalars& sc) {
  mi = mi + sc.one_minus_beta1 * (g - mi);
  vi = vi * sc.beta2 + sc.one_minus_beta2 * g * g;
  const float denom = sqrtf(vi) / sc.bc2_sqrt + sc.eps;
  a = a - sc.lr_step * (mi / denom);
  a = fminf(fmaxf(a, 0.f), 1.f);
  sl = (up <= 0.f) ? 0.f : ((lo >= 0.f) ? 1.f : a);
}

// grid (B, column chunks): one domain row per blockIdx.x, VEC consecutive columns per thread.
template <int VEC>
__global__ void __launch_bounds__(128) adam_step_kernel(float* __restrict__ alpha, float* __restrict__ m, float* __restrict__ v,
                                                        float* __restrict__ grad, const int* __restrict__ improve,
                                                        float* __restrict__ best_alpha, const float* __restrict__ pre_l,
                                                        const float* __restrict__ pre_u, float* __restrict__ slope_l,
                                                        AdamScalars sc, int do_update, int n) {
  const int b = blockIdx.x;
  const int j = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (j >= n) return;
  const size_t i = (size_t)b * n + j;
  const bool imp = improve[b] != 0;
  if (VEC == 4) {
    float4 a = *reinterpret_cast<const float4*>(alpha + i);
    if (imp) *reinterpret_cast<float4*>(best_alpha + i) = a;
    if (!do_update) return;
    float4 g = *reinterpret_cast<const float4*>(grad + i);
    float4 mi = *reinterpret_cast<const float4*>(m + i), vi = *reinterpret_cast<const float4*>(v + i);
    const float4 lo = *reinterpret_cast<const float4*>(pre_l + i), up = *reinterpret_cast<const float4*>(pre_u + i);
    float4 sl;
    adam_one(a.x, mi.x, vi.x, g.x * sc.grad_scale, lo.x, up.x, sl.x, sc);
    adam_one(a.y, mi.y, vi.y, g.y * sc.grad_scale, lo.y, up.y, sl.y, sc);
    adam_one(a.z, mi.z, vi.z, g.z * sc.grad_scale, lo.z, up.z, sl.z, sc);
    adam_one(a.w, mi.w, vi.w, g.w * sc.grad_scale, lo.w, up.w, sl.w, sc);
    *reinterpret_cast<float4*>(grad + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(m + i) = mi;
    *reinterpret_cast<float4*>(v + i) = vi;
    *reinterpret_cast<float4*>(alpha + i) = a;
    *reinterpret_cast<float4*>(slope_l + i) = sl;
  } else {
    float a = alpha[i];
    if (imp) best_alpha[i] = a;
    if (!do_update) return;
    float mi = m[i], vi = v[i], sl;
    adam_one(a, mi, vi, grad[i] * sc.grad_scale, pre_l[i], pre_u[i], sl, sc);
    grad[i] = 0.f;
    m[i] = mi;
    v[i] = vi;
    alpha[i] = a;
    slope_l[i] = sl;
  }
}

int launch_adam_step(float* alpha, float* m, float* v, float* grad, const int* improve, float* best_alpha,
                     const float* pre_l, const float* pre_u, float* slope_l, AdamScalars sc, int do_update, int B, int n,
                     cudaStream_t stream) {
  bool vec = (n % 4 == 0);
  const void* ptrs[] = {alpha, m, v, grad, best_alpha, pre_l, pre_u, slope_l};
  for (const void* q : ptrs) if (reinterpret_cast<uintptr_t>(q) & 15u) vec = false;
  timing_begin(T_ADAM, stream);
  if (vec) {
    dim3 grid(B, ceil_div(n / 4, 128));
    adam_step_kernel<4><<<grid, 128, 0, stream>>>(alpha, m, v, grad, improve, best_alpha, pre_l, pre_u, slope_l, sc, do_update, n);
  } else {
    dim3 grid(B, ceil_div(n, 128));
    adam_step_kernel<1><<<grid, 128, 0, stream>>>(alpha, m, v, grad, improve, best_alpha, pre_l, pre_u, slope_l, sc, do_update, n);
  }
  // the optimiser's own traffic: read alpha, m, v, grad and write alpha, m, v (28 B per element); the kernel also
  // reads the pre-activation bounds, clears the gradient and writes the next lower slope and the best-alpha snapshot
  // (up to 48 B per element in all), which replaces separate relaxation / snapshot passes
  timing_end(T_ADAM, stream, (do_update ? 28.0 : 8.0) * (double)B * n, do_update ? 10.0 * (double)B * n : 0.0);
  BF_CHECK_LAUNCH("adam_step_kernel");
  return BF_OK;
}

__global__ void scale_copy_kernel(const float* __restrict__ src, float scale, float* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = src[i] * scale;
}

int launch_scale_copy(const float* src, float scale, float* dst, long long n, cudaStream_t stream) {
  scale_copy_kernel<<<ew_grid(n, 256), 256, 0, stream>>>(src, scale, dst, n);
  BF_CHECK_LAUNCH("scale_copy_kernel");
  return BF_OK;
}

// ---- shared-alpha mode: one alpha per neuron for the whole batch ----------------
// Whole-batch objective (mean of every lower bound) and strict best-of on one scalar.
// A single block sums in a fixed order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(1024) shared_metric_kernel(const float* __restrict__ cur, long long M,
                                                             float* __restrict__ best_metric, int* __restrict__ improve,
                                                             int first) {
  __shared__ float red[1024];
  float s = 0.f;
  for (long long i = threadIdx.x; i < M; i += blockDim.x) s += cur[i];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int w = blockDim.x / 2; w > 0; w >>= 1) {
    if ((int)threadIdx.x < w) red[threadIdx.x] += red[threadIdx.x + w];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float metric = red[0] / (float)M;
    const bool imp = first || (metric > best_metric[0]);
    if (imp) best_metric[0] = metric;
    improve[0] = imp ? 1 : 0;
  }
}

int launch_shared_metric(const float* cur, long long M, float* best_metric, int* improve, int first, cudaStream_t stream) {
  shared_metric_kernel<<<1, 1024, 0, stream>>>(cur, M, best_metric, improve, first);
  BF_CHECK_LAUNCH("shared_metric_kernel");
  return BF_OK;
}

__global__ void copy_if_kernel(const float* __restrict__ src, float* __restrict__ dst, long long n, const int* __restrict__ flag) {
  if (flag[0] == 0) return;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dst[i] = src[i];
}

int launch_copy_if(const float* src, float* dst, long long n, const int* flag, cudaStream_t stream) {
  copy_if_kernel<<<ew_grid(n, 256), 256, 0, stream>>>(src, dst, n, flag);
  BF_CHECK_LAUNCH("copy_if_kernel");
  return BF_OK;
}

// Column sums of a per-domain gradient in two fixed-order stages: grid (column blocks, row chunks)
// writes part[chunk, j] = sum over the chunk's rows of grad[b, j] (times -split[b, j] for a beta
// gradient) and clears what it read.
__global__ void __launch_bounds__(128) grad_colsum_kernel(float* __restrict__ grad, const int8_t* __restrict__ split,
                                                          int split_stride, float* __restrict__ part, int B, int n,
                                                          int rows_per_chunk) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const int b0 = blockIdx.y * rows_per_chunk;
  const int b1 = min(B, b0 + rows_per_chunk);
  float s = 0.f;
  for (int b = b0; b < b1; ++b) {
    const size_t i = (size_t)b * n + j;
    const float g = grad[i];
    s += split ? g * -(float)split[(size_t)b * split_stride + j] : g;
    grad[i] = 0.f;
  }
  part[(size_t)blockIdx.y * n + j] = s;
}

// Adam on one shared parameter vector: alpha is projected to [0,1], beta to [0,inf).
__global__ void __launch_bounds__(128) shared_adam_kernel(float* __restrict__ param, float* __restrict__ m, float* __restrict__ v,
                                                          const float* __restrict__ part, int chunks,
                                                          const int* __restrict__ improve, float* __restrict__ best,
                                                          AdamScalars sc, int do_update, int is_beta, int n) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  float a = param[j];
  if (improve[0] != 0) best[j] = a;
  if (!do_update) return;
  float g = 0.f;
  for (int c = 0; c < chunks; ++c) g += part[(size_t)c * n + j];
  g *= sc.grad_scale;
  float mi = m[j], vi = v[j];
  mi = mi + sc.one_minus_beta1 * (g - mi);
  vi = vi * sc.beta2 + sc.one_minus_beta2 * g * g;
  const float denom = sqrtf(vi) / sc.bc2_sqrt + sc.eps;
  a = fmaxf(a - sc.lr_step * (mi / denom), 0.f);
  if (!is_beta) a = fminf(a, 1.f);
  m[j] = mi;
  v[j] = vi;
  param[j] = a;
}

int shared_alpha_chunks(int B) { return B < 64 ? B : 64; }

int launch_shared_adam(float* param, float* m, float* v, float* grad, const int8_t* split, int split_stride, float* part,
                       const int* improve, float* best, AdamScalars sc, int do_update, int is_beta, int B, int n,
                       cudaStream_t stream) {
  const int chunks = shared_alpha_chunks(B);
  if (do_update) {
    dim3 grid(ceil_div(n, 128), chunks);
    grad_colsum_kernel<<<grid, 128, 0, stream>>>(grad, split, split_stride, part, B, n, ceil_div(B, chunks));
    BF_CHECK_LAUNCH("grad_colsum_kernel");
  }
  shared_adam_kernel<<<ceil_div(n, 128), 128, 0, stream>>>(param, m, v, part, chunks, improve, best, sc, do_update, is_beta, n);
  BF_CHECK_LAUNCH("shared_adam_kernel");
  return BF_OK;
}

// Split term of a shared beta: add[b, j] = -beta[j] * split[b, j].
__global__ void __launch_bounds__(128) shared_beta_add_kernel(const float* __restrict__ beta, const int8_t* __restrict__ split,
                                                              int split_stride, float* __restrict__ add, int n) {
  const int b = blockIdx.x;
  const int j = blockIdx.y * blockDim.x + threadIdx.x;
  if (j >= n) return;
  add[(size_t)b * n + j] = -beta[j] * (float)split[(size_t)b * split_stride + j];
}

int launch_shared_beta_add(const float* beta, const int8_t* split, int split_stride, float* add, int B, int n, cudaStream_t stream) {
  dim3 grid(B, ceil_div(n, 128));
  shared_beta_add_kernel<<<grid, 128, 0, stream>>>(beta, split, split_stride, add, n);
  BF_CHECK_LAUNCH("shared_beta_add_kernel");
  return BF_OK;
}

// ---- objective influence of a ReLU: out[b, j] = max(out[b, j], max_s |A[b, s, j]|) --------------
__global__ void __launch_bounds__(256) colmax_abs_kernel(const float* __restrict__ A, float* __restrict__ out, int S, int n) {
  const int b = blockIdx.x;
  const int j = blockIdx.y * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const float* a = A + (size_t)b * S * n + j;
  float m = out[(size_t)b * n + j];
  for (int s = 0; s < S; ++s) m = fmaxf(m, fabsf(a[(size_t)s * n]));
  out[(size_t)b * n + j] = m;
}

int launch_colmax_abs(const float* A, float* out, int B, int S, int n, cudaStream_t stream) {
  dim3 grid(B, ceil_div(n, 256));
  colmax_abs_kernel<<<grid, 256, 0, stream>>>(A, out, S, n);
  BF_CHECK_LAUNCH("colmax_abs_kernel");
  return BF_OK;
}

// ---- gradient sweep pieces for layers without a fused epilogue (conv) --------------------------------
// Adjoint step of one ReLU on rows: g = layer output at the adjoint point (in), h = d*g + e (out, in place),
// grad[b,j] += sum over the domain's rows of [unstable][Ahat >= 0] Ahat*g and, with beta parameters,
// gsum[b,j] += sum over the domain's rows of g, each row times gw[b*S+s] when gw is given (the beta gradient is
// -split * gsum; gw carries d objective / d row for min / softmin).  One thread per (domain, neuron),
// rows of the domain in order: no atomics.
__global__ void __launch_bounds__(256) relu_adjoint_rows_kernel(float* __restrict__ G, const float* __restrict__ Ahat,
                                                                const float* __restrict__ dpos, const float* __restrict__ dneg,
                                                                const float* __restrict__ eneg, const float* __restrict__ pre_l,
                                                                const float* __restrict__ pre_u, float* __restrict__ grad,
                                                                float* __restrict__ gsum, const float* __restrict__ gw, int S, int n) {
  const int b = blockIdx.x;
  const int j = blockIdx.y * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const size_t o = (size_t)b * n + j;
  const float dp = dpos[o], dn = dneg[o], en = eneg ? eneg[o] : 0.f;
  const bool amb = pre_l[o] < 0.f && pre_u[o] > 0.f;
  float acc = 0.f, gs = 0.f;
  for (int s = 0; s < S; ++s) {
    const size_t i = ((size_t)b * S + s) * n + j;
    const float a = Ahat[i], g = G[i];
    const bool sel = a >= 0.f;
    gs = gw ? fmaf(gw[(size_t)b * S + s], g, gs) : gs + g;
    if (sel && amb) acc = fmaf(a, g, acc);
    G[i] = sel ? dp * g : fmaf(dn, g, en);
  }
  grad[o] += acc;
  if (gsum) gsum[o] += gs;
}

int launch_relu_adjoint_rows(float* G, const float* Ahat, const float* dpos, const float* dneg, const float* eneg,
                             const float* pre_l, const float* pre_u, float* grad, float* gsum, int B, int S, int n,
                             cudaStream_t stream, const float* gw) {
  dim3 grid(B, ceil_div(n, 256));
  relu_adjoint_rows_kernel<<<grid, 256, 0, stream>>>(G, Ahat, dpos, dneg, eneg, pre_l, pre_u, grad, gsum, gw, S, n);
  BF_CHECK_LAUNCH("relu_adjoint_rows_kernel");
  return BF_OK;
}

// Start vector of the gradient sweep for a box: h0 = mid - sgn(A0) * rad, written over A0.
__global__ void h0_box_kernel(float* __restrict__ A0, const float* __restrict__ mid, const float* __restrict__ rad, long long total,
                              int S, int n0) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / n0;
    const size_t o = (size_t)(m / S) * n0 + (size_t)(i - m * n0);
    const float a = A0[i];
    const float sg = (a > 0.f) ? 1.f : ((a < 0.f) ? -1.f : 0.f);
    A0[i] = mid[o] - sg * rad[o];
  }
}

int launch_h0_box(float* A0, const float* mid, const float* rad, int B, int S, int n0, cudaStream_t stream) {
  const long long total = (long long)B * S * n0;
  h0_box_kernel<<<ew_grid(total, 256), 256, 0, stream>>>(A0, mid, rad, total, S, n0);
  BF_CHECK_LAUNCH("h0_box_kernel");
  return BF_OK;
}

// ---- adaptive alpha start ------------------------------------------------------
__global__ void alpha_adaptive_init_kernel(const float* __restrict__ l, const float* __restrict__ u, float* __restrict__ alpha,
                                           long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const float lo = l[i], up = u[i];
    alpha[i] = (lo >= 0.f || (lo < 0.f && up > 0.f && up > -lo)) ? 1.f : 0.f;
  }
}

// ---- verdicts ---------------------------------------------------------------
// A NaN on any spec row poisons the minimum (fminf alone would drop it), so such a domain is never proven;
// a domain whose split assignment is empty (infeasible flag) carries meaningless bounds and is not proven either.
__global__ void verdict_kernel(const float* __restrict__ lower, float threshold, float tol, const int* __restrict__ infeasible,
                               int8_t* __restrict__ verdict, float* __restrict__ min_lower, int B, int S) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float mn = lower[(size_t)b * S];
  for (int k = 1; k < S; ++k) {
    const float v = lower[(size_t)b * S + k];
    mn = (v != v || mn != mn) ? nanf("") : fminf(mn, v);
  }
  const bool ok = (mn >= threshold - tol) && !(infeasible && infeasible[b] != 0);
  verdict[b] = ok ? 1 : 0;
  if (min_lower) min_lower[b] = mn;
}

int launch_verdict(const float* lower, float threshold, float tol, const int* infeasible, int8_t* verdict, float* min_lower,
                   int B, int S, cudaStream_t stream) {
  verdict_kernel<<<ceil_div(B, 128), 128, 0, stream>>>(lower, threshold, tol, infeasible, verdict, min_lower, B, S);
  BF_CHECK_LAUNCH("verdict_kernel");
  return BF_OK;
}

// Results of a call whose tensor-core kernels gave up on a bounded wait are undefined: when the chain's status word
// is set, every bound of the call is overwritten with NaN (which no verdict accepts) instead of being handed on.
__global__ void poison_on_status_kernel(const int* __restrict__ status, float* __restrict__ a, long long na,
                                        float* __restrict__ b, long long nb) {
  if (*status == 0) return;
  const float bad = nanf("");
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < na + nb; i += (long long)gridDim.x * blockDim.x) {
    if (i < na) a[i] = bad;
    else b[i - na] = bad;
  }
}

int launch_poison_on_status(const int* status, float* a, long long na, float* b, long long nb, cudaStream_t stream) {
  if (!status || (!a && !b)) return BF_OK;
  if (!a) na = 0;
  if (!b) nb = 0;
  poison_on_status_kernel<<<ew_grid(na + nb, 256), 256, 0, stream>>>(status, a, na, b, nb);
  BF_CHECK_LAUNCH("poison_on_status_kernel");
  return BF_OK;
}

}  // namespace bf

// ---- small interval / coefficient helpers for graphs that are not chains --------------------------
namespace bf {
__global__ void interval_relu_kernel(const float* __restrict__ l, const float* __restrict__ u, float* __restrict__ ol,
                                     float* __restrict__ ou, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    ol[i] = fmaxf(l[i], 0.f);
    ou[i] = fmaxf(u[i], 0.f);
  }
}
__global__ void interval_add_kernel(const float* __restrict__ al, const float* __restrict__ au, const float* __restrict__ bl,
                                    const float* __restrict__ bu, float* __restrict__ ol, float* __restrict__ ou, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    ol[i] = al[i] + bl[i];
    ou[i] = au[i] + bu[i];
  }
}
// Interval product: the smallest and largest of the four corner products (domains/interval.py:102-112).
__global__ void interval_mul_kernel(const float* __restrict__ al, const float* __restrict__ au, const float* __restrict__ bl,
                                    const float* __restrict__ bu, float* __restrict__ ol, float* __restrict__ ou, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float p0 = al[i] * bl[i], p1 = al[i] * bu[i], p2 = au[i] * bl[i], p3 = au[i] * bu[i];
    ol[i] = fminf(fminf(p0, p1), fminf(p2, p3));
    ou[i] = fmaxf(fmaxf(p0, p1), fmaxf(p2, p3));
  }
}
__global__ void accumulate_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dst[i] += src[i];
}
}  // namespace bf

extern "C" int bf_interval_relu(const float* l, const float* u, float* out_l, float* out_u, long long n, bf_stream_t stream) {
  BF_REQUIRE(l && u && out_l && out_u && n > 0, BF_E_INVALID, "bf_interval_relu: bad argument");
  bf::interval_relu_kernel<<<bf::ew_grid(n, 256), 256, 0, bf::as_stream(stream)>>>(l, u, out_l, out_u, n);
  BF_CHECK_LAUNCH("interval_relu_kernel");
  return BF_OK;
}

extern "C" int bf_interval_add(const float* a_l, const float* a_u, const float* b_l, const float* b_u, float* out_l, float* out_u,
                               long long n, bf_stream_t stream) {
  BF_REQUIRE(a_l && a_u && b_l && b_u && out_l && out_u && n > 0, BF_E_INVALID, "bf_interval_add: bad argument");
  bf::interval_add_kernel<<<bf::ew_grid(n, 256), 256, 0, bf::as_stream(stream)>>>(a_l, a_u, b_l, b_u, out_l, out_u, n);
  BF_CHECK_LAUNCH("interval_add_kernel");
  return BF_OK;
}

extern "C" int bf_interval_mul(const float* a_l, const float* a_u, const float* b_l, const float* b_u, float* out_l, float* out_u,
                               long long n, bf_stream_t stream) {
  BF_REQUIRE(a_l && a_u && b_l && b_u && out_l && out_u && n > 0, BF_E_INVALID, "bf_interval_mul: bad argument");
  bf::interval_mul_kernel<<<bf::ew_grid(n, 256), 256, 0, bf::as_stream(stream)>>>(a_l, a_u, b_l, b_u, out_l, out_u, n);
  BF_CHECK_LAUNCH("interval_mul_kernel");
  return BF_OK;
}

extern "C" int bf_accumulate(float* dst, const float* src, long long n, bf_stream_t stream) {
  BF_REQUIRE(dst && src && n > 0, BF_E_INVALID, "bf_accumulate: bad argument");
  bf::accumulate_kernel<<<bf::ew_grid(n, 256), 256, 0, bf::as_stream(stream)>>>(dst, src, n);
  BF_CHECK_LAUNCH("accumulate_kernel");
  return BF_OK;
}

extern "C" int bf_relu_relax(const float* l, const float* u, const float* alpha, int alpha_stride, float* alpha_u,
                             float* beta_u, float* alpha_l, int B, int n, bf_stream_t stream) {
  BF_REQUIRE(l && u && alpha_u && beta_u && alpha_l, BF_E_INVALID, "bf_relu_relax: null tensor");
  BF_REQUIRE(B > 0 && n > 0, BF_E_INVALID, "bf_relu_relax: sizes must be positive");
  BF_REQUIRE(!alpha || alpha_stride == 0 || alpha_stride == n, BF_E_INVALID, "bf_relu_relax: alpha_stride must be 0 or n");
  return bf::launch_relu_relax(l, u, alpha, alpha_stride, alpha_u, beta_u, alpha_l, B, n, bf::as_stream(stream));
}

extern "C" int bf_alpha_adaptive_init(const float* l, const float* u, float* alpha, int B, int n, bf_stream_t stream) {
  BF_REQUIRE(l && u && alpha, BF_E_INVALID, "bf_alpha_adaptive_init: null tensor");
  BF_REQUIRE(B > 0 && n > 0, BF_E_INVALID, "bf_alpha_adaptive_init: sizes must be positive");
  const long long total = (long long)B * n;
  bf::alpha_adaptive_init_kernel<<<bf::ew_grid(total, 256), 256, 0, bf::as_stream(stream)>>>(l, u, alpha, total);
  BF_CHECK_LAUNCH("alpha_adaptive_init_kernel");
  return BF_OK;
}

extern "C" int bf_concretize(const float* A, const float* mid, const float* rad, const float* bias_in, float* out, int side,
                             int B, int S, int n0, bf_stream_t stream) {
  BF_REQUIRE(A && mid && rad && out, BF_E_INVALID, "bf_concretize: null tensor");
  BF_REQUIRE(B > 0 && S > 0 && n0 > 0, BF_E_INVALID, "bf_concretize: sizes must be positive");
  BF_REQUIRE(side == BF_SIDE_LOWER || side == BF_SIDE_UPPER, BF_E_INVALID, "bf_concretize: bad side");
  BF_REQUIRE((long long)B * S < 2147483647LL, BF_E_INVALID, "bf_concretize: B*S overflows int");
  return bf::launch_concretize(A, mid, rad, bias_in, out, side, B, S, n0, bf::as_stream(stream));
}

extern "C" int bf_verdict(const float* lower, float threshold, float tol, int8_t* verdict, float* min_lower, int B, int S,
                          bf_stream_t stream) {
  return bf_verdict_masked(lower, threshold, tol, nullptr, verdict, min_lower, B, S, stream);
}

extern "C" int bf_verdict_masked(const float* lower, float threshold, float tol, const int* infeasible, int8_t* verdict,
                                 float* min_lower, int B, int S, bf_stream_t stream) {
  BF_REQUIRE(lower && verdict, BF_E_INVALID, "bf_verdict: null tensor");
  BF_REQUIRE(B > 0 && S > 0, BF_E_INVALID, "bf_verdict: sizes must be positive");
  return bf::launch_verdict(lower, threshold, tol, infeasible, verdict, min_lower, B, S, bf::as_stream(stream));
}

// ---- beta parameters (split-constraint multipliers) and branching scores -------------
namespace bf {

// gradient of the loss w.r.t. beta_j is grad_scale * (-s_j) * sum_s g[s,j]  (add_j = -beta_j * s_j enters the lower
// coefficients, d lower / d add_j = g_j); entries without a split never move.  Same Adam recurrences as alpha,
// projection to beta >= 0.
__global__ void __launch_bounds__(128) beta_step_kernel(float* __restrict__ beta, float* __restrict__ m, float* __restrict__ v,
                                                        float* __restrict__ gsum, const int8_t* __restrict__ split,
                                                        int split_stride, const int* __restrict__ improve,
                                                        float* __restrict__ best_beta, float* __restrict__ add, AdamScalars sc,
                                                        int do_update, int n) {
  const int b = blockIdx.x;
  const int j = blockIdx.y * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const size_t i = (size_t)b * n + j;
  const float s = split ? (float)split[(size_t)b * split_stride + j] : 0.f;
  float bt = beta[i];
  if (improve != nullptr && best_beta != nullptr && improve[b] != 0) best_beta[i] = bt;
  if (do_update) {
    const float g = gsum[i] * sc.grad_scale * (-s);
    gsum[i] = 0.f;
    float mi = m[i], vi = v[i];
    mi = mi + sc.one_minus_beta1 * (g - mi);
    vi = vi * sc.beta2 + sc.one_minus_beta2 * g * g;
    const float denom = sqrtf(vi) / sc.bc2_sqrt + sc.eps;
    bt = fmaxf(bt - sc.lr_step * (mi / denom), 0.f);
    m[i] = mi;
    v[i] = vi;
    beta[i] = bt;
  }
  add[i] = -bt * s;
}

int launch_beta_step(float* beta, float* m, float* v, float* gsum, const int8_t* split, int split_stride, const int* improve,
                     float* best_beta, float* add, AdamScalars sc, int do_update, int B, int n, cudaStream_t stream) {
  dim3 grid(B, ceil_div(n, 128));
  beta_step_kernel<<<grid, 128, 0, stream>>>(beta, m, v, gsum, split, split_stride, improve, best_beta, add, sc, do_update, n);
  BF_CHECK_LAUNCH("beta_step_kernel");
  return BF_OK;
}

__global__ void fill_kernel(float* __restrict__ dst, float value, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = value;
}

// Widest unstable gap of one ReLU per domain: one warp per domain, first index wins ties; the caller
// combines ReLUs in chain order with a strict comparison (earlier ReLUs win ties).
__global__ void __launch_bounds__(256) branch_score_kernel(const float* __restrict__ l, const float* __restrict__ u, int n, int B,
                                                           int relu_index, float* __restrict__ best_gap,
                                                           int* __restrict__ best_relu, int* __restrict__ best_idx) {
  const int b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  float gap = -INFINITY;
  int idx = 0x7fffffff;
  for (int j = lane; j < n; j += 32) {
    const float lo = l[(size_t)b * n + j], up = u[(size_t)b * n + j];
    if (lo < 0.f && up > 0.f) {
      const float g = fmaxf(up - lo, 0.f);
      if (g > gap) { gap = g; idx = j; }  // j increases: the first index of a tie is kept
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float og = __shfl_xor_sync(0xffffffffu, gap, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (og > gap || (og == gap && oi < idx)) { gap = og; idx = oi; }
  }
  if (lane == 0 && gap > best_gap[b]) {
    best_gap[b] = gap;
    best_relu[b] = relu_index;
    best_idx[b] = idx;
  }
}

}  // namespace bf

extern "C" int bf_branch_scores(const float* const* pre_l, const float* const* pre_u, const int* widths, int n_relu,
                                float* best_gap, int* best_relu, int* best_idx, int B, bf_stream_t stream_) {
  BF_REQUIRE(pre_l && pre_u && widths && best_gap && best_relu && best_idx, BF_E_INVALID, "bf_branch_scores: null argument");
  BF_REQUIRE(B > 0 && n_relu >= 0, BF_E_INVALID, "bf_branch_scores: bad sizes");
  cudaStream_t stream = bf::as_stream(stream_);
  // best_relu / best_idx start at -1 ("no unstable neuron"), best_gap at -inf
  if (cudaMemsetAsync(best_relu, 0xff, sizeof(int) * (size_t)B, stream) != cudaSuccess ||
      cudaMemsetAsync(best_idx, 0xff, sizeof(int) * (size_t)B, stream) != cudaSuccess) {
    bf::set_error("bf_branch_scores: cudaMemsetAsync failed");
    return BF_E_CUDA;
  }
  bf::fill_kernel<<<bf::ceil_div(B, 256), 256, 0, stream>>>(best_gap, -INFINITY, B);
  BF_CHECK_LAUNCH("fill_kernel");
  for (int r = 0; r < n_relu; ++r) {
    BF_REQUIRE(pre_l[r] && pre_u[r] && widths[r] > 0, BF_E_INVALID, "bf_branch_scores: bad ReLU %d", r);
    bf::branch_score_kernel<<<bf::ceil_div((long long)B * 32, 256), 256, 0, stream>>>(pre_l[r], pre_u[r], widths[r], B, r, best_gap,
                                                                                  best_relu, best_idx);
    BF_CHECK_LAUNCH("branch_score_kernel");
  }
  return BF_OK;
}

// ---- building blocks for graphs that are not chains ---------------------------------------------
namespace bf {

// ReLU split on the bounds of a value: s = +1 -> l = max(l, 0); s = -1 -> u = min(u, 0); a domain with l > u
// afterwards on any neuron is flagged.  One block row per domain.
__global__ void __launch_bounds__(256) relu_split_apply_kernel(float* __restrict__ l, float* __restrict__ u,
                                                               const int8_t* __restrict__ split, int split_stride,
                                                               int* __restrict__ infeasible, int n) {
  const int b = blockIdx.x;
  bool bad = false;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < n; j += gridDim.y * blockDim.x) {
    const size_t o = (size_t)b * n + j;
    const int s = split[(size_t)b * split_stride + j];
    float lo = l[o], up = u[o];
    if (s > 0) lo = fmaxf(lo, 0.f);
    if (s < 0) up = fminf(up, 0.f);
    l[o] = lo;
    u[o] = up;
    bad |= lo > up;
  }
  if (infeasible && __syncthreads_or(bad ? 1 : 0) && threadIdx.x == 0) atomicOr(&infeasible[b], 1);
}

int launch_relu_split_apply(float* l, float* u, const int8_t* split, int split_stride, int* infeasible, int B, int n,
                            cudaStream_t stream) {
  dim3 grid(B, std::min(ceil_div(n, 256), 64));
  relu_split_apply_kernel<<<grid, 256, 0, stream>>>(l, u, split, split_stride, infeasible, n);
  BF_CHECK_LAUNCH("relu_split_apply_kernel");
  return BF_OK;
}

// Intersection of the bounds of a value with a constraint interval, in place: l = max(l, cl), u = min(u, cu); a domain
// with l > u afterwards on any neuron is flagged.  One block row per domain.
__global__ void __launch_bounds__(256) interval_intersect_kernel(float* __restrict__ l, float* __restrict__ u, const float* __restrict__ cl,
                                                                 const float* __restrict__ cu, int* __restrict__ infeasible, int n) {
  const int b = blockIdx.x;
  bool bad = false;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < n; j += gridDim.y * blockDim.x) {
    const size_t o = (size_t)b * n + j;
    const float lo = fmaxf(l[o], cl[o]), up = fminf(u[o], cu[o]);
    l[o] = lo;
    u[o] = up;
    bad |= lo > up;
  }
  if (infeasible && __syncthreads_or(bad ? 1 : 0) && threadIdx.x == 0) atomicOr(&infeasible[b], 1);
}

int launch_interval_intersect(float* l, float* u, const float* cl, const float* cu, int* infeasible, int B, int n, cudaStream_t stream) {
  dim3 grid(B, std::min(ceil_div(n, 256), 64));
  interval_intersect_kernel<<<grid, 256, 0, stream>>>(l, u, cl, cu, infeasible, n);
  BF_CHECK_LAUNCH("interval_intersect_kernel");
  return BF_OK;
}

// A[b, s, :] += v[b, :] (v_stride = n) or += v[:] (v_stride = 0)
__global__ void rows_add_broadcast_kernel(float* __restrict__ A, const float* __restrict__ v, int v_stride, long long total, int S,
                                          int n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / n;
    A[i] += v[(size_t)(m / S) * v_stride + (size_t)(i - m * n)];
  }
}

int launch_rows_add_broadcast(float* A, const float* v, int v_stride, int B, int S, int n, cudaStream_t stream) {
  const long long total = (long long)B * S * n;
  rows_add_broadcast_kernel<<<ew_grid(total, 256), 256, 0, stream>>>(A, v, v_stride, total, S, n);
  BF_CHECK_LAUNCH("rows_add_broadcast_kernel");
  return BF_OK;
}

}  // namespace bf
