// Conv2d layers (NCHW activations, OIHW weights, groups = 1, dilation = 1):
// interval propagation in centre/radius form and the CROWN backward transformer
// (ReLU backward + transposed convolution of the coefficient rows).
#include "kernels.cuh"

namespace bf {

// ---------------------------------------------------------------------------
// IBP conv2d: one thread per output element; weights are warp-uniform loads
// (a warp covers consecutive output columns of one output channel).
// ---------------------------------------------------------------------------
struct IbpConvArgs {
  const float* in_a; const float* in_b; int in_mode; int relu_in;
  const float* W; const float* bias;
  const int8_t* split; int split_stride;
  const float* cons_l; const float* cons_u;
  float* out_l; float* out_u; int* infeasible;
  int B, Ci, Hi, Wi, Co, Ho, Wo, kh, kw, sh, sw, ph, pw;
};

__global__ void __launch_bounds__(256) ibp_conv2d_kernel(IbpConvArgs g) {
  const long long n_out = (long long)g.Co * g.Ho * g.Wo;
  const long long total = (long long)g.B * n_out;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int wo = (int)(idx % g.Wo);
    const int ho = (int)((idx / g.Wo) % g.Ho);
    const int co = (int)((idx / ((long long)g.Wo * g.Ho)) % g.Co);
    const int b = (int)(idx / n_out);
    float accC = 0.f, accR = 0.f;
    const int h0 = ho * g.sh - g.ph, w0 = wo * g.sw - g.pw;
    for (int ci = 0; ci < g.Ci; ++ci) {
      const float* wa = g.W + ((size_t)co * g.Ci + ci) * g.kh * g.kw;
      const size_t in_off = ((size_t)b * g.Ci + ci) * g.Hi * g.Wi;
      for (int r = 0; r < g.kh; ++r) {
        const int hi = h0 + r;
        if (hi < 0 || hi >= g.Hi) continue;
        for (int s = 0; s < g.kw; ++s) {
          const int wi = w0 + s;
          if (wi < 0 || wi >= g.Wi) continue;
          const float w = __ldg(wa + r * g.kw + s);
          float a = __ldg(g.in_a + in_off + (size_t)hi * g.Wi + wi);
          float bb = __ldg(g.in_b + in_off + (size_t)hi * g.Wi + wi);
          float c, rad;
          if (g.in_mode == BF_IN_LOWER_UPPER) {
            if (g.relu_in) { a = fmaxf(a, 0.f); bb = fmaxf(bb, 0.f); }
            c = (a + bb) * 0.5f;
            rad = (bb - a) * 0.5f;
          } else {
            c = a;
            rad = bb;
          }
          accC = fmaf(c, w, accC);
          accR = fmaf(rad, fabsf(w), accR);
        }
      }
    }
    const float bias = g.bias ? __ldg(g.bias + co) : 0.f;
    float lo = (accC - accR) + bias, up = (accC + accR) + bias;
    const long long j = idx - (long long)b * n_out;
    bool bad = false;
    if (g.cons_l) {
      lo = fmaxf(lo, g.cons_l[idx]);
      up = fminf(up, g.cons_u[idx]);
      bad |= lo > up;
    }
    if (g.split) {
      const int s = g.split[(size_t)b * g.split_stride + j];
      if (s > 0) lo = fmaxf(lo, 0.f);
      if (s < 0) up = fminf(up, 0.f);
      bad |= lo > up;
    }
    g.out_l[idx] = lo;
    g.out_u[idx] = up;
    if (bad && g.infeasible) g.infeasible[b] = 1;
  }
}

int launch_ibp_conv2d(const float* in_a, const float* in_b, int in_mode, int relu_in, const float* W, const float* bias,
                      const int8_t* split, int split_stride, const float* cons_l, const float* cons_u, float* out_l,
                      float* out_u, int* infeasible, int B, const bf_layer_desc& L, cudaStream_t stream) {
  IbpConvArgs g{in_a, in_b, in_mode, relu_in, W, bias, split, split_stride, cons_l, cons_u, out_l, out_u, infeasible,
                B, L.Ci, L.Hi, L.Wi, L.Co, L.Ho, L.Wo, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw};
  const long long total = (long long)B * L.Co * L.Ho * L.Wo;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  ibp_conv2d_kernel<<<(int)blocks, 256, 0, stream>>>(g);
  BF_CHECK_LAUNCH("ibp_conv2d_kernel");
  return BF_OK;
}

// ---------------------------------------------------------------------------
// ReLU backward on coefficient rows (one warp per row), used in front of the
// transposed convolution:  Lam = A * slope_sel ; delta (+)= sum A*icpt_sel + Lam*bias[channel]
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) relu_bwd_rows_kernel(const float* __restrict__ A, const float* __restrict__ dpos,
                                                            const float* __restrict__ dneg, const float* __restrict__ epos,
                                                            const float* __restrict__ eneg, const float* __restrict__ bias,
                                                            int chan_size, float* __restrict__ Lam, float* __restrict__ delta,
                                                            int accumulate, int M, int S, int n) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int m = warp; m < M; m += nwarps) {
    const float* a = A + (size_t)m * n;
    const size_t off = (size_t)(m / S) * n;
    float acc = 0.f;
    for (int k = lane; k < n; k += 32) {
      const float v = a[k];
      float lam = v;
      if (dpos) {
        const bool sel = v >= 0.f;
        lam = v * (sel ? dpos[off + k] : dneg[off + k]);
        const float e = sel ? (epos ? epos[off + k] : 0.f) : (eneg ? eneg[off + k] : 0.f);
        acc = fmaf(v, e, acc);
      }
      if (bias) acc = fmaf(lam, __ldg(bias + k / chan_size), acc);
      if (Lam) Lam[(size_t)m * n + k] = lam;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0 && delta) delta[m] = accumulate ? (delta[m] + acc) : acc;
  }
}

// ---------------------------------------------------------------------------
// Transposed convolution of coefficient rows (gather form): one thread per
// (row, input pixel) accumulating ACC input channels in registers; the weight
// slice W[co0:co0+CO_CHUNK, ci0:ci0+ACC, :, :] is staged in shared memory with
// the input channel innermost so that one 128-bit read feeds four FMAs.
// ---------------------------------------------------------------------------
struct ConvTArgs {
  const float* Lam;  // [M, Co, Ho, Wo]
  const float* W;    // [Co, Ci, kh, kw]
  float* out;        // [M, Ci, Hi, Wi]
  int M, Ci, Hi, Wi, Co, Ho, Wo, kh, kw, sh, sw, ph, pw;
  int co_chunk;
};

template <int ACC>
__global__ void __launch_bounds__(256) conv_transpose_rows_kernel(ConvTArgs g) {
  extern __shared__ __align__(16) float wsm[];  // [co_chunk][kh][kw][ACC]
  const int m = blockIdx.x;
  const int pix = blockIdx.y * blockDim.x + threadIdx.x;
  const int ci0 = blockIdx.z * ACC;
  const int npix = g.Hi * g.Wi;
  const bool active = pix < npix;
  const int hi = active ? pix / g.Wi : 0, wi = active ? pix % g.Wi : 0;
  float acc[ACC];
#pragma unroll
  for (int c = 0; c < ACC; ++c) acc[c] = 0.f;
  const int taps = g.kh * g.kw;
  const float* lam_m = g.Lam + (size_t)m * g.Co * g.Ho * g.Wo;

  for (int co0 = 0; co0 < g.Co; co0 += g.co_chunk) {
    const int nco = min(g.co_chunk, g.Co - co0);
    __syncthreads();
    for (int e = threadIdx.x; e < nco * taps * ACC; e += blockDim.x) {
      const int c = e % ACC;
      const int t = (e / ACC) % taps;
      const int co = e / (ACC * taps);
      const int ci = ci0 + c;
      wsm[e] = (ci < g.Ci) ? __ldg(g.W + ((size_t)(co0 + co) * g.Ci + ci) * taps + t) : 0.f;
    }
    __syncthreads();
    if (!active) continue;
    for (int r = 0; r < g.kh; ++r) {
      const int hn = hi + g.ph - r;
      if (hn < 0 || hn % g.sh != 0) continue;
      const int ho = hn / g.sh;
      if (ho >= g.Ho) continue;
      for (int s = 0; s < g.kw; ++s) {
        const int wn = wi + g.pw - s;
        if (wn < 0 || wn % g.sw != 0) continue;
        const int wo = wn / g.sw;
        if (wo >= g.Wo) continue;
        const float* lp = lam_m + ((size_t)co0 * g.Ho + ho) * g.Wo + wo;
        const float* wp = wsm + (r * g.kw + s) * ACC;
        for (int co = 0; co < nco; ++co) {
          const float v = lp[(size_t)co * g.Ho * g.Wo];
          const float4* w4 = reinterpret_cast<const float4*>(wp + (size_t)co * taps * ACC);
#pragma unroll
          for (int c = 0; c < ACC / 4; ++c) {
            const float4 w = w4[c];
            acc[4 * c + 0] = fmaf(v, w.x, acc[4 * c + 0]);
            acc[4 * c + 1] = fmaf(v, w.y, acc[4 * c + 1]);
            acc[4 * c + 2] = fmaf(v, w.z, acc[4 * c + 2]);
            acc[4 * c + 3] = fmaf(v, w.w, acc[4 * c + 3]);
          }
        }
      }
    }
  }
  if (!active) return;
#pragma unroll
  for (int c = 0; c < ACC; ++c) {
    const int ci = ci0 + c;
    if (ci < g.Ci) g.out[((size_t)m * g.Ci + ci) * npix + pix] = acc[c];
  }
}

size_t crown_bwd_conv2d_scratch_bytes(int M, const bf_layer_desc& L) { return (size_t)M * L.n_out * sizeof(float); }

template <int ACC>
static int launch_convT(const ConvTArgs& g0, cudaStream_t stream) {
  ConvTArgs g = g0;
  const int taps = g.kh * g.kw;
  int co_chunk = (64 * 1024) / (taps * ACC * (int)sizeof(float));
  if (co_chunk < 1) co_chunk = 1;
  if (co_chunk > g.Co) co_chunk = g.Co;
  g.co_chunk = co_chunk;
  const int smem = co_chunk * taps * ACC * (int)sizeof(float);
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(conv_transpose_rows_kernel<ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    attr_done = true;
  }
  BF_REQUIRE(smem <= 96 * 1024, BF_E_UNSUPPORTED, "conv backward: kernel window of %d taps is too large", taps);
  const int npix = g.Hi * g.Wi;
  const int threads = npix >= 256 ? 256 : ((npix + 31) / 32) * 32;
  dim3 grid(g.M, ceil_div(npix, threads), ceil_div(g.Ci, ACC));
  BF_REQUIRE(grid.y <= 65535 && grid.z <= 65535, BF_E_UNSUPPORTED, "conv backward: feature map too large");
  conv_transpose_rows_kernel<ACC><<<grid, threads, smem, stream>>>(g);
  BF_CHECK_LAUNCH("conv_transpose_rows_kernel");
  return BF_OK;
}

int launch_crown_bwd_conv2d(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                            const float* W, const float* bias, float* A_prev, float* delta, int accumulate, int M, int S,
                            const bf_layer_desc& L, void* scratch, cudaStream_t stream) {
  const float* lam = A;
  const bool need_pro = (dpos != nullptr) || (bias != nullptr) || (delta != nullptr && !accumulate);
  if (need_pro) {
    float* lam_out = dpos ? static_cast<float*>(scratch) : nullptr;
    BF_REQUIRE(!dpos || scratch, BF_E_WORKSPACE, "conv backward: scratch missing");
    int blocks = ceil_div(M, 8);
    if (blocks > 148 * 8) blocks = 148 * 8;
    relu_bwd_rows_kernel<<<blocks, 256, 0, stream>>>(A, dpos, dneg, epos, eneg, bias, L.Ho * L.Wo, lam_out, delta, accumulate,
                                                    M, S, L.n_out);
    BF_CHECK_LAUNCH("relu_bwd_rows_kernel");
    if (dpos) lam = lam_out;
  }
  if (!A_prev) return BF_OK;
  ConvTArgs g{lam, W, A_prev, M, L.Ci, L.Hi, L.Wi, L.Co, L.Ho, L.Wo, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, 0};
  if (L.Ci <= 4) return launch_convT<4>(g, stream);
  if (L.Ci <= 16) return launch_convT<16>(g, stream);
  return launch_convT<32>(g, stream);
}

}  // namespace bf

extern "C" int bf_ibp_conv2d(const float* in_a, const float* in_b, int in_mode, int relu_in, const float* W,
                             const float* bias, const int8_t* split, int split_stride, const float* cons_l,
                             const float* cons_u, float* out_l, float* out_u, int* infeasible, int B, int Ci, int Hi,
                             int Wi, int Co, int kh, int kw, int sh, int sw, int ph, int pw, bf_stream_t stream) {
  BF_REQUIRE(in_a && in_b && W && out_l && out_u, BF_E_INVALID, "bf_ibp_conv2d: null tensor");
  BF_REQUIRE(B > 0 && Ci > 0 && Hi > 0 && Wi > 0 && Co > 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0 && ph >= 0 && pw >= 0,
             BF_E_INVALID, "bf_ibp_conv2d: bad geometry");
  BF_REQUIRE(!(relu_in && in_mode == BF_IN_MID_RAD), BF_E_INVALID, "bf_ibp_conv2d: relu_in needs lower/upper inputs");
  BF_REQUIRE((cons_l == nullptr) == (cons_u == nullptr), BF_E_INVALID, "bf_ibp_conv2d: give both constraint tensors or none");
  bf_layer_desc L{};
  L.op = BF_OP_CONV2D; L.Ci = Ci; L.Hi = Hi; L.Wi = Wi; L.Co = Co; L.kh = kh; L.kw = kw; L.sh = sh; L.sw = sw; L.ph = ph; L.pw = pw;
  L.Ho = (Hi + 2 * ph - kh) / sh + 1;
  L.Wo = (Wi + 2 * pw - kw) / sw + 1;
  BF_REQUIRE(L.Ho > 0 && L.Wo > 0, BF_E_INVALID, "bf_ibp_conv2d: empty output");
  L.n_in = Ci * Hi * Wi; L.n_out = Co * L.Ho * L.Wo;
  BF_REQUIRE(!split || split_stride == 0 || split_stride == L.n_out, BF_E_INVALID, "bf_ibp_conv2d: split_stride must be 0 or Co*Ho*Wo");
  return bf::launch_ibp_conv2d(in_a, in_b, in_mode, relu_in, W, bias, split, split_stride, cons_l, cons_u, out_l, out_u,
                               infeasible, B, L, bf::as_stream(stream));
}

// Bytes of scratch the fused ReLU + Conv2d backward needs for the scaled coefficients.
extern "C" size_t bf_crown_relu_conv2d_bwd_scratch_bytes(int B, int S, int Co, int Ho, int Wo) {
  return (size_t)B * S * Co * Ho * Wo * sizeof(float);
}

extern "C" int bf_crown_relu_conv2d_bwd(const float* A, int side, const float* alpha_u, const float* alpha_l,
                                        const float* beta_u, const float* beta_l, const float* W, const float* bias,
                                        float* A_prev, float* delta, int accumulate, void* scratch, size_t scratch_bytes,
                                        int B, int S, int Ci, int Hi, int Wi, int Co, int Ho, int Wo, int kh, int kw, int sh,
                                        int sw, int ph, int pw, bf_stream_t stream) {
  BF_REQUIRE(A && W, BF_E_INVALID, "bf_crown_relu_conv2d_bwd: A and W must be non-null");
  BF_REQUIRE(B > 0 && S > 0 && Ci > 0 && Co > 0 && Hi > 0 && Wi > 0 && Ho > 0 && Wo > 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0,
             BF_E_INVALID, "bf_crown_relu_conv2d_bwd: bad geometry");
  BF_REQUIRE(side == BF_SIDE_LOWER || side == BF_SIDE_UPPER, BF_E_INVALID, "bf_crown_relu_conv2d_bwd: bad side");
  BF_REQUIRE(Ho == (Hi + 2 * ph - kh) / sh + 1 && Wo == (Wi + 2 * pw - kw) / sw + 1, BF_E_INVALID,
             "bf_crown_relu_conv2d_bwd: output size does not match the convolution geometry");
  BF_REQUIRE((long long)B * S < 2147483647LL, BF_E_INVALID, "bf_crown_relu_conv2d_bwd: B*S overflows int");
  const bool relu = alpha_u || alpha_l || beta_u || beta_l;
  BF_REQUIRE(!relu || (alpha_u && alpha_l), BF_E_INVALID, "bf_crown_relu_conv2d_bwd: alpha_u and alpha_l must both be given");
  BF_REQUIRE(!relu || (scratch && scratch_bytes >= bf_crown_relu_conv2d_bwd_scratch_bytes(B, S, Co, Ho, Wo)), BF_E_WORKSPACE,
             "bf_crown_relu_conv2d_bwd: scratch of %zu bytes needed", bf_crown_relu_conv2d_bwd_scratch_bytes(B, S, Co, Ho, Wo));
  const float *dpos = nullptr, *dneg = nullptr, *epos = nullptr, *eneg = nullptr;
  if (relu) {
    if (side == BF_SIDE_LOWER) { dpos = alpha_l; dneg = alpha_u; epos = beta_l; eneg = beta_u; }
    else { dpos = alpha_u; dneg = alpha_l; epos = beta_u; eneg = beta_l; }
  }
  bf_layer_desc L{};
  L.op = BF_OP_CONV2D; L.Ci = Ci; L.Hi = Hi; L.Wi = Wi; L.Co = Co; L.Ho = Ho; L.Wo = Wo; L.kh = kh; L.kw = kw;
  L.sh = sh; L.sw = sw; L.ph = ph; L.pw = pw; L.n_in = Ci * Hi * Wi; L.n_out = Co * Ho * Wo;
  return bf::launch_crown_bwd_conv2d(A, dpos, dneg, epos, eneg, W, bias, A_prev, delta, accumulate, B * S, S, L, scratch,
                                     bf::as_stream(stream));
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the fused ReLU + Conv2d backward.
//
// Some callers cannot obtain device memory at the moment they need this kernel:
// a verification service whose device pool is sized at start-up and then
// frozen, a plugin loaded into a process that already owns all device memory,
// or a host runtime that forbids cudaMalloc / cudaFree on its request path
// because those calls synchronise the whole device.
// For them the scratch that holds the ReLU-scaled coefficients lives in a
// fixed-size array inside the library image instead of a caller buffer.
// ---------------------------------------------------------------------------
#define BF_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)
static __device__ __align__(256) unsigned char g_noalloc_scratch[BF_NOALLOC_SCRATCH_BYTES];

// In host code the array's name is only a handle; the device address is resolved
// once per device (with that device current) and cached here.
static void* g_noalloc_scratch_addr[64] = {nullptr};

extern "C" size_t bf_crown_relu_conv2d_bwd_noalloc_max_bytes(void) { return (size_t)BF_NOALLOC_SCRATCH_BYTES; }

extern "C" int bf_crown_relu_conv2d_bwd_noalloc(const float* A, int side, const float* alpha_u, const float* alpha_l,
                                                const float* beta_u, const float* beta_l, const float* W, const float* bias,
                                                float* A_prev, float* delta, int accumulate, int B, int S, int Ci, int Hi,
                                                int Wi, int Co, int Ho, int Wo, int kh, int kw, int sh, int sw, int ph, int pw,
                                                bf_stream_t stream) {
  BF_REQUIRE(B > 0 && S > 0 && Co > 0 && Ho > 0 && Wo > 0, BF_E_INVALID, "bf_crown_relu_conv2d_bwd_noalloc: bad geometry");
  const size_t need = bf_crown_relu_conv2d_bwd_scratch_bytes(B, S, Co, Ho, Wo);
  BF_REQUIRE(need <= (size_t)BF_NOALLOC_SCRATCH_BYTES, BF_E_WORKSPACE,
             "bf_crown_relu_conv2d_bwd_noalloc: B*S*Co*Ho*Wo*4 = %zu bytes exceeds the built-in scratch of %u bytes; "
             "use bf_crown_relu_conv2d_bwd with a caller buffer",
             need, BF_NOALLOC_SCRATCH_BYTES);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    bf::set_error("bf_crown_relu_conv2d_bwd_noalloc: cannot identify the current device");
    return BF_E_CUDA;
  }
  void* scratch = g_noalloc_scratch_addr[dev];
  if (scratch == nullptr) {
    // first call on this device: resolve the symbol's device address (do this before any stream capture)
    cudaError_t e = cudaGetSymbolAddress(&scratch, g_noalloc_scratch);
    if (e != cudaSuccess || scratch == nullptr) {
      bf::set_error("bf_crown_relu_conv2d_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return BF_E_CUDA;
    }
    g_noalloc_scratch_addr[dev] = scratch;
  }
  return bf_crown_relu_conv2d_bwd(A, side, alpha_u, alpha_l, beta_u, beta_l, W, bias, A_prev, delta, accumulate, scratch,
                                  (size_t)BF_NOALLOC_SCRATCH_BYTES, B, S, Ci, Hi, Wi, Co, Ho, Wo, kh, kw, sh, sw, ph, pw, stream);
}
