// Conv2d layers (NCHW activations, OIHW weights, groups = 1, dilation = 1):
// interval propagation in centre/radius form and the CROWN backward transformer
// (ReLU backward + transposed convolution of the coefficient rows).
#include "kernels.cuh"

namespace bf {

// ---------------------------------------------------------------------------
// IBP conv2d: one thread per output element; weights are warp-uniform loads
// (a warp covers consecutive output columns of one output channel).
// ---------------------------------------------------------------------------
struct ConvGeom {
  int Ci, Hi, Wi, Co, Ho, Wo, kh, kw, sh, sw, ph, pw;
};

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
  timing_begin(T_IBP_CONV, stream);
  ibp_conv2d_kernel<<<(int)blocks, 256, 0, stream>>>(g);
  timing_end(T_IBP_CONV, stream, 4.0 * ((double)L.Co * L.Ci * L.kh * L.kw + L.Co) + 8.0 * (double)B * (L.n_in + L.n_out),
             4.0 * (double)total * L.Ci * L.kh * L.kw);
  BF_CHECK_LAUNCH("ibp_conv2d_kernel");
  return BF_OK;
}

// ---------------------------------------------------------------------------
// Forward convolution of rows (the gradient sweep of the alpha optimiser pushes its adjoint
// points through the layers in forward direction): out[m] = conv2d(in[m], W) + bias, one thread
// per output element.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) conv_forward_rows_kernel(const float* __restrict__ in, const float* __restrict__ W,
                                                                const float* __restrict__ bias, float* __restrict__ out,
                                                                long long total, ConvGeom g) {
  const long long n_out = (long long)g.Co * g.Ho * g.Wo;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int wo = (int)(idx % g.Wo);
    const int ho = (int)((idx / g.Wo) % g.Ho);
    const int co = (int)((idx / ((long long)g.Wo * g.Ho)) % g.Co);
    const long long m = idx / n_out;
    const int h0 = ho * g.sh - g.ph, w0 = wo * g.sw - g.pw;
    float acc = 0.f;
    for (int ci = 0; ci < g.Ci; ++ci) {
      const float* wa = W + ((size_t)co * g.Ci + ci) * g.kh * g.kw;
      const float* ip = in + ((size_t)m * g.Ci + ci) * g.Hi * g.Wi;
      for (int r = 0; r < g.kh; ++r) {
        const int hi = h0 + r;
        if (hi < 0 || hi >= g.Hi) continue;
        for (int sc = 0; sc < g.kw; ++sc) {
          const int wi = w0 + sc;
          if (wi < 0 || wi >= g.Wi) continue;
          acc = fmaf(__ldg(ip + (size_t)hi * g.Wi + wi), __ldg(wa + r * g.kw + sc), acc);
        }
      }
    }
    out[idx] = acc + (bias ? __ldg(bias + co) : 0.f);
  }
}

int launch_conv_forward_rows(const float* in, const float* W, const float* bias, float* out, int M, const bf_layer_desc& L,
                             cudaStream_t stream) {
  ConvGeom g{L.Ci, L.Hi, L.Wi, L.Co, L.Ho, L.Wo, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw};
  const long long total = (long long)M * L.n_out;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  conv_forward_rows_kernel<<<(int)blocks, 256, 0, stream>>>(in, W, bias, out, total, g);
  BF_CHECK_LAUNCH("conv_forward_rows_kernel");
  return BF_OK;
}

// ---------------------------------------------------------------------------
// ReLU backward on coefficient rows, in front of the transposed convolution:
//   Lam = A * slope_sel (+ add, the split term of beta-CROWN) ;  delta (+)= sum_k A*icpt_sel + Lam*bias[channel]
// grid (row, column chunk): a block streams RELU_ROWS_CHUNK columns of one row
// and leaves one partial sum (fixed summation order); sum_partials_kernel adds
// the chunks of a row.
// ---------------------------------------------------------------------------
constexpr int RELU_ROWS_CHUNK = 4096;

__global__ void __launch_bounds__(256) relu_bwd_rows_kernel(const float* __restrict__ A, const float* __restrict__ dpos,
                                                            const float* __restrict__ dneg, const float* __restrict__ epos,
                                                            const float* __restrict__ eneg, const float* __restrict__ add,
                                                            const float* __restrict__ bias, int chan_size,
                                                            float* __restrict__ Lam, float* __restrict__ partial,
                                                            float* __restrict__ delta, int accumulate, int chunk, int S, int n,
                                                            int vec) {
  const int m = blockIdx.x;
  const int k0 = blockIdx.y * chunk;
  const int k1 = min(n, k0 + chunk);
  const float* a = A + (size_t)m * n;
  const size_t off = (size_t)(m / S) * n;
  float acc = 0.f;
  if (vec) {  // n % 4 == 0 and 16-byte aligned rows: four columns per access
    for (int k = k0 + 4 * (int)threadIdx.x; k < k1; k += 4 * 256) {
      const float4 v4 = *reinterpret_cast<const float4*>(a + k);
      float v[4] = {v4.x, v4.y, v4.z, v4.w};
      float lam[4] = {v4.x, v4.y, v4.z, v4.w};
      if (dpos) {
        const float4 p4 = *reinterpret_cast<const float4*>(dpos + off + k), n4 = *reinterpret_cast<const float4*>(dneg + off + k);
        const float p[4] = {p4.x, p4.y, p4.z, p4.w}, q[4] = {n4.x, n4.y, n4.z, n4.w};
        float ep[4] = {0.f, 0.f, 0.f, 0.f}, en[4] = {0.f, 0.f, 0.f, 0.f};
        if (epos) { const float4 e4 = *reinterpret_cast<const float4*>(epos + off + k); ep[0] = e4.x; ep[1] = e4.y; ep[2] = e4.z; ep[3] = e4.w; }
        if (eneg) { const float4 e4 = *reinterpret_cast<const float4*>(eneg + off + k); en[0] = e4.x; en[1] = e4.y; en[2] = e4.z; en[3] = e4.w; }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const bool sel = v[c] >= 0.f;
          lam[c] = v[c] * (sel ? p[c] : q[c]);
          acc = fmaf(v[c], sel ? ep[c] : en[c], acc);
        }
        if (add) {
          const float4 a4 = *reinterpret_cast<const float4*>(add + off + k);
          lam[0] += a4.x; lam[1] += a4.y; lam[2] += a4.z; lam[3] += a4.w;
        }
      }
      if (bias) {
        int ch = k / chan_size, rem = k - ch * chan_size;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          acc = fmaf(lam[c], __ldg(bias + ch), acc);
          if (++rem == chan_size) { rem = 0; ++ch; }
        }
      }
      if (Lam) *reinterpret_cast<float4*>(Lam + (size_t)m * n + k) = make_float4(lam[0], lam[1], lam[2], lam[3]);
    }
  } else {
    for (int k = k0 + (int)threadIdx.x; k < k1; k += 256) {
      const float v = a[k];
      float lam = v;
      if (dpos) {
        const bool sel = v >= 0.f;
        lam = v * (sel ? dpos[off + k] : dneg[off + k]);
        const float e = sel ? (epos ? epos[off + k] : 0.f) : (eneg ? eneg[off + k] : 0.f);
        acc = fmaf(v, e, acc);
        if (add) lam += add[off + k];
      }
      if (bias) acc = fmaf(lam, __ldg(bias + k / chan_size), acc);
      if (Lam) Lam[(size_t)m * n + k] = lam;
    }
  }
  if (!partial && !delta) return;
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w];
    if (partial) partial[(size_t)m * gridDim.y + blockIdx.y] = t;   // several chunks per row: summed by sum_partials_kernel
    else delta[m] = accumulate ? (delta[m] + t) : t;                // one block per row
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

// ---------------------------------------------------------------------------
// Transposed convolution, row-segment form, for square kernels with equal stride and padding
// in both directions (KS, ST, PD compile-time).  A thread owns a segment of 16 consecutive
// input-image pixels of one image row for TCI input channels (16*TCI accumulators).  The lanes
// of a warp are 32 different segments (image rows, or rows of further coefficient rows when the
// image is small) of the same channel group: a coefficient read is one conflict-free 16-byte
// word per lane, a weight read is a broadcast.  Per output channel and kernel row a thread loads
// the NL coefficient words its segment can touch and the KS*TCI weights, and does
// 16*KS*TCI/ST multiply-adds on registers (all indices compile-time).  The block stages, per
// chunk of cc output channels, the zero-padded coefficient tiles [MR][cc][LH][NLT] and the weights
// [cc][KS*KS][CIB] with cp.async into one of two buffers while it computes on the other.
// ---------------------------------------------------------------------------
// VEC: the coefficient tile starts on a 16-byte boundary of the image row (SH extra columns on the
// left) so that it can be staged with 16-byte copies; needs Wo % 4 == 0.
template <int KS, int ST, int PD, bool VEC, int TWP = 16>
struct RowSeg {
  static constexpr int TW = TWP;                              // pixels per thread (16, or 8 for narrow windows)
  static constexpr int C0 = (KS - 1 - PD + ST - 1) / ST;       // coefficient columns left of the segment's first pixel
  static constexpr int SH = VEC ? ((C0 + 3) / 4 * 4 - C0) : 0;
  static constexpr int C0E = C0 + SH;
  static constexpr int NL = (((TW - 1 + PD) / ST + C0E + 1) + 3) / 4 * 4;
  static constexpr int Q0 = SH / 4;                           // first 16-byte word of a row that holds a needed column
  static_assert(PD <= KS - 1 && TW % ST == 0 && (TW / ST) % 4 == 0, "unsupported geometry");
  // row pitch: a multiple of 4 words whose count of 16-byte words is odd, so that the 16-byte reads of
  // eight consecutive tile rows (a quarter warp) fall into different bank groups
  __host__ __device__ static int tile_w(int sx) {
    const int w4 = (((TW * sx - 1 + PD) / ST + C0E + 1) + 3) / 4;
    return 4 * (w4 | 1);
  }
  __host__ __device__ static int tile_h(int th) { return (th - 1 + PD) / ST + C0 + 1; }
};

struct RowSegArgs {
  ConvTArgs c;
  int sxl;      // log2 of the 16-pixel segments per image row in a block
  int thl;      // log2 of the image rows per block
  int mrl;      // log2 of the coefficient rows per block  (2^(sxl+thl+mrl) segments = 256 / channel groups)
  int cigl;     // log2 of the channel groups per block (TCI channels each)
  int cc;       // output channels staged per chunk (divides Co)
  int tiles_x, tiles_y;
  int rowl;     // log2 of the threads that copy one coefficient-tile row while staging
};

// Asynchronous global->shared copies; `ok == false` writes zeros instead (src is not read).
__device__ __forceinline__ void cp_async_f32(float* smem_dst, const float* gsrc, bool ok) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int bytes = ok ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_f32x4(float* smem_dst, const float* gsrc, bool ok) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int bytes = ok ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int KS, int ST, int PD, int TCI, bool VEC, int TWP>
__global__ void __launch_bounds__(256, (TCI > 1 && TWP > 8 ? 2 : 3)) conv_transpose_rowseg_kernel(RowSegArgs a) {
  using G = RowSeg<KS, ST, PD, VEC, TWP>;
  extern __shared__ __align__(16) float rs_smem[];
  const ConvTArgs& g = a.c;
  const int sx = 1 << a.sxl, th = 1 << a.thl, MR = 1 << a.mrl;
  const int cibl = a.cigl + (TCI == 4 ? 2 : 0);
  const int cib = 1 << cibl;                             // input channels per block
  const int cc = a.cc;
  const int LH = G::tile_h(th), NLT = G::tile_w(sx);
  const int tile = LH * NLT;
  const int nrows = MR * cc * LH;                        // coefficient-tile rows per chunk
  const int lam_words = nrows * NLT;                     // [MR][cc][LH][NLT]
  const int w_row = KS * cib + 4;                        // one kernel row of weights + 16 bytes: rows r and r+1 (image rows of
                                                         // different parity read them in one instruction) fall into different banks
  const int w_words = (cc * KS * w_row + 3) & ~3;        // [cc][KS][KS*cib + 4], padded so that the second buffer stays 16-byte aligned
  const int buf_words = lam_words + w_words;
  constexpr int ROW_ZERO = -2147483647 - 1;
  int* row_off = reinterpret_cast<int*>(rs_smem + 2 * buf_words);  // [nrows] source offset of each tile row, ROW_ZERO: all zeros
  const int m0 = blockIdx.x << a.mrl;
  const int h0 = (blockIdx.y / a.tiles_x) << a.thl;
  const int w0 = (blockIdx.y % a.tiles_x) * (G::TW * sx);
  const int ci0 = blockIdx.z << cibl;
  const int nsegl = a.sxl + a.thl + a.mrl;
  const int seg = threadIdx.x & ((1 << nsegl) - 1);
  const int cig = threadIdx.x >> nsegl;
  const int hi = h0 + (seg & (th - 1));                 // lanes of a warp: consecutive image rows
  const int colseg = (seg >> a.thl) & (sx - 1);
  const int mr = seg >> (a.sxl + a.thl);
  const int ho_lo = h0 / ST - G::C0;
  const int wo_lo = w0 / ST - G::C0E;
  const int howo = g.Ho * g.Wo;
  const size_t lam_row = (size_t)g.Co * howo;
  const bool row_ok = hi < g.Hi && (w0 + colseg * G::TW) < g.Wi && (m0 + mr) < g.M;

  // source offset (floats, relative to the block's first coefficient row and the chunk's first output channel)
  for (int row = threadIdx.x; row < nrows; row += 256) {
    const int hl = row % LH, cm = row / LH;
    const int co = cm % cc, smr = cm / cc;
    const int ho = ho_lo + hl;
    const bool ok = (m0 + smr < g.M) && ho >= 0 && ho < g.Ho;
    row_off[row] = ok ? (int)(smr * lam_row) + co * howo + ho * g.Wo + wo_lo : ROW_ZERO;
  }
  __syncthreads();

  // staging: 2^rowl threads copy one tile row (16-byte words when VEC), 256 >> rowl rows per step
  const int rsub = threadIdx.x & ((1 << a.rowl) - 1);
  const int rrow = threadIdx.x >> a.rowl;
  const int rstep = 256 >> a.rowl;
  const int jcol = VEC ? 4 * rsub : rsub;
  const bool col_in = jcol < NLT;
  const bool col_ok = col_in && (wo_lo + jcol) >= 0 && (wo_lo + jcol) < g.Wo;  // VEC: words are all-in or all-out (Wo % 4 == 0)
  const float* lam_base = g.Lam + (size_t)m0 * lam_row;
  // weights: thread -> fixed input channel, walks (output channel, tap)
  const int wci = threadIdx.x & (cib - 1);
  const int wq0 = threadIdx.x >> cibl;
  const int wqstep = 256 >> cibl;
  const bool wci_ok = ci0 + wci < g.Ci;
  const float* w_base = g.W + (size_t)(ci0 + wci) * (KS * KS);
  auto stage = [&](int buf, int co0) {
    float* lamS = rs_smem + buf * buf_words;
    float* wS = lamS + lam_words;
    if (col_in) {
      const float* src0 = lam_base + (size_t)co0 * howo + jcol;
      for (int row = rrow; row < nrows; row += rstep) {
        const int off = row_off[row];
        const bool ok = col_ok && off != ROW_ZERO;
        if (VEC) cp_async_f32x4(lamS + row * NLT + jcol, ok ? src0 + off : g.Lam, ok);
        else cp_async_f32(lamS + row * NLT + jcol, ok ? src0 + off : g.Lam, ok);
      }
    }
    for (int q = wq0; q < cc * KS * KS; q += wqstep) {
      const int co = q / (KS * KS);
      const int t = q - co * (KS * KS), r = t / KS;
      cp_async_f32(wS + (co * KS + r) * w_row + (t - r * KS) * cib + wci, wci_ok ? w_base + (size_t)((co0 + co) * g.Ci) * (KS * KS) + (q - co * (KS * KS)) : g.W, wci_ok);
    }
    cp_async_commit();
  };

  float acc[TCI][G::TW];
#pragma unroll
  for (int c = 0; c < TCI; ++c)
#pragma unroll
    for (int i = 0; i < G::TW; ++i) acc[c][i] = 0.f;

  // kernel rows this image row meets: r = r_first + ST * jr (jr < JR, r < KS); they map to tile rows hl_top - jr
  constexpr int JR = (KS + ST - 1) / ST;
  const int r_first = (hi + PD) % ST;
  const int hl_top = (hi + PD - r_first) / ST - ho_lo;
  const int lam_thread = (mr * cc * LH + hl_top) * NLT + colseg * (G::TW / ST);
  const int w_thread = r_first * w_row + cig * TCI;

  stage(0, 0);
  int buf = 0;
  for (int co0 = 0; co0 < g.Co; co0 += cc, buf ^= 1) {
    const bool more = co0 + cc < g.Co;
    if (more) {
      stage(buf ^ 1, co0 + cc);  // the other buffer was released by the barrier that ended the previous iteration
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (row_ok) {
      const float* lam_t = rs_smem + buf * buf_words + lam_thread;
      const float* w_t = rs_smem + buf * buf_words + lam_words + w_thread;
      for (int co = 0; co < cc; ++co) {
        const float* lam_co = lam_t + co * tile;
        const float* w_co = w_t + co * KS * w_row;
#pragma unroll
        for (int jr = 0; jr < JR; ++jr) {
          if (KS % ST != 0 && r_first + ST * jr >= KS) break;
          float w[KS][TCI];
#pragma unroll
          for (int sct = 0; sct < KS; ++sct) {
            if (TCI == 4) {
              const float4 w4 = *reinterpret_cast<const float4*>(w_co + jr * ST * w_row + sct * cib);
              w[sct][0] = w4.x; w[sct][1 % TCI] = w4.y; w[sct][2 % TCI] = w4.z; w[sct][3 % TCI] = w4.w;
            } else {
#pragma unroll
              for (int c = 0; c < TCI; ++c) w[sct][c] = w_co[jr * ST * w_row + sct * cib + c];
            }
          }
          const float4* lp = reinterpret_cast<const float4*>(lam_co - jr * NLT);
          float L[G::NL];
#pragma unroll
          for (int q = G::Q0; q < G::NL / 4; ++q) {
            const float4 t4 = lp[q];
            L[4 * q + 0] = t4.x; L[4 * q + 1] = t4.y; L[4 * q + 2] = t4.z; L[4 * q + 3] = t4.w;
          }
#pragma unroll
          for (int sct = 0; sct < KS; ++sct) {
#pragma unroll
            for (int i = 0; i < G::TW; ++i) {
              if ((i + PD - sct) % ST == 0) {
#pragma unroll
                for (int c = 0; c < TCI; ++c) acc[c][i] = fmaf(L[(i + PD - sct) / ST + G::C0E], w[sct][c], acc[c][i]);
              }
            }
          }
        }
      }
    }
    __syncthreads();
  }
  if (!row_ok) return;
  const int wleft = g.Wi - (w0 + colseg * G::TW);
#pragma unroll
  for (int c = 0; c < TCI; ++c) {
    const int ci = ci0 + cig * TCI + c;
    if (ci >= g.Ci) break;
    float* op = g.out + (((size_t)(m0 + mr) * g.Ci + ci) * g.Hi + hi) * g.Wi + w0 + colseg * G::TW;
    if (wleft >= G::TW && (reinterpret_cast<uintptr_t>(op) & 15u) == 0) {
#pragma unroll
      for (int q = 0; q < G::TW / 4; ++q)
        reinterpret_cast<float4*>(op)[q] = make_float4(acc[c][4 * q], acc[c][4 * q + 1], acc[c][4 * q + 2], acc[c][4 * q + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < G::TW; ++i)
        if (i < wleft) op[i] = acc[c][i];
    }
  }
}

static int ilog2_ceil(int v) {
  int l = 0;
  while ((1 << l) < v) ++l;
  return l;
}

template <int KS, int ST, int PD, int TCI, bool VEC, int TWP>
static int launch_rowseg_tci(const ConvTArgs& g, cudaStream_t stream) {
  using G = RowSeg<KS, ST, PD, VEC, TWP>;
  RowSegArgs a{};
  a.c = g;
  // channel groups per block: up to 32 input channels side by side
  int cig = ceil_div(g.Ci, TCI);
  if (cig > 32 / TCI) cig = 32 / TCI;
  a.cigl = ilog2_ceil(cig);
  const int nsegl = 8 - a.cigl;  // 256 threads
  const int segs_row = ceil_div(g.Wi, G::TW);
  a.sxl = ilog2_ceil(segs_row);
  if (a.sxl > nsegl - 1) a.sxl = nsegl - 1;  // leave at least two image rows per block
  a.thl = ilog2_ceil(g.Hi);
  if (a.thl > nsegl - a.sxl) a.thl = nsegl - a.sxl;
  if ((1 << a.thl) % ST != 0) return BF_E_UNSUPPORTED;
  a.mrl = nsegl - a.sxl - a.thl;
  a.tiles_x = ceil_div(segs_row, 1 << a.sxl);
  a.tiles_y = ceil_div(g.Hi, 1 << a.thl);
  const int nlt = G::tile_w(1 << a.sxl);
  a.rowl = ilog2_ceil(VEC ? nlt / 4 : nlt);
  if (a.rowl > 8) return BF_E_UNSUPPORTED;
  const int cib = TCI << a.cigl;
  const size_t per_co = ((size_t)(1 << a.mrl) * G::tile_h(1 << a.thl) * nlt + (size_t)KS * (KS * cib + 4)) * sizeof(float);
  const size_t budget = (TCI > 1 ? 48 : 32) * 1024;  // per buffer; two buffers per block, two or three blocks per SM
  int cc = (int)(budget / per_co);
  if (cc > 16) cc = 16;
  if (cc > g.Co) cc = g.Co;
  if (cc < 1) return BF_E_UNSUPPORTED;
  while (g.Co % cc != 0) --cc;  // a divisor of Co: every chunk is full
  a.cc = cc;
  const size_t lam_words = (size_t)(1 << a.mrl) * cc * G::tile_h(1 << a.thl) * nlt;
  const size_t w_words = ((size_t)cc * KS * (KS * cib + 4) + 3) & ~(size_t)3;
  const size_t smem = 2 * (lam_words + w_words) * sizeof(float) + (size_t)(1 << a.mrl) * cc * G::tile_h(1 << a.thl) * sizeof(int);
  static SmemOptIn opt_in;
  if (int rc = ensure_dynamic_smem(conv_transpose_rowseg_kernel<KS, ST, PD, TCI, VEC, TWP>, 110 * 1024, opt_in, "conv_transpose_rowseg_kernel")) return rc;
  dim3 grid(ceil_div(g.M, 1 << a.mrl), a.tiles_x * a.tiles_y, ceil_div(g.Ci, cib));
  if (grid.y > 65535 || grid.z > 65535) return BF_E_UNSUPPORTED;
  conv_transpose_rowseg_kernel<KS, ST, PD, TCI, VEC, TWP><<<grid, 256, smem, stream>>>(a);
  BF_CHECK_LAUNCH("conv_transpose_rowseg_kernel");
  return BF_OK;
}

template <int KS, int ST, int PD>
static int launch_rowseg(const ConvTArgs& g, cudaStream_t stream) {
  const bool vec = (g.Wo % 4 == 0) && ((reinterpret_cast<uintptr_t>(g.Lam) & 15u) == 0);
  if (g.Ci <= 2) return vec ? launch_rowseg_tci<KS, ST, PD, 1, true, 16>(g, stream) : launch_rowseg_tci<KS, ST, PD, 1, false, 16>(g, stream);
  // 8-pixel segments when they waste fewer lanes than 16-pixel ones (narrow windows of the windowed sweeps)
  const bool narrow = ((g.Wi + 7) / 8) * 8 < ((g.Wi + 15) / 16) * 16;
  if (narrow) return vec ? launch_rowseg_tci<KS, ST, PD, 4, true, 8>(g, stream) : launch_rowseg_tci<KS, ST, PD, 4, false, 8>(g, stream);
  return vec ? launch_rowseg_tci<KS, ST, PD, 4, true, 16>(g, stream) : launch_rowseg_tci<KS, ST, PD, 4, false, 16>(g, stream);
}

// Row-segment kernel for the geometries it is instantiated for; BF_E_UNSUPPORTED otherwise.
static int launch_convT_rowseg(const ConvTArgs& g, cudaStream_t stream) {
  if (g.kh != g.kw || g.sh != g.sw || g.ph != g.pw) return BF_E_UNSUPPORTED;
  if (g.kh == 3 && g.sh == 1 && g.ph == 1) return launch_rowseg<3, 1, 1>(g, stream);
  if (g.kh == 4 && g.sh == 2 && g.ph == 1) return launch_rowseg<4, 2, 1>(g, stream);
  if (g.kh == 3 && g.sh == 2 && g.ph == 1) return launch_rowseg<3, 2, 1>(g, stream);
  // zero padding: the windowed sweeps below run every transposed convolution in window coordinates
  if (g.kh == 3 && g.sh == 1 && g.ph == 0) return launch_rowseg<3, 1, 0>(g, stream);
  if (g.kh == 4 && g.sh == 2 && g.ph == 0) return launch_rowseg<4, 2, 0>(g, stream);
  if (g.kh == 3 && g.sh == 2 && g.ph == 0) return launch_rowseg<3, 2, 0>(g, stream);
  if (g.kh == 5 && g.sh == 1 && g.ph == 2) return launch_rowseg<5, 1, 2>(g, stream);
  return BF_E_UNSUPPORTED;
}

// scaled coefficients [M, n_out] followed by the per-chunk partial sums of the intercept term [M, chunks]
static size_t relu_rows_lam_bytes(int M, int n_out) { return ((size_t)M * n_out * sizeof(float) + 255) & ~(size_t)255; }
size_t crown_bwd_conv2d_scratch_bytes(int M, const bf_layer_desc& L) {
  return relu_rows_lam_bytes(M, L.n_out) + (size_t)M * ceil_div(L.n_out, RELU_ROWS_CHUNK) * sizeof(float);
}

template <int ACC>
static int launch_convT(const ConvTArgs& g0, cudaStream_t stream) {
  ConvTArgs g = g0;
  const int taps = g.kh * g.kw;
  int co_chunk = (64 * 1024) / (taps * ACC * (int)sizeof(float));
  if (co_chunk < 1) co_chunk = 1;
  if (co_chunk > g.Co) co_chunk = g.Co;
  g.co_chunk = co_chunk;
  const int smem = co_chunk * taps * ACC * (int)sizeof(float);
  static SmemOptIn opt_in;
  if (int rc = ensure_dynamic_smem(conv_transpose_rows_kernel<ACC>, 96 * 1024, opt_in, "conv_transpose_rows_kernel")) return rc;
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
                            const bf_layer_desc& L, void* scratch, cudaStream_t stream, const float* add = nullptr) {
  const float* lam = A;
  const bool need_pro = (dpos != nullptr) || (bias != nullptr) || (delta != nullptr && !accumulate);
  if (need_pro) {
    BF_REQUIRE(!dpos || scratch, BF_E_WORKSPACE, "conv backward: scratch missing");
    float* lam_out = dpos ? static_cast<float*>(scratch) : nullptr;
    // without scratch (no ReLU) a block streams a whole row
    const int chunk = scratch ? RELU_ROWS_CHUNK : L.n_out;
    const int nchunks = ceil_div(L.n_out, chunk);
    float* partial = (delta && nchunks > 1) ? reinterpret_cast<float*>(static_cast<char*>(scratch) + relu_rows_lam_bytes(M, L.n_out)) : nullptr;
    BF_REQUIRE(nchunks <= 65535, BF_E_UNSUPPORTED, "conv backward: layer too wide");
    const void* ptrs[] = {A, dpos, dneg, epos, eneg, add, lam_out};
    int vec = (L.n_out % 4 == 0) ? 1 : 0;
    for (const void* q : ptrs) if (reinterpret_cast<uintptr_t>(q) & 15u) vec = 0;
    dim3 grid(M, nchunks);
    timing_begin(T_RELU_ROWS, stream);
    relu_bwd_rows_kernel<<<grid, 256, 0, stream>>>(A, dpos, dneg, epos, eneg, dpos ? add : nullptr, bias, L.Ho * L.Wo, lam_out, partial, delta, accumulate,
                                                  chunk, S, L.n_out, vec);
    // rows in (+ out when a ReLU scales them) and the slope / intercept vectors of every domain
    timing_end(T_RELU_ROWS, stream, (lam_out ? 8.0 : 4.0) * (double)M * L.n_out + (dpos ? 12.0 * (double)(M / S) * L.n_out : 0.0),
               4.0 * (double)M * L.n_out);
    BF_CHECK_LAUNCH("relu_bwd_rows_kernel");
    if (partial) {
      int rc = launch_sum_partials(accumulate ? delta : nullptr, partial, nchunks, delta, M, stream);
      if (rc != BF_OK) return rc;
    }
    if (dpos) lam = lam_out;
  }
  if (!A_prev) return BF_OK;
  ConvTArgs g{lam, W, A_prev, M, L.Ci, L.Hi, L.Wi, L.Co, L.Ho, L.Wo, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, 0};
  static const bool gather_only = getenv("BF_B200_CONV_GATHER") != nullptr;  // A/B switch, read once per process
  const double conv_bytes = 4.0 * (double)M * (L.n_out + L.n_in) + 4.0 * (double)L.Co * L.Ci * L.kh * L.kw;
  const double conv_flops = 2.0 * (double)M * L.n_out * L.Ci * L.kh * L.kw;
  timing_begin(T_CONV_T, stream);
  int rc = gather_only ? BF_E_UNSUPPORTED : launch_convT_rowseg(g, stream);
  if (rc == BF_E_UNSUPPORTED) {
    if (L.Ci <= 4) rc = launch_convT<4>(g, stream);
    else if (L.Ci <= 16) rc = launch_convT<16>(g, stream);
    else rc = launch_convT<32>(g, stream);
  }
  timing_end(T_CONV_T, stream, conv_bytes, conv_flops);
  return rc;
}

// ---------------------------------------------------------------------------
// Backward step of a conv2d layer for coefficient rows that are rows first..first+S-1 of the
// identity (the start of an intermediate-bound sweep): row j = (co, ho, wo) maps to the kernel
// patch W[co, :, :, :] placed at (ho*sh - ph, wo*sw - pw), the same for every domain, and its
// bias term is bias[co].  One thread per output element; nothing is multiplied.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) onehot_conv_rows_kernel(const float* __restrict__ W, const float* __restrict__ bias,
                                                               float* __restrict__ out, float* __restrict__ delta, int first,
                                                               int S, int vec, ConvTArgs g) {
  // grid (coefficient row, group of input channels): the row's output position is decoded once per block
  const int m = blockIdx.x;
  const int j = first + m % S;
  const int co = j / (g.Ho * g.Wo), rem = j - co * (g.Ho * g.Wo);
  const int ho = rem / g.Wo, wo = rem - ho * g.Wo;
  const int h_top = ho * g.sh - g.ph, w_left = wo * g.sw - g.pw;  // image position of kernel tap (0, 0)
  if (blockIdx.y == 0 && threadIdx.x == 0 && delta) delta[m] = bias ? __ldg(bias + co) : 0.f;
  const int ci_per_block = (g.Ci + gridDim.y - 1) / gridDim.y;
  const int ci_end = min(g.Ci, (int)(blockIdx.y + 1) * ci_per_block);
  for (int ci = blockIdx.y * ci_per_block; ci < ci_end; ++ci) {
  const float* wp = W + ((size_t)co * g.Ci + ci) * g.kh * g.kw;
  float* op = out + ((size_t)m * g.Ci + ci) * g.Hi * g.Wi;
  if (vec) {  // Wi % 4 == 0 and 16-byte aligned rows
    const int w4 = g.Wi >> 2;
    for (int p = threadIdx.x; p < g.Hi * w4; p += 256) {
      const int hi = p / w4, wi = (p - hi * w4) << 2;
      const int r = hi - h_top;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (r >= 0 && r < g.kh) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int sc = wi + q - w_left;
          if (sc >= 0 && sc < g.kw) v[q] = __ldg(wp + r * g.kw + sc);
        }
      }
      *reinterpret_cast<float4*>(op + (size_t)hi * g.Wi + wi) = make_float4(v[0], v[1], v[2], v[3]);
    }
  } else {
    for (int p = threadIdx.x; p < g.Hi * g.Wi; p += 256) {
      const int hi = p / g.Wi, wi = p - hi * g.Wi;
      const int r = hi - h_top, sc = wi - w_left;
      op[p] = (r >= 0 && r < g.kh && sc >= 0 && sc < g.kw) ? __ldg(wp + r * g.kw + sc) : 0.f;
    }
  }
  }
}

// grid-stride launch: enough blocks to fill the machine, at most one block per 256 elements
static int onehot_grid(long long total) {
  const long long blocks = (total + 255) / 256;
  return (int)(blocks < 148LL * 16 ? blocks : 148LL * 16);
}

int launch_onehot_conv_rows(int first, const float* W, const float* bias, float* A_prev, float* delta, int M, int S,
                            const bf_layer_desc& L, cudaStream_t stream) {
  ConvTArgs g{nullptr, W, A_prev, M, L.Ci, L.Hi, L.Wi, L.Co, L.Ho, L.Wo, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, 0};
  BF_REQUIRE(L.Ci <= 65535, BF_E_UNSUPPORTED, "conv backward: too many input channels");
  const int vec = (L.Wi % 4 == 0 && (reinterpret_cast<uintptr_t>(A_prev) & 15u) == 0) ? 1 : 0;
  // about 16 KB of output per block once there are enough rows to fill the machine
  int groups = L.Ci;
  const int per_block = 16384 / (L.Hi * L.Wi * 4);
  if (M >= 148 * 8 && per_block > 1) groups = ceil_div(L.Ci, per_block);
  dim3 grid(M, groups);
  onehot_conv_rows_kernel<<<grid, 256, 0, stream>>>(W, bias, A_prev, delta, first, S, vec, g);
  BF_CHECK_LAUNCH("onehot_conv_rows_kernel");
  return BF_OK;
}

// ---------------------------------------------------------------------------
// Windowed coefficient rows.  A row that started as a row of the identity on a conv layer's output is zero
// outside a small window of every feature map below it: kh x kw after the first backward step, and
// (WH-1)*stride + k after each further transposed convolution.  While the window is smaller than the
// feature map the sweep keeps only the window, [M, C, WH, WW] per row, whose image position follows from
// the row's output pixel (ho, wo):  top = ho*sy + ty, left = wo*sx + tx.  A transposed convolution in
// window coordinates is the ordinary one with zero padding (the kernels above, geometry Ho=WH, Wo=WW);
// what falls outside the feature map is cleared by the next ReLU pass or ignored by the concretisation.
// ---------------------------------------------------------------------------

// first backward step: the window is the kernel itself (one warp per row)
__global__ void __launch_bounds__(256) onehot_conv_window_kernel(const float* __restrict__ W, const float* __restrict__ bias,
                                                                 float* __restrict__ out, float* __restrict__ delta, WindowGeom w,
                                                                 int per) {
  const int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (m >= w.M) return;
  const int cb = (w.first + m % w.S) / (w.HoB * w.WoB);
  const float* src = W + (size_t)cb * per;
  float* dst = out + (size_t)m * per;
  for (int r = lane; r < per; r += 32) dst[r] = __ldg(src + r);
  if (lane == 0 && delta) delta[m] = bias ? __ldg(bias + cb) : 0.f;
}

// ReLU backward on windows: Lam = A * slope_sel inside the feature map, 0 outside;
// delta += sum A * icpt_sel + Lam * bias[channel].  T threads per row (T = 32 ... 256, by window size), 256 / T
// rows per block.  A thread owns positions of the WH x WW window plane and walks the channels: the image pixel of a
// position, whether it lies inside the feature map and both offsets are computed once per position.  The kernel is bound
// by the latency of its reads (the window value, then the slope and intercept that value selects, gathered from the
// feature map), so the channel loop handles eight channels at a time: eight window values in flight, then eight slopes.
// When the plane is smaller than T the threads split into T / plane channel groups (thread = group * plane + position).
template <int T>
__global__ void __launch_bounds__(256) relu_bwd_window_kernel(const float* __restrict__ A, const float* __restrict__ dpos,
                                                              const float* __restrict__ dneg, const float* __restrict__ epos,
                                                              const float* __restrict__ eneg, const float* __restrict__ bias,
                                                              float* __restrict__ Lam, float* __restrict__ delta, WindowGeom w) {
  __shared__ float red[8];
  const int m = blockIdx.x * (256 / T) + threadIdx.x / T;
  const int t = threadIdx.x % T;
  const bool live = m < w.M;  // whole warps: T is a multiple of 32
  float acc = 0.f;
  if (live) {
    const int j = w.first + m % w.S;
    const int rem = j % (w.HoB * w.WoB);
    const int top = (rem / w.WoB) * w.sy + w.ty, left = (rem % w.WoB) * w.sx + w.tx;
    const int plane = w.WH * w.WW;
    const int HW = w.H * w.W;
    const size_t dom = (size_t)(m / w.S) * w.C * HW;
    const float* a_row = A + (size_t)m * w.C * plane;
    float* lo_row = Lam + (size_t)m * w.C * plane;
    const int groups = (plane < T) ? T / plane : 1;          // channel groups when the plane is smaller than T
    const int c0 = (plane < T) ? t / plane : 0;              // this thread's first channel
    const int p0 = (plane < T) ? t - c0 * plane : t;         // and its first position
    const int pstep = (plane < T) ? plane : T;               // plane < T: a single position per thread
    if (c0 < groups) {
      const size_t astep = (size_t)groups * plane, kstep = (size_t)groups * HW;
      for (int pos = p0; pos < plane; pos += pstep) {
        const int y = pos / w.WW, x = pos - y * w.WW;
        const int Y = top + y, X = left + x;
        const bool inside = Y >= 0 && Y < w.H && X >= 0 && X < w.W;
        const float* a = a_row + (size_t)c0 * plane + pos;
        float* lo = lo_row + (size_t)c0 * plane + pos;
        if (!inside) {
          for (int c = c0; c < w.C; c += groups, lo += astep) *lo = 0.f;
          continue;
        }
        size_t k = dom + (size_t)c0 * HW + (size_t)Y * w.W + X;
        int c = c0;
        constexpr int U = 8;   // channels in flight
        for (; c + (U - 1) * groups < w.C; c += U * groups, a += U * astep, lo += U * astep, k += U * kstep) {
          float v[U], sl[U], ic[U];
#pragma unroll
          for (int q = 0; q < U; ++q) v[q] = a[q * astep];
#pragma unroll
          for (int q = 0; q < U; ++q) {
            const size_t kq = k + q * kstep;
            const bool sel = v[q] >= 0.f;
            sl[q] = sel ? dpos[kq] : dneg[kq];
            ic[q] = sel ? (epos ? epos[kq] : 0.f) : (eneg ? eneg[kq] : 0.f);
          }
#pragma unroll
          for (int q = 0; q < U; ++q) {
            const float lam = v[q] * sl[q];
            acc = fmaf(v[q], ic[q], acc);
            if (bias) acc = fmaf(lam, __ldg(bias + c + q * groups), acc);
            lo[q * astep] = lam;
          }
        }
        for (; c < w.C; c += groups, a += astep, lo += astep, k += kstep) {
          const float v = *a;
          const bool sel = v >= 0.f;
          const float lam = v * (sel ? dpos[k] : dneg[k]);
          acc = fmaf(v, sel ? (epos ? epos[k] : 0.f) : (eneg ? eneg[k] : 0.f), acc);
          if (bias) acc = fmaf(lam, __ldg(bias + c), acc);
          *lo = lam;
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (T == 32) {
    if (live && t == 0) delta[m] += acc;
  } else {
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (live && t == 0) {
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < T / 32; ++i) sum += red[(threadIdx.x >> 5) + i];
      delta[m] += sum;
    }
  }
}

// window -> full feature map (zeros elsewhere, what falls outside the map is dropped)
__global__ void __launch_bounds__(256) window_to_dense_kernel(const float* __restrict__ Awin, float* __restrict__ dense, WindowGeom w) {
  const int m = blockIdx.x;
  const int j = w.first + m % w.S;
  const int rem = j % (w.HoB * w.WoB);
  const int top = (rem / w.WoB) * w.sy + w.ty, left = (rem % w.WoB) * w.sx + w.tx;
  const int n = w.C * w.H * w.W, n_win = w.C * w.WH * w.WW;
  for (int k = threadIdx.x; k < n; k += 256) {
    const int c = k / (w.H * w.W), r2 = k - c * (w.H * w.W);
    const int y = r2 / w.W - top, x = r2 % w.W - left;
    dense[(size_t)m * n + k] = (y >= 0 && y < w.WH && x >= 0 && x < w.WW) ? Awin[(size_t)m * n_win + (c * w.WH + y) * w.WW + x] : 0.f;
  }
}

// box concretisation of windows on the network input: out[m] = sum A*mid -/+ |A|*rad over the window inside the image + delta
__global__ void __launch_bounds__(256) concretize_window_kernel(const float* __restrict__ Awin, const float* __restrict__ mid,
                                                                const float* __restrict__ rad, const float* __restrict__ delta,
                                                                float* __restrict__ out, float sgn, WindowGeom w) {
  const int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (m >= w.M) return;
  const int j = w.first + m % w.S;
  const int rem = j % (w.HoB * w.WoB);
  const int top = (rem / w.WoB) * w.sy + w.ty, left = (rem % w.WoB) * w.sx + w.tx;
  const int n_win = w.C * w.WH * w.WW;
  const size_t dom = (size_t)(m / w.S) * w.C * w.H * w.W;
  float acc = 0.f;
  // four elements of a lane per iteration: their index arithmetic first, then all loads, then the sums in element order
  // (the loop is bound by the latency of its gathered reads, like the ReLU pass on windows)
  for (int e0 = lane; e0 < n_win; e0 += 128) {
    float v[4], cm[4], cr[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = e0 + 32 * q;
      v[q] = cm[q] = cr[q] = 0.f;
      if (e < n_win) {
        const int c = e / (w.WH * w.WW), r2 = e - c * (w.WH * w.WW);
        const int Y = top + r2 / w.WW, X = left + r2 % w.WW;
        if (Y >= 0 && Y < w.H && X >= 0 && X < w.W) {
          const size_t k = dom + ((size_t)c * w.H + Y) * w.W + X;
          v[q] = Awin[(size_t)m * n_win + e];
          cm[q] = mid[k];
          cr[q] = rad[k];
        }
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {   // an element outside the window or the image contributes exact zeros
      acc = fmaf(v[q], cm[q], acc);
      acc = fmaf(sgn * fabsf(v[q]), cr[q], acc);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[m] = acc + (delta ? delta[m] : 0.f);
}

int launch_onehot_conv_window(const float* W, const float* bias, float* out, float* delta, const WindowGeom& w, int M, int Ci, int kk,
                              cudaStream_t stream) {
  onehot_conv_window_kernel<<<ceil_div((long long)M * 32, 256), 256, 0, stream>>>(W, bias, out, delta, w, Ci * kk);
  BF_CHECK_LAUNCH("onehot_conv_window_kernel");
  return BF_OK;
}

int launch_relu_bwd_window(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                           const float* bias, float* Lam, float* delta, const WindowGeom& w, int M, cudaStream_t stream) {
  const int n_win = w.C * w.WH * w.WW;
  timing_begin(T_RELU_WINDOW, stream);
  if (n_win <= 512)
    relu_bwd_window_kernel<32><<<ceil_div(M, 8), 256, 0, stream>>>(A, dpos, dneg, epos, eneg, bias, Lam, delta, w);
  else if (n_win <= 1536)
    relu_bwd_window_kernel<64><<<ceil_div(M, 4), 256, 0, stream>>>(A, dpos, dneg, epos, eneg, bias, Lam, delta, w);
  else if (n_win <= 4096)
    relu_bwd_window_kernel<128><<<ceil_div(M, 2), 256, 0, stream>>>(A, dpos, dneg, epos, eneg, bias, Lam, delta, w);
  else
    relu_bwd_window_kernel<256><<<M, 256, 0, stream>>>(A, dpos, dneg, epos, eneg, bias, Lam, delta, w);
  // window rows in and out; the slopes and intercepts are gathered per element (three values of the row's domain)
  timing_end(T_RELU_WINDOW, stream, 8.0 * (double)M * n_win + 12.0 * (double)M * n_win, 4.0 * (double)M * n_win);
  BF_CHECK_LAUNCH("relu_bwd_window_kernel");
  return BF_OK;
}

int launch_window_to_dense(const float* Awin, float* dense, const WindowGeom& w, int M, cudaStream_t stream) {
  window_to_dense_kernel<<<M, 256, 0, stream>>>(Awin, dense, w);
  BF_CHECK_LAUNCH("window_to_dense_kernel");
  return BF_OK;
}

int launch_concretize_window(const float* Awin, const float* mid, const float* rad, const float* delta, float* out, int side,
                             const WindowGeom& w, int M, cudaStream_t stream) {
  concretize_window_kernel<<<ceil_div((long long)M * 32, 256), 256, 0, stream>>>(Awin, mid, rad, delta, out,
                                                                               side == BF_SIDE_LOWER ? -1.f : 1.f, w);
  BF_CHECK_LAUNCH("concretize_window_kernel");
  return BF_OK;
}

// Same for a linear layer: coefficient row j is row j of W, its bias term bias[j].
__global__ void __launch_bounds__(256) onehot_linear_rows_kernel(const float* __restrict__ W, const float* __restrict__ bias,
                                                                 float* __restrict__ out, float* __restrict__ delta, int first,
                                                                 int S, int n_in, long long total) {
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(e / n_in);
    const int k = (int)(e - (long long)m * n_in);
    const int j = first + m % S;
    out[e] = __ldg(W + (size_t)j * n_in + k);
    if (k == 0 && delta) delta[m] = bias ? __ldg(bias + j) : 0.f;
  }
}

int launch_onehot_linear_rows(int first, const float* W, const float* bias, float* A_prev, float* delta, int M, int S, int n_in,
                              cudaStream_t stream) {
  const long long total = (long long)M * n_in;
  onehot_linear_rows_kernel<<<onehot_grid(total), 256, 0, stream>>>(W, bias, A_prev, delta, first, S, n_in, total);
  BF_CHECK_LAUNCH("onehot_linear_rows_kernel");
  return BF_OK;
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
  bf_layer_desc L{};
  L.n_out = Co * Ho * Wo;
  return bf::crown_bwd_conv2d_scratch_bytes(B * S, L);
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
  // without slopes the scratch is optional; one that is too small for the chunked intercept sums is not used at all
  // (a block then streams a whole coefficient row)
  if (!relu && scratch_bytes < bf_crown_relu_conv2d_bwd_scratch_bytes(B, S, Co, Ho, Wo)) scratch = nullptr;
  return bf::launch_crown_bwd_conv2d(A, dpos, dneg, epos, eneg, W, bias, A_prev, delta, accumulate, B * S, S, L, scratch,
                                     bf::as_stream(stream));
}

// ReLU backward alone (graphs where the ReLU's producer is not a single affine layer, e.g. after an add):
// A_prev = A * slope_sel, delta (+)= sum A * icpt_sel (+ add term on the lower side is not needed here).
extern "C" size_t bf_crown_relu_bwd_scratch_bytes(int B, int S, int n) {
  return (size_t)B * S * bf::ceil_div(n, bf::RELU_ROWS_CHUNK) * sizeof(float);
}

extern "C" int bf_crown_relu_bwd(const float* A, int side, const float* alpha_u, const float* alpha_l, const float* beta_u,
                                 const float* beta_l, float* A_prev, float* delta, int accumulate, void* scratch,
                                 size_t scratch_bytes, int B, int S, int n, bf_stream_t stream_) {
  BF_REQUIRE(A && alpha_u && alpha_l && A_prev, BF_E_INVALID, "bf_crown_relu_bwd: null tensor");
  BF_REQUIRE(B > 0 && S > 0 && n > 0 && (long long)B * S < 2147483647LL, BF_E_INVALID, "bf_crown_relu_bwd: bad sizes");
  BF_REQUIRE(side == BF_SIDE_LOWER || side == BF_SIDE_UPPER, BF_E_INVALID, "bf_crown_relu_bwd: bad side");
  const float *dpos, *dneg, *epos, *eneg;
  if (side == BF_SIDE_LOWER) { dpos = alpha_l; dneg = alpha_u; epos = beta_l; eneg = beta_u; }
  else { dpos = alpha_u; dneg = alpha_l; epos = beta_u; eneg = beta_l; }
  const int M = B * S;
  const int nchunks = bf::ceil_div(n, bf::RELU_ROWS_CHUNK);
  float* partial = nullptr;
  if (delta && nchunks > 1) {
    BF_REQUIRE(scratch && scratch_bytes >= bf_crown_relu_bwd_scratch_bytes(B, S, n), BF_E_WORKSPACE,
               "bf_crown_relu_bwd: scratch of %zu bytes needed", bf_crown_relu_bwd_scratch_bytes(B, S, n));
    partial = static_cast<float*>(scratch);
  }
  BF_REQUIRE(nchunks <= 65535, BF_E_UNSUPPORTED, "bf_crown_relu_bwd: layer too wide");
  const void* ptrs[] = {A, dpos, dneg, epos, eneg, A_prev};
  int vec = (n % 4 == 0) ? 1 : 0;
  for (const void* q : ptrs) if (reinterpret_cast<uintptr_t>(q) & 15u) vec = 0;
  cudaStream_t stream = bf::as_stream(stream_);
  dim3 grid(M, nchunks);
  bf::relu_bwd_rows_kernel<<<grid, 256, 0, stream>>>(A, dpos, dneg, epos, eneg, nullptr, nullptr, 1, A_prev, partial, delta, accumulate,
                                                    bf::RELU_ROWS_CHUNK, S, n, vec);
  BF_CHECK_LAUNCH("relu_bwd_rows_kernel");
  if (partial) return bf::launch_sum_partials(accumulate ? delta : nullptr, partial, nchunks, delta, M, stream);
  return BF_OK;
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
