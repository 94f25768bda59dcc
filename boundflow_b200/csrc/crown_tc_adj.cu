// Adjoint (gradient) sweep step of a linear layer on the 5th-generation tensor cores, feature-major:
//     g[m, n] = sum_k h_prev[m, k] * W[n, k] + b[n]
//     h[m, n] = d_sel[dom(m), n] * g + e_sel[dom(m), n]             (sel by the sign of the saved coefficient)
//     grad[dom, n] += [unstable] [coef >= 0] coef[m, n] * g[m, n]   (summed over the domain's rows)
// The MMA's M side (128 tensor-memory lanes) is a tile of 128 layer OUTPUT FEATURES taken from the
// pre-packed static weight images, its N side (256 accumulator columns) is a block of 256
// coefficient rows produced on the fly.  After tcgen05.ld a thread therefore owns one feature n
// and 32 consecutive rows m in registers:
//   * every global access of the epilogue (saved coefficients in, h out) is a coalesced 128-byte
//     row segment across the warp, without a transpose through shared memory;
//   * the slopes / intercepts / unstable flag of (domain, n) live in five registers and change
//     every S rows, warp-uniformly;
//   * the per-domain sums over rows are running sums in registers, flushed with one atomic per
//     (domain, n) and row chunk.
// 3xTF32 split operands as in the backward kernel: a*b ~= a_hi*b_hi + a_lo*b_hi + a_hi*b_lo.
// One CTA owns 256 rows x up to two feature tiles (accumulators side by side in the 512
// tensor-memory columns); one produced k-block feeds both feature tiles' MMAs.
// Every wait is bounded: on expiry the CTA raises a status word, stops, frees its tensor memory
// and returns.
#include "kernels.cuh"
#include "tc_primitives.cuh"

namespace bf {
namespace tca {

using namespace bf::tc;

constexpr int FT = 128;                 // features per accumulator (MMA M)
constexpr int RB = 256;                 // coefficient rows per CTA (MMA N)
constexpr int BK = 32;                  // fp32 per k-block row = 128 bytes
constexpr int P_TILE = RB * BK * 4;     // bytes of one produced tile (hi or lo)
constexpr int S_TILE = FT * BK * 4;     // bytes of one static tile (hi or lo)
constexpr int P_STAGES = 2;
constexpr int S_STAGES = 3;
constexpr int WARPS = 16;               // producers during the main loop, then the epilogue
constexpr int PRODUCERS = WARPS * 32;
constexpr int ROWS_PER_THREAD = RB / (PRODUCERS / 8);  // 8 threads cover one 128-byte row
constexpr int COPY_WARP = WARPS;
constexpr int MMA_WARP = WARPS + 1;
constexpr int THREADS = (WARPS + 2) * 32;
constexpr int PREFETCH_KB = 4;
constexpr int SMEM_BYTES = 2048 + P_STAGES * 2 * P_TILE + S_STAGES * 2 * S_TILE;

enum { PRO_PLAIN = 0, PRO_H0 = 2 };

struct Params {
  const float* A;            // [M,K]: h of the previous layer, or the input coefficients (PRO_H0)
  const unsigned char* Wpk;  // packed hi/lo images, [feature tiles][nkb][2][128][128 B]
  int M, N, K, S, nkb, nft, vecK;
  const float* mid_k; const float* rad_k;   // PRO_H0: [D,K]
  const float* nbias; const float* Ahat; const float* dpos; const float* dneg; const float* epos; const float* eneg;
  const float* pre_l; const float* pre_u; float* hout; float* grad; float* gsum;
  int* status;
  int wave;                  // CTAs resident at once (one per SM): distance to the CTA that follows on a freed SM
};

struct Control {
  unsigned long long p_full[P_STAGES];
  unsigned long long p_empty[P_STAGES];
  unsigned long long s_full[S_STAGES];
  unsigned long long s_empty[S_STAGES];
  unsigned long long accum;
  uint32_t tmem_base;
  int abort_flag;
};

struct Slopes {
  float dp, dn, ep, en, amb;
};

__device__ __forceinline__ Slopes load_slopes(const Params& p, int d, int n, bool ok) {
  Slopes s;
  const size_t off = (size_t)d * p.N + n;
  s.dp = ok ? __ldg(p.dpos + off) : 0.f;
  s.dn = ok ? __ldg(p.dneg + off) : 0.f;
  s.ep = (ok && p.epos) ? __ldg(p.epos + off) : 0.f;
  s.en = (ok && p.eneg) ? __ldg(p.eneg + off) : 0.f;
  const float pl = ok ? __ldg(p.pre_l + off) : 0.f;
  const float pu = ok ? __ldg(p.pre_u + off) : 0.f;
  s.amb = (pl < 0.f && pu > 0.f) ? 1.f : 0.f;
  return s;
}

// ---- epilogue pieces -----------------------------------------------------------------------
// A lane owns one feature n; rows arrive eight at a time (v[u] = g[row + u][n]).
constexpr int TBLD = 5;                       // domains of one 32-row chunk served from the shared-memory slope table (S >= 8)
constexpr int TBL_FLOATS = TBLD * 6 * 32;     // [domain][dpos, dneg, epos, eneg, pre_l, pre_u][lane]

struct ChunkState {
  Slopes cur, nxt;     // slopes of the current domain and (register path) of the one after it
  float run, run2;     // running per-domain sums: alpha gradient, g itself (beta gradient)
  int d;               // current domain
  unsigned off_st;     // byte offset of the next h element inside the CTA's row slab
  const float* tb;     // this lane's column of the chunk's slope table, or null (register path)
  int k, nd;           // table path: index of the current domain inside the chunk, domains in the chunk
};

__device__ __forceinline__ void cp_async4(uint32_t dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

// Starts the asynchronous copy of the slopes of the chunk's domains d0 .. d0 + nd - 1 at feature n into this lane's table column.
__device__ __forceinline__ void table_fill(const Params& p, float* tb, int d0, int nd, int n) {
  for (int dl = 0; dl < nd; ++dl) {
    const size_t off = (size_t)(d0 + dl) * p.N + n;
    const uint32_t dst = smem_u32(tb + dl * 6 * 32);
    cp_async4(dst, p.dpos + off);
    cp_async4(dst + 128, p.dneg + off);
    if (p.epos) cp_async4(dst + 256, p.epos + off);
    if (p.eneg) cp_async4(dst + 384, p.eneg + off);
    cp_async4(dst + 512, p.pre_l + off);
    cp_async4(dst + 640, p.pre_u + off);
  }
}

__device__ __forceinline__ Slopes table_read(const Params& p, const float* tb, int k) {
  const float* t = tb + k * 6 * 32;
  Slopes s;
  s.dp = t[0];
  s.dn = t[32];
  s.ep = p.epos ? t[64] : 0.f;
  s.en = p.eneg ? t[96] : 0.f;
  s.amb = (t[128] < 0.f && t[160] > 0.f) ? 1.f : 0.f;
  return s;
}

__device__ __forceinline__ void row_step(ChunkState& st, float a, float g, float nb, char* __restrict__ hout_cta, unsigned rowstride,
                                         bool st_ok) {
  const float gg = g + nb;
  const bool sel = a >= 0.f;
  const float h = fmaf(sel ? st.cur.dp : st.cur.dn, gg, sel ? st.cur.ep : st.cur.en);
  float* dst = reinterpret_cast<float*>(hout_cta + st.off_st);
  if (st_ok) *dst = h;
  st.off_st += rowstride;
  const float r1 = fmaf(a * st.cur.amb, gg, st.run);
  st.run = sel ? r1 : st.run;
  st.run2 += gg;
}

// the row just processed was the last one of domain st.d inside this chunk
template <bool TBL>
__device__ __forceinline__ void boundary_step(const Params& p, ChunkState& st, int n, bool n_ok, int D) {
  if (n_ok) {
    atomicAdd(&p.grad[(size_t)st.d * p.N + n], st.run);
    if (p.gsum) atomicAdd(&p.gsum[(size_t)st.d * p.N + n], st.run2);
  }
  st.run = 0.f;
  st.run2 = 0.f;
  ++st.d;
  if (TBL) {
    st.k = min(st.k + 1, st.nd - 1);
    st.cur = table_read(p, st.tb, st.k);
  } else {
    st.cur = st.nxt;
    st.nxt = load_slopes(p, min(st.d + 1, D - 1), n, n_ok);
  }
}

// Eight existing rows with at most one domain boundary, after row B (B == 8: none): straight-line code.
template <int B, bool TBL>
__device__ __forceinline__ void group_static(const Params& p, ChunkState& st, const float (&v)[8], const float (&ah)[8], float nb,
                                             char* __restrict__ hout_cta, unsigned rowstride, bool st_ok, int n, bool n_ok, int D) {
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    row_step(st, ah[u], v[u], nb, hout_cta, rowstride, st_ok);
    if (u == B) boundary_step<TBL>(p, st, n, n_ok, D);
  }
}

// Epilogue of one 32-row x 32-feature chunk whose accumulator sits at tensor-memory address taddr.
// vmask / bmask come from warp votes (rows that exist; rows that end a domain inside the chunk),
// so every branch below is warp-uniform by construction.  Rows are handled in groups of eight
// (rolled, to keep the code small); a group of existing rows with at most one boundary -- every
// group when a domain has eight rows or more -- runs as straight-line code selected by the
// boundary position, other groups row by row.  The saved coefficients of the next group are
// loaded while the current one is processed.  TBL: the slopes of the chunk's domains were copied
// to this lane's shared-memory table column (tb) ahead of time; otherwise they are loaded from
// global memory one domain ahead.
template <bool TBL>
__device__ __forceinline__ void adjoint_chunk(const Params& p, uint32_t taddr, const char* __restrict__ ahat_cta,
                                              char* __restrict__ hout_cta, unsigned off, unsigned rowstride, int n, bool n_ok,
                                              bool st_ok, float nb, int d, int D, unsigned vmask, unsigned bmask, const float* tb,
                                              int nd) {
  ChunkState st;
  st.tb = tb;
  st.k = 0;
  st.nd = nd;
  if (TBL) {
    st.cur = table_read(p, tb, 0);
    st.nxt = st.cur;
  } else {
    st.cur = load_slopes(p, d, n, n_ok);
    st.nxt = load_slopes(p, min(d + 1, D - 1), n, n_ok);
  }
  st.run = 0.f;
  st.run2 = 0.f;
  st.d = d;
  st.off_st = off;
  unsigned off_ld = off;
  float ahn[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    ahn[u] = 0.f;
    if (vmask & (1u << u)) ahn[u] = __ldg(reinterpret_cast<const float*>(ahat_cta + off_ld));
    off_ld += rowstride;
  }
#pragma unroll 1
  for (int jb = 0; jb < 32; jb += 8) {
    const unsigned vm = (vmask >> jb) & 0xffu, bm = (bmask >> jb) & 0xffu;
    if (vm == 0u) break;
    const unsigned vmn = (jb < 24) ? ((vmask >> (jb + 8)) & 0xffu) : 0u;
    float v[8], ah[8];
    tmem_ld8(taddr + (uint32_t)jb, v);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      ah[u] = ahn[u];
      if (vmn & (1u << u)) ahn[u] = __ldg(reinterpret_cast<const float*>(ahat_cta + off_ld));
      off_ld += rowstride;
    }
    if (vm == 0xffu && (bm & (bm - 1u)) == 0u) {
      switch (bm ? (__ffs((int)bm) - 1) : 8) {
        case 0: group_static<0, TBL>(p, st, v, ah, nb, hout_cta, rowstride, st_ok, n, n_ok, D); break;
        case 1: group_static<1, TBL>(p, st, v, ah, nb, hout_cta, rowstride, st_ok, n, n_ok, D); break;
        case 2: group_static<2, TBL>(p, st, v, ah, nb, hout_cta, rowstride, st_ok, n, n_ok, D); break;
        case 3: group_static<3, TBL>(p, st, v, ah, nb, hout_cta, rowstride, st_ok, n, n_ok, D); break;
        case 4: group_static<4, TBL>(p, st, v, ah, nb, hout_cta, rowstride, st_ok, n, n_ok, D); break;
        case 5: group_static<5, TBL>(p, st, v, ah, nb, hout_cta, rowstride, st_ok, n, n_ok, D); break;
        case 6: group_static<6, TBL>(p, st, v, ah, nb, hout_cta, rowstride, st_ok, n, n_ok, D); break;
        case 7: group_static<7, TBL>(p, st, v, ah, nb, hout_cta, rowstride, st_ok, n, n_ok, D); break;
        default: group_static<8, TBL>(p, st, v, ah, nb, hout_cta, rowstride, st_ok, n, n_ok, D); break;
      }
    } else {
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (vm & (1u << u)) {
          row_step(st, ah[u], v[u], nb, hout_cta, rowstride, st_ok);
          if (bm & (1u << u)) boundary_step<TBL>(p, st, n, n_ok, D);
        }
      }
    }
  }
}

// Work split of one CTA (THREADS = 576):
//   warps 0-15  produce the coefficient-row operand during the main loop (ROWS_PER_THREAD rows x one
//               16-byte chunk per thread and k-block), then run the epilogue (warp w reads
//               tensor-memory lane quarter w%4 = 32 features, row chunks w/4 and w/4 + 4)
//   warp 16     lane 0 issues the bulk copies of the packed weight images
//   warp 17     lane 0 issues the MMAs; the warp allocates / frees tensor memory
template <int PRO>
__global__ void __launch_bounds__(THREADS, 1) crown_tc_adjoint_kernel(Params p) {
  extern __shared__ unsigned char raw_smem[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1024 + 1023) & ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(tiles - 1024);
  unsigned char* s_tiles = tiles + P_STAGES * 2 * P_TILE;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // x = feature-tile pair, y = row block: the CTAs that share a row block are launched side by side, so the
  // second read of its rows hits L2
  const int m0 = blockIdx.y * RB;
  const int ft0 = blockIdx.x * 2;                      // first feature tile of this CTA
  const int nf = min(2, p.nft - ft0);                  // feature tiles handled here
  const int nbase = ft0 * FT;                          // first feature
  const uint32_t tmem_cols = (nf == 1) ? 256u : 512u;
  volatile int* abort_flag = &ctl->abort_flag;
  int copies_issued = 0;  // bulk copies this thread has issued (meaningful in the copy thread only)

  if (tid == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(smem_u32(&ctl->p_full[s]), PRODUCERS);
      mbar_init(smem_u32(&ctl->p_empty[s]), 1);
    }
    for (int s = 0; s < S_STAGES; ++s) {
      mbar_init(smem_u32(&ctl->s_full[s]), 1);
      mbar_init(smem_u32(&ctl->s_empty[s]), 1);
    }
    mbar_init(smem_u32(&ctl->accum), 1);
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp < WARPS) {
    // ------------------------------------------------------------------ row-operand producers
    const int c = tid & 7;        // 16-byte chunk inside the 128-byte k-block row
    const int rg = tid >> 3;      // row group of this thread
    const int row0 = m0 + rg * ROWS_PER_THREAD;
    const bool vK = p.vecK != 0;
    // every k-block is complete and 16-byte aligned (the usual case): loads need no bounds logic
    const bool fastK = vK && (p.K % BK == 0);
    auto ldk = [&](const float* row, int k) -> float4 {
      if (fastK) return __ldg(reinterpret_cast<const float4*>(row + k));
      return (k < p.K) ? load4_guard(row, k, p.K, vK) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    int dom[ROWS_PER_THREAD];
#pragma unroll
    for (int i = 0; i < ROWS_PER_THREAD; ++i) dom[i] = (row0 + i < p.M) ? ((row0 + i) / p.S) : 0;

    float4 a_next[ROWS_PER_THREAD];
    auto load_block = [&](int kb) {
      const int k = kb * BK + c * 4;
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) {
        const int m = row0 + i;
        a_next[i] = (m < p.M) ? ldk(p.A + (size_t)m * p.K, k) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (c == 0 && m < p.M && (kb + PREFETCH_KB) * BK < p.K)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.A + (size_t)m * p.K + (size_t)(kb + PREFETCH_KB) * BK));
      }
    };

    load_block(0);
    bool alive = true;
    const int pf_kb = max(1, p.nkb - 5);  // late enough that the lines are still in L2 when the epilogue starts
    for (int kb = 0; kb < p.nkb; ++kb) {
      float4 a_cur[ROWS_PER_THREAD];
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) a_cur[i] = a_next[i];
      if (kb + 1 < p.nkb) load_block(kb + 1);
      if (kb == pf_kb) {
        // the epilogue will read this tile's saved coefficients: start pulling their lines into L2 now
        const int lpr = nf * (FT / 32);  // 128-byte lines per row
        for (int idx = tid; idx < RB * lpr; idx += PRODUCERS) {
          const int r = idx / lpr, col = nbase + (idx - r * lpr) * 32;
          if (m0 + r < p.M && col < p.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.Ahat + (size_t)(m0 + r) * p.N + col));
        }
      }
      const int k = kb * BK + c * 4;
      const bool ok = k < p.K;
      if (PRO == PRO_H0) {
#pragma unroll
        for (int i = 0; i < ROWS_PER_THREAD; ++i) {
          if (row0 + i < p.M && ok) {
            const size_t off = (size_t)dom[i] * p.K;
            const float4 md = ldk(p.mid_k + off, k);
            const float4 rd = ldk(p.rad_k + off, k);
            // lanes of this float4 beyond K stay 0: a, mid and rad were all loaded guarded
            float4 a = a_cur[i];
            a.x = md.x - sgnf(a.x) * rd.x; a.y = md.y - sgnf(a.y) * rd.y;
            a.z = md.z - sgnf(a.z) * rd.z; a.w = md.w - sgnf(a.w) * rd.w;
            a_cur[i] = a;
          }
        }
      }
      const int s = kb % P_STAGES;
      const uint32_t phase = (uint32_t)(kb / P_STAGES) & 1u;
      if (!mbar_wait(smem_u32(&ctl->p_empty[s]), phase ^ 1u, abort_flag)) { alive = false; break; }
      unsigned char* t_hi = tiles + (size_t)s * 2 * P_TILE;
      unsigned char* t_lo = t_hi + P_TILE;
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) {
        const float4 a = a_cur[i];
        float4 hi, lo;
        hi.x = tf32_round(a.x); hi.y = tf32_round(a.y); hi.z = tf32_round(a.z); hi.w = tf32_round(a.w);
        lo.x = tf32_round(a.x - hi.x); lo.y = tf32_round(a.y - hi.y); lo.z = tf32_round(a.z - hi.z); lo.w = tf32_round(a.w - hi.w);
        const int rl = rg * ROWS_PER_THREAD + i;  // row inside the tile; 8-row swizzle atoms
        const int off = (rl >> 3) * 1024 + (rl & 7) * 128 + ((c ^ (rl & 7)) << 4);
        *reinterpret_cast<float4*>(t_hi + off) = hi;
        *reinterpret_cast<float4*>(t_lo + off) = lo;
      }
      fence_proxy_async();
      mbar_arrive(smem_u32(&ctl->p_full[s]));
    }

    // ------------------------------------------------------------------ epilogue (same sixteen warps)
    if (alive && mbar_wait(smem_u32(&ctl->accum), 0, abort_flag)) {
      tc_fence_after();
      {
        // The CTA that will start when this wave retires reads its first k-blocks from cold HBM pages;
        // pull those lines into L2 now (L2 is shared, so it does not matter which SM runs that CTA).
        const int lin = (int)(blockIdx.x + gridDim.x * blockIdx.y) + p.wave;
        const int ny = lin / (int)gridDim.x;  // its row block
        if (ny < (int)gridDim.y) {
          const int r = tid >> 1, half = tid & 1;  // 256 rows x two 128-byte k-blocks
          const int m = ny * RB + r;
          if (m < p.M && (half * BK) < p.K) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.A + (size_t)m * p.K + half * BK));
        }
      }
      const int q = warp & 3;          // tensor-memory lane quarter = features q*32 .. q*32+31 of a feature tile
      const int part = warp >> 2;      // this warp takes row chunks part, part + 4
      const int D = (p.M + p.S - 1) / p.S;
      // byte offsets inside this CTA's 256-row slab stay below 2^32 (N < 2^22 features)
      const unsigned rowstride = (unsigned)p.N * 4u;
      const char* __restrict__ ahat_cta = reinterpret_cast<const char*>(p.Ahat + (size_t)m0 * p.N);
      char* __restrict__ hout_cta = reinterpret_cast<char*>(p.hout + (size_t)m0 * p.N);
      // All MMAs have completed, so the pipeline stages are free: each warp keeps two slope tables there
      // (double buffer: the next chunk's slopes are copied asynchronously while the current chunk is processed).
      float* tbl = reinterpret_cast<float*>(tiles) + warp * (2 * TBL_FLOATS) + lane;
      const int nchunks = 2 * nf;  // chunk i: feature tile i >> 1, row chunk part + 4 * (i & 1)
      auto chunk_geom = [&](int i, int& t, int& rbase, int& d0, int& nd) -> bool {
        t = i >> 1;
        rbase = m0 + (part + (WARPS / 4) * (i & 1)) * 32;
        if (i >= nchunks || rbase >= p.M || nbase + t * FT + q * 32 >= p.N) return false;
        d0 = rbase / p.S;
        nd = min(rbase + 31, p.M - 1) / p.S - d0 + 1;
        return true;
      };
      auto feature_of = [&](int t) { return min(nbase + t * FT + q * 32 + lane, p.N - 1); };
      {
        int t, rbase, d0, nd;
        if (chunk_geom(0, t, rbase, d0, nd) && nd <= TBLD) table_fill(p, tbl, d0, nd, feature_of(t));
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
      for (int i = 0; i < nchunks; ++i) {
        {
          int t, rbase, d0, nd;
          if (chunk_geom(i + 1, t, rbase, d0, nd) && nd <= TBLD) table_fill(p, tbl + ((i + 1) & 1) * TBL_FLOATS, d0, nd, feature_of(t));
          asm volatile("cp.async.commit_group;" ::: "memory");
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // this chunk's table has landed
        int t, rbase, d, nd;
        if (!chunk_geom(i, t, rbase, d, nd)) continue;
        const int n_raw = nbase + t * FT + q * 32 + lane;
        const bool n_ok = n_raw < p.N;
        const int n = min(n_raw, p.N - 1);             // addresses stay valid; stores and sums are predicated on n_ok
        const bool st_ok = n_ok && p.hout != nullptr;
        const float nb = p.nbias ? __ldg(p.nbias + n) : 0.f;
        const int ch = (rbase - m0) >> 5;
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(t * RB + ch * 32);
        const int rl = rbase + lane;
        const unsigned vmask = __ballot_sync(0xffffffffu, rl < p.M);
        const unsigned bmask = __ballot_sync(0xffffffffu, (rl + 1) % p.S == 0 || rl == p.M - 1 || lane == 31) & vmask;
        const unsigned off = (unsigned)(ch * 32) * rowstride + (unsigned)n * 4u;
        const float* tb = tbl + (i & 1) * TBL_FLOATS;
        if (nd <= TBLD)
          adjoint_chunk<true>(p, taddr, ahat_cta, hout_cta, off, rowstride, n, n_ok, st_ok, nb, d, D, vmask, bmask, tb, nd);
        else
          adjoint_chunk<false>(p, taddr, ahat_cta, hout_cta, off, rowstride, n, n_ok, st_ok, nb, d, D, vmask, bmask, tb, nd);
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      tc_fence_before();
    }
  } else if (warp == COPY_WARP) {
    // ------------------------------------------------------------------ bulk-copy issue for the weight images
    if (lane == 0) {
      int it = 0;
      for (int kb = 0; kb < p.nkb; ++kb) {
        for (int t = 0; t < nf; ++t, ++it) {
          const int s = it % S_STAGES;
          const uint32_t phase = (uint32_t)(it / S_STAGES) & 1u;
          if (!mbar_wait(smem_u32(&ctl->s_empty[s]), phase ^ 1u, abort_flag)) { kb = p.nkb; break; }
          const uint32_t bar = smem_u32(&ctl->s_full[s]);
          const unsigned char* src = p.Wpk + ((size_t)(ft0 + t) * p.nkb + kb) * (2 * S_TILE);
          mbar_arrive_expect_tx(bar, (uint32_t)(2 * S_TILE));
          bulk_copy_g2s(smem_u32(s_tiles + (size_t)s * 2 * S_TILE), src, (uint32_t)(2 * S_TILE), bar);
        }
      }
      copies_issued = it;
    }
  } else {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      // D[features, rows] += W_tile[features, k] * H_tile[rows, k]^T: M = 128 features, N = 256 rows, both operands K-major
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(RB >> 3) << 17) | ((uint32_t)(FT >> 4) << 24);
      // descriptors of stage 0; a stage (or the lo image) further on is a plain add (the 14-bit address field cannot
      // overflow: shared-memory addresses stay below 256 KB)
      const uint64_t h_desc0 = make_desc(smem_u32(tiles)), w_desc0 = make_desc(smem_u32(s_tiles));
      bool ok = true;
      int it = 0;
      for (int kb = 0; kb < p.nkb && ok; ++kb) {
        const int sp = kb % P_STAGES;
        if (!mbar_wait(smem_u32(&ctl->p_full[sp]), (uint32_t)(kb / P_STAGES) & 1u, abort_flag)) { ok = false; break; }
        const uint64_t dhh = h_desc0 + (uint64_t)(sp * ((2 * P_TILE) >> 4));
        for (int t = 0; t < nf; ++t, ++it) {
          const int ss = it % S_STAGES;
          if (!mbar_wait(smem_u32(&ctl->s_full[ss]), (uint32_t)(it / S_STAGES) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t dwh = w_desc0 + (uint64_t)(ss * ((2 * S_TILE) >> 4));
          const uint32_t d_tmem = tmem_base + (uint32_t)(t * RB);
          mma_kblock_3xtf32(d_tmem, dwh, dwh + (S_TILE >> 4), dhh, dhh + (P_TILE >> 4), idesc, kb > 0 ? 1u : 0u);
          mma_commit(smem_u32(&ctl->s_empty[ss]));  // frees the weight stage when these MMAs have read it
        }
        if (ok) mma_commit(smem_u32(&ctl->p_empty[sp]));
      }
      if (ok) mma_commit(smem_u32(&ctl->accum));
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncthreads();
  if (ctl->abort_flag) {
    if (tid == 0 && p.status) atomicExch(p.status, 1);
    // bulk copies that were already issued must land before the CTA's shared memory is released
    if (warp == COPY_WARP && lane == 0) drain_bulk_copies(ctl->s_full, S_STAGES, copies_issued);
    __syncthreads();
  }
  if (warp == MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

}  // namespace tca

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

template <int PRO>
static int tca_launch(tca::Params& p, cudaStream_t stream, const char* name) {
  static SmemOptIn opt_in;
  if (int rc = ensure_dynamic_smem(tca::crown_tc_adjoint_kernel<PRO>, tca::SMEM_BYTES, opt_in, name)) return rc;
  dim3 grid((p.nft + 1) / 2, ceil_div(p.M, tca::RB));
  tca::crown_tc_adjoint_kernel<PRO><<<grid, tca::THREADS, tca::SMEM_BYTES, stream>>>(p);
  BF_CHECK_LAUNCH(name);
  g_tc_launches.fetch_add(1, std::memory_order_relaxed);
  return BF_OK;
}

int tc_adjoint_tile_rows() { return tca::FT; }

int launch_crown_adjoint_linear_tc_fm(const float* Hprev, int first_layer, const float* mid, const float* rad,
                                      const unsigned char* Wpk, const float* nbias, const float* Ahat, const float* dpos,
                                      const float* dneg, const float* epos, const float* eneg, const float* pre_l,
                                      const float* pre_u, float* hout, float* grad, float* gsum, int M, int S, int K, int N,
                                      int* status, cudaStream_t stream) {
  tca::Params p{};
  p.A = Hprev; p.Wpk = Wpk; p.M = M; p.N = N; p.K = K; p.S = S;
  p.nkb = (K + tca::BK - 1) / tca::BK;
  p.nft = (N + tca::FT - 1) / tca::FT;
  p.vecK = (K % 4 == 0);
  const void* kptrs[] = {Hprev, mid, rad};
  for (const void* q : kptrs) if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) p.vecK = 0;
  p.mid_k = mid; p.rad_k = rad;
  p.nbias = nbias; p.Ahat = Ahat; p.dpos = dpos; p.dneg = dneg; p.epos = epos; p.eneg = eneg;
  p.pre_l = pre_l; p.pre_u = pre_u; p.hout = hout; p.grad = grad; p.gsum = gsum;
  p.status = status;
  p.wave = sm_count();
  timing_begin(T_ADJ, stream);
  int rc = first_layer ? tca_launch<tca::PRO_H0>(p, stream, "crown_tc_adjoint_kernel<h0>")
                       : tca_launch<tca::PRO_PLAIN>(p, stream, "crown_tc_adjoint_kernel");
  timing_end(T_ADJ, stream, 4.0 * (double)M * K + 8.0 * (double)M * N, 2.0 * (double)M * K * N);
  return rc;
}

}  // namespace bf
