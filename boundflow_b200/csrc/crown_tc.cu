// CROWN backward / adjoint contractions on the 5th-generation tensor cores
// (tcgen05.mma kind::tf32, accumulators in tensor memory) with 3xTF32 split
// operands for fp32-faithful results:
//     a*b ~= a_hi*b_hi + a_lo*b_hi + a_hi*b_lo,   x_hi = tf32(x), x_lo = tf32(x - x_hi)
//
// One CTA computes 128 rows x up to two column sub-tiles of BN columns (BN <= 256, multiple of
// 16; the two accumulators sit side by side in the 512 tensor-memory columns) of
//     C[M,N] = f(A)[M,K] * B[K,N]
// * B (the layer weight, static) is pre-split into hi/lo and pre-packed per (column sub-tile,
//   32-wide k-block) into the exact shared-memory image the MMA reads (K-major rows of 128
//   bytes, 128-byte swizzle); one bulk asynchronous copy (cp.async.bulk, completion on an
//   mbarrier) brings a k-block's hi+lo image in.
// * A changes per call and needs the ReLU-backward prologue (sign-selected slope per domain,
//   intercept and bias row sums), so sixteen producer warps load it with coalesced 128-bit
//   loads (one k-block ahead in registers, further ahead as L2 prefetches), transform, split
//   and write the swizzled hi/lo tiles; one produced k-block feeds both sub-tiles' MMAs.
// * One thread issues the MMAs; tcgen05.commit releases shared-memory stages and finally
//   signals the same sixteen warps, which read the accumulators with tcgen05.ld, transpose
//   32x32 blocks through shared memory and do coalesced 128-bit row accesses (store, fused
//   concretisation partial sums, or the adjoint step with its per-domain gradient sums).
// Every wait is bounded: on expiry the CTA raises a status word, stops, frees its tensor
// memory and returns (the host reports the status; nothing traps).
#include <stdlib.h>

#include "kernels.cuh"
#include "tc_primitives.cuh"

namespace bf {
namespace tc {

constexpr int BM = 128;
constexpr int BK = 32;                  // fp32 per k-block row = 128 bytes
constexpr int MAX_BN = 256;
constexpr int A_TILE = BM * BK * 4;     // bytes of one A tile (hi or lo)
constexpr int A_STAGES = 2;
constexpr int MAX_B_STAGES = 4;
constexpr int PROD_WARPS = 16;
constexpr int ROWS_PER_THREAD = BM / (PROD_WARPS * 4);  // 8 threads cover one 128-byte row
constexpr int COL_PARTS = PROD_WARPS / 4;               // epilogue warps per TMEM lane quarter
constexpr int PRODUCERS = PROD_WARPS * 32;
constexpr int COPY_WARP = PROD_WARPS;       // bulk-copy issue
constexpr int MMA_WARP = PROD_WARPS + 1;    // MMA issue, TMEM alloc / free
constexpr int THREADS = (PROD_WARPS + 2) * 32;
constexpr int PREFETCH_KB = 4;              // k-blocks of L2 prefetch distance for the A operand
constexpr int TBL_MAX = 5;                  // domains per 32 rows served from the epilogue's slope table (S >= 8)
constexpr int STG_LD = 36;                  // leading dimension of the per-warp epilogue transpose buffer

enum { MODE_BWD = 0, MODE_ADJ = 1 };
enum { PRO_PLAIN = 0, PRO_RELU = 1, PRO_H0 = 2 };

struct Params {
  // operands
  const float* A;            // [M,K]
  const unsigned char* Bpk;  // packed hi/lo images, [ntiles][nkb][2][BN][128 B]
  int M, N, K, S, BN, nkb, ntiles, b_stages;
  int vecK, vecN;
  // prologue (see gemm_ffma.cuh for the meaning)
  const float* dpos; const float* dneg; const float* epos; const float* eneg; const float* add; const float* kbias;
  const float* mid_k; const float* rad_k;   // PRO_H0: [D,K]
  float* delta; int accumulate;
  // backward epilogue
  float* out;                // [M,N] or null
  const float* mid_n; const float* rad_n;   // [D,N] with `partial`
  float* partial;            // [M, COL_PARTS*gridDim.y] or null
  float conc_sign;           // -1 lower, +1 upper
  // adjoint epilogue
  const float* nbias; const float* Ahat; const float* e_dpos; const float* e_dneg; const float* e_epos; const float* e_eneg;
  const float* pre_l; const float* pre_u; float* hout; float* grad;
  float* gsum;               // [D,N] or null: per-domain sums of g (beta gradient)
  const float* gw;           // [M] or null: weight of each row in gsum (d objective / d row for min / softmin)
  int* status;               // device word, set non-zero when a wait expired
};

// Shared-memory control block placed in front of the (1024-byte aligned) tiles.
struct Control {
  unsigned long long a_full[A_STAGES];
  unsigned long long a_empty[A_STAGES];
  unsigned long long b_full[MAX_B_STAGES];
  unsigned long long b_empty[MAX_B_STAGES];
  unsigned long long accum;
  unsigned long long peer_b_full[MAX_B_STAGES];  // CTA pairs: in the leader, "the peer's B stage has landed"
  uint32_t tmem_base;
  int abort_flag;
};

// Work split of one CTA (THREADS = 576):
//   warps 0-15  A producers during the main loop (ROWS_PER_THREAD tile rows x one 16-byte chunk per
//               thread and k-block), then the epilogue (warp w reads TMEM lane quarter w%4, column
//               chunks w/4, w/4 + COL_PARTS, ...)
//   warp 16     lane 0 issues the bulk copies of the packed weight images
//   warp 17     lane 0 issues the MMAs; the warp allocates / frees tensor memory
// A CTA owns 128 rows and up to two column sub-tiles of BN columns (accumulators side by side in
// tensor memory), so one produced A k-block feeds two sets of MMAs.
//
// PAIR: two CTAs of a cluster (consecutive row blocks, same column sub-tiles) run as one tcgen05 cta_group::2 unit.
// Each CTA produces its own 128 A rows and copies HALF of each weight image (rows [rank*BN/2, +BN/2) of hi and lo);
// the leader (cluster rank 0) issues 256-row MMAs that make each CTA's tensor core read its own A tile and its own
// B half, so the shared-memory operand traffic per CTA and k-block falls from 2 x (A + B) to 2 x A + B.  Producers of
// both CTAs arrive on the leader's a_full; the peer's MMA warp forwards "B half landed" to the leader; the leader's
// commits arrive on the stage / accumulator barriers of both CTAs.
// Status: opt-in (BF_B200_BWD_PAIRS=1), bit-identical results.  Measured on B200 over the backward launches of a
// 8192-subdomain alpha step (73728 rows, 512- and 784-wide layers): 277 us per launch against 243 us for independent
// CTAs.  A third less operand traffic per CTA does not pay for coupling two CTAs' producers to one MMA stream with two
// A stages: the MMAs of a k-block now wait for the slower of 32 producer warps.
template <int MODE, int PRO, bool PAIR>
__global__ void __launch_bounds__(THREADS, 1) crown_tc_kernel(Params p) {
  extern __shared__ unsigned char raw_smem[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1024 + 1023) & ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(tiles - 1024);
  unsigned char* b_tiles = tiles + A_STAGES * 2 * A_TILE;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * BM;
  const int nt0 = blockIdx.y * 2;                       // first column sub-tile of this CTA
  const int nh = min(2, p.ntiles - nt0);                // sub-tiles handled here
  const int ncol0 = nt0 * p.BN;                         // first global column
  const int ncols = nh * p.BN;                          // accumulator columns in use
  const int b_bytes = 2 * p.BN * 128;                   // hi + lo image of one k-block of one sub-tile
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // position in the CTA pair; 0 leads
  const int b_stage_bytes = PAIR ? b_bytes / 2 : b_bytes;  // a pair member holds half of the rows of both images
  const uint32_t tmem_cols = (ncols <= 256) ? 256u : 512u;
  volatile int* abort_flag = &ctl->abort_flag;
  int copies_issued = 0;  // bulk copies this thread has issued (meaningful in the copy thread only)

  if (tid == 0) {
    for (int s = 0; s < A_STAGES; ++s) {
      mbar_init(smem_u32(&ctl->a_full[s]), PAIR ? 2 * PROD_WARPS : PROD_WARPS);
      mbar_init(smem_u32(&ctl->a_empty[s]), 1);
    }
    for (int s = 0; s < p.b_stages; ++s) {
      mbar_init(smem_u32(&ctl->b_full[s]), 1);
      mbar_init(smem_u32(&ctl->b_empty[s]), 1);
      mbar_init(smem_u32(&ctl->peer_b_full[s]), 1);
    }
    mbar_init(smem_u32(&ctl->accum), 1);
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    if (PAIR) {  // the same warp of both CTAs allocates the same columns
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(tmem_cols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(tmem_cols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp < PROD_WARPS) {
    // ------------------------------------------------------------------ A producers
    const int c = tid & 7;        // 16-byte chunk inside the 128-byte k-block row
    const int rg = tid >> 3;      // row pair of this thread
    const int row0 = m0 + rg * ROWS_PER_THREAD;
    const bool vK = p.vecK != 0;
    // every k-block is complete and 16-byte aligned (the usual case): loads need no bounds logic
    const bool fastK = vK && (p.K % BK == 0);
    auto ldk = [&](const float* row, int k) -> float4 {
      if (fastK) return __ldg(reinterpret_cast<const float4*>(row + k));
      return (k < p.K) ? load4_guard(row, k, p.K, vK) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    const bool want_delta = (PRO == PRO_RELU) && p.delta != nullptr && blockIdx.y == 0;
    int dom[ROWS_PER_THREAD];
#pragma unroll
    for (int i = 0; i < ROWS_PER_THREAD; ++i) dom[i] = (row0 + i < p.M) ? ((row0 + i) / p.S) : 0;
    float rowacc[ROWS_PER_THREAD];
#pragma unroll
    for (int i = 0; i < ROWS_PER_THREAD; ++i) rowacc[i] = 0.f;

    // The coefficient rows stream from HBM: they are loaded one k-block ahead into registers and
    // their lines are pulled into L2 PREFETCH_KB k-blocks ahead.  The per-domain slope vectors are
    // L2-resident and are loaded when a k-block is processed.
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
    for (int kb = 0; kb < p.nkb; ++kb) {
      float4 a_cur[ROWS_PER_THREAD];
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) a_cur[i] = a_next[i];
      if (kb + 1 < p.nkb) load_block(kb + 1);
      if (MODE == MODE_ADJ && kb == 1) {
        // the epilogue will read this tile's saved coefficients: start pulling their lines into L2 now
        const int lpr = (ncols + 31) >> 5;  // 128-byte lines per row
        for (int idx = tid; idx < BM * lpr; idx += PRODUCERS) {
          const int r = idx / lpr, col = ncol0 + (idx - r * lpr) * 32;
          if (m0 + r < p.M && col < p.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.Ahat + (size_t)(m0 + r) * p.N + col));
        }
      }

      const int k = kb * BK + c * 4;
      const bool ok = k < p.K;
      const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
      float4 kbv = z4;
      float4 sv[ROWS_PER_THREAD][5];  // dpos, dneg, epos|mid, eneg|rad, add of each row's domain
      if (PRO == PRO_RELU) {
        if (want_delta && p.kbias) kbv = ldk(p.kbias, k);
        if (p.dpos) {
#pragma unroll
          for (int i = 0; i < ROWS_PER_THREAD; ++i) {
            const size_t off = (size_t)dom[i] * p.K;
            sv[i][0] = ldk(p.dpos + off, k);
            sv[i][1] = ldk(p.dneg + off, k);
            sv[i][2] = (want_delta && p.epos) ? ldk(p.epos + off, k) : z4;
            sv[i][3] = (want_delta && p.eneg) ? ldk(p.eneg + off, k) : z4;
            sv[i][4] = p.add ? ldk(p.add + off, k) : z4;
          }
        }
      } else if (PRO == PRO_H0) {
#pragma unroll
        for (int i = 0; i < ROWS_PER_THREAD; ++i) {
          const size_t off = (size_t)dom[i] * p.K;
          sv[i][2] = ldk(p.mid_k + off, k);
          sv[i][3] = ldk(p.rad_k + off, k);
        }
      }

      const int s = kb % A_STAGES;
      const uint32_t phase = (uint32_t)(kb / A_STAGES) & 1u;
      if (!mbar_wait_warp(smem_u32(&ctl->a_empty[s]), phase ^ 1u, abort_flag)) { alive = false; break; }  // warp-uniform outcome
      unsigned char* a_hi = tiles + (size_t)s * 2 * A_TILE;
      unsigned char* a_lo = a_hi + A_TILE;
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) {
        float4 a = a_cur[i];
        const int m = row0 + i;
        if (PRO == PRO_RELU) {
          if (p.dpos != nullptr && m < p.M) {
            const float4 dp = sv[i][0], dn = sv[i][1], ep = sv[i][2], en = sv[i][3], ad = sv[i][4];
            if (want_delta) {
              float r = rowacc[i];
#define BF_TC_SEL(cc)                                       \
  {                                                         \
    const bool sel = a.cc >= 0.f;                           \
    const float lam = a.cc * (sel ? dp.cc : dn.cc) + ad.cc; \
    r = fmaf(a.cc, sel ? ep.cc : en.cc, r);                 \
    r = fmaf(lam, kbv.cc, r);                               \
    a.cc = lam;                                             \
  }
              BF_TC_SEL(x) BF_TC_SEL(y) BF_TC_SEL(z) BF_TC_SEL(w)
#undef BF_TC_SEL
              rowacc[i] = r;
            } else {
              a.x = a.x * (a.x >= 0.f ? dp.x : dn.x) + ad.x;
              a.y = a.y * (a.y >= 0.f ? dp.y : dn.y) + ad.y;
              a.z = a.z * (a.z >= 0.f ? dp.z : dn.z) + ad.z;
              a.w = a.w * (a.w >= 0.f ? dp.w : dn.w) + ad.w;
            }
          } else if (want_delta) {
            rowacc[i] += a.x * kbv.x + a.y * kbv.y + a.z * kbv.z + a.w * kbv.w;
          }
        } else if (PRO == PRO_H0) {
          if (m < p.M && ok) {
            const float4 md = sv[i][2], rd = sv[i][3];
            // lanes of this float4 beyond K stay 0: a, mid and rad were all loaded guarded
            a.x = md.x - sgnf(a.x) * rd.x; a.y = md.y - sgnf(a.y) * rd.y;
            a.z = md.z - sgnf(a.z) * rd.z; a.w = md.w - sgnf(a.w) * rd.w;
          }
        }
        float4 hi, lo;
        hi.x = tf32_round(a.x); hi.y = tf32_round(a.y); hi.z = tf32_round(a.z); hi.w = tf32_round(a.w);
        lo.x = tf32_round(a.x - hi.x); lo.y = tf32_round(a.y - hi.y); lo.z = tf32_round(a.z - hi.z); lo.w = tf32_round(a.w - hi.w);
        const int rl = rg * ROWS_PER_THREAD + i;  // row inside the tile; 8-row swizzle atoms
        const int off = (rl >> 3) * 1024 + (rl & 7) * 128 + ((c ^ (rl & 7)) << 4);
        *reinterpret_cast<float4*>(a_hi + off) = hi;
        *reinterpret_cast<float4*>(a_lo + off) = lo;
      }
      fence_proxy_async();
      // one arrival per warp: every lane has made its writes visible to the async proxy; the warp barrier orders them
      // before lane 0's releasing arrive (512 separate arrivals on one barrier word would serialise in shared memory)
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->a_full[s]), 0));
        else mbar_arrive(smem_u32(&ctl->a_full[s]));
      }
    }

    if (PRO == PRO_RELU) {
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) {
        float v = rowacc[i];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        const int m = row0 + i;
        if (alive && want_delta && c == 0 && m < p.M) p.delta[m] = p.accumulate ? (p.delta[m] + v) : v;
      }
    }

    // ------------------------------------------------------------------ epilogue (same eight warps)
    if (alive && mbar_wait(smem_u32(&ctl->accum), 0, abort_flag)) {
      tc_fence_after();
      const int q = warp & 3;          // TMEM lane quarter = rows q*32 .. q*32+31 of the tile
      const int part = warp >> 2;      // this warp takes every COL_PARTS-th 32-column chunk
      float* stg = reinterpret_cast<float*>(tiles) + warp * (32 * STG_LD);  // per-warp 32 x 36 transpose buffer
      const int row_base = m0 + q * 32;
      const int my_row = row_base + lane;  // thread-per-row view right after tcgen05.ld
      const int rs = lane >> 3, c4 = lane & 7;  // (row sub-index, 16-byte column chunk) view after the transpose
      const bool vN = p.vecN != 0;
      float conc = 0.f;
      // adjoint: domains covered by this warp's 32 rows and their per-chunk table
      float* tbl = reinterpret_cast<float*>(tiles) + PROD_WARPS * (32 * STG_LD) + warp * (TBL_MAX * 5 * 32);
      float* stg2 = reinterpret_cast<float*>(tiles) + PROD_WARPS * (32 * STG_LD + TBL_MAX * 5 * 32) + warp * (32 * 33);  // g itself, for the beta gradient
      const int d0 = (row_base < p.M) ? row_base / p.S : 0;
      const int nd = (row_base < p.M) ? (min(row_base + 31, p.M - 1) / p.S - d0 + 1) : 0;
      const bool tbl_ok = nd <= TBL_MAX;
      for (int c0 = part * 32; c0 < ncols; c0 += 32 * COL_PARTS) {
        float v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
        const int colbase = ncol0 + c0;
        if (MODE == MODE_BWD && p.partial != nullptr && my_row < p.M) {
          const size_t off = (size_t)(my_row / p.S) * p.N;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int col = colbase + j;
            if (col < p.N) {
              const float4 md = load4_guard(p.mid_n + off, col, p.N, vN);
              const float4 rd = load4_guard(p.rad_n + off, col, p.N, vN);
              conc += v[j] * md.x + p.conc_sign * fabsf(v[j]) * rd.x;
              conc += v[j + 1] * md.y + p.conc_sign * fabsf(v[j + 1]) * rd.y;
              conc += v[j + 2] * md.z + p.conc_sign * fabsf(v[j + 2]) * rd.z;
              conc += v[j + 3] * md.w + p.conc_sign * fabsf(v[j + 3]) * rd.w;
            }
          }
        }
        const bool need_rows = (MODE == MODE_ADJ) || (p.out != nullptr);
        if (!need_rows) continue;
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(&stg[lane * STG_LD + 4 * j]) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        __syncwarp();
        const int col = colbase + c4 * 4;
        if (MODE == MODE_BWD) {
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + rs;
            const int row = row_base + r;
            if (row < p.M && col < p.N) {
              const float4 val = *reinterpret_cast<const float4*>(&stg[r * STG_LD + c4 * 4]);
              store4_guard(p.out + (size_t)row * p.N, col, p.N, vN, val);
            }
          }
        } else {
          // All loads of this chunk are issued before any is consumed: the coefficient rows
          // (one float4 per (row, 4 columns)), and one table row per domain of this warp's 32
          // rows with the slopes / intercepts / unstable flag of the chunk's 32 columns.
          float4 nb = make_float4(0.f, 0.f, 0.f, 0.f);
          if (p.nbias && col < p.N) nb = load4_guard(p.nbias, col, p.N, vN);
          float4 ah[8];
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int row = row_base + it * 4 + rs;
            ah[it] = (row < p.M && col < p.N) ? load4_guard(p.Ahat + (size_t)row * p.N, col, p.N, vN) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
          if (tbl_ok) {
            const int colj = colbase + lane;
            float t[TBL_MAX][5];
#pragma unroll
            for (int dl = 0; dl < TBL_MAX; ++dl) {
              const bool okd = dl < nd && colj < p.N;
              const size_t off = (size_t)(d0 + (okd ? dl : 0)) * p.N + (okd ? colj : 0);
              t[dl][0] = okd ? __ldg(p.e_dpos + off) : 0.f;
              t[dl][1] = okd ? __ldg(p.e_dneg + off) : 0.f;
              t[dl][2] = (okd && p.e_epos) ? __ldg(p.e_epos + off) : 0.f;
              t[dl][3] = (okd && p.e_eneg) ? __ldg(p.e_eneg + off) : 0.f;
              const float pl = okd ? __ldg(p.pre_l + off) : 0.f;
              const float pu = okd ? __ldg(p.pre_u + off) : 0.f;
              t[dl][4] = (pl < 0.f && pu > 0.f) ? 1.f : 0.f;
            }
#pragma unroll
            for (int dl = 0; dl < TBL_MAX; ++dl)
#pragma unroll
              for (int a5 = 0; a5 < 5; ++a5) tbl[(dl * 5 + a5) * 32 + lane] = t[dl][a5];
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + rs;
            const int row = row_base + r;
            float4 contrib = make_float4(0.f, 0.f, 0.f, 0.f);
            float4 ggv = contrib;
            if (row < p.M && col < p.N) {
              const float4 g4 = *reinterpret_cast<const float4*>(&stg[r * STG_LD + c4 * 4]);
              ggv = make_float4(g4.x + nb.x, g4.y + nb.y, g4.z + nb.z, g4.w + nb.w);
              const int d = row / p.S;
              float4 dp, dn, ep, en, am;
              if (tbl_ok) {
                const float* tb = tbl + (size_t)(d - d0) * 5 * 32 + c4 * 4;
                dp = *reinterpret_cast<const float4*>(tb);
                dn = *reinterpret_cast<const float4*>(tb + 32);
                ep = *reinterpret_cast<const float4*>(tb + 64);
                en = *reinterpret_cast<const float4*>(tb + 96);
                am = *reinterpret_cast<const float4*>(tb + 128);
              } else {  // more than TBL_MAX domains inside 32 rows (small S): direct loads
                const size_t off = (size_t)d * p.N;
                dp = load4_guard(p.e_dpos + off, col, p.N, vN);
                dn = load4_guard(p.e_dneg + off, col, p.N, vN);
                ep = make_float4(0.f, 0.f, 0.f, 0.f);
                en = ep;
                if (p.e_epos) ep = load4_guard(p.e_epos + off, col, p.N, vN);
                if (p.e_eneg) en = load4_guard(p.e_eneg + off, col, p.N, vN);
                const float4 pl = load4_guard(p.pre_l + off, col, p.N, vN);
                const float4 pu = load4_guard(p.pre_u + off, col, p.N, vN);
                am.x = (pl.x < 0.f && pu.x > 0.f) ? 1.f : 0.f; am.y = (pl.y < 0.f && pu.y > 0.f) ? 1.f : 0.f;
                am.z = (pl.z < 0.f && pu.z > 0.f) ? 1.f : 0.f; am.w = (pl.w < 0.f && pu.w > 0.f) ? 1.f : 0.f;
              }
              const float4 a4 = ah[it];
              float4 h;
#define BF_TC_ADJ(cc)                                                 \
  {                                                                   \
    const float gg = g4.cc + nb.cc;                                   \
    const bool sel = a4.cc >= 0.f;                                    \
    h.cc = (sel ? dp.cc : dn.cc) * gg + (sel ? ep.cc : en.cc);        \
    contrib.cc = (sel && am.cc != 0.f) ? a4.cc * gg : 0.f;            \
  }
              BF_TC_ADJ(x) BF_TC_ADJ(y) BF_TC_ADJ(z) BF_TC_ADJ(w)
#undef BF_TC_ADJ
              if (p.hout) store4_guard(p.hout + (size_t)row * p.N, col, p.N, vN, h);
            }
            *reinterpret_cast<float4*>(&stg[r * STG_LD + c4 * 4]) = contrib;  // in place: same lane read this chunk
            if (p.gsum) {
              float* g2 = stg2 + r * 33 + c4 * 4;
              g2[0] = (col + 0 < p.N) ? ggv.x : 0.f; g2[1] = (col + 1 < p.N) ? ggv.y : 0.f;
              g2[2] = (col + 2 < p.N) ? ggv.z : 0.f; g2[3] = (col + 3 < p.N) ? ggv.w : 0.f;
            }
          }
          __syncwarp();
          // per-domain column sums over this warp's 32 rows; at most two warps/tiles touch one (domain, column)
          const int colj = colbase + lane;
          const int nrows = min(32, p.M - row_base);
          if (tbl_ok) {
#pragma unroll
            for (int dl = 0; dl < TBL_MAX; ++dl) {
              if (dl < nd) {
                const int r_lo = max((d0 + dl) * p.S - row_base, 0);
                const int r_hi = min((d0 + dl + 1) * p.S - row_base, nrows);
                float run = 0.f;
                for (int r = r_lo; r < r_hi; ++r) run += stg[r * STG_LD + lane];
                if (colj < p.N) atomicAdd(&p.grad[(size_t)(d0 + dl) * p.N + colj], run);
              }
            }
          } else {
            float run = 0.f;
            int run_d = -1;
            for (int r = 0; r < nrows; ++r) {
              const int d = (row_base + r) / p.S;
              if (d != run_d) {
                if (run_d >= 0 && colj < p.N) atomicAdd(&p.grad[(size_t)run_d * p.N + colj], run);
                run = 0.f;
                run_d = d;
              }
              run += stg[r * STG_LD + lane];
            }
            if (run_d >= 0 && colj < p.N) atomicAdd(&p.grad[(size_t)run_d * p.N + colj], run);
          }
          if (p.gsum) {
            float run = 0.f;
            int run_d = -1;
            for (int r = 0; r < nrows; ++r) {
              const int d = (row_base + r) / p.S;
              if (d != run_d) {
                if (run_d >= 0 && colj < p.N) atomicAdd(&p.gsum[(size_t)run_d * p.N + colj], run);
                run = 0.f;
                run_d = d;
              }
              run = p.gw ? fmaf(__ldg(p.gw + row_base + r), stg2[r * 33 + lane], run) : run + stg2[r * 33 + lane];
            }
            if (run_d >= 0 && colj < p.N) atomicAdd(&p.gsum[(size_t)run_d * p.N + colj], run);
          }
        }
      }
      if (MODE == MODE_BWD && p.partial != nullptr && my_row < p.M)
        p.partial[(size_t)my_row * (COL_PARTS * gridDim.y) + COL_PARTS * blockIdx.y + part] = conc;
      tc_fence_before();
    }
  } else if (warp == COPY_WARP) {
    // ------------------------------------------------------------------ bulk-copy issue for B
    if (lane == 0) {
      int it = 0;
      for (int kb = 0; kb < p.nkb; ++kb) {
        for (int h = 0; h < nh; ++h, ++it) {
          const int s = it % p.b_stages;
          const uint32_t phase = (uint32_t)(it / p.b_stages) & 1u;
          if (!mbar_wait(smem_u32(&ctl->b_empty[s]), phase ^ 1u, abort_flag)) { kb = p.nkb; break; }
          const uint32_t bar = smem_u32(&ctl->b_full[s]);
          const unsigned char* src = p.Bpk + ((size_t)(nt0 + h) * p.nkb + kb) * b_bytes;
          mbar_arrive_expect_tx(bar, (uint32_t)b_stage_bytes);
          if (PAIR) {  // this CTA's half of the rows of the hi image, then of the lo image
            const uint32_t half = (uint32_t)b_stage_bytes / 2;
            const uint32_t dst = smem_u32(b_tiles + (size_t)s * b_stage_bytes);
            bulk_copy_g2s(dst, src + rank * half, half, bar);
            bulk_copy_g2s(dst + half, src + (size_t)p.BN * 128 + rank * half, half, bar);
          } else {
            bulk_copy_g2s(smem_u32(b_tiles + (size_t)s * b_bytes), src, (uint32_t)b_bytes, bar);
          }
        }
      }
      copies_issued = it;
    }
  } else {
    // ------------------------------------------------------------------ MMA issue
    if (PAIR && rank != 0) {
      // peer of a pair: tell the leader when this CTA's half of a B stage has landed
      if (lane == 0) {
        int it = 0;
        for (int kb = 0; kb < p.nkb; ++kb) {
          for (int h = 0; h < nh; ++h, ++it) {
            const int sb = it % p.b_stages;
            if (!mbar_wait(smem_u32(&ctl->b_full[sb]), (uint32_t)(it / p.b_stages) & 1u, abort_flag)) { kb = p.nkb; break; }
            mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->peer_b_full[sb]), 0));
          }
        }
      }
    } else if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.BN >> 3) << 17) | ((uint32_t)((PAIR ? 2 * BM : BM) >> 4) << 24);
      // descriptors of stage 0; a stage (or the lo image) further on is a plain add (the 14-bit address field cannot
      // overflow: shared-memory addresses stay below 256 KB)
      const uint64_t a_desc0 = make_desc(smem_u32(tiles)), b_desc0 = make_desc(smem_u32(b_tiles));
      bool ok = true;
      int it = 0;
      for (int kb = 0; kb < p.nkb && ok; ++kb) {
        const int sa = kb % A_STAGES;
        if (!mbar_wait(smem_u32(&ctl->a_full[sa]), (uint32_t)(kb / A_STAGES) & 1u, abort_flag)) { ok = false; break; }
        const uint64_t dah = a_desc0 + (uint64_t)(sa * ((2 * A_TILE) >> 4));
        for (int h = 0; h < nh; ++h, ++it) {
          const int sb = it % p.b_stages;
          if (!mbar_wait(smem_u32(&ctl->b_full[sb]), (uint32_t)(it / p.b_stages) & 1u, abort_flag)) { ok = false; break; }
          if (PAIR && !mbar_wait(smem_u32(&ctl->peer_b_full[sb]), (uint32_t)(it / p.b_stages) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t dbh = b_desc0 + (uint64_t)(sb * (b_stage_bytes >> 4));
          const uint32_t d_tmem = tmem_base + (uint32_t)(h * p.BN);
          if (PAIR) {
            mma_kblock_3xtf32_pair(d_tmem, dah, dah + (A_TILE >> 4), dbh, dbh + (uint64_t)(b_stage_bytes >> 5), idesc, kb > 0 ? 1u : 0u);
            mma_commit_pair(smem_u32(&ctl->b_empty[sb]));
          } else {
            mma_kblock_3xtf32(d_tmem, dah, dah + (A_TILE >> 4), dbh, dbh + (uint64_t)((p.BN * 128) >> 4), idesc, kb > 0 ? 1u : 0u);
            mma_commit(smem_u32(&ctl->b_empty[sb]));  // frees the B stage when these MMAs have read it
          }
        }
        if (ok) { if (PAIR) mma_commit_pair(smem_u32(&ctl->a_empty[sa])); else mma_commit(smem_u32(&ctl->a_empty[sa])); }
      }
      if (ok) { if (PAIR) mma_commit_pair(smem_u32(&ctl->accum)); else mma_commit(smem_u32(&ctl->accum)); }
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncthreads();
  if (ctl->abort_flag) {
    if (tid == 0 && p.status) atomicExch(p.status, 1);
    // bulk copies that were already issued must land before the CTA's shared memory is released
    if (warp == COPY_WARP && lane == 0) drain_bulk_copies(ctl->b_full, p.b_stages, copies_issued);
    __syncthreads();
  }
  if (PAIR) {
    // neither CTA may free its tensor memory or leave while the other can still arrive on its barriers or run MMAs
    // that write its accumulators
    tc_fence_before();
    cluster_sync_all();
  }
  if (warp == MMA_WARP) {
    tc_fence_after();
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ---------------------------------------------------------------------------
// Weight packing: B[n][k] (k contiguous) -> per (n-tile, k-block) swizzled hi/lo images
// ---------------------------------------------------------------------------
__global__ void pack_weights_kernel(const float* __restrict__ W, int ldw, int transposed, int N, int K, int BN, int nkb,
                                    unsigned char* __restrict__ out, long long total_chunks) {
  // one thread per 16-byte chunk (4 k values) of one row of one image pair
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_chunks; idx += (long long)gridDim.x * blockDim.x) {
    const int cch = (int)(idx & 7);
    long long t = idx >> 3;
    const int r = (int)(t % BN);
    t /= BN;
    const int kb = (int)(t % nkb);
    const int nt = (int)(t / nkb);
    const int n = nt * BN + r;
    float w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = kb * BK + cch * 4 + q;
      float x = 0.f;
      if (n < N && k < K) x = transposed ? W[(size_t)k * ldw + n] : W[(size_t)n * ldw + k];
      w[q] = x;
    }
    float4 hi, lo;
    hi.x = tf32_rna(w[0]); hi.y = tf32_rna(w[1]); hi.z = tf32_rna(w[2]); hi.w = tf32_rna(w[3]);
    lo.x = tf32_rna(w[0] - hi.x); lo.y = tf32_rna(w[1] - hi.y); lo.z = tf32_rna(w[2] - hi.z); lo.w = tf32_rna(w[3] - hi.w);
    unsigned char* img = out + ((size_t)nt * nkb + kb) * (size_t)(2 * BN * 128);
    const int off = (r >> 3) * 1024 + (r & 7) * 128 + ((cch ^ (r & 7)) << 4);
    *reinterpret_cast<float4*>(img + off) = hi;
    *reinterpret_cast<float4*>(img + (size_t)BN * 128 + off) = lo;
  }
}

}  // namespace tc

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
void tc_tile_shape(int N, int K, int* BN, int* ntiles, int* nkb) {
  const int nt = (N + tc::MAX_BN - 1) / tc::MAX_BN;
  int bn = (N + nt - 1) / nt;
  bn = ((bn + 15) / 16) * 16;
  *BN = bn;
  *ntiles = nt;
  *nkb = (K + tc::BK - 1) / tc::BK;
}

int crown_tc_partial_tiles(int N, int K) {
  int BN, nt, nkb;
  tc_tile_shape(N, K, &BN, &nt, &nkb);
  return tc::COL_PARTS * ((nt + 1) / 2);  // one partial sum per CTA column and epilogue warp group
}

// tile_rows > 0 forces the image height (the feature-major adjoint kernel wants 128-row images)
static void tc_pack_shape(int N, int K, int tile_rows, int* BN, int* nt, int* nkb) {
  tc_tile_shape(N, K, BN, nt, nkb);
  if (tile_rows > 0) {
    *BN = tile_rows;
    *nt = (N + tile_rows - 1) / tile_rows;
  }
}

size_t tc_packed_bytes(int N, int K, int tile_rows) {
  int BN, nt, nkb;
  tc_pack_shape(N, K, tile_rows, &BN, &nt, &nkb);
  return (size_t)nt * nkb * 2 * BN * 128;
}

int tc_pack_weights(const float* W, int rows, int cols, int transposed, unsigned char* out, cudaStream_t stream, int tile_rows) {
  // logical B[n][k]: transposed == 0: W is [N=rows][K=cols]; transposed != 0: W is [K=rows][N=cols]
  const int N = transposed ? cols : rows, K = transposed ? rows : cols;
  int BN, nt, nkb;
  tc_pack_shape(N, K, tile_rows, &BN, &nt, &nkb);
  const long long total = (long long)nt * nkb * BN * 8;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  tc::pack_weights_kernel<<<(int)blocks, 256, 0, stream>>>(W, cols, transposed, N, K, BN, nkb, out, total);
  BF_CHECK_LAUNCH("pack_weights_kernel");
  return BF_OK;
}

static int tc_smem_bytes(int BN, int* b_stages_out) {
  const int b_bytes = 2 * BN * 128;
  int b_stages = (200 * 1024 - tc::A_STAGES * 2 * tc::A_TILE) / b_bytes;
  if (b_stages > tc::MAX_B_STAGES) b_stages = tc::MAX_B_STAGES;
  if (b_stages < 2) b_stages = 2;
  *b_stages_out = b_stages;
  const int mainloop = tc::A_STAGES * 2 * tc::A_TILE + b_stages * b_bytes;
  // the epilogue reuses the tile area for per-warp buffers: transpose block, slope table, second block (beta gradient)
  const int epilogue = tc::PROD_WARPS * (32 * tc::STG_LD + tc::TBL_MAX * 5 * 32 + 32 * 33) * (int)sizeof(float);
  return (mainloop > epilogue ? mainloop : epilogue) + 2048;  // + control block and alignment slack
}

template <int MODE, int PRO, bool PAIR = false>
static int tc_launch(tc::Params& p, int ntiles, cudaStream_t stream, const char* name) {
  int b_stages;
  const int smem = tc_smem_bytes(p.BN, &b_stages);
  p.b_stages = b_stages;
  p.ntiles = ntiles;
  static SmemOptIn opt_in;
  if (int rc = ensure_dynamic_smem(tc::crown_tc_kernel<MODE, PRO, PAIR>, 227 * 1024, opt_in, name)) return rc;
  dim3 grid(ceil_div(p.M, tc::BM), (ntiles + 1) / 2);
  if (PAIR) {
    grid.x = (grid.x + 1) & ~1u;  // whole pairs; a CTA past the last row block produces zero rows and stores nothing
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(tc::THREADS);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, tc::crown_tc_kernel<MODE, PRO, PAIR>, p);
    if (e != cudaSuccess) {
      set_error("%s: cluster launch failed: %s", name, cudaGetErrorString(e));
      return BF_E_CUDA;
    }
  } else {
    tc::crown_tc_kernel<MODE, PRO, PAIR><<<grid, tc::THREADS, smem, stream>>>(p);
  }
  BF_CHECK_LAUNCH(name);
  g_tc_launches.fetch_add(1, std::memory_order_relaxed);
  return BF_OK;
}

int launch_crown_bwd_linear_tc(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                               const float* add, const unsigned char* Wpk, const float* kbias, float* A_prev, float* delta,
                               int accumulate, const float* mid, const float* rad, float* partial, int side, int M, int S, int K,
                               int N, int* status, cudaStream_t stream, bool cta_pairs) {
  tc::Params p{};
  int nt;
  tc_tile_shape(N, K, &p.BN, &nt, &p.nkb);
  p.A = A; p.Bpk = Wpk; p.M = M; p.N = N; p.K = K; p.S = S;
  p.vecK = (K % 4 == 0);
  const void* kptrs[] = {A, dpos, dneg, epos, eneg, add, kbias};
  for (const void* q : kptrs) if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) p.vecK = 0;
  p.vecN = (N % 4 == 0);
  const void* nptrs[] = {mid, rad, A_prev};
  for (const void* q : nptrs) if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) p.vecN = 0;
  p.dpos = dpos; p.dneg = dneg; p.epos = epos; p.eneg = eneg; p.add = add; p.kbias = kbias;
  p.delta = delta; p.accumulate = accumulate;
  p.out = A_prev; p.mid_n = mid; p.rad_n = rad; p.partial = partial;
  p.conc_sign = (side == BF_SIDE_LOWER) ? -1.f : 1.f;
  p.status = status;
  timing_begin(T_BWD, stream);
  // cta_pairs (BF_B200_BWD_PAIRS=1, read by the callers once per call): the row blocks run as CTA pairs (tcgen05 cta_group::2)
  const bool pairs = cta_pairs && M > tc::BM;
  int rc = pairs ? tc_launch<tc::MODE_BWD, tc::PRO_RELU, true>(p, nt, stream, "crown_tc_kernel<bwd,pair>")
                 : tc_launch<tc::MODE_BWD, tc::PRO_RELU>(p, nt, stream, "crown_tc_kernel<bwd>");
  timing_end(T_BWD, stream, 4.0 * (double)M * K + (A_prev ? 4.0 * (double)M * N : 0.0), 2.0 * (double)M * K * N);
  return rc;
}

int launch_crown_adjoint_linear_tc(const float* Hprev, int first_layer, const float* mid, const float* rad,
                                   const unsigned char* Wpk, const float* nbias, const float* Ahat, const float* dpos,
                                   const float* dneg, const float* epos, const float* eneg, const float* pre_l,
                                   const float* pre_u, float* hout, float* grad, float* gsum, int M, int S, int K, int N,
                                   int* status, cudaStream_t stream, const float* gw) {
  tc::Params p{};
  int nt;
  tc_tile_shape(N, K, &p.BN, &nt, &p.nkb);
  p.A = Hprev; p.Bpk = Wpk; p.M = M; p.N = N; p.K = K; p.S = S;
  p.vecK = (K % 4 == 0);
  const void* kptrs[] = {Hprev, mid, rad};
  for (const void* q : kptrs) if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) p.vecK = 0;
  p.vecN = (N % 4 == 0);
  const void* nptrs[] = {nbias, Ahat, dpos, dneg, epos, eneg, pre_l, pre_u, hout};
  for (const void* q : nptrs) if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) p.vecN = 0;
  p.mid_k = mid; p.rad_k = rad;
  p.nbias = nbias; p.Ahat = Ahat; p.e_dpos = dpos; p.e_dneg = dneg; p.e_epos = epos; p.e_eneg = eneg;
  p.pre_l = pre_l; p.pre_u = pre_u; p.hout = hout; p.grad = grad; p.gsum = gsum; p.gw = gw;
  p.status = status;
  timing_begin(T_ADJ, stream);
  int rc = first_layer ? tc_launch<tc::MODE_ADJ, tc::PRO_H0>(p, nt, stream, "crown_tc_kernel<adjoint,h0>")
                       : tc_launch<tc::MODE_ADJ, tc::PRO_PLAIN>(p, nt, stream, "crown_tc_kernel<adjoint>");
  timing_end(T_ADJ, stream, 4.0 * (double)M * K + 8.0 * (double)M * N, 2.0 * (double)M * K * N);
  return rc;
}

}  // namespace bf
