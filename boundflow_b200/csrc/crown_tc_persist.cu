// Persistent, warp-specialised CROWN backward contraction on the 5th-generation tensor cores
// (tcgen05.mma kind::tf32, 3xTF32 split operands, accumulators in tensor memory).
//
//     A_prev[M,N] = relu_bwd(A)[M,K] * W^T[K,N]      (+ intercept / bias row sums, + fused box concretisation)
//
// One CTA per SM walks a static list of 128-row x BN-column tiles (BN <= 256).  The two halves of
// tensor memory (2 x 256 columns) hold the accumulators of two consecutive tiles, so a tile's
// epilogue runs while the next tile's MMAs are being issued; producers, the weight-copy thread and
// the MMA thread never stop between tiles.  Roles:
//   warps 0-15   A producers: coalesced 128-bit loads of the coefficient rows (one k-block ahead in
//                registers across tile boundaries, further ahead as L2 prefetches), ReLU-backward
//                prologue (sign-selected slope per domain, intercept / bias row sums), hi/lo TF32
//                split, 128-byte-swizzled K-major tiles in shared memory
//   warps 16-19  epilogue: warp q reads tensor-memory lane quarter q (rows 32q..32q+31 of the tile)
//                with tcgen05.ld, transposes 32x32 blocks through shared memory and stores coalesced
//                128-bit row segments; on the first layer it also forms the concretisation partial sums
//   warp 20      lane 0 issues the bulk copies (cp.async.bulk + mbarrier complete_tx) of the packed
//                hi/lo weight images
//   warp 21      lane 0 issues the MMAs; the warp allocates / frees tensor memory
// Synchronisation is by mbarriers only (a_full/a_empty, b_full/b_empty per pipeline stage, acc_full/
// acc_empty per accumulator buffer).  Every wait is bounded: on expiry the CTA raises the status word,
// every role leaves its loop, the copy thread waits (bounded) for its copies in flight, tensor memory is
// freed and the kernel returns; nothing traps.
//
// Status: opt-in (environment variable BF_B200_BWD_PERSISTENT=1), not the default.  Measured on B200 on a
// 73728 x 512 x 512 layer (8192 subdomains x 9 specs): 233 us against 190 us for the one-tile-per-CTA kernel
// (crown_tc.cu, 128 x 512 tiles).  Per-role cycle counts of an instrumented build (clock64 around every wait, CTA 0;
// the stamps slow that build to 369 us, so they give shares, not absolute times) show why: a 128 x 256 tile halves
// the MMA work that one produced coefficient block feeds (12 MMAs instead of 24) while the producers need the same time
// per 128 x 32 block whether it feeds 12 or 24 MMAs, so the MMA thread waits for coefficient tiles half of the time.
// Further measurements with the same build on the same layer: with the producers doing nothing but arriving on
// their barrier (no loads, no transform, no stores) this kernel reaches 173 us (223 TFLOP/s fp32-equivalent; 201 us
// with its weight copies on, which a 128 x 256 tile needs twice as often per MMA), i.e. 140 clock cycles per MMA plus
// about 20 % of barrier round trips with two coefficient stages - so the one-tile-per-CTA kernel (196-200 TFLOP/s with
// the full prologue) is within about 12 % of what this pipeline structure can give.  Tried on the one-tile kernel
// without gain: CTA pairs sharing the weight tile (crown_tc.cu, PAIR: 277 us against 243 us per launch), the slope
// vectors loaded a k-block ahead in registers (96-register cap of 576-thread CTAs, spills: 256 us) or software-
// pipelined per row (247.5 us against 247.8 us).
// The kernel stays for problems with few row blocks, where its narrower tiles (a half or a quarter of a packed
// weight image) give more CTAs work: a 1152 x 256 x 256 layer launches 36 tiles instead of 9 and runs in 23 us
// instead of 26 us.
#include <stdlib.h>

#include "kernels.cuh"
#include "tc_primitives.cuh"

namespace bf {
namespace tcp {

using namespace bf::tc;

constexpr int BM = 128;
constexpr int BK = 32;                  // fp32 per k-block row = 128 bytes
constexpr int MAX_BN = 256;
constexpr int A_TILE = BM * BK * 4;     // bytes of one A tile (hi or lo)
constexpr int A_STAGES = 2;
constexpr int MAX_B_STAGES = 4;
constexpr int PROD_WARPS = 16;
constexpr int EPI_WARPS = 4;
constexpr int ROWS_PER_THREAD = BM / (PROD_WARPS * 4);  // 8 threads cover one 128-byte row
constexpr int PRODUCERS = PROD_WARPS * 32;
constexpr int EPI_WARP0 = PROD_WARPS;                   // a multiple of 4: epilogue warp w owns lane quarter w % 4
constexpr int COPY_WARP = PROD_WARPS + EPI_WARPS;
constexpr int MMA_WARP = COPY_WARP + 1;
constexpr int THREADS = (MMA_WARP + 1) * 32;
constexpr int PREFETCH_KB = 4;          // k-blocks of L2 prefetch distance for the A operand
constexpr int STG_LD = 36;              // leading dimension of the per-warp epilogue transpose buffer
constexpr int EPI_BYTES = EPI_WARPS * 32 * STG_LD * 4;
constexpr uint32_t TMEM_COLS = 512;     // two accumulator buffers of 256 columns

struct Params {
  const float* A;            // [M,K]
  const unsigned char* Bpk;  // packed hi/lo images, [ntiles_pack][nkb][2][BN_pack][128 B]
  int M, N, K, S;
  int BN;                    // tile width (columns), BN_pack / split
  int BN_pack, split;        // packed image height and how many tiles share one image
  int nkb, ncolt, nrowb, b_stages;
  int vecK, vecN;
  // ReLU-backward prologue (see gemm_ffma.cuh for the meaning)
  // slopes for non-negative / negative coefficients and ONE intercept vector that applies to the coefficients of one
  // sign (e_on_pos != 0: the non-negative ones); callers with two intercept vectors or a beta term use the classic kernel
  const float* dpos; const float* dneg; const float* evec; int e_on_pos; const float* kbias;
  float* delta; int accumulate;
  // epilogue
  float* out;                // [M,N] or null
  const float* mid_n; const float* rad_n;   // [D,N] with `partial`
  float* partial;            // [M, ncolt] or null
  float conc_sign;           // -1 lower, +1 upper
  int* status;               // device word, set non-zero when a wait expired
};


struct Control {
  unsigned long long a_full[A_STAGES];
  unsigned long long a_empty[A_STAGES];
  unsigned long long b_full[MAX_B_STAGES];
  unsigned long long b_empty[MAX_B_STAGES];
  unsigned long long acc_full[2];
  unsigned long long acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// FULLK: K is a multiple of the 32-wide k-block and every K-side pointer is 16-byte aligned (no guards on the loads).
template <bool FULLK>
__global__ void __launch_bounds__(THREADS, 1) crown_tc_persistent_kernel(Params p) {
  extern __shared__ unsigned char raw_smem[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1024 + 1023) & ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(tiles - 1024);
  unsigned char* b_tiles = tiles + A_STAGES * 2 * A_TILE;
  const int b_bytes = 2 * p.BN * 128;                   // hi + lo image of one k-block of one tile
  float* epi_smem = reinterpret_cast<float*>(b_tiles + (size_t)p.b_stages * b_bytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &ctl->abort_flag;
  const int total_tiles = p.nrowb * p.ncolt;
  // tiles of this CTA: t = blockIdx.x + i * gridDim.x; consecutive t share a row block, so the CTAs that read the
  // same coefficient rows (for different column tiles) run at the same time and share them through L2
  const int my_tiles = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  int copies_issued = 0;  // bulk copies this thread has issued (meaningful in the copy thread only)

  if (tid == 0) {
    for (int s = 0; s < A_STAGES; ++s) {
      mbar_init(smem_u32(&ctl->a_full[s]), PRODUCERS);
      mbar_init(smem_u32(&ctl->a_empty[s]), 1);
    }
    for (int s = 0; s < p.b_stages; ++s) {
      mbar_init(smem_u32(&ctl->b_full[s]), 1);
      mbar_init(smem_u32(&ctl->b_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->acc_full[b]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[b]), EPI_WARPS);
    }
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp < PROD_WARPS) {
    // ------------------------------------------------------------------ A producers
    // The producers are instruction-bound (they must finish a 128 x 32 block in the time of twelve MMAs), so the
    // loop below avoids everything avoidable: no integer divisions (running cursors instead), unguarded 128-bit
    // loads when FULLK says every k-block is complete and aligned, and the TF32 split done with two integer
    // operations per value instead of a conversion instruction.
    const int c = tid & 7;        // 16-byte chunk inside the 128-byte k-block row
    const int rg = tid >> 3;      // row group of this thread
    const int n_iter = my_tiles * p.nkb;   // pipeline iterations of this CTA: (tile, k-block) pairs
    const int kcol = c * 4;
    auto ld4 = [&](const float* row, int k) -> float4 {
      if (FULLK) return __ldg(reinterpret_cast<const float4*>(row + k));
      return (k < p.K) ? load4_guard(row, k, p.K, p.vecK != 0) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto tile_row0 = [&](int ti) { return (((int)blockIdx.x + ti * (int)gridDim.x) / p.ncolt) * BM + rg * ROWS_PER_THREAD; };
    // cursor of the block that is loaded next (one iteration ahead of the one being processed, also across a tile
    // boundary) and cursor of the block whose lines are pulled into L2 (PREFETCH_KB iterations further)
    int l_ti = 0, l_kb = 0, l_row = tile_row0(0);
    int f_ti = 0, f_kb = 0, f_row = l_row, f_g = 0;
    for (; f_g < PREFETCH_KB + 1; ++f_g)
      if (++f_kb == p.nkb) { f_kb = 0; ++f_ti; f_row = tile_row0(f_ti); }
    float4 a_next[ROWS_PER_THREAD];
    auto load_next = [&]() {
      const int k = l_kb * BK + kcol;
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) {
        const int m = l_row + i;
        a_next[i] = (m < p.M) ? ld4(p.A + (size_t)m * p.K, k) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      if (++l_kb == p.nkb) { l_kb = 0; ++l_ti; l_row = tile_row0(l_ti); }
      if (f_g < n_iter) {
        if (c == 0 && f_kb * BK < p.K) {
#pragma unroll
          for (int i = 0; i < ROWS_PER_THREAD; ++i)
            if (f_row + i < p.M) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.A + (size_t)(f_row + i) * p.K + (size_t)f_kb * BK));
        }
        ++f_g;
        if (++f_kb == p.nkb) { f_kb = 0; ++f_ti; f_row = tile_row0(f_ti); }
      }
    };
    if (n_iter > 0) load_next();
    bool alive = true;
    int g = 0;
    for (int ti = 0; ti < my_tiles && alive; ++ti) {
      const int t = (int)blockIdx.x + ti * (int)gridDim.x;
      const int rb = t / p.ncolt, ct = t - rb * p.ncolt;
      const int row0 = rb * BM + rg * ROWS_PER_THREAD;
      const bool want_delta = p.delta != nullptr && ct == 0;   // the row sums are formed once per row block
      size_t doff[ROWS_PER_THREAD];
      float rowacc[ROWS_PER_THREAD];
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) {
        doff[i] = (size_t)((row0 + i < p.M) ? ((row0 + i) / p.S) : 0) * p.K;
        rowacc[i] = 0.f;
      }
      for (int kb = 0; kb < p.nkb; ++kb, ++g) {
        float4 a_cur[ROWS_PER_THREAD];
#pragma unroll
        for (int i = 0; i < ROWS_PER_THREAD; ++i) a_cur[i] = a_next[i];
        if (g + 1 < n_iter) load_next();

        const int k = kb * BK + kcol;
        const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 kbv = z4;
        float4 sv[ROWS_PER_THREAD][3];  // dpos, dneg, intercept of each row's domain
        if (want_delta && p.kbias) kbv = ld4(p.kbias, k);
        if (p.dpos) {
#pragma unroll
          for (int i = 0; i < ROWS_PER_THREAD; ++i) {
            sv[i][0] = ld4(p.dpos + doff[i], k);
            sv[i][1] = ld4(p.dneg + doff[i], k);
            sv[i][2] = (want_delta && p.evec) ? ld4(p.evec + doff[i], k) : z4;
          }
        }

        const int s = g % A_STAGES;
        const uint32_t phase = (uint32_t)(g / A_STAGES) & 1u;
        if (!mbar_wait_warp(smem_u32(&ctl->a_empty[s]), phase ^ 1u, abort_flag)) { alive = false; break; }
        unsigned char* a_hi = tiles + (size_t)s * 2 * A_TILE;
        unsigned char* a_lo = a_hi + A_TILE;
#pragma unroll
        for (int i = 0; i < ROWS_PER_THREAD; ++i) {
          float4 a = a_cur[i];
          const int m = row0 + i;
          if (p.dpos != nullptr && m < p.M) {
            const float4 dp = sv[i][0], dn = sv[i][1], ev = sv[i][2];
            if (want_delta) {
              float r = rowacc[i];
              const bool eop = p.e_on_pos != 0;
#define BF_TCP_SEL(cc)                                      \
  {                                                         \
    const bool sel = a.cc >= 0.f;                           \
    const float lam = a.cc * (sel ? dp.cc : dn.cc);         \
    r = fmaf(a.cc, (sel == eop) ? ev.cc : 0.f, r);          \
    r = fmaf(lam, kbv.cc, r);                               \
    a.cc = lam;                                             \
  }
              BF_TCP_SEL(x) BF_TCP_SEL(y) BF_TCP_SEL(z) BF_TCP_SEL(w)
#undef BF_TCP_SEL
              rowacc[i] = r;
            } else {
              a.x *= (a.x >= 0.f ? dp.x : dn.x);
              a.y *= (a.y >= 0.f ? dp.y : dn.y);
              a.z *= (a.z >= 0.f ? dp.z : dn.z);
              a.w *= (a.w >= 0.f ? dp.w : dn.w);
            }
          } else if (want_delta) {
            rowacc[i] += a.x * kbv.x + a.y * kbv.y + a.z * kbv.z + a.w * kbv.w;
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
        mbar_arrive(smem_u32(&ctl->a_full[s]));
      }
      if (alive && want_delta) {
#pragma unroll
        for (int i = 0; i < ROWS_PER_THREAD; ++i) {
          float v = rowacc[i];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          const int m = row0 + i;
          if (c == 0 && m < p.M) p.delta[m] = p.accumulate ? (p.delta[m] + v) : v;
        }
      }
    }
  } else if (warp < COPY_WARP) {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;          // tensor-memory lane quarter = rows q*32 .. q*32+31 of the tile
    float* stg = epi_smem + (warp - EPI_WARP0) * (32 * STG_LD);  // per-warp 32 x 36 transpose buffer
    const int rs = lane >> 3, c4 = lane & 7;  // (row sub-index, 16-byte column chunk) view after the transpose
    const bool vN = p.vecN != 0;
    for (int ti = 0; ti < my_tiles; ++ti) {
      const int t = (int)blockIdx.x + ti * (int)gridDim.x;
      const int rb = t / p.ncolt, ct = t - rb * p.ncolt;
      const int buf = ti & 1;
      if (!mbar_wait_warp(smem_u32(&ctl->acc_full[buf]), (uint32_t)(ti >> 1) & 1u, abort_flag)) break;
      tc_fence_after();
      const int row_base = rb * BM + q * 32;
      const int my_row = row_base + lane;  // thread-per-row view right after tcgen05.ld
      const int ncol0 = ct * p.BN;
      // this tile owns columns [ncol0, ncol_end): the 32-column chunks below may overhang a tile whose width is not a
      // multiple of 32 (into accumulator columns that hold nothing) or N (zero padding of the packed weights)
      const int ncol_end = min(p.N, ncol0 + p.BN);
      float conc = 0.f;
      for (int c0 = 0; c0 < p.BN; c0 += 32) {
        const int colbase = ncol0 + c0;
        if (colbase >= ncol_end) break;
        float v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * MAX_BN + c0), v);
        if (p.partial != nullptr && my_row < p.M) {
          const size_t off = (size_t)(my_row / p.S) * p.N;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int col = colbase + j;
            if (col < ncol_end) {   // tile widths are multiples of 16, so a group of four columns is inside or outside as a whole
              const float4 md = load4_guard(p.mid_n + off, col, p.N, vN);
              const float4 rd = load4_guard(p.rad_n + off, col, p.N, vN);
              conc += v[j] * md.x + p.conc_sign * fabsf(v[j]) * rd.x;
              conc += v[j + 1] * md.y + p.conc_sign * fabsf(v[j + 1]) * rd.y;
              conc += v[j + 2] * md.z + p.conc_sign * fabsf(v[j + 2]) * rd.z;
              conc += v[j + 3] * md.w + p.conc_sign * fabsf(v[j + 3]) * rd.w;
            }
          }
        }
        if (p.out == nullptr) continue;
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(&stg[lane * STG_LD + 4 * j]) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        __syncwarp();
        const int col = colbase + c4 * 4;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r = it * 4 + rs;
          const int row = row_base + r;
          if (row < p.M && col < ncol_end) {
            const float4 val = *reinterpret_cast<const float4*>(&stg[r * STG_LD + c4 * 4]);
            store4_guard(p.out + (size_t)row * p.N, col, ncol_end, vN, val);
          }
        }
      }
      // this warp has read its quarter of the buffer: hand it back to the MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[buf]));
      if (p.partial != nullptr && my_row < p.M) p.partial[(size_t)my_row * p.ncolt + ct] = conc;
    }
  } else if (warp == COPY_WARP) {
    // ------------------------------------------------------------------ bulk-copy issue for the weight images
    if (lane == 0) {
      int it = 0;
      const uint32_t half = (uint32_t)(p.BN * 128);
      for (int ti = 0; ti < my_tiles; ++ti) {
        const int t = (int)blockIdx.x + ti * (int)gridDim.x;
        const int ct = t % p.ncolt;
        const int nt_pack = ct / p.split, r0 = (ct - nt_pack * p.split) * p.BN;  // image and first row inside it
        bool ok = true;
        for (int kb = 0; kb < p.nkb; ++kb, ++it) {
          const int s = it % p.b_stages;
          const uint32_t phase = (uint32_t)(it / p.b_stages) & 1u;
          if (!mbar_wait(smem_u32(&ctl->b_empty[s]), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t bar = smem_u32(&ctl->b_full[s]);
          const unsigned char* img = p.Bpk + ((size_t)nt_pack * p.nkb + kb) * (size_t)(2 * p.BN_pack * 128);
          const uint32_t dst = smem_u32(b_tiles + (size_t)s * b_bytes);
          mbar_arrive_expect_tx(bar, 2 * half);
          if (p.split == 1) {
            bulk_copy_g2s(dst, img, 2 * half, bar);
          } else {  // rows r0 .. r0+BN of the hi image and of the lo image
            bulk_copy_g2s(dst, img + (size_t)r0 * 128, half, bar);
            bulk_copy_g2s(dst + half, img + (size_t)(p.BN_pack + r0) * 128, half, bar);
          }
        }
        if (!ok) break;
      }
      copies_issued = it;
    }
  } else {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      // descriptors of stage 0; a stage (or the lo image) further on is a plain add (the 14-bit address field cannot
      // overflow: shared-memory addresses stay below 256 KB)
      const uint64_t a_desc0 = make_desc(smem_u32(tiles)), b_desc0 = make_desc(smem_u32(b_tiles));
      bool ok = true;
      int it = 0;
      for (int ti = 0; ti < my_tiles && ok; ++ti) {
        const int buf = ti & 1;
        // the epilogue warps must have drained this buffer (its previous use was tile ti - 2)
        if (!mbar_wait(smem_u32(&ctl->acc_empty[buf]), ((uint32_t)(ti >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * MAX_BN);
        for (int kb = 0; kb < p.nkb; ++kb, ++it) {
          const int sa = it % A_STAGES, sb = it % p.b_stages;
          if (!mbar_wait(smem_u32(&ctl->a_full[sa]), (uint32_t)(it / A_STAGES) & 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&ctl->b_full[sb]), (uint32_t)(it / p.b_stages) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t dah = a_desc0 + (uint64_t)(sa * ((2 * A_TILE) >> 4));
          const uint64_t dbh = b_desc0 + (uint64_t)(sb * (b_bytes >> 4));
          mma_kblock_3xtf32(d_tmem, dah, dah + (A_TILE >> 4), dbh, dbh + (uint64_t)((p.BN * 128) >> 4), idesc, kb > 0 ? 1u : 0u);
          mma_commit(smem_u32(&ctl->b_empty[sb]));  // frees both stages when these MMAs have read them
          mma_commit(smem_u32(&ctl->a_empty[sa]));
        }
        if (ok) mma_commit(smem_u32(&ctl->acc_full[buf]));
      }
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
  if (warp == MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace tcp


// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int sm_count_of_current_device() {
  static std::atomic<int> cached[MAX_DEVICES];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) dev = 0;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// Tile width for a problem: the packed images are BN_pack rows high; a tile may take 1/2 or 1/4 of an image when the
// full-width tiles would leave SMs without work (small M) and the narrower width is still a legal MMA N (multiple of 16).
static void persist_tile_shape(int M, int N, int K, int sms, int* BN, int* split, int* ncolt, int* BN_pack, int* nkb) {
  int nt_pack;
  tc_tile_shape(N, K, BN_pack, &nt_pack, nkb);
  const int nrowb = ceil_div(M, tcp::BM);
  int sp = 1;
  while (sp < 4 && nrowb * ceil_div(N, *BN_pack / sp) < sms && (*BN_pack / (sp * 2)) % 16 == 0 && *BN_pack / (sp * 2) >= 32) sp *= 2;
  *split = sp;
  *BN = *BN_pack / sp;
  *ncolt = ceil_div(N, *BN);
}

int crown_tc_persist_partial_tiles(int M, int N, int K) {
  int BN, split, ncolt, BN_pack, nkb;
  persist_tile_shape(M, N, K, sm_count_of_current_device(), &BN, &split, &ncolt, &BN_pack, &nkb);
  return ncolt;
}

int crown_tc_persist_max_partial_tiles(int N) {
  // narrowest tile the shape rule can choose: a quarter of the packed width, at least 32 columns
  int BN_pack, nt, nkb;
  tc_tile_shape(N, 32, &BN_pack, &nt, &nkb);
  int bn = BN_pack;
  for (int sp = 1; sp < 4 && (bn / 2) % 16 == 0 && bn / 2 >= 32; sp *= 2) bn /= 2;
  return ceil_div(N, bn);
}

bool crown_tc_persistent_supports(const float* epos, const float* eneg, const float* add) {
  return add == nullptr && !(epos != nullptr && eneg != nullptr);
}

int launch_crown_bwd_linear_tc_persistent(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                                          const float* add, const unsigned char* Wpk, const float* kbias, float* A_prev,
                                          float* delta, int accumulate, const float* mid, const float* rad, float* partial,
                                          int side, int M, int S, int K, int N, int* status, cudaStream_t stream) {
  if (!crown_tc_persistent_supports(epos, eneg, add)) {
    set_error("crown_tc_persistent_kernel: two intercept vectors or a beta term need the classic kernel");
    return BF_E_UNSUPPORTED;
  }
  tcp::Params p{};
  const int sms = sm_count_of_current_device();
  persist_tile_shape(M, N, K, sms, &p.BN, &p.split, &p.ncolt, &p.BN_pack, &p.nkb);
  p.nrowb = ceil_div(M, tcp::BM);
  p.A = A; p.Bpk = Wpk; p.M = M; p.N = N; p.K = K; p.S = S;
  p.vecK = (K % 4 == 0);
  const void* kptrs[] = {A, dpos, dneg, epos, eneg, kbias};
  for (const void* q : kptrs) if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) p.vecK = 0;
  p.vecN = (N % 4 == 0);
  const void* nptrs[] = {mid, rad, A_prev};
  for (const void* q : nptrs) if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) p.vecN = 0;
  p.dpos = dpos; p.dneg = dneg; p.evec = epos ? epos : eneg; p.e_on_pos = epos != nullptr; p.kbias = kbias;
  p.delta = delta; p.accumulate = accumulate;
  p.out = A_prev; p.mid_n = mid; p.rad_n = rad; p.partial = partial;
  p.conc_sign = (side == BF_SIDE_LOWER) ? -1.f : 1.f;
  p.status = status;
  const int b_bytes = 2 * p.BN * 128;
  const int budget = 225 * 1024 - 2048 - tcp::A_STAGES * 2 * tcp::A_TILE - tcp::EPI_BYTES;
  int b_stages = budget / b_bytes;
  if (b_stages > tcp::MAX_B_STAGES) b_stages = tcp::MAX_B_STAGES;
  if (b_stages < 2) {
    set_error("crown_tc_persistent_kernel: tile of %d columns does not fit two weight stages", p.BN);
    return BF_E_UNSUPPORTED;
  }
  p.b_stages = b_stages;
  const int smem = 2048 + tcp::A_STAGES * 2 * tcp::A_TILE + b_stages * b_bytes + tcp::EPI_BYTES;
  const bool fullk = p.vecK && (K % tcp::BK == 0);
  static SmemOptIn opt_in[2];
  if (int rc = fullk ? ensure_dynamic_smem(tcp::crown_tc_persistent_kernel<true>, 227 * 1024, opt_in[1], "crown_tc_persistent_kernel")
                     : ensure_dynamic_smem(tcp::crown_tc_persistent_kernel<false>, 227 * 1024, opt_in[0], "crown_tc_persistent_kernel"))
    return rc;
  const int total_tiles = p.nrowb * p.ncolt;
  const int grid = total_tiles < sms ? total_tiles : sms;
  timing_begin(T_BWD, stream);
  if (fullk) tcp::crown_tc_persistent_kernel<true><<<grid, tcp::THREADS, smem, stream>>>(p);
  else tcp::crown_tc_persistent_kernel<false><<<grid, tcp::THREADS, smem, stream>>>(p);
  timing_end(T_BWD, stream, 4.0 * (double)M * K + (A_prev ? 4.0 * (double)M * N : 0.0), 2.0 * (double)M * K * N);
  BF_CHECK_LAUNCH("crown_tc_persistent_kernel");
  g_tc_launches.fetch_add(1, std::memory_order_relaxed);
  return BF_OK;
}

}  // namespace bf
