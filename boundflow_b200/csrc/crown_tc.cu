// CROWN backward / adjoint contractions on the 5th-generation tensor cores
// (tcgen05.mma kind::tf32, accumulators in tensor memory) with 3xTF32 split
// operands for fp32-faithful results:
//     a*b ~= a_hi*b_hi + a_lo*b_hi + a_hi*b_lo,   x_hi = tf32(x), x_lo = tf32(x - x_hi)
//
// One CTA computes a 128 x BN tile (BN <= 256, multiple of 16) of
//     C[M,N] = f(A)[M,K] * B[K,N]
// * B (the layer weight, static) is pre-split into hi/lo and pre-packed per
//   (n-tile, 32-wide k-block) into the exact shared-memory image the MMA reads
//   (K-major rows of 128 bytes, 128-byte swizzle); one bulk asynchronous copy
//   (cp.async.bulk, completion on an mbarrier) brings a k-block's hi+lo image in.
// * A changes per call and needs the ReLU-backward prologue (sign-selected slope
//   per domain, intercept and bias row sums), so four producer warps load it with
//   coalesced 128-bit loads, transform, split and write the swizzled hi/lo tiles.
// * One thread issues the MMAs; tcgen05.commit releases shared-memory stages and
//   finally signals the epilogue warps, which read the accumulators with
//   tcgen05.ld, transpose through shared memory and write coalesced rows.
// Every wait is bounded: on expiry the CTA raises a status word, stops, frees its
// tensor memory and returns (the host reports the status; nothing traps).
#include "kernels.cuh"

namespace bf {
namespace tc {

constexpr int BM = 128;
constexpr int BK = 32;                  // fp32 per k-block row = 128 bytes
constexpr int MAX_BN = 256;
constexpr int A_TILE = BM * BK * 4;     // bytes of one A tile (hi or lo)
constexpr int PRODUCERS = 128;          // warps 0-3
constexpr int THREADS = 192;            // + warp 4 (bulk-copy issue) + warp 5 (MMA issue, TMEM alloc)
constexpr int TMEM_COLS = 256;
constexpr long long WAIT_LIMIT = 4000000000LL;  // clock cycles (~2 s) before a wait gives up

enum { MODE_BWD = 0, MODE_ADJ = 1 };
enum { PRO_PLAIN = 0, PRO_RELU = 1, PRO_H0 = 2 };

struct Params {
  // operands
  const float* A;            // [M,K]
  const unsigned char* Bpk;  // packed hi/lo images, [ntiles][nkb][2][BN][128 B]
  int M, N, K, S, BN, nkb, stages;
  int vecK, vecN;
  // prologue (see gemm_ffma.cuh for the meaning)
  const float* dpos; const float* dneg; const float* epos; const float* eneg; const float* add; const float* kbias;
  const float* mid_k; const float* rad_k;   // PRO_H0: [D,K]
  float* delta; int accumulate;
  // backward epilogue
  float* out;                // [M,N] or null
  const float* mid_n; const float* rad_n;   // [D,N] with `partial`
  float* partial;            // [M, gridDim.y] or null
  float conc_sign;           // -1 lower, +1 upper
  // adjoint epilogue
  const float* nbias; const float* Ahat; const float* e_dpos; const float* e_dneg; const float* e_epos; const float* e_eneg;
  const float* pre_l; const float* pre_u; float* hout; float* grad;
  int* status;               // device word, set non-zero when a wait expired
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when another thread aborted or the limit was reached.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > WAIT_LIMIT) {
      *abort_flag = 1;
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  // K-major, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart (SBO), LBO unused (= 1), descriptor version 1.
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(z), "r"(z), "r"(z), "r"(z)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
__device__ __forceinline__ float sgnf(float a) { return (a > 0.f) ? 1.f : ((a < 0.f) ? -1.f : 0.f); }

// Shared-memory control block placed in front of the (1024-byte aligned) tiles.
struct Control {
  unsigned long long full[4];
  unsigned long long empty[4];
  unsigned long long accum;
  uint32_t tmem_base;
  int abort_flag;
};

template <int MODE, int PRO>
__global__ void __launch_bounds__(THREADS, 1) crown_tc_kernel(Params p) {
  extern __shared__ unsigned char raw_smem[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1024 + 1023) & ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(tiles - 1024);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * BM;
  const int nt = blockIdx.y;
  const int n0 = nt * p.BN;
  const int b_bytes = 2 * p.BN * 128;              // hi + lo image of one k-block
  const int stage_bytes = 2 * A_TILE + b_bytes;
  volatile int* abort_flag = &ctl->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), PRODUCERS + 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    mbar_init(smem_u32(&ctl->accum), 1);
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp < 4) {
    // ------------------------------------------------------------------ A producers
    const int c = tid & 7;        // 16-byte chunk inside the 128-byte k-block row
    const int rg = tid >> 3;      // 8-row group (= swizzle atom) of this thread
    const int row0 = m0 + rg * 8;
    const bool vK = p.vecK != 0;
    const int d_first = (row0 < p.M) ? (row0 / p.S) : 0;
    const int d_last = (min(row0 + 7, p.M - 1) >= row0) ? (min(row0 + 7, p.M - 1) / p.S) : d_first;
    float rowacc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) rowacc[i] = 0.f;

    float4 a_next[8];
    float4 s_next[2][5];  // per domain set: dpos, dneg, epos|mid, eneg|rad, add
    float4 kb_next;
    auto load_block = [&](int kb) {
      const int k = kb * BK + c * 4;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int m = row0 + i;
        a_next[i] = (m < p.M && k < p.K) ? load4_guard(p.A + (size_t)m * p.K, k, p.K, vK) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      kb_next = z;
      if (PRO == PRO_RELU) {
        if (p.kbias && k < p.K) kb_next = load4_guard(p.kbias, k, p.K, vK);
        if (p.dpos) {
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const size_t off = (size_t)(q == 0 ? d_first : d_last) * p.K;
            const bool ok = k < p.K;
            s_next[q][0] = ok ? load4_guard(p.dpos + off, k, p.K, vK) : z;
            s_next[q][1] = ok ? load4_guard(p.dneg + off, k, p.K, vK) : z;
            s_next[q][2] = (ok && p.epos) ? load4_guard(p.epos + off, k, p.K, vK) : z;
            s_next[q][3] = (ok && p.eneg) ? load4_guard(p.eneg + off, k, p.K, vK) : z;
            s_next[q][4] = (ok && p.add) ? load4_guard(p.add + off, k, p.K, vK) : z;
          }
        }
      } else if (PRO == PRO_H0) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const size_t off = (size_t)(q == 0 ? d_first : d_last) * p.K;
          const bool ok = k < p.K;
          s_next[q][2] = ok ? load4_guard(p.mid_k + off, k, p.K, vK) : z;
          s_next[q][3] = ok ? load4_guard(p.rad_k + off, k, p.K, vK) : z;
        }
      }
    };

    load_block(0);
    bool alive = true;
    for (int kb = 0; kb < p.nkb && alive; ++kb) {
      float4 a_cur[8], s_cur[2][5];
      const float4 kbv = kb_next;
#pragma unroll
      for (int i = 0; i < 8; ++i) a_cur[i] = a_next[i];
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int j = 0; j < 5; ++j) s_cur[q][j] = s_next[q][j];
      if (kb + 1 < p.nkb) load_block(kb + 1);

      const int s = kb % p.stages;
      const uint32_t phase = (uint32_t)(kb / p.stages) & 1u;
      if (!mbar_wait(smem_u32(&ctl->empty[s]), phase ^ 1u, abort_flag)) { alive = false; break; }
      unsigned char* a_hi = tiles + (size_t)s * stage_bytes;
      unsigned char* a_lo = a_hi + A_TILE;
      const int k = kb * BK + c * 4;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 a = a_cur[i];
        const int m = row0 + i;
        if (PRO == PRO_RELU) {
          if (p.dpos != nullptr && m < p.M) {
            const int d = m / p.S;
            float4 dp, dn, ep, en, ad;
            if (d == d_first) { dp = s_cur[0][0]; dn = s_cur[0][1]; ep = s_cur[0][2]; en = s_cur[0][3]; ad = s_cur[0][4]; }
            else if (d == d_last) { dp = s_cur[1][0]; dn = s_cur[1][1]; ep = s_cur[1][2]; en = s_cur[1][3]; ad = s_cur[1][4]; }
            else {  // more than two domains inside 8 rows (S < 7): direct loads
              const size_t off = (size_t)d * p.K;
              const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
              const bool ok = k < p.K;
              dp = ok ? load4_guard(p.dpos + off, k, p.K, vK) : z;
              dn = ok ? load4_guard(p.dneg + off, k, p.K, vK) : z;
              ep = (ok && p.epos) ? load4_guard(p.epos + off, k, p.K, vK) : z;
              en = (ok && p.eneg) ? load4_guard(p.eneg + off, k, p.K, vK) : z;
              ad = (ok && p.add) ? load4_guard(p.add + off, k, p.K, vK) : z;
            }
            float r = rowacc[i];
#define BF_TC_SEL(cc)                                      \
  {                                                        \
    const bool sel = a.cc >= 0.f;                          \
    const float lam = a.cc * (sel ? dp.cc : dn.cc) + ad.cc; \
    r += a.cc * (sel ? ep.cc : en.cc);                     \
    r = fmaf(lam, kbv.cc, r);                              \
    a.cc = lam;                                            \
  }
            BF_TC_SEL(x) BF_TC_SEL(y) BF_TC_SEL(z) BF_TC_SEL(w)
#undef BF_TC_SEL
            rowacc[i] = r;
          } else {
            rowacc[i] += a.x * kbv.x + a.y * kbv.y + a.z * kbv.z + a.w * kbv.w;
          }
        } else if (PRO == PRO_H0) {
          if (m < p.M && k < p.K) {
            const int d = m / p.S;
            float4 md, rd;
            if (d == d_first) { md = s_cur[0][2]; rd = s_cur[0][3]; }
            else if (d == d_last) { md = s_cur[1][2]; rd = s_cur[1][3]; }
            else {
              const size_t off = (size_t)d * p.K;
              md = load4_guard(p.mid_k + off, k, p.K, vK);
              rd = load4_guard(p.rad_k + off, k, p.K, vK);
            }
            a.x = md.x - sgnf(a.x) * rd.x; a.y = md.y - sgnf(a.y) * rd.y;
            a.z = md.z - sgnf(a.z) * rd.z; a.w = md.w - sgnf(a.w) * rd.w;
            // lanes of this float4 beyond K stay 0 because mid/rad were loaded guarded
          }
        }
        float4 hi, lo;
        hi.x = tf32_rna(a.x); hi.y = tf32_rna(a.y); hi.z = tf32_rna(a.z); hi.w = tf32_rna(a.w);
        lo.x = tf32_rna(a.x - hi.x); lo.y = tf32_rna(a.y - hi.y); lo.z = tf32_rna(a.z - hi.z); lo.w = tf32_rna(a.w - hi.w);
        const int off = rg * 1024 + i * 128 + ((c ^ i) << 4);
        *reinterpret_cast<float4*>(a_hi + off) = hi;
        *reinterpret_cast<float4*>(a_lo + off) = lo;
      }
      fence_proxy_async();
      mbar_arrive(smem_u32(&ctl->full[s]));
    }

    if (PRO == PRO_RELU) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v = rowacc[i];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        const int m = row0 + i;
        if (alive && p.delta != nullptr && nt == 0 && c == 0 && m < p.M) p.delta[m] = p.accumulate ? (p.delta[m] + v) : v;
      }
    }

    // ------------------------------------------------------------------ epilogue (same four warps)
    if (alive && mbar_wait(smem_u32(&ctl->accum), 0, abort_flag)) {
      tc_fence_after();
      float* stage = reinterpret_cast<float*>(tiles) + warp * (32 * 33);  // per-warp 32x33 transpose buffer
      const int my_row = m0 + warp * 32 + lane;                          // TMEM lane = tile row
      const bool vN = p.vecN != 0;
      float conc = 0.f;
      // adjoint: running per-domain column sums, flushed with atomicAdd when the domain changes
      for (int c0 = 0; c0 < p.BN; c0 += 32) {
        float v[32];
        tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
        if (MODE == MODE_BWD && p.partial != nullptr && my_row < p.M) {
          const size_t off = (size_t)(my_row / p.S) * p.N;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int col = n0 + c0 + j;
            if (c0 + j < p.BN && col < p.N) {
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
        if (need_rows) {
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 32; ++j) stage[lane * 33 + j] = v[j];
          __syncwarp();
          const int col = n0 + c0 + lane;
          const bool col_ok = (c0 + lane < p.BN) && (col < p.N);
          float run = 0.f;
          int run_d = -1;
          for (int r = 0; r < 32; ++r) {
            const int row = m0 + warp * 32 + r;
            if (row >= p.M) break;
            const float val = stage[r * 33 + lane];
            if (MODE == MODE_BWD) {
              if (col_ok) p.out[(size_t)row * p.N + col] = val;
            } else {
              const int d = row / p.S;
              if (d != run_d) {
                if (run_d >= 0 && col_ok) atomicAdd(&p.grad[(size_t)run_d * p.N + col], run);
                run = 0.f;
                run_d = d;
              }
              if (col_ok) {
                const size_t off = (size_t)d * p.N + col;
                const float gg = val + (p.nbias ? __ldg(p.nbias + col) : 0.f);
                const float ah = __ldg(p.Ahat + (size_t)row * p.N + col);
                const bool sel = ah >= 0.f;
                const float dsel = sel ? __ldg(p.e_dpos + off) : __ldg(p.e_dneg + off);
                const float esel = sel ? (p.e_epos ? __ldg(p.e_epos + off) : 0.f) : (p.e_eneg ? __ldg(p.e_eneg + off) : 0.f);
                if (p.hout) p.hout[(size_t)row * p.N + col] = dsel * gg + esel;
                if (sel && __ldg(p.pre_l + off) < 0.f && __ldg(p.pre_u + off) > 0.f) run += ah * gg;
              }
            }
          }
          if (MODE == MODE_ADJ && run_d >= 0 && col_ok) atomicAdd(&p.grad[(size_t)run_d * p.N + col], run);
        }
      }
      if (MODE == MODE_BWD && p.partial != nullptr && my_row < p.M) p.partial[(size_t)my_row * gridDim.y + nt] = conc;
      tc_fence_before();
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ bulk-copy issue for B
    if (lane == 0) {
      const unsigned char* src = p.Bpk + (size_t)nt * p.nkb * b_bytes;
      for (int kb = 0; kb < p.nkb; ++kb) {
        const int s = kb % p.stages;
        const uint32_t phase = (uint32_t)(kb / p.stages) & 1u;
        if (!mbar_wait(smem_u32(&ctl->empty[s]), phase ^ 1u, abort_flag)) break;
        const uint32_t bar = smem_u32(&ctl->full[s]);
        mbar_arrive_expect_tx(bar, (uint32_t)b_bytes);
        bulk_copy_g2s(smem_u32(tiles + (size_t)s * stage_bytes + 2 * A_TILE), src + (size_t)kb * b_bytes, (uint32_t)b_bytes, bar);
      }
    }
  } else {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < p.nkb; ++kb) {
        const int s = kb % p.stages;
        const uint32_t phase = (uint32_t)(kb / p.stages) & 1u;
        if (!mbar_wait(smem_u32(&ctl->full[s]), phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_hi = smem_u32(tiles + (size_t)s * stage_bytes);
        const uint32_t a_lo = a_hi + A_TILE;
        const uint32_t b_hi = a_hi + 2 * A_TILE;
        const uint32_t b_lo = b_hi + p.BN * 128;
#pragma unroll
        for (int j = 0; j < BK / 8; ++j) {
          const uint64_t dah = make_desc(a_hi + j * 32), dal = make_desc(a_lo + j * 32);
          const uint64_t dbh = make_desc(b_hi + j * 32), dbl = make_desc(b_lo + j * 32);
          mma_tf32(tmem_base, dal, dbh, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          mma_tf32(tmem_base, dah, dbl, idesc, 1u);
          mma_tf32(tmem_base, dah, dbh, idesc, 1u);
        }
        mma_commit(smem_u32(&ctl->empty[s]));  // frees the stage when these MMAs have read it
      }
      if (ok) mma_commit(smem_u32(&ctl->accum));
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncthreads();
  if (ctl->abort_flag) {
    if (tid == 0 && p.status) atomicExch(p.status, 1);
    // give bulk copies that were already issued time to land before the CTA's shared memory is released
    if (tid == 0) {
      for (int s = 0; s < p.stages; ++s) {
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&ctl->full[s]), 0) && !mbar_try_wait(smem_u32(&ctl->full[s]), 1) && clock64() - t0 < 200000000LL) {
        }
      }
    }
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
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
  return nt;
}

size_t tc_packed_bytes(int N, int K) {
  int BN, nt, nkb;
  tc_tile_shape(N, K, &BN, &nt, &nkb);
  return (size_t)nt * nkb * 2 * BN * 128;
}

int tc_pack_weights(const float* W, int rows, int cols, int transposed, unsigned char* out, cudaStream_t stream) {
  // logical B[n][k]: transposed == 0: W is [N=rows][K=cols]; transposed != 0: W is [K=rows][N=cols]
  const int N = transposed ? cols : rows, K = transposed ? rows : cols;
  int BN, nt, nkb;
  tc_tile_shape(N, K, &BN, &nt, &nkb);
  const long long total = (long long)nt * nkb * BN * 8;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  tc::pack_weights_kernel<<<(int)blocks, 256, 0, stream>>>(W, cols, transposed, N, K, BN, nkb, out, total);
  BF_CHECK_LAUNCH("pack_weights_kernel");
  return BF_OK;
}

static int tc_smem_bytes(int BN, int* stages_out) {
  const int stage = 2 * tc::A_TILE + 2 * BN * 128;
  int stages = (200 * 1024) / stage;
  if (stages > 4) stages = 4;
  if (stages < 2) stages = 2;
  *stages_out = stages;
  return stages * stage + 2048;  // control block + alignment slack
}

template <int MODE, int PRO>
static int tc_launch(tc::Params& p, int ntiles, cudaStream_t stream, const char* name) {
  int stages;
  const int smem = tc_smem_bytes(p.BN, &stages);
  p.stages = stages;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(tc::crown_tc_kernel<MODE, PRO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      set_error("%s: cannot raise the dynamic shared memory limit: %s", name, cudaGetErrorString(e));
      return BF_E_CUDA;
    }
    attr_done = true;
  }
  dim3 grid(ceil_div(p.M, tc::BM), ntiles);
  tc::crown_tc_kernel<MODE, PRO><<<grid, tc::THREADS, smem, stream>>>(p);
  BF_CHECK_LAUNCH(name);
  return BF_OK;
}

int launch_crown_bwd_linear_tc(const float* A, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                               const float* add, const unsigned char* Wpk, const float* kbias, float* A_prev, float* delta,
                               int accumulate, const float* mid, const float* rad, float* partial, int side, int M, int S, int K,
                               int N, int* status, cudaStream_t stream) {
  tc::Params p{};
  int nt;
  tc_tile_shape(N, K, &p.BN, &nt, &p.nkb);
  p.A = A; p.Bpk = Wpk; p.M = M; p.N = N; p.K = K; p.S = S;
  p.vecK = (K % 4 == 0);
  const void* kptrs[] = {A, dpos, dneg, epos, eneg, add, kbias};
  for (const void* q : kptrs) if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) p.vecK = 0;
  p.vecN = (N % 4 == 0);
  const void* nptrs[] = {mid, rad};
  for (const void* q : nptrs) if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) p.vecN = 0;
  p.dpos = dpos; p.dneg = dneg; p.epos = epos; p.eneg = eneg; p.add = add; p.kbias = kbias;
  p.delta = delta; p.accumulate = accumulate;
  p.out = A_prev; p.mid_n = mid; p.rad_n = rad; p.partial = partial;
  p.conc_sign = (side == BF_SIDE_LOWER) ? -1.f : 1.f;
  p.status = status;
  timing_begin(0, stream);
  int rc = tc_launch<tc::MODE_BWD, tc::PRO_RELU>(p, nt, stream, "crown_tc_kernel<bwd>");
  timing_end(0, stream);
  return rc;
}

int launch_crown_adjoint_linear_tc(const float* Hprev, int first_layer, const float* mid, const float* rad,
                                   const unsigned char* Wpk, const float* nbias, const float* Ahat, const float* dpos,
                                   const float* dneg, const float* epos, const float* eneg, const float* pre_l,
                                   const float* pre_u, float* hout, float* grad, int M, int S, int K, int N, int* status,
                                   cudaStream_t stream) {
  tc::Params p{};
  int nt;
  tc_tile_shape(N, K, &p.BN, &nt, &p.nkb);
  p.A = Hprev; p.Bpk = Wpk; p.M = M; p.N = N; p.K = K; p.S = S;
  p.vecK = (K % 4 == 0);
  const void* kptrs[] = {Hprev, mid, rad};
  for (const void* q : kptrs) if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) p.vecK = 0;
  p.vecN = 0;
  p.mid_k = mid; p.rad_k = rad;
  p.nbias = nbias; p.Ahat = Ahat; p.e_dpos = dpos; p.e_dneg = dneg; p.e_epos = epos; p.e_eneg = eneg;
  p.pre_l = pre_l; p.pre_u = pre_u; p.hout = hout; p.grad = grad;
  p.status = status;
  timing_begin(1, stream);
  int rc = first_layer ? tc_launch<tc::MODE_ADJ, tc::PRO_H0>(p, nt, stream, "crown_tc_kernel<adjoint,h0>")
                       : tc_launch<tc::MODE_ADJ, tc::PRO_PLAIN>(p, nt, stream, "crown_tc_kernel<adjoint>");
  timing_end(1, stream);
  return rc;
}

}  // namespace bf
