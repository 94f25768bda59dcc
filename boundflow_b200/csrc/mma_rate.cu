// Measurement aid: issue rate of tcgen05.mma kind::tf32 on every SM.
//
// One CTA per SM; its thread 0 issues `iters` MMAs (M = 128, N = n_cols, K = 8, A and B from shared memory through
// 128-byte-swizzle descriptors, accumulator in tensor memory) back to back, commits them to an mbarrier and waits for it
// with the bounded wait of the product kernels.  The cycles between the first issue and the arrival of the commit are
// written per CTA.  The operand tiles hold zeros: the pipe's rate does not depend on the values.  The figure says what
// the tensor pipe itself sustains, next to which the product kernels' MMA rate inside their producer / epilogue
// pipeline is read (the bench's roofline fields use the measured bf16 GEMM throughput, not this number).
#include <stdint.h>

#include "kernels.cuh"
#include "tc_primitives.cuh"

namespace bf {

using namespace bf::tc;

constexpr int RATE_THREADS = 128;
constexpr int RATE_A_BYTES = 128 * 32 * 4;   // 128 rows x 32 floats: four K = 8 slices, only the first is read

__global__ void __launch_bounds__(RATE_THREADS) tf32_mma_rate_kernel(int n_cols, int iters, long long* __restrict__ cycles,
                                                                     int* __restrict__ status) {
  extern __shared__ unsigned char rate_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* rate_smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(rate_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ unsigned long long bar;
  __shared__ uint32_t tmem_base_sh;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int total_floats = (RATE_A_BYTES + n_cols * 128) / 4;
  float* z = reinterpret_cast<float*>(rate_smem);
  for (int i = tid; i < total_floats; i += RATE_THREADS) z[i] = 0.f;
  const uint32_t tmem_cols = (n_cols <= 32) ? 32u : (n_cols <= 64) ? 64u : (n_cols <= 128) ? 128u : 256u;
  if (tid == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_proxy_async();   // the zero fill is read by the tensor core through the async proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_sh;
  if (tid == 0) {
    // instruction descriptor: fp32 accumulator, tf32 operands, both K-major, N / 8, M / 16
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n_cols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const uint64_t da = make_desc(smem_u32(rate_smem));
    const uint64_t db = make_desc(smem_u32(rate_smem + RATE_A_BYTES));
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) mma_tf32(tmem_base, da, db, idesc, i > 0 ? 1u : 0u);
    mma_commit(smem_u32(&bar));
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag);
    const long long t1 = clock64();
    cycles[blockIdx.x] = ok ? (t1 - t0) : -1;
    if (!ok) atomicExch(status, 1);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

}  // namespace bf

extern "C" int bf_tf32_mma_rate(int n_cols, int iters, int n_ctas, long long* cycles, int* status, bf_stream_t stream) {
  BF_REQUIRE(cycles && status, BF_E_INVALID, "bf_tf32_mma_rate: null output");
  BF_REQUIRE(n_cols >= 16 && n_cols <= 256 && n_cols % 16 == 0 && iters > 0 && iters <= 1000000 && n_ctas > 0 && n_ctas <= 4096,
             BF_E_INVALID, "bf_tf32_mma_rate: n_cols must be a multiple of 16 in [16, 256], iters in [1, 10^6], n_ctas in [1, 4096]");
  const size_t smem = (size_t)bf::RATE_A_BYTES + (size_t)n_cols * 128 + 1024;
  static bf::SmemOptIn opt_in;
  if (int rc = bf::ensure_dynamic_smem(bf::tf32_mma_rate_kernel, 64 * 1024, opt_in, "tf32_mma_rate_kernel")) return rc;
  bf::tf32_mma_rate_kernel<<<n_ctas, bf::RATE_THREADS, smem, bf::as_stream(stream)>>>(n_cols, iters, cycles, status);
  BF_CHECK_LAUNCH("tf32_mma_rate_kernel");
  return BF_OK;
}
