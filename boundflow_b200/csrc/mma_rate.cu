// Stand-alone micro-benchmark (not part of libbf_b200.so): cycles per tcgen05.mma kind::tf32 (M = 128, N = 256 or 128,
// K = 8) issued back to back by one thread per SM on all SMs, with the A operand in shared memory or in tensor memory.
// It gives the tensor-pipe rate the 3xTF32 contraction kernels are measured against.
//     python -m boundflow_b200.csrc.build --mma-rate     (builds boundflow_b200/csrc/mma_rate and runs it)
// Every wait is bounded; operands are zeros.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  const uint32_t z = 0;
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
               ::"r"(d), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(z), "r"(z), "r"(z), "r"(z) : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_tmem, uint64_t db, uint32_t idesc, uint32_t acc) {
  const uint32_t z = 0;
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
               ::"r"(d), "r"(a_tmem), "l"(db), "r"(idesc), "r"(acc), "r"(z), "r"(z), "r"(z), "r"(z) : "memory");
}

template <int MODE>  // 0: A smem, 1: A tmem
__global__ void __launch_bounds__(128, 1) rate_kernel(int BN, int iters, long long* cycles, int* status) {
  extern __shared__ unsigned char raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  __shared__ unsigned long long bar;
  __shared__ uint32_t tmem_base_sh;
  const int tid = threadIdx.x, warp = tid >> 5;
  // zero the operand tiles (A 16 KB, B BN*128 B)
  for (int i = tid; i < (16384 + BN * 128) / 4; i += 128) reinterpret_cast<uint32_t*>(tiles)[i] = 0;
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&tmem_base_sh)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_sh;
  if (MODE == 1) {
    // fill the A region of tensor memory (columns 256..319) with zeros: every warp writes its lane quarter
    const uint32_t z = 0;
    for (int c = 0; c < 64; c += 8) {
      const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + 256u + (uint32_t)c;
      asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                   ::"r"(taddr), "r"(z), "r"(z), "r"(z), "r"(z), "r"(z), "r"(z), "r"(z), "r"(z) : "memory");
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  long long t0 = 0, t1 = 0;
  int bad = 0;
  if (tid == 0) {
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const uint32_t a_s = smem_u32(tiles), b_s = a_s + 16384;
    t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (MODE == 0) mma_ss(tmem, make_desc(a_s + j * 32), make_desc(b_s + j * 32), idesc, 1u);
        else mma_ts(tmem, tmem + 256u + (uint32_t)(j * 8), make_desc(b_s + j * 32), idesc, 1u);
      }
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
    // bounded wait
    uint32_t ok = 0;
    const long long w0 = clock64();
    while (!ok) {
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(ok) : "r"(smem_u32(&bar)), "r"(0u) : "memory");
      if (clock64() - w0 > 4000000000LL) { bad = 1; break; }
    }
    t1 = clock64();
    if (bad) *status = 1;
    cycles[blockIdx.x] = t1 - t0;
  }
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}

int main() {
  long long* cyc; int* status;
  cudaMalloc(&cyc, 148 * sizeof(long long)); cudaMalloc(&status, 4); cudaMemset(status, 0, 4);
  const int iters = 2000;
  cudaFuncSetAttribute(rate_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  cudaFuncSetAttribute(rate_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  for (int mode = 0; mode < 2; ++mode)
    for (int BN : {256, 128}) {
      for (int rep = 0; rep < 2; ++rep) {
        if (mode == 0) rate_kernel<0><<<148, 128, 60 * 1024>>>(BN, iters, cyc, status);
        else rate_kernel<1><<<148, 128, 60 * 1024>>>(BN, iters, cyc, status);
        cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { printf("mode %d BN %d: %s\n", mode, BN, cudaGetErrorString(e)); return 1; }
      }
      long long h[148]; int st;
      cudaMemcpy(h, cyc, sizeof(h), cudaMemcpyDeviceToHost); cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
      double avg = 0; for (int i = 0; i < 148; ++i) avg += (double)h[i]; avg /= 148;
      const double per = avg / (iters * 4.0);
      printf("A from %s, N=%d: %.1f clk per MMA (128xNx8), %.0f MAC/clk/SM, status %d\n", mode ? "tmem" : "smem", BN, per, 128.0 * BN * 8 / per, st);
    }
  return 0;
}
