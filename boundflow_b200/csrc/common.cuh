// Shared host/device helpers of the bound-propagation kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/bf_b200.h"

namespace bf {

// ---- error reporting -------------------------------------------------------
void set_error(const char* fmt, ...);
extern std::atomic<unsigned long long> g_launches;
extern std::atomic<unsigned long long> g_tc_launches;  // launches of the tcgen05 contraction kernels among them

inline void count_launch(int n = 1) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

#define BF_REQUIRE(cond, code, ...)  \
  do {                               \
    if (!(cond)) {                   \
      bf::set_error(__VA_ARGS__);    \
      return (code);                 \
    }                                \
  } while (0)

#define BF_CHECK_LAUNCH(name)                                                   \
  do {                                                                          \
    cudaError_t e__ = cudaGetLastError();                                       \
    if (e__ != cudaSuccess) {                                                   \
      bf::set_error("%s: launch failed: %s", (name), cudaGetErrorString(e__)); \
      return BF_E_CUDA;                                                         \
    }                                                                           \
    bf::count_launch();                                                         \
  } while (0)

// Optional per-launch device timing of the hot kernels.  Off by default; when on, a CUDA event pair
// brackets every launch of a kernel that has a slot, and the launcher states the algorithmic work of
// that launch (bytes that must cross HBM, floating-point operations), so that a caller can form
// achieved GB/s and FLOP/s per kernel over any region it runs.
enum TimingSlotId {
  T_BWD = 0,          // backward contraction (tcgen05 or FFMA tiles)
  T_ADJ = 1,          // adjoint contraction
  T_THIN = 2,         // top layer of a sweep (spec width <= 16): store-bound
  T_IBP_LINEAR = 3,
  T_IBP_CONV = 4,
  T_ADAM = 5,
  T_CONCRETIZE = 6,   // stand-alone concretisation of coefficient rows
  T_RELU_WINDOW = 7,  // ReLU scaling of windowed coefficient rows
  T_CONV_T = 8,       // transposed convolution
  T_RELU_ROWS = 9,    // ReLU scaling of full coefficient rows (conv path)
  T_SLOTS = 10
};
void timing_begin(int slot, cudaStream_t stream);
void timing_end(int slot, cudaStream_t stream, double bytes = 0.0, double flops = 0.0);

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute of a kernel: every launcher that needs
// more than 48 KB keeps one of these tables (a function-local static) and raises the limit once per device.
constexpr int MAX_DEVICES = 64;
struct SmemOptIn {
  std::atomic<int> bytes[MAX_DEVICES];
};
template <typename Kernel>
inline int ensure_dynamic_smem(Kernel kernel, int bytes, SmemOptIn& table, const char* name) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) dev = -1;
  if (dev >= 0 && table.bytes[dev].load(std::memory_order_acquire) >= bytes) return BF_OK;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    set_error("%s: cannot raise the dynamic shared memory limit to %d bytes: %s", name, bytes, cudaGetErrorString(e));
    return BF_E_CUDA;
  }
  if (dev >= 0) table.bytes[dev].store(bytes, std::memory_order_release);
  return BF_OK;
}

inline cudaStream_t as_stream(bf_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// ---- device helpers --------------------------------------------------------
__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Loads 4 consecutive floats p[idx..idx+3] with a bound `n_valid` (elements of
// this row that exist from idx on); out-of-range lanes read as 0.
__device__ __forceinline__ float4 load4_guard(const float* __restrict__ row, int idx, int n, bool vec_ok) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (vec_ok && idx + 3 < n) {
    v = __ldg(reinterpret_cast<const float4*>(row + idx));
  } else {
    if (idx + 0 < n) v.x = __ldg(row + idx + 0);
    if (idx + 1 < n) v.y = __ldg(row + idx + 1);
    if (idx + 2 < n) v.z = __ldg(row + idx + 2);
    if (idx + 3 < n) v.w = __ldg(row + idx + 3);
  }
  return v;
}

// Same for data written earlier in the same stream by another kernel but which
// must not go through the read-only path (plain loads).
__device__ __forceinline__ float4 load4_plain(const float* row, int idx, int n, bool vec_ok) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (vec_ok && idx + 3 < n) {
    v = *reinterpret_cast<const float4*>(row + idx);
  } else {
    if (idx + 0 < n) v.x = row[idx + 0];
    if (idx + 1 < n) v.y = row[idx + 1];
    if (idx + 2 < n) v.z = row[idx + 2];
    if (idx + 3 < n) v.w = row[idx + 3];
  }
  return v;
}

__device__ __forceinline__ void store4_guard(float* row, int idx, int n, bool vec_ok, float4 v) {
  if (vec_ok && idx + 3 < n) {
    *reinterpret_cast<float4*>(row + idx) = v;
  } else {
    if (idx + 0 < n) row[idx + 0] = v.x;
    if (idx + 1 < n) row[idx + 1] = v.y;
    if (idx + 2 < n) row[idx + 2] = v.z;
    if (idx + 3 < n) row[idx + 3] = v.w;
  }
}

}  // namespace bf
