// Shared between the chain drivers (chain.cu, chain_alpha.cu).
#pragma once
#include <vector>

#include "kernels.cuh"

struct bf_chain {
  std::vector<bf_layer_desc> layers;
  std::vector<int> relu_layers;  // layer index of every ReLU, chain order
  int n0 = 0;
  int max_width = 0;
  bool linear_relu_alternating = false;  // linear (relu linear)*
  std::vector<int> affine_layers;        // layer index of every Linear / Conv2d, chain order
  bool affine_relu_alternating = false;  // affine (relu affine)* once flatten layers are dropped
  bool has_conv = false;
  // tensor-core path: per layer, packed hi/lo weight images for the backward (W^T as B) and
  // adjoint (W as B) orientation inside a caller-owned buffer, plus a device status word
  std::vector<const unsigned char*> pk_bwd, pk_adj, pk_adj_fm;  // pk_adj_fm: 128-row images for the feature-major adjoint kernel
  int* status = nullptr;
  // A/B switches (environment variables BF_B200_*), refreshed at the start of every whole-chain call and read by
  // the per-layer dispatch of that call
  struct Switches {
    bool force_ffma = false;        // BF_B200_FORCE_FFMA=1: FP32 FFMA tiles instead of the tensor-core kernels
    int adjoint_kernel = 0;         // 0 automatic, 1 row-major (BF_B200_ADJ_ROWMAJOR=1), 2 feature-major (BF_B200_ADJ_FEATURE_MAJOR=1)
    bool no_windows = false;        // BF_B200_NO_WINDOWS set: identity-row sweeps keep full feature maps
    bool persistent_bwd = false;    // BF_B200_BWD_PERSISTENT=1: persistent warp-specialised backward kernel (128 x 256 tiles, double-buffered
                                    // accumulators) instead of the one-tile-per-CTA kernel; measured slower on wide layers, see crown_tc_persist.cu
    bool pair_bwd = false;          // BF_B200_BWD_PAIRS=1: backward contraction as CTA pairs (tcgen05 cta_group::2); measured slower, A/B switch
    int tc_min_rows = 256;          // coefficient rows from which Linear layers run on the tensor-core kernels (BF_B200_TC_MIN_ROWS)
    bool tc_auto = true;            // BF_B200_TC_MIN_ROWS unset: in addition, a layer whose 64 x 64 FFMA tiles fit one wave (two CTAs per
                                    // SM) stays on the FFMA kernels, which are faster there and follow the reference's fp32 rounding
  };
  mutable Switches sw;
};

namespace bf {

static inline size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  template <typename T>
  T* take(size_t n) {
    T* p = reinterpret_cast<T*>(base + off);
    off += align_up(n * sizeof(T));
    return p;
  }
};


// Re-reads the BF_B200_* environment switches into chain->sw (called once per whole-chain entry point).
void refresh_switches(const bf_chain* c);
// True when a sweep over M coefficient rows may have run tensor-core kernels (whose status word then guards the results).
bool tc_may_run(const bf_chain* c, int M);

// Backward contraction of linear layer `layer` (tensor-core path when the packed weights exist and the
// problem is large enough, FFMA tiles otherwise); *ptiles receives the number of column tiles of the
// concretisation partial-sum buffer.
int dispatch_bwd(const bf_chain* c, int layer, const float* A, const float* dpos, const float* dneg, const float* epos,
                 const float* eneg, const float* add, float* A_prev, float* delta, int accumulate, const float* mid,
                 const float* rad, float* partial, int side, int M, int S, int* ptiles, cudaStream_t stream);
int dispatch_adjoint(const bf_chain* c, int layer, const float* Hprev, int first_layer, const float* mid, const float* rad,
                     const float* Ahat, const float* dpos, const float* dneg, const float* epos, const float* eneg,
                     const float* pre_l, const float* pre_u, float* hout, float* grad, float* gsum, int M, int S,
                     cudaStream_t stream, const float* gw = nullptr);

}  // namespace bf
