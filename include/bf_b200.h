/*
 * bf_b200.h -- C ABI of the B200 (sm_100a) bound-propagation backend.
 *
 * The reference project (BoundFlow) has no FFI: its plug points are Python
 * protocols.  Each entry point below names the reference interface whose
 * arithmetic it replaces (path:line inside the reference project).  All
 * pointers are DEVICE pointers owned by the caller unless stated otherwise,
 * all tensors are contiguous row-major fp32 unless stated otherwise, every call
 * is asynchronous on `stream` and allocates nothing.  Return value: 0 on
 * success, a negative BF_E_* code otherwise (bf_last_error_string() explains).
 *
 * Shapes: B = domains (inputs or BaB subdomains), S = spec rows per domain,
 * M = B*S coefficient rows, n = neurons of a layer.
 */
#ifndef BF_B200_H
#define BF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* bf_stream_t; /* a cudaStream_t */

#define BF_OK 0
#define BF_E_INVALID (-1)     /* bad argument (null pointer, non-positive size, ...) */
#define BF_E_UNSUPPORTED (-2) /* legal request this backend does not implement */
#define BF_E_WORKSPACE (-3)   /* workspace too small */
#define BF_E_CUDA (-4)        /* a CUDA runtime call failed */

#define BF_SIDE_LOWER 0
#define BF_SIDE_UPPER 1

#define BF_IN_LOWER_UPPER 0 /* (in_a, in_b) = (lower, upper) */
#define BF_IN_MID_RAD 1     /* (in_a, in_b) = (midpoint, radius) */
#define BF_IN_CENTER_DEV 2  /* bf_chain_ibp only: in_a = ball centre [B,n0], in_b = eps * dual norm of the first
                               Linear layer's weight rows [n_1] (from bf_row_dual_norms): Lp-ball input */

#define BF_NORM_BOX 0 /* per-element box given as midpoint + radius (also the L-inf ball: radius == eps) */
#define BF_NORM_INF 3 /* Lp ball given as centre + eps, p = inf (dual norm: sum |x|) */
#define BF_NORM_L2 2  /* p = 2 (dual norm: sqrt(sum x^2)) */
#define BF_NORM_L1 1  /* p = 1 (dual norm: max |x|) */

#define BF_OP_LINEAR 1
#define BF_OP_CONV2D 2
#define BF_OP_RELU 3
#define BF_OP_FLATTEN 4

#define BF_REDUCE_MEAN 0 /* per-domain objective = mean over spec rows */
#define BF_REDUCE_SUM 1  /* per-domain objective = sum over spec rows  */
#define BF_REDUCE_MIN 2  /* per-domain objective = smallest spec row */
#define BF_REDUCE_SOFTMIN 3 /* per-domain objective = -tau * logsumexp(-rows / tau) */

#define BF_OBJECTIVE_GAP 2  /* minimise reduce(upper - lower) */
#define BF_OBJECTIVE_BOTH 3 /* maximise lb_weight * reduce(lower) - ub_weight * reduce(upper) */

/* Library identity and diagnostics. */
int bf_version(void);
const char* bf_last_error_string(void);
/* Number of kernels this library has launched since it was loaded, and how many of those were the
 * tcgen05 (tensor-core) contraction kernels. */
unsigned long long bf_launch_count(void);
unsigned long long bf_tc_launch_count(void);

/* Measurement aid (no counterpart in the reference): when enabled, every launch of a kernel
 * that has a timing slot is bracketed by a CUDA event pair on its own stream, and the launcher adds
 * the algorithmic work of that launch (bytes that must cross HBM once, floating-point operations)
 * to the slot.  bf_kernel_timing_read[_work] waits for the recorded events and returns the number
 * of launches, their summed device time and the summed work since the last enable.
 * Slots (bf_kernel_timing_slots() of them, named by bf_kernel_timing_slot_name):
 *   0 CROWN backward contraction      1 adjoint (gradient) contraction   2 thin top-layer kernel
 *   3 interval Linear                 4 interval Conv2d                  5 Adam / projection step
 *   6 stand-alone concretisation      7 ReLU scaling of windowed rows    8 transposed convolution
 *   9 ReLU scaling of full coefficient rows
 * Safe to call from several host threads (one mutex guards the slots); meant for benchmarks. */
void bf_kernel_timing_enable(int on);
int bf_kernel_timing_slots(void);
const char* bf_kernel_timing_slot_name(int slot);
int bf_kernel_timing_read(int slot, int* launches, float* total_ms);
int bf_kernel_timing_read_work(int slot, int* launches, float* total_ms, double* bytes, double* flops);

/* ------------------------------------------------------------------------
 * Layer-level kernels
 * ---------------------------------------------------------------------- */

/* Interval linear layer, optionally preceded by the interval ReLU and followed
 * by the pre-activation constraint intersection and the ReLU split clamp.
 *   replaces IntervalDomain.affine_transformer, boundflow/domains/interval.py:79-86
 *            (W+/W- form; computed here in centre/radius form W*c+b -/+ |W|*r),
 *            BoxPerturbation.concretize_matmul, boundflow/runtime/perturbation.py:282-325
 *            (in_mode = BF_IN_MID_RAD or a box given as lower/upper),
 *            relu_transformer interval.py:88-91 (relu_in != 0),
 *            the constraint intersection boundflow/runtime/crown_ibp.py:186-209,
 *            _apply_relu_split crown_ibp.py:70-98.
 * in_a,in_b [B,n_in]; W [n_out,n_in]; bias [n_out] or NULL;
 * split int8 [B,n_out] in {-1,0,+1} or NULL, split_stride = n_out or 0 (one row for all domains);
 * cons_l,cons_u [B,n_out] or NULL; out_l,out_u [B,n_out];
 * infeasible int32 [B] or NULL: set to 1 where a clamp produced lower > upper (never cleared). */
int bf_ibp_linear(const float* in_a, const float* in_b, int in_mode, int relu_in,
                  const float* W, const float* bias,
                  const int8_t* split, int split_stride,
                  const float* cons_l, const float* cons_u,
                  float* out_l, float* out_u, int* infeasible,
                  int B, int n_in, int n_out, bf_stream_t stream);

/* Interval Conv2d (NCHW input, OIHW weight, groups = 1, dilation = 1), same
 * fusion options as bf_ibp_linear.
 *   replaces IntervalDomain.affine_transformer conv2d branch, boundflow/domains/interval.py:57-74. */
int bf_ibp_conv2d(const float* in_a, const float* in_b, int in_mode, int relu_in,
                  const float* W, const float* bias,
                  const int8_t* split, int split_stride,
                  const float* cons_l, const float* cons_u,
                  float* out_l, float* out_u, int* infeasible,
                  int B, int Ci, int Hi, int Wi, int Co, int kh, int kw,
                  int sh, int sw, int ph, int pw, bf_stream_t stream);

/* ReLU relaxation from pre-activation bounds.
 *   replaces _relu_relax crown_ibp.py:722-758 and the alpha override
 *            _relu_backward_relaxation crown_ibp.py:1176-1208.
 * l,u [B,n]; alpha [B,n] (alpha_stride = n) or [n] (alpha_stride = 0) or NULL;
 * outputs [B,n]: alpha_u (upper slope), beta_u (upper intercept), alpha_l
 * (lower slope: 1 / 0 for stable neurons, clamp(alpha,0,1) or 0 for unstable). */
int bf_relu_relax(const float* l, const float* u, const float* alpha, int alpha_stride,
                  float* alpha_u, float* beta_u, float* alpha_l,
                  int B, int n, bf_stream_t stream);

/* Start value of the per-domain lower slopes: 1 where l >= 0 or (l < 0 < u and u > -l), else 0.
 *   replaces _initial_alpha_state, boundflow/runtime/native_alpha_beta_optimizer_schedule.py:635-656.
 * l,u,alpha [B,n]. */
int bf_alpha_adaptive_init(const float* l, const float* u, float* alpha, int B, int n, bf_stream_t stream);

/* Fused ReLU backward + Linear backward region for one side (lower or upper).
 *   replaces FusedCrownExecutor.run for kind == "linear", boundflow/runtime/fused_crown.py:97-123
 *            (eager oracle fused_crown.py:330-363; TVM kernel backends/tvm/fused_crown_linear.py:85-156),
 *            i.e. _backprop_relu_step_dense_reference crown_ibp.py:1262-1298 followed by
 *            _backprop_linear_step crown_ibp.py:1073-1090.
 * A [B,S,n_cur] coefficients w.r.t. the ReLU output;
 * alpha_u, alpha_l, beta_u, beta_l [B,n_cur] (beta_l may be NULL = 0; passing all four
 * NULL skips the ReLU, giving the plain Linear backward);
 * add [B,n_cur] or NULL: term added to the scaled coefficients of every spec row (beta-CROWN);
 * W [n_cur,n_prev], bias [n_cur] or NULL;
 * A_prev [B,S,n_prev] (may be NULL when only delta is wanted);
 * delta [B,S]: sum_j A*beta_sel + sum_j A_scaled*bias; if accumulate != 0 it is added to the
 * existing contents of `delta`, otherwise it overwrites them. */
int bf_crown_relu_linear_bwd(const float* A, int side,
                             const float* alpha_u, const float* alpha_l,
                             const float* beta_u, const float* beta_l,
                             const float* add,
                             const float* W, const float* bias,
                             float* A_prev, float* delta, int accumulate,
                             int B, int S, int n_cur, int n_prev, bf_stream_t stream);

/* Tensor-core variant of bf_crown_relu_linear_bwd for callers that keep a layer's weight between calls
 * (the fused-region executor, graphs that are not chains).  No counterpart in the reference, whose
 * contraction is a cuBLAS call made by torch.einsum (boundflow/runtime/linear_operator.py:585-586).
 *   bf_linear_pack: splits W [n_cur,n_prev] into hi/lo TF32 parts and writes the shared-memory images of the
 *            tcgen05 kernel, preceded by a status word, into `pack` (device, 256-byte aligned,
 *            bf_linear_pack_bytes(n_cur, n_prev) bytes).  Repack when W changes.
 *   bf_crown_relu_linear_bwd_packed: same arguments and results as bf_crown_relu_linear_bwd plus the pack;
 *            runs the tcgen05 3xTF32 kernel when B*S >= 256 and both widths are >= 32, the FP32 FFMA
 *            tiles otherwise (or when pack is NULL).  If a bounded wait inside the kernel ever expires the
 *            outputs of that call are overwritten with NaN and the pack's status word stays non-zero
 *            (bf_linear_pack_status, synchronous). */
size_t bf_linear_pack_bytes(int n_cur, int n_prev);
int bf_linear_pack(const float* W, int n_cur, int n_prev, void* pack, size_t pack_bytes, bf_stream_t stream);
int bf_linear_pack_status(const void* pack, int* status);
int bf_crown_relu_linear_bwd_packed(const float* A, int side,
                                    const float* alpha_u, const float* alpha_l,
                                    const float* beta_u, const float* beta_l,
                                    const float* add,
                                    const float* W, const float* bias, const void* pack,
                                    float* A_prev, float* delta, int accumulate,
                                    int B, int S, int n_cur, int n_prev, bf_stream_t stream);

/* Fused ReLU backward + Conv2d backward (transposed convolution) for one side.
 *   replaces FusedCrownExecutor.run for kind == "conv2d", fused_crown.py:365-400
 *            (TVM kernel backends/tvm/fused_crown_conv2d.py:202-344), i.e.
 *            _backprop_conv2d_step crown_ibp.py:1106-1173 with Conv2dLinearOperator.to_dense
 *            boundflow/runtime/linear_operator.py:1067-1092.
 * A [B,S,Co*Ho*Wo]; slopes [B,Co*Ho*Wo]; W OIHW [Co,Ci,kh,kw]; bias [Co] or NULL;
 * A_prev [B,S,Ci*Hi*Wi]; delta [B,S] as above.  groups = 1, dilation = 1; any kernel size,
 * stride and padding with 0 <= output_padding < stride.  `scratch` (device,
 * bf_crown_relu_conv2d_bwd_scratch_bytes) holds the ReLU-scaled coefficients between the
 * two passes and, for wide layers, partial sums of delta.  Without slopes (no ReLU) it is
 * optional: NULL, or a buffer smaller than bf_crown_relu_conv2d_bwd_scratch_bytes, is simply not
 * used; with slopes a buffer of at least that size is required (BF_E_WORKSPACE otherwise). */
size_t bf_crown_relu_conv2d_bwd_scratch_bytes(int B, int S, int Co, int Ho, int Wo);
int bf_crown_relu_conv2d_bwd(const float* A, int side,
                             const float* alpha_u, const float* alpha_l,
                             const float* beta_u, const float* beta_l,
                             const float* W, const float* bias,
                             float* A_prev, float* delta, int accumulate,
                             void* scratch, size_t scratch_bytes,
                             int B, int S, int Ci, int Hi, int Wi, int Co, int Ho, int Wo,
                             int kh, int kw, int sh, int sw, int ph, int pw, bf_stream_t stream);

/* Building blocks for graphs that are not chains (residual add, fan-out): the reference routes them in
 * _run_crown_backward_from_trace, boundflow/runtime/crown_ibp.py:1748-2030.
 *   bf_crown_relu_bwd: ReLU backward alone, _backprop_relu_step_dense_reference crown_ibp.py:1211-1298:
 *            A_prev = A * slope_sel, delta (+)= sum_k A * intercept_sel.  A, A_prev [B,S,n] (may alias);
 *            slopes [B,n]; scratch (bf_crown_relu_bwd_scratch_bytes) only for n > 4096 with delta.
 *   bf_accumulate: dst += src, _accumulate_backward_state crown_ibp.py:879-913.
 *   bf_interval_relu / bf_interval_add / bf_interval_mul: IntervalDomain.relu_transformer /
 *            elementwise_transformer("add" | "mul"), boundflow/domains/interval.py:88-114 (mul: the smallest and
 *            largest of the four corner products; same-shape operands, the caller expands a broadcast one). */
size_t bf_crown_relu_bwd_scratch_bytes(int B, int S, int n);
int bf_crown_relu_bwd(const float* A, int side, const float* alpha_u, const float* alpha_l,
                      const float* beta_u, const float* beta_l, float* A_prev, float* delta, int accumulate,
                      void* scratch, size_t scratch_bytes, int B, int S, int n, bf_stream_t stream);
int bf_accumulate(float* dst, const float* src, long long n, bf_stream_t stream);
int bf_interval_relu(const float* l, const float* u, float* out_l, float* out_u, long long n, bf_stream_t stream);
int bf_interval_add(const float* a_l, const float* a_u, const float* b_l, const float* b_u,
                    float* out_l, float* out_u, long long n, bf_stream_t stream);
int bf_interval_mul(const float* a_l, const float* a_u, const float* b_l, const float* b_u,
                    float* out_l, float* out_u, long long n, bf_stream_t stream);

/* Allocation-free variant of bf_crown_relu_conv2d_bwd.  It has no counterpart in the
 * reference.  It exists for callers that cannot hand over (or obtain) device scratch when
 * they call: services whose device pool is sized at start-up and then frozen, plugins loaded
 * into a process that already owns all device memory, runtimes that ban cudaMalloc / cudaFree
 * on the request path because those calls synchronise the device.
 * The ReLU-scaled coefficients are staged in an array that is part of the library image
 * (bf_crown_relu_conv2d_bwd_noalloc_max_bytes() = 16 MiB, held on every GPU that loads the
 * library until the process exits); requests whose bf_crown_relu_conv2d_bwd_scratch_bytes
 * (about B*S*Co*Ho*Wo*4 bytes) is beyond that return BF_E_WORKSPACE.  The first call on each device looks up the array's device address; make
 * that call with the device current and before any stream capture.  No call allocates or
 * frees memory.  The array is shared by all calls and keeps the last call's contents (every
 * element a call reads was written by that same call, so nothing needs clearing); two calls
 * whose kernels may overlap on the GPU (different streams) race on it. */
size_t bf_crown_relu_conv2d_bwd_noalloc_max_bytes(void);
int bf_crown_relu_conv2d_bwd_noalloc(const float* A, int side,
                                     const float* alpha_u, const float* alpha_l,
                                     const float* beta_u, const float* beta_l,
                                     const float* W, const float* bias,
                                     float* A_prev, float* delta, int accumulate,
                                     int B, int S, int Ci, int Hi, int Wi, int Co, int Ho, int Wo,
                                     int kh, int kw, int sh, int sw, int ph, int pw, bf_stream_t stream);

/* Concretisation of an affine form over a box (or L-inf ball: rad == eps).
 *   replaces BoxPerturbation.concretize_affine perturbation.py:327-359 and
 *            LpBallPerturbation.concretize_affine (p = inf) perturbation.py:175-222.
 * A [B,S,n0]; mid, rad [B,n0]; bias_in [B,S] or NULL; out [B,S]:
 *   lower: A.mid - |A|.rad + bias_in     upper: A.mid + |A|.rad + bias_in */
int bf_concretize(const float* A, const float* mid, const float* rad, const float* bias_in,
                  float* out, int side, int B, int S, int n0, bf_stream_t stream);

/* IBP linear layer with one weight matrix per batch element -- the output spec merged into the
 * last layer (W' = C @ W, b' = C @ b; _fuse_linear_spec_into_last_linear,
 * boundflow/planner/interval_v1.py:85-163), evaluated as the batched-W branch of
 * PythonTaskExecutor.run_ibp, boundflow/runtime/task_executor.py:231-245:
 * out = mid @ W'^T -/+ rad @ |W'|^T + b'.  in_l, in_u [B,n_in] (relu_in != 0: clamped at 0 first);
 * W [B,S,n_in]; bias [B,S] or NULL; out_l, out_u [B,S]. */
int bf_ibp_linear_batched(const float* in_l, const float* in_u, int relu_in, const float* W, const float* bias,
                          float* out_l, float* out_u, int B, int S, int n_in, bf_stream_t stream);

/* Lp-ball input sets (p = 1, 2, inf), the non-box branch of the reference's perturbations.
 *   bf_row_dual_norms: out[r] = scale * ||W[r,:]||_q (q dual to p) -- the row norms of
 *            LpBallPerturbation.concretize_matmul, boundflow/runtime/perturbation.py:102-134.
 *   bf_ibp_linear_lp: first Linear layer on a ball: centre @ W^T + b -/+ row_dev, then the
 *            same constraint / split clamps as bf_ibp_linear (row_dev [n_out] from bf_row_dual_norms
 *            with scale = eps).
 *   bf_concretize_lp: A.centre -/+ eps * ||A_row||_q + bias_in, replaces
 *            LpBallPerturbation.concretize_affine perturbation.py:175-222 (row norms
 *            boundflow/runtime/linear_operator.py:365-372). */
int bf_row_dual_norms(const float* W, int n_rows, int n_cols, int p, float scale, float* out, bf_stream_t stream);
int bf_ibp_linear_lp(const float* center, const float* row_dev, const float* W, const float* bias,
                     const int8_t* split, int split_stride, const float* cons_l, const float* cons_u,
                     float* out_l, float* out_u, int* infeasible, int B, int n_in, int n_out, bf_stream_t stream);
int bf_concretize_lp(const float* A, const float* center, float eps, int p, const float* bias_in,
                     float* out, int side, int B, int S, int n0, bf_stream_t stream);

/* First-layer infeasibility certificate per domain
 *   replaces _is_infeasible_split_first_layer_convex_combo, boundflow/runtime/alpha_beta_crown.py:391-532
 *            (half-spaces of a Linear first layer, _collect_first_layer_split_halfspaces 262-388), which the
 *            reference evaluates for batch size 1 only; here every domain of the batch gets its own.
 * split int8 [B,n1] (row stride split_stride: n1, or 0 for one shared row) on the FIRST ReLU, W1 [n1,n0],
 * b1 [n1] or NULL, box mid/rad [B,n0].  Per domain: half-spaces s_j*(W1[j].x + b1[j]) >= 0 in ascending j;
 * weights softmax(logits), logits start at 0; up to `steps` Adam(lr) steps on
 * max_box (sum w_i a_i).x + sum w_i c_i, stopping at the first value < -tol (one half-space: tested directly).
 * infeasible int32 [B]: 1 certificate found, 0 none, -1 not evaluated (more than
 * bf_first_layer_certificate_max_halfspaces() half-spaces); best_value float [B] or NULL: smallest maximum
 * seen; n_halfspaces int32 [B] or NULL. */
int bf_first_layer_certificate_max_halfspaces(void);
int bf_first_layer_certificate(const int8_t* split, int split_stride, const float* W1, const float* b1,
                               const float* mid, const float* rad, int* infeasible, float* best_value,
                               int* n_halfspaces, int steps, float lr, float tol, int B, int n1, int n0,
                               bf_stream_t stream);
/* The same on an L1 / L2 ball (p = BF_NORM_L1 | BF_NORM_L2) around center [B,n0]: the maximum of a combination is
 * a.center + eps * ||a||_q, LpBallPerturbation.concretize_affine boundflow/runtime/perturbation.py:175-222 (the reference's
 * certificate calls spec.perturbation.concretize_affine, alpha_beta_crown.py:439-441, 476-478). */
int bf_first_layer_certificate_lp(const int8_t* split, int split_stride, const float* W1, const float* b1,
                                  const float* center, float eps, int p, int* infeasible, float* best_value,
                                  int* n_halfspaces, int steps, float lr, float tol, int B, int n1, int n0,
                                  bf_stream_t stream);

/* Half-space rows of a Conv2d FIRST layer for the certificate above
 *   replaces the conv2d branch of _collect_first_layer_split_halfspaces, boundflow/runtime/alpha_beta_crown.py:325-387
 *            (one-hot row through DenseLinearOperator.conv2d_right(...).to_dense()).
 * rows int32 [n_rows]: flat indices (co*Ho + ho)*Wo + wo of the layer's outputs, usually the split neurons of the
 * batch in ascending order; out_W [n_rows, Ci*Hi*Wi] receives the filter W[co] (OIHW) placed at
 * (ho*sh - ph, wo*sw - pw), out_b [n_rows] or NULL receives bias[co] (0 without bias).  The result, with the split
 * columns gathered in the same order, is what bf_first_layer_certificate takes as W1 / b1 / split.  groups = 1,
 * dilation = 1. */
int bf_conv2d_dense_rows(const float* W, const float* bias, const int* rows, int n_rows, float* out_W, float* out_b,
                         int Ci, int Hi, int Wi, int Co, int Ho, int Wo, int kh, int kw, int sh, int sw, int ph, int pw,
                         bf_stream_t stream);

/* Verdict per domain: proven iff min over spec rows of the lower bound >= threshold - tol.
 *   replaces the node test in solve_bab_mlp, boundflow/runtime/bab.py:881-895
 *            (bounds.lower.min() then >=: a NaN bound never proves a node, and neither does it here).
 * lower [B,S]; verdict int8 [B] (1 proven, 0 not); min_lower [B] or NULL (NaN when any row is NaN).
 * bf_verdict_masked additionally takes the per-domain infeasible flags of the IBP sweep
 * (int32 [B] or NULL): a flagged domain's bounds are meaningless, its verdict is 0. */
int bf_verdict_masked(const float* lower, float threshold, float tol, const int* infeasible, int8_t* verdict,
                      float* min_lower, int B, int S, bf_stream_t stream);
int bf_verdict(const float* lower, float threshold, float tol, int8_t* verdict, float* min_lower,
               int B, int S, bf_stream_t stream);

/* ------------------------------------------------------------------------
 * Whole-chain drivers (host loops over the kernels above; no host sync)
 * ---------------------------------------------------------------------- */

typedef struct bf_layer_desc {
  int op;            /* BF_OP_* */
  const float* W;    /* linear [n_out,n_in]; conv2d OIHW; NULL otherwise */
  const float* bias; /* [n_out] / [Co] or NULL */
  int n_in, n_out;   /* flattened feature counts in / out of this layer */
  int Ci, Hi, Wi, Co, Ho, Wo, kh, kw, sh, sw, ph, pw; /* conv2d only */
} bf_layer_desc;

typedef struct bf_chain bf_chain; /* opaque: a validated copy of the layer list */

int bf_chain_create(const bf_layer_desc* layers, int n_layers, bf_chain** out);
void bf_chain_destroy(bf_chain* chain);
int bf_chain_num_relu(const bf_chain* chain);

/* Tensor-core path set-up (no counterpart in the reference, whose GEMMs are cuBLAS calls made
 * by torch.einsum, boundflow/runtime/linear_operator.py:585-586).  The CROWN backward and
 * adjoint contractions of Linear layers run as tcgen05 (kind::tf32) tiles with 3xTF32 split
 * operands once the static weights have been split into hi/lo parts and packed into the
 * shared-memory image the MMA consumes.  bf_chain_tc_prepare does that packing into a
 * caller-owned device buffer of bf_chain_tc_bytes(chain) bytes (256-byte aligned) that must
 * outlive the chain; without it, or with the environment variable BF_B200_FORCE_FFMA=1, or
 * for tiny problems, the FP32 FFMA kernels are used.  Every wait inside the tensor-core
 * kernels is bounded; bf_chain_tc_status (synchronous) returns non-zero in *status if a
 * wait ever expired, in which case results of that call are invalid. */
size_t bf_chain_tc_bytes(const bf_chain* chain);
int bf_chain_tc_prepare(bf_chain* chain, void* buffer, size_t bytes, bf_stream_t stream);
int bf_chain_tc_status(const bf_chain* chain, int* status);

/* One IBP sweep that records every ReLU pre-activation.
 *   replaces _forward_ibp_trace_mlp crown_ibp.py:101-342 (and the op loop of
 *            PythonTaskExecutor.run_ibp boundflow/runtime/task_executor.py:127-358,
 *            TVMTaskExecutor.run_ibp boundflow/runtime/tvm_executor.py:730-1034).
 * in_a,in_b [B,n0] per in_mode; `splits`, `cons_l`, `cons_u`, `pre_l`, `pre_u` are HOST arrays
 * of device pointers, one entry per ReLU in chain order (entries or whole arrays may be NULL
 * for splits/constraints); pre_l[r],pre_u[r] [B,n_r] receive the clamped pre-activation
 * bounds; out_l,out_u [B,n_last] the chain output bounds; infeasible int32 [B] or NULL.
 * scratch: 2 * B * max_width floats (device) used when a layer's output is not a ReLU input. */
int bf_chain_ibp(const bf_chain* chain, const float* in_a, const float* in_b, int in_mode,
                 const int8_t* const* splits, const int* split_strides,
                 const float* const* cons_l, const float* const* cons_u,
                 float* const* pre_l, float* const* pre_u,
                 float* out_l, float* out_u, int* infeasible,
                 float* scratch, size_t scratch_bytes, int B, bf_stream_t stream);

size_t bf_chain_crown_workspace_bytes(const bf_chain* chain, int B, int S, int upto_layer);

/* One CROWN backward sweep + concretisation for one side.
 *   replaces _run_crown_backward_from_trace crown_ibp.py:1669-2051 for chain graphs
 *            (run_crown_ibp_mlp crown_ibp.py:2054, run_crown_ibp_mlp_from_forward_trace crown_ibp.py:2136).
 * Bounds C @ (output of layers[0:upto_layer]) (upto_layer = number of layers for the chain
 * output).  C [B,S,O] (a spec shared by all domains is expanded by the caller).
 * alpha_u/beta_u/alpha_l: HOST arrays of device pointers per ReLU, each [B,n_r] (from
 * bf_relu_relax); add: per ReLU [B,n_r] or NULL entries / NULL array, added to the coefficients of the requested side
 * behind the ReLU (relu_pre_add_coeff_l for BF_SIDE_LOWER, relu_pre_add_coeff_u for BF_SIDE_UPPER, crown_ibp.py:1270-1296).
 * Input set: norm_p = BF_NORM_BOX with mid, rad [B,n0] (eps ignored), or an Lp ball with
 * mid = centre [B,n0], rad = NULL and norm_p in {BF_NORM_INF, BF_NORM_L2, BF_NORM_L1}.  out [B,S]. */
int bf_chain_crown(const bf_chain* chain, int upto_layer, int side,
                   const float* C,
                   const float* const* alpha_u, const float* const* beta_u, const float* const* alpha_l,
                   const float* const* add,
                   const float* mid, const float* rad, int norm_p, float eps, float* out,
                   void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);

/* bf_chain_crown that also records the objective influence of every ReLU below the bounded value:
 * influence[r][b, j] = max(influence[r][b, j], max_s |A[b, s, j]|) with A the coefficients that reach
 * ReLU r in this sweep.  Calling it for both sides on zero-filled buffers gives
 * max(max_s |A_u|, max_s |A_l|), the tensor run_crown_ibp_mlp_with_relu_influence_from_forward_trace
 * returns (boundflow/runtime/crown_ibp.py:1810-1834, 2201-2240).  influence: HOST array of device
 * pointers [B,n_r] (NULL entries are skipped). */
int bf_chain_crown_influence(const bf_chain* chain, int upto_layer, int side,
                             const float* C,
                             const float* const* alpha_u, const float* const* beta_u, const float* const* alpha_l,
                             const float* const* add,
                             const float* mid, const float* rad, int norm_p, float eps, float* out,
                             float* const* influence,
                             void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);

/* bf_chain_crown for spec rows that are rows first_row .. first_row+S-1 of the identity, the same
 * for every domain: the sweeps that bound an intermediate value neuron by neuron
 * (run_crown_ibp_mlp_from_forward_trace(output_value=name, linear_spec_C=I_chunk) as composed in
 * boundflow/runtime/native_intermediate_refinement.py:923-973).  layers[upto_layer-1] must be the
 * affine layer that produces the bounded value.  Its backward step then copies weight rows /
 * kernel patches instead of multiplying an identity by them; everything else, and every other
 * argument, is as in bf_chain_crown (same workspace size). */
int bf_chain_crown_onehot(const bf_chain* chain, int upto_layer, int side, int first_row,
                          const float* const* alpha_u, const float* const* beta_u, const float* const* alpha_l,
                          const float* const* add,
                          const float* mid, const float* rad, int norm_p, float eps, float* out,
                          void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);

size_t bf_chain_alpha_workspace_bytes(const bf_chain* chain, int B, int S);
/* Input set of the alpha / beta entry points below: as in bf_chain_crown -- norm_p = BF_NORM_BOX with
 * mid, rad [B,n0], or an Lp ball with mid = centre, rad = NULL, eps and norm_p in
 * {BF_NORM_INF, BF_NORM_L2, BF_NORM_L1} (LpBallPerturbation.concretize_affine,
 * boundflow/runtime/perturbation.py:175-222; the gradient sweep then starts from
 * centre - eps * d||A_0||_q / dA_0). */

/* Per-domain alpha-CROWN: steps+1 lower-bound evaluations, analytic alpha gradient,
 * Adam(lr, 0.9, 0.999, 1e-8), projection to [0,1], strict per-domain best tracking, and
 * one upper-bound evaluation at the best alpha.  Chains affine (ReLU affine)* of Linear / Conv2d layers (flatten layers anywhere); beta needs Linear layers only.
 *   replaces run_alpha_beta_crown_mlp(per_batch_params=True, objective="lower") with beta at
 *            zero, boundflow/runtime/alpha_beta_crown.py:643-941 (loop 756-923), whose gradient
 *            comes from torch autograd through crown_ibp.py:1211-1298.
 * pre_l,pre_u: HOST arrays of device pointers [B,n_r] (from bf_chain_ibp);
 * alpha: HOST array of device pointers [B,n_r], in: start values, out: values after the last step;
 * best_alpha: same layout, out: alpha of each domain's best evaluation;
 * best_lower,best_upper [B,S] (best_upper may be NULL to skip the upper sweep);
 * best_metric [B] or NULL. */
int bf_chain_alpha_crown(const bf_chain* chain,
                         const float* C,
                         const float* const* pre_l, const float* const* pre_u,
                         float* const* alpha, float* const* best_alpha,
                         const float* mid, const float* rad, int norm_p, float eps,
                         float* best_lower, float* best_upper, float* best_metric,
                         int steps, float lr, int spec_reduce,
                         void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);

/* alpha-beta-CROWN: as bf_chain_alpha_crown, plus one multiplier beta >= 0 per (domain, split
 * neuron) whose term -beta*s (s = split sign) is added to the lower coefficients at that ReLU and
 * which the same Adam recurrences update (gradient -s * sum over spec rows of the adjoint value).
 *   replaces run_alpha_beta_crown_mlp(per_batch_params=True, objective="lower"),
 *            boundflow/runtime/alpha_beta_crown.py:643-941, with _beta_to_relu_pre_add_coeff 615-640.
 * beta, best_beta: HOST arrays of device pointers [B,n_r] (in: start values / out: last and best);
 * splits: HOST array of int8 device pointers [B,n_r] (or [1,n_r] with split_strides[r] == 0; NULL
 * entries = no split at that ReLU).  beta == NULL degenerates to bf_chain_alpha_crown.
 * Workspace: bf_chain_alpha_beta_workspace_bytes. */
size_t bf_chain_alpha_beta_workspace_bytes(const bf_chain* chain, int B, int S);
int bf_chain_alpha_beta_crown(const bf_chain* chain,
                              const float* C,
                              const float* const* pre_l, const float* const* pre_u,
                              float* const* alpha, float* const* best_alpha,
                              float* const* beta, float* const* best_beta,
                              const int8_t* const* splits, const int* split_strides,
                              const float* mid, const float* rad, int norm_p, float eps,
                              float* best_lower, float* best_upper, float* best_metric,
                              int steps, float lr, int spec_reduce,
                              void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);
/* The same loop with every spec reduction of the reference's objective="lower" (_objective_metric / _loss,
 * boundflow/runtime/alpha_beta_crown.py:535-612, per-domain form 787-818): spec_reduce BF_REDUCE_MEAN, _SUM,
 * _MIN (smallest spec row) or _SOFTMIN (-soft_tau * logsumexp(-rows / soft_tau), soft_tau > 0).  For _MIN and
 * _SOFTMIN the gradient sweep weights every spec row by d objective / d lower (one-hot at the first minimum, or
 * softmax(-rows / soft_tau)): the weights scale the coefficients kept at every ReLU (alpha gradient) and, with beta
 * parameters, the per-domain sums of the adjoint values (beta gradient; these layers then run on the row-major
 * tensor-core adjoint kernel or the FFMA tiles, which carry the row weight). */
int bf_chain_alpha_beta_crown_reduce(const bf_chain* chain,
                                     const float* C,
                                     const float* const* pre_l, const float* const* pre_u,
                                     float* const* alpha, float* const* best_alpha,
                                     float* const* beta, float* const* best_beta,
                                     const int8_t* const* splits, const int* split_strides,
                                     const float* mid, const float* rad, int norm_p, float eps,
                                     float* best_lower, float* best_upper, float* best_metric,
                                     int steps, float lr, int spec_reduce, float soft_tau,
                                     void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);

/* The alpha loop for the objectives that involve both bounds (objective="gap" | "both" of
 * run_alpha_beta_crown_mlp, boundflow/runtime/alpha_beta_crown.py:807-818 with _objective_metric / _loss 535-612;
 * these objectives carry no beta term, 763-785).  The caller passes PAIRED spec rows: C is [B, 2S, n_out] holding
 * the S rows c_s of every domain followed by their negations -c_s, so that row S+s's lower bound is minus row s's
 * upper bound and one lower-side sweep with one gradient sweep serves both bounds.  best_rows [B, 2S] receives, per
 * domain, the rows of its best iteration: lower = best_rows[:, :S], upper = -best_rows[:, S:].  objective is
 * BF_OBJECTIVE_GAP or BF_OBJECTIVE_BOTH, spec_reduce BF_REDUCE_MEAN, _MIN or _SOFTMIN (upper-side max / softmax are
 * taken as min / softmin of the negated rows); lb_weight / ub_weight apply to BF_OBJECTIVE_BOTH.
 * objective="upper" needs no entry point of its own: it is objective="lower" on the negated rows -C.
 * Workspace: bf_chain_alpha_workspace_bytes(chain, B, 2 * S). */
int bf_chain_alpha_crown_objective(const bf_chain* chain,
                                   const float* C_paired,
                                   const float* const* pre_l, const float* const* pre_u,
                                   float* const* alpha, float* const* best_alpha,
                                   const float* mid, const float* rad, int norm_p, float eps,
                                   float* best_rows, float* best_metric,
                                   int steps, float lr, int objective, int spec_reduce, float soft_tau,
                                   float lb_weight, float ub_weight,
                                   void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);

/* The pieces of the per-domain alpha / beta loop as separate entry points, for graphs that are not chains (residual
 * add, concat, fan-out): the reference's alpha-beta function accepts such graphs because its sweep is the generic
 * _run_crown_backward_from_trace (boundflow/runtime/crown_ibp.py:1669-2051) under autograd; here the caller walks the
 * graph and calls, per value, the layer-level backward entry points above plus:
 *   bf_relu_split_apply   _apply_relu_split, crown_ibp.py:70-98, on the bounds of one ReLU input, in place: split +1
 *                         clamps l to >= 0, -1 clamps u to <= 0; infeasible[b] (int32, may be NULL) is OR-ed with
 *                         "some neuron has l > u".  split int8 [B,n] (stride n) or [1,n] (stride 0).
 *   bf_interval_intersect the constraint intersection crown_ibp.py:186-209 on the bounds of one ReLU input, in place:
 *                         l = max(l, cons_l), u = min(u, cons_u) ([B,n] each); infeasible[b] (int32, may be NULL) is OR-ed
 *                         with "some neuron has l > u".
 *   bf_rows_add_broadcast A[b,s,:] += v[b,:] (v_stride = n) or v[:] (v_stride = 0): the split term -beta*s added to the
 *                         lower coefficients after a ReLU backward step (alpha_beta_crown.py:615-640), and the bias of a
 *                         forward Linear step on rows.
 *   bf_adjoint_start_box  start of the gradient sweep: A0 [B,S,n0] (final lower coefficients) becomes
 *                         h0 = mid - sgn(A0) * rad in place, the point at which the lower bound is attained.
 *   bf_adjoint_start_lp   the same for an Lp ball (p = BF_NORM_L1 | _L2 | _INF): h0 = centre - eps * (the unit-ball point
 *                         that attains the dual norm of the row), LpBallPerturbation.concretize_affine
 *                         perturbation.py:175-222.
 *   bf_rows_conv2d_fwd    forward convolution of M rows [M,Ci,Hi,Wi] -> [M,Co,Ho,Wo] (+ bias): the gradient sweep's
 *                         step through a Conv2d layer.  (A Linear layer on rows is bf_crown_relu_linear_bwd without
 *                         slopes on the transposed weight, plus bf_rows_add_broadcast for the bias.)
 *   bf_relu_adjoint_rows  G [B,S,n] holds the relaxed network's value at a ReLU input (the forward image of h0), Ahat
 *                         [B,S,n] the lower coefficients that arrived at the ReLU's output in the backward sweep:
 *                         grad[b,j] += sum_s [l<0<u][Ahat>=0] Ahat*G, gsum[b,j] += sum_s row_weight[b,s]*G (gsum NULL
 *                         without beta; row_weight NULL = 1, else d objective / d row for min / softmin), then G
 *                         becomes the ReLU's output on the chosen line (alpha_l*G where Ahat >= 0, alpha_u*G + beta_u
 *                         elsewhere), in place.
 *   bf_alpha_select_best  per-domain objective reduce_s(cur[b,s]) (BF_REDUCE_*), strict best-of against best_metric
 *                         (first != 0 initialises), improve[b] flags, best_lower rows copied on improvement;
 *                         row_weight [B,S] or NULL receives d objective / d cur for _MIN / _SOFTMIN
 *                         (alpha_beta_crown.py:787-902).
 *   bf_alpha_adam_step    torch.optim.Adam step t (0-based; betas 0.9 / 0.999, eps 1e-8) on alpha with gradient
 *                         grad * (-1/S for _MEAN, -1 otherwise), projection to [0,1], grad cleared; best_alpha receives
 *                         the alpha BEFORE the step where improve[b] != 0; slope_l receives the next lower slope
 *                         (0 if u <= 0, 1 if l >= 0, alpha otherwise); do_update == 0 only snapshots (913-923).
 *   bf_beta_adam_step     the same for beta >= 0 with gradient -split * gsum (gsum cleared), and add = -beta*split
 *                         for the next sweep; improve / best_beta may be NULL. */
int bf_relu_split_apply(float* l, float* u, const int8_t* split, int split_stride, int* infeasible, int B, int n,
                        bf_stream_t stream);
int bf_interval_intersect(float* l, float* u, const float* cons_l, const float* cons_u, int* infeasible, int B, int n,
                          bf_stream_t stream);
int bf_rows_add_broadcast(float* A, const float* v, int v_stride, int B, int S, int n, bf_stream_t stream);
int bf_adjoint_start_box(float* A0, const float* mid, const float* rad, int B, int S, int n0, bf_stream_t stream);
int bf_adjoint_start_lp(float* A0, const float* center, float eps, int p, int B, int S, int n0, bf_stream_t stream);
int bf_rows_conv2d_fwd(const float* in, const float* W, const float* bias, float* out, int M, int Ci, int Hi, int Wi,
                       int Co, int Ho, int Wo, int kh, int kw, int sh, int sw, int ph, int pw, bf_stream_t stream);
int bf_relu_adjoint_rows(float* G, const float* Ahat, const float* alpha_u, const float* alpha_l, const float* beta_u,
                         const float* pre_l, const float* pre_u, float* grad, float* gsum, const float* row_weight, int B,
                         int S, int n, bf_stream_t stream);
int bf_alpha_select_best(const float* cur, float* best_lower, float* best_metric, int* improve, int first, int spec_reduce,
                         float soft_tau, float* row_weight, int B, int S, bf_stream_t stream);
int bf_alpha_adam_step(float* alpha, float* m, float* v, float* grad, const int* improve, float* best_alpha,
                       const float* pre_l, const float* pre_u, float* slope_l, int t, float lr, int spec_reduce, int S,
                       int do_update, int B, int n, bf_stream_t stream);
int bf_beta_adam_step(float* beta, float* m, float* v, float* gsum, const int8_t* split, int split_stride,
                      const int* improve, float* best_beta, float* add, int t, float lr, int spec_reduce, int S,
                      int do_update, int B, int n, bf_stream_t stream);

/* The remaining pieces, for the other objectives and the shared-parameter mode on such graphs:
 *   bf_alpha_select_best_paired  cur [B,2S] holds the lower bounds of S spec rows followed by those of their negations
 *                         (upper[b,s] = -cur[b,S+s]); per-domain objective BF_OBJECTIVE_GAP = -reduce_s(upper - lower) or
 *                         BF_OBJECTIVE_BOTH = lb_weight * reduce_s(lower) - ub_weight * reduce_s(upper) with reduce = mean |
 *                         min (max on the upper side) | softmin (alpha_beta_crown.py:787-818), strict best-of as above;
 *                         row_weight [B,2S] or NULL receives d objective / d cur (all >= 0 for weights >= 0).
 *   bf_rows_scale         A[r,:] *= w[r] for M rows of n: the row weights applied to the coefficients kept at every ReLU
 *                         before the gradient sweep.
 *   bf_rows_colmax_abs    out[b,j] = max(out[b,j], max_s |A[b,s,j]|): the objective influence of a ReLU from the
 *                         coefficients that reach it (crown_ibp.py:1810-1834), one call per side.
 *   bf_shared_metric      whole-batch metric mean(values[0..M)) with strict best-of against best_metric[0]; improve[0]
 *                         (alpha_crown.py:215-220; first != 0 initialises).
 *   bf_copy_if            dst = src when flag[0] != 0 (the batch's best bounds).
 *   bf_shared_adam_step   Adam step t on ONE parameter row [n] shared by the batch: gradient = grad_scale * sum_b grad[b,j]
 *                         (times -split[b,j] when `split` is given: a shared beta), grad cleared; alpha projected to [0,1],
 *                         beta (is_beta != 0) to >= 0; best receives the parameter BEFORE the step when improve[0] != 0;
 *                         scratch holds bf_shared_adam_scratch_floats(B, n) floats; do_update == 0 only snapshots.
 *   bf_shared_beta_add    add[b,j] = -beta[j] * split[b,j]: the split term of a shared beta for the next sweep. */
int bf_alpha_select_best_paired(const float* cur, float* best_rows, float* best_metric, int* improve, int first, int objective,
                                int spec_reduce, float soft_tau, float lb_weight, float ub_weight, float* row_weight, int B,
                                int S, bf_stream_t stream);
int bf_rows_scale(float* A, const float* w, long long M, int n, bf_stream_t stream);
int bf_rows_colmax_abs(const float* A, float* out, int B, int S, int n, bf_stream_t stream);
int bf_shared_metric(const float* values, long long M, float* best_metric, int* improve, int first, bf_stream_t stream);
int bf_copy_if(const float* src, float* dst, long long n, const int* flag, bf_stream_t stream);
size_t bf_shared_adam_scratch_floats(int B, int n);
int bf_shared_adam_step(float* param, float* m, float* v, float* grad, const int8_t* split, int split_stride, float* scratch,
                        const int* improve, float* best, int t, float lr, float grad_scale, int do_update, int is_beta, int B,
                        int n, bf_stream_t stream);
int bf_shared_beta_add(const float* beta, const int8_t* split, int split_stride, float* add, int B, int n, bf_stream_t stream);

/* Branching hint: per domain the ReLU (chain order) and neuron with the widest gap u - l among
 * unstable neurons (l < 0 < u); earlier ReLUs and lower indices win ties; -1/-1 when none.
 *   replaces _branch_choices_from_relu_pre, boundflow/runtime/alpha_beta_crown.py:145-182.
 * pre_l, pre_u: HOST arrays of device pointers [B,widths[r]]; outputs best_gap float [B],
 * best_relu / best_idx int32 [B]. */
int bf_branch_scores(const float* const* pre_l, const float* const* pre_u, const int* widths, int n_relu,
                     float* best_gap, int* best_relu, int* best_idx, int B, bf_stream_t stream);

/* Gradient of  -sum_b reduce_s lower[b,s]  w.r.t. every per-domain alpha at the given alpha
 * (the tensor torch autograd hands to Adam in alpha_beta_crown.py:913-917), plus the lower
 * bounds themselves.  grad: HOST array of device pointers [B,n_r]; lower [B,S]. */
int bf_chain_alpha_grad(const bf_chain* chain,
                        const float* C,
                        const float* const* pre_l, const float* const* pre_u,
                        const float* const* alpha,
                        const float* mid, const float* rad, int norm_p, float eps,
                        float* const* grad, float* lower, int spec_reduce,
                        void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);

/* alpha(-beta)-CROWN with ONE alpha (and one beta) per neuron shared by every domain and spec row:
 * replaces run_alpha_crown_mlp, boundflow/runtime/alpha_crown.py:137-261, and the shared-parameter
 * mode (per_batch_params=False) of run_alpha_beta_crown_mlp, boundflow/runtime/alpha_beta_crown.py:643-941,
 * for objective="lower", spec_reduce="mean".  steps+1 lower sweeps at the broadcast parameters;
 * loss = -mean over all B*S lower bounds; gradient = column sums over the batch of the per-domain
 * adjoint gradient (two fixed-order stages; beta: of -split * sum_s g); Adam; alpha clamped to [0,1],
 * beta to >= 0; strict best-of on the scalar metric, which keeps the whole batch's bounds and the
 * parameters of the best iteration.
 * alpha / best_alpha (and beta / best_beta, or NULL for alpha only): HOST arrays of device pointers
 * [n_r], updated in place; splits: HOST array of int8 device pointers [B,n_r] (row stride
 * split_strides[r], 0 = one shared row) or NULL entries, needed with beta; best_lower [B,S];
 * best_upper [B,S] or NULL (one upper sweep at the best alpha); best_metric: device float[1] or NULL.
 * Workspace: bf_chain_alpha_shared_workspace_bytes(chain, B, S, with_beta). */
size_t bf_chain_alpha_shared_workspace_bytes(const bf_chain* chain, int B, int S, int with_beta);
int bf_chain_alpha_crown_shared(const bf_chain* chain,
                                const float* C,
                                const float* const* pre_l, const float* const* pre_u,
                                float* const* alpha, float* const* best_alpha,
                                float* const* beta, float* const* best_beta,
                                const int8_t* const* splits, const int* split_strides,
                                const float* mid, const float* rad, int norm_p, float eps,
                                float* best_lower, float* best_upper, float* best_metric,
                                int steps, float lr,
                                void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);
/* The shared-alpha loop with the other objectives and spec reductions of run_alpha_crown_mlp
 * (boundflow/runtime/alpha_crown.py:93-134, 137-261: `objective`, `spec_reduce`, `soft_tau`, `lb_weight`, `ub_weight`):
 * the whole-batch metric is the mean over the domains of the per-domain objective.  objective 0 = "lower" on the S rows
 * as given (spec_reduce BF_REDUCE_MEAN, _MIN or _SOFTMIN; best_rows [B,S], best_upper [B,S] or NULL); BF_OBJECTIVE_GAP /
 * _BOTH take PAIRED rows like bf_chain_alpha_crown_objective (C [B,2S,n_out], best_rows [B,2S], best_upper ignored;
 * workspace for 2*S rows); "upper" is "lower" on the negated rows.  Alpha only. */
int bf_chain_alpha_crown_shared_objective(const bf_chain* chain,
                                          const float* C,
                                          const float* const* pre_l, const float* const* pre_u,
                                          float* const* alpha, float* const* best_alpha,
                                          const float* mid, const float* rad, int norm_p, float eps,
                                          float* best_rows, float* best_upper, float* best_metric,
                                          int steps, float lr, int objective, int spec_reduce, float soft_tau,
                                          float lb_weight, float ub_weight,
                                          void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);
/* bf_chain_alpha_crown_shared with the min / softmin spec reductions of the lower objective AND beta parameters
 * (run_alpha_beta_crown_mlp(per_batch_params=False, spec_reduce=...), boundflow/runtime/alpha_beta_crown.py:787-805): the
 * per-row weights d objective / d lower scale the kept coefficients (alpha gradient) and the per-domain sums of the
 * adjoint values (beta gradient).  spec_reduce BF_REDUCE_MEAN | _MIN | _SOFTMIN; other arguments as above. */
int bf_chain_alpha_beta_crown_shared_reduce(const bf_chain* chain,
                                            const float* C,
                                            const float* const* pre_l, const float* const* pre_u,
                                            float* const* alpha, float* const* best_alpha,
                                            float* const* beta, float* const* best_beta,
                                            const int8_t* const* splits, const int* split_strides,
                                            const float* mid, const float* rad, int norm_p, float eps,
                                            float* best_lower, float* best_upper, float* best_metric,
                                            int steps, float lr, int spec_reduce, float soft_tau,
                                            void* workspace, size_t workspace_bytes, int B, int S, bf_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* BF_B200_H */
