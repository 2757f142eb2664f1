// Shared declarations of the sm_100a training-step library: status handling, launch bookkeeping, the
// activation functions of the reference (Header_Files/Neural_Network/Activation_Functions.hpp:34-183) as device
// functions, and the interfaces between the translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <utility>

#include "myea_b200.h"

namespace myea {

// ---------------------------------------------------------------------------------------------------------
// Execution context of one handle: stream, error slot written by kernels whose bounded waits ran out,
// launch counter and optional per-class event timing.
// ---------------------------------------------------------------------------------------------------------
enum TimerClass { TC_GEMM = 0, TC_SPLIT = 1, TC_NORM = 2, TC_ELEMENTWISE = 3, TC_OPTIMIZER = 4, TC_RECURRENT = 5, TC_COMM = 6, TC_OTHER = 7 };

struct Context {
  int device = 0;
  cudaStream_t stream = nullptr;
  int *d_error_flag = nullptr;  // device int: 0 = fine, otherwise the code of the first kernel that gave up waiting
  uint64_t launches = 0;
  bool profiling = false;
  double class_ms[MYEA_TIMER_CLASSES] = {0};
  uint64_t class_launches[MYEA_TIMER_CLASSES] = {0};
  double gemm_flops = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::string error;
  int gemm_engine = 0;  // 0 = tcgen05 3xTF32, 1 = FP32 FMA
  int gemm_bn = 0;      // forced N tile of the tcgen05 kernel (0 = heuristic)
  bool dependent_launch = true;  // programmatic dependent launch for the kernels that support it
  float *sk_ws = nullptr;               // partial sums of tiles split along K (gemm_splitk_reserve)
  unsigned int *sk_counters = nullptr;  // arrival counters of those tiles, all zero between launches
  int sk_clusters = 0;                  // clusters the workspace has slots for

  void begin(TimerClass) {
    if (profiling) cudaEventRecord(ev0, stream);
  }
  void end(TimerClass c, int n_launch = 1) {
    launches += n_launch;
    class_launches[c] += n_launch;
    if (profiling) {
      cudaEventRecord(ev1, stream);
      cudaEventSynchronize(ev1);
      float ms = 0.f;
      cudaEventElapsedTime(&ms, ev0, ev1);
      class_ms[c] += ms;
    }
  }
};

// ---------------------------------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched through launch_dependent() may begin (block scheduling, barrier
// and tensor-memory setup) while the kernel before it in the stream is still draining; it must call
// grid_dependency_wait() before its first access to global memory - the wait returns when the preceding kernel has
// completed and its writes are visible - and calls grid_dependency_release() so that ITS successor may start early too.
// Launched the ordinary way the two calls do nothing.
// ---------------------------------------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_dependent(const Context &ctx, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = (ctx.dependent_launch && !ctx.profiling) ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

// ---------------------------------------------------------------------------------------------------------
// Activation functions, value and derivative, exactly as the reference codes them (steepness 1):
// tanh is 2/(1+e^-2z)-1 (Activation_Functions.hpp:45), sigmoid 1/(1+e^-z) (:40); the ELU derivative below zero is
// alpha*y with y = e^z-1 (:93-94), not alpha*e^z; the softmax derivative is 1 (cross-entropy pairing).
// ---------------------------------------------------------------------------------------------------------
// piecewise-linear approximation through six points (v_k, r_k), constant lo / hi outside (AF_STEPWISE_real, :28-31)
__host__ __device__ __forceinline__ float af_stepwise(float z, const float *v, const float *r, float lo, float hi) {
  if (z < v[0]) return lo;
  if (!(z < v[5])) return hi;
  const int k = z < v[1] ? 0 : (z < v[2] ? 1 : (z < v[3] ? 2 : (z < v[4] ? 3 : 4)));
  return (((r[k + 1] - r[k]) * (z - v[k])) / (v[k + 1] - v[k])) + r[k];
}

__host__ __device__ __forceinline__ float af_fire(uint32_t af, float z) {
  switch (af) {
    case MYEA_AF_TANH: return 2.0f / (1.0f + expf(-2.0f * z)) - 1.0f;
    case MYEA_AF_SIGMOID: return 1.0f / (1.0f + expf(-z));
    case MYEA_AF_RELU: return z < 0.0f ? 0.0f : z;
    case MYEA_AF_LEAKY_RELU: case MYEA_AF_PARAMETRIC_RELU: return z < 0.0f ? 0.01f * z : z;
    case MYEA_AF_ELU: return z < 0.0f ? (expf(z) - 1.0f) : z;
    case MYEA_AF_SELU: return 1.0507009873554804934193349852946f * (z <= 0.0f ? 1.6732632423543772848170429916717f * expf(z) - 1.6732632423543772848170429916717f : z);
    case MYEA_AF_LINEAR_PIECE: return z < 0.0f ? 0.0f : (z > 1.0f ? 1.0f : z);
    case MYEA_AF_LINEAR_PIECE_SYMMETRIC: return z < -1.0f ? -1.0f : (z > 1.0f ? 1.0f : z);
    case MYEA_AF_SIGMOID_STEPWISE: {
      const float v[6] = {-2.64665246f, -1.47221947f, -0.549306154f, 0.549306154f, 1.47221935f, 2.64665294f};
      const float r[6] = {0.00499999989f, 0.0500000007f, 0.25f, 0.75f, 0.949999988f, 0.995000005f};
      return af_stepwise(z, v, r, 0.0f, 1.0f);
    }
    case MYEA_AF_TANH_STEPWISE: {
      const float v[6] = {-2.64665294f, -1.47221935f, -0.549306154f, 0.549306154f, 1.47221935f, 2.64665294f};
      const float r[6] = {-0.99000001f, -0.899999976f, -0.5f, 0.5f, 0.899999976f, 0.99000001f};
      return af_stepwise(z, v, r, -1.0f, 1.0f);
    }
    case MYEA_AF_THRESHOLD: return z < 0.0f ? 0.0f : 1.0f;
    case MYEA_AF_THRESHOLD_SYMMETRIC: return z < 0.0f ? -1.0f : 1.0f;
    case MYEA_AF_GAUSSIAN: return expf(-z * z);
    case MYEA_AF_GAUSSIAN_SYMMETRIC: return expf(-z * z) * 2.0f - 1.0f;
    case MYEA_AF_GAUSSIAN_STEPWISE: return 0.0f;
    case MYEA_AF_ELLIOT: return (z / 2.0f) / (1.0f + fabsf(z)) + 0.5f;
    case MYEA_AF_ELLIOT_SYMMETRIC: return z / (1.0f + fabsf(z));
    case MYEA_AF_SINE: return sinf(z) / 2.0f + 0.5f;
    case MYEA_AF_SINE_SYMMETRIC: return sinf(z);
    case MYEA_AF_COSINE: return cosf(z) / 2.0f + 0.5f;
    case MYEA_AF_COSINE_SYMMETRIC: return cosf(z);
    case MYEA_AF_ISRU: return z * (1.0f / sqrtf(1.0f + z * z));
    case MYEA_AF_ISRLU: return z < 0.0f ? z * (1.0f / sqrtf(1.0f + z * z)) : z;
    default: return z;  // linear
  }
}

// Activation_Function_Derive (Neural_Network.cpp:3157-3199) at steepness 1.  The threshold functions and the stepwise
// Gaussian are not in that switch: its default branch hands back the VALUE, and so does this one.  ISRU / ISRLU divide the
// value by the summation; at a summation of exactly zero (0 / 0 in the reference) the limit 1 is used.
__host__ __device__ __forceinline__ float af_derive(uint32_t af, float z, float y) {
  switch (af) {
    case MYEA_AF_TANH: case MYEA_AF_TANH_STEPWISE: return 1.0f - y * y;
    case MYEA_AF_SIGMOID: case MYEA_AF_SIGMOID_STEPWISE: return y * (1.0f - y);
    case MYEA_AF_RELU: return z < 0.0f ? 0.0f : 1.0f;
    case MYEA_AF_LEAKY_RELU: case MYEA_AF_PARAMETRIC_RELU: return z < 0.0f ? 0.01f : 1.0f;
    case MYEA_AF_ELU: return z < 0.0f ? y : 1.0f;
    case MYEA_AF_SELU: return 1.0507009873554804934193349852946f * (z <= 0.0f ? (y + 1.6732632423543772848170429916717f) : 1.0f);
    case MYEA_AF_GAUSSIAN: return -2.0f * z * y;
    case MYEA_AF_GAUSSIAN_SYMMETRIC: return -2.0f * z * (y + 1.0f);
    case MYEA_AF_ELLIOT: { const float a = 1.0f + fabsf(z); return 1.0f / (2.0f * a * a); }
    case MYEA_AF_ELLIOT_SYMMETRIC: { const float a = 1.0f + fabsf(z); return 1.0f / (a * a); }
    case MYEA_AF_SINE: return cosf(z) / 2.0f;
    case MYEA_AF_SINE_SYMMETRIC: return cosf(z);
    case MYEA_AF_COSINE: return -sinf(z) / 2.0f;
    case MYEA_AF_COSINE_SYMMETRIC: return -sinf(z);
    case MYEA_AF_ISRU: { if (z == 0.0f) return 1.0f; const float q = y / z; return q * q * q; }
    case MYEA_AF_ISRLU: { if (!(z < 0.0f)) return 1.0f; const float q = y / z; return q * q * q; }
    case MYEA_AF_THRESHOLD: case MYEA_AF_THRESHOLD_SYMMETRIC: case MYEA_AF_GAUSSIAN_STEPWISE: return y;
    default: return 1.0f;  // linear, linear piece (symmetric), softmax
  }
}

// which arrays af_derive reads: the summation (pre-activation) and / or the value
__host__ __device__ __forceinline__ bool af_derive_reads_summation(uint32_t af) {
  switch (af) {
    case MYEA_AF_TANH: case MYEA_AF_TANH_STEPWISE: case MYEA_AF_SIGMOID: case MYEA_AF_SIGMOID_STEPWISE: case MYEA_AF_THRESHOLD:
    case MYEA_AF_THRESHOLD_SYMMETRIC: case MYEA_AF_GAUSSIAN_STEPWISE: case MYEA_AF_LINEAR: case MYEA_AF_LINEAR_PIECE:
    case MYEA_AF_LINEAR_PIECE_SYMMETRIC: case MYEA_AF_SOFTMAX: return false;
    default: return true;
  }
}
__host__ __device__ __forceinline__ bool af_derive_reads_value(uint32_t af) {
  switch (af) {
    case MYEA_AF_RELU: case MYEA_AF_LEAKY_RELU: case MYEA_AF_PARAMETRIC_RELU: case MYEA_AF_ELLIOT: case MYEA_AF_ELLIOT_SYMMETRIC: case MYEA_AF_SINE:
    case MYEA_AF_SINE_SYMMETRIC: case MYEA_AF_COSINE: case MYEA_AF_COSINE_SYMMETRIC: case MYEA_AF_LINEAR: case MYEA_AF_LINEAR_PIECE:
    case MYEA_AF_LINEAR_PIECE_SYMMETRIC: case MYEA_AF_SOFTMAX: return false;
    default: return true;
  }
}

// ---------------------------------------------------------------------------------------------------------
// Dense contraction  C[M,N] (+)= A[M,K] * B[N,K]^T  with a fused epilogue.
// ---------------------------------------------------------------------------------------------------------
// The reference's sigmoid / tanh of the LSTM gates (Activation_Functions.hpp:40, :45)
__host__ __device__ inline float sigmoid_ref(float x) { return 1.0f / (1.0f + expf(-x)); }
__host__ __device__ inline float tanh_ref(float x) { return 2.0f / (1.0f + expf(-2.0f * x)) - 1.0f; }

struct Epilogue {
  float *C = nullptr;
  long long ldc = 0;
  int accumulate = 0;            // C += acc instead of C = acc
  const float *bias = nullptr;   // [N], added to every row
  const float *addend = nullptr; // [M,N] (pitch ld_addend) added before the activation derivative (skip-connection error)
  long long ld_addend = 0;
  uint32_t deriv_af = 0;         // != 0: result *= f'(pre, y) of this activation
  const float *aux_pre = nullptr;  // [M,N] pre-activation source (may be null when f' only needs y)
  const float *aux_y = nullptr;    // [M,N] activation output
  long long ld_aux = 0;
  const float *col_scale = nullptr;  // pre = aux_pre * col_scale[n] + col_shift[n] when non-null (normalization folded in)
  const float *col_shift = nullptr;
  // Column statistics of the result, emitted by the epilogue so that no separate pass has to re-read it (tensor-core
  // kernels, 16-byte aligned arrays, N a multiple of 32): for every block of 32 output rows, col_stats[0][block][n] and
  // col_stats[1][block][n] (pitch stats_blocks * N between the two) receive
  //   stats_kind 1:  sum of the stored values, sum of their squares           (batch-normalization forward sums)
  //   stats_kind 2:  sum of the stored values d, sum of d * (aux_pre - col_mean[n])   (its backward sums; needs deriv_af)
  int stats_kind = 0;
  float *col_stats = nullptr;
  long long stats_blocks = 0;
  const float *col_mean = nullptr;
  // seg_rows != 0: the output rows come in up to 4 segments of seg_rows rows; row m of the product is row
  // (m mod seg_rows) of the array that starts at C + seg_off[m / seg_rows] (the four gate matrices of an LSTM layer
  // inside the reference's per-block parameter layout: one contraction instead of four)
  long long seg_rows = 0;
  long long seg_off[4] = {0, 0, 0, 0};
};

// A fp32 matrix operand given by strides: element (r, k) at ptr[r * stride_r + k * stride_k]; one of the two
// strides is 1.
struct Operand {
  const float *ptr = nullptr;
  long long rows = 0, k = 0;
  long long stride_r = 0, stride_k = 0;
  const float *lo = nullptr;  // optional second addend with the same strides (value = ptr[..] + lo[..]); FMA engine only
};

// K-major hi / lo panels of one operand, pitch kp floats (a multiple of 32): what the tensor-core kernel reads with TMA.
// `hi`: TF32-rounded values in fp32 containers.  `lo`: the CROSS panel, per 8 K elements 16 bf16 = [lo x8 | hi x8] for the
// left operand (role A) and [hi x8 | lo x8] for the right operand (role B), so that one K = 16 BF16 MMA of an A group with
// a B group yields lo_a*hi_b + hi_a*lo_b.
enum { PANEL_ROLE_A = 0, PANEL_ROLE_B = 1 };
// An MN-major panel set (major == PANEL_MN) describes the operand TRANSPOSED: the arrays are [k][kp] (hi, fp32) and
// [2 * round_up(k, 8)][kp] (cross, bf16; per 8 K rows 16 panel rows, lo rows / hi rows ordered by role), the operand's
// `rows` run along the contiguous axis.  Only the 256 x 256 kernel reads this form; it needs kp to be a multiple of 64.
enum { PANEL_K = 0, PANEL_MN = 1 };
struct Panels {
  float *hi = nullptr, *lo = nullptr;
  long long rows = 0, k = 0, kp = 0;
  int role = PANEL_ROLE_A;
  int major = PANEL_K;
};

struct GemmScratch {   // hi/lo K-major panels of both operands, reused by every contraction of a handle
  float *base = nullptr;
  size_t floats = 0;
};

size_t gemm_scratch_floats(long long M, long long N, long long K);
size_t panel_floats(long long rows, long long k);
Panels panels_at(float *mem, long long rows, long long k, int role);
int gemm_prepare(Context &ctx, const Operand &op, float *mem, Panels *out, int role);
int gemm_prepare_into(Context &ctx, const Operand &op, const Panels &dst, long long row_offset, long long k_offset);
// The same with the source rows landing on every `row_step`-th panel row starting at row_offset (interleaving several
// matrices row by row into one panel set); K-major sources only.
int gemm_prepare_interleaved(Context &ctx, const Operand &op, const Panels &dst, long long row_offset, long long row_step);
int gemm_panels(Context &ctx, const Panels &A, long long a_row0, long long M, const Panels &B, long long b_row0, long long N,
                const Epilogue &epi);
// TMA descriptor of a K-major panel [rows][kp] (hi, or cross seen as 32-bit words): boxes of 32 floats of K x box_rows
// rows, 128-byte swizzle; K ends at round_up(k, 8) and rows at `rows` (the hardware fills the rest of a box with zeros)
bool make_panel_map(CUtensorMap *map, const float *panel, long long rows, long long k, long long kp, int box_rows);
// One pass over a row-major source S[R][C] that serves BOTH readings of it: `as_rows` is the K-major operand
// (rows = R, K = C) and `as_cols` the MN-major operand (rows = C, K = R); they share the hi panel.  Either output may
// be null.  `mem` needs shared_panel_floats(R, C) floats.
size_t shared_panel_floats(long long R, long long C);
int gemm_prepare_shared(Context &ctx, const float *src, long long stride_r, long long R, long long C, float *mem, int role_rows,
                        Panels *as_rows, int role_cols, Panels *as_cols);
// true when a contraction of this shape runs on the 256 x 256 kernel (the only one that takes MN-major operands)
bool gemm_takes_mn_major(const Context &ctx, long long M, long long N);
// The Panels of gemm_prepare_shared's layout in `mem` without writing them (for a producer kernel that writes them itself),
// and what such a producer needs to know: where the three panels lie and which cross-term order each reading wants.
// Only for R and C that are multiples of 8 (no padding rows or columns to clear).
struct PanelSink {
  float *hi = nullptr;            // [R][kp] TF32-rounded values
  float *cross_k = nullptr;       // [R][kp] cross panel of the row reading (null: not wanted)
  uint16_t *cross_mn = nullptr;   // [2 R][kp] bf16 cross panel of the column reading (null: not wanted)
  long long kp = 0;
  int role_k = 0, role_mn = 0;    // PANEL_ROLE_A / _B of the two readings
};
void shared_panel_layout(float *mem, long long R, long long C, int role_rows, Panels *as_rows, int role_cols, Panels *as_cols, PanelSink *sink);
// whether the epilogue of a tensor-core contraction with this description can emit column statistics (stats_kind)
bool epilogue_takes_stats(const Context &ctx, const Epilogue &e, long long N);
// Launches split kernels + the tensor-core kernel (engine 0) or the FP32 FMA kernel (engine 1) on ctx.stream.
int gemm_nt(Context &ctx, const Operand &A, const Operand &B, const Epilogue &epi, const GemmScratch &scratch);
// Optional workspace that lets the 256 x 256 tensor-core kernel split the tiles of a partial last wave along K
// (39 MB per context); without it that kernel computes whole tiles only.
int gemm_splitk_reserve(Context &ctx);
void gemm_splitk_release(Context &ctx);

// ---------------------------------------------------------------------------------------------------------
// Bandwidth-bound kernels (kernels_elementwise.cu, optimizer.cu)
// ---------------------------------------------------------------------------------------------------------
struct NormParams {        // one normalized layer
  uint32_t type = 0;       // MYEA_NORM_*
  float momentum = 0.999f, epsilon = 1e-5f, r_max = 1.f, d_max = 0.f;
  const float *gamma = nullptr, *beta = nullptr;   // in the flat parameter buffer
  float *d_gamma = nullptr, *d_beta = nullptr;     // in the flat derivative buffer
  float *mean = nullptr, *sigma = nullptr, *r = nullptr, *d = nullptr;  // [H] batch statistics of the last forward
  float *mean_avg = nullptr, *sigma_avg = nullptr;                      // [H] running averages
  float *col_scale = nullptr, *col_shift = nullptr;                     // [H] y = z*col_scale + col_shift
  float *partial = nullptr;  // [2][chunks][H] workspace of the column reductions
  int chunks = 0;
};

// Cross-GPU sum of a small device vector, supplied by the communicator when the batch is sharded over `world` ranks.
struct SumHook {
  int world = 1;
  void *user = nullptr;
  int (*all_reduce)(void *user, float *buf, size_t n) = nullptr;
  // split form: `begin` starts the sum on a side stream once everything queued so far has finished, `end` makes the
  // main stream wait for it; work queued on the main stream in between runs beside the exchange
  int (*begin)(void *user, float *buf, size_t n) = nullptr;
  int (*end)(void *user) = nullptr;
};
// something independent of the sums that can be queued while they travel (may be null)
struct OverlapWork {
  int (*run)(void *arg) = nullptr;
  void *arg = nullptr;
};

// z [rows,H] -> batch statistics (training) or running statistics (inference) -> col_scale / col_shift
// fused_chunks > 0: np.partial already holds the column sums of `fused_chunks` row blocks (written by the epilogue of the
// contraction that produced z), no pass over z is made
int norm_forward_stats(Context &ctx, const float *z, long long rows, long long H, const NormParams &np, int training,
                       const SumHook *hook = nullptr, const OverlapWork *meanwhile = nullptr, int fused_chunks = 0);
// out = dropout(f(z*col_scale+col_shift)) ; col_scale null = no normalization. mask: uint8[H] or null; keep_scale = 1/p for inverted dropout
// sink (may be null): the result is also written as operand panels of the contraction that reads it next
bool activation_writes_panels(uint32_t af);
int activation_forward(Context &ctx, const float *z, float *out, long long rows, long long H, uint32_t af,
                       const float *col_scale, const float *col_shift, const uint8_t *mask, float keep_scale, const PanelSink *sink = nullptr);
// in place: d *= f'(z * col_scale + col_shift, y) (col_scale null: the summation itself)
int activation_backward(Context &ctx, float *d, const float *z, const float *y, long long rows, long long H, uint32_t af, const float *col_scale,
                        const float *col_shift);
int softmax_forward(Context &ctx, const float *z, float *out, long long rows, long long H);
// delta_af [rows,H] (error after the activation derivative) -> error before the normalization, plus d_gamma / d_beta
int norm_backward(Context &ctx, const float *z, const float *delta_af, float *delta_out, long long rows, long long H,
                  const NormParams &np, const SumHook *hook = nullptr, int fused_chunks = 0, const PanelSink *sink = nullptr);
// delta = f'(pre,y) * (y - desired); loss / accuracy accumulators (double[2] + uint64) on the device
int output_error(Context &ctx, const float *pre, const float *y, const float *desired, float *delta, long long rows,
                 long long H, uint32_t af, uint32_t loss, uint32_t accuracy, float accuracy_variance, double *d_acc,
                 unsigned long long *d_count);
// out[j] (+)= sum_rows in[r][j]
int column_sum(Context &ctx, const float *in, long long rows, long long H, float *out, int accumulate, float *partial,
               int chunks);
int fill_zero(Context &ctx, float *p, size_t n);

struct OptLaunch {
  uint32_t type = 0;
  float lr_t = 0, beta1 = 0, beta2 = 0, epsilon = 0, weight_decay = 0, lower = 0, upper = 0;
  float gd_lr = 0, momentum = 0;
  int nesterov = 0;
  float rprop_increase = 1.2f, rprop_decrease = 0.5f, rprop_min = 1e-6f, rprop_max = 50.f, rprop_zero = 0.1f;  // iRPROP+
  int rprop_error_is_worse = 0;
  const float *clip_scale = nullptr;  // device float: multiply the gradient by it first (global-norm clip), may be null
};
int optimizer_update(Context &ctx, const OptLaunch &o, float *w, float *g, float *m, float *v, float *vhat,
                     float *prev_delta, const float *mask, size_t n);
// every row of w[rows][cols] whose Euclidean norm is >= max_norm is scaled to norm max_norm (Euclidean_Norm__Loop,
// Neural_Network__Regularization__Max_Norm_Constraints.cpp:48-88)
int row_max_norm(Context &ctx, float *w, long long rows, long long cols, float max_norm);
// the same for the weight runs of `blocks` LSTM blocks whose first parameter is `first` (one direction has `cells` cells)
int lstm_max_norm(Context &ctx, float *params, long long first, long long blocks, long long stride, long long n_in, long long cells,
                  long long cells_per_block, float max_norm);
// d_out[0] = sum g^2 (double)
int sum_squares(Context &ctx, const float *g, size_t n, double *d_out, bool accumulate = false);  // d_out (+)= sum of g^2
// clip_scale[0] = norm >= clip ? clip / norm : 1
int clip_scale_from_norm(Context &ctx, const double *d_sumsq, float clip, float *d_scale);

}  // namespace myea
