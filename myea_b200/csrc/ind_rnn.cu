// Independently recurrent fully connected layers (Ind-RNN): every unit sees its own previous output through one
// recurrent weight,   pre_t = z_t + u * y_{t-1},   y_t = f(pre_t)   (z_t: the layer's summation, normalized if it is).
//
// Reference routines: Forward_Pass__FC_Ind_RNN (Neural_Network__Recurrent_Forward_Pass__OpenMP.cpp, Loop twin :813-860),
// Backward_Pass__FC__DF_Ind_RNN (Neural_Network__Backward_Pass__Loop.cpp:1296-1372): with D_t the error arriving on y_t,
//   dAF_t = f'(pre_t, y_t) * (D_t + u * dAF_{t+1}),
// and Update_Derivative_Weight__FC_Ind_RNN (Neural_Network__Recurrent_Update_Derivative_Weight__Loop.cpp:461-):
//   du += sum over t >= 1 and rows of dAF_t * y_{t-1}.
// The weights' contraction over all time steps stays one GEMM; the recurrence is an elementwise kernel per time step
// (4-5 arrays of [B, units] each: HBM-bound, launch-latency-bound for small layers).
#include "net.cuh"

#include <algorithm>

namespace myea {

// one time step forward: pre = z * col_scale + col_shift + u * y_prev ; y = f(pre) (* mask, * keep_scale)
__global__ void __launch_bounds__(256) ind_rnn_forward_kernel(const float *__restrict__ z, const float *__restrict__ y_prev, const float *__restrict__ u,
                                                              float *__restrict__ pre, float *__restrict__ y, long long rows, long long H, uint32_t af,
                                                              const float *__restrict__ col_scale, const float *__restrict__ col_shift,
                                                              const uint8_t *__restrict__ mask, float keep_scale) {
  const long long total = rows * H;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long c = i % H;
    float p = col_scale != nullptr ? fmaf(z[i], col_scale[c], col_shift[c]) : z[i];
    if (y_prev != nullptr) p += u[c] * y_prev[i];
    pre[i] = p;
    float v = af_fire(af, p);
    if (keep_scale != 1.0f) v *= keep_scale;
    if (mask != nullptr && mask[c] == 0) v = 0.f;
    y[i] = v;
  }
}

// one time step backward, in place on d (D_t in, dAF_t out): d = f'(pre, y) * (d + u * d_next)
__global__ void __launch_bounds__(256) ind_rnn_backward_kernel(float *__restrict__ d, const float *__restrict__ d_next, const float *__restrict__ u,
                                                               const float *__restrict__ pre, const float *__restrict__ y, long long rows, long long H,
                                                               uint32_t af) {
  const long long total = rows * H;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float f = af_derive(af, pre[i], y[i]);
    // the reference's order of operations: D * f' first, then + u * f' * dAF_next
    float v = d[i] * f;
    if (d_next != nullptr) v += u[i % H] * f * d_next[i];
    d[i] = v;
  }
}

// out[r][c] = d[r + shift][c] * y[r][c] for the rows that have a successor step (`shift` = rows of one time step)
__global__ void __launch_bounds__(256) ind_rnn_products_kernel(const float *__restrict__ d, const float *__restrict__ y, long long rows, long long H,
                                                               long long shift, float *__restrict__ out) {
  const long long total = rows * H;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = d[i + shift * H] * y[i];
}

__global__ void __launch_bounds__(256) clamp_kernel(float *__restrict__ w, long long n, float lo, float hi) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < n) w[i] = w[i] < lo ? lo : (w[i] > hi ? hi : w[i]);
}

static int grid_for(long long total) { return static_cast<int>(std::max<long long>(1, std::min<long long>((total + 255) / 256, 148 * 16))); }

int ind_rnn_forward_step(Context &ctx, const float *z, const float *y_prev, const float *u, float *pre, float *y, long long rows, long long H, uint32_t af,
                         const float *col_scale, const float *col_shift, const uint8_t *mask, float keep_scale) {
  if (rows <= 0) return MYEA_OK;
  ctx.begin(TC_RECURRENT);
  ind_rnn_forward_kernel<<<grid_for(rows * H), 256, 0, ctx.stream>>>(z, y_prev, u, pre, y, rows, H, af, col_scale, col_shift, mask, keep_scale);
  ctx.end(TC_RECURRENT);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

int ind_rnn_backward_step(Context &ctx, float *d, const float *d_next, const float *u, const float *pre, const float *y, long long rows, long long H,
                          uint32_t af) {
  if (rows <= 0) return MYEA_OK;
  ctx.begin(TC_RECURRENT);
  ind_rnn_backward_kernel<<<grid_for(rows * H), 256, 0, ctx.stream>>>(d, d_next, u, pre, y, rows, H, af);
  ctx.end(TC_RECURRENT);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// du[c] += sum over the first `rows` rows of d[r + shift][c] * y[r][c]; `scratch`: rows * H floats
int ind_rnn_recurrent_derivative(Context &ctx, const float *d, const float *y, long long rows, long long H, long long shift, float *scratch, float *du,
                                 float *partial, int chunks) {
  if (rows <= 0) return MYEA_OK;
  ctx.begin(TC_RECURRENT);
  ind_rnn_products_kernel<<<grid_for(rows * H), 256, 0, ctx.stream>>>(d, y, rows, H, shift, scratch);
  ctx.end(TC_RECURRENT);
  if (cudaGetLastError() != cudaSuccess) return MYEA_E_CUDA;
  return column_sum(ctx, scratch, rows, H, du, 1, partial, chunks);
}

// Default bound of an independently recurrent layer's recurrent weights
// (Compute__Regularization__Constraint_Recurrent_Weight__Default, …Constraint_Recurrent_Weight.cpp:43-80): +-(MAG / c)^(1/T),
// MAG = clip(clip_gradient, 2, 10), c = 0.9^(T/10) for symmetric activation functions and 1 for the others
float ind_rnn_weight_bound(float clip_gradient, uint32_t type_activation_function, long long T) {
  const float cg = clip_gradient > 0.f ? clip_gradient : 1.f;
  const float mag = cg < 2.f ? 2.f : (cg > 10.f ? 10.f : cg);
  const float t = static_cast<float>(T);
  bool symmetric = false;
  switch (type_activation_function) {
    case MYEA_AF_COSINE_SYMMETRIC: case MYEA_AF_ELLIOT_SYMMETRIC: case MYEA_AF_GAUSSIAN_SYMMETRIC: case MYEA_AF_LINEAR_PIECE_SYMMETRIC:
    case MYEA_AF_SINE_SYMMETRIC: case MYEA_AF_TANH: case MYEA_AF_TANH_STEPWISE: case MYEA_AF_THRESHOLD_SYMMETRIC: symmetric = true; break;
    default: break;
  }
  return symmetric ? powf(mag / powf(0.9f, t / 10.f), 1.f / t) : powf(mag, 1.f / t);
}

// Update_Weight_Regularization__Constraint_Recurrent_Weight__FC_Ind_RNN (:317-334): w = clip(w, -bound, bound)
int ind_rnn_clamp(Context &ctx, float *w, long long n, float bound) {
  if (n <= 0) return MYEA_OK;
  ctx.begin(TC_OPTIMIZER);
  clamp_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, ctx.stream>>>(w, n, -bound, bound);
  ctx.end(TC_OPTIMIZER);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

}  // namespace myea
