// One fused parameter update over the flat parameter buffer, the global-norm clip that precedes it and the
// derivative reset that follows it: Update_Parameters__Adam (Neural_Network__Adam.cpp:39-95), AMSGrad
// (Neural_Network__AMSGrad.cpp), AdaBound / AMSBound (Neural_Network__AdaBound.cpp, …AMSBound.cpp), gradient descent,
// momentum and Nesterov (Neural_Network__Gradient_Descent.cpp, …_Momentum.cpp, Neural_Network__Nesterov_Accelerated_Gradient.cpp), iRPROP+
// (Neural_Network__iRPROP_plus.cpp),
// Clip_Gradient / Euclidean_Norm (Neural_Network__Clip_Gradient.cpp:82-94, …Regularization__Max_Norm_Constraints.cpp:48-87).
// Pure HBM streaming: every array is read and written once with 128-bit accesses; the optimizer is a uniform branch.
#include "common.cuh"

#include <algorithm>

namespace myea {

struct OptArrays {
  float *w, *g, *m, *v, *vhat, *prev;
  const float *mask;
};

__device__ __forceinline__ float opt_one(const OptLaunch &o, float w, float g, float &m, float &v, float &vhat, float &prev, float mask) {
  const float decay = (o.weight_decay != 0.f) ? mask * o.weight_decay * w : 0.f;
  switch (o.type) {
    case MYEA_OPT_ADAM: {
      m = o.beta1 * m + (1.f - o.beta1) * g;
      v = o.beta2 * v + (1.f - o.beta2) * g * g;
      return w - (o.lr_t * m / (sqrtf(v) + o.epsilon) + decay);
    }
    case MYEA_OPT_AMSGRAD: {
      m = o.beta1 * m + (1.f - o.beta1) * g;
      v = o.beta2 * v + (1.f - o.beta2) * g * g;
      vhat = fmaxf(vhat, v);
      return w - (o.lr_t * m / (sqrtf(vhat) + o.epsilon) + decay);
    }
    case MYEA_OPT_ADABOUND: {
      m = o.beta1 * m + (1.f - o.beta1) * g;
      v = o.beta2 * v + (1.f - o.beta2) * g * g;
      const float step = fminf(fmaxf(o.lr_t / (sqrtf(v) + o.epsilon), o.lower), o.upper);
      return w - (step * m + decay);
    }
    case MYEA_OPT_AMSBOUND: {
      m = o.beta1 * m + (1.f - o.beta1) * g;
      v = o.beta2 * v + (1.f - o.beta2) * g * g;
      vhat = fmaxf(vhat, v);
      const float step = fminf(fmaxf(o.lr_t / (sqrtf(vhat) + o.epsilon), o.lower), o.upper);
      return w - (step * m + decay);
    }
    case MYEA_OPT_IRPROP_PLUS: {
      // Update_Parameter__iRPROP_plus__Loop (Neural_Network__iRPROP_plus.cpp:30-120).  m: previous derivative,
      // v: previous step (a cleared 0 stands for rprop_delta_zero, Clear_Optimizer, Train.cpp:163-190), prev: previous
      // delta weight.  No decay term: the reference has none on this path.
      if (v == 0.f) v = o.rprop_zero;
      const float same = m * g;
      const float sign = static_cast<float>(0.f < g) - static_cast<float>(g < 0.f);
      if (same > 0.f) {
        v = fminf(v * o.rprop_increase, o.rprop_max);
        prev = -sign * v;
        m = g;
        return w + prev;
      }
      if (same < 0.f) {
        v = fmaxf(v * o.rprop_decrease, o.rprop_min);
        m = 0.f;
        return o.rprop_error_is_worse ? w - prev : w;
      }
      prev = -sign * v;
      m = g;
      return w + prev;
    }
    default: {  // gradient descent family
      if (o.momentum == 0.f) return w - (o.gd_lr * g + decay);
      if (!o.nesterov) {
        // delta = lr*g + momentum*previous delta ; w -= delta
        const float delta = o.gd_lr * g + o.momentum * prev;
        prev = delta;
        return w - (delta + decay);
      }
      // Nesterov exactly as the reference codes it (Neural_Network__Nesterov_Accelerated_Gradient.cpp:48,59):
      // delta = lr*g + momentum*previous delta ; w -= momentum*delta - lr*g
      const float delta = o.gd_lr * g + o.momentum * prev;
      prev = delta;
      return w - (o.momentum * delta - o.gd_lr * g + decay);
    }
  }
}

template <bool HAS_VHAT, bool HAS_PREV>
__global__ void __launch_bounds__(256) optimizer_kernel(const OptLaunch o, const OptArrays a, size_t n) {
  const float scale = o.clip_scale != nullptr ? *o.clip_scale : 1.0f;
  const size_t n4 = n >> 2;
  const bool adam_like = o.type != MYEA_OPT_GD;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float4 w = reinterpret_cast<float4 *>(a.w)[i];
    float4 g = reinterpret_cast<float4 *>(a.g)[i];
    float4 m = make_float4(0, 0, 0, 0), v = m, vh = m, pv = m, mk = make_float4(1, 1, 1, 1);
    if (adam_like) { m = reinterpret_cast<float4 *>(a.m)[i]; v = reinterpret_cast<float4 *>(a.v)[i]; }
    if (HAS_VHAT) vh = reinterpret_cast<float4 *>(a.vhat)[i];
    if (HAS_PREV) pv = reinterpret_cast<float4 *>(a.prev)[i];
    if (o.weight_decay != 0.f && a.mask != nullptr) mk = reinterpret_cast<const float4 *>(a.mask)[i];
    w.x = opt_one(o, w.x, g.x * scale, m.x, v.x, vh.x, pv.x, mk.x);
    w.y = opt_one(o, w.y, g.y * scale, m.y, v.y, vh.y, pv.y, mk.y);
    w.z = opt_one(o, w.z, g.z * scale, m.z, v.z, vh.z, pv.z, mk.z);
    w.w = opt_one(o, w.w, g.w * scale, m.w, v.w, vh.w, pv.w, mk.w);
    reinterpret_cast<float4 *>(a.w)[i] = w;
    reinterpret_cast<float4 *>(a.g)[i] = make_float4(0, 0, 0, 0);
    if (adam_like) { reinterpret_cast<float4 *>(a.m)[i] = m; reinterpret_cast<float4 *>(a.v)[i] = v; }
    if (HAS_VHAT) reinterpret_cast<float4 *>(a.vhat)[i] = vh;
    if (HAS_PREV) reinterpret_cast<float4 *>(a.prev)[i] = pv;
  }
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const size_t i = (n4 << 2) + threadIdx.x;
    float m = adam_like ? a.m[i] : 0.f, v = adam_like ? a.v[i] : 0.f, vh = HAS_VHAT ? a.vhat[i] : 0.f, pv = HAS_PREV ? a.prev[i] : 0.f;
    const float mk = (o.weight_decay != 0.f && a.mask != nullptr) ? a.mask[i] : 1.f;
    a.w[i] = opt_one(o, a.w[i], a.g[i] * scale, m, v, vh, pv, mk);
    a.g[i] = 0.f;
    if (adam_like) { a.m[i] = m; a.v[i] = v; }
    if (HAS_VHAT) a.vhat[i] = vh;
    if (HAS_PREV) a.prev[i] = pv;
  }
}

int optimizer_update(Context &ctx, const OptLaunch &o, float *w, float *g, float *m, float *v, float *vhat, float *prev_delta,
                     const float *mask, size_t n) {
  OptArrays a{w, g, m, v, vhat, prev_delta, mask};
  const bool has_vhat = (o.type == MYEA_OPT_AMSGRAD || o.type == MYEA_OPT_AMSBOUND);
  const bool has_prev = (o.type == MYEA_OPT_GD && o.momentum != 0.f) || o.type == MYEA_OPT_IRPROP_PLUS;
  if ((has_vhat && vhat == nullptr) || (has_prev && prev_delta == nullptr) || (o.type != MYEA_OPT_GD && (m == nullptr || v == nullptr)))
    return MYEA_E_INVALID;
  const int blocks = static_cast<int>(std::max<size_t>(1, std::min<size_t>(((n >> 2) + 255) / 256, 148 * 16)));
  ctx.begin(TC_OPTIMIZER);
  if (has_vhat) optimizer_kernel<true, false><<<blocks, 256, 0, ctx.stream>>>(o, a, n);
  else if (has_prev) optimizer_kernel<false, true><<<blocks, 256, 0, ctx.stream>>>(o, a, n);
  else optimizer_kernel<false, false><<<blocks, 256, 0, ctx.stream>>>(o, a, n);
  ctx.end(TC_OPTIMIZER);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// sum of squares of the whole derivative buffer, double accumulation across blocks
__global__ void __launch_bounds__(256) sum_squares_kernel(const float *__restrict__ g, size_t n, double *out) {
  __shared__ float sh[8];
  float s = 0.f;
  const size_t n4 = n >> 2;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float4 t = reinterpret_cast<const float4 *>(g)[i];
    s += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) { const float t = g[(n4 << 2) + threadIdx.x]; s += t * t; }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < 8; ++w) t += static_cast<double>(sh[w]);
    atomicAdd(out, t);
  }
}

int sum_squares(Context &ctx, const float *g, size_t n, double *d_out, bool accumulate) {
  ctx.begin(TC_OPTIMIZER);
  if (!accumulate) cudaMemsetAsync(d_out, 0, sizeof(double), ctx.stream);
  const int blocks = static_cast<int>(std::max<size_t>(1, std::min<size_t>(((n >> 2) + 255) / 256, 148 * 8)));
  sum_squares_kernel<<<blocks, 256, 0, ctx.stream>>>(g, n, d_out);
  ctx.end(TC_OPTIMIZER);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

__global__ void clip_scale_kernel(const double *sumsq, float clip, float *scale) {
  const float norm = sqrtf(static_cast<float>(*sumsq));
  *scale = norm >= clip ? clip / norm : 1.0f;
}

int clip_scale_from_norm(Context &ctx, const double *d_sumsq, float clip, float *d_scale) {
  clip_scale_kernel<<<1, 1, 0, ctx.stream>>>(d_sumsq, clip, d_scale);
  ctx.launches += 1;
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// one block per row: sum of squares (fp32 partials, tree), then the scale
__global__ void __launch_bounds__(256) row_max_norm_kernel(float *__restrict__ w, long long cols, float max_norm) {
  __shared__ float sh[256];
  float *row = w + static_cast<long long>(blockIdx.x) * cols;
  float acc = 0.f;
  for (long long j = threadIdx.x; j < cols; j += blockDim.x) acc = fmaf(row[j], row[j], acc);
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s];
    __syncthreads();
  }
  const float norm = sqrtf(sh[0]);
  if (norm >= max_norm) {
    const float scale = max_norm / norm;
    for (long long j = threadIdx.x; j < cols; j += blockDim.x) row[j] *= scale;
  }
}

// LSTM blocks (Update_Weight_Regularization__Max_Norm_Constraints__LSTMs, …Max_Norm_Constraints.cpp:167-310): every run
// of weights is a vector of its own - per cell the input and the recurrent weights of the cell input, per block those
// of the three gates, and the three peephole runs.  One thread block per run: grid (blocks of the layer, 2 cpb + 9).
// The reference tests `first_index > start` with start = 0: a run that begins at parameter 0 is passed over.
__global__ void __launch_bounds__(256) lstm_max_norm_kernel(float *__restrict__ params, long long first, long long stride, long long I, long long C,
                                                            long long cpb, float max_norm) {
  __shared__ float sh[256];
  const long long s = blockIdx.y, base = first + static_cast<long long>(blockIdx.x) * stride;
  long long at, len;
  if (s < 2 * cpb) {
    at = base + (s >> 1) * (I + C) + ((s & 1) ? I : 0);
    len = (s & 1) ? C : I;
  } else {
    const long long g = s - 2 * cpb, g0 = base + cpb * (I + C);
    if (g < 3) { at = g0 + g * I; len = I; }
    else if (g < 6) { at = g0 + 3 * I + (g - 3) * C; len = C; }
    else { at = g0 + 3 * I + 3 * C + (g - 6) * cpb; len = cpb; }
  }
  if (at == 0) return;
  float *v = params + at;
  float acc = 0.f;
  for (long long j = threadIdx.x; j < len; j += blockDim.x) acc = fmaf(v[j], v[j], acc);
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (int h = 128; h > 0; h >>= 1) {
    if (threadIdx.x < h) sh[threadIdx.x] += sh[threadIdx.x + h];
    __syncthreads();
  }
  const float norm = sqrtf(sh[0]);
  if (norm >= max_norm) {
    const float scale = max_norm / norm;
    for (long long j = threadIdx.x; j < len; j += blockDim.x) v[j] *= scale;
  }
}

int lstm_max_norm(Context &ctx, float *params, long long first, long long blocks, long long stride, long long n_in, long long cells,
                  long long cells_per_block, float max_norm) {
  if (blocks <= 0) return MYEA_OK;
  ctx.begin(TC_OPTIMIZER);
  lstm_max_norm_kernel<<<dim3(static_cast<unsigned>(blocks), static_cast<unsigned>(2 * cells_per_block + 9)), 256, 0, ctx.stream>>>(
      params, first, stride, n_in, cells, cells_per_block, max_norm);
  ctx.end(TC_OPTIMIZER);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

int row_max_norm(Context &ctx, float *w, long long rows, long long cols, float max_norm) {
  if (rows <= 0 || cols <= 0) return MYEA_OK;
  ctx.begin(TC_OPTIMIZER);
  row_max_norm_kernel<<<static_cast<unsigned>(rows), 256, 0, ctx.stream>>>(w, cols, max_norm);
  ctx.end(TC_OPTIMIZER);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

}  // namespace myea
