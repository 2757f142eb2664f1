// Average and max pooling layers over the units of the layer below (one-dimensional windows).
//
// Reference routines: Forward_Pass__Average_Pooling / __Max_Pooling (Neural_Network__Forward_Pass__OpenMP.cpp, Loop twin
// :4537-4582, :5069-5136), Backward_Pass__Average_Pooling / __Max_Pooling (Neural_Network__Backward_Pass__Loop.cpp:1004-1040,
// :1139-1175), output width from Assign__Post__Layer (Neural_Network__Compile.cpp:250-271).
// Output j reads the positions j * stride + k * dilation - padding, k < kernel, that fall inside the input.  The
// average divides by the kernel size whatever falls outside; the maximum treats a position outside as the value 0 and
// remembers which position won (the first of equals), and its backward pass hands the error to that position alone.
// Both are HBM-bound elementwise passes: 4 bytes read per input element, 4 (+4 for the index) written per output.
#include "net.cuh"

#include <algorithm>

namespace myea {

struct PoolShape {
  long long rows, n_in, n_out, kernel, stride, padding, dilation;
};

__global__ void __launch_bounds__(256) pooling_forward_kernel(const PoolShape s, const float *__restrict__ in, float *__restrict__ out,
                                                              int *__restrict__ winner) {
  const long long total = s.rows * s.n_out;
  const float scale = 1.0f / static_cast<float>(s.kernel);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / s.n_out, j = i - r * s.n_out;
    const float *x = in + r * s.n_in;
    if (winner == nullptr) {
      float sum = 0.f;
      for (long long k = 0; k < s.kernel; ++k) {
        const long long p = j * s.stride + k * s.dilation;
        if (p < s.padding || p >= s.n_in + s.padding) continue;
        sum += x[p - s.padding];
      }
      out[i] = sum * scale;
    } else {
      long long best = 0;
      float top = -3.402823466e+38f;
      for (long long k = 0; k < s.kernel; ++k) {
        const long long p = j * s.stride + k * s.dilation;
        if (p < s.padding || p >= s.n_in + s.padding) {
          if (top < 0.f) { best = p; top = 0.f; }
        } else if (top < x[p - s.padding]) {
          best = p;
          top = x[p - s.padding];
        }
      }
      winner[i] = static_cast<int>(best);
      out[i] = top;
    }
  }
}

// d_in[r][p] = sum over the outputs whose window holds position p of their share of the error: one thread per INPUT
// element gathers (no atomics, and the sum runs in output order as the reference's accumulation does)
__global__ void __launch_bounds__(256) pooling_backward_kernel(const PoolShape s, const float *__restrict__ d_out, const int *__restrict__ winner,
                                                               float *__restrict__ d_in) {
  const long long total = s.rows * s.n_in;
  const float scale = 1.0f / static_cast<float>(s.kernel);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / s.n_in, c = i - r * s.n_in, p = c + s.padding;
    const float *d = d_out + r * s.n_out;
    // outputs j with j * stride <= p <= j * stride + (kernel - 1) * dilation
    const long long reach = (s.kernel - 1) * s.dilation;
    const long long j_lo = p > reach ? (p - reach + s.stride - 1) / s.stride : 0;
    const long long j_hi = (p / s.stride < s.n_out - 1) ? p / s.stride : s.n_out - 1;
    float sum = 0.f;
    for (long long j = j_lo; j <= j_hi; ++j) {
      const long long off = p - j * s.stride;
      if (winner == nullptr) {
        if (s.dilation == 0) { if (off == 0) sum += d[j] * scale * static_cast<float>(s.kernel); }  // every k lands on the same position
        else if (off % s.dilation == 0 && off / s.dilation < s.kernel) sum += d[j] * scale;
      } else if (winner[r * s.n_out + j] == static_cast<int>(p)) {
        sum += d[j];
      }
    }
    d_in[i] = sum;
  }
}

static PoolShape shape_of(const LayerPlan &L, long long rows) {
  PoolShape s;
  s.rows = rows; s.n_in = L.n_in; s.n_out = L.n_out;
  s.kernel = static_cast<long long>(L.desc.unit_parameters[0]); s.stride = static_cast<long long>(L.desc.unit_parameters[1]);
  s.padding = static_cast<long long>(L.desc.unit_parameters[2]); s.dilation = static_cast<long long>(L.desc.unit_parameters[3]);
  return s;
}

static int grid_for(long long total) { return static_cast<int>(std::max<long long>(1, std::min<long long>((total + 255) / 256, 148 * 16))); }

// width of a pooling layer over `n_in` units (Assign__Post__Layer: the average ignores the dilation, the maximum counts it)
long long pooling_output_width(const myea_layer_desc &d, long long n_in) {
  const double kernel = static_cast<double>(d.unit_parameters[0]), stride = static_cast<double>(d.unit_parameters[1]);
  const double padding = static_cast<double>(d.unit_parameters[2]), dilation = static_cast<double>(d.unit_parameters[3]);
  if (stride <= 0.0 || kernel <= 0.0) return 0;
  const double span = d.type_layer == MYEA_LAYER_AVERAGE_POOLING ? static_cast<double>(n_in) + 2.0 * padding - kernel
                                                                  : static_cast<double>(n_in) + 2.0 * padding - dilation * (kernel - 1.0) - 1.0;
  const double q = span / stride + 1.0;
  const double w = d.unit_parameters[4] == 0 ? floor(q) : ceil(q);
  return w < 1.0 ? 0 : static_cast<long long>(w);
}

int pooling_forward(myea_b200_net *net, LayerPlan &L, const float *input, long long rows) {
  Context &ctx = net->ctx;
  ctx.begin(TC_ELEMENTWISE);
  pooling_forward_kernel<<<grid_for(rows * L.n_out), 256, 0, ctx.stream>>>(shape_of(L, rows), input, L.values, L.pool_winner);
  ctx.end(TC_ELEMENTWISE);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// error on the layer's outputs (L.errors) -> error on its inputs
int pooling_backward(myea_b200_net *net, LayerPlan &L, float *d_input, long long rows) {
  Context &ctx = net->ctx;
  ctx.begin(TC_ELEMENTWISE);
  pooling_backward_kernel<<<grid_for(rows * L.n_in), 256, 0, ctx.stream>>>(shape_of(L, rows), L.errors, L.pool_winner, d_input);
  ctx.end(TC_ELEMENTWISE);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

}  // namespace myea
