// Residual blocks of fully connected layers with ShakeDrop, in the reference's pre-activation order.
//
// Reference (Source_Files/Neural_Network/): Forward_Pass__Residual / __Residual__Layer / __Residual__FC
// (Neural_Network__Forward_Pass__OpenMP.cpp:3930-4500), Forward_Pass__Dropout__ShakeDrop (:5021-5056),
// Forward_Pass__Zero_Padded_Identity (:5158-5236); Backward_Pass__Residual__Block / __Residual__FC
// (Neural_Network__Backward_Pass__OpenMP.cpp:351-534), Backward_Pass__Gradient__Residual__FC (:822-950),
// Backward_Pass__Dropout__ShakeDrop (:1009-1042).
//
// A block of depth D behind residual layer R, fed by x (the output of the layer before R):
//   layer 1 (block input):  s1 = W1 x (+ b1)                      no activation in front of the first layer
//   layer k > 1:            v_k = dropout(f_k(norm_k(s_{k-1})))   normalization and activation act on the layer's INPUT
//                           s_k = W_k v_k (+ b_k when the layer is not normalized)
//   block output:           r = x + ShakeDrop(s_D)                training: rows whose mask is set are multiplied by
//                                                                 alpha[row, :]; inference: everything times (1 - p)
// A block layer's `summations` are its outputs, its `values` hold v_k (what Update_Derivative_Weight multiplies the
// error with).  Backward: the error on r passes unchanged to x (skip connection) and, multiplied by beta[row, :] on the
// masked rows, to s_D; layer k > 1 sends W_k^T delta_k through f_k' and the normalization backward to s_{k-1}; the layer
// feeding the block receives skip error + W_1^T delta_1, with its own activation derivative fused when it is a fully
// connected layer.  ShakeDrop's alpha, beta and row mask are inputs (the reference draws them on the fly).
#include "net.cuh"

#include <algorithm>

namespace myea {

int fc_finish_backward(myea_b200_net *net, LayerPlan &L, long long rows);

#define RRC(expr) do { int rc__ = (expr); if (rc__ != MYEA_OK) return rc__; } while (0)

// out = x + s * (row masked ? coef[row, :] : 1) * scale      (forward, coef = alpha)
// out = d * (row masked ? coef[row, :] : 1)                  (backward, x == nullptr, coef = beta)
template <int VEC>
__global__ void __launch_bounds__(256) shakedrop_kernel(const float *__restrict__ x, const float *__restrict__ s, float *__restrict__ out,
                                                        const uint8_t *__restrict__ mask, const float *__restrict__ coef, float scale,
                                                        long long rows, long long H) {
  const long long hv = H / VEC, total = rows * hv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / hv, c = (i - r * hv) * VEC;
    const bool m = mask != nullptr && mask[r] != 0;
    float sv[VEC], xv[VEC], cv[VEC];
    if (VEC == 4) {
      const float4 t = *reinterpret_cast<const float4 *>(s + r * H + c);
      sv[0] = t.x; sv[1] = t.y; sv[2] = t.z; sv[3] = t.w;
      if (x != nullptr) { const float4 u = *reinterpret_cast<const float4 *>(x + r * H + c); xv[0] = u.x; xv[1] = u.y; xv[2] = u.z; xv[3] = u.w; }
      if (m) { const float4 w = *reinterpret_cast<const float4 *>(coef + r * H + c); cv[0] = w.x; cv[1] = w.y; cv[2] = w.z; cv[3] = w.w; }
    } else {
      sv[0] = s[r * H + c];
      if (x != nullptr) xv[0] = x[r * H + c];
      if (m) cv[0] = coef[r * H + c];
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float v = m ? sv[k] * cv[k] : sv[k];
      if (scale != 1.0f) v *= scale;
      sv[k] = x != nullptr ? xv[k] + v : v;
    }
    if (VEC == 4) *reinterpret_cast<float4 *>(out + r * H + c) = make_float4(sv[0], sv[1], sv[2], sv[3]);
    else out[r * H + c] = sv[0];
  }
}

// The same with a block whose output is narrower or wider than its input (zero-padded identity,
// Forward_Pass__Zero_Padded_Identity, Neural_Network__Forward_Pass__OpenMP.cpp:5158-5236): the result has
// R = max(A, W) columns; the narrower of the two addends sits `pad` columns in.
//   forward:  out[r, c] = x[r, c - oa] (inside [0, A)) + s[r, c - os] * (masked row ? coef[r, c - os] : 1) * scale (inside [0, W))
__global__ void __launch_bounds__(256) shakedrop_pad_forward_kernel(const float *__restrict__ x, long long A, long long oa, const float *__restrict__ s,
                                                                    long long W, long long os, float *__restrict__ out, long long R,
                                                                    const uint8_t *__restrict__ mask, const float *__restrict__ coef, float scale,
                                                                    long long rows) {
  const long long total = rows * R;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / R, c = i - r * R;
    float v = 0.f;
    const long long ca = c - oa, cs = c - os;
    if (cs >= 0 && cs < W) {
      float t = s[r * W + cs];
      if (mask != nullptr && mask[r] != 0) t *= coef[r * R + cs];
      if (scale != 1.0f) t *= scale;
      v = t;
    }
    if (ca >= 0 && ca < A) v = x[r * A + ca] + v;
    out[i] = v;
  }
}
//   backward (Backward_Pass__Residual, …Backward_Pass__OpenMP.cpp:1155-1215, then the ShakeDrop factor):
//   out[r, c] = d[r, c + os] * (masked row ? coef[r, c] : 1)        for the W columns of the block's last layer
__global__ void __launch_bounds__(256) shakedrop_pad_backward_kernel(const float *__restrict__ d, long long R, long long os, float *__restrict__ out,
                                                                     long long W, const uint8_t *__restrict__ mask, const float *__restrict__ coef,
                                                                     long long rows) {
  const long long total = rows * W;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / W, c = i - r * W;
    float v = d[r * R + c + os];
    if (mask != nullptr && mask[r] != 0) v *= coef[r * R + c];
    out[i] = v;
  }
}

static int launch_shakedrop(Context &ctx, const float *x, const float *s, float *out, const uint8_t *mask, const float *coef, float scale,
                            long long rows, long long H) {
  ctx.begin(TC_ELEMENTWISE);
  const bool vec4 = (H % 4 == 0);
  const long long total = rows * (vec4 ? H / 4 : H);
  const int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>((total + 255) / 256, 148 * 16)));
  if (vec4) shakedrop_kernel<4><<<blocks, 256, 0, ctx.stream>>>(x, s, out, mask, coef, scale, rows, H);
  else shakedrop_kernel<1><<<blocks, 256, 0, ctx.stream>>>(x, s, out, mask, coef, scale, rows, H);
  ctx.end(TC_ELEMENTWISE);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// columns the narrower addend of a zero-padded identity sits in (Assign__Post__Layer, Neural_Network__Compile.cpp:272-277)
static long long residual_padding(long long A, long long W) { return ((A > W ? A - W : W - A) + 1) / 2; }

int residual_check(myea_b200_net *net, int r) {
  LayerPlan &R = net->layers[r];
  if (net->T != 1) { net->ctx.error = "residual blocks in recurrent networks are not built"; return MYEA_E_UNSUPPORTED; }
  for (int k = 1; k <= R.block_depth; ++k) {
    const LayerPlan &L = net->layers[r + k];
    if (L.has_norm && (k == 1 || L.n_in != L.n_out)) { net->ctx.error = "normalization on the first layer of a block, or on a block layer whose input and output widths differ, is not built"; return MYEA_E_UNSUPPORTED; }
    if (L.mask_bernoulli != nullptr && L.n_in != L.n_out) { net->ctx.error = "dropout on a block layer whose input and output widths differ is not built"; return MYEA_E_UNSUPPORTED; }
    if (L.desc.type_activation_function == MYEA_AF_SOFTMAX) { net->ctx.error = "softmax inside a block"; return MYEA_E_INVALID; }
  }
  return MYEA_OK;
}

// input of block layer k's contraction (what its weight derivative multiplies the error with)
const float *residual_fc_input(myea_b200_net *net, int r, int k) {
  return k == 1 ? net->layers[net->layers[r].input_layer].values : net->layers[r + k].values;
}

int residual_forward(myea_b200_net *net, int r) {
  LayerPlan &R = net->layers[r];
  RRC(residual_check(net, r));
  Context &ctx = net->ctx;
  const long long rows = net->pitch();
  const float *x = net->layers[R.input_layer].values;
  for (int k = 1; k <= R.block_depth; ++k) {
    LayerPlan &L = net->layers[r + k];
    const float *in = x;
    if (k > 1) {
      const float *prev = net->layers[r + k - 1].summations;
      const float *cs = nullptr, *ch = nullptr;
      if (L.has_norm) {
        RRC(norm_forward_stats(ctx, prev, rows, L.n_in, L.norm, net->training ? 1 : 0, &net->hook));
        cs = L.norm.col_scale;
        ch = L.norm.col_shift;
      }
      const uint8_t *mask = (net->training && L.mask_bernoulli != nullptr) ? L.mask_bernoulli : nullptr;
      const float scale = net->training ? (mask != nullptr ? L.keep_scale : 1.f) : L.infer_scale;
      RRC(activation_forward(ctx, prev, L.values, rows, L.n_in, L.desc.type_activation_function, cs, ch, mask, scale));
      in = L.values;
    }
    Epilogue e;
    e.C = L.summations;
    e.ldc = L.n_out;
    e.bias = L.use_bias ? net->params + L.idx.first_bias_connection_index : nullptr;
    RRC(fc_product_forward(net, L, in, rows, e));
  }
  const LayerPlan &last = net->layers[r + R.block_depth];
  const bool shake = R.desc.type_dropout == MYEA_DROPOUT_SHAKEDROP;
  const uint8_t *mask = (shake && net->training) ? R.shake_mask : nullptr;
  const float scale = (shake && !net->training) ? 1.0f - R.desc.dropout_values[0] : 1.0f;
  // what the block adds to the shortcut: its last layer's output, normalized first when the residual layer itself
  // carries a normalization (Forward_Pass__Residual, …Forward_Pass__OpenMP.cpp:3861-3998)
  const float *s = last.summations;
  const long long A = R.n_in, W = last.n_out;
  if (R.has_norm) {
    RRC(norm_forward_stats(ctx, last.summations, rows, W, R.norm, net->training ? 1 : 0, &net->hook));
    RRC(activation_forward(ctx, last.summations, R.summations, rows, W, MYEA_AF_LINEAR, R.norm.col_scale, R.norm.col_shift, nullptr, 1.f));
    s = R.summations;
  }
  if (A == W) return launch_shakedrop(ctx, x, s, R.values, mask, R.shake_alpha, scale, rows, R.n_out);
  const long long pad = residual_padding(A, W);
  ctx.begin(TC_ELEMENTWISE);
  const long long total = rows * R.n_out;
  const int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>((total + 255) / 256, 148 * 16)));
  shakedrop_pad_forward_kernel<<<blocks, 256, 0, ctx.stream>>>(x, A, A < W ? pad : 0, s, W, W < A ? pad : 0, R.values, R.n_out, mask, R.shake_alpha, scale, rows);
  ctx.end(TC_ELEMENTWISE);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// R.deriv holds the error on the block's output.  Leaves every block layer's `errors` final and writes the complete
// error of the layer feeding the block (its `deriv`, then its own normalization backward when it is fully connected).
int residual_backward(myea_b200_net *net, int r) {
  LayerPlan &R = net->layers[r];
  Context &ctx = net->ctx;
  const long long rows = net->pitch();
  LayerPlan &last = net->layers[r + R.block_depth];
  const bool shake = R.desc.type_dropout == MYEA_DROPOUT_SHAKEDROP;
  // error on the last layer's output: the block error (its W columns out of the R of the block output), times beta on
  // the masked rows, then through the residual layer's own normalization when it has one
  // (Backward_Pass__Residual__Block, …Backward_Pass__OpenMP.cpp:351-452)
  {
    const long long A = R.n_in, W = last.n_out;
    float *dst = R.has_norm ? R.summations : last.errors;  // R.summations: the normalized copy is not needed any more
    if (A == W) {
      RRC(launch_shakedrop(ctx, nullptr, R.deriv, dst, shake ? R.shake_mask : nullptr, R.shake_beta, 1.0f, rows, R.n_out));
    } else {
      ctx.begin(TC_ELEMENTWISE);
      const long long total = rows * W;
      const int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>((total + 255) / 256, 148 * 16)));
      shakedrop_pad_backward_kernel<<<blocks, 256, 0, ctx.stream>>>(R.deriv, R.n_out, W < A ? residual_padding(A, W) : 0, dst, W, shake ? R.shake_mask : nullptr,
                                                                    R.shake_beta, rows);
      ctx.end(TC_ELEMENTWISE);
    }
    if (R.has_norm) RRC(norm_backward(ctx, last.summations, dst, last.errors, rows, W, R.norm, &net->hook));
  }
  for (int k = R.block_depth; k > 1; --k) {
    LayerPlan &L = net->layers[r + k];
    LayerPlan &below = net->layers[r + k - 1];
    Epilogue e;
    e.C = L.has_norm ? L.deriv : below.errors;  // without normalization the result IS the error on the layer below's output
    e.ldc = L.n_in;
    e.deriv_af = L.desc.type_activation_function;
    e.aux_pre = below.summations;
    e.aux_y = L.values;
    e.ld_aux = L.n_in;
    if (L.has_norm) { e.col_scale = L.norm.col_scale; e.col_shift = L.norm.col_shift; }
    RRC(fc_product_backward(net, L, rows, e));
    if (L.has_norm) RRC(norm_backward(ctx, below.summations, L.deriv, below.errors, rows, L.n_in, L.norm, &net->hook));
  }
  // the layer feeding the block: skip error + W_1^T delta_1, then its own activation derivative / normalization
  LayerPlan &first = net->layers[r + 1];
  LayerPlan &F = net->layers[R.input_layer];
  if (R.input_layer < 1) return MYEA_OK;  // the block reads the network input: nothing to propagate to
  Epilogue e;
  e.C = F.deriv;
  e.ldc = first.n_in;
  // the skip connection: the A columns of the block error that lie over the shortcut
  e.addend = R.deriv + (R.n_in < R.n_out ? residual_padding(R.n_in, R.n_out) : 0);
  e.ld_addend = R.n_out;
  if (F.type == MYEA_LAYER_FULLY_CONNECTED) {
    e.deriv_af = F.desc.type_activation_function;
    e.aux_pre = F.summations;
    e.aux_y = F.values;
    e.ld_aux = F.n_out;
    if (F.has_norm) { e.col_scale = F.norm.col_scale; e.col_shift = F.norm.col_shift; }
  } else if (F.type != MYEA_LAYER_RESIDUAL) {
    net->ctx.error = "a residual block fed by an LSTM layer is not built";
    return MYEA_E_UNSUPPORTED;
  }
  RRC(fc_product_backward(net, first, rows, e));
  if (F.type == MYEA_LAYER_FULLY_CONNECTED) RRC(fc_finish_backward(net, F, rows));
  return MYEA_OK;
}

}  // namespace myea
