// C ABI of the training step: network construction (index map + device buffers) and the five step functions,
// one per member function of the reference's `class Neural_Network` that its training loop calls
// (Dataset.cpp:637-691: Forward_Pass, Compute__Error, Backward_Pass, Update_Derivative_Weight; :7654-7690 Update_Parameter).
#include "net.cuh"

#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <new>

using namespace myea;

namespace myea {
// lstm.cu
int lstm_create(myea_b200_net *net, LayerPlan &L);
void lstm_destroy(LayerPlan &L);
int lstm_forward(myea_b200_net *net, LayerPlan &L, const float *input, long long n_in);
int lstm_backward(myea_b200_net *net, LayerPlan &L);
int lstm_backward_to_input(myea_b200_net *net, LayerPlan &L, float *prev_deriv, const LayerPlan &prev, const Epilogue *finish = nullptr);
int lstm_update_derivative_weight(myea_b200_net *net, LayerPlan &L, const float *input, long long n_in);
int lstm_set_zoneout(myea_b200_net *net, LayerPlan &L, const uint8_t *state, const uint8_t *output, uint64_t count);
float *lstm_output_errors(LayerPlan &L);
// residual.cu
int residual_forward(myea_b200_net *net, int layer);
size_t comm_bucket_count(const myea_b200_net *net);
int comm_bucket_wait(myea_b200_net *net, size_t i, size_t *offset, size_t *n, size_t *slice_offset, size_t *slice_n);
int comm_bucket_gather(myea_b200_net *net, size_t i);
int comm_gather_join(myea_b200_net *net);
int comm_wait_gathers(myea_b200_net *net, size_t offset, size_t n);
void comm_set_scatter(myea_b200_net *net, bool on);
bool comm_any_scattered(const myea_b200_net *net);
int comm_gather_state(myea_b200_net *net, float *buf);
int comm_unscatter(myea_b200_net *net);
void comm_buckets_done(myea_b200_net *net);
int residual_backward(myea_b200_net *net, int layer);
const float *residual_fc_input(myea_b200_net *net, int r, int k);
// comm.cu
int comm_all_reduce_sum(myea_b200_net *net, float *buf, size_t n);
int comm_all_reduce_sum_f64(myea_b200_net *net, double *buf, size_t n);
int comm_reduce_bucket_async(myea_b200_net *net, size_t offset, size_t n);
int comm_join(myea_b200_net *net);
int comm_world(const myea_b200_net *net);
int comm_rank(const myea_b200_net *net);
void comm_destroy(myea_b200_net *net);
}  // namespace myea

#define CK(expr)                                                              \
  do {                                                                        \
    cudaError_t e__ = (expr);                                                 \
    if (e__ != cudaSuccess) {                                                 \
      net->ctx.error = std::string(#expr) + ": " + cudaGetErrorString(e__);   \
      return MYEA_E_CUDA;                                                     \
    }                                                                         \
  } while (0)
#define RC(expr)                 \
  do {                           \
    int rc__ = (expr);           \
    if (rc__ != MYEA_OK) return rc__; \
  } while (0)

static int fail(myea_b200_net *net, int code, const char *msg) {
  net->ctx.error = msg;
  return code;
}

static bool layer_in_block(const myea_b200_net *net, int l, int *block_layer) {
  for (int r = 1; r < static_cast<int>(net->layers.size()); ++r)
    if (net->layers[r].type == MYEA_LAYER_RESIDUAL && l > r && l <= r + net->layers[r].block_depth) {
      if (block_layer) *block_layer = r;
      return true;
    }
  return false;
}

template <typename T>
static int dev_alloc(myea_b200_net *net, T **p, size_t count, bool zero = true) {
  void *q = nullptr;
  const size_t bytes = std::max<size_t>(count, 1) * sizeof(T);
  if (cudaMalloc(&q, bytes) != cudaSuccess) {
    net->ctx.error = "cudaMalloc failed";
    return MYEA_E_CUDA;
  }
  net->allocations.push_back(q);
  if (zero && cudaMemsetAsync(q, 0, bytes, net->ctx.stream) != cudaSuccess) return MYEA_E_CUDA;
  *p = static_cast<T *>(q);
  return MYEA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Index map: Compile (Neural_Network__Compile.cpp:426-785) -> Prepare__Connections__FC/LSTM, Prepare__Bias__FC/LSTM
// (Neural_Network__Prepare_Connections.cpp:20-252); normalized-unit slots as Allocate__Normalized_Unit lays them out
// (Neural_Network__Allocate.cpp:2378-2460): once ANY layer is normalized, gamma for every unit of every layer (input,
// residual and output layers included) is appended after the biases, then beta for every unit.
// ---------------------------------------------------------------------------------------------------------
int myea::build_index_map(myea_b200_net *net) {
  const myea_net_desc &d = net->desc;
  const uint32_t n = d.number_layers;
  net->layers.assign(n, LayerPlan());
  // widths
  for (uint32_t l = 0; l < n; ++l) {
    LayerPlan &L = net->layers[l];
    L.desc = d.layers[l];
    L.type = d.layers[l].type_layer;
    memset(&L.idx, 0, sizeof(L.idx));
    switch (L.type) {
      case MYEA_LAYER_FC_INDEPENDENTLY_RECURRENT:  // a fully connected layer with one recurrent weight per unit on top
        L.type = MYEA_LAYER_FULLY_CONNECTED;
        L.ind_rnn = true;
        L.n_out = static_cast<long long>(d.layers[l].unit_parameters[0]);
        if (l == 0 || l + 1 == n) return fail(net, MYEA_E_INVALID, "an independently recurrent layer is a hidden layer");
        break;
      case MYEA_LAYER_FULLY_CONNECTED: L.n_out = static_cast<long long>(d.layers[l].unit_parameters[0]); break;
      case MYEA_LAYER_LSTM: {
        const long long blocks = static_cast<long long>(d.layers[l].unit_parameters[0]);
        const long long cpb = std::max<long long>(1, static_cast<long long>(d.layers[l].unit_parameters[1]));
        // a bidirectional layer outputs [forward | backward] side by side (the reference keeps number_outputs at the
        // one-direction width and overlaps the two directions' buffers, which is not a usable definition)
        L.n_out = blocks * cpb * (d.layers[l].use_bidirectional ? 2 : 1);
        break;
      }
      case MYEA_LAYER_RESIDUAL: L.block_depth = static_cast<int>(d.layers[l].unit_parameters[0]); break;
      case MYEA_LAYER_AVERAGE_POOLING:
      case MYEA_LAYER_MAX_POOLING:
        // a window over the units of the layer before, which has to have a width of its own already
        if (l == 0 || net->layers[l - 1].type == MYEA_LAYER_RESIDUAL) return fail(net, MYEA_E_UNSUPPORTED, "a pooling layer next to a residual block is not built");
        if (d.layers[l].type_dropout != MYEA_DROPOUT_NONE || d.layers[l].type_normalization != MYEA_NORM_NONE)
          return fail(net, MYEA_E_INVALID, "pooling layers take neither dropout nor normalization");
        L.n_out = pooling_output_width(d.layers[l], net->layers[l - 1].n_out);
        break;
      default: return fail(net, MYEA_E_UNSUPPORTED, "layer type not built (fully connected, LSTM, residual, average / max pooling)");
    }
    if (L.type != MYEA_LAYER_RESIDUAL && L.n_out <= 0) return fail(net, MYEA_E_INVALID, "layer with zero units");
  }
  if (net->layers[0].type != MYEA_LAYER_FULLY_CONNECTED || net->layers[n - 1].type != MYEA_LAYER_FULLY_CONNECTED)
    return fail(net, MYEA_E_INVALID, "input and output layers must be fully connected");
  // a residual layer's width is the width of the last layer of its block (Assign__Post__Layers, Compile.cpp:222-424)
  for (uint32_t l = 1; l < n; ++l) {
    LayerPlan &L = net->layers[l];
    if (L.type == MYEA_LAYER_RESIDUAL) {
      if (L.block_depth < 1 || l + L.block_depth >= n) return fail(net, MYEA_E_INVALID, "residual block runs past the output layer");
      for (int k = 1; k <= L.block_depth; ++k)
        if (net->layers[l + k].type != MYEA_LAYER_FULLY_CONNECTED || net->layers[l + k].ind_rnn)
          return fail(net, MYEA_E_UNSUPPORTED, "residual blocks of fully connected layers only");
      // the block output is as wide as the wider of the shortcut and the block's last layer (zero-padded identity); the
      // shortcut is the layer before, or the residual layer of the block that ends there
      uint32_t feeder = l - 1;
      for (uint32_t q = 1; q < l; ++q)
        if (net->layers[q].type == MYEA_LAYER_RESIDUAL && q + net->layers[q].block_depth == l - 1) feeder = q;
      L.n_out = std::max(net->layers[feeder].n_out, net->layers[l + L.block_depth].n_out);
    }
  }
  for (uint32_t l = 1; l < n; ++l) {
    const uint32_t t = net->layers[l].type;
    if ((t == MYEA_LAYER_AVERAGE_POOLING || t == MYEA_LAYER_MAX_POOLING) && layer_in_block(net, static_cast<int>(l) - 1, nullptr))
      return fail(net, MYEA_E_UNSUPPORTED, "a pooling layer next to a residual block is not built");
  }
  // inputs: a layer reads the layer before it; the first layer of a residual block reads the layer before the
  // residual layer, and the layer after a block reads the block's output (held by the residual layer)
  for (uint32_t l = 1; l < n; ++l) {
    net->layers[l].input_layer = static_cast<int>(l) - 1;
    net->layers[l].n_in = net->layers[l - 1].n_out;
  }
  for (uint32_t l = 1; l < n; ++l) {
    LayerPlan &L = net->layers[l];
    if (L.type != MYEA_LAYER_RESIDUAL) continue;
    net->layers[l + 1].input_layer = static_cast<int>(l) - 1;
    net->layers[l + 1].n_in = net->layers[l - 1].n_out;
    const uint32_t after = l + L.block_depth + 1;
    if (after < n) { net->layers[after].input_layer = static_cast<int>(l); net->layers[after].n_in = L.n_out; }
  }
  // weights
  uint64_t tw = 0;
  for (uint32_t l = 1; l < n; ++l) {
    LayerPlan &L = net->layers[l];
    const bool has_connections = L.type == MYEA_LAYER_FULLY_CONNECTED || L.type == MYEA_LAYER_LSTM;
    L.idx.number_inputs = has_connections ? L.n_in : 0;  // residual and pooling layers have no connections of their own
    L.idx.number_outputs = L.n_out;
    if (L.type == MYEA_LAYER_FULLY_CONNECTED) {
      L.idx.first_connection_index = tw;
      tw += static_cast<uint64_t>(L.n_out) * L.n_in;
      if (L.ind_rnn) tw += static_cast<uint64_t>(L.n_out);  // the units' self connections (Prepare__Connections__FC_Ind_RNN)
      L.idx.last_connection_index = tw;
    } else if (L.type == MYEA_LAYER_LSTM) {
      const uint64_t blocks = L.desc.unit_parameters[0] << (L.desc.use_bidirectional ? 1 : 0);
      const uint64_t cpb = std::max<uint64_t>(1, L.desc.unit_parameters[1]);
      const uint64_t cells_dir = L.desc.unit_parameters[0] * cpb;  // cells of one direction
      // per block: per cell [W_z,in (in) | W_z,rec (cells)], then W_i,in W_f,in W_o,in (in each), W_i,rec W_f,rec W_o,rec
      // (cells each), then peepholes p_i p_f p_o (cells per block each)
      L.idx.block_stride = cpb * (L.n_in + cells_dir) + 3 * L.n_in + 3 * cells_dir + 3 * cpb;
      L.idx.first_connection_index = tw;
      tw += blocks * L.idx.block_stride;
      L.idx.last_connection_index = tw;
    }
  }
  net->layers[0].idx.number_outputs = net->layers[0].n_out;
  net->total_weights = tw;
  // biases
  uint64_t tb = 0;
  for (uint32_t l = 1; l < n; ++l) {
    LayerPlan &L = net->layers[l];
    if (L.type == MYEA_LAYER_FULLY_CONNECTED) {
      L.idx.first_bias_connection_index = tw + tb;
      tb += L.n_out;
      L.idx.last_bias_connection_index = tw + tb;
    } else if (L.type == MYEA_LAYER_LSTM) {
      const uint64_t dirs = L.desc.use_bidirectional ? 2 : 1;
      const uint64_t cells = L.n_out, blocks = L.desc.unit_parameters[0] * dirs;
      // Prepare__Bias__LSTM overwrites first_bias_connection_index with (base + cells): the stored range is
      // [base + cells, base + cells + 3*blocks) although cells + 3*blocks slots are counted.
      L.idx.first_bias_connection_index = tw + tb + cells;
      tb += cells + 3 * blocks;
      L.idx.last_bias_connection_index = tw + tb;
    }
  }
  net->total_bias = tb;
  net->total_parameters = tw + tb;
  // normalized units
  net->any_norm = false;
  for (uint32_t l = 1; l < n; ++l) net->any_norm = net->any_norm || d.layers[l].type_normalization != MYEA_NORM_NONE;
  net->total_norm_units = 0;
  if (net->any_norm) {
    // units a layer normalizes (Prepare__Normalized__Layer / ..__Residual_Layer, Neural_Network__Layer_Normalization.cpp:43-154):
    // its own outputs; inside a residual block its INPUT (the block runs normalization -> activation -> weights); for a
    // residual layer the outputs of the block's last layer
    uint64_t units = 0;
    for (uint32_t l = 0; l < n; ++l) {
      LayerPlan &L = net->layers[l];
      L.norm_unit_offset = static_cast<long long>(units);
      if (L.type == MYEA_LAYER_LSTM && d.layers[l].type_normalization != MYEA_NORM_NONE)
        return fail(net, MYEA_E_UNSUPPORTED, "normalization of an LSTM layer's own gates and cell inputs is not built");
      long long own = L.n_out;
      if (L.type == MYEA_LAYER_LSTM) {  // three per cell and six per block, counted although the layer does not normalize
        const long long dirs = d.layers[l].use_bidirectional ? 2 : 1;
        own = 3 * L.n_out + 6 * static_cast<long long>(d.layers[l].unit_parameters[0]) * dirs;
      }
      if (L.type == MYEA_LAYER_RESIDUAL) own = net->layers[l + L.block_depth].n_out;
      if (L.type == MYEA_LAYER_AVERAGE_POOLING || L.type == MYEA_LAYER_MAX_POOLING) own = 0;  // Prepare__Normalized__Layer: none
      else if (l > 0 && layer_in_block(net, static_cast<int>(l), nullptr)) own = L.n_in;
      L.idx.number_units_norm = static_cast<uint64_t>(own);
      units += static_cast<uint64_t>(own);
    }
    net->total_norm_units = units;
    for (uint32_t l = 0; l < n; ++l) {
      LayerPlan &L = net->layers[l];
      L.idx.scale_index = net->total_parameters + L.norm_unit_offset;
      L.idx.shift_index = net->total_parameters + units + L.norm_unit_offset;
    }
    net->total_parameters += 2 * units;
  }
  return MYEA_OK;
}

static int allocate_buffers(myea_b200_net *net) {
  const size_t P = net->total_parameters;
  const long long rows = net->T * net->B;
  RC(dev_alloc(net, &net->params, P + 4));
  RC(dev_alloc(net, &net->grads, P + 4));
  RC(dev_alloc(net, &net->m1, P + 4));
  RC(dev_alloc(net, &net->m2, P + 4));
  RC(dev_alloc(net, &net->m2hat, P + 4));
  RC(dev_alloc(net, &net->prev_delta, P + 4));
  RC(dev_alloc(net, &net->mask_reg, P + 4));
  RC(dev_alloc(net, &net->d_loss_acc, 2));
  RC(dev_alloc(net, &net->d_loss_count, 1));
  RC(dev_alloc(net, &net->d_sumsq, 1));
  RC(dev_alloc(net, &net->d_clip_scale, 1));
  RC(dev_alloc(net, &net->d_loss_tmp, 3));
  RC(dev_alloc(net, &net->ctx.d_error_flag, 1));
  RC(gemm_splitk_reserve(net->ctx));
  RC(dev_alloc(net, &net->d_input, rows * net->layers[0].n_out));
  RC(dev_alloc(net, &net->d_desired, rows * net->layers.back().n_out));
  long long max_h = 1;
  size_t scratch = 0;
  for (size_t l = 1; l < net->layers.size(); ++l) {
    LayerPlan &L = net->layers[l];
    max_h = std::max(max_h, std::max(L.n_out, L.n_in));
    L.is_output = (l + 1 == net->layers.size());
    if (L.type == MYEA_LAYER_FULLY_CONNECTED) {
      L.has_norm = L.desc.type_normalization != MYEA_NORM_NONE;
      L.use_bias = !L.has_norm;
      if (L.has_norm && !L.desc.use_layer_normalization_before_activation && !layer_in_block(net, static_cast<int>(l), nullptr))
        return fail(net, MYEA_E_UNSUPPORTED, "normalization after the activation is not built");
      // a layer inside a residual block keeps its normalized / activated INPUT in `values` and `deriv`
      const long long wide = layer_in_block(net, static_cast<int>(l), nullptr) ? std::max(L.n_out, L.n_in) : L.n_out;
      RC(dev_alloc(net, &L.summations, rows * L.n_out));
      if (L.ind_rnn) RC(dev_alloc(net, &L.pre_af, rows * L.n_out));
      RC(dev_alloc(net, &L.values, rows * wide));
      RC(dev_alloc(net, &L.deriv, rows * wide));
      if (L.has_norm) RC(dev_alloc(net, &L.errors, rows * L.n_out));
      else L.errors = L.deriv;
      if (gemm_takes_mn_major(net->ctx, rows, L.n_out) &&
          gemm_takes_mn_major(net->ctx, rows, L.n_in) && gemm_takes_mn_major(net->ctx, L.n_out, L.n_in) && net->ctx.gemm_engine == 0) {
        L.shared_panels = true;
        RC(dev_alloc(net, &L.in_panel_mem, shared_panel_floats(rows, L.n_in)));
        RC(dev_alloc(net, &L.w_panel_mem, shared_panel_floats(L.n_out, L.n_in)));
        RC(dev_alloc(net, &L.d_panel_mem, shared_panel_floats(rows, L.n_out)));
      }
      scratch = std::max(scratch, gemm_scratch_floats(rows, L.n_out, L.n_in));   // forward
      scratch = std::max(scratch, gemm_scratch_floats(rows, L.n_in, L.n_out));   // backward data
      scratch = std::max(scratch, gemm_scratch_floats(L.n_out, L.n_in, rows));   // backward weight
      if (L.desc.type_dropout == MYEA_DROPOUT_BERNOULLI || L.desc.type_dropout == MYEA_DROPOUT_BERNOULLI_INVERTED) {
        const float p = L.desc.dropout_values[0];
        if (!(p > 0.f && p <= 1.f)) return fail(net, MYEA_E_INVALID, "retention probability must be in (0, 1]");
        RC(dev_alloc(net, &L.mask_bernoulli, net->T * L.n_out));
        CK(cudaMemsetAsync(L.mask_bernoulli, 1, net->T * L.n_out, net->ctx.stream));
        // inverted: kept units are scaled by 1/p while training, nothing at inference; plain Bernoulli: no scaling
        // while training, every unit times p at inference (…Forward_Pass__OpenMP.cpp:4907-4990)
        L.keep_scale = L.desc.type_dropout == MYEA_DROPOUT_BERNOULLI_INVERTED ? 1.0f / p : 1.0f;
        L.infer_scale = L.desc.type_dropout == MYEA_DROPOUT_BERNOULLI ? p : 1.0f;
      }
    } else if (L.type == MYEA_LAYER_LSTM) {
      RC(lstm_create(net, L));
    } else if (L.type == MYEA_LAYER_AVERAGE_POOLING || L.type == MYEA_LAYER_MAX_POOLING) {
      RC(dev_alloc(net, &L.values, rows * L.n_out));
      RC(dev_alloc(net, &L.deriv, rows * L.n_out));
      L.errors = L.deriv;  // no activation of its own: the error on its outputs is the error its backward pass spreads
      if (L.type == MYEA_LAYER_MAX_POOLING) RC(dev_alloc(net, &L.pool_winner, rows * L.n_out));
    } else if (L.type == MYEA_LAYER_RESIDUAL) {
      RC(dev_alloc(net, &L.values, rows * L.n_out));
      RC(dev_alloc(net, &L.deriv, rows * L.n_out));
      L.errors = L.deriv;
      L.has_norm = L.desc.type_normalization != MYEA_NORM_NONE;  // normalization of the block's output before the skip add
      if (L.has_norm) RC(dev_alloc(net, &L.summations, rows * L.n_out));
      if (L.desc.type_dropout == MYEA_DROPOUT_SHAKEDROP) {
        RC(dev_alloc(net, &L.shake_mask, net->B));
        RC(dev_alloc(net, &L.shake_alpha, net->B * L.n_out));
        RC(dev_alloc(net, &L.shake_beta, net->B * L.n_out));
      }
    }
  }
  net->layers[0].values = net->d_input;
  // normalization state
  if (net->any_norm) {
    // every time step keeps statistics of its own (gamma and beta are shared): arrays of T * units values, one layer
    // after the other, each layer as [T][its units] (Allocate__Normalized_Unit, Neural_Network__Allocate.cpp:2643-2700)
    const size_t U = net->total_norm_units * static_cast<size_t>(net->T);
    RC(dev_alloc(net, &net->norm_mean_avg, U));
    RC(dev_alloc(net, &net->norm_sigma_avg, U));
    RC(dev_alloc(net, &net->norm_stats, U * 6));
    // partial sums of up to norm_chunks row blocks (the contractions' epilogues emit one per 32 rows) | 3 coefficients |
    // 2 cross-GPU sums
    net->norm_chunks = static_cast<int>(std::max<long long>(net->reduce_chunks, (rows + 31) / 32));
    RC(dev_alloc(net, &net->norm_partial, static_cast<size_t>(2 * net->norm_chunks + 5) * max_h));
    for (size_t l = 1; l < net->layers.size(); ++l) {
      LayerPlan &L = net->layers[l];
      if (!L.has_norm) continue;
      NormParams &np = L.norm;
      np.type = L.desc.type_normalization;
      np.momentum = net->desc.normalization_momentum_average > 0.f ? net->desc.normalization_momentum_average : 0.999f;
      np.epsilon = net->desc.normalization_epsilon > 0.f ? net->desc.normalization_epsilon : 1e-5f;
      np.r_max = net->desc.batch_renormalization_r_correction_maximum > 0.f ? net->desc.batch_renormalization_r_correction_maximum : 1.f;
      np.d_max = net->desc.batch_renormalization_d_correction_maximum > 0.f ? net->desc.batch_renormalization_d_correction_maximum : 0.f;
      np.gamma = net->params + L.idx.scale_index;
      np.beta = net->params + L.idx.shift_index;
      np.d_gamma = net->grads + L.idx.scale_index;
      np.d_beta = net->grads + L.idx.shift_index;
      const size_t o = static_cast<size_t>(L.norm_unit_offset) * static_cast<size_t>(net->T);  // time step 0 of this layer
      np.mean_avg = net->norm_mean_avg + o;
      np.sigma_avg = net->norm_sigma_avg + o;
      np.mean = net->norm_stats + 0 * U + o;
      np.sigma = net->norm_stats + 1 * U + o;
      np.r = net->norm_stats + 2 * U + o;
      np.d = net->norm_stats + 3 * U + o;
      np.col_scale = net->norm_stats + 4 * U + o;
      np.col_shift = net->norm_stats + 5 * U + o;
      np.partial = net->norm_partial;
      np.chunks = net->norm_chunks;
    }
  }
  RC(dev_alloc(net, &net->reduce_partial, static_cast<size_t>(net->reduce_chunks) * max_h));
  net->scratch.floats = std::max(net->scratch.floats, scratch + 64);
  RC(dev_alloc(net, &net->scratch.base, net->scratch.floats, false));
  return MYEA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// create / destroy / queries
// ---------------------------------------------------------------------------------------------------------
extern "C" int myea_b200_create(myea_handle *out, const myea_net_desc *desc, int device) {
  if (out == nullptr || desc == nullptr) return MYEA_E_INVALID;
  *out = nullptr;
  if (desc->number_layers < 2 || desc->number_layers > MYEA_MAX_LAYERS || desc->batch_size == 0 || desc->number_recurrent_depth == 0)
    return MYEA_E_INVALID;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) return MYEA_E_CUDA;  // no GPU: fail loudly, there is no CPU path
  if (device < 0 || device >= count) return MYEA_E_INVALID;
  if (cudaSetDevice(device) != cudaSuccess) return MYEA_E_CUDA;
  myea_b200_net *net = new (std::nothrow) myea_b200_net();
  if (net == nullptr) return MYEA_E_INVALID;
  net->desc = *desc;
  net->ctx.device = device;
  net->T = static_cast<long long>(desc->number_recurrent_depth);
  net->B = static_cast<long long>(desc->batch_size);
  net->active_B = net->B;
  const char *eng = getenv("MYEA_B200_GEMM_ENGINE");  // 1 = the exact FP32 FMA engine (tests use it to tell tensor-core effects apart)
  if (eng != nullptr && eng[0] == '1') net->ctx.gemm_engine = 1;
  *out = net;  // returned even on failure so that the caller can read last_error, then destroy
  if (cudaStreamCreateWithFlags(&net->ctx.stream, cudaStreamNonBlocking) != cudaSuccess) return fail(net, MYEA_E_CUDA, "cudaStreamCreate failed");
  cudaEventCreate(&net->ctx.ev0);
  cudaEventCreate(&net->ctx.ev1);
  if (cudaStreamCreateWithFlags(&net->copy_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&net->ev_desired_ready, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&net->ev_desired_free, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&net->ev_input_ready, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&net->ev_input_free, cudaEventDisableTiming) != cudaSuccess)
    return fail(net, MYEA_E_CUDA, "cudaStreamCreate / cudaEventCreate failed");
  RC(myea::build_index_map(net));
  net->full_pitch = net->T > 1;
  for (const LayerPlan &L : net->layers) net->full_pitch = net->full_pitch || L.type == MYEA_LAYER_LSTM;
  RC(allocate_buffers(net));
  CK(cudaStreamSynchronize(net->ctx.stream));
  return MYEA_OK;
}

extern "C" void myea_b200_destroy(myea_handle net) {
  if (net == nullptr) return;
  cudaSetDevice(net->ctx.device);
  if (net->ctx.stream) cudaStreamSynchronize(net->ctx.stream);
  comm_destroy(net);
  for (auto &L : net->layers) lstm_destroy(L);
  for (void *p : net->allocations) cudaFree(p);
  gemm_splitk_release(net->ctx);
  for (void *p : {static_cast<void *>(net->ds_inputs), static_cast<void *>(net->ds_outputs), static_cast<void *>(net->ds_batch_inputs),
                  static_cast<void *>(net->ds_batch_outputs), static_cast<void *>(net->ds_order)})
    if (p != nullptr) cudaFree(p);
  if (net->ctx.ev0) cudaEventDestroy(net->ctx.ev0);
  if (net->ctx.ev1) cudaEventDestroy(net->ctx.ev1);
  if (net->copy_stream) { cudaStreamSynchronize(net->copy_stream); cudaStreamDestroy(net->copy_stream); }
  if (net->ev_desired_ready) cudaEventDestroy(net->ev_desired_ready);
  if (net->ev_desired_free) cudaEventDestroy(net->ev_desired_free);
  if (net->ev_input_ready) cudaEventDestroy(net->ev_input_ready);
  if (net->ev_input_free) cudaEventDestroy(net->ev_input_free);
  if (net->ctx.stream) cudaStreamDestroy(net->ctx.stream);
  delete net;
}

extern "C" const char *myea_b200_last_error(myea_handle net) { return net ? net->ctx.error.c_str() : "null handle"; }

extern "C" int myea_b200_sizes(myea_handle net, uint64_t *P, uint64_t *W, uint64_t *bias, uint64_t *norm_units) {
  if (net == nullptr) return MYEA_E_INVALID;
  if (P) *P = net->total_parameters;
  if (W) *W = net->total_weights;
  if (bias) *bias = net->total_bias;
  if (norm_units) *norm_units = net->total_norm_units;
  return MYEA_OK;
}

extern "C" int myea_b200_layer_index(myea_handle net, uint32_t layer, myea_layer_index *out) {
  if (net == nullptr || out == nullptr || layer >= net->layers.size()) return MYEA_E_INVALID;
  *out = net->layers[layer].idx;
  return MYEA_OK;
}

static float *select_buffer(myea_b200_net *net, int which, size_t *count) {
  *count = net->total_parameters;
  switch (which) {
    case MYEA_BUF_PARAMETERS: return net->params;
    case MYEA_BUF_DERIVATIVES: return net->grads;
    case MYEA_BUF_FIRST_MOMENT: case MYEA_BUF_PREVIOUS_DERIVATIVES: return net->m1;
    case MYEA_BUF_SECOND_MOMENT: case MYEA_BUF_PREVIOUS_STEPS: return net->m2;
    case MYEA_BUF_SECOND_MOMENT_HAT: return net->m2hat;
    case MYEA_BUF_MASK_REGULARIZED: return net->mask_reg;
    case MYEA_BUF_PREVIOUS_DELTA: return net->prev_delta;
    case MYEA_BUF_NORM_MEAN_AVERAGE: *count = net->total_norm_units * static_cast<uint64_t>(net->T); return net->norm_mean_avg;
    case MYEA_BUF_NORM_VARIANCE_AVERAGE: *count = net->total_norm_units * static_cast<uint64_t>(net->T); return net->norm_sigma_avg;
    default: *count = 0; return nullptr;
  }
}

extern "C" int myea_b200_upload(myea_handle net, int which, const float *host, uint64_t offset, uint64_t count) {
  if (net == nullptr || host == nullptr) return MYEA_E_INVALID;
  size_t n = 0;
  float *dst = select_buffer(net, which, &n);
  if (dst == nullptr || offset > n || count > n - offset) return fail(net, MYEA_E_INVALID, "upload: buffer selector or range out of bounds");
  CK(cudaSetDevice(net->ctx.device));
  RC(comm_gather_join(net));
  CK(cudaMemcpyAsync(dst + offset, host, count * sizeof(float), cudaMemcpyHostToDevice, net->ctx.stream));
  CK(cudaStreamSynchronize(net->ctx.stream));
  if (dst == net->params) {
    for (auto &L : net->layers) L.w_valid = false;  // weight panels of the last forward pass no longer match
  }
  return MYEA_OK;
}

extern "C" int myea_b200_download(myea_handle net, int which, float *host, uint64_t offset, uint64_t count) {
  if (net == nullptr || host == nullptr) return MYEA_E_INVALID;
  size_t n = 0;
  float *src = select_buffer(net, which, &n);
  if (src == nullptr || offset > n || count > n - offset) return fail(net, MYEA_E_INVALID, "download: buffer selector or range out of bounds");
  CK(cudaSetDevice(net->ctx.device));
  // under a sharded update every rank keeps the optimizer state of its slices only: reading such a buffer back gathers
  // the slices first (collective: every rank has to make the call)
  RC(comm_gather_join(net));
  if (net->comm != nullptr && (src == net->m1 || src == net->m2 || src == net->m2hat || src == net->prev_delta)) RC(comm_gather_state(net, src));
  CK(cudaMemcpyAsync(host, src + offset, count * sizeof(float), cudaMemcpyDeviceToHost, net->ctx.stream));
  CK(cudaStreamSynchronize(net->ctx.stream));
  return MYEA_OK;
}

extern "C" int myea_b200_set_mask_bernoulli(myea_handle net, uint32_t layer, const uint8_t *mask, uint64_t count) {
  if (net == nullptr || mask == nullptr || layer >= net->layers.size()) return MYEA_E_INVALID;
  LayerPlan &L = net->layers[layer];
  if (L.mask_bernoulli == nullptr || count != static_cast<uint64_t>(net->T * L.n_out)) return fail(net, MYEA_E_INVALID, "layer has no Bernoulli mask of that size");
  CK(cudaMemcpyAsync(L.mask_bernoulli, mask, count, cudaMemcpyHostToDevice, net->ctx.stream));
  CK(cudaStreamSynchronize(net->ctx.stream));
  return MYEA_OK;
}

extern "C" int myea_b200_set_mask_zoneout(myea_handle net, uint32_t layer, const uint8_t *mask_state, const uint8_t *mask_output,
                                          uint64_t count) {
  if (net == nullptr || mask_state == nullptr || mask_output == nullptr || layer >= net->layers.size()) return MYEA_E_INVALID;
  LayerPlan &L = net->layers[layer];
  if (L.type != MYEA_LAYER_LSTM) return fail(net, MYEA_E_INVALID, "zoneout masks belong to LSTM layers");
  return lstm_set_zoneout(net, L, mask_state, mask_output, count);
}

extern "C" int myea_b200_set_shakedrop(myea_handle net, uint32_t layer, const uint8_t *mask, const float *alpha, const float *beta,
                                       uint64_t batch) {
  if (net == nullptr || mask == nullptr || alpha == nullptr || beta == nullptr || layer >= net->layers.size()) return MYEA_E_INVALID;
  LayerPlan &L = net->layers[layer];
  if (L.shake_mask == nullptr || batch != static_cast<uint64_t>(net->B)) return fail(net, MYEA_E_INVALID, "layer has no ShakeDrop state of that batch size");
  CK(cudaMemcpyAsync(L.shake_mask, mask, batch, cudaMemcpyHostToDevice, net->ctx.stream));
  CK(cudaMemcpyAsync(L.shake_alpha, alpha, batch * L.n_out * sizeof(float), cudaMemcpyHostToDevice, net->ctx.stream));
  CK(cudaMemcpyAsync(L.shake_beta, beta, batch * L.n_out * sizeof(float), cudaMemcpyHostToDevice, net->ctx.stream));
  CK(cudaStreamSynchronize(net->ctx.stream));
  return MYEA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Forward pass
// ---------------------------------------------------------------------------------------------------------
namespace myea {

// One fully connected layer on `rows` rows: z = x W^T (+ b); normalization statistics; activation; dropout.
// Forward_Pass__FC (Neural_Network__Forward_Pass__Loop.cpp:350-790 is the per-layer driver).
// (a short last batch may fall below the 256 x 256 kernel's shapes: then the layer goes the per-contraction way)
static bool fc_uses_shared_panels(const myea_b200_net *net, const LayerPlan &L, long long rows) {
  return L.shared_panels && gemm_takes_mn_major(net->ctx, rows, L.n_out) && gemm_takes_mn_major(net->ctx, rows, L.n_in);
}

// The weight panels of a layer depend on no activation: a forward pass whose inputs come from the host makes them all
// while the inputs are still on their way (see forward_impl).
static int fc_prepare_weights(myea_b200_net *net, LayerPlan &L) {
  const bool tr = net->training;
  RC(comm_wait_gathers(net, L.idx.first_connection_index, L.idx.last_connection_index - L.idx.first_connection_index));
  RC(gemm_prepare_shared(net->ctx, net->params + L.idx.first_connection_index, L.n_in, L.n_out, L.n_in, L.w_panel_mem, PANEL_ROLE_B, &L.w_rows,
                         PANEL_ROLE_B, tr ? &L.w_cols : nullptr));
  L.w_prepared = true;
  return MYEA_OK;
}

int fc_product_forward(myea_b200_net *net, LayerPlan &L, const float *input, long long rows, const Epilogue &e) {
  const float *w = net->params + L.idx.first_connection_index;
  // the other ranks' slices of this layer's updated weights (a sharded update gathers them layer by layer)
  RC(comm_wait_gathers(net, L.idx.first_connection_index, L.idx.last_connection_index - L.idx.first_connection_index));
  if (fc_uses_shared_panels(net, L, rows)) {
    // while training, the same pass also writes the column readings the backward contractions will want
    const bool tr = net->training;
    if (L.in_ready_src == input && L.in_ready_rows == rows) {
      // the kernel that produced `input` has written these panels already (fc_forward of the layer before)
    } else {
      RC(gemm_prepare_shared(net->ctx, input, L.n_in, rows, L.n_in, L.in_panel_mem, PANEL_ROLE_A, &L.in_rows, PANEL_ROLE_B, tr ? &L.in_cols : nullptr));
    }
    L.in_ready_src = nullptr;
    if (!L.w_prepared) RC(fc_prepare_weights(net, L));
    L.w_prepared = false;
    L.in_valid = L.w_valid = tr;
    L.in_src = input;
    L.d_valid = false;
    return gemm_panels(net->ctx, L.in_rows, 0, rows, L.w_rows, 0, L.n_out, e);
  }
  L.in_valid = L.w_valid = L.d_valid = false;
  Operand a{input, rows, L.n_in, L.n_in, 1};
  Operand b{w, L.n_out, L.n_in, L.n_in, 1};
  return gemm_nt(net->ctx, a, b, e, net->scratch);
}

int fc_product_backward(myea_b200_net *net, LayerPlan &N, long long rows, const Epilogue &e) {
  if (N.shared_panels && N.w_valid) {
    if (!N.d_valid)  // (the normalization backward of N may have written them already)
      RC(gemm_prepare_shared(net->ctx, N.errors, N.n_out, rows, N.n_out, N.d_panel_mem, PANEL_ROLE_A, &N.d_rows, PANEL_ROLE_A, &N.d_cols));
    N.d_valid = true;
    return gemm_panels(net->ctx, N.d_rows, 0, rows, N.w_cols, 0, N.n_in, e);
  }
  Operand a{N.errors, rows, N.n_out, N.n_out, 1};
  Operand b{net->params + N.idx.first_connection_index, N.n_in, N.n_out, 1, N.n_in};  // W[out,in] read as [in rows, K=out]
  return gemm_nt(net->ctx, a, b, e, net->scratch);
}

// the normalization state of time step t of a layer
static NormParams norm_at_step(const LayerPlan &L, long long t) {
  NormParams np = L.norm;
  const long long o = t * static_cast<long long>(L.idx.number_units_norm);
  np.mean += o; np.sigma += o; np.r += o; np.d += o; np.mean_avg += o; np.sigma_avg += o; np.col_scale += o; np.col_shift += o;
  return np;
}

int fc_forward(myea_b200_net *net, LayerPlan &L, const float *input, long long rows) {
  // normalization with batch statistics / dropout with masks: as the network's state says, unless a pre-training pass
  // runs this layer in another role (LayerPlan::mode_norm, mode_drop)
  const bool norm_train = L.mode_norm < 0 ? net->training : L.mode_norm != 0;
  const bool drop_train = L.mode_drop < 0 ? net->training : L.mode_drop != 0;
  Epilogue e;
  e.C = L.summations;
  e.ldc = L.n_out;
  e.bias = L.use_bias ? net->params + L.idx.first_bias_connection_index : nullptr;
  // batch statistics: the contraction's epilogue leaves the column sums of every 32-row block behind, where it can
  int fused_chunks = 0;
  const bool timewise_norm = (L.has_norm && net->T > 1) || L.ind_rnn;  // a recurrent network normalizes every time step by itself
  if (L.has_norm && norm_train && !timewise_norm) {
    Epilogue probe = e;
    probe.stats_kind = 1;
    probe.col_stats = L.norm.partial;
    probe.stats_blocks = (rows + 31) / 32;
    if (probe.stats_blocks <= L.norm.chunks && epilogue_takes_stats(net->ctx, probe, L.n_out)) {
      e = probe;
      fused_chunks = static_cast<int>(probe.stats_blocks);
    }
  }
  RC(fc_product_forward(net, L, input, rows, e));
  const size_t li = static_cast<size_t>(&L - net->layers.data());
  // the layer that reads this one's output from shared operand panels gets them from the activation kernel
  PanelSink sink;
  bool use_sink = false;
  if (li + 1 < net->layers.size() && !timewise_norm && activation_writes_panels(L.desc.type_activation_function) && (rows & 7) == 0 && (L.n_out & 7) == 0 &&
      net->ctx.gemm_engine == 0) {
    LayerPlan &N = net->layers[li + 1];
    if (N.type == MYEA_LAYER_FULLY_CONNECTED && N.input_layer == static_cast<int>(li) && fc_uses_shared_panels(net, N, rows)) {
      shared_panel_layout(N.in_panel_mem, rows, N.n_in, PANEL_ROLE_A, &N.in_rows, PANEL_ROLE_B, net->training ? &N.in_cols : nullptr, &sink);
      N.in_ready_src = L.values;
      N.in_ready_rows = rows;
      use_sink = true;
    }
  }
  if (L.ind_rnn) {
    // the recurrence runs step by step on the summations of all steps (one contraction above): per step the statistics of
    // a normalized layer, then pre = z' + u * y_prev and the activation
    if (L.desc.type_activation_function == MYEA_AF_SOFTMAX) return MYEA_E_UNSUPPORTED;
    const long long pitch = rows / net->T;
    const uint8_t *mask = (drop_train && L.mask_bernoulli != nullptr) ? L.mask_bernoulli : nullptr;
    const float scale = drop_train ? (mask != nullptr ? L.keep_scale : 1.f) : L.infer_scale;
    const float *u = net->params + L.idx.first_connection_index + static_cast<uint64_t>(L.n_out) * L.n_in;
    for (long long t = 0; t < net->T; ++t) {
      const long long off = t * pitch * L.n_out;
      const float *cs = nullptr, *ch = nullptr;
      if (L.has_norm) {
        const NormParams np = norm_at_step(L, t);
        RC(norm_forward_stats(net->ctx, L.summations + off, net->active_B, L.n_out, np, norm_train ? 1 : 0, &net->hook, nullptr, 0));
        cs = np.col_scale; ch = np.col_shift;
      }
      RC(ind_rnn_forward_step(net->ctx, L.summations + off, t > 0 ? L.values + off - pitch * L.n_out : nullptr, u, L.pre_af + off, L.values + off, pitch,
                              L.n_out, L.desc.type_activation_function, cs, ch, mask != nullptr ? mask + t * L.n_out : nullptr, scale));
    }
    return MYEA_OK;
  }
  if (timewise_norm) {
    // statistics, running averages and coefficients of step t live at t * units behind those of step 0; the rows a short
    // batch leaves unused take part in no sum (Forward_Pass__Batch_Normalization__Training__Loop(time_step, ...),
    // Neural_Network__Forward_Pass__Loop.cpp:4673-4750)
    if (L.desc.type_activation_function == MYEA_AF_SOFTMAX) return MYEA_E_UNSUPPORTED;
    const long long pitch = rows / net->T;
    const uint8_t *mask = (drop_train && L.mask_bernoulli != nullptr) ? L.mask_bernoulli : nullptr;
    const float scale = drop_train ? (mask != nullptr ? L.keep_scale : 1.f) : L.infer_scale;
    for (long long t = 0; t < net->T; ++t) {
      const NormParams np = norm_at_step(L, t);
      const long long off = t * pitch * L.n_out;
      RC(norm_forward_stats(net->ctx, L.summations + off, net->active_B, L.n_out, np, norm_train ? 1 : 0, &net->hook, nullptr, 0));
      RC(activation_forward(net->ctx, L.summations + off, L.values + off, pitch, L.n_out, L.desc.type_activation_function, np.col_scale, np.col_shift,
                            mask != nullptr ? mask + t * L.n_out : nullptr, scale, nullptr));
    }
    return MYEA_OK;
  }
  const float *cs = nullptr, *ch = nullptr;
  if (L.has_norm) {
    // data-parallel ranks exchange the column sums here; the next layer's weight panels depend on nothing that is in
    // flight and are made while the sums travel
    struct Next { myea_b200_net *net; LayerPlan *layer; } next{net, nullptr};
    if (li + 1 < net->layers.size()) {
      LayerPlan &N = net->layers[li + 1];
      if (N.type == MYEA_LAYER_FULLY_CONNECTED && !N.w_prepared && fc_uses_shared_panels(net, N, rows)) next.layer = &N;
    }
    OverlapWork work;
    work.arg = &next;
    work.run = [](void *arg) { Next *p = static_cast<Next *>(arg); return fc_prepare_weights(p->net, *p->layer); };
    RC(norm_forward_stats(net->ctx, L.summations, rows, L.n_out, L.norm, norm_train ? 1 : 0, &net->hook, next.layer != nullptr ? &work : nullptr,
                          fused_chunks));
    cs = L.norm.col_scale;
    ch = L.norm.col_shift;
  }
  if (L.desc.type_activation_function == MYEA_AF_SOFTMAX) {
    if (L.has_norm) return MYEA_E_UNSUPPORTED;
    return softmax_forward(net->ctx, L.summations, L.values, rows, L.n_out);
  }
  const uint8_t *mask = (drop_train && L.mask_bernoulli != nullptr) ? L.mask_bernoulli : nullptr;
  const float scale = drop_train ? (mask != nullptr ? L.keep_scale : 1.f) : L.infer_scale;
  if (mask != nullptr && net->T > 1) {
    // a recurrent network draws one mask per time step (mask[t][unit], Forward_Pass__Dropout__Bernoulli__Training__Loop,
    // Neural_Network__Forward_Pass__Loop.cpp:4947-4970): one activation pass per step, each with its own mask row
    if (use_sink) net->layers[li + 1].in_ready_src = nullptr;
    const long long step_rows = rows / net->T;
    for (long long t = 0; t < net->T; ++t)
      RC(activation_forward(net->ctx, L.summations + t * step_rows * L.n_out, L.values + t * step_rows * L.n_out, step_rows, L.n_out,
                            L.desc.type_activation_function, cs, ch, mask + t * L.n_out, scale, nullptr));
    return MYEA_OK;
  }
  if (use_sink && ((reinterpret_cast<uintptr_t>(cs) | reinterpret_cast<uintptr_t>(ch)) & 15) != 0) {  // unaligned coefficients: the plain kernel, and the reader splits
    use_sink = false;
    net->layers[li + 1].in_ready_src = nullptr;
  }
  RC(activation_forward(net->ctx, L.summations, L.values, rows, L.n_out, L.desc.type_activation_function, cs, ch, mask, scale, use_sink ? &sink : nullptr));
  return MYEA_OK;
}

}  // namespace myea

// Forward_Pass(batch_size_received, ...) accepts any batch up to the allocated one (the last batch of
// Dataset::Train_Batch_BP is smaller, Dataset.cpp:667-691).  A feed-forward network (one time step) keeps plain
// [rows][units] buffers and simply runs fewer rows.  Recurrent buffers are [T][B][units] with the allocated B as the
// pitch, as in the reference: a shorter batch fills the first rows of every time step, the rows behind them are
// computed along as padding - zero inputs, zero output error, hence zero deltas and no share in any derivative - and
// are not counted in the loss.
static int batch_for_forward(myea_b200_net *net, uint64_t batch) {
  const long long b = static_cast<long long>(batch);
  if (b == net->B) return MYEA_OK;
  if (b < 1 || b > net->B) return fail(net, MYEA_E_INVALID, "batch must be between 1 and the batch size the network was created for");
  if (net->comm != nullptr) return fail(net, MYEA_E_UNSUPPORTED, "with a communicator attached every rank takes full batches");
  return MYEA_OK;
}
// rows the kernels of the step in flight run over, and the rows per time step among them
static long long pitch_rows(const myea_b200_net *net) { return net->pitch(); }
static long long step_rows_total(const myea_b200_net *net) { return net->T * pitch_rows(net); }
// host or device block packed [T][active_B][units] -> [T][pitch][units], padding rows zeroed
static int copy_batch_in(myea_b200_net *net, float *dst, const float *src, long long units, cudaMemcpyKind kind, cudaStream_t stream) {
  const long long pitch = pitch_rows(net), b = net->active_B;
  if (b == pitch) {
    CK(cudaMemcpyAsync(dst, src, net->T * b * units * sizeof(float), kind, stream));
    return MYEA_OK;
  }
  CK(cudaMemcpy2DAsync(dst, pitch * units * sizeof(float), src, b * units * sizeof(float), b * units * sizeof(float), net->T, kind, stream));
  CK(cudaMemset2DAsync(dst + b * units, pitch * units * sizeof(float), 0, (pitch - b) * units * sizeof(float), net->T, stream));
  return MYEA_OK;
}
static int batch_in_flight(myea_b200_net *net, uint64_t batch) {
  if (static_cast<long long>(batch) != net->active_B) return fail(net, MYEA_E_INVALID, "batch must equal the batch of the last forward pass");
  return MYEA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Autoencoder pre-training (Set__Pre_Training_Level, Neural_Network__Indexing.cpp:20-51): at level k >= 1 only hidden
// layer k (the "coded" layer) and its mirror image, layer n - k (the "decoded" layer), are trained: the layers before k
// encode the input in inference behaviour (the one feeding layer k with its training dropout), layer k and layer n - k
// run in training behaviour with dropout reduced to its inference scaling, the decoded layer reads the coded layer's
// output, and its output is compared with what the coded layer read (the targets of the call at level 1)
// (FF__Forward_Pass_Batch__Pre_Training, …Forward_Pass__Loop.cpp:205-326; FF__Compute__Error :120;
// FF__Backward_Pass_Batch__Pre_Training, …Backward_Pass__Loop.cpp:211-296; FF__Update_Derivative_Weight_Batch__Pre_Training,
// …Update_Derivative_Weight__Loop.cpp:135-182).
// ---------------------------------------------------------------------------------------------------------
static int pre_training_layers(myea_b200_net *net, int *coded, int *decoded) {
  const int n = static_cast<int>(net->layers.size()), k = static_cast<int>(net->pre_training_level);
  *coded = k;
  *decoded = n - k;
  return MYEA_OK;
}

extern "C" int myea_b200_set_pre_training_level(myea_handle net, uint64_t level) {
  if (net == nullptr) return MYEA_E_INVALID;
  const uint64_t n = net->layers.size();
  if (level == 0) { net->pre_training_level = 0; return MYEA_OK; }
  if (n < 3 || level > (n - 3) / 2 + 1) return fail(net, MYEA_E_INVALID, "pre-training level above the number of layer pairs");
  if (net->T != 1 || net->comm != nullptr) return fail(net, MYEA_E_UNSUPPORTED, "pre-training of recurrent or data-parallel networks is not built");
  const LayerPlan &K = net->layers[level], &D = net->layers[n - level];
  for (uint64_t l = 1; l <= level; ++l)
    if (net->layers[l].type != MYEA_LAYER_FULLY_CONNECTED || net->layers[l].ind_rnn || layer_in_block(net, static_cast<int>(l), nullptr))
      return fail(net, MYEA_E_UNSUPPORTED, "pre-training is built for plain fully connected layers");
  if (D.type != MYEA_LAYER_FULLY_CONNECTED || D.ind_rnn || layer_in_block(net, static_cast<int>(n - level), nullptr))
    return fail(net, MYEA_E_UNSUPPORTED, "pre-training is built for plain fully connected layers");
  if (D.n_in != K.n_out || D.n_out != K.n_in) return fail(net, MYEA_E_INVALID, "the decoded layer is not the mirror image of the coded layer");
  if (K.has_norm || D.has_norm) return fail(net, MYEA_E_UNSUPPORTED, "normalization on the coded or decoded layer is not built");
  if (D.desc.type_activation_function == MYEA_AF_SOFTMAX && n - level != n - 1) return fail(net, MYEA_E_INVALID, "softmax on a hidden layer");
  net->pre_training_level = static_cast<uint32_t>(level);
  return MYEA_OK;
}

static int forward_pre_training(myea_b200_net *net, long long rows) {
  int k = 0, dl = 0;
  RC(pre_training_layers(net, &k, &dl));
  for (int l = 1; l < k; ++l) {  // encode: inference behaviour; the layer feeding the coded layer keeps its training dropout
    LayerPlan &L = net->layers[l];
    L.mode_norm = 0;
    L.mode_drop = (l == k - 1 && net->training) ? 1 : 0;
    const int rc = fc_forward(net, L, net->layers[L.input_layer].values, rows);
    L.mode_norm = L.mode_drop = -1;
    RC(rc);
  }
  LayerPlan &K = net->layers[k], &D = net->layers[dl];
  K.mode_drop = 0;  // (coded dropout is a flag this library does not carry: the layer scales as at inference)
  int rc = fc_forward(net, K, net->layers[K.input_layer].values, rows);
  K.mode_drop = -1;
  RC(rc);
  D.mode_drop = 0;
  rc = fc_forward(net, D, K.values, rows);
  D.mode_drop = -1;
  return rc;
}

static int forward_impl(myea_b200_net *net, uint64_t batch, const float *src, cudaMemcpyKind kind, int training) {
  if (net == nullptr || src == nullptr) return MYEA_E_INVALID;
  RC(batch_for_forward(net, batch));
  CK(cudaSetDevice(net->ctx.device));
  net->training = training != 0;
  net->active_B = static_cast<long long>(batch);
  const long long rows = step_rows_total(net);
  const int n = static_cast<int>(net->layers.size());
  for (auto &L : net->layers) { L.w_prepared = false; L.in_ready_src = nullptr; }
  // After a sharded update the gathers of the updated parameters may still be travelling.  Biases and normalization
  // parameters are waited for here, every fully connected layer's weights where the layer first reads them, and
  // everything that is left before any other kind of layer.
  RC(comm_wait_gathers(net, net->total_weights, net->total_parameters - net->total_weights));
  if (kind == cudaMemcpyHostToDevice) {
    // inputs from the host: copy them on the side stream (once everything already queued has finished with d_input)
    // and split every large layer's weights meanwhile - the copy takes longer than all those passes together
    CK(cudaEventRecord(net->ev_input_free, net->ctx.stream));
    CK(cudaStreamWaitEvent(net->copy_stream, net->ev_input_free, 0));
    RC(copy_batch_in(net, net->d_input, src, net->layers[0].n_out, kind, net->copy_stream));
    CK(cudaEventRecord(net->ev_input_ready, net->copy_stream));
    for (int l = 1; l < n; ++l) {
      LayerPlan &L = net->layers[l];
      if (L.type == MYEA_LAYER_FULLY_CONNECTED && fc_uses_shared_panels(net, L, rows)) RC(fc_prepare_weights(net, L));
    }
    CK(cudaStreamWaitEvent(net->ctx.stream, net->ev_input_ready, 0));
  } else {
    RC(copy_batch_in(net, net->d_input, src, net->layers[0].n_out, kind, net->ctx.stream));
  }
  if (net->pre_training_level != 0) {
    RC(comm_gather_join(net));
    return forward_pre_training(net, rows);
  }
  for (int l = 1; l < n;) {
    LayerPlan &L = net->layers[l];
    const LayerPlan &in = net->layers[L.input_layer];
    if (L.type != MYEA_LAYER_FULLY_CONNECTED || L.ind_rnn) RC(comm_gather_join(net));
    if (L.type == MYEA_LAYER_FULLY_CONNECTED) {
      if (layer_in_block(net, l, nullptr)) return fail(net, MYEA_E_INVALID, "block layer outside its block");
      RC(fc_forward(net, L, in.values, rows));
      ++l;
    } else if (L.type == MYEA_LAYER_LSTM) {
      RC(lstm_forward(net, L, in.values, L.n_in));
      ++l;
    } else if (L.type == MYEA_LAYER_AVERAGE_POOLING || L.type == MYEA_LAYER_MAX_POOLING) {
      RC(pooling_forward(net, L, in.values, rows));
      ++l;
    } else {  // residual block: consumes layers l+1 .. l+depth
      RC(residual_forward(net, l));
      l += L.block_depth + 1;
    }
  }
  return comm_gather_join(net);
}

extern "C" int myea_b200_forward(myea_handle net, uint64_t batch, const float *inputs, int training) {
  return forward_impl(net, batch, inputs, cudaMemcpyHostToDevice, training);
}
extern "C" int myea_b200_forward_device(myea_handle net, uint64_t batch, const float *inputs, int training) {
  return forward_impl(net, batch, inputs, cudaMemcpyDeviceToDevice, training);
}

// ---------------------------------------------------------------------------------------------------------
// Output error
// ---------------------------------------------------------------------------------------------------------
static int compute_error_impl(myea_b200_net *net, uint64_t batch, const float *src, cudaMemcpyKind kind) {
  if (net == nullptr || src == nullptr) return MYEA_E_INVALID;
  RC(batch_in_flight(net, batch));
  CK(cudaSetDevice(net->ctx.device));
  if (net->pre_training_level != 0) {
    // the decoded layer answers as the output layer; above level 1 it is compared with what the coded layer read
    int k = 0, dl = 0;
    RC(pre_training_layers(net, &k, &dl));
    LayerPlan &D = net->layers[dl];
    const long long rows = step_rows_total(net);
    const float *desired = net->layers[k - 1].values;
    if (k <= 1) {
      CK(cudaStreamWaitEvent(net->ctx.stream, net->ev_desired_free, 0));
      CK(cudaMemcpyAsync(net->d_desired, src, rows * D.n_out * sizeof(float), kind, net->ctx.stream));
      desired = net->d_desired;
    }
    RC(output_error(net->ctx, D.summations, D.values, desired, D.errors, rows, D.n_out, D.desc.type_activation_function, net->desc.type_loss_function,
                    net->desc.type_accuracy_function, net->desc.accuracy_variance > 0.f ? net->desc.accuracy_variance : 0.49f, net->d_loss_acc,
                    net->d_loss_count));
    CK(cudaEventRecord(net->ev_desired_free, net->ctx.stream));
    return MYEA_OK;
  }
  LayerPlan &L = net->layers.back();
  const long long pitch = pitch_rows(net), rows = net->T * pitch;
  if (kind == cudaMemcpyHostToDevice) {
    // host targets: copy beside the forward pass still in flight on the main stream (the last use of d_desired by an
    // error kernel is behind ev_desired_free), and let the main stream wait for the copy only now
    CK(cudaStreamWaitEvent(net->copy_stream, net->ev_desired_free, 0));
    RC(copy_batch_in(net, net->d_desired, src, L.n_out, kind, net->copy_stream));
    CK(cudaEventRecord(net->ev_desired_ready, net->copy_stream));
    CK(cudaStreamWaitEvent(net->ctx.stream, net->ev_desired_ready, 0));
  } else {
    RC(copy_batch_in(net, net->d_desired, src, L.n_out, kind, net->ctx.stream));
  }
  // Recurrent networks only score the steps t >= number_time_delays; earlier steps get a zero error
  // (RNN__Compute__Error, Neural_Network__Recurrent_Compute__Error__OpenMP.cpp:22-159).
  const long long t0 = net->T > 1 ? std::min<long long>(static_cast<long long>(net->desc.number_time_delays), net->T) : 0;
  const float variance = net->desc.accuracy_variance > 0.f ? net->desc.accuracy_variance : 0.49f;
  if (net->active_B == pitch) {
    const long long skip = t0 * pitch;
    if (skip > 0) RC(fill_zero(net->ctx, L.errors, skip * L.n_out));
    if (rows > skip) {
      const size_t off = static_cast<size_t>(skip) * L.n_out;
      RC(output_error(net->ctx, L.summations + off, L.values + off, net->d_desired + off, L.errors + off, rows - skip, L.n_out,
                      L.desc.type_activation_function, net->desc.type_loss_function, net->desc.type_accuracy_function, variance,
                      net->d_loss_acc, net->d_loss_count));
    }
  } else {
    // short batch of a recurrent network: every time step scores its first active_B rows, all other rows carry no error
    RC(fill_zero(net->ctx, L.errors, rows * L.n_out));
    for (long long t = t0; t < net->T; ++t) {
      const size_t off = static_cast<size_t>(t * pitch) * L.n_out;
      RC(output_error(net->ctx, L.summations + off, L.values + off, net->d_desired + off, L.errors + off, net->active_B, L.n_out,
                      L.desc.type_activation_function, net->desc.type_loss_function, net->desc.type_accuracy_function, variance,
                      net->d_loss_acc, net->d_loss_count));
    }
  }
  CK(cudaEventRecord(net->ev_desired_free, net->ctx.stream));
  return MYEA_OK;
}

extern "C" int myea_b200_compute_error(myea_handle net, uint64_t batch, const float *desired) {
  return compute_error_impl(net, batch, desired, cudaMemcpyHostToDevice);
}
extern "C" int myea_b200_compute_error_device(myea_handle net, uint64_t batch, const float *desired) {
  return compute_error_impl(net, batch, desired, cudaMemcpyDeviceToDevice);
}

extern "C" int myea_b200_reset_loss(myea_handle net) {
  if (net == nullptr) return MYEA_E_INVALID;
  CK(cudaMemsetAsync(net->d_loss_acc, 0, 2 * sizeof(double), net->ctx.stream));
  CK(cudaMemsetAsync(net->d_loss_count, 0, sizeof(unsigned long long), net->ctx.stream));
  return MYEA_OK;
}

extern "C" int myea_b200_get_loss(myea_handle net, double *loss_sum, uint64_t *number_loss, double *accuracy_sum) {
  if (net == nullptr) return MYEA_E_INVALID;
  double acc[2] = {0, 0};
  unsigned long long cnt = 0;
  CK(cudaMemcpyAsync(acc, net->d_loss_acc, sizeof(acc), cudaMemcpyDeviceToHost, net->ctx.stream));
  CK(cudaMemcpyAsync(&cnt, net->d_loss_count, sizeof(cnt), cudaMemcpyDeviceToHost, net->ctx.stream));
  CK(cudaStreamSynchronize(net->ctx.stream));
  if (net->comm != nullptr) {  // Merge__Post__Training across ranks: every rank must call get_loss
    double all[3] = {acc[0], acc[1], static_cast<double>(cnt)};
    CK(cudaMemcpyAsync(net->d_loss_tmp, all, sizeof(all), cudaMemcpyHostToDevice, net->ctx.stream));
    RC(comm_all_reduce_sum_f64(net, net->d_loss_tmp, 3));
    CK(cudaMemcpyAsync(all, net->d_loss_tmp, sizeof(all), cudaMemcpyDeviceToHost, net->ctx.stream));
    CK(cudaStreamSynchronize(net->ctx.stream));
    acc[0] = all[0]; acc[1] = all[1]; cnt = static_cast<unsigned long long>(all[2] + 0.5);
  }
  if (loss_sum) *loss_sum = acc[0];
  if (accuracy_sum) *accuracy_sum = acc[1];
  if (number_loss) *number_loss = cnt;
  return MYEA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Backward pass: error propagation, last hidden layer -> first hidden layer
// FF__Backward_Pass_Batch (Neural_Network__Backward_Pass__OpenMP.cpp:24-155), RNN__ (…Recurrent_Backward_Pass__OpenMP.cpp:24-181)
// ---------------------------------------------------------------------------------------------------------
namespace myea {

// error arriving on layer `L`'s outputs from the fully connected layer `next`:  D = delta_next * W_next, with the
// activation derivative of L fused into the epilogue when L is fully connected (Backward_Pass__FC :1044-1082 followed
// by Backward_Pass__FC__DF :1225-1263), then the normalization backward (:1346-1709).
int fc_backward_from_fc(myea_b200_net *net, LayerPlan &L, const LayerPlan &next, const float *next_errors, long long rows,
                        float *dst, bool fuse_derivative) {
  Epilogue e;
  e.C = dst;
  e.ldc = next.n_in;
  L.bwd_fused_chunks = 0;
  if (fuse_derivative) {
    const uint32_t af = L.desc.type_activation_function;
    e.deriv_af = af;
    // the derivative of tanh / sigmoid is a function of the output alone, that of ReLU of the pre-activation alone
    // (Activation_Functions.hpp); an array the derivative does not read is not fetched
    const bool wants_pre = af_derive_reads_summation(af), wants_y = af_derive_reads_value(af);
    e.aux_pre = wants_pre ? L.summations : nullptr;
    e.aux_y = wants_y ? L.values : nullptr;
    e.ld_aux = L.n_out;
    if (L.has_norm) {
      if (wants_pre) { e.col_scale = L.norm.col_scale; e.col_shift = L.norm.col_shift; }
      // the sums of the normalization backward (error, error x centred summation) from the same epilogue
      Epilogue probe = e;
      probe.stats_kind = 2;
      probe.aux_pre = L.summations;
      probe.col_scale = L.norm.col_scale;
      probe.col_shift = L.norm.col_shift;
      probe.col_stats = L.norm.partial;
      probe.col_mean = L.norm.mean;
      probe.stats_blocks = (rows + 31) / 32;
      if (next_errors == next.errors && probe.stats_blocks <= L.norm.chunks && epilogue_takes_stats(net->ctx, probe, L.n_out)) {
        e = probe;
        L.bwd_fused_chunks = static_cast<int>(probe.stats_blocks);
      }
    }
  }
  if (next_errors != next.errors) {  // (not the case today) an error array other than the layer's own: no shared panels
    Operand a{next_errors, rows, next.n_out, next.n_out, 1};
    Operand b{net->params + next.idx.first_connection_index, next.n_in, next.n_out, 1, next.n_in};
    return gemm_nt(net->ctx, a, b, e, net->scratch);
  }
  return fc_product_backward(net, const_cast<LayerPlan &>(next), rows, e);
}

int fc_finish_backward(myea_b200_net *net, LayerPlan &L, long long rows) {
  if (!L.has_norm) return MYEA_OK;
  // the layer's errors are read next by the error propagation below it (rows) and by its weight derivative (columns),
  // both from shared operand panels: the kernel that writes the errors writes those panels as well
  PanelSink sink;
  // (the panel-writing kernel reads the layer's statistics eight columns at a time: they lie behind those of the
  // normalized layers before this one, whose unit counts need not be multiples of four - then the plain kernel runs and
  // the readers of the errors split them themselves, as the forward pass does with unaligned coefficients)
  const uintptr_t stat_bits = reinterpret_cast<uintptr_t>(L.norm.mean) | reinterpret_cast<uintptr_t>(L.norm.partial) |
                              reinterpret_cast<uintptr_t>(L.summations) | reinterpret_cast<uintptr_t>(L.deriv) | reinterpret_cast<uintptr_t>(L.errors);
  const bool use_sink = L.shared_panels && L.in_valid && net->ctx.gemm_engine == 0 && (rows & 7) == 0 && (L.n_out & 7) == 0 && (stat_bits & 15) == 0 &&
                        gemm_takes_mn_major(net->ctx, rows, L.n_out) && gemm_takes_mn_major(net->ctx, rows, L.n_in);
  if (use_sink) shared_panel_layout(L.d_panel_mem, rows, L.n_out, PANEL_ROLE_A, &L.d_rows, PANEL_ROLE_A, &L.d_cols, &sink);
  RC(norm_backward(net->ctx, L.summations, L.deriv, L.errors, rows, L.n_out, L.norm, &net->hook, L.bwd_fused_chunks, use_sink ? &sink : nullptr));
  L.bwd_fused_chunks = 0;
  if (use_sink) L.d_valid = true;
  return MYEA_OK;
}

}  // namespace myea

extern "C" int myea_b200_backward(myea_handle net, uint64_t batch) {
  if (net == nullptr) return MYEA_E_INVALID;
  RC(batch_in_flight(net, batch));
  if (!net->training) return fail(net, MYEA_E_INVALID, "can not back propagate in inference mode");
  CK(cudaSetDevice(net->ctx.device));
  RC(comm_gather_join(net));
  const long long rows = step_rows_total(net);
  const int n = static_cast<int>(net->layers.size());
  if (net->pre_training_level != 0) {  // the decoded layer's error reaches the coded layer and stops there
    int k = 0, dl = 0;
    RC(pre_training_layers(net, &k, &dl));
    LayerPlan &K = net->layers[k], &D = net->layers[dl];
    RC(fc_backward_from_fc(net, K, D, D.errors, rows, K.deriv, true));
    return fc_finish_backward(net, K, rows);
  }
  // `l` is a layer whose error is complete; send it to the layer feeding it, finish that layer, move down
  int l = n - 1;
  while (l >= 1) {
    LayerPlan &N = net->layers[l];
    if (N.type == MYEA_LAYER_RESIDUAL) {  // the block handles its own layers and the layer feeding it
      RC(residual_backward(net, l));
      l = N.input_layer;
      continue;
    }
    const int p = N.input_layer;
    if (p < 1) break;
    LayerPlan &P = net->layers[p];
    const bool n_pool = N.type == MYEA_LAYER_AVERAGE_POOLING || N.type == MYEA_LAYER_MAX_POOLING;
    // the error of N carried to the outputs of P, without P's activation derivative
    auto send_plain = [&](float *dst) -> int {
      if (N.type == MYEA_LAYER_FULLY_CONNECTED) return fc_backward_from_fc(net, P, N, N.errors, rows, dst, false);
      if (n_pool) return pooling_backward(net, N, dst, rows);
      return lstm_backward_to_input(net, N, dst, P, nullptr);
    };
    if (P.type == MYEA_LAYER_FULLY_CONNECTED) {
      if (P.ind_rnn) {
        // the error over all rows first, then backwards through time dAF_t = f'(pre_t) * (D_t + u * dAF_{t+1}), in place, and
        // the normalization backward of each step behind it
        RC(send_plain(P.deriv));
        const long long pitch = rows / net->T;
        const float *u = net->params + P.idx.first_connection_index + static_cast<uint64_t>(P.n_out) * P.n_in;
        for (long long t = net->T - 1; t >= 0; --t) {
          const long long off = t * pitch * P.n_out;
          RC(ind_rnn_backward_step(net->ctx, P.deriv + off, t + 1 < net->T ? P.deriv + off + pitch * P.n_out : nullptr, u, P.pre_af + off, P.values + off,
                                   pitch, P.n_out, P.desc.type_activation_function));
        }
        if (P.has_norm) {
          for (long long t = 0; t < net->T; ++t) {
            const NormParams np = norm_at_step(P, t);
            const long long off = t * pitch * P.n_out;
            RC(norm_backward(net->ctx, P.summations + off, P.deriv + off, P.errors + off, net->active_B, P.n_out, np, &net->hook, 0, nullptr));
          }
          if (net->active_B < pitch)
            CK(cudaMemset2DAsync(P.errors + net->active_B * P.n_out, pitch * P.n_out * sizeof(float), 0, (pitch - net->active_B) * P.n_out * sizeof(float),
                                 net->T, net->ctx.stream));
        }
        l = p;
        continue;
      }
      if (P.has_norm && net->T > 1) {
        // per-time-step normalization: the error over all rows first, then step by step the activation derivative on
        // that step's normalized summations and the normalization backward with that step's statistics
        RC(send_plain(P.deriv));
        const long long pitch = rows / net->T;
        for (long long t = 0; t < net->T; ++t) {
          const NormParams np = norm_at_step(P, t);
          const long long off = t * pitch * P.n_out;
          RC(activation_backward(net->ctx, P.deriv + off, P.summations + off, P.values + off, net->active_B, P.n_out, P.desc.type_activation_function,
                                 np.col_scale, np.col_shift));
          RC(norm_backward(net->ctx, P.summations + off, P.deriv + off, P.errors + off, net->active_B, P.n_out, np, &net->hook, 0, nullptr));
        }
        if (net->active_B < pitch)  // rows a short batch leaves unused carry no error
          CK(cudaMemset2DAsync(P.errors + net->active_B * P.n_out, pitch * P.n_out * sizeof(float), 0, (pitch - net->active_B) * P.n_out * sizeof(float),
                               net->T, net->ctx.stream));
        l = p;
        continue;
      }
      if (N.type == MYEA_LAYER_FULLY_CONNECTED) {
        RC(fc_backward_from_fc(net, P, N, N.errors, rows, P.deriv, true));
      } else if (n_pool) {  // a pooling layer above: its backward pass has no epilogue to carry P's activation derivative
        P.bwd_fused_chunks = 0;
        RC(pooling_backward(net, N, P.deriv, rows));
        RC(activation_backward(net->ctx, P.deriv, P.summations, P.values, rows, P.n_out, P.desc.type_activation_function,
                               P.has_norm ? P.norm.col_scale : nullptr, P.has_norm ? P.norm.col_shift : nullptr));
      } else {  // an LSTM layer above: its input contraction carries P's activation derivative in the epilogue
        Epilogue fin;
        const uint32_t af = P.desc.type_activation_function;
        fin.deriv_af = af;
        fin.aux_pre = af_derive_reads_summation(af) ? P.summations : nullptr;
        fin.aux_y = af_derive_reads_value(af) ? P.values : nullptr;
        fin.ld_aux = P.n_out;
        P.bwd_fused_chunks = 0;
        RC(lstm_backward_to_input(net, N, P.deriv, P, &fin));
      }
      RC(fc_finish_backward(net, P, rows));
    } else if (P.type == MYEA_LAYER_LSTM) {
      RC(send_plain(lstm_output_errors(P)));
      RC(lstm_backward(net, P));
    } else if (P.type == MYEA_LAYER_AVERAGE_POOLING || P.type == MYEA_LAYER_MAX_POOLING) {
      RC(send_plain(P.deriv));  // P.errors == P.deriv: nothing of its own to finish
    } else {  // residual block feeding N: its output has no activation of its own
      if (N.type != MYEA_LAYER_FULLY_CONNECTED) return fail(net, MYEA_E_UNSUPPORTED, "a residual block below an LSTM or pooling layer is not built");
      RC(fc_backward_from_fc(net, P, N, N.errors, rows, P.deriv, false));
    }
    l = p;
  }
  return MYEA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Derivative-weight accumulation
// Update_Derivative_Weight__FC (Neural_Network__Update_Derivative_Weight__OpenMP.cpp:178-216) + bias (:218-242)
// ---------------------------------------------------------------------------------------------------------
namespace myea {
int fc_update_derivative_weight(myea_b200_net *net, LayerPlan &L, const float *input, long long rows) {
  Operand a{L.errors, L.n_out, rows, 1, L.n_out};  // delta^T: [out rows, K = batch]
  Operand b{input, L.n_in, rows, 1, L.n_in};       // input^T: [in rows, K = batch]
  Epilogue e;
  e.C = net->grads + L.idx.first_connection_index;
  e.ldc = L.n_in;
  e.accumulate = 1;
  if (L.shared_panels && L.in_valid && input == L.in_src) {
    if (!L.d_valid) {  // no error propagation below this layer (first hidden layer): only the column reading is needed
      RC(gemm_prepare_shared(net->ctx, L.errors, L.n_out, rows, L.n_out, L.d_panel_mem, PANEL_ROLE_A, nullptr, PANEL_ROLE_A, &L.d_cols));
    }
    RC(gemm_panels(net->ctx, L.d_cols, 0, L.n_out, L.in_cols, 0, L.n_in, e));
    L.d_valid = false;  // the errors of the next step will differ
  } else {
    RC(gemm_nt(net->ctx, a, b, e, net->scratch));
  }
  if (L.use_bias)
    RC(column_sum(net->ctx, L.errors, rows, L.n_out, net->grads + L.idx.first_bias_connection_index, 1, net->reduce_partial, net->reduce_chunks));
  return MYEA_OK;
}
}  // namespace myea

extern "C" int myea_b200_update_derivative_weight(myea_handle net, uint64_t batch) {
  if (net == nullptr) return MYEA_E_INVALID;
  RC(batch_in_flight(net, batch));
  CK(cudaSetDevice(net->ctx.device));
  const long long rows = step_rows_total(net);
  if (net->comm != nullptr && net->grads_reduced)
    return fail(net, MYEA_E_UNSUPPORTED, "with a communicator attached, call update_parameter after every update_derivative_weight (the derivative buckets of this step were already summed over the ranks)");
  // Reduce-scatter instead of all-reduce where the update works on slices: not under the max-norm constraint (whole
  // rows), which the last update's description announced
  comm_set_scatter(net, net->comm != nullptr && net->sharded_update);
  if (net->pre_training_level != 0) {  // the two layers of the pair only
    int k = 0, dl = 0;
    RC(pre_training_layers(net, &k, &dl));
    LayerPlan &K = net->layers[k], &D = net->layers[dl];
    RC(fc_update_derivative_weight(net, D, K.values, rows));
    return fc_update_derivative_weight(net, K, net->layers[K.input_layer].values, rows);
  }
  // Every layer's error is known by now, so the order is free.  One GPU: last layer first.  Data parallel: FIRST layer
  // first - its bucket is then the first to be summed, updated and gathered, and the next forward pass, which waits
  // for each layer's gather only where it reads that layer, finds the lower layers' parameters in place while the
  // upper layers' are still travelling.
  const int n_layers = static_cast<int>(net->layers.size());
  for (int step = 1; step < n_layers; ++step) {
    const int l = net->comm != nullptr ? step : n_layers - step;
    LayerPlan &L = net->layers[l];
    if (L.type == MYEA_LAYER_FULLY_CONNECTED) {
      const float *input = net->layers[L.input_layer].values;
      int blk = 0;
      if (layer_in_block(net, l, &blk)) input = residual_fc_input(net, blk, l - blk);  // normalized / activated copy kept by the block
      RC(fc_update_derivative_weight(net, L, input, rows));
      if (L.ind_rnn && net->T > 1) {
        // recurrent weights: dAF of step t with the output of step t - 1 (the pre-activation buffer is free by now and
        // holds the products)
        const long long pitch = rows / net->T;
        RC(ind_rnn_recurrent_derivative(net->ctx, L.deriv, L.values, (net->T - 1) * pitch, L.n_out, pitch, L.pre_af,
                                        net->grads + L.idx.first_connection_index + static_cast<uint64_t>(L.n_out) * L.n_in, net->reduce_partial,
                                        net->reduce_chunks));
      }
    } else if (L.type == MYEA_LAYER_LSTM) {
      RC(lstm_update_derivative_weight(net, L, net->layers[L.input_layer].values, L.n_in));
    }
    if (net->comm != nullptr && L.idx.last_connection_index > L.idx.first_connection_index)
      RC(comm_reduce_bucket_async(net, L.idx.first_connection_index, L.idx.last_connection_index - L.idx.first_connection_index));
  }
  if (net->comm != nullptr) {  // biases and normalization scales / shifts: one last bucket behind the weights
    RC(comm_reduce_bucket_async(net, net->total_weights, net->total_parameters - net->total_weights));
    net->grads_reduced = true;
  }
  return MYEA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Parameter update: merge across GPUs, clip, optimizer, zero the derivatives
// Update_Parameter (Neural_Network.cpp:4719-4900)
// ---------------------------------------------------------------------------------------------------------
extern "C" int myea_b200_update_parameter(myea_handle net, uint64_t batch, uint64_t training_size, const myea_opt_desc *opt) {
  if (net == nullptr || opt == nullptr || training_size == 0) return MYEA_E_INVALID;
  CK(cudaSetDevice(net->ctx.device));
  RC(comm_gather_join(net));
  const size_t P = net->total_parameters;
  // The update is element by element, so each derivative bucket can be applied as soon as ITS sum over the ranks has
  // arrived, while the later buckets are still on the wire - and only on this rank's slice of it where the bucket was
  // reduce-scattered.  A global-norm clip works on slices too (every rank squares what it holds and the sums are added
  // over the ranks) but has to see every bucket before the first update; the max-norm constraint needs whole rows.
  const bool needs_whole = opt->regularization__max_norm_constraints != 0.f;
  net->sharded_update = !needs_whole;  // what the NEXT step's buckets may assume
  bool by_bucket = net->comm != nullptr && net->grads_reduced && !needs_whole && comm_bucket_count(net) > 0 && (net->total_weights & 3) == 0;
  for (const auto &L : net->layers)  // the update kernel reads float4: every bucket has to start on a 16-byte boundary
    if (L.type != MYEA_LAYER_RESIDUAL && (L.idx.first_connection_index & 3) != 0) by_bucket = false;
  if (net->comm != nullptr && !by_bucket) {
    // slices that were reduce-scattered for an update that now wants whole buffers: gather them first
    if (net->grads_reduced && comm_any_scattered(net)) RC(comm_unscatter(net));
    if (net->grads_reduced) RC(comm_join(net));            // buckets issued by update_derivative_weight
    else RC(comm_all_reduce_sum(net, net->grads, P));      // nothing was issued: reduce everything now
    net->grads_reduced = false;
  }
  for (auto &L : net->layers) L.w_valid = false;  // the weights change below
  OptLaunch o;
  o.type = opt->type_optimizer_function;
  struct ReadyBucket { size_t i, n, off, slice; };
  std::vector<ReadyBucket> ready;  // buckets whose sums were waited for ahead of the update loop (clip only)
  if (opt->use_clip_gradient) {
    if (by_bucket) {
      // the norm needs every bucket's sum before the first update: a reduce-scattered bucket contributes this rank's
      // slice, an all-reduced one (every rank holds all of it) is counted by rank 0 alone
      CK(cudaMemsetAsync(net->d_sumsq, 0, sizeof(double), net->ctx.stream));
      const size_t count = comm_bucket_count(net);
      for (size_t k = 0; k < count; ++k) {
        ReadyBucket b{k == 0 ? count - 1 : k - 1, 0, 0, 0};
        size_t bucket_off = 0;
        RC(comm_bucket_wait(net, b.i, &bucket_off, &b.n, &b.off, &b.slice));
        if (b.slice != b.n || comm_rank(net) == 0) RC(sum_squares(net->ctx, net->grads + b.off, b.slice, net->d_sumsq, true));
        ready.push_back(b);
      }
      RC(comm_all_reduce_sum_f64(net, net->d_sumsq, 1));
    } else {
      RC(sum_squares(net->ctx, net->grads, P, net->d_sumsq));
    }
    RC(clip_scale_from_norm(net->ctx, net->d_sumsq, opt->clip_gradient, net->d_clip_scale));
    o.clip_scale = net->d_clip_scale;
  }
  net->optimizer_time_step += 1.f;
  const float t = net->optimizer_time_step;
  // decoupled weight decay, "normalized" by default (Train.cpp:284-286); fp32 arithmetic as the reference
  float wd = opt->regularization__weight_decay;
  if (wd != 0.f && opt->use_normalized_weight_decay)
    wd = wd * sqrtf(static_cast<float>(batch) / (static_cast<float>(training_size) * (opt->epoch_time_step > 0.f ? opt->epoch_time_step : 1.f)));
  o.weight_decay = wd;
  switch (o.type) {
    case MYEA_OPT_ADAM:
    case MYEA_OPT_AMSGRAD:
    case MYEA_OPT_ADABOUND:
    case MYEA_OPT_AMSBOUND: {
      o.beta1 = opt->adam_beta1;
      o.beta2 = opt->adam_beta2;
      o.epsilon = opt->adam_epsilon;
      const float lr = opt->adam_learning_rate;
      o.lr_t = opt->use_adam_bias_correction ? lr * sqrtf(1.f - powf(o.beta2, t)) / (1.f - powf(o.beta1, t)) : lr;
      o.lower = opt->learning_rate_final * (1.f - 1.f / (opt->learning_gamma * t + 1.f));
      o.upper = opt->learning_rate_final * (1.f + 1.f / (opt->learning_gamma * t));
      break;
    }
    case MYEA_OPT_NOSADAM: {
      // Adam whose second-moment decay changes with time (Neural_Network__NosAdam.cpp:97-160): the bias correction keeps
      // using the fixed adam_beta2; the running sum B lives on the handle like adam_previous_beta2 on the reference object
      const float gamma = opt->adam_gamma > 0.f ? opt->adam_gamma : 0.1f;
      const float pw = powf(t, -gamma);
      o.type = MYEA_OPT_ADAM;
      o.beta1 = opt->adam_beta1;
      o.beta2 = net->nosadam_previous_beta2 / (net->nosadam_previous_beta2 + pw);
      o.epsilon = opt->adam_epsilon;
      const float lr = opt->adam_learning_rate;
      o.lr_t = opt->use_adam_bias_correction ? lr * sqrtf(1.f - powf(opt->adam_beta2, t)) / (1.f - powf(opt->adam_beta1, t)) : lr;
      net->nosadam_previous_beta2 += pw;
      break;
    }
    case MYEA_OPT_GD:
      o.gd_lr = opt->learning_rate;
      o.momentum = opt->learning_momentum;
      o.nesterov = opt->use_nesterov != 0;
      break;
    case MYEA_OPT_IRPROP_PLUS:
      o.weight_decay = 0.f;
      o.rprop_increase = opt->rprop_increase_factor > 0.f ? opt->rprop_increase_factor : 1.2f;
      o.rprop_decrease = opt->rprop_decrease_factor > 0.f ? opt->rprop_decrease_factor : 0.5f;
      o.rprop_min = opt->rprop_delta_min > 0.f ? opt->rprop_delta_min : 1e-6f;
      o.rprop_max = opt->rprop_delta_max > 0.f ? opt->rprop_delta_max : 50.f;
      o.rprop_zero = opt->rprop_delta_zero > 0.f ? opt->rprop_delta_zero : 0.1f;
      o.rprop_error_is_worse = opt->loss_rprop > opt->previous_loss_rprop ? 1 : 0;
      break;
    default: return fail(net, MYEA_E_UNSUPPORTED, "optimizer not built (Adam, AMSGrad, NosAdam, AdaBound, AMSBound, gradient descent / momentum / Nesterov, iRPROP+)");
  }
  const float max_norm = opt->regularization__max_norm_constraints;
  if (by_bucket) {
    const size_t count = comm_bucket_count(net);
    size_t covered = 0;
    // the bucket of the biases and normalization parameters was issued last but is gathered first: the next forward
    // pass reads it before anything else
    for (size_t k = 0; k < count; ++k) {
      size_t i = k == 0 ? count - 1 : k - 1;
      size_t bucket_off = 0, n = 0, off = 0, slice = 0;
      if (!ready.empty()) { i = ready[k].i; n = ready[k].n; off = ready[k].off; slice = ready[k].slice; }
      else RC(comm_bucket_wait(net, i, &bucket_off, &n, &off, &slice));
      if ((off & 3) != 0) return fail(net, MYEA_E_INVALID, "derivative bucket does not start on a 16-byte boundary");
      RC(optimizer_update(net->ctx, o, net->params + off, net->grads + off, net->m1 + off, net->m2 + off, net->m2hat + off, net->prev_delta + off,
                          net->mask_reg + off, slice));
      RC(comm_bucket_gather(net, i));  // the other ranks' slices of the updated parameters (nothing for an all-reduced bucket)
      covered += n;
    }
    comm_buckets_done(net);  // the gathers stay open: the next reader of the parameters waits for them
    net->grads_reduced = false;
    if (covered != P) return fail(net, MYEA_E_INVALID, "derivative buckets do not cover the parameter buffer");
  } else {
    RC(optimizer_update(net->ctx, o, net->params, net->grads, net->m1, net->m2, net->m2hat, net->prev_delta, net->mask_reg, P));
  }
  // independently recurrent layers keep their recurrent weights inside their bound (Update_Parameter: Use__Regularization__Constraint_Recurrent_Weight)
  for (const auto &L : net->layers)
    if (L.ind_rnn)
      RC(ind_rnn_clamp(net->ctx, net->params + L.idx.first_connection_index + static_cast<uint64_t>(L.n_out) * L.n_in, L.n_out,
                       ind_rnn_weight_bound(net->desc.clip_gradient, L.desc.type_activation_function, net->T)));
  if (max_norm != 0.f) {
    // Update_Weight_Regularization__Max_Norm_Constraints__Neurons (…Max_Norm_Constraints.cpp:147-165): one weight row per neuron
    for (const auto &L : net->layers)
      if (L.type == MYEA_LAYER_FULLY_CONNECTED) RC(row_max_norm(net->ctx, net->params + L.idx.first_connection_index, L.n_out, L.n_in, max_norm));
    for (const auto &L : net->layers)
      if (L.type == MYEA_LAYER_LSTM) {
        const long long dirs = L.desc.use_bidirectional ? 2 : 1, cpb = std::max<long long>(1, static_cast<long long>(L.desc.unit_parameters[1]));
        RC(lstm_max_norm(net->ctx, net->params, static_cast<long long>(L.idx.first_connection_index), static_cast<long long>(L.desc.unit_parameters[0]) * dirs,
                         static_cast<long long>(L.idx.block_stride), L.n_in, L.n_out / dirs, cpb, max_norm));
      }
  }
  return MYEA_OK;
}

extern "C" int myea_b200_clear_training_arrays(myea_handle net) {
  if (net == nullptr) return MYEA_E_INVALID;
  const size_t bytes = (net->total_parameters + 4) * sizeof(float);
  CK(cudaMemsetAsync(net->grads, 0, bytes, net->ctx.stream));
  CK(cudaMemsetAsync(net->m1, 0, bytes, net->ctx.stream));
  CK(cudaMemsetAsync(net->m2, 0, bytes, net->ctx.stream));
  CK(cudaMemsetAsync(net->m2hat, 0, bytes, net->ctx.stream));
  CK(cudaMemsetAsync(net->prev_delta, 0, bytes, net->ctx.stream));
  net->optimizer_time_step = 0.f;
  net->nosadam_previous_beta2 = 0.f;
  return MYEA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Read-back helpers, synchronisation, profiling
// ---------------------------------------------------------------------------------------------------------
// rows of the step in flight, packed [T][active_B][units] for the caller (the device pitch is the allocated B when
// the network is recurrent)
static int copy_out(myea_b200_net *net, const float *src, long long units, float *host, uint64_t count) {
  const long long pitch = pitch_rows(net), b = net->active_B;
  if (src == nullptr || count > static_cast<uint64_t>(net->T * b * units)) return fail(net, MYEA_E_INVALID, "layer has no such buffer, or count too large");
  if (b == pitch) {
    CK(cudaMemcpyAsync(host, src, count * sizeof(float), cudaMemcpyDeviceToHost, net->ctx.stream));
  } else {
    const uint64_t per_step = static_cast<uint64_t>(b * units);
    for (uint64_t t = 0; t * per_step < count; ++t)
      CK(cudaMemcpyAsync(host + t * per_step, src + t * pitch * units, std::min<uint64_t>(per_step, count - t * per_step) * sizeof(float),
                         cudaMemcpyDeviceToHost, net->ctx.stream));
  }
  CK(cudaStreamSynchronize(net->ctx.stream));
  return MYEA_OK;
}

extern "C" int myea_b200_get_outputs(myea_handle net, uint32_t layer, float *host, uint64_t count) {
  if (net == nullptr || host == nullptr || layer >= net->layers.size()) return MYEA_E_INVALID;
  LayerPlan &L = net->layers[layer];
  return copy_out(net, L.values, L.n_out, host, count);
}

extern "C" int myea_b200_get_errors(myea_handle net, uint32_t layer, float *host, uint64_t count) {
  if (net == nullptr || host == nullptr || layer >= net->layers.size() || layer == 0) return MYEA_E_INVALID;
  LayerPlan &L = net->layers[layer];
  const float *src = L.type == MYEA_LAYER_LSTM ? lstm_output_errors(L) : L.errors;
  return copy_out(net, src, L.n_out, host, count);
}

extern "C" int myea_b200_synchronize(myea_handle net) {
  if (net == nullptr) return MYEA_E_INVALID;
  CK(cudaSetDevice(net->ctx.device));
  int flag = 0;
  RC(comm_gather_join(net));
  CK(cudaMemcpyAsync(&flag, net->ctx.d_error_flag, sizeof(int), cudaMemcpyDeviceToHost, net->ctx.stream));
  CK(cudaStreamSynchronize(net->ctx.stream));
  if (flag != 0) {
    char msg[96];
    snprintf(msg, sizeof(msg), "a kernel gave up a bounded wait (code %d)", flag);
    return fail(net, MYEA_E_KERNEL, msg);
  }
  return MYEA_OK;
}

extern "C" void *myea_b200_stream(myea_handle net) { return net ? net->ctx.stream : nullptr; }
extern "C" uint64_t myea_b200_kernel_launches(myea_handle net) { return net ? net->ctx.launches : 0; }

extern "C" int myea_b200_profile(myea_handle net, int enable) {
  if (net == nullptr) return MYEA_E_INVALID;
  net->ctx.profiling = enable != 0;
  return MYEA_OK;
}

extern "C" int myea_b200_profile_read(myea_handle net, double ms[MYEA_TIMER_CLASSES], uint64_t launches[MYEA_TIMER_CLASSES],
                                      double gemm_flops[1], int reset) {
  if (net == nullptr) return MYEA_E_INVALID;
  for (int i = 0; i < MYEA_TIMER_CLASSES; ++i) {
    if (ms) ms[i] = net->ctx.class_ms[i];
    if (launches) launches[i] = net->ctx.class_launches[i];
  }
  if (gemm_flops) gemm_flops[0] = net->ctx.gemm_flops;
  if (reset) {
    for (int i = 0; i < MYEA_TIMER_CLASSES; ++i) { net->ctx.class_ms[i] = 0; net->ctx.class_launches[i] = 0; }
    net->ctx.gemm_flops = 0;
  }
  return MYEA_OK;
}
