// Test infrastructure, not product code.
//
// C-ABI driver around the UNMODIFIED reference `class Neural_Network` (compiled from the reference checkout by
// oracle/build_ref.sh).  It takes the same descriptors as the product library (include/myea_b200.h) and mirrors
// its entry points one to one, so a parity test builds the same network on both sides, feeds both the same
// weights / masks / inputs and compares buffers.  Only tests, smoke() and the CPU-baseline leg of bench.py load it.
//
// Call order inside ref_create follows what the reference's own harness does
// (Neural_Network_Launcher_Windows/Source_Files/debug.cpp:1145-1480): Compile, activation functions, loss /
// accuracy / optimizer, batch size, normalization, dropout, weight decay, clip.  Parameters are left as Compile
// allocated them (zero); the caller writes them through ref_buffer().  The reference's own initializers are never
// called on LSTM networks: Initialize__Constant__LSTM__Bias (Neural_Network.cpp:5090-5111) writes past the
// parameter buffer.
#include "stdafx.hpp"
#include "myea_b200.h"

#include <omp.h>
#include <chrono>
#include <cstring>
#include <vector>

using namespace MyEA::Common;

namespace {
struct RefNet {
  Neural_Network nn;
  myea_net_desc desc;
  int threads = 1;
  size_t n_inputs = 0, n_outputs = 0, T = 1;
  std::vector<std::vector<T_>> xrows, yrows;   // T_ is the reference's scalar: float, or double in the COMPILE_DOUBLE build
  std::vector<const T_ *> xptr, yptr;
};

void apply_opt(Neural_Network &nn, const myea_opt_desc &o) {
  nn.learning_rate = o.learning_rate;
  nn.learning_momentum = o.learning_momentum;
  nn.use_Nesterov = o.use_nesterov != 0;
  nn.adam_learning_rate = o.adam_learning_rate;
  nn.adam_beta1 = o.adam_beta1;
  nn.adam_beta2 = o.adam_beta2;
  nn.adam_epsilon = o.adam_epsilon;
  nn.learning_rate_final = o.learning_rate_final;
  nn.learning_gamma = o.learning_gamma;
  nn.use_adam_bias_correction = o.use_adam_bias_correction != 0;
  nn.use_normalized_weight_decay = o.use_normalized_weight_decay != 0;
  nn.epoch_time_step = o.epoch_time_step;
  if (o.adam_gamma > 0.f) nn.adam_gamma = o.adam_gamma;
  nn.Set__Regularization__Max_Norm_Constraints(o.regularization__max_norm_constraints);
  nn.Set__Regularization__L1(o.regularization__l1);
  nn.Set__Regularization__L2(o.regularization__l2);
  if (o.rprop_increase_factor > 0.f) nn.rprop_increase_factor = o.rprop_increase_factor;
  if (o.rprop_decrease_factor > 0.f) nn.rprop_decrease_factor = o.rprop_decrease_factor;
  if (o.rprop_delta_min > 0.f) nn.rprop_delta_min = o.rprop_delta_min;
  if (o.rprop_delta_max > 0.f) nn.rprop_delta_max = o.rprop_delta_max;
  if (o.rprop_delta_zero > 0.f) nn.rprop_delta_zero = o.rprop_delta_zero;
  if (o.type_optimizer_function == MYEA_OPT_IRPROP_PLUS) {
    nn.loss_rprop = o.loss_rprop;
    nn.previous_loss_rprop = o.previous_loss_rprop;
  }
}

// [T][B][W] packed block -> one contiguous [T*W] row per sample (Neural_Network__Assign_Inputs.cpp:273-304).
void unpack_rows(const float *tbw, size_t T, size_t B, size_t W, std::vector<std::vector<T_>> &rows,
                 std::vector<const T_ *> &ptrs) {
  rows.resize(B);
  ptrs.resize(B);
  for (size_t b = 0; b < B; ++b) {
    rows[b].resize(T * W);
    for (size_t t = 0; t < T; ++t)
      for (size_t j = 0; j < W; ++j) rows[b][t * W + j] = static_cast<T_>(tbw[(t * B + b) * W + j]);
    ptrs[b] = rows[b].data();
  }
}
}  // namespace

extern "C" {

void *ref_create(const myea_net_desc *d, const myea_opt_desc *opt, int threads) {
  if (d == nullptr || d->number_layers < 2 || d->number_layers > MYEA_MAX_LAYERS) return nullptr;
  RefNet *r = new RefNet();
  r->desc = *d;
  r->threads = threads < 1 ? 1 : threads;
  r->T = d->number_recurrent_depth;
  std::vector<Layer_Parameters> lp(d->number_layers);
  for (uint32_t i = 0; i < d->number_layers; ++i) {
    lp[i].type_layer = static_cast<ENUM_TYPE_LAYER>(d->layers[i].type_layer);
    lp[i].use_bidirectional = d->layers[i].use_bidirectional != 0;
    for (int k = 0; k < 5; ++k) lp[i].unit_parameters[k] = d->layers[i].unit_parameters[k];
  }
  Neural_Network &nn = r->nn;
  if (!nn.Compile(d->number_layers, d->number_recurrent_depth, static_cast<ENUM_TYPE_NETWORKS>(d->type_network),
                  lp.data(), size_t(1) << 40)) {
    delete r;
    return nullptr;
  }
  if (d->number_recurrent_depth > 1) nn.Set__Number_Time_Delays(d->number_time_delays);
  for (uint32_t i = 1; i < d->number_layers; ++i) {
    const myea_layer_desc &L = d->layers[i];
    if ((L.type_layer == MYEA_LAYER_FULLY_CONNECTED || L.type_layer == MYEA_LAYER_FC_INDEPENDENTLY_RECURRENT) && L.type_activation_function != 0)
      nn.Set__Layer_Activation_Function(i, static_cast<ENUM_TYPE_ACTIVATION_FUNCTION>(L.type_activation_function));
  }
  nn.Set__Loss_Function(static_cast<ENUM_TYPE_LOSS_FUNCTIONS>(d->type_loss_function));
  nn.Set__Accuracy_Function(static_cast<ENUM_TYPE_ACCURACY_FUNCTIONS>(d->type_accuracy_function));
  if (d->accuracy_variance > 0.f) nn.Set__Accurancy_Variance(d->accuracy_variance);
  if (opt != nullptr) {
    nn.Set__Optimizer_Function(static_cast<ENUM_TYPE_OPTIMIZER_FUNCTIONS>(opt->type_optimizer_function));
    apply_opt(nn, *opt);
  }
  if (r->threads > 1) {
    nn.Set__OpenMP(true);
    nn.Set__Maximum_Thread_Usage(100.0);
  }
  if (!nn.Update__Batch_Size(d->batch_size)) { delete r; return nullptr; }
  if (nn.batch_size != d->batch_size) {  // the memory limit silently shrank the batch: BN statistics would change
    delete r;
    return nullptr;
  }
  if (r->threads > 1) {
    nn.Update__Thread_Size(r->threads);
    omp_set_num_threads(static_cast<int>(nn.number_threads));
    r->threads = static_cast<int>(nn.number_threads);
  }
  bool ok = true;
  for (uint32_t i = 1; i < d->number_layers; ++i) {
    const myea_layer_desc &L = d->layers[i];
    if (L.type_normalization != MYEA_NORM_NONE) {
      ok = ok && nn.Set__Layer_Normalization(i, static_cast<ENUM_TYPE_LAYER_NORMALIZATION>(L.type_normalization));
      nn.ptr_array_layers[i].use_layer_normalization_before_activation = L.use_layer_normalization_before_activation != 0;
    }
  }
  if (d->normalization_momentum_average > 0.f) nn.Set__Normalization_Momentum_Average(d->normalization_momentum_average);
  if (d->normalization_epsilon > 0.f) nn.Set__Normalization_Epsilon(d->normalization_epsilon);
  if (d->batch_renormalization_r_correction_maximum > 0.f)
    nn.Set__Batch_Renormalization_r_Correction_Maximum(d->batch_renormalization_r_correction_maximum);
  if (d->batch_renormalization_d_correction_maximum > 0.f)
    nn.Set__Batch_Renormalization_d_Correction_Maximum(d->batch_renormalization_d_correction_maximum);
  for (uint32_t i = 1; i < d->number_layers; ++i) {
    const myea_layer_desc &L = d->layers[i];
    if (L.type_dropout != MYEA_DROPOUT_NONE) {
      const T_ values[3] = {static_cast<T_>(L.dropout_values[0]), static_cast<T_>(L.dropout_values[1]), static_cast<T_>(L.dropout_values[2])};
      ok = ok && nn.Set__Dropout(i, static_cast<ENUM_TYPE_LAYER_DROPOUT>(L.type_dropout), values, false);
    }
  }
  if (opt != nullptr) {
    if (opt->regularization__weight_decay != 0.f) ok = ok && nn.Set__Regularization__Weight_Decay(opt->regularization__weight_decay);
    if (opt->use_clip_gradient) {
      nn.Set__Clip_Gradient(true);
      nn.Set__Clip_Gradient(opt->clip_gradient);
    }
  }
  if (!ok) { delete r; return nullptr; }
  // The reference seeds its ShakeDrop generators from the clock (Neural_Network__Allocate.cpp:296, :314).  Seed them
  // through their public Seed() instead, so that a test sees the same draws on every run (an activation kink that a
  // particular draw happens to put within rounding distance of zero would otherwise fail one run in ten).
  if (nn.ptr_array_Class_Generator_Bernoulli_ShakeDrop != nullptr && nn.ptr_array_Class_Generator_Real_ShakeDrop != nullptr) {
    for (size_t g = 0; g < nn.number_threads; ++g) {
      nn.ptr_array_Class_Generator_Bernoulli_ShakeDrop[g].Seed(5413u + static_cast<unsigned int>(g));
      nn.ptr_array_Class_Generator_Real_ShakeDrop[g].Seed(7919u + static_cast<unsigned int>(g));
    }
  }
  r->n_inputs = nn.number_inputs;
  r->n_outputs = nn.number_outputs;
  nn.type_state_propagation = ENUM_TYPE_STATE_PROPAGATION::TYPE_STATE_PROPAGATION_TRAINING;
  nn.Clear_Training_Arrays();
  return r;
}

void ref_destroy(void *h) { delete static_cast<RefNet *>(h); }

// Set__Pre_Training_Level (Neural_Network__Indexing.cpp:20-51): 0 = the whole network, k >= 1 = train the k-th layer pair
// of an autoencoder (hidden layer k and its mirror image)
int ref_set_pre_training_level(void *h, uint64_t level) {
  return static_cast<RefNet *>(h)->nn.Set__Pre_Training_Level(level) ? 0 : -1;
}

// bytes of the reference's scalar type in this build: 4 (float) or 8 (COMPILE_DOUBLE); buffers, outputs and errors
// cross this interface in that type, inputs and targets always arrive as float
int ref_scalar_bytes(void) { return static_cast<int>(sizeof(T_)); }

int ref_threads(void *h) { return static_cast<RefNet *>(h)->threads; }

int ref_sizes(void *h, uint64_t *P, uint64_t *W, uint64_t *bias, uint64_t *norm_units) {
  Neural_Network &nn = static_cast<RefNet *>(h)->nn;
  *P = nn.total_parameters;
  *W = nn.total_weights;
  *bias = nn.total_bias;
  *norm_units = nn.total_normalized_units;
  return 0;
}

int ref_layer_index(void *h, uint32_t layer, myea_layer_index *out) {
  Neural_Network &nn = static_cast<RefNet *>(h)->nn;
  if (layer >= nn.total_layers) return -1;
  Layer *L = nn.ptr_array_layers + layer;
  std::memset(out, 0, sizeof(*out));
  if (layer > 0 && L->type_layer != ENUM_TYPE_LAYER::TYPE_LAYER_RESIDUAL) {
    out->first_connection_index = *L->ptr_first_connection_index;
    out->last_connection_index = *L->ptr_last_connection_index;
    out->first_bias_connection_index = L->first_bias_connection_index;
    out->last_bias_connection_index = L->last_bias_connection_index;
  }
  out->number_outputs = *L->ptr_number_outputs;
  if (L->type_layer == ENUM_TYPE_LAYER::TYPE_LAYER_LSTM) {
    Block_unit *b = L->ptr_array_block_units;
    out->block_stride = b->last_index_connection - b->first_index_connection;
    out->number_inputs = b->last_index_feedforward_connection_input_gate - b->first_index_feedforward_connection_input_gate;
  } else if (layer > 0 && (L->type_layer == ENUM_TYPE_LAYER::TYPE_LAYER_FULLY_CONNECTED ||
                           L->type_layer == ENUM_TYPE_LAYER::TYPE_LAYER_FULLY_CONNECTED_INDEPENDENTLY_RECURRENT)) {
    out->number_inputs = *L->ptr_array_neuron_units->ptr_number_connections;
  }
  if (nn.total_normalized_units != 0 && L->ptr_array_normalized_units != nullptr) {
    out->scale_index = L->ptr_array_normalized_units->normalized_batch_units.ptr_scale - nn.ptr_array_parameters;
    out->shift_index = L->ptr_array_normalized_units->normalized_batch_units.ptr_shift - nn.ptr_array_parameters;
    out->number_units_norm = L->ptr_last_normalized_unit - L->ptr_array_normalized_units;
  }
  return 0;
}

T_ *ref_buffer(void *h, int which) {
  Neural_Network &nn = static_cast<RefNet *>(h)->nn;
  switch (which) {
    case MYEA_BUF_PARAMETERS: return nn.ptr_array_parameters;
    case MYEA_BUF_DERIVATIVES: return nn.ptr_array_derivatives_parameters;
    case MYEA_BUF_FIRST_MOMENT: return nn.ptr_array_previous_biased_first_moment;
    case MYEA_BUF_SECOND_MOMENT: return nn.ptr_array_previous_biased_second_moment;
    case MYEA_BUF_SECOND_MOMENT_HAT: return nn.ptr_array_previous_biased_second_moment_hat;
    case MYEA_BUF_MASK_REGULARIZED: return nn.ptr_array_mask_regularized_parameters;
    case MYEA_BUF_NORM_MEAN_AVERAGE: return nn.ptr_array_normalized_batch_units_means_averages;
    case MYEA_BUF_NORM_VARIANCE_AVERAGE: return nn.ptr_array_normalized_batch_units_variances_averages;
    case MYEA_BUF_PREVIOUS_DELTA: return nn.ptr_array_previous_delta_parameters;
    case MYEA_BUF_PREVIOUS_DERIVATIVES: return nn.ptr_array_previous_derivatives_parameters;
    case MYEA_BUF_PREVIOUS_STEPS: return nn.ptr_array_previous_steps;
    default: return nullptr;
  }
}

int ref_set_mask_bernoulli(void *h, uint32_t layer, const uint8_t *mask, uint64_t count) {
  Neural_Network &nn = static_cast<RefNet *>(h)->nn;
  bool *dst = nn.ptr_array_layers[layer].ptr_array__mask__dropout__bernoulli;
  if (dst == nullptr) return -1;
  for (uint64_t i = 0; i < count; ++i) dst[i] = mask[i] != 0;
  return 0;
}

// masks arrive as bool[T][cells]; the reference keeps one pointer per cell with a stride of `cells` between steps.
int ref_set_mask_zoneout(void *h, uint32_t layer, const uint8_t *state, const uint8_t *output, uint64_t count) {
  RefNet *r = static_cast<RefNet *>(h);
  Layer *L = r->nn.ptr_array_layers + layer;
  size_t C = L->ptr_last_cell_unit - L->ptr_array_cell_units;
  if (count != r->T * C || L->ptr_array_cell_units->ptr_mask_dropout_zoneout_state == nullptr) return -1;
  for (size_t c = 0; c < C; ++c)
    for (size_t t = 0; t < r->T; ++t) {
      L->ptr_array_cell_units[c].ptr_mask_dropout_zoneout_state[t * C] = state[t * C + c] != 0;
      L->ptr_array_cell_units[c].ptr_mask_dropout_zoneout_output[t * C] = output[t * C + c] != 0;
    }
  return 0;
}

int ref_set_training(void *h, int training) {
  static_cast<RefNet *>(h)->nn.type_state_propagation =
      training ? ENUM_TYPE_STATE_PROPAGATION::TYPE_STATE_PROPAGATION_TRAINING
               : ENUM_TYPE_STATE_PROPAGATION::TYPE_STATE_PROPAGATION_INFERENCE;
  return 0;
}

int ref_load_batch(void *h, uint64_t B, const float *X_TBI, const float *Y_TBO) {
  RefNet *r = static_cast<RefNet *>(h);
  if (X_TBI) unpack_rows(X_TBI, r->T, B, r->n_inputs, r->xrows, r->xptr);
  if (Y_TBO) unpack_rows(Y_TBO, r->T, B, r->n_outputs, r->yrows, r->yptr);
  return 0;
}

// The four calls of Dataset::Train_Batch_BP_{Loop,OpenMP} (Dataset.cpp:637-691) on the loaded batch.
// `stages` bit mask: 1 forward, 2 compute error, 4 backward, 8 update derivative weight.
int ref_run(void *h, uint64_t B, int stages) {
  RefNet *r = static_cast<RefNet *>(h);
  Neural_Network &nn = r->nn;
  if (r->threads > 1) {
    omp_set_num_threads(r->threads);
#pragma omp parallel
    {
      if (stages & 1) nn.Forward_Pass(B, r->xptr.data());
      if (stages & 2) nn.Compute__Error(B, r->yptr.data());
      if (stages & 4) nn.Backward_Pass(B);
      if (stages & 8) nn.Update_Derivative_Weight(B, nn.ptr_array_layers + 1, nn.ptr_last_layer);
    }
    if (stages & 8) {
      nn.Merge__Post__Training();
    }
  } else {
    if (stages & 1) nn.Forward_Pass(B, r->xptr.data());
    if (stages & 2) nn.Compute__Error(B, r->yptr.data());
    if (stages & 4) nn.Backward_Pass(B);
    if (stages & 8) nn.Update_Derivative_Weight(B, nn.ptr_array_layers + 1, nn.ptr_last_layer);
  }
  return 0;
}

// Per-thread derivative slices are only summed inside Update_Parameter__OpenMP; a test that wants to read the
// gradient in OpenMP mode merges first (Neural_Network__Merge.cpp:20-50).
int ref_merge_derivatives(void *h) {
  RefNet *r = static_cast<RefNet *>(h);
  if (r->threads > 1) r->nn.Merge_Derivatives_Parameters(0, r->nn.total_parameters);  // opens its own parallel loops
  return 0;
}

int ref_update_parameter(void *h, uint64_t B, uint64_t N, const myea_opt_desc *opt) {
  RefNet *r = static_cast<RefNet *>(h);
  if (opt) apply_opt(r->nn, *opt);
  r->nn.Update_Parameter(B, N);
  return 0;
}

int ref_reset_loss(void *h) { static_cast<RefNet *>(h)->nn.Reset__Loss(); return 0; }

int ref_get_loss(void *h, double *loss_sum, uint64_t *number_loss, double *accuracy_sum) {
  Neural_Network &nn = static_cast<RefNet *>(h)->nn;
  *loss_sum = nn.ptr_array_loss_values[0];
  *number_loss = nn.ptr_array_number_loss[0];
  *accuracy_sum = nn.ptr_array_accuracy_values[0][0];
  return 0;
}

// outputs of `layer` for the batch of the last forward pass, packed [T][B][outputs]
int ref_get_outputs(void *h, uint32_t layer, uint64_t B, T_ *out) {
  RefNet *r = static_cast<RefNet *>(h);
  Neural_Network &nn = r->nn;
  Layer *L = nn.ptr_array_layers + layer;
  size_t W = *L->ptr_number_outputs;
  for (size_t t = 0; t < r->T; ++t)
    for (size_t b = 0; b < B; ++b) std::memcpy(out + (t * B + b) * W, nn.Get__Outputs(L, b, t), W * sizeof(T_));
  return 0;
}

// delta of `layer` after the backward pass, packed [T][B][units]: FC = Neuron_unit::ptr_array_errors,
// LSTM = Cell_unit::ptr_delta_cell_output (error arriving on the cell outputs)
int ref_get_errors(void *h, uint32_t layer, uint64_t B, T_ *out) {
  RefNet *r = static_cast<RefNet *>(h);
  Neural_Network &nn = r->nn;
  Layer *L = nn.ptr_array_layers + layer;
  size_t W = *L->ptr_number_outputs;
  const T_ *src = nullptr;
  if (L->type_layer == ENUM_TYPE_LAYER::TYPE_LAYER_FULLY_CONNECTED) src = L->ptr_array_neuron_units->ptr_array_errors;
  else if (L->type_layer == ENUM_TYPE_LAYER::TYPE_LAYER_LSTM) src = L->ptr_array_cell_units->ptr_delta_cell_output;
  if (src == nullptr) return -1;
  for (size_t t = 0; t < r->T; ++t)
    for (size_t b = 0; b < B; ++b)
      std::memcpy(out + (t * B + b) * W, src + (t * nn.batch_size + b) * W, W * sizeof(T_));
  return 0;
}

// Wall-clock milliseconds of `steps` full training steps (4 calls + Update_Parameter) on the loaded batch,
// after `warmup` untimed ones: the CPU baseline of the bench.
double ref_time_steps(void *h, uint64_t B, uint64_t N, int warmup, int steps) {
  RefNet *r = static_cast<RefNet *>(h);
  for (int i = 0; i < warmup; ++i) { ref_run(h, B, 15); r->nn.Update_Parameter(B, N); }
  auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < steps; ++i) { ref_run(h, B, 15); r->nn.Update_Parameter(B, N); }
  auto t1 = std::chrono::steady_clock::now();
  return std::chrono::duration<double, std::milli>(t1 - t0).count();
}

// Makes the ShakeDrop draws of the NEXT training step explicit without touching the reference: copies of its two
// generator objects are advanced through exactly the draw sequence the step will make (Loop mode, one generator of each
// kind) - forward, blocks in layer order, rows in order: one Bernoulli(p) draw per row and, when it is set, `width`
// draws of U(-1, 1) (Neural_Network__Forward_Pass__Loop.cpp:5016-5045); backward, blocks in reverse order, `width`
// draws of U(0, 1) from the same real generator for every row whose mask is set
// (Neural_Network__Backward_Pass__Loop.cpp:1050-1077).  Blocks are packed in layer order: masks [block][B],
// alpha / beta [block][B * width].  Returns the number of ShakeDrop blocks, or -1.
int ref_shakedrop_replay(void *h, uint64_t B, uint8_t *masks, float *alpha, float *beta) {
  RefNet *r = static_cast<RefNet *>(h);
  Neural_Network &nn = r->nn;
  if (nn.ptr_array_Class_Generator_Bernoulli_ShakeDrop == nullptr || nn.ptr_array_Class_Generator_Real_ShakeDrop == nullptr) return -1;
  MyEA::Random::Bernoulli<T_> bern;
  MyEA::Random::Floating<T_> real;
  bern = nn.ptr_array_Class_Generator_Bernoulli_ShakeDrop[0];
  real = nn.ptr_array_Class_Generator_Real_ShakeDrop[0];
  // widths: pitch of a block's rows in alpha / beta (the residual layer's outputs); drawn: coefficients the reference
  // draws per row = outputs of the block's LAST layer (narrower than the pitch under a zero-padded identity)
  std::vector<size_t> blocks, widths, drawn, offsets;
  size_t off = 0;
  for (size_t l = 1; l < nn.total_layers; ++l) {
    Layer *L = nn.ptr_array_layers + l;
    if (L->type_layer == ENUM_TYPE_LAYER::TYPE_LAYER_RESIDUAL && L->type_dropout == ENUM_TYPE_LAYER_DROPOUT::TYPE_LAYER_DROPOUT_SHAKEDROP) {
      blocks.push_back(l);
      widths.push_back(*L->ptr_number_outputs);
      drawn.push_back(*(L + L->block_depth)->ptr_number_outputs);
      offsets.push_back(off);
      off += B * *L->ptr_number_outputs;
    }
  }
  for (size_t k = 0; k < blocks.size(); ++k) {
    Layer *L = nn.ptr_array_layers + blocks[k];
    bern.Probability(L->dropout_values[0]);
    real.Range(-1_T, 1_T);
    for (size_t b = 0; b < B; ++b) {
      const bool m = bern();
      masks[k * B + b] = m ? 1 : 0;
      for (size_t j = 0; j < widths[k]; ++j) alpha[offsets[k] + b * widths[k] + j] = (m && j < drawn[k]) ? static_cast<float>(real()) : 1.0f;
    }
  }
  for (size_t k = blocks.size(); k-- > 0;) {
    real.Range(0_T, 1_T);
    for (size_t b = 0; b < B; ++b)
      for (size_t j = 0; j < widths[k]; ++j) beta[offsets[k] + b * widths[k] + j] = (masks[k * B + b] && j < drawn[k]) ? static_cast<float>(real()) : 1.0f;
  }
  return static_cast<int>(blocks.size());
}

// The reference's own checkpoint writers (Neural_Network__Save.cpp:23 and :204) on this network.
int ref_save(void *h, const char *path_dimension, const char *path_general) {
  Neural_Network &nn = static_cast<RefNet *>(h)->nn;
  if (path_dimension != nullptr && !nn.Save_Dimension_Parameters(path_dimension)) return -1;
  if (path_general != nullptr && !nn.Save_General_Parameters(path_general)) return -1;
  return 0;
}

// The reference's own checkpoint reader (Neural_Network__Load.cpp:2323) into a fresh object; the handle supports
// ref_sizes / ref_layer_index / ref_buffer / ref_layer_state / ref_general_state.
void *ref_load(const char *path_dimension, const char *path_general) {
  RefNet *r = new RefNet();
  if (!r->nn.Load(path_dimension, path_general, size_t(1) << 40)) {
    delete r;
    return nullptr;
  }
  r->n_inputs = r->nn.number_inputs;
  r->n_outputs = r->nn.number_outputs;
  r->T = r->nn.number_recurrent_depth;
  return r;
}

// Per-layer configuration of a loaded object, in descriptor form.
int ref_layer_state(void *h, uint32_t layer, myea_layer_desc *out) {
  Neural_Network &nn = static_cast<RefNet *>(h)->nn;
  if (layer >= nn.total_layers) return -1;
  Layer *L = nn.ptr_array_layers + layer;
  std::memset(out, 0, sizeof(*out));
  out->type_layer = L->type_layer;
  out->use_bidirectional = L->use_bidirectional;
  out->type_activation_function = L->ptr_array_AF_units != L->ptr_last_AF_unit
                                      ? static_cast<uint32_t>(*L->ptr_array_AF_units->ptr_type_activation_function) : 0u;
  out->type_normalization = L->type_normalization;
  out->use_layer_normalization_before_activation = L->use_layer_normalization_before_activation;
  out->type_dropout = L->type_dropout;
  for (int k = 0; k < 3; ++k) out->dropout_values[k] = L->dropout_values[k];
  out->unit_parameters[0] = *L->ptr_number_outputs;
  return 0;
}

// Network-level training state of a loaded object: v[0..] = learning_rate, learning_momentum, adam_learning_rate,
// adam_beta1, adam_beta2, adam_epsilon, regularization__weight_decay, clip_gradient, normalization_momentum_average,
// normalization_epsilon, accuracy_variance, regularization__max_norm_constraints; u[0..] = type_optimizer_function,
// type_loss_function, type_accuracy_function, use_Nesterov, use_clip_gradient, type_network, number_recurrent_depth,
// number_time_delays.
int ref_general_state(void *h, float v[12], uint64_t u[8]) {
  Neural_Network &nn = static_cast<RefNet *>(h)->nn;
  v[0] = nn.learning_rate; v[1] = nn.learning_momentum; v[2] = nn.adam_learning_rate; v[3] = nn.adam_beta1;
  v[4] = nn.adam_beta2; v[5] = nn.adam_epsilon; v[6] = nn.regularization__weight_decay; v[7] = nn.clip_gradient;
  v[8] = nn.normalization_momentum_average; v[9] = nn.normalization_epsilon; v[10] = nn.accuracy_variance;
  v[11] = nn.regularization__max_norm_constraints;
  u[0] = nn.type_optimizer_function; u[1] = nn.type_loss_function; u[2] = nn.type_accuracy_function;
  u[3] = nn.use_Nesterov; u[4] = nn.use_clip_gradient; u[5] = nn.type_network; u[6] = nn.number_recurrent_depth;
  u[7] = nn.number_time_delays;
  return 0;
}

}  // extern "C"
