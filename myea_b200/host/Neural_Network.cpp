// See Neural_Network.hpp.  Every member is a thin adapter from the reference's calling convention (row pointers, bool
// results, printed diagnostics) to the C ABI.
#include "Neural_Network.hpp"

#include <stdio.h>
#include <string.h>

namespace MyEA { namespace B200 {

Neural_Network::~Neural_Network() { Deinitialize__CUDA(); }

bool Neural_Network::fail(char const *where, int status) {
  error_ = std::string(where) + ": " + (ptr_device_Neural_Network ? myea_b200_last_error(ptr_device_Neural_Network) : "no device network");
  fprintf(stderr, "%s: ERROR: status %d: %s\n", where, status, error_.c_str());
  return false;
}

bool Neural_Network::Compile(size_t number_layers, size_t depth, unsigned int type_network, Layer_Parameters const *lp, size_t) {
  if (number_layers < 2 || number_layers > MYEA_MAX_LAYERS || lp == nullptr || depth == 0) return fail("Compile", MYEA_E_INVALID);
  memset(&desc_, 0, sizeof(desc_));
  memset(&opt_, 0, sizeof(opt_));
  desc_.number_layers = static_cast<uint32_t>(number_layers);
  desc_.type_network = type_network;
  desc_.number_recurrent_depth = depth;
  desc_.type_loss_function = MYEA_LOSS_MSE;
  for (size_t l = 0; l < number_layers; ++l) {
    myea_layer_desc &d = desc_.layers[l];
    d.type_layer = lp[l].type_layer;
    d.use_bidirectional = lp[l].use_bidirectional ? 1u : 0u;
    for (int k = 0; k < 5; ++k) d.unit_parameters[k] = lp[l].unit_parameters[k];
    d.type_activation_function = MYEA_AF_LINEAR;
    d.use_layer_normalization_before_activation = 1u;
  }
  opt_.type_optimizer_function = MYEA_OPT_GD;
  total_layers = number_layers;
  number_recurrent_depth = depth;
  number_inputs = lp[0].unit_parameters[0];
  number_outputs = lp[number_layers - 1].unit_parameters[0];
  return true;
}

bool Neural_Network::Set__Layer_Activation_Function(size_t l, unsigned int af) {
  if (l == 0 || l >= total_layers) return fail("Set__Layer_Activation_Function", MYEA_E_INVALID);
  desc_.layers[l].type_activation_function = af;
  return true;
}

bool Neural_Network::Set__Layer_Normalization(size_t l, unsigned int type, bool, bool) {
  if (l == 0 || l >= total_layers) return fail("Set__Layer_Normalization", MYEA_E_INVALID);
  desc_.layers[l].type_normalization = type;
  return true;
}

bool Neural_Network::Set__Dropout(size_t l, unsigned int type, float const v[], bool) {
  if (l == 0 || l >= total_layers || v == nullptr) return fail("Set__Dropout", MYEA_E_INVALID);
  desc_.layers[l].type_dropout = type;
  desc_.layers[l].dropout_values[0] = v[0];
  desc_.layers[l].dropout_values[1] = type == MYEA_DROPOUT_ZONEOUT ? v[1] : 0.f;
  return true;
}

bool Neural_Network::Update__Batch_Size(size_t desired, bool) {
  if (desired == 0 || is_device_initialized) return desired == batch_size;  // carved buffers are fixed once on the device
  batch_size = desired;
  desc_.batch_size = desired;
  return true;
}

bool Neural_Network::Initialize__CUDA(size_t device) {
  if (is_device_initialized) return true;
  if (batch_size == 0) return fail("Initialize__CUDA", MYEA_E_INVALID);
  int rc = myea_b200_create(&ptr_device_Neural_Network, &desc_, static_cast<int>(device));
  if (rc != MYEA_OK) {
    fail("Initialize__CUDA", rc);
    myea_b200_destroy(ptr_device_Neural_Network);
    ptr_device_Neural_Network = nullptr;
    return false;
  }
  if (!adopt_device()) return false;
  is_device_initialized = true;
  return Copy__Parameters__Host_To_Device();
}

// sizes, index map and the public host arrays of a freshly created device network
bool Neural_Network::adopt_device(void) {
  uint64_t P, W, Bn, U;
  myea_b200_sizes(ptr_device_Neural_Network, &P, &W, &Bn, &U);
  total_parameters = P; total_weights = W; total_bias = Bn; total_normalized_units = U;
  index_.resize(total_layers);
  for (size_t l = 0; l < total_layers; ++l) myea_b200_layer_index(ptr_device_Neural_Network, static_cast<uint32_t>(l), &index_[l]);
  for (int k = 0; k < 6; ++k) host_[k].assign(P, 0.f);
  host_[6].assign(U * number_recurrent_depth, 0.f);   // running averages: one set per time step
  host_[7].assign(U * number_recurrent_depth, 1.f);
  ptr_array_parameters = host_[0].data();
  ptr_array_derivatives_parameters = host_[1].data();
  ptr_array_previous_biased_first_moment = host_[2].data();
  ptr_array_previous_biased_second_moment = host_[3].data();
  ptr_array_previous_biased_second_moment_hat = host_[4].data();
  ptr_array_mask_regularized_parameters = host_[5].data();
  ptr_array_normalized_batch_units_means_averages = host_[6].data();
  ptr_array_normalized_batch_units_variances_averages = host_[7].data();
  for (size_t i = 0; i < W; ++i) host_[5][i] = 1.f;   // weights are regularized, biases and scales / shifts are not
  if (U) for (size_t i = 0; i < U; ++i) host_[0][W + Bn + i] = 1.f;   // scales start at one
  return true;
}

bool Neural_Network::Deinitialize__CUDA(void) {
  if (ptr_device_Neural_Network != nullptr) myea_b200_destroy(ptr_device_Neural_Network);
  ptr_device_Neural_Network = nullptr;
  is_device_initialized = false;
  return true;
}

bool Neural_Network::Copy__Parameters__Host_To_Device(void) {
  if (!is_device_initialized) return fail("Copy__Parameters__Host_To_Device", MYEA_E_INVALID);
  myea_handle h = ptr_device_Neural_Network;
  int rc = myea_b200_upload(h, MYEA_BUF_PARAMETERS, ptr_array_parameters, 0, total_parameters);
  if (rc == MYEA_OK) rc = myea_b200_upload(h, MYEA_BUF_MASK_REGULARIZED, ptr_array_mask_regularized_parameters, 0, total_parameters);
  if (rc == MYEA_OK && total_normalized_units) rc = myea_b200_upload(h, MYEA_BUF_NORM_MEAN_AVERAGE, ptr_array_normalized_batch_units_means_averages, 0, total_normalized_units * number_recurrent_depth);
  if (rc == MYEA_OK && total_normalized_units) rc = myea_b200_upload(h, MYEA_BUF_NORM_VARIANCE_AVERAGE, ptr_array_normalized_batch_units_variances_averages, 0, total_normalized_units * number_recurrent_depth);
  return rc == MYEA_OK ? true : fail("Copy__Parameters__Host_To_Device", rc);
}

bool Neural_Network::Copy__Parameters__Device_To_Host(void) {
  if (!is_device_initialized) return fail("Copy__Parameters__Device_To_Host", MYEA_E_INVALID);
  int rc = myea_b200_download(ptr_device_Neural_Network, MYEA_BUF_PARAMETERS, ptr_array_parameters, 0, total_parameters);
  return rc == MYEA_OK ? true : fail("Copy__Parameters__Device_To_Host", rc);
}

bool Neural_Network::Copy__Derivatives_Parameters__Device_To_Host(void) {
  if (!is_device_initialized) return fail("Copy__Derivatives_Parameters__Device_To_Host", MYEA_E_INVALID);
  int rc = myea_b200_download(ptr_device_Neural_Network, MYEA_BUF_DERIVATIVES, ptr_array_derivatives_parameters, 0, total_parameters);
  return rc == MYEA_OK ? true : fail("Copy__Derivatives_Parameters__Device_To_Host", rc);
}

bool Neural_Network::Copy__Optimizer_Paramaters__Device_To_Host(void) {
  if (!is_device_initialized) return fail("Copy__Optimizer_Paramaters__Device_To_Host", MYEA_E_INVALID);
  myea_handle h = ptr_device_Neural_Network;
  int rc = myea_b200_download(h, MYEA_BUF_FIRST_MOMENT, ptr_array_previous_biased_first_moment, 0, total_parameters);
  if (rc == MYEA_OK) rc = myea_b200_download(h, MYEA_BUF_SECOND_MOMENT, ptr_array_previous_biased_second_moment, 0, total_parameters);
  if (rc == MYEA_OK) rc = myea_b200_download(h, MYEA_BUF_SECOND_MOMENT_HAT, ptr_array_previous_biased_second_moment_hat, 0, total_parameters);
  return rc == MYEA_OK ? true : fail("Copy__Optimizer_Paramaters__Device_To_Host", rc);
}

bool Neural_Network::Copy__Batch_Normalization_Neurons__Device_To_Host(void) {
  if (!is_device_initialized || total_normalized_units == 0) return is_device_initialized;
  myea_handle h = ptr_device_Neural_Network;
  int rc = myea_b200_download(h, MYEA_BUF_NORM_MEAN_AVERAGE, ptr_array_normalized_batch_units_means_averages, 0, total_normalized_units * number_recurrent_depth);
  if (rc == MYEA_OK) rc = myea_b200_download(h, MYEA_BUF_NORM_VARIANCE_AVERAGE, ptr_array_normalized_batch_units_variances_averages, 0, total_normalized_units * number_recurrent_depth);
  return rc == MYEA_OK ? true : fail("Copy__Batch_Normalization_Neurons__Device_To_Host", rc);
}

bool Neural_Network::Upload__Mask_Dropout_Bernoulli(size_t l, bool const *mask, size_t count) {
  static_assert(sizeof(bool) == 1, "masks are one byte per unit");
  int rc = myea_b200_set_mask_bernoulli(ptr_device_Neural_Network, static_cast<uint32_t>(l), reinterpret_cast<uint8_t const *>(mask), count);
  return rc == MYEA_OK ? true : fail("Upload__Mask_Dropout_Bernoulli", rc);
}

bool Neural_Network::Upload__Mask_Dropout_Zoneout(size_t l, bool const *state, bool const *output, size_t count) {
  int rc = myea_b200_set_mask_zoneout(ptr_device_Neural_Network, static_cast<uint32_t>(l), reinterpret_cast<uint8_t const *>(state),
                                      reinterpret_cast<uint8_t const *>(output), count);
  return rc == MYEA_OK ? true : fail("Upload__Mask_Dropout_Zoneout", rc);
}

bool Neural_Network::Upload__Dropout_ShakeDrop(size_t l, bool const *mask, float const *alpha, float const *beta, size_t batch) {
  int rc = myea_b200_set_shakedrop(ptr_device_Neural_Network, static_cast<uint32_t>(l), reinterpret_cast<uint8_t const *>(mask), alpha, beta, batch);
  return rc == MYEA_OK ? true : fail("Upload__Dropout_ShakeDrop", rc);
}

bool Neural_Network::Draw__Masks(void) {
  int rc = myea_b200_generate_masks(ptr_device_Neural_Network, seed_dropout, draws_++);
  return rc == MYEA_OK ? true : fail("Draw__Masks", rc);
}

// row pointers (one [T * width] row per sample, Neural_Network__Assign_Inputs.cpp:273-304) -> packed [T][B][width]
bool Neural_Network::pack(float const *const *rows, size_t B, size_t width, std::vector<float> &dst) {
  if (rows == nullptr) return false;
  dst.resize(number_recurrent_depth * B * width);
  for (size_t b = 0; b < B; ++b)
    for (size_t t = 0; t < number_recurrent_depth; ++t) memcpy(&dst[(t * B + b) * width], rows[b] + t * width, width * sizeof(float));
  return true;
}

void Neural_Network::Forward_Pass(size_t B, float const *const *X, long long, long long) {
  if (!is_device_initialized || !pack(X, B, number_inputs, stage_x_)) { fail("Forward_Pass", MYEA_E_INVALID); return; }
  int rc = myea_b200_forward(ptr_device_Neural_Network, B, stage_x_.data(), type_state_propagation >= 1 ? 1 : 0);
  if (rc != MYEA_OK) fail("Forward_Pass", rc);
}

void Neural_Network::Compute__Error(size_t B, float const *const *Y) {
  if (!is_device_initialized || !pack(Y, B, number_outputs, stage_y_)) { fail("Compute__Error", MYEA_E_INVALID); return; }
  int rc = myea_b200_compute_error(ptr_device_Neural_Network, B, stage_y_.data());
  if (rc != MYEA_OK) fail("Compute__Error", rc);
}

void Neural_Network::Backward_Pass(size_t B) {
  int rc = is_device_initialized ? myea_b200_backward(ptr_device_Neural_Network, B) : MYEA_E_INVALID;
  if (rc != MYEA_OK) fail("Backward_Pass", rc);
}

void Neural_Network::Update_Derivative_Weight(size_t B) {
  int rc = is_device_initialized ? myea_b200_update_derivative_weight(ptr_device_Neural_Network, B) : MYEA_E_INVALID;
  if (rc != MYEA_OK) fail("Update_Derivative_Weight", rc);
}

// the public optimizer members are the state of record, as in the reference; the descriptor follows them
void Neural_Network::sync_optimizer(void) {
  opt_.learning_rate = learning_rate; opt_.learning_momentum = learning_momentum; opt_.use_nesterov = use_Nesterov ? 1u : 0u;
  opt_.adam_learning_rate = adam_learning_rate; opt_.adam_beta1 = adam_beta1; opt_.adam_beta2 = adam_beta2; opt_.adam_epsilon = adam_epsilon;
  opt_.learning_rate_final = learning_rate_final; opt_.learning_gamma = learning_gamma;
  opt_.use_adam_bias_correction = use_adam_bias_correction ? 1u : 0u;
  opt_.use_normalized_weight_decay = use_normalized_weight_decay ? 1u : 0u;
  opt_.epoch_time_step = epoch_time_step;
  opt_.rprop_increase_factor = rprop_increase_factor; opt_.rprop_decrease_factor = rprop_decrease_factor;
  opt_.rprop_delta_min = rprop_delta_min; opt_.rprop_delta_max = rprop_delta_max; opt_.rprop_delta_zero = rprop_delta_zero;
  opt_.loss_rprop = loss_rprop; opt_.previous_loss_rprop = previous_loss_rprop;
}

bool Neural_Network::Save_General_Parameters(std::string const &path) {
  sync_optimizer();
  int rc = myea_b200_checkpoint_format_general(&desc_, &opt_, path.c_str());
  return rc == MYEA_OK ? true : fail("Save_General_Parameters", rc);
}

bool Neural_Network::Save_Dimension_Parameters(std::string const &path) {
  if (!is_device_initialized) return fail("Save_Dimension_Parameters", MYEA_E_INVALID);
  int rc = myea_b200_save_dimension_parameters(ptr_device_Neural_Network, path.c_str());
  return rc == MYEA_OK ? true : fail("Save_Dimension_Parameters", rc);
}

bool Neural_Network::Load(std::string const &path_dimension, std::string const &path_general, size_t desired_batch_size, size_t device) {
  if (is_device_initialized || desired_batch_size == 0) return fail("Load", MYEA_E_INVALID);
  int rc = myea_b200_checkpoint_parse(path_dimension.c_str(), path_general.c_str(), desired_batch_size, &desc_, &opt_, nullptr, 0, nullptr, nullptr, 0,
                                      nullptr, nullptr);
  if (rc == MYEA_OK) rc = myea_b200_load(&ptr_device_Neural_Network, path_dimension.c_str(), path_general.c_str(), desired_batch_size, static_cast<int>(device), nullptr);
  if (rc != MYEA_OK) {
    error_ = std::string("Load: ") + myea_b200_checkpoint_last_error();
    fprintf(stderr, "%s\n", error_.c_str());
    if (ptr_device_Neural_Network != nullptr) myea_b200_destroy(ptr_device_Neural_Network);
    ptr_device_Neural_Network = nullptr;
    return false;
  }
  total_layers = desc_.number_layers;
  number_recurrent_depth = desc_.number_recurrent_depth;
  number_inputs = desc_.layers[0].unit_parameters[0];
  number_outputs = desc_.layers[total_layers - 1].unit_parameters[0];
  batch_size = desired_batch_size;
  learning_rate = opt_.learning_rate; learning_momentum = opt_.learning_momentum; use_Nesterov = opt_.use_nesterov != 0;
  adam_learning_rate = opt_.adam_learning_rate; adam_beta1 = opt_.adam_beta1; adam_beta2 = opt_.adam_beta2; adam_epsilon = opt_.adam_epsilon;
  learning_rate_final = opt_.learning_rate_final; learning_gamma = opt_.learning_gamma;
  use_adam_bias_correction = opt_.use_adam_bias_correction != 0;
  use_normalized_weight_decay = opt_.use_normalized_weight_decay != 0;
  if (opt_.rprop_increase_factor > 0.f) rprop_increase_factor = opt_.rprop_increase_factor;
  if (opt_.rprop_decrease_factor > 0.f) rprop_decrease_factor = opt_.rprop_decrease_factor;
  if (opt_.rprop_delta_min > 0.f) rprop_delta_min = opt_.rprop_delta_min;
  if (opt_.rprop_delta_max > 0.f) rprop_delta_max = opt_.rprop_delta_max;
  if (opt_.rprop_delta_zero > 0.f) rprop_delta_zero = opt_.rprop_delta_zero;
  if (!adopt_device()) return false;
  is_device_initialized = true;
  return Copy__Parameters__Device_To_Host() && (total_normalized_units == 0 || Copy__Batch_Normalization_Neurons__Device_To_Host());
}

void Neural_Network::Update_Parameter(size_t B, size_t N) {
  sync_optimizer();
  int rc = is_device_initialized ? myea_b200_update_parameter(ptr_device_Neural_Network, B, N, &opt_) : MYEA_E_INVALID;
  if (rc != MYEA_OK) fail("Update_Parameter", rc);
}

void Neural_Network::Clear_Training_Arrays(void) {
  if (is_device_initialized) myea_b200_clear_training_arrays(ptr_device_Neural_Network);
}

void Neural_Network::Reset__Loss(void) {
  if (is_device_initialized) myea_b200_reset_loss(ptr_device_Neural_Network);
}

float Neural_Network::Get__Loss(void) {
  double s = 0, a = 0; uint64_t n = 0;
  if (!is_device_initialized || myea_b200_get_loss(ptr_device_Neural_Network, &s, &n, &a) != MYEA_OK || n == 0) return 1.f;
  return static_cast<float>(s / static_cast<double>(n));
}

float Neural_Network::Get__Accuracy(void) {
  double s = 0, a = 0; uint64_t n = 0;
  if (!is_device_initialized || myea_b200_get_loss(ptr_device_Neural_Network, &s, &n, &a) != MYEA_OK || number_accuracy_trial == 0) return 0.f;
  return static_cast<float>(a / static_cast<double>(number_accuracy_trial) * 100.0);
}

float const *Neural_Network::Get__Outputs(size_t data_index, size_t t) {
  if (!is_device_initialized) return nullptr;
  size_t const n = number_recurrent_depth * batch_size * number_outputs;
  outputs_.resize(n);
  if (myea_b200_get_outputs(ptr_device_Neural_Network, static_cast<uint32_t>(total_layers - 1), outputs_.data(), n) != MYEA_OK) return nullptr;
  return outputs_.data() + (t * batch_size + data_index) * number_outputs;
}

}}  // namespace MyEA::B200
