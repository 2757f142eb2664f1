// Host-side mirror of the reference's `class Neural_Network` (Header_Files/Neural_Network/Data.hpp:760-3293) for the
// training step: the same member names, argument meaning and "return false / print, never throw" behaviour, with
// every computation forwarded to the sm_100a library through the C ABI of include/myea_b200.h.  It holds no numerics
// of its own; without the library or without a GPU every step function reports failure.
//
// Differences a caller sees, all stemming from device residency:
//   * device memory is carved by Initialize__CUDA(), to be called once the topology, activation functions,
//     normalization, dropout, optimizer and batch size are set (the reference's Initialize__CUDA has the same place in
//     its GPU flow, Data.hpp:3112-3195); the public host arrays (ptr_array_parameters, ...) exist from then on;
//   * host arrays are synchronised explicitly with Copy__Parameters__Host_To_Device / __Device_To_Host, as in the
//     reference's GPU seam; dropout / zoneout masks and ShakeDrop coefficients are uploaded with the Upload__* members
//     after the caller (re)draws them in the public mask arrays.
#pragma once

#include <stddef.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "myea_b200.h"

namespace MyEA { namespace B200 {

struct Layer_Parameters {          // Data.hpp:56-80
  bool use_bidirectional = false;
  unsigned int type_layer = 0;     // ENUM_TYPE_LAYER value
  size_t unit_parameters[5] = {0};
};

class Neural_Network {
 public:
  Neural_Network() {}
  ~Neural_Network();
  Neural_Network(Neural_Network const &) = delete;
  Neural_Network &operator=(Neural_Network const &) = delete;

  // ---- construction (Neural_Network__Compile.cpp:426-785 and the Set__* family) ----
  bool Compile(size_t number_layers, size_t number_recurrent_depth, unsigned int type_network, Layer_Parameters const *ptr_array_layers_parameters,
               size_t maximum_allowable_memory = 0);
  bool Set__Layer_Activation_Function(size_t index_layer, unsigned int type_activation_function);
  bool Set__Layer_Normalization(size_t index_layer, unsigned int type_layer_normalization, bool reallocate = true, bool organize_pointers = true);
  bool Set__Dropout(size_t index_layer, unsigned int type_layer_dropout, float const value_dropout[], bool scale_weights = true);
  void Set__Loss_Function(unsigned int type) { desc_.type_loss_function = type; }
  void Set__Accuracy_Function(unsigned int type) { desc_.type_accuracy_function = type; }
  void Set__Optimizer_Function(unsigned int type) { opt_.type_optimizer_function = type; }
  bool Set__Accurancy_Variance(float v) { desc_.accuracy_variance = v; return v >= 0.f; }
  bool Set__Number_Time_Delays(size_t d) { desc_.number_time_delays = d; return d < desc_.number_recurrent_depth; }
  bool Set__Regularization__Weight_Decay(float v) { opt_.regularization__weight_decay = v; return v >= 0.f; }
  bool Set__Regularization__Max_Norm_Constraints(float v) { opt_.regularization__max_norm_constraints = v; return v >= 0.f; }
  // range checks of Set__Regularization__L1 / __L2 (Neural_Network__Regularization__L1.cpp:24-46); the step ignores both
  // penalties, as the reference's own does (see myea_opt_desc)
  bool Set__Regularization__L1(float v) { if (v < 0.f || v > 1.f) return false; opt_.regularization__l1 = v; return true; }
  bool Set__Regularization__L2(float v) { if (v < 0.f || v > 1.f) return false; opt_.regularization__l2 = v; return true; }
  void Set__Clip_Gradient(bool use) { opt_.use_clip_gradient = use ? 1u : 0u; }
  bool Set__Clip_Gradient(float v) { opt_.clip_gradient = v; return v > 0.f; }
  bool Set__Normalization_Momentum_Average(float v) { desc_.normalization_momentum_average = v; return v > 0.f && v <= 1.f; }
  bool Set__Normalization_Epsilon(float v) { desc_.normalization_epsilon = v; return v > 0.f; }
  bool Set__Batch_Renormalization_r_Correction_Maximum(float v) { desc_.batch_renormalization_r_correction_maximum = v; return v >= 1.f; }
  bool Set__Batch_Renormalization_d_Correction_Maximum(float v) { desc_.batch_renormalization_d_correction_maximum = v; return v >= 0.f; }
  // autoencoder pre-training (Neural_Network__Indexing.cpp:20-51): 0 = the whole network; needs the device network
  bool Set__Pre_Training_Level(size_t pre_training_level) {
    if (!is_device_initialized) return fail("Set__Pre_Training_Level", MYEA_E_INVALID);
    int const rc = myea_b200_set_pre_training_level(ptr_device_Neural_Network, pre_training_level);
    if (rc == MYEA_OK) this->pre_training_level = pre_training_level;
    return rc == MYEA_OK ? true : fail("Set__Pre_Training_Level", rc);
  }
  size_t pre_training_level = 0;
  bool Update__Batch_Size(size_t desired_batch_size, bool force_update = false);
  void Clear_Training_Arrays(void);

  // ---- device residency (Data.hpp:3112-3195) ----
  bool Set__CUDA(bool use_cuda, size_t /*maximum_allowable_memory*/ = 0) { use_CUDA = use_cuda; return true; }
  bool Initialize__CUDA(size_t device_index = 0);
  bool Deinitialize__CUDA(void);
  bool Copy__Parameters__Host_To_Device(void);
  bool Copy__Parameters__Device_To_Host(void);
  bool Copy__Optimizer_Paramaters__Device_To_Host(void);
  bool Copy__Batch_Normalization_Neurons__Device_To_Host(void);
  bool Copy__Derivatives_Parameters__Device_To_Host(void);
  bool Upload__Mask_Dropout_Bernoulli(size_t index_layer, bool const *mask, size_t count);
  bool Upload__Mask_Dropout_Zoneout(size_t index_layer, bool const *mask_state, bool const *mask_output, size_t count);
  bool Upload__Dropout_ShakeDrop(size_t index_layer, bool const *mask, float const *alpha, float const *beta, size_t batch);
  // Dropout_Bernoulli() / Dropout_Zoneout() and the ShakeDrop draws (Data.hpp:944-958): new masks and coefficients for
  // every layer, drawn on the device from (seed_dropout, number of calls so far); nothing is uploaded
  void Dropout_Bernoulli(void) { Draw__Masks(); }
  void Dropout_Zoneout(void) { Draw__Masks(); }
  bool Draw__Masks(void);
  unsigned long long seed_dropout = 5413u;

  // ---- the training step (Dataset.cpp:637-691, 7654-7690) ----
  void Forward_Pass(size_t batch_size, float const *const *ptr_array_inputs, long long input_layer = -1, long long output_layer = -1);
  void Compute__Error(size_t batch_size, float const *const *ptr_array_desireds_outputs);
  void Backward_Pass(size_t batch_size);
  void Update_Derivative_Weight(size_t batch_size);
  void Update_Parameter(size_t batch_size, size_t training_size);
  void Reset__Loss(void);
  float Get__Loss(void);       // accumulated loss / number of loss terms (mean squared error; cross-entropy sum / terms)
  float Get__Accuracy(void);   // accumulated hits / number_accuracy_trial * 100
  float const *Get__Outputs(size_t data_index, size_t time_step_index = 0);

  // ---- checkpoint files in the reference's text format (Neural_Network__Save.cpp:23, :204; Neural_Network__Load.cpp:2323) ----
  // Save_*: written from the device-resident state (parameters and normalization averages are copied back first, as
  // Save.cpp:227-237 does).  Load: call on a fresh object; it takes the place of Compile + Set__* and leaves the
  // network initialized on `device_index` for `desired_batch_size` rows with parameters uploaded.  The reference's
  // third argument (maximum allowable memory) has no meaning here and is replaced by the batch size the device
  // buffers are carved for.
  bool Save_General_Parameters(std::string const &path);
  bool Save_Dimension_Parameters(std::string const &path);
  bool Load(std::string const &path_dimension, std::string const &path_general, size_t desired_batch_size, size_t device_index = 0);

  char const *Get__Last_Error(void) const { return error_.c_str(); }

  // ---- public state, as in the reference (Data.hpp:2786-3048) ----
  size_t total_layers = 0, total_parameters = 0, total_weights = 0, total_bias = 0, total_normalized_units = 0;
  size_t number_recurrent_depth = 1, number_inputs = 0, number_outputs = 0, batch_size = 0, number_accuracy_trial = 0;
  unsigned int type_state_propagation = 1;  // ENUM_TYPE_STATE_PROPAGATION: 0 inference, 1 training
  bool use_CUDA = true, is_device_initialized = false;
  float learning_rate = 0.01f, learning_momentum = 0.9f, learning_rate_final = 0.1f, learning_gamma = 1e-3f;
  float adam_learning_rate = 0.001f, adam_beta1 = 0.9f, adam_beta2 = 0.999f, adam_epsilon = 1e-8f, epoch_time_step = 1.f;
  bool use_Nesterov = false, use_normalized_weight_decay = true, use_adam_bias_correction = true;
  float rprop_increase_factor = 1.2f, rprop_decrease_factor = 0.5f, rprop_delta_min = 1e-6f, rprop_delta_max = 50.f, rprop_delta_zero = 0.1f;
  float loss_rprop = 3.402823466e+38f, previous_loss_rprop = 3.402823466e+38f;  // iRPROP+ (Data.hpp, Dataset.cpp:575-579)
  float *ptr_array_parameters = nullptr;                     // [total_parameters]
  float *ptr_array_derivatives_parameters = nullptr;         // [total_parameters], merged
  float *ptr_array_previous_biased_first_moment = nullptr, *ptr_array_previous_biased_second_moment = nullptr,
        *ptr_array_previous_biased_second_moment_hat = nullptr, *ptr_array_mask_regularized_parameters = nullptr;
  float *ptr_array_normalized_batch_units_means_averages = nullptr, *ptr_array_normalized_batch_units_variances_averages = nullptr;
  myea_handle ptr_device_Neural_Network = nullptr;
  myea_layer_index const &Get__Layer_Index(size_t index_layer) const { return index_[index_layer]; }

 private:
  bool fail(char const *where, int status);
  void sync_optimizer(void);
  bool adopt_device(void);
  unsigned long long draws_ = 0;
  bool pack(float const *const *rows, size_t batch, size_t width, std::vector<float> &dst);
  myea_net_desc desc_ = {};
  myea_opt_desc opt_ = {};
  std::vector<myea_layer_index> index_;
  std::vector<float> host_[8], stage_x_, stage_y_, outputs_;
  std::string error_;
};

}}  // namespace MyEA::B200
