// The device-side network object behind a myea_handle: the reference's flat buffers and index map, the
// per-layer activation / error buffers, and the step functions.
#pragma once

#include <vector>

#include "common.cuh"

namespace myea {

struct LstmPlan;   // lstm.cu
struct LayerPlan;
struct CommState;  // comm.cu

struct LayerPlan {
  myea_layer_desc desc;
  myea_layer_index idx;
  uint32_t type = 0;
  long long n_in = 0, n_out = 0;  // widths per time step
  int input_layer = -1;            // layer whose outputs feed this one
  bool use_bias = false;           // FC: false under normalization (Layer::Use__Bias, Data.hpp:736)
  bool is_output = false;
  // [T*B, n_out] each
  float *summations = nullptr;  // z = W x (+ b)
  float *values = nullptr;      // layer output after activation and dropout
  float *deriv = nullptr;       // error after the activation derivative (input of the normalization backward)
  float *errors = nullptr;      // error w.r.t. z (what Update_Derivative_Weight and the previous layer read)
  bool has_norm = false;
  NormParams norm;
  uint8_t *mask_bernoulli = nullptr;  // [T*n_out]
  float keep_scale = 1.f;             // factor applied to kept units while training
  float infer_scale = 1.f;            // factor applied to every unit at inference
  LstmPlan *lstm = nullptr;
  // residual block (type RESIDUAL): see residual.cu
  int block_depth = 0;
  uint8_t *shake_mask = nullptr;      // [B]
  float *shake_alpha = nullptr, *shake_beta = nullptr;  // [B, n_out]
  long long norm_unit_offset = 0;     // units of earlier layers in the normalized-unit run
  // Operand panels shared by the three contractions of a large fully connected layer (all on the 256 x 256 kernel):
  // one split pass per tensor and step serves both of its readings.  input: forward (rows, role A) and dW (columns,
  // role B); weights: forward (rows, role B) and error propagation (columns, role B); errors: error propagation
  // (rows, role A) and dW (columns, role A).
  bool shared_panels = false;
  float *in_panel_mem = nullptr, *w_panel_mem = nullptr, *d_panel_mem = nullptr;
  Panels in_rows, in_cols, w_rows, w_cols, d_rows, d_cols;
  bool in_valid = false, w_valid = false, d_valid = false;
  bool w_prepared = false;  // the weight panels have already been made in this forward pass (hoisted under the input copy)
  const float *in_src = nullptr;  // the array the input panels were made from
  const float *in_ready_src = nullptr;  // set by the producer of this layer's input when IT has written the input panels
  long long in_ready_rows = 0;
  int bwd_fused_chunks = 0;       // row blocks whose normalization-backward sums the error-propagation epilogue has emitted
  int *pool_winner = nullptr;     // max pooling: [T*B, n_out] position (in the padded input) that gave each output
  // independently recurrent fully connected layer (type FULLY_CONNECTED here, ind_rnn set): n_out recurrent weights
  // behind the layer's n_out * n_in weights; pre_af = summation (normalized) + u * previous output, what the activation sees
  // roles of an autoencoder pre-training pass: -1 = as the network's state says, 0 = inference behaviour (running
  // statistics / dropout scaling), 1 = training behaviour (batch statistics / dropout masks)
  int mode_norm = -1, mode_drop = -1;
  bool ind_rnn = false;
  float *pre_af = nullptr;        // [T*B, n_out]
};

// independently recurrent layers (ind_rnn.cu)
int ind_rnn_forward_step(Context &ctx, const float *z, const float *y_prev, const float *u, float *pre, float *y, long long rows, long long H, uint32_t af,
                         const float *col_scale, const float *col_shift, const uint8_t *mask, float keep_scale);
int ind_rnn_backward_step(Context &ctx, float *d, const float *d_next, const float *u, const float *pre, const float *y, long long rows, long long H,
                          uint32_t af);
float ind_rnn_weight_bound(float clip_gradient, uint32_t type_activation_function, long long T);
int ind_rnn_clamp(Context &ctx, float *w, long long n, float bound);
int ind_rnn_recurrent_derivative(Context &ctx, const float *d, const float *y, long long rows, long long H, long long shift, float *scratch, float *du,
                                 float *partial, int chunks);

// pooling layers (pooling.cu)
long long pooling_output_width(const myea_layer_desc &d, long long n_in);
int pooling_forward(myea_b200_net *net, LayerPlan &L, const float *input, long long rows);
int pooling_backward(myea_b200_net *net, LayerPlan &L, float *d_input, long long rows);

// z = input * W^T of a fully connected layer and D = errors * W (error on the layer's inputs), from the layer's shared
// operand panels when it has them, else through gemm_nt; `e` carries destination and fused extras (net.cu)
int fc_product_forward(myea_b200_net *net, LayerPlan &L, const float *input, long long rows, const Epilogue &e);
int fc_product_backward(myea_b200_net *net, LayerPlan &N, long long rows, const Epilogue &e);

}  // namespace myea

struct myea_b200_net;
namespace myea {
// fills net->layers (widths, input layers, index map) and the parameter totals from net->desc; host arithmetic only
int build_index_map(myea_b200_net *net);
}  // namespace myea

struct myea_b200_net {
  myea::Context ctx;
  myea_net_desc desc;
  std::vector<myea::LayerPlan> layers;
  uint64_t total_parameters = 0, total_weights = 0, total_bias = 0, total_norm_units = 0;
  long long T = 1, B = 0;
  long long active_B = 0;  // samples of the batch in flight: B, or fewer for the last batch of an epoch
  bool full_pitch = false; // recurrent (T > 1 or an LSTM layer): buffers keep the allocated B as the row pitch of a time step
  long long pitch() const { return full_pitch ? B : active_B; }  // rows per time step the kernels of the step in flight run over
  bool any_norm = false;
  // flat buffers, [P] (norm averages: [total_norm_units])
  float *params = nullptr, *grads = nullptr, *m1 = nullptr, *m2 = nullptr, *m2hat = nullptr, *prev_delta = nullptr,
        *mask_reg = nullptr;
  float *norm_mean_avg = nullptr, *norm_sigma_avg = nullptr;
  float *norm_stats = nullptr;  // [total_norm_units][6]: mean, sigma, r, d, col_scale, col_shift
  float *norm_partial = nullptr;
  float *reduce_partial = nullptr;
  int reduce_chunks = 64;
  int norm_chunks = 64;        // row blocks the normalization partial-sum workspace has room for
  float *d_input = nullptr;    // [T*B, inputs]
  float *d_desired = nullptr;  // [T*B, outputs]
  myea::GemmScratch scratch;
  double *d_loss_acc = nullptr;  // [2] loss sum, accuracy sum
  unsigned long long *d_loss_count = nullptr;
  double *d_sumsq = nullptr;
  float *d_clip_scale = nullptr;
  float optimizer_time_step = 0.f;
  float nosadam_previous_beta2 = 0.f;  // adam_previous_beta2 (Data.hpp:2953)
  bool training = true;
  uint32_t pre_training_level = 0;  // 0: the whole network; k >= 1: hidden layer k and its mirror image are trained as an autoencoder
  myea::CommState *comm = nullptr;
  myea::SumHook hook;            // cross-GPU sum of normalization column sums (world 1: unused)
  bool grads_reduced = false;    // this step's derivative buckets have already been handed to the communicator
  bool sharded_update = true;    // the last update was element by element (no clip, no max-norm): buckets may be reduce-scattered
  double *d_loss_tmp = nullptr;  // [3] staging for the cross-GPU sum of the loss accumulators
  // dataset kept on the device for the epoch loop (epoch.cu): rows [example][T * width], the staged batch, the order
  float *ds_inputs = nullptr, *ds_outputs = nullptr, *ds_batch_inputs = nullptr, *ds_batch_outputs = nullptr;
  unsigned long long *ds_order = nullptr;
  uint64_t ds_examples = 0, ds_order_capacity = 0;
  // targets arriving from the host are copied on a stream of their own, so that the copy runs under the forward pass
  // that is still executing; the two events order it against the error kernel's use of d_desired
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t ev_desired_ready = nullptr, ev_desired_free = nullptr;
  cudaEvent_t ev_input_ready = nullptr, ev_input_free = nullptr;  // the same for inputs arriving from the host
  std::vector<void *> allocations;
};
