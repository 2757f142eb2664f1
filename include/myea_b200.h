/*
 * myea_b200.h — C ABI of the B200 (sm_100a) implementation of the MyEA training step.
 *
 * One handle = one `class Neural_Network` of the reference (Header_Files/Neural_Network/Data.hpp:760-3293)
 * living on one GPU.  The entry points are one-to-one with the member functions the reference's training
 * loop calls (Source_Files/Neural_Network/Dataset.cpp:637-691, 7654-7690); each declaration cites the member
 * it replaces.  Plain pointers and sizes only; host memory is owned by the caller, device memory by the
 * library.  Every function returns 0 on success or a negative MYEA_E_* status and never aborts or traps;
 * myea_b200_last_error() gives the message.  One host thread per handle; calls are asynchronous on the
 * handle's stream, download / compute_error results synchronise.
 *
 * Enumerator values are the reference's own (Common_Library/include/Enums/ *.hpp) so that a host class can
 * pass its enums through unchanged.
 */
#ifndef MYEA_B200_H
#define MYEA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MYEA_MAX_LAYERS 64

/* status codes */
#define MYEA_OK 0
#define MYEA_E_INVALID (-1)     /* bad argument / unsupported topology            */
#define MYEA_E_CUDA (-2)        /* a CUDA runtime / driver call failed            */
#define MYEA_E_KERNEL (-3)      /* a kernel reported a bounded-wait timeout       */
#define MYEA_E_UNSUPPORTED (-4) /* valid in the reference, not built here         */
#define MYEA_E_COMM (-5)        /* NCCL failure                                   */

/* ENUM_TYPE_LAYER (Enum_Type_Layer.hpp:25) */
#define MYEA_LAYER_AVERAGE_POOLING 1u /* unit_parameters: kernel size, stride, padding, dilation, ceil mode (Compile.cpp:51-58) */
#define MYEA_LAYER_FULLY_CONNECTED 4u
#define MYEA_LAYER_FC_INDEPENDENTLY_RECURRENT 5u /* a fully connected layer whose units also see their own previous output through
                                                   one recurrent weight each (Ind-RNN; Prepare__Connections__FC_Ind_RNN) */
#define MYEA_LAYER_LSTM 8u
#define MYEA_LAYER_MAX_POOLING 9u     /* the same five values */
#define MYEA_LAYER_RESIDUAL 10u
/* ENUM_TYPE_NETWORKS (Enum_Type_Networks.hpp:25) */
#define MYEA_NETWORK_AUTOENCODER 1u
#define MYEA_NETWORK_FEEDFORWARD 3u
#define MYEA_NETWORK_RECURRENT 4u
/* ENUM_TYPE_ACTIVATION_FUNCTION (Enum_Type_Activation_Functions.hpp:25) */
#define MYEA_AF_COSINE 1u
#define MYEA_AF_COSINE_SYMMETRIC 2u
#define MYEA_AF_ELU 3u
#define MYEA_AF_ELLIOT 4u
#define MYEA_AF_ELLIOT_SYMMETRIC 5u
#define MYEA_AF_GAUSSIAN 6u
#define MYEA_AF_GAUSSIAN_STEPWISE 7u /* the reference's value is the constant 0 (Activation_Functions.hpp: AF_FIRE) */
#define MYEA_AF_GAUSSIAN_SYMMETRIC 8u
#define MYEA_AF_ISRU 9u
#define MYEA_AF_ISRLU 10u
#define MYEA_AF_LINEAR 11u
#define MYEA_AF_LINEAR_PIECE 12u
#define MYEA_AF_LINEAR_PIECE_SYMMETRIC 13u
#define MYEA_AF_LEAKY_RELU 14u
#define MYEA_AF_PARAMETRIC_RELU 15u /* fixed slope 0.01 in the reference (AF_PRELU_ALPHA) */
#define MYEA_AF_RELU 16u
#define MYEA_AF_SELU 17u
#define MYEA_AF_SIGMOID 18u
#define MYEA_AF_SINE 19u
#define MYEA_AF_SIGMOID_STEPWISE 20u
#define MYEA_AF_SINE_SYMMETRIC 21u
#define MYEA_AF_SOFTMAX 22u
#define MYEA_AF_TANH 23u
#define MYEA_AF_TANH_STEPWISE 24u
#define MYEA_AF_THRESHOLD 25u           /* no derivative in the reference (Activation_Function_Derive falls through */
#define MYEA_AF_THRESHOLD_SYMMETRIC 26u /* to `return value`); the same factor is used here */
/* ENUM_TYPE_LAYER_NORMALIZATION (Enum_Type_Layer_Normalization.hpp) */
#define MYEA_NORM_NONE 0u
#define MYEA_NORM_BATCH_NORMALIZATION 1u
#define MYEA_NORM_BATCH_RENORMALIZATION 2u
/* ENUM_TYPE_LAYER_DROPOUT (Enum_Type_Layer_Dropout.hpp:25) */
#define MYEA_DROPOUT_NONE 0u
#define MYEA_DROPOUT_BERNOULLI 2u
#define MYEA_DROPOUT_BERNOULLI_INVERTED 3u
#define MYEA_DROPOUT_SHAKEDROP 5u
#define MYEA_DROPOUT_ZONEOUT 7u
/* ENUM_TYPE_LOSS_FUNCTIONS / ENUM_TYPE_ACCURACY_FUNCTIONS (Enum_Type_Loss_Functions.hpp:25,58) */
#define MYEA_LOSS_CROSS_ENTROPY 2u
#define MYEA_LOSS_MSE 10u
#define MYEA_ACCURACY_NONE 0u
#define MYEA_ACCURACY_CROSS_ENTROPY 1u
#define MYEA_ACCURACY_DISTANCE 3u
/* ENUM_TYPE_OPTIMIZER_FUNCTIONS (Enum_Type_Optimizer_Functions.hpp) */
#define MYEA_OPT_ADABOUND 1u
#define MYEA_OPT_ADAM 2u
#define MYEA_OPT_AMSBOUND 4u
#define MYEA_OPT_AMSGRAD 5u
#define MYEA_OPT_GD 6u
#define MYEA_OPT_IRPROP_PLUS 8u
#define MYEA_OPT_NOSADAM 9u

/* One layer, as `struct Layer_Parameters` (Data.hpp:56-80) plus the per-layer Set__* state. */
typedef struct myea_layer_desc {
  uint32_t type_layer;        /* MYEA_LAYER_*                                                     */
  uint32_t use_bidirectional; /* Layer_Parameters::use_bidirectional (LSTM only)                  */
  uint64_t unit_parameters[5];/* [0] FC: neurons, LSTM: blocks, RESIDUAL: block depth; [1] LSTM: cells per block */
  uint32_t type_activation_function; /* Set__Layer_Activation_Function (Data.hpp:2749)           */
  uint32_t type_normalization;       /* Set__Layer_Normalization       (Data.hpp:2697)           */
  uint32_t use_layer_normalization_before_activation; /* reference default: 1                    */
  uint32_t type_dropout;             /* Set__Dropout                   (Data.hpp:2667)           */
  float dropout_values[3];    /* Bernoulli: retention probability; ShakeDrop: drop probability; Zoneout: cell, hidden */
  uint32_t reserved;
} myea_layer_desc;

/* Whole network: the arguments of Neural_Network::Compile (Data.hpp:2531) plus network-level Set__* state. */
typedef struct myea_net_desc {
  uint32_t number_layers;        /* including the input layer (layer 0, an FC desc holding the input width) */
  uint32_t type_network;         /* MYEA_NETWORK_*                                              */
  uint64_t number_recurrent_depth; /* T; 1 for feed-forward                                      */
  uint64_t number_time_delays;   /* Set__Number_Time_Delays (Data.hpp:2666)                      */
  uint64_t batch_size;           /* rows the activation buffers are carved for (Update__Batch_Size, Data.hpp:2559) */
  uint32_t type_loss_function;   /* Set__Loss_Function     (Data.hpp:832)                        */
  uint32_t type_accuracy_function; /* Set__Accuracy_Function (Data.hpp:833)                      */
  float accuracy_variance;       /* DISTANCE accuracy tolerance                                  */
  float normalization_momentum_average; /* Data.hpp:2966 */
  float normalization_epsilon;   /* Data.hpp:2967                                                */
  float batch_renormalization_r_correction_maximum; /* Data.hpp:2746                             */
  float batch_renormalization_d_correction_maximum; /* Data.hpp:2747                             */
  float clip_gradient; /* the class's clip_gradient member (Set__Clip_Gradient(T_), Data.hpp:2718) as far as it shapes the network:
                          independently recurrent layers keep their recurrent weights inside +-(MAG / c)^(1/T) after every update,
                          MAG = clip(clip_gradient, 2, 10), c = 0.9^(T/10) for symmetric activations and 1 otherwise
                          (Compute__Regularization__Constraint_Recurrent_Weight__Default); 0 = the class default 1 */
  myea_layer_desc layers[MYEA_MAX_LAYERS];
} myea_net_desc;

/* Optimizer state of the reference object read by Update_Parameter (Data.hpp:2940-2957). */
typedef struct myea_opt_desc {
  uint32_t type_optimizer_function; /* MYEA_OPT_*                                               */
  uint32_t use_adam_bias_correction;
  float learning_rate;        /* GD learning rate                                                */
  float learning_momentum;    /* GD momentum (0 = plain GD)                                      */
  uint32_t use_nesterov;
  float adam_learning_rate, adam_beta1, adam_beta2, adam_epsilon;
  float learning_rate_final, learning_gamma; /* AdaBound / AMSBound                              */
  float regularization__weight_decay;
  uint32_t use_normalized_weight_decay;
  uint32_t use_clip_gradient; /* Set__Clip_Gradient(bool)  (Data.hpp:837)                        */
  float clip_gradient;        /* Set__Clip_Gradient(T_)    (Data.hpp:2718)                       */
  float epoch_time_step;      /* divisor of the normalized weight decay (Train.cpp:284-286)      */
  float adam_gamma;           /* NosAdam: beta2_t = B/(B + t^-gamma), B += t^-gamma (Neural_Network__NosAdam.cpp:97-160); 0 = the class default 0.1 */
  float regularization__max_norm_constraints; /* Set__Regularization__Max_Norm_Constraints (Data.hpp:2744): after the update every
                                                 neuron's weight row with norm >= c is scaled to norm c; 0 = off */
  /* iRPROP+ (Neural_Network__iRPROP_plus.cpp:30-187); 0 in a factor or bound = the class default
   * (1.2, 0.5, 1e-6, 50, 0.1).  loss_rprop / previous_loss_rprop are the two members Dataset::Train_Epoch keeps
   * (Dataset.cpp:575-579): a weight whose derivative changed sign is stepped back only when loss_rprop >
   * previous_loss_rprop.  The reference assigns previous = current before the batch and the new loss after it, so
   * inside its own training loop the two are always equal at update time; a caller may pass them differently. */
  float rprop_increase_factor, rprop_decrease_factor, rprop_delta_min, rprop_delta_max, rprop_delta_zero;
  float loss_rprop, previous_loss_rprop;
  /* Set__Regularization__L1 / __L2 (Data.hpp:2742-2743).  Accepted, kept in checkpoints, and WITHOUT effect on the step, as
   * in the reference: Update_Parameter hands (batch, 0, total_weights) to routines that take (start, end, batch)
   * (Neural_Network.cpp:4729-4741, 4832-4844 against Neural_Network__Regularization__L1.cpp:99-128, __L2.cpp alike), so
   * their loops run from `batch` to 0 and never execute. */
  float regularization__l1, regularization__l2;
} myea_opt_desc;

/* Where one layer's parameters sit in the flat [P] buffer: the index map that
 * Prepare__Connections__FC/LSTM and Prepare__Bias__FC/LSTM (Neural_Network__Prepare_Connections.cpp:20-252)
 * and Allocate__Normalized_Unit (Neural_Network__Allocate.cpp:2378-2460) build.  Bit-exact with the reference. */
typedef struct myea_layer_index {
  uint64_t first_connection_index, last_connection_index;
  uint64_t first_bias_connection_index, last_bias_connection_index; /* LSTM: already shifted by the cell count, as the reference does */
  uint64_t scale_index, shift_index; /* gamma / beta of this layer's first unit; valid once any layer is normalized */
  uint64_t number_inputs, number_outputs;
  uint64_t block_stride;      /* LSTM: floats per block = 4*in + 4*cells + 3*cells_per_block     */
  uint64_t number_units_norm; /* units of this layer counted in the normalized-unit run          */
} myea_layer_index;

typedef struct myea_b200_net *myea_handle;

/* buffer selectors for upload / download */
#define MYEA_BUF_PARAMETERS 0     /* ptr_array_parameters                         (Data.hpp:3017 block) */
#define MYEA_BUF_DERIVATIVES 1    /* ptr_array_derivatives_parameters, merged [P]                       */
#define MYEA_BUF_FIRST_MOMENT 2   /* ptr_array_previous_biased_first_moment                             */
#define MYEA_BUF_SECOND_MOMENT 3  /* ptr_array_previous_biased_second_moment                            */
#define MYEA_BUF_SECOND_MOMENT_HAT 4 /* ptr_array_previous_biased_second_moment_hat (AMSGrad)           */
#define MYEA_BUF_MASK_REGULARIZED 5  /* ptr_array_mask_regularized_parameters                           */
#define MYEA_BUF_NORM_MEAN_AVERAGE 6     /* normalized_batch_units.ptr_mean_average: units x time steps, [layer][T][units] */
#define MYEA_BUF_NORM_VARIANCE_AVERAGE 7 /* normalized_batch_units.ptr_variance_average, same layout                       */
#define MYEA_BUF_PREVIOUS_DELTA 8 /* ptr_array_previous_delta_parameters (GD momentum, iRPROP+)         */
#define MYEA_BUF_PREVIOUS_DERIVATIVES 9 /* ptr_array_previous_derivatives_parameters (iRPROP+); shares the first-moment storage  */
#define MYEA_BUF_PREVIOUS_STEPS 10      /* ptr_array_previous_steps (iRPROP+; 0 reads as rprop_delta_zero); shares the second-moment storage */

/* Neural_Network::Compile + Set__* + Update__Batch_Size (Neural_Network__Compile.cpp:426-785,
 * Neural_Network__Update.cpp:187-231): builds the index map, carves device buffers for batch_size rows. */
int myea_b200_create(myea_handle *out, const myea_net_desc *desc, int device);
/* Neural_Network::Deallocate (Neural_Network__Deallocate.cpp) */
void myea_b200_destroy(myea_handle h);
const char *myea_b200_last_error(myea_handle h);

/* total_parameters / total_weights / total_bias (Data.hpp:2925-2935) and the per-layer index map. */
int myea_b200_sizes(myea_handle h, uint64_t *total_parameters, uint64_t *total_weights, uint64_t *total_bias,
                    uint64_t *total_normalized_units);
int myea_b200_layer_index(myea_handle h, uint32_t layer, myea_layer_index *out);

/* Copy__Parameters__Host_To_Device / …Device_To_Host, Copy__Optimizer_Paramaters__Device_To_Host,
 * Copy__Batch_Normalization_Neurons__Device_To_Host (Data.hpp:3112-3195): `count` floats from `offset`. */
int myea_b200_upload(myea_handle h, int which, const float *host, uint64_t offset, uint64_t count);
int myea_b200_download(myea_handle h, int which, float *host, uint64_t offset, uint64_t count);

/* Layer::ptr_array__mask__dropout__bernoulli (Data.hpp:611): bool[T][units] of layer `layer`, true = keep. */
int myea_b200_set_mask_bernoulli(myea_handle h, uint32_t layer, const uint8_t *mask, uint64_t count);
/* Cell_unit::ptr_mask_dropout_zoneout_state / _output (Data.hpp:484-485), gathered as bool[T][cells]
 * (both directions: [T][2*cells]); true = compute, false = keep the previous value. */
int myea_b200_set_mask_zoneout(myea_handle h, uint32_t layer, const uint8_t *mask_state, const uint8_t *mask_output,
                               uint64_t count);
/* Device-side replacement of Dropout_Bernoulli (Neural_Network__Dropout__Bernoulli__Loop.cpp:70-90), Dropout_Zoneout
 * (Neural_Network__Dropout__Zoneout__Loop.cpp:57-100) and the ShakeDrop draws of the forward / backward passes
 * (Neural_Network__Forward_Pass__Loop.cpp:5016-5045): fills every mask and coefficient array of the network on the GPU
 * with a counter-based generator (Philox4x32-10).  The draws are a pure function of (seed, step, layer, kind, element),
 * identical on every GPU; statistically, not bit for bit, comparable to the reference's std::mt19937 streams.
 * myea_b200_download_mask reads one array back (uint8 masks, float coefficients; zoneout as [T][dirs*cells]). */
#define MYEA_MASK_BERNOULLI 0
#define MYEA_MASK_ZONEOUT_STATE 1
#define MYEA_MASK_ZONEOUT_OUTPUT 2
#define MYEA_MASK_SHAKEDROP 3
#define MYEA_MASK_SHAKEDROP_ALPHA 4
#define MYEA_MASK_SHAKEDROP_BETA 5
int myea_b200_generate_masks(myea_handle h, uint64_t seed, uint64_t step);
int myea_b200_download_mask(myea_handle h, uint32_t layer, int kind, void *host, uint64_t bytes);

/* The caller of the step, with the dataset resident on the device.
 * myea_b200_dataset_set: `number_examples` rows of [T * inputs] and [T * outputs] floats, example-major, as
 *   Dataset::ptr_array_inputs_array[i] / ptr_array_outputs_array[i] point to them.
 * myea_b200_train_epoch: Dataset_Mini_Batch::Training_Loop (Dataset__Mini_Batch.cpp:394-436) over
 *   Dataset::Train_Batch_BP_Loop (Dataset.cpp:667-691): for every mini-batch of `order` (the host shuffles, as
 *   Dataset_Mini_Batch::Shuffle does) - reset loss, then per sub-batch of the network's batch size gather, forward,
 *   error, backward, derivative accumulation - then Update_Parameter(mini_batch_size, examples of the dataset).
 *   `mean_loss`: Get__Loss(TYPE_DATASET_NONE) averaged over the mini-batches; `accuracy_sum`: summed accuracy hits.
 *   mask_seed != 0 draws new masks before mini-batch i with myea_b200_generate_masks(seed, first_step + i).
 *   The caller advances opt->epoch_time_step between epochs as the reference does.
 *   A mini-batch is walked in sub-batches of the network's batch size, the last one shorter, and the last mini-batch
 *   of the epoch may be shorter too, as in the reference; recurrent (and multi-GPU) networks take full batches only
 *   (MYEA_E_UNSUPPORTED otherwise).
 * myea_b200_evaluate: the forward-only loop of Dataset::Testing: inference-mode forward (running normalization
 *   statistics, dropout scaling) and loss / accuracy accumulation over `number_examples` examples (`order` may be
 *   null: the first examples of the dataset); a recurrent network needs a multiple of its batch size. */
int myea_b200_dataset_set(myea_handle h, uint64_t number_examples, const float *inputs, const float *outputs);
int myea_b200_train_epoch(myea_handle h, const uint64_t *order, uint64_t number_examples, uint64_t mini_batch_size,
                          const myea_opt_desc *opt, uint64_t mask_seed, uint64_t first_step, double *mean_loss, double *accuracy_sum);
int myea_b200_evaluate(myea_handle h, const uint64_t *order, uint64_t number_examples, double *loss, double *loss_sum,
                       uint64_t *number_loss, double *accuracy_sum);

/* Checkpoint files in the reference's text format, written from and read into the device-resident network.
 * myea_b200_save_dimension_parameters: Neural_Network::Save_Dimension_Parameters (Neural_Network__Save.cpp:204-624),
 *   the `.nn` file: dimensions, every connection with its weight, biases, normalization scale / shift / running
 *   averages.  Parameters and averages are copied from the device first, as the reference does (Save.cpp:227-237).
 * myea_b200_save_general_parameters: Neural_Network::Save_General_Parameters (Save.cpp:23-202), the `.net` file:
 *   optimizer, loss, accuracy, regularization and normalization settings, taken from the handle's description and
 *   `opt`; fields of optimizers that are not built here carry the reference constructor's values.
 * myea_b200_load: Neural_Network::Load (Neural_Network__Load.cpp:2323): builds the network both files describe for
 *   `batch_size` rows on `device`, uploads parameters and averages, and returns the optimizer settings in `opt` (may
 *   be null).  Optimizer moments are in neither file (the reference does not save them): a loaded network starts
 *   with zero moments; its regularization mask covers the weights, as the reference builds it.  Bidirectional LSTM layers, pooling and independently recurrent layers: MYEA_E_UNSUPPORTED.
 * Both files are byte-identical to the reference's for the same network state, and each side reads the other's.
 *
 * The format / parse halves work on host arrays and need no GPU:
 * myea_b200_checkpoint_format_dimension / _format_general write the two files from a description, `parameters`
 *   [total_parameters] and the two average arrays (null without normalization) of total_normalized_units x
 *   number_recurrent_depth values: every time step keeps averages of its own, laid out layer after layer, each layer as
 *   [time step][its units] (Allocate__Normalized_Unit, Neural_Network__Allocate.cpp:2643-2700);
 * myea_b200_checkpoint_parse reads them back: with `parameters` null it returns the description (batch_size filled
 *   in from the argument) and the two totals; with arrays of at least those sizes it fills them as well.
 *   `path_general` may be null (description fields that live in the `.net` file then stay 0 = class default).
 * myea_b200_checkpoint_last_error: why the last parse / load on this thread failed. */
int myea_b200_save_dimension_parameters(myea_handle h, const char *path);
int myea_b200_save_general_parameters(myea_handle h, const myea_opt_desc *opt, const char *path);
int myea_b200_load(myea_handle *out, const char *path_dimension, const char *path_general, uint64_t batch_size, int device,
                   myea_opt_desc *opt);
int myea_b200_checkpoint_format_dimension(const myea_net_desc *desc, const float *parameters, const float *mean_average,
                                          const float *variance_average, const char *path);
int myea_b200_checkpoint_format_general(const myea_net_desc *desc, const myea_opt_desc *opt, const char *path);
int myea_b200_checkpoint_parse(const char *path_dimension, const char *path_general, uint64_t batch_size, myea_net_desc *desc,
                               myea_opt_desc *opt, float *parameters, uint64_t parameters_capacity, float *mean_average,
                               float *variance_average, uint64_t norm_capacity, uint64_t *total_parameters,
                               uint64_t *total_normalized_units);
const char *myea_b200_checkpoint_last_error(void);

/* ShakeDrop draws of one residual block made explicit: mask bool[B] (Layer::ptr_array__mask__dropout__shakedrop,
 * Data.hpp:612), forward coefficients alpha[B][units] and backward coefficients beta[B][units]
 * (Neural_Network__Forward_Pass__OpenMP.cpp:5021-5056, Neural_Network__Backward_Pass__OpenMP.cpp:1009-1042). */
int myea_b200_set_shakedrop(myea_handle h, uint32_t layer, const uint8_t *mask, const float *alpha, const float *beta,
                            uint64_t batch);

/* bool Set__Pre_Training_Level(size_t) (Neural_Network__Indexing.cpp:20-51): 0 = the whole network (default); k >= 1 = the step
 * functions train hidden layer k and its mirror image, layer number_layers - k, as one autoencoder pair: layers before k
 * encode in inference behaviour, the decoded layer reads the coded layer's output and is compared with what the coded
 * layer read (at level 1: the targets passed to compute_error, normally the inputs).  The decoded layer's answer is
 * read with myea_b200_get_outputs(h, number_layers - k, ...).  Feed-forward networks of plain fully connected layers,
 * no normalization on the two layers of the pair, no communicator. */
int myea_b200_set_pre_training_level(myea_handle h, uint64_t level);

/* void Forward_Pass(size_t B, T_ const *const *X, …) (Data.hpp:2896). X is the packed [T][B][inputs] block the
 * host class gathers from the reference's row pointers; host memory. training: type_state_propagation (Data.hpp:3048).
 * `batch` may be anything from 1 to the batch size the network was created for when the network is feed-forward
 * (one time step); recurrent networks and networks with a communicator take the full batch only.  The calls that
 * follow (compute_error, backward, update_derivative_weight) take the batch of the last forward pass. */
int myea_b200_forward(myea_handle h, uint64_t batch, const float *inputs_TBI, int training);
/* same, inputs already resident on this handle's GPU */
int myea_b200_forward_device(myea_handle h, uint64_t batch, const float *device_inputs_TBI, int training);
/* void Compute__Error(size_t B, T_ const *const *Y) (Data.hpp:1033). Y packed [T][B][outputs]. The loss sum, the
 * number of loss terms and the accuracy count are ACCUMULATED into the handle (ptr_array_loss_values,
 * ptr_array_number_loss, ptr_array_accuracy_values) and read with myea_b200_get_loss. */
int myea_b200_compute_error(myea_handle h, uint64_t batch, const float *desired_TBO);
int myea_b200_compute_error_device(myea_handle h, uint64_t batch, const float *device_desired_TBO);
/* Reset__Loss (Data.hpp:823) / the accumulators behind Get__Loss (Data.hpp:2913). */
int myea_b200_reset_loss(myea_handle h);
int myea_b200_get_loss(myea_handle h, double *loss_sum, uint64_t *number_loss, double *accuracy_sum);
/* void Backward_Pass(size_t B) (Data.hpp:1709) */
int myea_b200_backward(myea_handle h, uint64_t batch);
/* void Update_Derivative_Weight(size_t B, Layer *first, Layer const *end) (Data.hpp:2199), over all layers */
int myea_b200_update_derivative_weight(myea_handle h, uint64_t batch);
/* void Update_Parameter(size_t B, size_t N_train) (Data.hpp:849): merge (all-reduce when a communicator is
 * attached), clip, optimizer, zero the derivatives. */
int myea_b200_update_parameter(myea_handle h, uint64_t batch, uint64_t training_size, const myea_opt_desc *opt);
/* Clear_Training_Arrays (Data.hpp:2438): zero derivatives and optimizer moments, optimizer_time_step = 0. */
int myea_b200_clear_training_arrays(myea_handle h);
/* Layer outputs of the last forward pass, [T][B][outputs] (Get__Outputs, Data.hpp:2903), to host memory. */
int myea_b200_get_outputs(myea_handle h, uint32_t layer, float *host, uint64_t count);
/* Layer errors (Neuron_unit::ptr_array_errors / cell delta of an LSTM) of the last backward pass. */
int myea_b200_get_errors(myea_handle h, uint32_t layer, float *host, uint64_t count);

/* Merge_Derivatives_Parameters (Neural_Network__Merge.cpp:20-50) across GPUs: attach this handle to an NCCL
 * communicator of `world` ranks. `unique_id` is the 128-byte ncclUniqueId made by rank 0
 * (myea_b200_comm_unique_id) and carried to the other ranks by the caller.
 * With a communicator every rank runs the step on its rows of the batch; update_derivative_weight hands each layer's
 * derivatives to the communicator (reduce-scatter where the range divides evenly over the ranks and the update is
 * element by element, else all-reduce), update_parameter updates this rank's slices and gathers the updated parameters,
 * so that all ranks hold identical parameters afterwards (where the ranks can map each other's memory, slices and
 * updated parameters travel as peer copies with arrival words instead of library collectives; a forward pass waits
 * for a layer's parameters only where it reads them).  The optimizer state (moments, previous deltas) of a slice
 * lives on the rank that owns it: myea_b200_download of such a buffer gathers the slices first and is therefore
 * COLLECTIVE - every rank has to make the call. */
int myea_b200_comm_unique_id(uint8_t id_out[128]);
int myea_b200_comm_init(myea_handle h, int world, int rank, const uint8_t unique_id[128]);

/* Blocks until the handle's stream is idle; returns MYEA_E_KERNEL if any kernel flagged a timeout. */
int myea_b200_synchronize(myea_handle h);
/* The handle's cudaStream_t (for event timing by the caller) and counters. */
void *myea_b200_stream(myea_handle h);
uint64_t myea_b200_kernel_launches(myea_handle h);

/* Stand-alone dense contraction used by the step, exposed for kernel-level tests and roofline timing:
 * C[M,N] (+)= A[M,K] · B[N,K]^T, fp32 in HOST memory, computed on tcgen05 with split precision (TF32 main
 * product + bf16 cross terms; bit 0 of `engine` clear) or with the FP32 FMA kernel (bit 0 set).  Bits 8..16 of
 * `engine` force a tile shape (0 heuristic, 128 single CTA, 2 CTA pair 256x128, 3 CTA pair 256x256, 4 the same
 * without splitting tiles along K); bit 17 / bit 18: A / B is handed over transposed, [K][M] / [K][N] row-major,
 * and read as it lies (256x256 kernel only); bit 19: C = (A·B^T) .* relu'(C on entry), the fused activation-derivative
 * epilogue of the error-propagation product, for kernel-level tests (bits 20 / 21: timing variants of it).  `elapsed_ms` (may be null) receives the mean device time of `repeats`
 * extra runs.  Replaces the triple loops
 * Forward_Pass__FC / Backward_Pass__FC / Update_Derivative_Weight__FC
 * (Neural_Network__Forward_Pass__OpenMP.cpp:4517, …Backward_Pass__OpenMP.cpp:1044, …Update_Derivative_Weight__OpenMP.cpp:178). */
int myea_b200_gemm_nt(int device, int engine, uint64_t M, uint64_t N, uint64_t K, const float *A, const float *B,
                      float *C, int accumulate, float *elapsed_ms, int repeats);

/* No counterpart in the reference.  The same contraction for callers that cannot allocate device memory in the call
 * path (a host that reserved all GPU memory up front, a tick-driven trading loop that cannot absorb cudaMalloc's
 * device-wide synchronisation or its failure): C[M,N] (+)= A[M,K] * B[N,K]^T with A, B, C DEVICE pointers owned by
 * the caller and the operand-panel scratch in a fixed 32 MiB array inside the library image, so the call performs no
 * cudaMalloc / cudaFree.  Limit: 2*(M+N)*round_up(K,32)+64 floats <= 8 Mi floats, else MYEA_E_INVALID with a message in
 * error_message (optional, error_capacity bytes).  Every GPU that loads the library holds the array until exit.  All
 * calls share it: calls that overlap on the GPU race and must be serialised by the caller.  The first call on a
 * device looks up the array's device address.  The call is synchronous (it returns after the stream is idle and has
 * read a status word back), so never make it on a stream that is being captured.  It makes `device` current for its
 * own work and restores the caller's current device before returning. */
#define MYEA_STATIC_SCRATCH_BYTES (32u << 20)
int myea_b200_gemm_nt_static(int device, uint64_t M, uint64_t N, uint64_t K, const float *device_A, const float *device_B,
                             float *device_C, int accumulate, void *stream, char *error_message, size_t error_capacity);

/* Per-kernel-class device time of the handle since the last call with reset!=0 (CUDA events on the handle's
 * stream); classes: 0 gemm, 1 split/pack, 2 normalization, 3 elementwise, 4 optimizer, 5 recurrent cell. */
#define MYEA_TIMER_CLASSES 8
int myea_b200_profile(myea_handle h, int enable);
int myea_b200_profile_read(myea_handle h, double ms[MYEA_TIMER_CLASSES], uint64_t launches[MYEA_TIMER_CLASSES],
                           double gemm_flops[1], int reset);

#ifdef __cplusplus
}
#endif
#endif /* MYEA_B200_H */
