// The caller of the step: one epoch of mini-batch training and the evaluation pass over a dataset that stays on the
// device.  Replaces Dataset_Mini_Batch::Training_Loop (Dataset__Mini_Batch.cpp:394-436) with Dataset::Train_Batch_BP_Loop
// (Dataset.cpp:667-691) inside it, and the forward-only loop of Dataset::Testing / Measure_Accuracy.
// The reference keeps one row pointer per example ([T * width] floats each) and hands the network a window of those
// pointers; here the rows live in two device arrays and a gather kernel builds each batch in the network's
// [T][B][width] layout from the (host-shuffled) order, so an epoch moves no example over PCIe.
#include "net.cuh"

namespace myea {

// dst[(t * B + b) * W + j] = src[order[first + b] * T * W + t * W + j]
__global__ void __launch_bounds__(256) gather_batch_kernel(const float *__restrict__ src, const unsigned long long *__restrict__ order,
                                                           long long first, long long B, long long T, long long W, float *__restrict__ dst) {
  const long long total = T * B * W;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long j = i % W, tb = i / W, b = tb % B, t = tb / B;
    dst[i] = src[order[first + b] * T * W + t * W + j];
  }
}
__global__ void __launch_bounds__(256) gather_batch_vec4_kernel(const float4 *__restrict__ src, const unsigned long long *__restrict__ order,
                                                                long long first, long long B, long long T, long long W4, float4 *__restrict__ dst) {
  const long long total = T * B * W4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long j = i % W4, tb = i / W4, b = tb % B, t = tb / B;
    dst[i] = src[order[first + b] * T * W4 + t * W4 + j];
  }
}

static int gather(myea_b200_net *net, const float *src, long long first, long long B, long long W, float *dst) {
  Context &ctx = net->ctx;
  const long long total = net->T * B * W;
  ctx.begin(TC_ELEMENTWISE);
  if ((W & 3) == 0) {
    const int blocks = static_cast<int>(std::min<long long>((total / 4 + 255) / 256, 148 * 16));
    gather_batch_vec4_kernel<<<std::max(blocks, 1), 256, 0, ctx.stream>>>(reinterpret_cast<const float4 *>(src), net->ds_order, first, B, net->T,
                                                                          W / 4, reinterpret_cast<float4 *>(dst));
  } else {
    const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
    gather_batch_kernel<<<std::max(blocks, 1), 256, 0, ctx.stream>>>(src, net->ds_order, first, B, net->T, W, dst);
  }
  ctx.end(TC_ELEMENTWISE);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

static int set_order(myea_b200_net *net, const uint64_t *order, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i)
    if (order[i] >= net->ds_examples) { net->ctx.error = "an index of the order is past the end of the dataset"; return MYEA_E_INVALID; }
  if (n > net->ds_order_capacity) {
    if (net->ds_order != nullptr) cudaFree(net->ds_order);
    net->ds_order = nullptr;
    if (cudaMalloc(&net->ds_order, n * sizeof(unsigned long long)) != cudaSuccess) { net->ds_order_capacity = 0; return MYEA_E_CUDA; }
    net->ds_order_capacity = n;
  }
  if (cudaMemcpyAsync(net->ds_order, order, n * sizeof(unsigned long long), cudaMemcpyHostToDevice, net->ctx.stream) != cudaSuccess) return MYEA_E_CUDA;
  return cudaStreamSynchronize(net->ctx.stream) == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;  // `order` is the caller's memory
}

// Get__Loss(TYPE_DATASET_NONE) (Neural_Network__Loss.cpp:99-205) of the accumulators of one mini-batch
static double reference_loss(const myea_b200_net *net, double loss_sum, uint64_t number_loss) {
  if (number_loss == 0) return 1.0;
  if (net->desc.type_loss_function == MYEA_LOSS_CROSS_ENTROPY) {
    const uint64_t outputs = static_cast<uint64_t>(net->layers.back().n_out);
    return loss_sum / static_cast<double>(number_loss / outputs);
  }
  return loss_sum / static_cast<double>(number_loss);
}

}  // namespace myea

using namespace myea;

extern "C" int myea_b200_dataset_set(myea_handle net, uint64_t number_examples, const float *inputs, const float *outputs) {
  if (net == nullptr || inputs == nullptr || outputs == nullptr || number_examples == 0) return MYEA_E_INVALID;
  if (cudaSetDevice(net->ctx.device) != cudaSuccess) return MYEA_E_CUDA;
  const size_t wi = static_cast<size_t>(net->T * net->layers[0].n_out), wo = static_cast<size_t>(net->T * net->layers.back().n_out);
  for (float **p : {&net->ds_inputs, &net->ds_outputs, &net->ds_batch_inputs, &net->ds_batch_outputs}) {
    if (*p != nullptr) cudaFree(*p);
    *p = nullptr;
  }
  net->ds_examples = 0;
  if (cudaMalloc(&net->ds_inputs, number_examples * wi * sizeof(float)) != cudaSuccess ||
      cudaMalloc(&net->ds_outputs, number_examples * wo * sizeof(float)) != cudaSuccess ||
      cudaMalloc(&net->ds_batch_inputs, static_cast<size_t>(net->B) * wi * sizeof(float) + 16) != cudaSuccess ||
      cudaMalloc(&net->ds_batch_outputs, static_cast<size_t>(net->B) * wo * sizeof(float) + 16) != cudaSuccess) {
    net->ctx.error = "cudaMalloc failed (dataset)";
    return MYEA_E_CUDA;
  }
  if (cudaMemcpyAsync(net->ds_inputs, inputs, number_examples * wi * sizeof(float), cudaMemcpyHostToDevice, net->ctx.stream) != cudaSuccess ||
      cudaMemcpyAsync(net->ds_outputs, outputs, number_examples * wo * sizeof(float), cudaMemcpyHostToDevice, net->ctx.stream) != cudaSuccess ||
      cudaStreamSynchronize(net->ctx.stream) != cudaSuccess)
    return MYEA_E_CUDA;
  net->ds_examples = number_examples;
  return MYEA_OK;
}

extern "C" int myea_b200_train_epoch(myea_handle net, const uint64_t *order, uint64_t number_examples, uint64_t mini_batch_size,
                                     const myea_opt_desc *opt, uint64_t mask_seed, uint64_t first_step, double *mean_loss, double *accuracy_sum) {
  if (net == nullptr || order == nullptr || opt == nullptr || number_examples == 0) return MYEA_E_INVALID;
  if (net->ds_examples == 0) { net->ctx.error = "no dataset on the device (myea_b200_dataset_set)"; return MYEA_E_INVALID; }
  const uint64_t B = static_cast<uint64_t>(net->B);
  if (mini_batch_size == 0) return MYEA_E_INVALID;
  // Train_Batch_BP walks a mini-batch in sub-batches of the network's batch size, the last one shorter
  // (Dataset.cpp:667-691); the last mini-batch of the epoch may be shorter as well.  Ranks of a data-parallel job take
  // full batches only (see myea_b200_forward).
  if ((mini_batch_size % B != 0 || number_examples % mini_batch_size != 0) && net->comm != nullptr) {
    net->ctx.error = "train_epoch: a multi-GPU network needs a mini-batch that is a multiple of its batch size and divides the number of examples";
    return MYEA_E_UNSUPPORTED;
  }
  // With a communicator the derivative buckets are summed over the ranks inside update_derivative_weight, so a
  // mini-batch is exactly one batch: a second sub-batch would add to sums that have already travelled.
  if (net->comm != nullptr && mini_batch_size != B) {
    net->ctx.error = "train_epoch: with a communicator attached the mini-batch must equal the network's batch size";
    return MYEA_E_UNSUPPORTED;
  }
  if (cudaSetDevice(net->ctx.device) != cudaSuccess) return MYEA_E_CUDA;
  int rc = set_order(net, order, number_examples);
  if (rc != MYEA_OK) return rc;
  const long long wi = net->layers[0].n_out, wo = net->layers.back().n_out;
  const uint64_t mini_batches = (number_examples + mini_batch_size - 1) / mini_batch_size;
  double loss_total = 0.0, acc_total = 0.0;
  for (uint64_t mb = 0; mb < mini_batches; ++mb) {
    const uint64_t mb_first = mb * mini_batch_size;
    const uint64_t mb_size = std::min<uint64_t>(mini_batch_size, number_examples - mb_first);
    if (mask_seed != 0 && (rc = myea_b200_generate_masks(net, mask_seed, first_step + mb)) != MYEA_OK) return rc;
    if ((rc = myea_b200_reset_loss(net)) != MYEA_OK) return rc;
    for (uint64_t done = 0; done < mb_size; done += B) {  // derivatives accumulate over the sub-batches of one mini-batch
      const uint64_t b = std::min<uint64_t>(B, mb_size - done);
      const long long first = static_cast<long long>(mb_first + done);
      if ((rc = gather(net, net->ds_inputs, first, static_cast<long long>(b), wi, net->ds_batch_inputs)) != MYEA_OK) return rc;
      if ((rc = gather(net, net->ds_outputs, first, static_cast<long long>(b), wo, net->ds_batch_outputs)) != MYEA_OK) return rc;
      if ((rc = myea_b200_forward_device(net, b, net->ds_batch_inputs, 1)) != MYEA_OK) return rc;
      if ((rc = myea_b200_compute_error_device(net, b, net->ds_batch_outputs)) != MYEA_OK) return rc;
      if ((rc = myea_b200_backward(net, b)) != MYEA_OK) return rc;
      if ((rc = myea_b200_update_derivative_weight(net, b)) != MYEA_OK) return rc;
    }
    double ls = 0.0, as = 0.0;
    uint64_t nl = 0;
    if ((rc = myea_b200_get_loss(net, &ls, &nl, &as)) != MYEA_OK) return rc;
    loss_total += reference_loss(net, ls, nl);
    acc_total += as;
    if ((rc = myea_b200_update_parameter(net, mb_size, net->ds_examples, opt)) != MYEA_OK) return rc;
  }
  if (mean_loss != nullptr) *mean_loss = loss_total / static_cast<double>(mini_batches);
  if (accuracy_sum != nullptr) *accuracy_sum = acc_total;
  return MYEA_OK;
}

extern "C" int myea_b200_evaluate(myea_handle net, const uint64_t *order, uint64_t number_examples, double *loss, double *loss_sum,
                                  uint64_t *number_loss, double *accuracy_sum) {
  if (net == nullptr || number_examples == 0) return MYEA_E_INVALID;
  if (net->ds_examples == 0) { net->ctx.error = "no dataset on the device (myea_b200_dataset_set)"; return MYEA_E_INVALID; }
  const uint64_t B = static_cast<uint64_t>(net->B);
  if (number_examples % B != 0 && net->comm != nullptr) {
    net->ctx.error = "evaluate: a multi-GPU network needs a number of examples that is a multiple of its batch size";
    return MYEA_E_UNSUPPORTED;
  }
  if (cudaSetDevice(net->ctx.device) != cudaSuccess) return MYEA_E_CUDA;
  std::vector<uint64_t> identity;
  if (order == nullptr) {
    if (number_examples > net->ds_examples) return MYEA_E_INVALID;
    identity.resize(number_examples);
    for (uint64_t i = 0; i < number_examples; ++i) identity[i] = i;
    order = identity.data();
  }
  int rc = set_order(net, order, number_examples);
  if (rc != MYEA_OK) return rc;
  const long long wi = net->layers[0].n_out, wo = net->layers.back().n_out;
  if ((rc = myea_b200_reset_loss(net)) != MYEA_OK) return rc;
  for (uint64_t first = 0; first < number_examples; first += B) {
    const uint64_t b = std::min<uint64_t>(B, number_examples - first);
    if ((rc = gather(net, net->ds_inputs, static_cast<long long>(first), static_cast<long long>(b), wi, net->ds_batch_inputs)) != MYEA_OK) return rc;
    if ((rc = gather(net, net->ds_outputs, static_cast<long long>(first), static_cast<long long>(b), wo, net->ds_batch_outputs)) != MYEA_OK) return rc;
    if ((rc = myea_b200_forward_device(net, b, net->ds_batch_inputs, 0)) != MYEA_OK) return rc;   // inference: running statistics, no masks
    if ((rc = myea_b200_compute_error_device(net, b, net->ds_batch_outputs)) != MYEA_OK) return rc;
  }
  double ls = 0.0, as = 0.0;
  uint64_t nl = 0;
  if ((rc = myea_b200_get_loss(net, &ls, &nl, &as)) != MYEA_OK) return rc;
  if (loss != nullptr) *loss = reference_loss(net, ls, nl);
  if (loss_sum != nullptr) *loss_sum = ls;
  if (number_loss != nullptr) *number_loss = nl;
  if (accuracy_sum != nullptr) *accuracy_sum = as;
  return MYEA_OK;
}
