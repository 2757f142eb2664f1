// Checkpoint files in the reference's text format: the `.nn` file of Save_Dimension_Parameters
// (Neural_Network__Save.cpp:204-624: dimensions, every connection with its weight, normalization statistics) and the
// `.net` file of Save_General_Parameters (Neural_Network__Save.cpp:23-202: optimizer, loss, regularization and
// normalization settings), written from and read into the device-resident network, so that a model trained by the
// reference continues here and the other way round.  The text is produced byte for byte as the reference produces it:
// "\r\n" line ends, integers through std::to_string, reals as `ostream << defaultfloat << setprecision(16)` of the
// fp32 value (String.hpp:103-121), which is "%.16g" of the value widened to double and therefore round-trips exactly.
//
// Everything here is host code.  The format/parse halves take plain host arrays and need no GPU; the save/load halves
// move the parameters and the normalization averages between the device and those arrays.
//
// What the reference writes and this file follows:
//   * unit numbering is global per unit kind: neurons over all fully connected layers (input layer first), cells over
//     all LSTM layers, basic units over all residual layers; a connection names the unit it reads by that number,
//   * once any layer is normalized every layer lists its normalized units, with values only where the layer's own
//     type_normalization is set (Information__Layer__Normalization, Save.cpp:626-676),
//   * inside a residual block the first layer has no activation units and every later layer has as many as its input
//     is wide (Assign__Post__Residual_Layer, Neural_Network__Compile.cpp:340-400),
//   * an LSTM layer lists 3 * blocks bias values starting at the index already shifted by the cell count
//     (Information__Layer__Bias, Save.cpp:865-879, on the range Prepare__Bias__LSTM leaves),
//   * optimizer moments are not part of either file.
#include "net.cuh"

#include <cfloat>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

using namespace myea;

namespace {

const char *const NL = "\r\n";

std::string real(float v) {
  char buf[64];
  snprintf(buf, sizeof buf, "%.16g", static_cast<double>(v));
  return buf;
}
std::string real(double v, int precision) {
  char buf[64];
  snprintf(buf, sizeof buf, "%.*g", precision, v);
  return buf;
}
std::string num(uint64_t v) { return std::to_string(v); }

// ENUM_TYPE_LAYER_ACTIVATION of an activation function (Activation_Function__To__Class_Activation_Function,
// Train.cpp:454-497), for the functions this library runs
uint32_t activation_class(uint32_t af) {
  switch (af) {
    case MYEA_AF_COSINE_SYMMETRIC: case MYEA_AF_ELLIOT_SYMMETRIC: case MYEA_AF_GAUSSIAN_SYMMETRIC: case MYEA_AF_LINEAR_PIECE_SYMMETRIC:
    case MYEA_AF_SINE_SYMMETRIC: case MYEA_AF_TANH: case MYEA_AF_TANH_STEPWISE: case MYEA_AF_THRESHOLD_SYMMETRIC: return 5u;  // symmetric
    case MYEA_AF_COSINE: case MYEA_AF_ELU: case MYEA_AF_ELLIOT: case MYEA_AF_GAUSSIAN: case MYEA_AF_GAUSSIAN_STEPWISE: case MYEA_AF_ISRU:
    case MYEA_AF_ISRLU: case MYEA_AF_LINEAR: case MYEA_AF_LINEAR_PIECE: case MYEA_AF_SIGMOID: case MYEA_AF_SINE: case MYEA_AF_SIGMOID_STEPWISE:
    case MYEA_AF_THRESHOLD: return 1u;                                                                                           // asymmetric
    case MYEA_AF_LEAKY_RELU: case MYEA_AF_PARAMETRIC_RELU: case MYEA_AF_RELU: return 2u;                                          // rectifier
    case MYEA_AF_SELU: return 3u;                                                                                                // self-normalization
    case MYEA_AF_SOFTMAX: return 4u;
    default: return 0u;
  }
}

// a network description turned into the layer plan, with no device behind it
struct HostPlan {
  std::unique_ptr<myea_b200_net> net;
  std::vector<uint64_t> unit_base;  // first global unit number of each layer, in the numbering of its own unit kind
  std::vector<int> block_of;        // residual layer a layer sits in, or 0
  uint64_t neurons = 0, cells = 0, blocks = 0, basics = 0, basic_indices = 0, af_units = 0, af_ind_units = 0;
  std::vector<uint64_t> af_count;   // activation units each layer lists
  std::vector<uint64_t> ind_base;   // first global AF_Ind_recurrent unit number of an independently recurrent layer
  std::vector<int> reads;           // the layer whose units a layer's connections name
  std::string error;
};

int make_plan(const myea_net_desc *desc, HostPlan &P) {
  if (desc == nullptr || desc->number_layers < 2 || desc->number_layers > MYEA_MAX_LAYERS) { P.error = "bad network description"; return MYEA_E_INVALID; }
  P.net.reset(new myea_b200_net());
  P.net->desc = *desc;
  P.net->T = static_cast<long long>(desc->number_recurrent_depth);
  P.net->B = static_cast<long long>(desc->batch_size);
  const int rc = build_index_map(P.net.get());
  if (rc != MYEA_OK) { P.error = P.net->ctx.error; return rc; }
  const std::vector<LayerPlan> &Ls = P.net->layers;
  const size_t n = Ls.size();
  P.unit_base.assign(n, 0);
  P.block_of.assign(n, 0);
  P.af_count.assign(n, 0);
  P.reads.assign(n, 0);
  for (size_t l = 0; l < n; ++l)
    if (Ls[l].type == MYEA_LAYER_RESIDUAL)
      for (int k = 1; k <= Ls[l].block_depth; ++k) P.block_of[l + k] = static_cast<int>(l);
  // the first layer of a block reads what the residual layer reads (the previous block's output when blocks follow
  // one another); every other layer reads its own input layer
  for (size_t l = 1; l < n; ++l)
    P.reads[l] = (P.block_of[l] != 0 && static_cast<int>(l) == P.block_of[l] + 1) ? Ls[P.block_of[l]].input_layer : Ls[l].input_layer;
  for (size_t l = 0; l < n; ++l) {
    const LayerPlan &L = Ls[l];
    if (L.desc.use_bidirectional) { P.error = "bidirectional layers have no usable definition in the reference's files"; return MYEA_E_UNSUPPORTED; }
    switch (L.type) {
      case MYEA_LAYER_FULLY_CONNECTED:
        P.unit_base[l] = P.neurons;   // its readers name neuron units, also when the layer is independently recurrent (Save.cpp:731-738)
        P.neurons += L.n_out;
        if (L.ind_rnn) {  // it lists AF_Ind_recurrent units instead of plain activation units
          P.ind_base.resize(n, 0);
          P.ind_base[l] = P.af_ind_units;
          P.af_ind_units += L.n_out;
          break;
        }
        if (P.block_of[l] == 0) P.af_count[l] = L.n_out;
        else P.af_count[l] = (static_cast<int>(l) == P.block_of[l] + 1) ? 0 : L.n_in;
        P.af_units += P.af_count[l];
        break;
      case MYEA_LAYER_LSTM:
        P.unit_base[l] = P.cells;
        P.cells += L.n_out;
        P.blocks += L.desc.unit_parameters[0];
        break;
      case MYEA_LAYER_RESIDUAL:
      case MYEA_LAYER_AVERAGE_POOLING:   // Basic_unit, like the outputs of a residual block
        P.unit_base[l] = P.basics;
        P.basics += L.n_out;
        break;
      case MYEA_LAYER_MAX_POOLING:       // Basic_indice_unit
        P.unit_base[l] = P.basic_indices;
        P.basic_indices += L.n_out;
        break;
      default: P.error = "layer type not built"; return MYEA_E_UNSUPPORTED;
    }
  }
  return MYEA_OK;
}

// ENUM_TYPE_LAYER_CONNECTION_NAME (Enum_Type_Layer.hpp:56-68) of the layer a connection reads
const char *connection_name(uint32_t type_layer) {
  switch (type_layer) {
    case MYEA_LAYER_LSTM: return "connected_to_cell";
    case MYEA_LAYER_RESIDUAL: case MYEA_LAYER_AVERAGE_POOLING: return "connected_to_basic";
    case MYEA_LAYER_MAX_POOLING: return "connected_to_basic_indice";
    default: return "connected_to_neuron";
  }
}

struct Writer {
  const HostPlan &P;
  const float *params, *mean, *sigma;
  std::string out;
  Writer(const HostPlan &p, const float *a, const float *m, const float *s) : P(p), params(a), mean(m), sigma(s) {}
  const myea_b200_net &net() const { return *P.net; }

  void line(int indent, const std::string &key, const std::string &value) {
    out.append(static_cast<size_t>(indent), ' ');
    out += key;
    if (!value.empty()) { out += ' '; out += value; }
    out += NL;
  }
  void weight(uint64_t index) { line(10, "weight[" + num(index) + "]", real(params[index])); }

  void dropout(const LayerPlan &L, bool hidden) {
    line(4, "type_dropout", num(L.desc.type_dropout));
    if (hidden) line(6, "use_coded_dropout", "0");
    // Set__Dropout stores the values only with a dropout type; without one the reference's three slots stay 0
    for (int k = 0; k < 3; ++k) line(6, "dropout_values[" + num(k) + "]", real(L.desc.type_dropout == MYEA_DROPOUT_NONE ? 0.f : L.desc.dropout_values[k]));
  }

  void normalization(const LayerPlan &L) {
    line(4, "type_normalization", num(L.desc.type_normalization));
    if (L.type == MYEA_LAYER_FULLY_CONNECTED) line(6, "use_layer_normalization_before_activation", num(L.desc.use_layer_normalization_before_activation ? 1 : 0));
    const uint64_t units = net().any_norm ? L.idx.number_units_norm : 0;
    line(6, "number_normalized_units", num(units));
    const uint64_t T = static_cast<uint64_t>(net().T);
    for (uint64_t u = 0; u < units; ++u) {
      line(8, "NormU[" + num(u) + "]", "");
      if (L.desc.type_normalization == MYEA_NORM_NONE) continue;
      line(10, "scale", real(params[L.idx.scale_index + u]));
      line(10, "shift", real(params[L.idx.shift_index + u]));
      for (uint64_t t = 0; t < T; ++t) {
        const uint64_t at = static_cast<uint64_t>(L.norm_unit_offset) * T + t * units + u;  // [layer][T][units]
        line(10, "mean_average[" + num(t) + "]", real(mean[at]));
        line(10, "variance_average[" + num(t) + "]", real(sigma[at]));
      }
    }
  }

  void sparsity_and_constraints(const LayerPlan *L = nullptr) {
    line(4, "use_tied_parameter", "0");
    line(4, "k_sparsity", "0");
    line(4, "alpha_sparsity", "1");
    if (L != nullptr && L->ind_rnn) {  // the default bound of the layer's recurrent weights
      const float b = ind_rnn_weight_bound(net().desc.clip_gradient, L->desc.type_activation_function, net().T);
      line(4, "constraint_recurrent_weight_lower_bound", real(-b));
      line(4, "constraint_recurrent_weight_upper_bound", real(b));
      return;
    }
    line(4, "constraint_recurrent_weight_lower_bound", "0");
    line(4, "constraint_recurrent_weight_upper_bound", "0");
  }

  void neurons(size_t l, const char *count_key) {
    const LayerPlan &L = net().layers[l];
    const LayerPlan &in = net().layers[P.reads[l]];
    const char *name = connection_name(in.type);
    const uint64_t base = P.unit_base[P.reads[l]];
    line(4, count_key, num(L.n_out));
    for (long long i = 0; i < L.n_out; ++i) {
      line(6, "Neuron_unit[" + num(i) + "]", "");
      line(8, "number_connections", num(L.n_in));
      const uint64_t first = L.idx.first_connection_index + static_cast<uint64_t>(i) * L.n_in;
      for (long long j = 0; j < L.n_in; ++j) {
        line(10, name, num(base + j));
        weight(first + j);
      }
    }
  }

  void activation_units(size_t l) {
    const LayerPlan &L = net().layers[l];
    line(4, "number_AF_units", num(P.af_count[l]));
    for (uint64_t i = 0; i < P.af_count[l]; ++i) {
      line(6, "AF[" + num(i) + "]", "");
      line(8, "activation_steepness", "1");
      line(8, "activation_function", num(L.desc.type_activation_function));
    }
  }

  // Information__Layer__AF_Ind_Recurrent (Save.cpp:844-863): activation and the self connection of every unit
  void ind_recurrent_units(size_t l) {
    const LayerPlan &L = net().layers[l];
    line(4, "number_AF_Ind_recurrent_units", num(L.n_out));
    const uint64_t first = L.idx.first_connection_index + static_cast<uint64_t>(L.n_out) * L.n_in;
    for (long long i = 0; i < L.n_out; ++i) {
      line(6, "AF_Ind_R[" + num(i) + "]", "");
      line(8, "activation_steepness", "1");
      line(8, "activation_function", num(L.desc.type_activation_function));
      line(8, "connected_to_AF_Ind_R", num(P.ind_base[l] + i));
      line(8, "weight[" + num(first + i) + "]", real(params[first + i]));
    }
  }

  void bias(const LayerPlan &L) {
    const uint64_t count = L.idx.last_bias_connection_index - L.idx.first_bias_connection_index;
    line(4, "number_bias_parameters", num(count));
    for (uint64_t k = 0; k < count; ++k) line(6, "weight[" + num(L.idx.first_bias_connection_index + k) + "]", real(params[L.idx.first_bias_connection_index + k]));
  }

  // one block: Layer__LSTM_Information__Connection (Save.cpp:958-1098) walks the block's parameters in storage order
  void lstm_blocks(size_t l) {
    const LayerPlan &L = net().layers[l];
    const LayerPlan &in = net().layers[P.reads[l]];
    const char *name = connection_name(in.type);
    const uint64_t in_base = P.unit_base[P.reads[l]], cell_base = P.unit_base[l];
    const uint64_t blocks = L.desc.unit_parameters[0], cpb = std::max<uint64_t>(1, L.desc.unit_parameters[1]);
    const uint64_t cells = blocks * cpb, n_in = static_cast<uint64_t>(L.n_in);
    line(4, "number_block_units", num(blocks));
    line(4, "number_cell_units", num(cells));
    for (uint64_t b = 0; b < blocks; ++b) {
      line(6, "Block[" + num(b) + "]", "");
      line(8, "activation_function", num(MYEA_AF_TANH));
      line(8, "activation_steepness", "1");
      line(8, "number_connections", num(L.idx.block_stride));
      uint64_t w = L.idx.first_connection_index + b * L.idx.block_stride;
      auto feedforward = [&]() { for (uint64_t j = 0; j < n_in; ++j) { line(10, name, num(in_base + j)); weight(w++); } };
      auto recurrent = [&]() { for (uint64_t j = 0; j < cells; ++j) { line(10, "connected_to_cell", num(cell_base + j)); weight(w++); } };
      auto peephole = [&]() { for (uint64_t j = 0; j < cpb; ++j) { line(10, "connected_to_cell", num(cell_base + b * cpb + j)); weight(w++); } };
      for (uint64_t c = 0; c < cpb; ++c) { feedforward(); recurrent(); }
      for (int g = 0; g < 3; ++g) feedforward();
      for (int g = 0; g < 3; ++g) recurrent();
      for (int g = 0; g < 3; ++g) peephole();
    }
  }
};

}  // namespace

namespace {

int write_file(const char *path, const std::string &text, std::string &error) {
  std::ofstream f(path, std::ios::out | std::ios::binary | std::ios::trunc);
  if (!f.is_open()) { error = std::string("cannot open ") + path; return MYEA_E_INVALID; }
  f.write(text.data(), static_cast<std::streamsize>(text.size()));
  f.flush();
  if (f.fail()) { error = std::string("write failed on ") + path; return MYEA_E_INVALID; }
  return MYEA_OK;
}

// the `.nn` text (Save_Dimension_Parameters, Save.cpp:239-570)
int format_dimension(const HostPlan &P, const float *params, const float *mean, const float *sigma, std::string &text) {
  const myea_b200_net &net = *P.net;
  const std::vector<LayerPlan> &Ls = net.layers;
  const size_t n = Ls.size();
  Writer w(P, params, mean, sigma);
  w.out.reserve(64 + static_cast<size_t>(net.total_parameters) * 64);
  w.line(0, "|===| DIMENSION |===|", "");
  w.line(0, "type_network", num(net.desc.type_network));
  w.line(0, "number_layers", num(n));
  w.line(0, "number_recurrent_depth", num(net.desc.number_recurrent_depth));
  w.line(0, "number_time_delays", num(net.desc.number_time_delays));
  w.line(0, "use_first_layer_as_input", "1");
  w.line(0, "use_last_layer_as_output", "1");
  w.line(0, "total_basic_units", num(P.basics));
  w.line(0, "total_basic_indice_units", num(P.basic_indices));
  w.line(0, "total_neuron_units", num(P.neurons));
  w.line(0, "total_AF_units", num(P.af_units));
  w.line(0, "total_AF_Ind_recurrent_units", num(P.af_ind_units));
  w.line(0, "total_block_units", num(P.blocks));
  w.line(0, "total_cell_units", num(P.cells));
  w.line(0, "total_normalized_units", num(net.total_norm_units));
  w.line(0, "total_parameters", num(net.total_parameters));
  w.line(0, "total_weights", num(net.total_weights));
  w.line(0, "total_bias", num(net.total_bias));

  w.line(2, "Input layer:", "");
  w.line(4, "type_layer", num(Ls[0].type));
  w.line(4, "type_activation", "0");
  w.dropout(Ls[0], false);
  w.line(4, "number_inputs", num(Ls[0].n_out));

  for (size_t l = 1; l + 1 < n; ++l) {
    const LayerPlan &L = Ls[l];
    w.line(2, "Hidden layer " + num(l) + ":", "");
    w.line(4, "type_layer", num(L.desc.type_layer));
    w.line(4, "use_bidirectional", "0");
    switch (L.type) {
      case MYEA_LAYER_FULLY_CONNECTED:
        w.line(4, "type_activation", num(activation_class(L.desc.type_activation_function)));
        w.dropout(L, true);
        w.normalization(L);
        w.sparsity_and_constraints(&L);
        w.neurons(l, "number_neuron_units");
        if (L.ind_rnn) w.ind_recurrent_units(l);
        else w.activation_units(l);
        w.bias(L);
        break;
      case MYEA_LAYER_LSTM:
        w.line(4, "type_activation", "5");  // Prepare__Connections__LSTM sets TYPE_ACTIVATION_SYMMETRIC (Prepare_Connections.cpp:119)
        w.dropout(L, true);
        w.normalization(L);
        w.sparsity_and_constraints();
        w.lstm_blocks(l);
        w.bias(L);
        break;
      case MYEA_LAYER_AVERAGE_POOLING:
      case MYEA_LAYER_MAX_POOLING:   // (Save.cpp:305-311, 487-493; the ceil mode is not in the file)
        w.line(4, "kernel_size", num(L.desc.unit_parameters[0]));
        w.line(4, "stride", num(L.desc.unit_parameters[1]));
        w.line(4, "padding", num(L.desc.unit_parameters[2]));
        w.line(4, "dilation", num(L.desc.unit_parameters[3]));
        w.line(4, L.type == MYEA_LAYER_MAX_POOLING ? "number_basic_indice_units" : "number_basic_units", num(L.n_out));
        break;
      case MYEA_LAYER_RESIDUAL: {
        const long long a = Ls[L.input_layer].n_out, b = Ls[l + L.block_depth].n_out;
        w.line(4, "block_depth", num(static_cast<uint64_t>(L.block_depth)));
        w.line(4, "padding", num(static_cast<uint64_t>(((a > b ? a - b : b - a) + 1) / 2)));
        w.dropout(L, true);
        w.normalization(L);
        w.line(4, "number_basic_units", num(L.n_out));
        break;
      }
      default: return MYEA_E_UNSUPPORTED;
    }
  }

  const LayerPlan &O = Ls[n - 1];
  w.line(2, "Output layer:", "");
  w.line(4, "type_layer", num(O.type));
  w.line(4, "type_activation", num(activation_class(O.desc.type_activation_function)));
  w.neurons(n - 1, "number_outputs");
  w.activation_units(n - 1);
  w.bias(O);
  w.line(0, "|END| DIMENSION |END|", "");
  text.swap(w.out);
  return MYEA_OK;
}

// value of a descriptor field where 0 stands for the reference class's default
float or_default(float v, float dflt) { return v > 0.f ? v : dflt; }

// the `.net` text (Save_General_Parameters, Save.cpp:42-149).  Fields of optimizers this library does not run
// (QuickProp, SARPROP, warm restarts) carry the reference constructor's values so that its loader accepts the file.
std::string format_general(const myea_net_desc &d, const myea_opt_desc &o) {
  std::string s;
  auto put = [&](const char *key, const std::string &value) { s += key; s += ' '; s += value; s += NL; };
  auto open = [&](const char *name) { s += "|===| "; s += name; s += " |===|"; s += NL; };
  auto close = [&](const char *name, bool blank = true) { s += "|END| "; s += name; s += " |END|"; s += NL; if (blank) s += NL; };
  open("GRADIENT DESCENT PARAMETERS");
  put("learning_rate", real(o.learning_rate));
  put("learning_rate_final", real(o.learning_rate_final));
  put("learning_momentum", real(o.learning_momentum));
  put("learning_gamma", real(o.learning_gamma));
  put("use_Nesterov", num(o.use_nesterov ? 1 : 0));
  close("GRADIENT DESCENT PARAMETERS");
  open("QUICKPROP PARAMETERS");
  put("quickprop_decay", real(-0.0001f));
  put("quickprop_mu", real(1.75f));
  close("QUICKPROP PARAMETERS");
  open("RESILLENT PROPAGATION PARAMETERS");
  put("rprop_increase_factor", real(or_default(o.rprop_increase_factor, 1.2f)));
  put("rprop_decrease_factor", real(or_default(o.rprop_decrease_factor, 0.5f)));
  put("rprop_delta_min", real(or_default(o.rprop_delta_min, 1e-6f)));
  put("rprop_delta_max", real(or_default(o.rprop_delta_max, 50.f)));
  put("rprop_delta_zero", real(or_default(o.rprop_delta_zero, 0.1f)));
  close("RESILLENT PROPAGATION PARAMETERS");
  open("SARPROP PARAMETERS");
  put("sarprop_weight_decay_shift", real(-6.644f));
  put("sarprop_step_error_threshold_factor", real(0.1f));
  put("sarprop_step_error_shift", real(1.385f));
  put("sarprop_temperature", real(0.015f));
  put("sarprop_epoch", "0");
  close("SARPROP PARAMETERS");
  open("ADAM PARAMETERS");
  put("adam_learning_rate", real(o.adam_learning_rate));
  put("adam_beta1", real(o.adam_beta1));
  put("adam_beta2", real(o.adam_beta2));
  put("adam_epsilon", real(o.adam_epsilon));
  put("adam_bias_correction", num(o.use_adam_bias_correction ? 1 : 0));
  put("adam_gamma", real(or_default(o.adam_gamma, 0.1f)));
  close("ADAM PARAMETERS");
  open("WARM RESTARTS PARAMETERS");
  put("use_Warm_Restarts", "0");
  put("warm_restarts_decay_learning_rate", real(1.f));
  put("warm_restarts_maximum_learning_rate", real(1.f));
  put("warm_restarts_minimum_learning_rate", real(1e-7f));
  put("warm_restarts_initial_T_i", "1");
  put("warm_restarts_multiplier", "2");
  close("WARM RESTARTS PARAMETERS");
  open("TRAINING PARAMETERS");
  put("type_optimizer_function", num(o.type_optimizer_function));
  put("type_loss_function", num(d.type_loss_function));
  put("type_accuracy_function", num(d.type_accuracy_function));
  put("bit_fail_limit", real(0.35f));
  put("pre_training_level", "0");
  put("use_clip_gradient", num(o.use_clip_gradient ? 1 : 0));
  put("clip_gradient", real(o.use_clip_gradient ? o.clip_gradient : or_default(o.clip_gradient, 1.f)));
  close("TRAINING PARAMETERS");
  open("REGULARIZATION PARAMETERS");
  put("regularization__max_norm_constraints", real(o.regularization__max_norm_constraints));
  put("regularization__l1", real(o.regularization__l1));
  put("regularization__l2", real(o.regularization__l2));
  put("regularization__srip", "0");
  put("regularization__weight_decay", real(o.regularization__weight_decay));
  put("use_normalized_weight_decay", num(o.use_normalized_weight_decay ? 1 : 0));
  close("REGULARIZATION PARAMETERS");
  open("NORMALIZATION PARAMETERS");
  put("normalization_momentum_average", real(or_default(d.normalization_momentum_average, 0.999f)));
  put("normalization_epsilon", real(or_default(d.normalization_epsilon, 1e-5f)));
  put("batch_renormalization_r_correction_maximum", real(or_default(d.batch_renormalization_r_correction_maximum, 1.f)));
  put("batch_renormalization_d_correction_maximum", real(or_default(d.batch_renormalization_d_correction_maximum, 0.f)));
  close("NORMALIZATION PARAMETERS");
  open("LOSS PARAMETERS");
  put("loss_training", real(FLT_MAX));
  put("loss_validating", real(FLT_MAX));
  put("loss_testing", real(FLT_MAX));
  close("LOSS PARAMETERS");
  open("ACCURANCY PARAMETERS");
  put("accuracy_variance", real(or_default(d.accuracy_variance, 0.49f)));
  put("accuracy_training", "0");
  put("accuracy_validating", "0");
  put("accuracy_testing", "0");
  close("ACCURANCY PARAMETERS");
  open("COMPUTATION PARAMETERS");
  put("use_CUDA", "0");
  put("use_OpenMP", "0");
  put("percentage_maximum_thread_usage", real(100.0, 9));
  put("maximum_batch_size", num(UINT64_MAX));
  close("COMPUTATION PARAMETERS", false);
  return s;
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------
// writing
// ---------------------------------------------------------------------------------------------------------
extern "C" int myea_b200_checkpoint_format_dimension(const myea_net_desc *desc, const float *parameters, const float *mean_average,
                                                     const float *variance_average, const char *path) {
  if (desc == nullptr || parameters == nullptr || path == nullptr) return MYEA_E_INVALID;
  HostPlan P;
  const int rc = make_plan(desc, P);
  if (rc != MYEA_OK) return rc;
  if (P.net->any_norm && (mean_average == nullptr || variance_average == nullptr)) return MYEA_E_INVALID;
  std::string text, error;
  const int fr = format_dimension(P, parameters, mean_average, variance_average, text);
  if (fr != MYEA_OK) return fr;
  return write_file(path, text, error);
}

extern "C" int myea_b200_checkpoint_format_general(const myea_net_desc *desc, const myea_opt_desc *opt, const char *path) {
  if (desc == nullptr || opt == nullptr || path == nullptr) return MYEA_E_INVALID;
  std::string error;
  return write_file(path, format_general(*desc, *opt), error);
}

extern "C" int myea_b200_save_dimension_parameters(myea_handle net, const char *path) {
  if (net == nullptr || path == nullptr) return MYEA_E_INVALID;
  HostPlan P;
  int rc = make_plan(&net->desc, P);
  if (rc != MYEA_OK) { net->ctx.error = P.error; return rc; }
  const uint64_t averages = net->total_norm_units * static_cast<uint64_t>(net->T);  // one set per time step
  std::vector<float> params(net->total_parameters + 1), mean(averages + 1), sigma(averages + 1);
  rc = myea_b200_download(net, MYEA_BUF_PARAMETERS, params.data(), 0, net->total_parameters);
  if (rc == MYEA_OK && averages != 0) {
    rc = myea_b200_download(net, MYEA_BUF_NORM_MEAN_AVERAGE, mean.data(), 0, averages);
    if (rc == MYEA_OK) rc = myea_b200_download(net, MYEA_BUF_NORM_VARIANCE_AVERAGE, sigma.data(), 0, averages);
  }
  if (rc != MYEA_OK) return rc;
  std::string text;
  rc = format_dimension(P, params.data(), mean.data(), sigma.data(), text);
  if (rc != MYEA_OK) { net->ctx.error = "layer type without a text form"; return rc; }
  return write_file(path, text, net->ctx.error);
}

extern "C" int myea_b200_save_general_parameters(myea_handle net, const myea_opt_desc *opt, const char *path) {
  if (net == nullptr || opt == nullptr || path == nullptr) return MYEA_E_INVALID;
  return write_file(path, format_general(net->desc, *opt), net->ctx.error);
}

// ---------------------------------------------------------------------------------------------------------
// reading
// ---------------------------------------------------------------------------------------------------------
namespace {

// the file as (key, value) lines; Load (Neural_Network__Load.cpp:2323-6880) reads the same pairs with `>>`
struct Lines {
  std::vector<std::pair<std::string, std::string>> kv;
  size_t at = 0;
  std::string error;

  bool read(const char *path) {
    std::ifstream f(path, std::ios::in | std::ios::binary);
    if (!f.is_open()) { error = std::string("cannot open ") + path; return false; }
    std::string line;
    while (std::getline(f, line)) {
      while (!line.empty() && (line.back() == '\r' || line.back() == ' ' || line.back() == '\n')) line.pop_back();
      size_t b = 0;
      while (b < line.size() && line[b] == ' ') ++b;
      if (b == line.size()) continue;
      if (line[b] == '|') { kv.emplace_back(line.substr(b), ""); continue; }  // section markers contain spaces
      const size_t sp = line.find(' ', b);
      if (sp == std::string::npos) kv.emplace_back(line.substr(b), "");
      else kv.emplace_back(line.substr(b, sp - b), line.substr(sp + 1));
    }
    return true;
  }
  bool done() const { return at >= kv.size(); }
  const std::string &key() const { static const std::string none; return done() ? none : kv[at].first; }
  bool fail(const std::string &what) {
    if (error.empty()) error = what + " (entry " + std::to_string(at) + (done() ? ", end of file" : ", found \"" + kv[at].first + "\"") + ")";
    return false;
  }
  // the next line must carry `name` (a "name[...]" key matches its stem when `stem` is set)
  bool take(const char *name, std::string *value, bool stem = false) {
    if (done()) return fail(std::string("expected ") + name);
    const std::string &k = kv[at].first;
    const size_t len = strlen(name);
    const bool ok = stem ? (k.compare(0, len, name) == 0 && k.size() > len && k[len] == '[') : (k == name);
    if (!ok) return fail(std::string("expected ") + name);
    if (value) *value = kv[at].second;
    ++at;
    return true;
  }
  bool take_u64(const char *name, uint64_t *v, bool stem = false) {
    std::string s;
    if (!take(name, &s, stem)) return false;
    char *end = nullptr;
    *v = strtoull(s.c_str(), &end, 10);
    return (end != s.c_str()) || fail(std::string("no integer after ") + name);
  }
  bool take_real(const char *name, float *v, bool stem = false) {
    std::string s;
    if (!take(name, &s, stem)) return false;
    char *end = nullptr;
    *v = static_cast<float>(strtod(s.c_str(), &end));
    return (end != s.c_str()) || fail(std::string("no number after ") + name);
  }
  // "weight[index] value": both numbers
  bool take_weight(uint64_t *index, float *v) {
    if (done() || kv[at].first.compare(0, 7, "weight[") != 0) return fail("expected weight[...]");
    *index = strtoull(kv[at].first.c_str() + 7, nullptr, 10);
    *v = static_cast<float>(strtod(kv[at].second.c_str(), nullptr));
    ++at;
    return true;
  }
};

struct NormValues { std::vector<float> scale, shift, mean, sigma; };  // mean / sigma: [t][unit]

struct Parsed {
  myea_net_desc desc;
  uint64_t total_parameters = 0, total_weights = 0, total_bias = 0, total_norm_units = 0;
  std::vector<std::pair<uint64_t, float>> weights;
  std::vector<NormValues> norm;  // per layer
  std::vector<uint64_t> af_units;
};

bool parse_dropout(Lines &in, myea_layer_desc &L, bool hidden) {
  uint64_t u = 0;
  if (!in.take_u64("type_dropout", &u)) return false;
  L.type_dropout = static_cast<uint32_t>(u);
  if (hidden && !in.take_u64("use_coded_dropout", &u)) return false;
  for (int k = 0; k < 3; ++k)
    if (!in.take_real("dropout_values", &L.dropout_values[k], true)) return false;
  return true;
}

bool parse_normalization(Lines &in, myea_layer_desc &L, NormValues &nv, uint64_t T, bool fully_connected) {
  uint64_t u = 0, units = 0;
  if (!in.take_u64("type_normalization", &u)) return false;
  L.type_normalization = static_cast<uint32_t>(u);
  L.use_layer_normalization_before_activation = 1;
  // the reference's writer leaves this line out for LSTM and residual layers (Save.cpp:636-644) although its reader
  // asks for it on LSTM layers (Load.cpp:5459), so the reference cannot read back its own files for recurrent
  // networks; both forms are taken here
  if (fully_connected || in.key() == "use_layer_normalization_before_activation") {
    if (!in.take_u64("use_layer_normalization_before_activation", &u)) return false;
    L.use_layer_normalization_before_activation = static_cast<uint32_t>(u);
  }
  if (!in.take_u64("number_normalized_units", &units)) return false;
  if (L.type_normalization != MYEA_NORM_NONE) {
    nv.scale.assign(units, 1.f);
    nv.shift.assign(units, 0.f);
    nv.mean.assign(units * T, 0.f);
    nv.sigma.assign(units * T, 1.f);
  }
  for (uint64_t i = 0; i < units; ++i) {
    if (!in.take("NormU", nullptr, true)) return false;
    if (L.type_normalization == MYEA_NORM_NONE) continue;
    if (!in.take_real("scale", &nv.scale[i]) || !in.take_real("shift", &nv.shift[i])) return false;
    for (uint64_t t = 0; t < T; ++t)
      if (!in.take_real("mean_average", &nv.mean[t * units + i], true) || !in.take_real("variance_average", &nv.sigma[t * units + i], true)) return false;
  }
  return true;
}

bool skip_sparsity_and_constraints(Lines &in, float *upper_bound = nullptr) {
  float f, hi = 0.f;
  uint64_t u;
  const bool ok = in.take_u64("use_tied_parameter", &u) && in.take_u64("k_sparsity", &u) && in.take_real("alpha_sparsity", &f) &&
                  in.take_real("constraint_recurrent_weight_lower_bound", &f) && in.take_real("constraint_recurrent_weight_upper_bound", &hi);
  if (upper_bound != nullptr) *upper_bound = hi;
  return ok;
}

bool parse_connections(Lines &in, uint64_t count, Parsed &out) {
  for (uint64_t j = 0; j < count; ++j) {
    uint64_t idx = 0;
    float v = 0.f;
    if (in.done() || in.key().compare(0, 13, "connected_to_") != 0) return in.fail("expected connected_to_*");
    ++in.at;
    if (!in.take_weight(&idx, &v)) return false;
    out.weights.emplace_back(idx, v);
  }
  return true;
}

bool parse_neurons(Lines &in, const char *count_key, myea_layer_desc &L, Parsed &out) {
  uint64_t n = 0, c = 0;
  if (!in.take_u64(count_key, &n)) return false;
  L.unit_parameters[0] = n;
  for (uint64_t i = 0; i < n; ++i)
    if (!in.take("Neuron_unit", nullptr, true) || !in.take_u64("number_connections", &c) || !parse_connections(in, c, out)) return false;
  return true;
}

bool parse_activation_units(Lines &in, myea_layer_desc &L, uint64_t *count) {
  uint64_t n = 0, af = 0;
  float steep = 1.f;
  if (!in.take_u64("number_AF_units", &n)) return false;
  *count = n;
  for (uint64_t i = 0; i < n; ++i) {
    if (!in.take("AF", nullptr, true) || !in.take_real("activation_steepness", &steep) || !in.take_u64("activation_function", &af)) return false;
    if (steep != 1.f) return in.fail("activation steepness other than 1 is not built");
    if (i == 0) L.type_activation_function = static_cast<uint32_t>(af);
    else if (L.type_activation_function != af) return in.fail("a layer mixing activation functions is not built");
  }
  return true;
}

bool parse_ind_recurrent_units(Lines &in, myea_layer_desc &L, Parsed &out) {
  uint64_t n = 0, af = 0, unit = 0, idx = 0;
  float steep = 1.f, v = 0.f;
  if (!in.take_u64("number_AF_Ind_recurrent_units", &n)) return false;
  for (uint64_t i = 0; i < n; ++i) {
    if (!in.take("AF_Ind_R", nullptr, true) || !in.take_real("activation_steepness", &steep) || !in.take_u64("activation_function", &af) ||
        !in.take_u64("connected_to_AF_Ind_R", &unit) || !in.take_weight(&idx, &v))
      return false;
    if (steep != 1.f) return in.fail("activation steepness other than 1 is not built");
    if (i == 0) L.type_activation_function = static_cast<uint32_t>(af);
    else if (L.type_activation_function != af) return in.fail("a layer mixing activation functions is not built");
    out.weights.emplace_back(idx, v);
  }
  return true;
}

bool parse_bias(Lines &in, Parsed &out) {
  uint64_t n = 0, idx = 0;
  float v = 0.f;
  if (!in.take_u64("number_bias_parameters", &n)) return false;
  for (uint64_t i = 0; i < n; ++i) {
    if (!in.take_weight(&idx, &v)) return false;
    out.weights.emplace_back(idx, v);
  }
  return true;
}

bool parse_lstm(Lines &in, myea_layer_desc &L, Parsed &out) {
  uint64_t blocks = 0, cells = 0, af = 0, c = 0;
  float steep = 1.f;
  if (!in.take_u64("number_block_units", &blocks) || !in.take_u64("number_cell_units", &cells)) return false;
  if (blocks == 0 || cells % blocks != 0) return in.fail("cells are not a multiple of blocks");
  L.unit_parameters[0] = blocks;
  L.unit_parameters[1] = cells / blocks;
  for (uint64_t b = 0; b < blocks; ++b) {
    if (!in.take("Block", nullptr, true) || !in.take_u64("activation_function", &af) || !in.take_real("activation_steepness", &steep) ||
        !in.take_u64("number_connections", &c) || !parse_connections(in, c, out)) return false;
    if (af != MYEA_AF_TANH) return in.fail("LSTM blocks with an input/output activation other than tanh are not built");
  }
  return true;
}

int parse_dimension(const char *path, Parsed &out, std::string &error) {
  Lines in;
  if (!in.read(path)) { error = in.error; return MYEA_E_INVALID; }
  memset(&out.desc, 0, sizeof(out.desc));
  myea_net_desc &d = out.desc;
  uint64_t u = 0, layers = 0, totals[8];
  bool ok = in.take("|===| DIMENSION |===|", nullptr) && in.take_u64("type_network", &u);
  d.type_network = static_cast<uint32_t>(u);
  ok = ok && in.take_u64("number_layers", &layers) && in.take_u64("number_recurrent_depth", &d.number_recurrent_depth) &&
       in.take_u64("number_time_delays", &d.number_time_delays) && in.take_u64("use_first_layer_as_input", &u) &&
       in.take_u64("use_last_layer_as_output", &u);
  static const char *const total_keys[8] = {"total_basic_units", "total_basic_indice_units", "total_neuron_units", "total_AF_units",
                                            "total_AF_Ind_recurrent_units", "total_block_units", "total_cell_units", "total_normalized_units"};
  for (int k = 0; ok && k < 8; ++k) ok = in.take_u64(total_keys[k], &totals[k]);
  ok = ok && in.take_u64("total_parameters", &out.total_parameters) && in.take_u64("total_weights", &out.total_weights) &&
       in.take_u64("total_bias", &out.total_bias);
  if (!ok) { error = in.error; return MYEA_E_INVALID; }
  if (layers < 2 || layers > MYEA_MAX_LAYERS || d.number_recurrent_depth == 0) { error = "layer count or recurrent depth out of range"; return MYEA_E_INVALID; }
  out.total_norm_units = totals[7];
  d.number_layers = static_cast<uint32_t>(layers);
  out.norm.assign(layers, NormValues());
  out.af_units.assign(layers, 0);
  const uint64_t T = d.number_recurrent_depth;

  myea_layer_desc &I = d.layers[0];
  ok = in.take("Input", nullptr) && in.take_u64("type_layer", &u);
  I.type_layer = static_cast<uint32_t>(u);
  ok = ok && in.take_u64("type_activation", &u) && parse_dropout(in, I, false) && in.take_u64("number_inputs", &I.unit_parameters[0]);
  I.use_layer_normalization_before_activation = 1;
  std::vector<uint64_t> width(layers, 0);  // units of each layer as the file states them
  width[0] = I.unit_parameters[0];
  for (uint64_t l = 1; ok && l + 1 < layers; ++l) {
    myea_layer_desc &L = d.layers[l];
    ok = in.take("Hidden", nullptr) && in.take_u64("type_layer", &u);
    L.type_layer = static_cast<uint32_t>(u);
    ok = ok && in.take_u64("use_bidirectional", &u);
    if (ok && u != 0) { error = "bidirectional layers have no usable definition in the reference's files"; return MYEA_E_UNSUPPORTED; }
    if (!ok) break;
    switch (L.type_layer) {
      case MYEA_LAYER_FULLY_CONNECTED:
        ok = in.take_u64("type_activation", &u) && parse_dropout(in, L, true) && parse_normalization(in, L, out.norm[l], T, true) &&
             skip_sparsity_and_constraints(in) && parse_neurons(in, "number_neuron_units", L, out) &&
             parse_activation_units(in, L, &out.af_units[l]) && parse_bias(in, out);
        break;
      case MYEA_LAYER_FC_INDEPENDENTLY_RECURRENT: {
        float bound = 0.f;
        ok = in.take_u64("type_activation", &u) && parse_dropout(in, L, true) && parse_normalization(in, L, out.norm[l], T, true) &&
             skip_sparsity_and_constraints(in, &bound) && parse_neurons(in, "number_neuron_units", L, out) &&
             parse_ind_recurrent_units(in, L, out) && parse_bias(in, out);
        out.af_units[l] = L.unit_parameters[0];  // (not the first layer of a block)
        // the bound is the default one for some clip_gradient between 2 and 10: recover that value (0 = the class default)
        if (ok && bound > 0.f && fabsf(bound - ind_rnn_weight_bound(0.f, L.type_activation_function, static_cast<long long>(T))) > 1e-6f * bound) {
          const float c = ind_rnn_weight_bound(0.f, L.type_activation_function, static_cast<long long>(T));
          const float guess = 2.f * powf(bound / c, static_cast<float>(T));  // bound = (MAG / k)^(1/T), c = (2 / k)^(1/T)
          // the power and its root do not invert each other to the last bit: take the neighbour of the guess that gives
          // this very bound back, so that a file written from the parsed description equals the file that was read
          d.clip_gradient = guess;
          float up = guess, down = guess;
          for (int step = 0; step < 64; ++step) {
            if (ind_rnn_weight_bound(up, L.type_activation_function, static_cast<long long>(T)) == bound) { d.clip_gradient = up; break; }
            if (ind_rnn_weight_bound(down, L.type_activation_function, static_cast<long long>(T)) == bound) { d.clip_gradient = down; break; }
            up = nextafterf(up, INFINITY);
            down = nextafterf(down, -INFINITY);
          }
        }
        break;
      }
      case MYEA_LAYER_LSTM:
        ok = in.take_u64("type_activation", &u) && parse_dropout(in, L, true) && parse_normalization(in, L, out.norm[l], T, false) &&
             skip_sparsity_and_constraints(in) && parse_lstm(in, L, out) && parse_bias(in, out);
        break;
      case MYEA_LAYER_RESIDUAL:
        ok = in.take_u64("block_depth", &L.unit_parameters[0]) && in.take_u64("padding", &u) && parse_dropout(in, L, true) &&
             parse_normalization(in, L, out.norm[l], T, false) && in.take_u64("number_basic_units", &u);
        width[l] = u;
        break;
      case MYEA_LAYER_AVERAGE_POOLING:
      case MYEA_LAYER_MAX_POOLING: {
        ok = in.take_u64("kernel_size", &L.unit_parameters[0]) && in.take_u64("stride", &L.unit_parameters[1]) &&
             in.take_u64("padding", &L.unit_parameters[2]) && in.take_u64("dilation", &L.unit_parameters[3]) &&
             in.take_u64(L.type_layer == MYEA_LAYER_MAX_POOLING ? "number_basic_indice_units" : "number_basic_units", &u);
        width[l] = u;
        // the file does not carry the ceil mode: it is the mode under which the stated number of units comes out
        L.unit_parameters[4] = 0;
        if (ok && pooling_output_width(L, static_cast<long long>(width[l - 1])) != static_cast<long long>(u)) L.unit_parameters[4] = 1;
        break;
      }
      default: error = "layer type " + std::to_string(L.type_layer) + " is not built"; return MYEA_E_UNSUPPORTED;
    }
    if (L.type_layer == MYEA_LAYER_FULLY_CONNECTED || L.type_layer == MYEA_LAYER_FC_INDEPENDENTLY_RECURRENT) width[l] = L.unit_parameters[0];
    if (L.type_layer == MYEA_LAYER_LSTM) width[l] = L.unit_parameters[0] * std::max<uint64_t>(1, L.unit_parameters[1]);
  }
  myea_layer_desc &O = d.layers[layers - 1];
  ok = ok && in.take("Output", nullptr) && in.take_u64("type_layer", &u);
  O.type_layer = static_cast<uint32_t>(u);
  O.use_layer_normalization_before_activation = 1;
  ok = ok && in.take_u64("type_activation", &u) && parse_neurons(in, "number_outputs", O, out) &&
       parse_activation_units(in, O, &out.af_units[layers - 1]) && parse_bias(in, out) && in.take("|END| DIMENSION |END|", nullptr);
  if (!ok) { error = in.error; return MYEA_E_INVALID; }
  // the first layer of a residual block lists no activation unit (its input is used as it is); give it the function of
  // the layer after it so that writing the network again yields the same activation class
  for (uint64_t l = 1; l + 2 < layers; ++l)
    if (d.layers[l].type_layer == MYEA_LAYER_FULLY_CONNECTED && out.af_units[l] == 0)
      d.layers[l].type_activation_function = d.layers[l + 1].type_activation_function != 0 ? d.layers[l + 1].type_activation_function : MYEA_AF_LINEAR;
  return MYEA_OK;
}

}  // namespace

namespace {

// the `.net` file: every "key value" line, looked up by key (Load_Parameters, Neural_Network__Load.cpp:82-2321)
int parse_general(const char *path, myea_net_desc &d, myea_opt_desc &o, std::string &error) {
  Lines in;
  if (!in.read(path)) { error = in.error; return MYEA_E_INVALID; }
  memset(&o, 0, sizeof(o));
  o.epoch_time_step = 1.f;
  size_t found = 0;
  for (const auto &kv : in.kv) {
    const std::string &k = kv.first;
    if (k.empty() || k[0] == '|') continue;
    const double v = strtod(kv.second.c_str(), nullptr);
    const float f = static_cast<float>(v);
    const uint32_t u = static_cast<uint32_t>(strtoull(kv.second.c_str(), nullptr, 10));
    ++found;
    if (k == "learning_rate") o.learning_rate = f;
    else if (k == "learning_rate_final") o.learning_rate_final = f;
    else if (k == "learning_momentum") o.learning_momentum = f;
    else if (k == "learning_gamma") o.learning_gamma = f;
    else if (k == "use_Nesterov") o.use_nesterov = u;
    else if (k == "rprop_increase_factor") o.rprop_increase_factor = f;
    else if (k == "rprop_decrease_factor") o.rprop_decrease_factor = f;
    else if (k == "rprop_delta_min") o.rprop_delta_min = f;
    else if (k == "rprop_delta_max") o.rprop_delta_max = f;
    else if (k == "rprop_delta_zero") o.rprop_delta_zero = f;
    else if (k == "adam_learning_rate") o.adam_learning_rate = f;
    else if (k == "adam_beta1") o.adam_beta1 = f;
    else if (k == "adam_beta2") o.adam_beta2 = f;
    else if (k == "adam_epsilon") o.adam_epsilon = f;
    else if (k == "adam_bias_correction") o.use_adam_bias_correction = u;
    else if (k == "adam_gamma") o.adam_gamma = f;
    else if (k == "type_optimizer_function") o.type_optimizer_function = u;
    else if (k == "type_loss_function") d.type_loss_function = u;
    else if (k == "type_accuracy_function") d.type_accuracy_function = u;
    else if (k == "use_clip_gradient") o.use_clip_gradient = u;
    else if (k == "clip_gradient") o.clip_gradient = f;
    else if (k == "regularization__max_norm_constraints") o.regularization__max_norm_constraints = f;
    else if (k == "regularization__weight_decay") o.regularization__weight_decay = f;
    else if (k == "use_normalized_weight_decay") o.use_normalized_weight_decay = u;
    else if (k == "normalization_momentum_average") d.normalization_momentum_average = f;
    else if (k == "normalization_epsilon") d.normalization_epsilon = f;
    else if (k == "batch_renormalization_r_correction_maximum") d.batch_renormalization_r_correction_maximum = f;
    else if (k == "batch_renormalization_d_correction_maximum") d.batch_renormalization_d_correction_maximum = f;
    else if (k == "accuracy_variance") d.accuracy_variance = f;
    else if (k == "regularization__l1") o.regularization__l1 = f;
    else if (k == "regularization__l2") o.regularization__l2 = f;
    else if (k == "regularization__srip" && v != 0.0) {
      error = k + " is set: that penalty is not built";
      return MYEA_E_UNSUPPORTED;
    } else if (k == "use_Warm_Restarts" && u != 0) {
      error = "warm restarts are not built";
      return MYEA_E_UNSUPPORTED;
    } else --found;
  }
  if (found < 20) { error = std::string(path) + " does not look like a general-parameters file"; return MYEA_E_INVALID; }
  return MYEA_OK;
}

// places what the `.nn` file held into flat arrays laid out by this library's index map, after checking that the map
// agrees with the totals the file states
int place(const Parsed &in, uint64_t batch_size, HostPlan &P, float *params, float *mean, float *sigma, std::string &error) {
  myea_net_desc d = in.desc;
  d.batch_size = batch_size == 0 ? 1 : batch_size;
  const int rc = make_plan(&d, P);
  if (rc != MYEA_OK) { error = P.error; return rc; }
  const myea_b200_net &net = *P.net;
  if (net.total_parameters != in.total_parameters || net.total_weights != in.total_weights || net.total_bias != in.total_bias ||
      net.total_norm_units != in.total_norm_units) {
    error = "the file's parameter totals differ from the layout of the layers it lists";
    return MYEA_E_INVALID;
  }
  if (params == nullptr) return MYEA_OK;
  std::fill(params, params + net.total_parameters, 0.f);
  for (uint64_t l = 0; l < net.layers.size() && net.any_norm; ++l) {  // units without a file entry: gamma 1, sigma 1 (Allocate__Normalized_Unit)
    const LayerPlan &L = net.layers[l];
    const uint64_t T = static_cast<uint64_t>(net.T), units = L.idx.number_units_norm;
    for (uint64_t u = 0; u < units; ++u) params[L.idx.scale_index + u] = 1.f;
    for (uint64_t i = 0; i < units * T; ++i) {   // running averages: [layer][T][units]
      mean[static_cast<uint64_t>(L.norm_unit_offset) * T + i] = 0.f;
      sigma[static_cast<uint64_t>(L.norm_unit_offset) * T + i] = 1.f;
    }
  }
  for (const auto &w : in.weights) {
    if (w.first >= net.total_weights + net.total_bias) { error = "weight index past the parameters"; return MYEA_E_INVALID; }
    params[w.first] = w.second;
  }
  for (uint64_t l = 0; l < net.layers.size(); ++l) {
    const NormValues &nv = in.norm[l];
    const LayerPlan &L = net.layers[l];
    if (nv.scale.empty()) continue;
    if (nv.scale.size() != L.idx.number_units_norm) { error = "normalized units of a layer differ from its width"; return MYEA_E_INVALID; }
    const uint64_t T = static_cast<uint64_t>(net.T), units = nv.scale.size();
    for (uint64_t u = 0; u < units; ++u) {
      params[L.idx.scale_index + u] = nv.scale[u];
      params[L.idx.shift_index + u] = nv.shift[u];
    }
    for (uint64_t i = 0; i < units * T && i < nv.mean.size(); ++i) {   // the file's [t][unit] order is the arrays' order
      mean[static_cast<uint64_t>(L.norm_unit_offset) * T + i] = nv.mean[i];
      sigma[static_cast<uint64_t>(L.norm_unit_offset) * T + i] = nv.sigma[i];
    }
  }
  return MYEA_OK;
}

thread_local std::string g_parse_error;

}  // namespace

extern "C" const char *myea_b200_checkpoint_last_error(void) { return g_parse_error.c_str(); }

extern "C" int myea_b200_checkpoint_parse(const char *path_dimension, const char *path_general, uint64_t batch_size, myea_net_desc *desc,
                                          myea_opt_desc *opt, float *parameters, uint64_t parameters_capacity, float *mean_average,
                                          float *variance_average, uint64_t norm_capacity, uint64_t *total_parameters,
                                          uint64_t *total_normalized_units) {
  g_parse_error.clear();
  if (path_dimension == nullptr || desc == nullptr) return MYEA_E_INVALID;
  Parsed in;
  int rc = parse_dimension(path_dimension, in, g_parse_error);
  if (rc != MYEA_OK) return rc;
  myea_opt_desc o;
  memset(&o, 0, sizeof(o));
  if (path_general != nullptr) {
    rc = parse_general(path_general, in.desc, o, g_parse_error);
    if (rc != MYEA_OK) return rc;
    // the general file states clip_gradient itself; where the bounds of the independently recurrent layers are the
    // default ones for that value, it replaces the value recovered from a bound
    if (in.desc.clip_gradient != 0.f && o.clip_gradient > 0.f) {
      const float from_bound = std::min(std::max(in.desc.clip_gradient, 2.f), 10.f), stated = std::min(std::max(o.clip_gradient, 2.f), 10.f);
      if (fabsf(from_bound - stated) <= 1e-4f * stated) in.desc.clip_gradient = o.clip_gradient;
    }
  }
  if (total_parameters) *total_parameters = in.total_parameters;
  if (total_normalized_units) *total_normalized_units = in.total_norm_units;
  const bool fill = parameters != nullptr;
  const uint64_t averages = in.total_norm_units * std::max<uint64_t>(1, in.desc.number_recurrent_depth);
  if (fill && (parameters_capacity < in.total_parameters ||
               (averages != 0 && (mean_average == nullptr || variance_average == nullptr || norm_capacity < averages)))) {
    g_parse_error = "arrays too small for the file's parameters";
    return MYEA_E_INVALID;
  }
  HostPlan P;
  rc = place(in, batch_size, P, fill ? parameters : nullptr, mean_average, variance_average, g_parse_error);
  if (rc != MYEA_OK) return rc;
  *desc = P.net->desc;
  if (opt != nullptr) *opt = o;
  return MYEA_OK;
}

extern "C" int myea_b200_load(myea_handle *out, const char *path_dimension, const char *path_general, uint64_t batch_size, int device,
                              myea_opt_desc *opt) {
  if (out == nullptr || batch_size == 0) return MYEA_E_INVALID;
  *out = nullptr;
  myea_net_desc desc;
  uint64_t P = 0, U = 0;
  int rc = myea_b200_checkpoint_parse(path_dimension, path_general, batch_size, &desc, opt, nullptr, 0, nullptr, nullptr, 0, &P, &U);
  if (rc != MYEA_OK) return rc;
  U *= std::max<uint64_t>(1, desc.number_recurrent_depth);  // running averages: one set per time step
  std::vector<float> params(P + 1), mean(U + 1), sigma(U + 1);
  rc = myea_b200_checkpoint_parse(path_dimension, path_general, batch_size, &desc, opt, params.data(), P, mean.data(), sigma.data(), U, nullptr, nullptr);
  if (rc != MYEA_OK) return rc;
  rc = myea_b200_create(out, &desc, device);
  if (rc != MYEA_OK) return rc;
  rc = myea_b200_upload(*out, MYEA_BUF_PARAMETERS, params.data(), 0, P);
  if (rc == MYEA_OK) {  // the regularization mask as the reference builds it: weights 1, biases and scale / shift 0 (Neural_Network__Indexing.cpp:50-76)
    std::vector<float> mask(P + 1, 0.f);
    std::fill(mask.begin(), mask.begin() + (*out)->total_weights, 1.f);
    rc = myea_b200_upload(*out, MYEA_BUF_MASK_REGULARIZED, mask.data(), 0, P);
  }
  if (rc == MYEA_OK && U != 0) {
    rc = myea_b200_upload(*out, MYEA_BUF_NORM_MEAN_AVERAGE, mean.data(), 0, U);
    if (rc == MYEA_OK) rc = myea_b200_upload(*out, MYEA_BUF_NORM_VARIANCE_AVERAGE, sigma.data(), 0, U);
  }
  if (rc != MYEA_OK) {  // a half-loaded network is of no use to the caller: keep the reason, give the handle back
    g_parse_error = std::string("load: copying the parsed state to the device failed: ") + myea_b200_last_error(*out);
    myea_b200_destroy(*out);
    *out = nullptr;
  }
  return rc;
}
