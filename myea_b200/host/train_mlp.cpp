// Example and self-check of the host mirror: config 1 of the benchmark list (MLP 64-256-256-10, tanh / softmax,
// cross-entropy, Adam, batch 128) trained for a few steps on seeded synthetic data, written the way the reference's
// own harness drives `class Neural_Network` (Neural_Network_Launcher_Windows/Source_Files/debug.cpp).
// Prints one line per step: "step <i> loss <mean cross-entropy term> accuracy <percent>".
// With a second argument <prefix> the trained network is then written to <prefix>.nn / <prefix>.net in the reference's
// checkpoint format, read back into a second object with Load, and both answer the batch in inference mode:
// "checkpoint round trip: identical" when every output agrees bit for bit.
// With a third argument <dir> the initial parameters, inputs and targets are read from <dir>/parameters.f32, inputs.f32
// and targets.f32 (raw little-endian floats, [P], [B][64], [B][10]) instead of being drawn, the optimizer is the one a
// fourth argument names (ENUM_TYPE_OPTIMIZER_FUNCTIONS value, default Adam), and the trained parameters are written to
// <dir>/parameters_out.f32: a test runs the reference's own class through the same member calls on the same files and
// compares.  An empty <prefix> ("") skips the checkpoint round trip.
#include <stdio.h>
#include <stdlib.h>

#include <random>
#include <string>
#include <vector>

#include "Neural_Network.hpp"

using MyEA::B200::Layer_Parameters;
using MyEA::B200::Neural_Network;

static bool read_floats(std::string const &path, float *dst, size_t count) {
  FILE *f = fopen(path.c_str(), "rb");
  if (f == nullptr) return false;
  size_t const got = fread(dst, sizeof(float), count, f);
  fclose(f);
  return got == count;
}

int main(int argc, char **argv) {
  int const steps = argc > 1 ? atoi(argv[1]) : 10;
  std::string const io_dir(argc > 3 ? argv[3] : "");
  unsigned int const optimizer = argc > 4 ? static_cast<unsigned int>(atoi(argv[4])) : MYEA_OPT_ADAM;
  size_t const B = 128, sizes[4] = {64, 256, 256, 10};
  Layer_Parameters lp[4];
  for (int i = 0; i < 4; ++i) { lp[i].type_layer = MYEA_LAYER_FULLY_CONNECTED; lp[i].unit_parameters[0] = sizes[i]; }
  Neural_Network nn;
  if (!nn.Compile(4, 1, MYEA_NETWORK_FEEDFORWARD, lp)) return 1;
  nn.Set__Layer_Activation_Function(1, MYEA_AF_TANH);
  nn.Set__Layer_Activation_Function(2, MYEA_AF_TANH);
  nn.Set__Layer_Activation_Function(3, MYEA_AF_SOFTMAX);
  nn.Set__Loss_Function(MYEA_LOSS_CROSS_ENTROPY);
  nn.Set__Accuracy_Function(MYEA_ACCURACY_CROSS_ENTROPY);
  nn.Set__Optimizer_Function(optimizer);
  if (!nn.Update__Batch_Size(B) || !nn.Initialize__CUDA(0)) return 1;
  std::mt19937 gen(0);
  for (int l = 1; l < 4; ++l) {  // Glorot-uniform, tanh gain 5/3 on the hidden layers
    float const gain = l < 3 ? 5.f / 3.f : 1.f, bound = gain * sqrtf(6.f / float(sizes[l - 1] + sizes[l]));
    std::uniform_real_distribution<float> u(-bound, bound);
    myea_layer_index const &ix = nn.Get__Layer_Index(l);
    for (uint64_t i = ix.first_connection_index; i < ix.last_connection_index; ++i) nn.ptr_array_parameters[i] = u(gen);
  }
  if (!io_dir.empty() && !read_floats(io_dir + "/parameters.f32", nn.ptr_array_parameters, nn.total_parameters)) return 5;
  if (!nn.Copy__Parameters__Host_To_Device()) return 1;
  std::uniform_real_distribution<float> ux(-1.f, 1.f);
  std::vector<std::vector<float>> X(B, std::vector<float>(64)), Y(B, std::vector<float>(10, 0.f));
  std::vector<float const *> xp(B), yp(B);
  for (size_t b = 0; b < B; ++b) {
    for (float &v : X[b]) v = ux(gen);
    Y[b][gen() % 10] = 1.f;
    xp[b] = X[b].data();
    yp[b] = Y[b].data();
  }
  if (!io_dir.empty()) {
    std::vector<float> xs(B * 64), ys(B * 10);
    if (!read_floats(io_dir + "/inputs.f32", xs.data(), xs.size()) || !read_floats(io_dir + "/targets.f32", ys.data(), ys.size())) return 5;
    for (size_t b = 0; b < B; ++b) {
      X[b].assign(xs.begin() + b * 64, xs.begin() + (b + 1) * 64);
      Y[b].assign(ys.begin() + b * 10, ys.begin() + (b + 1) * 10);
    }
  }
  nn.type_state_propagation = 1;
  nn.Clear_Training_Arrays();
  float first = 0.f, last = 0.f;
  for (int it = 0; it < steps; ++it) {
    nn.Reset__Loss();
    nn.Forward_Pass(B, xp.data());
    nn.Compute__Error(B, yp.data());
    nn.Backward_Pass(B);
    nn.Update_Derivative_Weight(B);
    nn.number_accuracy_trial = B;
    last = nn.Get__Loss();
    if (it == 0) first = last;
    printf("step %d loss %.6f accuracy %.2f\n", it, last, nn.Get__Accuracy());
    nn.Update_Parameter(B, B);
  }
  if (!nn.Copy__Parameters__Device_To_Host()) return 1;
  if (!io_dir.empty()) {
    FILE *f = fopen((io_dir + "/parameters_out.f32").c_str(), "wb");
    if (f == nullptr || fwrite(nn.ptr_array_parameters, sizeof(float), nn.total_parameters, f) != nn.total_parameters) return 5;
    fclose(f);
  }
  if (argc > 2 && argv[2][0] != '\0') {
    std::string const prefix(argv[2]);
    if (!nn.Save_Dimension_Parameters(prefix + ".nn") || !nn.Save_General_Parameters(prefix + ".net")) return 3;
    Neural_Network again;
    if (!again.Load(prefix + ".nn", prefix + ".net", B, 0)) return 3;
    nn.type_state_propagation = again.type_state_propagation = 0;
    nn.Forward_Pass(B, xp.data());
    again.Forward_Pass(B, xp.data());
    size_t differing = 0;
    for (size_t b = 0; b < B; ++b) {
      float const *p = nn.Get__Outputs(b), *q = again.Get__Outputs(b);
      for (size_t o = 0; o < sizes[3]; ++o) differing += (p[o] != q[o]) ? 1 : 0;
    }
    for (size_t i = 0; i < nn.total_parameters; ++i) differing += (nn.ptr_array_parameters[i] != again.ptr_array_parameters[i]) ? 1 : 0;
    printf("checkpoint round trip: %s\n", differing == 0 ? "identical" : "DIFFERENT");
    if (differing != 0) return 4;
  }
  return (last < first) ? 0 : 2;   // the loss must go down on a fixed batch
}
