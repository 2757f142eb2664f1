// Plan of one LSTM layer on the device (lstm.cu) and the persistent step kernels that walk its time steps
// (lstm_persistent.cu).
#pragma once

#include "net.cuh"

namespace myea {

struct LstmDir {
  long long w_base = 0;   // first parameter of this direction's blocks
  long long b_base = 0;   // [bz (C) | bi (C) | bf (C) | bo (C)]
  float *gates_in = nullptr;  // [T*B, 4C] input projection + bias, columns [z | i | f | o]
  float *act = nullptr;       // [T*B, 4C] activated gates
  float *cstate = nullptr, *cact = nullptr;  // [T*B, C] cell state, tanh(cell state)
  float *dgates = nullptr;    // [T*B, 4C] error w.r.t. the gate summations
  float *dcstate = nullptr;   // [T*B, C]
  uint8_t *zone_state = nullptr, *zone_output = nullptr;  // [T, C], 1 = compute, 0 = keep the previous value
};

struct LstmPlan {
  int dirs = 1;
  long long C = 0, n_in = 0, stride = 0;
  bool zoneout = false;
  LstmDir d[2];
  float *s_rec = nullptr;      // [B, 4C] recurrent projection of the current step
  float *panel_mem = nullptr;  // W_rec panels, their transpose, per-step operand panels
  size_t off_wrec = 0, off_wrect = 0, off_step = 0;
  float *partial = nullptr;    // [7][chunks][C]
  // cell fused into the recurrent contraction (C a multiple of 8, tensor-core engine): compact peepholes
  // [dirs][3][C], ping-pong operand panels of h (forward) and of the gate errors (backward)
  bool shared_dw = false;  // weight derivatives from untransposed (column-read) operand panels
  bool fuse = false;
  // With `fuse`, a step is two kernels: the contraction and an 8-cells-per-thread cell kernel that also writes the next
  // operand panels.  fuse_mask (MYEA_B200_LSTM_FUSE) moves the cell into the contraction's epilogue instead: bit 0
  // forward, bit 1 backward.  One kernel per step, but measured slower on C3 (the few threads that own accumulator
  // rows walk their cells one memory round trip after the other), so it is off by default.
  int fuse_mask = 0;
  float *peep_compact = nullptr;
  float *h_panels[2] = {nullptr, nullptr};
  float *dg_panels[2] = {nullptr, nullptr};
};

// One launch that walks ALL remaining time steps of one layer and direction (lstm_persistent.cu): the recurrent
// contraction of every step on the tensor cores, the cell arithmetic in its epilogue, the step's results written as the
// next step's operand panels, and a bounded grid-wide barrier between steps.  `first_step` is the first step of the
// walk this launch computes (the steps before it were computed by the per-step kernels and left their panels behind).
//   forward: steps s = 1 .. T-1 of direction `dir` (step s reads the h panels of buffer (s - 1) & 1)
//   backward: steps s = 1 .. T-1 of the walk against the direction (step s reads the gate-error panels of (s - 1) & 1)
// lstm_persistent_plan decides at creation whether the layer's shapes fit (every tile resident at once); the step
// functions return MYEA_E_UNSUPPORTED when they do not apply and the caller takes the per-step path.
struct LstmPersistent;
int lstm_persistent_plan(myea_b200_net *net, LayerPlan &L);
void lstm_persistent_destroy(LstmPlan *P);
bool lstm_persistent_ready(const LstmPlan *P);
int lstm_persistent_forward(myea_b200_net *net, LayerPlan &L, int dir, const Panels &w_rec_interleaved, const float *peep_compact, bool zoneout);
int lstm_persistent_backward(myea_b200_net *net, LayerPlan &L, int dir, const Panels &w_rec_transposed, const float *peep_compact);

}  // namespace myea
