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

struct LstmPersistent;
struct LstmPlan {
  int dirs = 1;
  long long C = 0, n_in = 0, stride = 0;
  bool zoneout = false;
  LstmDir d[2];
  float *s_rec = nullptr;      // [B, 4C] recurrent projection of the current step
  float *panel_mem = nullptr;  // W_rec panels, their transpose, per-step operand panels
  size_t off_wrec = 0, off_wrect = 0, off_step = 0;
  float *partial = nullptr;    // [7][chunks][C]
  bool shared_dw = false;  // weight derivatives from untransposed (column-read) operand panels
  // `fuse` (C a multiple of 8, tensor-core engine): the cell arithmetic of a step also writes the next step's operand
  // panels - ping-pong panels of h (forward) and of the gate errors (backward) - and reads compact peepholes
  // [dirs][3][C].  All steps but the first then run in one persistent launch (`persist`, lstm_persistent.cu) when the
  // layer's tiles fit the device at once, else as a contraction plus an 8-cells-per-thread cell kernel per step.
  bool fuse = false;
  float *peep_compact = nullptr;
  // both buffers of a ping-pong pair lie in one allocation, hi [2][rows][kp] then cross [2][rows][kp] with rows = the
  // batch rounded up to 128, so that one tensor map covers both
  Panels h_pan[2], dg_pan[2];
  LstmPersistent *persist = nullptr;
  // blocks of several cells (lstm_blocks.cu): K blocks of cpb cells per direction, gate rows of G = C + 3K columns
  // [z (C) | i (K) | f (K) | o (K)], weights gathered into dense matrices for the pass and their derivatives scattered back
  long long K = 0, cpb = 1;
  float *blk_w_in = nullptr, *blk_w_rec = nullptr, *blk_peep = nullptr;       // [G, in], [G, C], [3][C]
  float *blk_dw_in = nullptr, *blk_dw_rec = nullptr, *blk_dpeep = nullptr;
  float *blk_products = nullptr;                                               // [T*B, 3C]
};

int lstm_blocks_create(myea_b200_net *net, LayerPlan &L, LstmPlan *P);
int lstm_blocks_forward(myea_b200_net *net, LayerPlan &L, const float *input, long long n_in);
int lstm_blocks_backward(myea_b200_net *net, LayerPlan &L);
int lstm_blocks_backward_to_input(myea_b200_net *net, LayerPlan &L, float *prev_deriv, const LayerPlan &prev, const Epilogue *finish);
int lstm_blocks_update_derivative_weight(myea_b200_net *net, LayerPlan &L, const float *input, long long n_in);


// One launch that walks ALL remaining time steps of one layer and direction (lstm_persistent.cu): the recurrent
// contraction of every step on the tensor cores, the cell arithmetic in its epilogue, the step's results written as the
// next step's operand panels, and a bounded grid-wide barrier between steps.  The first step of a walk has no predecessor
// and is computed by the per-step kernels, which leave its panels behind.
//   forward: steps s = 1 .. T-1 of direction `dir` (step s reads the h panels of buffer (s - 1) & 1)
//   backward: steps s = 1 .. T-1 of the walk against the direction (step s reads the gate-error panels of (s - 1) & 1)
// lstm_persistent_plan decides at creation whether the layer's shapes fit (every tile resident at once); the step
// functions return MYEA_E_UNSUPPORTED when they do not apply and the caller takes the per-step path.
int lstm_persistent_plan(myea_b200_net *net, LayerPlan &L);
void lstm_persistent_destroy(LstmPlan *P);
bool lstm_persistent_ready(const LstmPlan *P);
int lstm_persistent_forward(myea_b200_net *net, LayerPlan &L, int dir, const Panels &w_rec_interleaved, const float *peep_compact, bool zoneout);
int lstm_persistent_backward(myea_b200_net *net, LayerPlan &L, int dir, const Panels &w_rec_transposed, const float *peep_compact);

}  // namespace myea
