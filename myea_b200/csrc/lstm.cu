// LSTM layer with peephole connections: forward pass, back-propagation through time, derivative-weight accumulation.
//
// Reference routines (Source_Files/Neural_Network/): forward Forward_Pass__LSTM__Gates_CIFO / __Gates_CIF_AF_State
// (and its Zoneout twin) / __States_AF / __Output (Neural_Network__Recurrent_Forward_Pass__OpenMP.cpp:859-1582), BPTT
// Backward_Pass__LSTM_Derivative__Output / __Cell_State_AF / __Gates_CIF_AF_State
// (Neural_Network__Recurrent_Backward_Pass__OpenMP.cpp:1130-1604), error to the previous layer Backward_Pass__LSTM (:1024-1120),
// Recurrent__Update_Derivative_Weight__LSTM + bias (Neural_Network__Recurrent_Update_Derivative_Weight__OpenMP.cpp:492-776).
//
// One cell per block (what every shipped configuration uses; blocks of several cells: lstm_blocks.cu).  Per step, with prev = the step before in the layer's direction:
//   z = tanh(Wz x + Rz h_prev + bz)          i = sig(Wi x + Ri h_prev + bi + pi*c_prev)
//   f = sig(Wf x + Rf h_prev + bf + pf*c_prev)   c = z*i + f*c_prev        (first step: no recurrent terms, no f)
//   o = sig(Wo x + Ro h_prev + bo + po*c)    h = tanh(c)*o
// Zoneout (forward only, as in the reference): where the state mask is false c = c_prev (0 at the first step), where
// the output mask is false h = h_prev (0 at the first step); the backward pass ignores the masks.
//
// Mapping to the GPU: the four gate matrices stay in the reference's interleaved per-block parameter layout and are read
// through strided operands into fused K-major panels ([4C, in], [4C, C] and their transposes), so the input projection
// of all T steps is ONE tensor-core contraction [T*B, in] x [in, 4C], each recurrent step is one [B, C] x [C, 4C]
// contraction plus one fused cell kernel (gate nonlinearities, peepholes, cell-state recurrence, zoneout select), each
// BPTT step is one [B, 4C] x [4C, C] contraction accumulated into the output error plus one fused cell-backward kernel,
// and the weight derivatives are contractions over K = T*B.  Bias and peephole derivatives are column reductions.
#include "lstm.cuh"
#include "panel_math.cuh"

#include <algorithm>

namespace myea {

// offsets of the gate matrices inside one block of the parameter buffer (Prepare__Connections__LSTM)
struct BlockOffsets {
  long long z_in, z_rec, in[3], rec[3], peep;  // in/rec: input, forget, output gate
};
static BlockOffsets block_offsets(long long n_in, long long C) {
  BlockOffsets o;
  o.z_in = 0;
  o.z_rec = n_in;
  o.in[0] = n_in + C; o.in[1] = 2 * n_in + C; o.in[2] = 3 * n_in + C;
  o.rec[0] = 4 * n_in + C; o.rec[1] = 4 * n_in + 2 * C; o.rec[2] = 4 * n_in + 3 * C;
  o.peep = 4 * n_in + 4 * C;
  return o;
}

// ---------------------------------------------------------------------------------------------------------
// fused cell kernels
// ---------------------------------------------------------------------------------------------------------

struct CellFwd {
  const float *gates_in;  // rows of step t: [B, 4C]
  const float *s_rec;     // [B, 4C] or null at the first step
  const float *c_prev;    // [B, C] or null
  const float *h_prev;    // [B, ldh] or null
  const float *peep;      // parameter pointer of block 0's p_i; block c at + c*stride, p_f +1, p_o +2
  long long stride;
  float *act, *cstate, *cact, *h;  // rows of step t
  long long ldh;
  const uint8_t *zone_state, *zone_output;  // [C] of step t, or null
  long long B, C;
};

__global__ void __launch_bounds__(256) lstm_cell_forward_kernel(const CellFwd p) {
  const long long total = p.B * p.C;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = i / p.C, c = i - b * p.C;
    const float *gi = p.gates_in + b * 4 * p.C;
    const bool first = p.s_rec == nullptr;
    const float *sr = first ? nullptr : p.s_rec + b * 4 * p.C;
    const float pi = p.peep[c * p.stride], pf = p.peep[c * p.stride + 1], po = p.peep[c * p.stride + 2];
    const float cp = first ? 0.f : p.c_prev[b * p.C + c];
    const float sz = gi[c] + (first ? 0.f : sr[c]);
    const float si = gi[p.C + c] + (first ? 0.f : sr[p.C + c] + pi * cp);
    const float z = tanh_ref(sz);
    const float ig = sigmoid_ref(si);
    float fg = 0.f;
    float cs = z * ig;
    if (!first) {
      fg = sigmoid_ref(gi[2 * p.C + c] + sr[2 * p.C + c] + pf * cp);
      cs += fg * cp;
    }
    if (p.zone_state != nullptr && !p.zone_state[c]) cs = cp;  // cp is 0 at the first step
    const float a = tanh_ref(cs);
    const float og = sigmoid_ref(gi[3 * p.C + c] + (first ? 0.f : sr[3 * p.C + c]) + po * cs);
    float h = a * og;
    if (p.zone_output != nullptr && !p.zone_output[c]) h = first ? 0.f : p.h_prev[b * p.ldh + c];
    float *act = p.act + b * 4 * p.C;
    act[c] = z; act[p.C + c] = ig; act[2 * p.C + c] = fg; act[3 * p.C + c] = og;
    p.cstate[b * p.C + c] = cs;
    p.cact[b * p.C + c] = a;
    p.h[b * p.ldh + c] = h;
  }
}

struct CellBwd {
  const float *dh;        // [B, ldh] error on the outputs of step t (recurrent contribution already added)
  long long ldh;
  const float *act, *cact;     // step t
  const float *c_prev;         // cell state of the previous step in the layer's direction, null at the first step
  const float *act_next, *dgates_next, *dc_next;  // step after t in the layer's direction, null at the last step
  const float *peep;
  long long stride;
  float *dgates, *dcstate;     // step t
  long long B, C;
};

__global__ void __launch_bounds__(256) lstm_cell_backward_kernel(const CellBwd p) {
  const long long total = p.B * p.C;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = i / p.C, c = i - b * p.C;
    const float *act = p.act + b * 4 * p.C;
    const float z = act[c], ig = act[p.C + c], fg = act[2 * p.C + c], og = act[3 * p.C + c];
    const float a = p.cact[b * p.C + c];
    const float pi = p.peep[c * p.stride], pf = p.peep[c * p.stride + 1], po = p.peep[c * p.stride + 2];
    const float dh = p.dh[b * p.ldh + c];
    const float d_o = og * (1.f - og) * (dh * a);
    float dc = dh * og * (1.f - a * a);
    dc += po * d_o;
    if (p.dgates_next != nullptr) {
      const float *dn = p.dgates_next + b * 4 * p.C;
      dc += pi * dn[p.C + c];
      dc += pf * dn[2 * p.C + c];
      dc += p.dc_next[b * p.C + c] * p.act_next[b * 4 * p.C + 2 * p.C + c];
    }
    const float dz = dc * ig * (1.f - z * z);
    const float di = (dc * z) * (ig * (1.f - ig));
    const float df = p.c_prev != nullptr ? (dc * p.c_prev[b * p.C + c]) * (fg * (1.f - fg)) : 0.f;
    float *dg = p.dgates + b * 4 * p.C;
    dg[c] = dz; dg[p.C + c] = di; dg[2 * p.C + c] = df; dg[3 * p.C + c] = d_o;
    p.dcstate[b * p.C + c] = dc;
  }
}

// Bias and peephole derivatives: per cell c, over all rows r of dgates [R, 4C]
//   out0..3 = sum dz, di, df, do ; out4 = sum di[r]*c[r - shift], out5 = sum df[r]*c[r - shift] (rows whose partner
//   exists), out6 = sum do[r]*c[r].   partial[k][chunk][c].
__global__ void __launch_bounds__(256) lstm_bias_peephole_reduce_kernel(const float *__restrict__ dgates, const float *__restrict__ cstate,
                                                                        long long R, long long C, long long shift, int chunks,
                                                                        float *__restrict__ partial) {
  __shared__ float sh[7][8][33];
  const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const long long c = static_cast<long long>(blockIdx.x) * 32 + cl;
  const long long per = (R + chunks - 1) / chunks;
  const long long r0 = blockIdx.y * per, r1 = min(R, r0 + per);
  float acc[7] = {0, 0, 0, 0, 0, 0, 0};
  if (c < C) {
    for (long long r = r0 + rl; r < r1; r += 8) {
      const float *dg = dgates + r * 4 * C;
      const float dz = dg[c], di = dg[C + c], df = dg[2 * C + c], d_o = dg[3 * C + c];
      acc[0] += dz; acc[1] += di; acc[2] += df; acc[3] += d_o;
      const long long rp = r - shift;
      if (rp >= 0 && rp < R) {
        const float cs = cstate[rp * C + c];
        acc[4] = fmaf(di, cs, acc[4]);
        acc[5] = fmaf(df, cs, acc[5]);
      }
      acc[6] = fmaf(d_o, cstate[r * C + c], acc[6]);
    }
  }
#pragma unroll
  for (int k = 0; k < 7; ++k) sh[k][rl][cl] = acc[k];
  __syncthreads();
  if (rl == 0 && c < C) {
#pragma unroll
    for (int k = 0; k < 7; ++k) {
      float t = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) t += sh[k][r][cl];
      partial[(static_cast<long long>(k) * chunks + blockIdx.y) * C + c] = t;
    }
  }
}

// 32 cells per block, the chunks of a sum spread over 8 threads per cell
__global__ void __launch_bounds__(256) lstm_bias_peephole_finalize_kernel(const float *__restrict__ partial, int chunks, long long C, float *d_bias,
                                                                          float *d_peep, long long stride) {
  __shared__ float sh[7][8][33];
  const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const long long c = static_cast<long long>(blockIdx.x) * 32 + cl;
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    float t = 0.f;
    if (c < C)
      for (int ch = rl; ch < chunks; ch += 8) t += partial[(static_cast<long long>(k) * chunks + ch) * C + c];
    sh[k][rl][cl] = t;
  }
  __syncthreads();
  if (rl != 0 || c >= C) return;
  float t[7];
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    t[k] = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t[k] += sh[k][r][cl];
  }
  // atomics: with the reference's shifted bias base the output-gate slots alias the next layer's bias slots, which another
  // kernel of the same stream also accumulates into; stream order already serialises them, the atomics are belt and braces
  atomicAdd(&d_bias[c], t[0]);
  atomicAdd(&d_bias[C + c], t[1]);
  atomicAdd(&d_bias[2 * C + c], t[2]);
  atomicAdd(&d_bias[3 * C + c], t[3]);
  d_peep[c * stride] += t[4];
  d_peep[c * stride + 1] += t[5];
  d_peep[c * stride + 2] += t[6];
}

// Cell kernels of the steps that have a predecessor / successor, 8 consecutive cells of one batch row per thread: the
// arithmetic of lstm_cell_forward_kernel / lstm_cell_backward_kernel, and the results also leave as the operand panels
// of the next step's contraction (no separate split pass).  p.kind selects; s_rec / rec_dh is the contraction's output.
__global__ void __launch_bounds__(256) lstm_cells8_forward_kernel(const LstmStep p, const float *__restrict__ s_rec, long long B) {
  grid_dependency_wait();
  grid_dependency_release();
  const long long groups = p.C >> 3, total = B * groups;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = i / groups, c0 = (i - b * groups) << 3;
    float gz[8], gi[8], gf[8], go[8], rec[32];
    const float *r = s_rec + b * 4 * p.C + c0;
    load8(gz, r); load8(gi, r + p.C); load8(gf, r + 2 * p.C); load8(go, r + 3 * p.C);
#pragma unroll
    for (int k = 0; k < 8; ++k) { rec[4 * k] = gz[k]; rec[4 * k + 1] = gi[k]; rec[4 * k + 2] = gf[k]; rec[4 * k + 3] = go[k]; }
    lstm_forward_cells8(p, rec, b, c0);
  }
}
// the error through time has already been added into p.dh by the contraction (accumulate epilogue): rec = 0
__global__ void __launch_bounds__(256) lstm_cells8_backward_kernel(const LstmStep p, long long B) {
  grid_dependency_wait();
  grid_dependency_release();
  const long long groups = p.C >> 3, total = B * groups;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = i / groups, c0 = (i - b * groups) << 3;
    const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    lstm_backward_cells8(p, zero, b, c0);
  }
}

// peepholes p_i, p_f, p_o of every cell, gathered from the blocks of the parameter buffer into [3][C]
__global__ void lstm_gather_peepholes_kernel(const float *__restrict__ peep, long long stride, long long C, float *__restrict__ out) {
  const long long c = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (c >= C) return;
  out[c] = peep[c * stride];
  out[C + c] = peep[c * stride + 1];
  out[2 * C + c] = peep[c * stride + 2];
}

// ---------------------------------------------------------------------------------------------------------
// plan
// ---------------------------------------------------------------------------------------------------------
template <typename T>
static int lalloc(myea_b200_net *net, T **p, size_t count) {
  void *q = nullptr;
  const size_t bytes = std::max<size_t>(count, 1) * sizeof(T);
  if (cudaMalloc(&q, bytes) != cudaSuccess) { net->ctx.error = "cudaMalloc failed (LSTM buffers)"; return MYEA_E_CUDA; }
  net->allocations.push_back(q);
  if (cudaMemsetAsync(q, 0, bytes, net->ctx.stream) != cudaSuccess) return MYEA_E_CUDA;
  *p = static_cast<T *>(q);
  return MYEA_OK;
}

#define LRC(expr) do { int rc__ = (expr); if (rc__ != MYEA_OK) return rc__; } while (0)

int lstm_create(myea_b200_net *net, LayerPlan &L) {
  const long long cpb = std::max<long long>(1, static_cast<long long>(L.desc.unit_parameters[1]));
  LstmPlan *P = new LstmPlan();
  L.lstm = P;
  P->dirs = L.desc.use_bidirectional ? 2 : 1;
  P->C = L.n_out / P->dirs;
  P->cpb = cpb;
  P->K = P->C / cpb;
  P->n_in = L.n_in;
  P->stride = static_cast<long long>(L.idx.block_stride);
  P->zoneout = L.desc.type_dropout == MYEA_DROPOUT_ZONEOUT;
  if (cpb != 1) return lstm_blocks_create(net, L, P);
  const long long rows = net->T * net->B, C = P->C;
  // biases: the reference stores first_bias_connection_index already shifted by the number of cells and then reads
  // [bz | bi | bf | bo] from it, so bo overlaps the next layer's bias slots.  Reproduced for the unidirectional layer;
  // the bidirectional layer (no usable reference) uses its true, unshifted block, one [bz|bi|bf|bo] run per direction.
  const long long fb = static_cast<long long>(L.idx.first_bias_connection_index);
  for (int d = 0; d < P->dirs; ++d) {
    LstmDir &D = P->d[d];
    D.w_base = static_cast<long long>(L.idx.first_connection_index) + d * C * P->stride;
    D.b_base = P->dirs == 1 ? fb : (fb - 2 * C) + d * 4 * C;
    if (D.b_base + 4 * C > static_cast<long long>(net->total_parameters)) {
      net->ctx.error = "LSTM output-gate bias would run past the parameter buffer (the next layer must be at least as wide as the LSTM layer)";
      return MYEA_E_INVALID;
    }
    LRC(lalloc(net, &D.gates_in, rows * 4 * C));
    LRC(lalloc(net, &D.act, rows * 4 * C));
    LRC(lalloc(net, &D.cstate, rows * C));
    LRC(lalloc(net, &D.cact, rows * C));
    LRC(lalloc(net, &D.dgates, rows * 4 * C));
    LRC(lalloc(net, &D.dcstate, rows * C));
    if (P->zoneout) {
      LRC(lalloc(net, &D.zone_state, net->T * C));
      LRC(lalloc(net, &D.zone_output, net->T * C));
      cudaMemsetAsync(D.zone_state, 1, net->T * C, net->ctx.stream);
      cudaMemsetAsync(D.zone_output, 1, net->T * C, net->ctx.stream);
    }
  }
  LRC(lalloc(net, &L.values, rows * L.n_out));
  LRC(lalloc(net, &L.deriv, rows * L.n_out));
  L.errors = L.deriv;
  LRC(lalloc(net, &P->s_rec, net->B * 4 * C));
  P->off_wrec = 0;
  const long long Cp = (C + 7) & ~7ll;
  P->off_wrect = P->off_wrec + panel_floats(4 * C, C) + 64;
  P->off_step = P->off_wrect + panel_floats(C, 4 * Cp) + 64;
  LRC(lalloc(net, &P->panel_mem, P->off_step + panel_floats(net->B, 4 * Cp) + 64));
  LRC(lalloc(net, &P->partial, static_cast<size_t>(7) * net->reduce_chunks * C));
  P->fuse = (C % 8 == 0) && net->ctx.gemm_engine == 0;
  if (P->fuse) {
    LRC(lalloc(net, &P->peep_compact, static_cast<size_t>(P->dirs) * 3 * C));
    // ping-pong operand panels, rows padded to whole 128-row tiles and zero (rows past the batch stay zero for ever)
    const long long prow = (net->B + 127) / 128 * 128;
    auto two_buffers = [&](long long k, Panels (&pan)[2]) -> int {
      const long long kp = (k + 31) / 32 * 32;
      float *mem = nullptr;
      LRC(lalloc(net, &mem, static_cast<size_t>(4 * prow * kp) + 64));
      for (int i = 0; i < 2; ++i) {
        pan[i] = Panels{};
        pan[i].hi = mem + i * prow * kp;
        pan[i].lo = mem + (2 + i) * prow * kp;
        pan[i].rows = net->B; pan[i].k = k; pan[i].kp = kp;
        pan[i].role = PANEL_ROLE_A; pan[i].major = PANEL_K;
      }
      return MYEA_OK;
    };
    LRC(two_buffers(C, P->h_pan));
    LRC(two_buffers(4 * Cp, P->dg_pan));
    LRC(lstm_persistent_plan(net, L));
  }
  // one-shot contractions use the handle's scratch: make sure it is large enough
  size_t need = 0;
  need = std::max(need, panel_floats(rows, L.n_in) + panel_floats(4 * C, L.n_in));            // input projection
  need = std::max(need, panel_floats(rows, 4 * Cp) + panel_floats(L.n_in, 4 * Cp));          // error to the previous layer
  need = std::max(need, panel_floats(4 * C, rows) + panel_floats(std::max(L.n_in, C), rows));  // weight derivatives
  P->shared_dw = net->ctx.gemm_engine == 0 && (C % 64) == 0 && (net->B % 8) == 0 && gemm_takes_mn_major(net->ctx, C, L.n_in) &&
                 gemm_takes_mn_major(net->ctx, C, C);
  if (P->shared_dw) need = std::max(need, shared_panel_floats(rows, 4 * C) + shared_panel_floats(rows, L.n_in) + shared_panel_floats(rows, L.n_out) + 256);
  net->scratch.floats = std::max(net->scratch.floats, need + 256);
  return MYEA_OK;
}

void lstm_destroy(LayerPlan &L) {
  lstm_persistent_destroy(L.lstm);
  delete L.lstm;
  L.lstm = nullptr;
}

float *lstm_output_errors(LayerPlan &L) { return L.deriv; }

int lstm_set_zoneout(myea_b200_net *net, LayerPlan &L, const uint8_t *state, const uint8_t *output, uint64_t count) {
  LstmPlan *P = L.lstm;
  if (P == nullptr || !P->zoneout || count != static_cast<uint64_t>(net->T * P->C * P->dirs)) {
    net->ctx.error = "layer has no zoneout masks of that size";
    return MYEA_E_INVALID;
  }
  // masks arrive as [T][dirs*C]
  for (int d = 0; d < P->dirs; ++d) {
    if (cudaMemcpy2DAsync(P->d[d].zone_state, P->C, state + d * P->C, P->dirs * P->C, P->C, net->T, cudaMemcpyHostToDevice, net->ctx.stream) != cudaSuccess ||
        cudaMemcpy2DAsync(P->d[d].zone_output, P->C, output + d * P->C, P->dirs * P->C, P->C, net->T, cudaMemcpyHostToDevice, net->ctx.stream) != cudaSuccess)
      return MYEA_E_CUDA;
  }
  return cudaStreamSynchronize(net->ctx.stream) == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// the per-direction zoneout arrays ([T][C] each) and probabilities of layer L, for the device-side mask generator
void lstm_zoneout_arrays(LayerPlan &L, int dir, uint8_t **state, uint8_t **output, long long *cells, int *dirs, float *p_state, float *p_output) {
  LstmPlan *P = L.lstm;
  *state = nullptr; *output = nullptr;
  if (P == nullptr || !P->zoneout || dir < 0 || dir >= P->dirs) return;
  *state = P->d[dir].zone_state;
  *output = P->d[dir].zone_output;
  *cells = P->C;
  *dirs = P->dirs;
  *p_state = L.desc.dropout_values[0];
  *p_output = L.desc.dropout_values[1];
}

static float *aligned_scratch(myea_b200_net *net) {
  return reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(net->scratch.base) + 255) & ~static_cast<uintptr_t>(255));
}

// [rows, 4C] gate matrix -> panel [rows, K = 4*Cp]: gate g occupies K columns [g*Cp, g*Cp + C); one pass when C is a
// multiple of 8, else one pass per gate (the panel builder zero-fills each gate's tail up to its group boundary)
static int prepare_gates(Context &ctx, const float *gates, long long rows, long long C, long long Cp, const Panels &dst) {
  if (Cp == C) return gemm_prepare_into(ctx, Operand{gates, rows, 4 * C, 4 * C, 1}, dst, 0, 0);
  for (int g = 0; g < 4; ++g) {
    int rc = gemm_prepare_into(ctx, Operand{gates + g * C, rows, C, 4 * C, 1}, dst, 0, g * Cp);
    if (rc != MYEA_OK) return rc;
  }
  return MYEA_OK;
}

// the 8-cell kernels: 128-thread blocks while 256-thread ones would leave SMs without a block (a 256 x 1024 step has
// 32768 threads: 128 blocks of 256 for 148 SMs), 256-thread blocks otherwise
static int cell_threads8(long long total) { return (total + 255) / 256 < 148 ? 128 : 256; }
static int cell_blocks8(long long total) {
  const long long t = cell_threads8(total);
  return static_cast<int>(std::max<long long>(1, std::min<long long>((total + t - 1) / t, 148 * 8)));
}
static int cell_blocks(long long total) { return static_cast<int>(std::max<long long>(1, std::min<long long>((total + 255) / 256, 148 * 8))); }

// ---------------------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------------------
int lstm_forward(myea_b200_net *net, LayerPlan &L, const float *input, long long n_in) {
  LstmPlan *P = L.lstm;
  if (P->cpb != 1) return lstm_blocks_forward(net, L, input, n_in);
  Context &ctx = net->ctx;
  const long long T = net->T, B = net->B, rows = T * B, C = P->C, ldh = L.n_out;
  const BlockOffsets off = block_offsets(n_in, C);
  float *scratch = aligned_scratch(net);
  Panels px;
  LRC(gemm_prepare(ctx, Operand{input, rows, n_in, n_in, 1}, scratch, &px, PANEL_ROLE_A));
  for (int d = 0; d < P->dirs; ++d) {
    LstmDir &D = P->d[d];
    const float *w = net->params + D.w_base;
    // fused input panel [4C, in], gate order z, i, f, o
    Panels pwin = panels_at(scratch + panel_floats(rows, n_in), 4 * C, n_in, PANEL_ROLE_B);
    LRC(gemm_prepare_into(ctx, Operand{w + off.z_in, C, n_in, P->stride, 1}, pwin, 0, 0));
    for (int g = 0; g < 3; ++g) LRC(gemm_prepare_into(ctx, Operand{w + off.in[g], C, n_in, P->stride, 1}, pwin, (g + 1) * C, 0));
    Epilogue e;
    e.C = D.gates_in;
    e.ldc = 4 * C;
    e.bias = net->params + D.b_base;
    LRC(gemm_panels(ctx, px, 0, rows, pwin, 0, 4 * C, e));
    // fused recurrent panel [4C, C]
    Panels pwrec = panels_at(P->panel_mem + P->off_wrec, 4 * C, C, PANEL_ROLE_B);
    float *peep_c = nullptr;
    if (P->fuse) {
      peep_c = P->peep_compact + static_cast<size_t>(d) * 3 * C;
      ctx.begin(TC_RECURRENT);
      lstm_gather_peepholes_kernel<<<static_cast<unsigned>((C + 255) / 256), 256, 0, ctx.stream>>>(w + off.peep, P->stride, C, peep_c);
      ctx.end(TC_RECURRENT);
    }
    const bool persistent = lstm_persistent_ready(P);
    if (persistent) {
      // rows interleaved cell by cell (row 4 * cell + gate): the 128 columns of a tile of the step's product then hold the
      // four gate sums of 32 cells side by side and the kernel finishes whole cells from its share of the tile
      LRC(gemm_prepare_interleaved(ctx, Operand{w + off.z_rec, C, C, P->stride, 1}, pwrec, 0, 4));
      for (int g = 0; g < 3; ++g) LRC(gemm_prepare_interleaved(ctx, Operand{w + off.rec[g], C, C, P->stride, 1}, pwrec, g + 1, 4));
    } else {
      LRC(gemm_prepare_into(ctx, Operand{w + off.z_rec, C, C, P->stride, 1}, pwrec, 0, 0));
      for (int g = 0; g < 3; ++g) LRC(gemm_prepare_into(ctx, Operand{w + off.rec[g], C, C, P->stride, 1}, pwrec, (g + 1) * C, 0));
    }
    const bool zone = P->zoneout && net->training;
    for (long long s = 0; s < T; ++s) {
      const long long t = d == 0 ? s : T - 1 - s;
      const long long tp = d == 0 ? t - 1 : t + 1;
      float *h_t = L.values + t * B * ldh + d * C;
      if (persistent && s > 0) {  // one launch walks steps 1 .. T-1
        LRC(lstm_persistent_forward(net, L, d, pwrec, peep_c, zone));
        break;
      }
      if (P->fuse && s > 0) {
        // recurrent contraction on the panels the previous step left, then the cell kernel; h_t leaves as the layer
        // output and as the operand panels of step s + 1
        const Panels &ph_prev = P->h_pan[(s - 1) & 1];
        const Panels &ph_next = P->h_pan[s & 1];
        Epilogue e;
        LstmStep f;
        f.C = C; f.ldh = ldh; f.kp = ph_next.kp;
        f.peep = peep_c;
        if (s + 1 < T) { f.p_hi = ph_next.hi; f.p_cross = ph_next.lo; }
        f.gates_in = D.gates_in + t * B * 4 * C;
        f.c_prev = D.cstate + tp * B * C;
        f.h_prev = L.values + tp * B * ldh + d * C;
        f.act = D.act + t * B * 4 * C;
        f.cstate = D.cstate + t * B * C;
        f.cact = D.cact + t * B * C;
        f.h = h_t;
        f.zone_state = zone ? D.zone_state + t * C : nullptr;
        f.zone_output = zone ? D.zone_output + t * C : nullptr;
        e.C = P->s_rec;
        e.ldc = 4 * C;
        LRC(gemm_panels(ctx, ph_prev, 0, B, pwrec, 0, 4 * C, e));
        ctx.begin(TC_RECURRENT);
        launch_dependent(ctx, lstm_cells8_forward_kernel, dim3(cell_blocks8(B * C / 8)), dim3(cell_threads8(B * C / 8)), 0, f, static_cast<const float *>(P->s_rec), B);
        ctx.end(TC_RECURRENT);
        continue;
      }
      CellFwd cf;
      cf.gates_in = D.gates_in + t * B * 4 * C;
      cf.s_rec = nullptr; cf.c_prev = nullptr; cf.h_prev = nullptr;
      if (s > 0) {
        const float *h_prev = L.values + tp * B * ldh + d * C;
        Panels ph;
        LRC(gemm_prepare(ctx, Operand{h_prev, B, C, ldh, 1}, P->panel_mem + P->off_step, &ph, PANEL_ROLE_A));
        Epilogue er;
        er.C = P->s_rec;
        er.ldc = 4 * C;
        LRC(gemm_panels(ctx, ph, 0, B, pwrec, 0, 4 * C, er));
        cf.s_rec = P->s_rec;
        cf.c_prev = D.cstate + tp * B * C;
        cf.h_prev = h_prev;
      }
      cf.peep = w + off.peep;
      cf.stride = P->stride;
      cf.act = D.act + t * B * 4 * C;
      cf.cstate = D.cstate + t * B * C;
      cf.cact = D.cact + t * B * C;
      cf.h = h_t;
      cf.ldh = ldh;
      cf.zone_state = zone ? D.zone_state + t * C : nullptr;
      cf.zone_output = zone ? D.zone_output + t * C : nullptr;
      cf.B = B; cf.C = C;
      ctx.begin(TC_RECURRENT);
      lstm_cell_forward_kernel<<<cell_blocks(B * C), 256, 0, ctx.stream>>>(cf);
      ctx.end(TC_RECURRENT);
      if (P->fuse && T > 1)  // first step: its output becomes the operand of the second step
        LRC(gemm_prepare_into(ctx, Operand{h_t, B, C, ldh, 1}, P->h_pan[0], 0, 0));
    }
  }
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// ---------------------------------------------------------------------------------------------------------
// BPTT: L.deriv holds the error arriving on the layer's outputs from its consumers
// ---------------------------------------------------------------------------------------------------------
int lstm_backward(myea_b200_net *net, LayerPlan &L) {
  LstmPlan *P = L.lstm;
  if (P->cpb != 1) return lstm_blocks_backward(net, L);
  Context &ctx = net->ctx;
  const long long T = net->T, B = net->B, C = P->C, ldh = L.n_out, n_in = P->n_in;
  const long long Cp = (C + 7) & ~7ll;  // each gate's K segment starts on a group-of-8 boundary
  const BlockOffsets off = block_offsets(n_in, C);
  for (int d = 0; d < P->dirs; ++d) {
    LstmDir &D = P->d[d];
    const float *w = net->params + D.w_base;
    // transposed recurrent panel [C (unit j of h), K = 4C (gate, cell)]
    Panels pwt = panels_at(P->panel_mem + P->off_wrect, C, 4 * Cp, PANEL_ROLE_B);
    LRC(gemm_prepare_into(ctx, Operand{w + off.z_rec, C, C, 1, P->stride}, pwt, 0, 0));
    for (int g = 0; g < 3; ++g) LRC(gemm_prepare_into(ctx, Operand{w + off.rec[g], C, C, 1, P->stride}, pwt, 0, (g + 1) * Cp));
    for (long long s = 0; s < T; ++s) {
      const long long t = d == 0 ? T - 1 - s : s;      // walk against the layer's direction
      const long long tn = d == 0 ? t + 1 : t - 1;     // the step after t in the layer's direction
      const long long tp = d == 0 ? t - 1 : t + 1;     // the step before t
      float *dh_t = L.deriv + t * B * ldh + d * C;
      if (lstm_persistent_ready(P) && s > 0) {  // one launch walks the remaining steps
        LRC(lstm_persistent_backward(net, L, d, pwt, P->peep_compact + static_cast<size_t>(d) * 3 * C));
        break;
      }
      if (P->fuse && s > 0) {
        // error through time (gate errors of the next step times W_rec) on the panels the previous step left, then the
        // cell's backward arithmetic; the gate errors of step t leave as arrays and as the next operand panels
        const Panels &pd_prev = P->dg_pan[(s - 1) & 1];
        const Panels &pd_next = P->dg_pan[s & 1];
        Epilogue e;
        LstmStep f;
        f.C = C; f.ldh = ldh; f.kp = pd_next.kp; f.Cp = Cp;
        f.peep = P->peep_compact + static_cast<size_t>(d) * 3 * C;
        if (s + 1 < T) { f.p_hi = pd_next.hi; f.p_cross = pd_next.lo; }
        f.dh = dh_t;
        f.b_act = D.act + t * B * 4 * C;
        f.b_cact = D.cact + t * B * C;
        f.b_c_prev = (tp >= 0 && tp < T) ? D.cstate + tp * B * C : nullptr;
        f.act_next = D.act + tn * B * 4 * C;
        f.dgates_next = D.dgates + tn * B * 4 * C;
        f.dc_next = D.dcstate + tn * B * C;
        f.dgates = D.dgates + t * B * 4 * C;
        f.dcstate = D.dcstate + t * B * C;
        e.C = dh_t;
        e.ldc = ldh;
        e.accumulate = 1;
        LRC(gemm_panels(ctx, pd_prev, 0, B, pwt, 0, C, e));
        ctx.begin(TC_RECURRENT);
        launch_dependent(ctx, lstm_cells8_backward_kernel, dim3(cell_blocks8(B * C / 8)), dim3(cell_threads8(B * C / 8)), 0, f, B);
        ctx.end(TC_RECURRENT);
        continue;
      }
      if (s > 0) {
        Panels pd = panels_at(P->panel_mem + P->off_step, B, 4 * Cp, PANEL_ROLE_A);
        LRC(prepare_gates(ctx, D.dgates + tn * B * 4 * C, B, C, Cp, pd));
        Epilogue e;
        e.C = dh_t;
        e.ldc = ldh;
        e.accumulate = 1;
        LRC(gemm_panels(ctx, pd, 0, B, pwt, 0, C, e));
      }
      CellBwd cb;
      cb.dh = dh_t;
      cb.ldh = ldh;
      cb.act = D.act + t * B * 4 * C;
      cb.cact = D.cact + t * B * C;
      cb.c_prev = (tp >= 0 && tp < T) ? D.cstate + tp * B * C : nullptr;
      cb.act_next = s > 0 ? D.act + tn * B * 4 * C : nullptr;
      cb.dgates_next = s > 0 ? D.dgates + tn * B * 4 * C : nullptr;
      cb.dc_next = s > 0 ? D.dcstate + tn * B * C : nullptr;
      cb.peep = w + off.peep;
      cb.stride = P->stride;
      cb.dgates = D.dgates + t * B * 4 * C;
      cb.dcstate = D.dcstate + t * B * C;
      cb.B = B; cb.C = C;
      ctx.begin(TC_RECURRENT);
      lstm_cell_backward_kernel<<<cell_blocks(B * C), 256, 0, ctx.stream>>>(cb);
      ctx.end(TC_RECURRENT);
      if (P->fuse && T > 1)  // last time step (first of the walk): its gate errors are the operand of the next contraction
        LRC(prepare_gates(ctx, D.dgates + t * B * 4 * C, B, C, Cp, P->dg_pan[0]));
    }
  }
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// error of the LSTM layer L propagated to the outputs of the layer feeding it: prev_deriv [T*B, n_in] = sum over
// directions of dgates [T*B, 4C] * W_in [4C, n_in].  `finish` (optional) carries the activation derivative of a fully
// connected layer below, applied by the epilogue of the last direction's contraction to the complete sum.
int lstm_backward_to_input(myea_b200_net *net, LayerPlan &L, float *prev_deriv, const LayerPlan &prev, const Epilogue *finish) {
  LstmPlan *P = L.lstm;
  if (P->cpb != 1) return lstm_blocks_backward_to_input(net, L, prev_deriv, prev, finish);
  Context &ctx = net->ctx;
  const long long rows = net->T * net->B, C = P->C, n_in = P->n_in;
  if (prev.n_out != n_in) return MYEA_E_INVALID;
  const long long Cp = (C + 7) & ~7ll;
  const BlockOffsets off = block_offsets(n_in, C);
  float *scratch = aligned_scratch(net);
  for (int d = 0; d < P->dirs; ++d) {
    LstmDir &D = P->d[d];
    const float *w = net->params + D.w_base;
    Panels pd = panels_at(scratch, rows, 4 * Cp, PANEL_ROLE_A);
    LRC(prepare_gates(ctx, D.dgates, rows, C, Cp, pd));
    Panels pwt = panels_at(scratch + panel_floats(rows, 4 * Cp), n_in, 4 * Cp, PANEL_ROLE_B);  // [n_in, K = 4 gates]
    LRC(gemm_prepare_into(ctx, Operand{w + off.z_in, n_in, C, 1, P->stride}, pwt, 0, 0));
    for (int g = 0; g < 3; ++g) LRC(gemm_prepare_into(ctx, Operand{w + off.in[g], n_in, C, 1, P->stride}, pwt, 0, (g + 1) * Cp));
    Epilogue e;
    if (finish != nullptr && d == P->dirs - 1) e = *finish;
    e.C = prev_deriv;
    e.ldc = n_in;
    if (d > 0 && finish != nullptr) { e.addend = prev_deriv; e.ld_addend = n_in; }  // the addend enters before the derivative
    else e.accumulate = d > 0 ? 1 : 0;
    LRC(gemm_panels(ctx, pd, 0, rows, pwt, 0, n_in, e));
  }
  return MYEA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// derivative weights: dW_in,g += dg^T x ; dW_rec,g += dg(next step)^T h ; peepholes and biases by column reductions
// ---------------------------------------------------------------------------------------------------------
int lstm_update_derivative_weight(myea_b200_net *net, LayerPlan &L, const float *input, long long n_in) {
  LstmPlan *P = L.lstm;
  if (P->cpb != 1) return lstm_blocks_update_derivative_weight(net, L, input, n_in);
  Context &ctx = net->ctx;
  const long long T = net->T, B = net->B, rows = T * B, C = P->C, ldh = L.n_out;
  const BlockOffsets off = block_offsets(n_in, C);
  float *scratch = aligned_scratch(net);
  for (int d = 0; d < P->dirs; ++d) {
    LstmDir &D = P->d[d];
    float *gw = net->grads + D.w_base;
    if (P->shared_dw) {
      // Both operands of every weight-derivative contraction are read through their columns (K = rows of the batch
      // and time axis), so one untransposed split pass per tensor serves all of them: gate errors, layer input, and
      // the layer's own outputs for the recurrent weights (a sub-range of K rows and of columns).
      float *mem_d = scratch;
      float *mem_x = mem_d + ((shared_panel_floats(rows, 4 * C) + 63) & ~static_cast<size_t>(63));
      float *mem_h = mem_x + ((shared_panel_floats(rows, n_in) + 63) & ~static_cast<size_t>(63));
      Panels pd, px, ph;
      LRC(gemm_prepare_shared(ctx, D.dgates, 4 * C, rows, 4 * C, mem_d, PANEL_ROLE_A, nullptr, PANEL_ROLE_A, &pd));
      LRC(gemm_prepare_shared(ctx, input, n_in, rows, n_in, mem_x, PANEL_ROLE_B, nullptr, PANEL_ROLE_B, &px));
      const long long in_off[4] = {off.z_in, off.in[0], off.in[1], off.in[2]};
      {  // the four gates in one contraction: row g*C + c of the product lands in block c at gate g's offset
        Epilogue e;
        e.C = gw;
        e.ldc = P->stride;
        e.accumulate = 1;
        e.seg_rows = C;
        for (int g = 0; g < 4; ++g) e.seg_off[g] = in_off[g];
        LRC(gemm_panels(ctx, pd, 0, 4 * C, px, 0, n_in, e));
      }
      if (T > 1) {
        LRC(gemm_prepare_shared(ctx, L.values, ldh, rows, ldh, mem_h, PANEL_ROLE_B, nullptr, PANEL_ROLE_B, &ph));
        const long long K = (T - 1) * B;
        // K rows of steps 1..T-1 of the gate errors against steps 0..T-2 of the outputs (forward direction), the
        // other way round for the backward direction: a K offset of B rows on one side
        Panels pdk = pd, phk = ph;
        const long long kd = d == 0 ? B : 0, kh = d == 0 ? 0 : B;
        pdk.hi += kd * pd.kp;
        pdk.lo = reinterpret_cast<float *>(reinterpret_cast<uint16_t *>(pd.lo) + 2 * kd * pd.kp);
        pdk.k = K;
        phk.hi += kh * ph.kp;
        phk.lo = reinterpret_cast<float *>(reinterpret_cast<uint16_t *>(ph.lo) + 2 * kh * ph.kp);
        phk.k = K;
        const long long rec_off[4] = {off.z_rec, off.rec[0], off.rec[1], off.rec[2]};
        Epilogue e;
        e.C = gw;
        e.ldc = P->stride;
        e.accumulate = 1;
        e.seg_rows = C;
        for (int g = 0; g < 4; ++g) e.seg_off[g] = rec_off[g];
        LRC(gemm_panels(ctx, pdk, 0, 4 * C, phk, d * C, C, e));
      }
    } else {
    // input weights: K = all T*B rows
    Panels pdt, pxt;
    LRC(gemm_prepare(ctx, Operand{D.dgates, 4 * C, rows, 1, 4 * C}, scratch, &pdt, PANEL_ROLE_A));                        // dgates^T [4C, rows]
    LRC(gemm_prepare(ctx, Operand{input, n_in, rows, 1, n_in}, scratch + panel_floats(4 * C, rows), &pxt, PANEL_ROLE_B));  // x^T [n_in, rows]
    const long long in_off[4] = {off.z_in, off.in[0], off.in[1], off.in[2]};
    for (int g = 0; g < 4; ++g) {
      Epilogue e;
      e.C = gw + in_off[g];
      e.ldc = P->stride;
      e.accumulate = 1;
      LRC(gemm_panels(ctx, pdt, g * C, C, pxt, 0, n_in, e));
    }
    // recurrent weights: pairs (gate error of the next step in the layer's direction, output of this step)
    if (T > 1) {
      const long long K = (T - 1) * B;
      const float *dg0 = d == 0 ? D.dgates + B * 4 * C : D.dgates;              // rows of steps 1..T-1 (forward) / 0..T-2 (backward)
      const float *h0 = d == 0 ? L.values + d * C : L.values + B * ldh + d * C;  // rows of steps 0..T-2 (forward) / 1..T-1 (backward)
      Panels pdr, pht;
      LRC(gemm_prepare(ctx, Operand{dg0, 4 * C, K, 1, 4 * C}, scratch, &pdr, PANEL_ROLE_A));
      LRC(gemm_prepare(ctx, Operand{h0, C, K, 1, ldh}, scratch + panel_floats(4 * C, K), &pht, PANEL_ROLE_B));
      const long long rec_off[4] = {off.z_rec, off.rec[0], off.rec[1], off.rec[2]};
      for (int g = 0; g < 4; ++g) {
        Epilogue e;
        e.C = gw + rec_off[g];
        e.ldc = P->stride;
        e.accumulate = 1;
        LRC(gemm_panels(ctx, pdr, g * C, C, pht, 0, C, e));
      }
    }
    }
    // biases and peepholes
    const int chunks = static_cast<int>(std::max<long long>(1, std::min<long long>(net->reduce_chunks, rows / 8)));
    ctx.begin(TC_RECURRENT);
    dim3 grid(static_cast<unsigned>((C + 31) / 32), chunks);
    lstm_bias_peephole_reduce_kernel<<<grid, 256, 0, ctx.stream>>>(D.dgates, D.cstate, rows, C, d == 0 ? B : -B, chunks, P->partial);
    lstm_bias_peephole_finalize_kernel<<<static_cast<unsigned>((C + 31) / 32), 256, 0, ctx.stream>>>(P->partial, chunks, C, net->grads + D.b_base,
                                                                                                    gw + off.peep, P->stride);
    ctx.end(TC_RECURRENT, 2);
  }
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

}  // namespace myea
