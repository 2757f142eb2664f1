// LSTM layers whose blocks hold SEVERAL cells (Layer::ptr_array_block_units with more than one Cell_unit each).
//
// The cells of a block share its input, forget and output gate; each gate sees the states of all the block's cells
// through its peepholes.  With C cells in K blocks (cpb = C / K cells each) a step is
//   z_j = tanh(Wz_j x + Rz_j h_prev + bz_j)                                         per cell j
//   i_k = sig(Wi_k x + Ri_k h_prev + bi_k + sum_{j in k} pi_j c_prev_j)             per block k (f_k alike)
//   c_j = z_j i_k + f_k c_prev_j ;  o_k = sig(Wo_k x + Ro_k h_prev + bo_k + sum_{j in k} po_j c_j) ;  h_j = tanh(c_j) o_k
// Reference routines: Forward_Pass__LSTM__Gates_CIFO / __Gates_CIF_AF_State / __States_AF / __Output
// (Neural_Network__Recurrent_Forward_Pass__OpenMP.cpp:859-1582), Backward_Pass__LSTM_Derivative__Output / __Cell_State_AF /
// __Gates_CIF_AF_State (Neural_Network__Recurrent_Backward_Pass__OpenMP.cpp:1130-1604), Backward_Pass__LSTM (:1024-1120),
// Recurrent__Update_Derivative_Weight__LSTM + bias (Neural_Network__Recurrent_Update_Derivative_Weight__OpenMP.cpp:492-776).
//
// Mapping to the GPU: the gate rows have G = C + 3K columns [z (C) | i (K) | f (K) | o (K)].  The weights of those G rows
// are gathered once per pass from the reference's per-block parameter layout into dense matrices W_in [G, in] and
// W_rec [G, C] (the biases already lie as one run of G values), every contraction then runs on the tensor-core GEMM, a
// cell kernel with one thread per (row, block) does the block's arithmetic, and the weight derivatives are scattered
// back into the parameter layout.  The single-cell layer (every shipped configuration) has its own, faster path in
// lstm.cu / lstm_persistent.cu.
#include "lstm.cuh"
#include "panel_math.cuh"

#include <algorithm>

namespace myea {

#define BRC(expr) do { int rc__ = (expr); if (rc__ != MYEA_OK) return rc__; } while (0)

// positions inside the flat parameter buffer (Prepare__Connections__LSTM, Neural_Network__Prepare_Connections.cpp): per
// block, per cell [Wz_in (in) | Wz_rec (C)], then Wi_in Wf_in Wo_in (in each), Wi_rec Wf_rec Wo_rec (C each), then the
// peepholes p_i p_f p_o (cpb each)
struct BlockLayout {
  long long base, stride, I, C, K, cpb;
  __host__ __device__ long long gate_base(long long k) const { return base + k * stride + cpb * (I + C); }
  __host__ __device__ long long w_in(long long row, long long col) const {
    if (row < C) return base + (row / cpb) * stride + (row % cpb) * (I + C) + col;
    const long long g = (row - C) / K, k = (row - C) % K;
    return gate_base(k) + g * I + col;
  }
  __host__ __device__ long long w_rec(long long row, long long col) const {
    if (row < C) return base + (row / cpb) * stride + (row % cpb) * (I + C) + I + col;
    const long long g = (row - C) / K, k = (row - C) % K;
    return gate_base(k) + 3 * I + g * C + col;
  }
  __host__ __device__ long long peephole(long long g, long long cell) const { return gate_base(cell / cpb) + 3 * I + 3 * C + g * cpb + cell % cpb; }
};

// dense [W_in (G x I) | W_rec (G x C) | peepholes (3 x C)] <-> parameter layout.  SCATTER: flat[pos] += dense[i]
template <bool SCATTER>
__global__ void __launch_bounds__(256) lstm_blocks_weights_kernel(const BlockLayout lay, float *__restrict__ flat, float *__restrict__ w_in,
                                                                  float *__restrict__ w_rec, float *__restrict__ peep) {
  const long long G = lay.C + 3 * lay.K, n_in = G * lay.I, n_rec = G * lay.C, total = n_in + n_rec + 3 * lay.C;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long pos;
    float *dense;
    if (i < n_in) { pos = lay.w_in(i / lay.I, i % lay.I); dense = w_in + i; }
    else if (i < n_in + n_rec) { const long long r = i - n_in; pos = lay.w_rec(r / lay.C, r % lay.C); dense = w_rec + r; }
    else { const long long r = i - n_in - n_rec; pos = lay.peephole(r / lay.C, r % lay.C); dense = peep + r; }
    if (SCATTER) flat[pos] += *dense;
    else *dense = flat[pos];
  }
}

struct BlocksFwd {
  const float *gates_in, *s_rec;   // rows of step t [B, G]; recurrent product [B, G] or null at the first step
  const float *c_prev, *h_prev;    // [B, C], [B, ldh]; null at the first step
  const float *peep;               // [3][C]
  float *act, *cstate, *cact, *h;  // rows of step t: [B, G], [B, C], [B, C], [B, ldh]
  const uint8_t *zone_state, *zone_output;  // [C] of step t, or null
  long long B, C, K, cpb, ldh;
};

__global__ void __launch_bounds__(128) lstm_blocks_forward_kernel(const BlocksFwd p) {
  const long long total = p.B * p.K, G = p.C + 3 * p.K;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = i / p.K, k = i - b * p.K, j0 = k * p.cpb;
    const bool first = p.s_rec == nullptr;
    const float *gi = p.gates_in + b * G;
    const float *sr = first ? nullptr : p.s_rec + b * G;
    const float *cp = first ? nullptr : p.c_prev + b * p.C;
    float si = gi[p.C + k], sf = gi[p.C + p.K + k], so = gi[p.C + 2 * p.K + k];
    if (!first) {
      si += sr[p.C + k]; sf += sr[p.C + p.K + k]; so += sr[p.C + 2 * p.K + k];
      for (long long j = j0; j < j0 + p.cpb; ++j) {
        si = fmaf(p.peep[j], cp[j], si);
        sf = fmaf(p.peep[p.C + j], cp[j], sf);
      }
    }
    const float ig = sigmoid_ref(si), fg = first ? 0.f : sigmoid_ref(sf);
    float *act = p.act + b * G;
    for (long long j = j0; j < j0 + p.cpb; ++j) {
      const float z = tanh_ref(gi[j] + (first ? 0.f : sr[j]));
      const float c_old = first ? 0.f : cp[j];
      float cs = z * ig;
      if (!first) cs += fg * c_old;
      if (p.zone_state != nullptr && !p.zone_state[j]) cs = c_old;
      act[j] = z;
      p.cstate[b * p.C + j] = cs;
      p.cact[b * p.C + j] = tanh_ref(cs);
      so = fmaf(p.peep[2 * p.C + j], cs, so);
    }
    const float og = sigmoid_ref(so);
    act[p.C + k] = ig; act[p.C + p.K + k] = fg; act[p.C + 2 * p.K + k] = og;
    for (long long j = j0; j < j0 + p.cpb; ++j) {
      float h = p.cact[b * p.C + j] * og;
      if (p.zone_output != nullptr && !p.zone_output[j]) h = first ? 0.f : p.h_prev[b * p.ldh + j];
      p.h[b * p.ldh + j] = h;
    }
  }
}

struct BlocksBwd {
  const float *dh;                  // [B, ldh] error on the outputs of step t, the part through time already added
  const float *act, *cact, *c_prev; // step t; c_prev null at the first step of the layer's direction
  const float *act_next, *dgates_next, *dc_next;  // the step after t in the layer's direction, null at its last step
  const float *peep;
  float *dgates, *dcstate;
  long long B, C, K, cpb, ldh;
};

__global__ void __launch_bounds__(128) lstm_blocks_backward_kernel(const BlocksBwd p) {
  const long long total = p.B * p.K, G = p.C + 3 * p.K;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = i / p.K, k = i - b * p.K, j0 = k * p.cpb;
    const float *act = p.act + b * G;
    const float ig = act[p.C + k], fg = act[p.C + p.K + k], og = act[p.C + 2 * p.K + k];
    float sum_o = 0.f;
    for (long long j = j0; j < j0 + p.cpb; ++j) sum_o = fmaf(p.dh[b * p.ldh + j], p.cact[b * p.C + j], sum_o);
    const float d_o = og * (1.f - og) * sum_o;
    const bool has_next = p.dgates_next != nullptr;
    const float di_n = has_next ? p.dgates_next[b * G + p.C + k] : 0.f, df_n = has_next ? p.dgates_next[b * G + p.C + p.K + k] : 0.f;
    const float f_n = has_next ? p.act_next[b * G + p.C + p.K + k] : 0.f;
    float sum_i = 0.f, sum_f = 0.f;
    float *dg = p.dgates + b * G;
    for (long long j = j0; j < j0 + p.cpb; ++j) {
      const float a = p.cact[b * p.C + j], z = act[j];
      float dc = p.dh[b * p.ldh + j] * og * (1.f - a * a);
      dc += p.peep[2 * p.C + j] * d_o;
      if (has_next) {
        dc += p.peep[j] * di_n;
        dc += p.peep[p.C + j] * df_n;
        dc += p.dc_next[b * p.C + j] * f_n;
      }
      dg[j] = dc * ig * (1.f - z * z);
      sum_i = fmaf(dc, z, sum_i);
      if (p.c_prev != nullptr) sum_f = fmaf(dc, p.c_prev[b * p.C + j], sum_f);
      p.dcstate[b * p.C + j] = dc;
    }
    dg[p.C + k] = sum_i * (ig * (1.f - ig));
    dg[p.C + p.K + k] = p.c_prev != nullptr ? sum_f * (fg * (1.f - fg)) : 0.f;
    dg[p.C + 2 * p.K + k] = d_o;
  }
}

// products whose column sums are the peephole derivatives: out [R, 3C] = [di(r) c(r - shift) | df(r) c(r - shift) | do(r) c(r)],
// gate errors taken from the cell's block, 0 where row r - shift does not exist
__global__ void __launch_bounds__(256) lstm_blocks_peephole_products_kernel(const float *__restrict__ dgates, const float *__restrict__ cstate,
                                                                            long long R, long long C, long long K, long long cpb, long long shift,
                                                                            float *__restrict__ out) {
  const long long total = R * C, G = C + 3 * K;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / C, j = i - r * C, k = j / cpb, rp = r - shift;
    const float *dg = dgates + r * G;
    const bool partner = rp >= 0 && rp < R;
    const float c_old = partner ? cstate[rp * C + j] : 0.f;
    float *o = out + r * 3 * C;
    o[j] = dg[C + k] * c_old;
    o[C + j] = dg[C + K + k] * c_old;
    o[2 * C + j] = dg[C + 2 * K + k] * cstate[r * C + j];
  }
}

template <typename T>
static int balloc(myea_b200_net *net, T **p, size_t count) {
  void *q = nullptr;
  const size_t bytes = std::max<size_t>(count, 1) * sizeof(T);
  if (cudaMalloc(&q, bytes) != cudaSuccess) { net->ctx.error = "cudaMalloc failed (LSTM buffers)"; return MYEA_E_CUDA; }
  net->allocations.push_back(q);
  if (cudaMemsetAsync(q, 0, bytes, net->ctx.stream) != cudaSuccess) return MYEA_E_CUDA;
  *p = static_cast<T *>(q);
  return MYEA_OK;
}

static int grid_for(long long total, int threads) { return static_cast<int>(std::max<long long>(1, std::min<long long>((total + threads - 1) / threads, 148 * 8))); }

static BlockLayout layout_of(const LstmPlan *P, int d) {
  BlockLayout lay;
  lay.base = P->d[d].w_base; lay.stride = P->stride; lay.I = P->n_in; lay.C = P->C; lay.K = P->K; lay.cpb = P->cpb;
  return lay;
}

int lstm_blocks_create(myea_b200_net *net, LayerPlan &L, LstmPlan *P) {
  const long long rows = net->T * net->B, C = P->C, K = P->K, G = C + 3 * K, I = P->n_in;
  const long long fb = static_cast<long long>(L.idx.first_bias_connection_index);
  for (int d = 0; d < P->dirs; ++d) {
    LstmDir &D = P->d[d];
    D.w_base = static_cast<long long>(L.idx.first_connection_index) + d * K * P->stride;
    // [bz (C) | bi (K) | bf (K) | bo (K)] from the reference's base, which is already shifted by the number of cells (its
    // tail overlaps the next layer's biases); a bidirectional layer uses its true block, one run per direction
    D.b_base = P->dirs == 1 ? fb : (fb - P->dirs * C) + d * G;
    if (D.b_base + G > static_cast<long long>(net->total_parameters)) {
      net->ctx.error = "LSTM gate biases would run past the parameter buffer (the next layer must be at least as wide as the LSTM layer has cells)";
      return MYEA_E_INVALID;
    }
    BRC(balloc(net, &D.gates_in, rows * G));
    BRC(balloc(net, &D.act, rows * G));
    BRC(balloc(net, &D.dgates, rows * G));
    BRC(balloc(net, &D.cstate, rows * C));
    BRC(balloc(net, &D.cact, rows * C));
    BRC(balloc(net, &D.dcstate, rows * C));
    if (P->zoneout) {
      BRC(balloc(net, &D.zone_state, net->T * C));
      BRC(balloc(net, &D.zone_output, net->T * C));
      cudaMemsetAsync(D.zone_state, 1, net->T * C, net->ctx.stream);
      cudaMemsetAsync(D.zone_output, 1, net->T * C, net->ctx.stream);
    }
  }
  BRC(balloc(net, &L.values, rows * L.n_out));
  BRC(balloc(net, &L.deriv, rows * L.n_out));
  L.errors = L.deriv;
  BRC(balloc(net, &P->s_rec, net->B * G));
  BRC(balloc(net, &P->blk_w_in, static_cast<size_t>(G * I)));
  BRC(balloc(net, &P->blk_w_rec, static_cast<size_t>(G * C)));
  BRC(balloc(net, &P->blk_peep, static_cast<size_t>(3 * C)));
  BRC(balloc(net, &P->blk_dw_in, static_cast<size_t>(G * I)));
  BRC(balloc(net, &P->blk_dw_rec, static_cast<size_t>(G * C)));
  BRC(balloc(net, &P->blk_dpeep, static_cast<size_t>(3 * C)));
  BRC(balloc(net, &P->blk_products, static_cast<size_t>(rows * 3 * C)));
  BRC(balloc(net, &P->partial, static_cast<size_t>(net->reduce_chunks) * std::max(3 * C, G)));
  size_t need = 0;
  need = std::max(need, gemm_scratch_floats(rows, G, I));      // input projection
  need = std::max(need, gemm_scratch_floats(net->B, G, C));    // recurrent step
  need = std::max(need, gemm_scratch_floats(net->B, C, G));    // error through time
  need = std::max(need, gemm_scratch_floats(rows, I, G));      // error to the previous layer
  need = std::max(need, gemm_scratch_floats(G, std::max(I, C), rows));  // weight derivatives
  net->scratch.floats = std::max(net->scratch.floats, need + 256);
  return MYEA_OK;
}

static int gather_weights(myea_b200_net *net, const LstmPlan *P, int d) {
  Context &ctx = net->ctx;
  const BlockLayout lay = layout_of(P, d);
  const long long total = (P->C + 3 * P->K) * (P->n_in + P->C) + 3 * P->C;
  ctx.begin(TC_RECURRENT);
  lstm_blocks_weights_kernel<false><<<grid_for(total, 256), 256, 0, ctx.stream>>>(lay, net->params, P->blk_w_in, P->blk_w_rec, P->blk_peep);
  ctx.end(TC_RECURRENT);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

int lstm_blocks_forward(myea_b200_net *net, LayerPlan &L, const float *input, long long n_in) {
  LstmPlan *P = L.lstm;
  Context &ctx = net->ctx;
  const long long T = net->T, B = net->B, rows = T * B, C = P->C, K = P->K, G = C + 3 * K, ldh = L.n_out;
  const bool zone = P->zoneout && net->training;
  for (int d = 0; d < P->dirs; ++d) {
    LstmDir &D = P->d[d];
    BRC(gather_weights(net, P, d));
    {
      Epilogue e;
      e.C = D.gates_in;
      e.ldc = G;
      e.bias = net->params + D.b_base;
      BRC(gemm_nt(ctx, Operand{input, rows, n_in, n_in, 1}, Operand{P->blk_w_in, G, n_in, n_in, 1}, e, net->scratch));
    }
    for (long long s = 0; s < T; ++s) {
      const long long t = d == 0 ? s : T - 1 - s, tp = d == 0 ? t - 1 : t + 1;
      BlocksFwd f;
      f.gates_in = D.gates_in + t * B * G;
      f.s_rec = nullptr; f.c_prev = nullptr; f.h_prev = nullptr;
      if (s > 0) {
        f.h_prev = L.values + tp * B * ldh + d * C;
        f.c_prev = D.cstate + tp * B * C;
        Epilogue e;
        e.C = P->s_rec;
        e.ldc = G;
        BRC(gemm_nt(ctx, Operand{f.h_prev, B, C, ldh, 1}, Operand{P->blk_w_rec, G, C, C, 1}, e, net->scratch));
        f.s_rec = P->s_rec;
      }
      f.peep = P->blk_peep;
      f.act = D.act + t * B * G;
      f.cstate = D.cstate + t * B * C;
      f.cact = D.cact + t * B * C;
      f.h = L.values + t * B * ldh + d * C;
      f.zone_state = zone ? D.zone_state + t * C : nullptr;
      f.zone_output = zone ? D.zone_output + t * C : nullptr;
      f.B = B; f.C = C; f.K = K; f.cpb = P->cpb; f.ldh = ldh;
      ctx.begin(TC_RECURRENT);
      lstm_blocks_forward_kernel<<<grid_for(B * K, 128), 128, 0, ctx.stream>>>(f);
      ctx.end(TC_RECURRENT);
    }
  }
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// BPTT: L.deriv holds the error arriving on the layer's outputs from its consumers
int lstm_blocks_backward(myea_b200_net *net, LayerPlan &L) {
  LstmPlan *P = L.lstm;
  Context &ctx = net->ctx;
  const long long T = net->T, B = net->B, C = P->C, K = P->K, G = C + 3 * K, ldh = L.n_out;
  for (int d = 0; d < P->dirs; ++d) {
    LstmDir &D = P->d[d];
    BRC(gather_weights(net, P, d));  // a bidirectional layer shares the dense buffers between its directions
    for (long long s = 0; s < T; ++s) {
      const long long t = d == 0 ? T - 1 - s : s;   // against the layer's direction
      const long long tn = d == 0 ? t + 1 : t - 1, tp = d == 0 ? t - 1 : t + 1;
      float *dh_t = L.deriv + t * B * ldh + d * C;
      if (s > 0) {  // dh_t += dgates(next step) [B, G] x W_rec [G, C]
        Epilogue e;
        e.C = dh_t;
        e.ldc = ldh;
        e.accumulate = 1;
        BRC(gemm_nt(ctx, Operand{D.dgates + tn * B * G, B, G, G, 1}, Operand{P->blk_w_rec, C, G, 1, C}, e, net->scratch));
      }
      BlocksBwd f;
      f.dh = dh_t;
      f.act = D.act + t * B * G;
      f.cact = D.cact + t * B * C;
      f.c_prev = (tp >= 0 && tp < T) ? D.cstate + tp * B * C : nullptr;
      f.act_next = s > 0 ? D.act + tn * B * G : nullptr;
      f.dgates_next = s > 0 ? D.dgates + tn * B * G : nullptr;
      f.dc_next = s > 0 ? D.dcstate + tn * B * C : nullptr;
      f.peep = P->blk_peep;
      f.dgates = D.dgates + t * B * G;
      f.dcstate = D.dcstate + t * B * C;
      f.B = B; f.C = C; f.K = K; f.cpb = P->cpb; f.ldh = ldh;
      ctx.begin(TC_RECURRENT);
      lstm_blocks_backward_kernel<<<grid_for(B * K, 128), 128, 0, ctx.stream>>>(f);
      ctx.end(TC_RECURRENT);
    }
  }
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// prev_deriv [T*B, n_in] = sum over directions of dgates [T*B, G] x W_in [G, n_in]; `finish` as in lstm_backward_to_input
int lstm_blocks_backward_to_input(myea_b200_net *net, LayerPlan &L, float *prev_deriv, const LayerPlan &prev, const Epilogue *finish) {
  LstmPlan *P = L.lstm;
  const long long rows = net->T * net->B, G = P->C + 3 * P->K, n_in = P->n_in;
  if (prev.n_out != n_in) return MYEA_E_INVALID;
  for (int d = 0; d < P->dirs; ++d) {
    BRC(gather_weights(net, P, d));
    Epilogue e;
    if (finish != nullptr && d == P->dirs - 1) e = *finish;
    e.C = prev_deriv;
    e.ldc = n_in;
    if (d > 0 && finish != nullptr) { e.addend = prev_deriv; e.ld_addend = n_in; }
    else e.accumulate = d > 0 ? 1 : 0;
    BRC(gemm_nt(net->ctx, Operand{P->d[d].dgates, rows, G, G, 1}, Operand{P->blk_w_in, n_in, G, 1, n_in}, e, net->scratch));
  }
  return MYEA_OK;
}

int lstm_blocks_update_derivative_weight(myea_b200_net *net, LayerPlan &L, const float *input, long long n_in) {
  LstmPlan *P = L.lstm;
  Context &ctx = net->ctx;
  const long long T = net->T, B = net->B, rows = T * B, C = P->C, K = P->K, G = C + 3 * K, ldh = L.n_out;
  const int chunks = static_cast<int>(std::max<long long>(1, std::min<long long>(net->reduce_chunks, rows / 8)));
  for (int d = 0; d < P->dirs; ++d) {
    LstmDir &D = P->d[d];
    {  // dW_in [G, in] = dgates^T x
      Epilogue e;
      e.C = P->blk_dw_in;
      e.ldc = n_in;
      BRC(gemm_nt(ctx, Operand{D.dgates, G, rows, 1, G}, Operand{input, n_in, rows, 1, n_in}, e, net->scratch));
    }
    if (T > 1) {  // dW_rec [G, C]: gate errors of the step after t (in the layer's direction) with the outputs of step t
      const long long Kr = (T - 1) * B;
      const float *dg0 = d == 0 ? D.dgates + B * G : D.dgates;
      const float *h0 = d == 0 ? L.values + d * C : L.values + B * ldh + d * C;
      Epilogue e;
      e.C = P->blk_dw_rec;
      e.ldc = C;
      BRC(gemm_nt(ctx, Operand{dg0, G, Kr, 1, G}, Operand{h0, C, Kr, 1, ldh}, e, net->scratch));
    } else {
      BRC(fill_zero(ctx, P->blk_dw_rec, static_cast<size_t>(G * C)));
    }
    ctx.begin(TC_RECURRENT);
    lstm_blocks_peephole_products_kernel<<<grid_for(rows * C, 256), 256, 0, ctx.stream>>>(D.dgates, D.cstate, rows, C, K, P->cpb, d == 0 ? B : -B,
                                                                                          P->blk_products);
    ctx.end(TC_RECURRENT);
    BRC(column_sum(ctx, P->blk_products, rows, 3 * C, P->blk_dpeep, 0, P->partial, chunks));
    const BlockLayout lay = layout_of(P, d);
    const long long total = G * (n_in + C) + 3 * C;
    ctx.begin(TC_RECURRENT);
    lstm_blocks_weights_kernel<true><<<grid_for(total, 256), 256, 0, ctx.stream>>>(lay, net->grads, P->blk_dw_in, P->blk_dw_rec, P->blk_dpeep);
    ctx.end(TC_RECURRENT);
    // biases: the G columns of the gate errors, summed over all rows, in the order they lie in the parameter buffer
    BRC(column_sum(ctx, D.dgates, rows, G, net->grads + D.b_base, 1, P->partial, chunks));
  }
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

}  // namespace myea
