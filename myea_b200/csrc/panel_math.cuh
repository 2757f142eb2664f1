// Device helpers shared by the contraction kernels and the LSTM cell kernels: the fp32 -> (TF32 hi, bf16 cross) split
// of 8 consecutive K elements and the arithmetic of one LSTM cell step for 8 consecutive cells of one batch row.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"

namespace myea {

__device__ __forceinline__ float round_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
__device__ __forceinline__ uint32_t bf16_bits(float x) { return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(x))); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) { return bf16_bits(a) | (bf16_bits(b) << 16); }

// one group of 8 K elements -> 8 hi floats and the 8 words of the cross group
__device__ __forceinline__ void split_group(const float (&v)[8], int role_b, int raw, float (&hi)[8], uint32_t (&cross)[8]) {
  float lo[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    hi[j] = raw ? v[j] : round_tf32(v[j]);
    lo[j] = v[j] - hi[j];
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t l = raw ? 0u : pack_bf16(lo[2 * j], lo[2 * j + 1]);
    const uint32_t h = raw ? 0u : pack_bf16(hi[2 * j], hi[2 * j + 1]);
    cross[j] = role_b ? h : l;
    cross[4 + j] = role_b ? l : h;
  }
}

__device__ __forceinline__ void load8(float (&d)[8], const float *p) {
  const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
  d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w; d[4] = b.x; d[5] = b.y; d[6] = b.z; d[7] = b.w;
}
__device__ __forceinline__ void store8(float *p, const float (&d)[8]) {
  *reinterpret_cast<float4 *>(p) = make_float4(d[0], d[1], d[2], d[3]);
  *reinterpret_cast<float4 *>(p + 4) = make_float4(d[4], d[5], d[6], d[7]);
}
// 8 consecutive K elements of one operand row written as panels (role A)
__device__ __forceinline__ void store_panel_group(float *hi_row, float *cross_row, const float (&v)[8]) {
  float h[8];
  uint32_t x[8];
  split_group(v, 0, 0, h, x);
  store8(hi_row, h);
  *reinterpret_cast<uint4 *>(cross_row) = make_uint4(x[0], x[1], x[2], x[3]);
  *reinterpret_cast<uint4 *>(cross_row + 4) = make_uint4(x[4], x[5], x[6], x[7]);
}

// One time step of an LSTM layer as the cell arithmetic sees it: the arrays of step t, of the step before / after it in
// the layer's direction, and where the results also leave as operand panels of the next step's contraction.
struct LstmStep {
  long long C = 0, ldh = 0, kp = 0;
  const float *peep = nullptr;  // compact peepholes [3][C]: p_i, p_f, p_o
  float *p_hi = nullptr, *p_cross = nullptr;  // operand panels written for the next step (role A, pitch kp), or null
  // forward (rows of step t unless said otherwise)
  const float *gates_in = nullptr, *c_prev = nullptr, *h_prev = nullptr;
  float *act = nullptr, *cstate = nullptr, *cact = nullptr, *h = nullptr;
  const uint8_t *zone_state = nullptr, *zone_output = nullptr;
  // backward
  float *dh = nullptr;  // [B, ldh] error on h of step t from above; the error through time is added in place
  const float *b_act = nullptr, *b_cact = nullptr, *b_c_prev = nullptr, *act_next = nullptr, *dgates_next = nullptr, *dc_next = nullptr;
  float *dgates = nullptr, *dcstate = nullptr;
  long long Cp = 0;  // K offset of gate g inside the gate-error panel is g * Cp
};

// LSTM forward cell for batch row b, cells [c0, c0 + 8), in two halves so that a caller can issue the loads before it
// waits for the recurrent sums: load8 fetches everything the step needs from memory, finish8 takes the recurrent sums
// (rec[4 * i + g] = gate g of cell c0 + i) and writes the results.  Same arithmetic, in the same order, as
// lstm_cell_forward_kernel (lstm.cu) on a step that has a predecessor.
struct LstmForwardIn {
  float gz[8], gi[8], gf[8], go[8], cp[8], hp[8], pi[8], pf[8], po[8];
  unsigned long long zs, zo;
};
// SELF: also fetch what this same cell wrote in the step before (cell state, output); a caller that still holds those
// values in registers passes false and fills in.cp / in.hp itself.  PEEP: fetch the peepholes.
template <bool SELF = true, bool PEEP = true>
__device__ __forceinline__ void lstm_forward_load8(const LstmStep &p, LstmForwardIn &in, long long b, long long c0) {
  const long long C = p.C;
  const float *g = p.gates_in + b * 4 * C + c0;
  load8(in.gz, g); load8(in.gi, g + C); load8(in.gf, g + 2 * C); load8(in.go, g + 3 * C);
  if (SELF) load8(in.cp, p.c_prev + b * C + c0);
  if (PEEP) { load8(in.pi, p.peep + c0); load8(in.pf, p.peep + C + c0); load8(in.po, p.peep + 2 * C + c0); }
  in.zs = p.zone_state != nullptr ? *reinterpret_cast<const unsigned long long *>(p.zone_state + c0) : ~0ull;
  in.zo = p.zone_output != nullptr ? *reinterpret_cast<const unsigned long long *>(p.zone_output + c0) : ~0ull;
  if (SELF && p.zone_output != nullptr) load8(in.hp, p.h_prev + b * p.ldh + c0);
}
struct LstmForwardOut {
  float z[8], ig[8], fg[8], og[8], cs[8], a[8], h[8];
};
__device__ __forceinline__ void lstm_forward_compute8(const LstmForwardIn &in, const float (&rec)[32], LstmForwardOut &o) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    o.z[i] = tanh_ref(in.gz[i] + rec[4 * i]);
    o.ig[i] = sigmoid_ref(in.gi[i] + (rec[4 * i + 1] + in.pi[i] * in.cp[i]));
    o.fg[i] = sigmoid_ref(in.gf[i] + rec[4 * i + 2] + in.pf[i] * in.cp[i]);
    float c = o.z[i] * o.ig[i];
    c += o.fg[i] * in.cp[i];
    if (((in.zs >> (8 * i)) & 0xFFull) == 0ull) c = in.cp[i];
    o.cs[i] = c;
    o.a[i] = tanh_ref(c);
    o.og[i] = sigmoid_ref(in.go[i] + rec[4 * i + 3] + in.po[i] * c);
    float hh = o.a[i] * o.og[i];
    if (((in.zo >> (8 * i)) & 0xFFull) == 0ull) hh = in.hp[i];
    o.h[i] = hh;
  }
}
// what the NEXT step's contraction reads: h as operand panels
__device__ __forceinline__ void lstm_forward_store_panels8(const LstmStep &p, const LstmForwardOut &o, long long b, long long c0) {
  if (p.p_hi != nullptr) store_panel_group(p.p_hi + b * p.kp + c0, p.p_cross + b * p.kp + c0, o.h);
}
// what the backward pass and the layers above read
__device__ __forceinline__ void lstm_forward_store_arrays8(const LstmStep &p, const LstmForwardOut &o, long long b, long long c0) {
  const long long C = p.C;
  float *act = p.act + b * 4 * C + c0;
  store8(act, o.z); store8(act + C, o.ig); store8(act + 2 * C, o.fg); store8(act + 3 * C, o.og);
  store8(p.cstate + b * C + c0, o.cs);
  store8(p.cact + b * C + c0, o.a);
  store8(p.h + b * p.ldh + c0, o.h);
}
__device__ __forceinline__ void lstm_forward_finish8(const LstmStep &p, const LstmForwardIn &in, const float (&rec)[32], long long b, long long c0) {
  LstmForwardOut o;
  lstm_forward_compute8(in, rec, o);
  lstm_forward_store_arrays8(p, o, b, c0);
  lstm_forward_store_panels8(p, o, b, c0);
}
__device__ __forceinline__ void lstm_forward_cells8(const LstmStep &p, const float (&rec)[32], long long b, long long c0) {
  LstmForwardIn in;
  lstm_forward_load8(p, in, b, c0);
  lstm_forward_finish8(p, in, rec, b, c0);
}

// LSTM backward cell for batch row b, cells [c0, c0 + 8): rec[i] is the error arriving on h of cell c0 + i through time.
// Same arithmetic as lstm_cell_backward_kernel on a step that has a successor; load8 / finish8 as above.
struct LstmBackwardIn {
  float dh[8], z[8], ig[8], fg[8], og[8], a[8], pi[8], pf[8], po[8], cp[8], dni[8], dnf[8], dcn[8], fn[8];
};
// SELF: also fetch what this same cell wrote in the step of the walk before (input / forget gate errors, cell-state
// error); PEEP: fetch the peepholes (see lstm_forward_load8)
template <bool SELF = true, bool PEEP = true>
__device__ __forceinline__ void lstm_backward_load8(const LstmStep &p, LstmBackwardIn &in, long long b, long long c0) {
  const long long C = p.C;
  load8(in.dh, p.dh + b * p.ldh + c0);
  const float *act = p.b_act + b * 4 * C + c0;
  load8(in.z, act); load8(in.ig, act + C); load8(in.fg, act + 2 * C); load8(in.og, act + 3 * C);
  load8(in.a, p.b_cact + b * C + c0);
  if (PEEP) { load8(in.pi, p.peep + c0); load8(in.pf, p.peep + C + c0); load8(in.po, p.peep + 2 * C + c0); }
  if (p.b_c_prev != nullptr) load8(in.cp, p.b_c_prev + b * C + c0);
  if (SELF) {
    const float *dn = p.dgates_next + b * 4 * C + c0;
    load8(in.dni, dn + C); load8(in.dnf, dn + 2 * C);
    load8(in.dcn, p.dc_next + b * C + c0);
  }
  load8(in.fn, p.act_next + b * 4 * C + 2 * C + c0);
}
struct LstmBackwardOut {
  float dh[8], dz[8], di[8], df[8], d_o[8], dc[8];
};
__device__ __forceinline__ void lstm_backward_compute8(const LstmBackwardIn &in, const float (&rec)[8], bool has_prev, LstmBackwardOut &o) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    o.dh[i] = in.dh[i] + rec[i];
    o.d_o[i] = in.og[i] * (1.f - in.og[i]) * (o.dh[i] * in.a[i]);
    float d = o.dh[i] * in.og[i] * (1.f - in.a[i] * in.a[i]);
    d += in.po[i] * o.d_o[i];
    d += in.pi[i] * in.dni[i];
    d += in.pf[i] * in.dnf[i];
    d += in.dcn[i] * in.fn[i];
    o.dc[i] = d;
    o.dz[i] = d * in.ig[i] * (1.f - in.z[i] * in.z[i]);
    o.di[i] = (d * in.z[i]) * (in.ig[i] * (1.f - in.ig[i]));
    o.df[i] = has_prev ? (d * in.cp[i]) * (in.fg[i] * (1.f - in.fg[i])) : 0.f;
  }
}
__device__ __forceinline__ void lstm_backward_store_panels8(const LstmStep &p, const LstmBackwardOut &o, long long b, long long c0) {
  if (p.p_hi != nullptr) {
    float *hi = p.p_hi + b * p.kp + c0, *cr = p.p_cross + b * p.kp + c0;
    store_panel_group(hi, cr, o.dz);
    store_panel_group(hi + p.Cp, cr + p.Cp, o.di);
    store_panel_group(hi + 2 * p.Cp, cr + 2 * p.Cp, o.df);
    store_panel_group(hi + 3 * p.Cp, cr + 3 * p.Cp, o.d_o);
  }
}
__device__ __forceinline__ void lstm_backward_store_arrays8(const LstmStep &p, const LstmBackwardOut &o, long long b, long long c0) {
  const long long C = p.C;
  store8(p.dh + b * p.ldh + c0, o.dh);
  float *dg = p.dgates + b * 4 * C + c0;
  store8(dg, o.dz); store8(dg + C, o.di); store8(dg + 2 * C, o.df); store8(dg + 3 * C, o.d_o);
  store8(p.dcstate + b * C + c0, o.dc);
}
__device__ __forceinline__ void lstm_backward_finish8(const LstmStep &p, const LstmBackwardIn &in, const float (&rec)[8], long long b, long long c0) {
  LstmBackwardOut o;
  lstm_backward_compute8(in, rec, p.b_c_prev != nullptr, o);
  lstm_backward_store_arrays8(p, o, b, c0);
  lstm_backward_store_panels8(p, o, b, c0);
}
__device__ __forceinline__ void lstm_backward_cells8(const LstmStep &p, const float (&rec)[8], long long b, long long c0) {
  LstmBackwardIn in;
  lstm_backward_load8(p, in, b, c0);
  lstm_backward_finish8(p, in, rec, b, c0);
}

}  // namespace myea
