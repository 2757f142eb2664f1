// Dense contractions of the training step on Blackwell tensor cores.
//
//   C[M,N] (+)= A[M,K] * B[N,K]^T        fp32 in, fp32 out
//
// replaces the three scalar triple loops of the reference: Forward_Pass__FC
// (Neural_Network__Forward_Pass__OpenMP.cpp:4517-4557), Backward_Pass__FC (…Backward_Pass__OpenMP.cpp:1044-1082) and
// Update_Derivative_Weight__FC (…Update_Derivative_Weight__OpenMP.cpp:178-216), and the LSTM gate products.
//
// Precision: split fp32 on the tensor cores.  Every fp32 operand x is split into hi = x rounded to TF32 and
// lo = x - hi (exact in fp32); the tensor core accumulates hi*hi (one TF32 instruction per 8 of K) and
// lo*hi + hi*lo (ONE bf16 K = 16 instruction per 8 of K, both terms packed into its K dimension) in fp32 in tensor
// memory; only lo*lo (2^-22 relative) is dropped.  See "Operand panels" below for the packing.
//
// Three kernels share the operand format and the epilogue:
//   gemm3x_tf32_tcgen05_kernel       one CTA, 128 x 128 tile, 192 threads (small M)
//   gemm3x_tf32_tcgen05_pair_kernel  CTA pair (cta_group::2), 256 x 128 tile
//   gemm3x_tf32_tcgen05_wide_kernel  CTA pair, persistent, 256 x 256 tiles, stream-K tail: the one large layers use
// Common structure:
//   warp 0   : TMA producer - cp.async.bulk.tensor 2D loads of the four K-major panels (A hi, A cross, B hi, B cross),
//              128-byte swizzle, 32 floats of K per stage, completing on a per-stage "full" mbarrier
//   warp 1   : allocates tensor memory; one elected lane issues the tcgen05.mma pairs, tcgen05.commit releases the
//              stage ("empty" mbarrier) and signals finished accumulators
//   others   : read accumulators with tcgen05.ld (each warp its own 32-lane quarter: the thread owns an output row),
//              fused bias / accumulate / skip-connection addend / activation derivative, float4 stores
// Every mbarrier wait is bounded (about one second of SM clock); a wait that runs out sets the handle's error flag
// and the CTA frees its tensor memory and returns.
//
// The FP32 FMA kernel at the end of the file is the second engine (exact fp32 products; selectable for debugging).
#include "common.cuh"
#include "panel_math.cuh"
#include "tcgen05.cuh"

#include <cudaTypedefs.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <mutex>

namespace myea {

struct GemmDims {
  int M, N, K;
};

// epilogue math for one element
// offset of output row m from e.C: plain pitch, or one of up to four row segments that start at their own offsets
__device__ __forceinline__ long long c_row(const Epilogue &e, long long m) {
  if (e.seg_rows == 0) return m * e.ldc;
  const int s = static_cast<int>(m >= e.seg_rows) + static_cast<int>(m >= 2 * e.seg_rows) + static_cast<int>(m >= 3 * e.seg_rows);
  return (m - s * e.seg_rows) * e.ldc + e.seg_off[s];
}

__device__ __forceinline__ float epilogue_value(const Epilogue &e, float acc, long long m, long long n) {
  float v = acc;
  if (e.bias != nullptr) v += e.bias[n];
  if (e.addend != nullptr) v += e.addend[m * e.ld_addend + n];
  if (e.deriv_af != 0u) {
    float pre = 0.f, y = 0.f;
    if (e.aux_pre != nullptr) {
      pre = e.aux_pre[m * e.ld_aux + n];
      if (e.col_scale != nullptr) pre = pre * e.col_scale[n] + e.col_shift[n];
    }
    if (e.aux_y != nullptr) y = e.aux_y[m * e.ld_aux + n];
    v *= af_derive(e.deriv_af, pre, y);
  }
  if (e.accumulate) v += e.C[c_row(e, m) + n];
  return v;
}

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }

// The vector path of the epilogue needs 16-byte aligned bases and pitches that are multiples of four floats.
__device__ __forceinline__ bool epilogue_vector_ok(const Epilogue &e) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(e.C) | reinterpret_cast<uintptr_t>(e.bias) | reinterpret_cast<uintptr_t>(e.addend) |
                         reinterpret_cast<uintptr_t>(e.aux_pre) | reinterpret_cast<uintptr_t>(e.aux_y) |
                         reinterpret_cast<uintptr_t>(e.col_scale) | reinterpret_cast<uintptr_t>(e.col_shift);
  return (bits & 15) == 0 && ((e.ldc | e.ld_addend | e.ld_aux | e.seg_off[0] | e.seg_off[1] | e.seg_off[2] | e.seg_off[3]) & 3) == 0;
}
// 0 plain (bias only), 1 activation derivative, 2 accumulate, 3 anything else
__device__ __forceinline__ int epilogue_mode(const Epilogue &e) {
  if (e.addend != nullptr) return 3;
  if (e.deriv_af != 0u) return e.accumulate ? 3 : 1;
  return e.accumulate ? 2 : 0;
}

// Epilogue of a 32-row x 32-column block, warp-collective: lane l holds row row0 + l (that is how tensor memory hands an
// accumulator to a warp), but global memory wants rows of 128 contiguous bytes.  The block goes through a 16 x 36
// float staging buffer in shared memory, half at a time: the owning lanes write their rows as float4 (conflict-free at
// pitch 36), then every lane takes one float4 column slot (lane % 8) of the rows lane / 8 + 4 i, so that each global
// instruction of the warp covers four full 128-byte row segments.  The loads of the four rows are issued before their
// first use.  ADD / DERIV / ACC say what MAY be present.  `tr`: this warp's 16 * 36 floats.
constexpr int TR_PITCH = 36;
constexpr int TR_WARP_FLOATS = 16 * TR_PITCH;

// x[i] *= f'(z[i], y[i]) for four float4; the activation is the same for the whole launch, so the switch is taken once
// per call and every case is straight-line code (a switch per element made this epilogue as long as a whole tile's
// main loop)
template <uint32_t AF>
__device__ __forceinline__ void derive4x4(float4 (&x)[4], const float4 (&z)[4], const float4 (&y)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[i].x *= af_derive(AF, z[i].x, y[i].x);
    x[i].y *= af_derive(AF, z[i].y, y[i].y);
    x[i].z *= af_derive(AF, z[i].z, y[i].z);
    x[i].w *= af_derive(AF, z[i].w, y[i].w);
  }
}
__device__ __forceinline__ void derive4x4_any(uint32_t af, float4 (&x)[4], const float4 (&z)[4], const float4 (&y)[4]) {
  switch (af) {
    case MYEA_AF_TANH: derive4x4<MYEA_AF_TANH>(x, z, y); break;
    case MYEA_AF_SIGMOID: derive4x4<MYEA_AF_SIGMOID>(x, z, y); break;
    case MYEA_AF_RELU: derive4x4<MYEA_AF_RELU>(x, z, y); break;
    case MYEA_AF_LEAKY_RELU: derive4x4<MYEA_AF_LEAKY_RELU>(x, z, y); break;
    case MYEA_AF_ELU: derive4x4<MYEA_AF_ELU>(x, z, y); break;
    case MYEA_AF_SELU: derive4x4<MYEA_AF_SELU>(x, z, y); break;
    case MYEA_AF_LINEAR: case MYEA_AF_LINEAR_PIECE: case MYEA_AF_LINEAR_PIECE_SYMMETRIC: case MYEA_AF_SOFTMAX: break;  // derivative 1
    default:  // the rarely used functions share one body that switches per element
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[i].x *= af_derive(af, z[i].x, y[i].x);
        x[i].y *= af_derive(af, z[i].y, y[i].y);
        x[i].z *= af_derive(af, z[i].z, y[i].z);
        x[i].w *= af_derive(af, z[i].w, y[i].w);
      }
      break;
  }
}

template <bool ADD, bool DERIV, bool ACC, int STATS = 0>
__device__ __forceinline__ void epilogue_block32(const Epilogue &e, float *tr, const float (&v)[32], int lane, long long row0, long long col0, int M) {
  const int c4 = (lane & 7) * 4, rsub = lane >> 3;
  const long long n = col0 + c4;
  const bool has_add = ADD && e.addend != nullptr, has_pre = DERIV && e.aux_pre != nullptr, has_y = DERIV && e.aux_y != nullptr;
  const bool affine = has_pre && e.col_scale != nullptr;
  const bool acc = ACC && e.accumulate;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 bias = e.bias != nullptr ? ld4(e.bias + n) : zero;
  const float4 cs = affine ? ld4(e.col_scale + n) : make_float4(1.f, 1.f, 1.f, 1.f), ch = affine ? ld4(e.col_shift + n) : zero;
  // The global reads of BOTH halves go out before anything else (one memory round trip per block instead of two);
  // the variant that may read all four arrays keeps to one half at a time for the sake of registers.
  constexpr bool AHEAD = !(ADD && DERIV && ACC);
  constexpr int SLOTS = AHEAD ? 8 : 4;
  float4 add[ADD ? SLOTS : 1], pre[DERIV ? SLOTS : 1], y[DERIV ? SLOTS : 1], old[ACC ? SLOTS : 1];
  auto load_rows = [&](int first_slot, int h0, int h1) {
#pragma unroll
    for (int h = h0; h < h1; ++h) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int s = first_slot + (h - h0) * 4 + i;
        const long long m = row0 + h * 16 + rsub + 4 * i;
        const bool in = m < M;
        if (ADD) add[s] = (has_add && in) ? ld4(e.addend + m * e.ld_addend + n) : zero;
        if (DERIV) {
          pre[s] = (has_pre && in) ? ld4(e.aux_pre + m * e.ld_aux + n) : zero;
          y[s] = (has_y && in) ? ld4(e.aux_y + m * e.ld_aux + n) : zero;
        }
        if (ACC) old[s] = (acc && in) ? ld4(e.C + c_row(e, m) + n) : zero;
      }
    }
  };
  // column statistics of this 32 x 32 block: this lane's four columns over its eight rows first
  float4 st0 = zero, st1 = zero;
  const float4 mu = (STATS == 2 && e.col_mean != nullptr) ? ld4(e.col_mean + n) : zero;
  if (AHEAD) load_rows(0, 0, 2);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!AHEAD) load_rows(0, h, h + 1);
    const int s0 = AHEAD ? h * 4 : 0;
    __syncwarp();
    if ((lane >> 4) == h) {
      float *dst = tr + (lane & 15) * TR_PITCH;
#pragma unroll
      for (int j = 0; j < 8; ++j) *reinterpret_cast<float4 *>(dst + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    __syncwarp();
    float4 x[4], z4[4], y4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[i] = *reinterpret_cast<const float4 *>(tr + (rsub + 4 * i) * TR_PITCH + c4);
      x[i].x += bias.x; x[i].y += bias.y; x[i].z += bias.z; x[i].w += bias.w;
      if (ADD) { x[i].x += add[s0 + i].x; x[i].y += add[s0 + i].y; x[i].z += add[s0 + i].z; x[i].w += add[s0 + i].w; }
      if (DERIV) {
        const float4 p = pre[s0 + i];
        z4[i] = make_float4(p.x * cs.x + ch.x, p.y * cs.y + ch.y, p.z * cs.z + ch.z, p.w * cs.w + ch.w);
        y4[i] = y[s0 + i];
      }
    }
    if (DERIV) derive4x4_any(e.deriv_af, x, z4, y4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long m = row0 + h * 16 + rsub + 4 * i;
      if (ACC) { x[i].x += old[s0 + i].x; x[i].y += old[s0 + i].y; x[i].z += old[s0 + i].z; x[i].w += old[s0 + i].w; }
      if (m < M) {
        *reinterpret_cast<float4 *>(e.C + c_row(e, m) + n) = x[i];
        if (STATS == 1) {
          st0.x += x[i].x; st0.y += x[i].y; st0.z += x[i].z; st0.w += x[i].w;
          st1.x = fmaf(x[i].x, x[i].x, st1.x); st1.y = fmaf(x[i].y, x[i].y, st1.y); st1.z = fmaf(x[i].z, x[i].z, st1.z); st1.w = fmaf(x[i].w, x[i].w, st1.w);
        }
        if (STATS == 2) {
          const float4 p = pre[s0 + i];  // the raw array the derivative was taken on (before the folded normalization)
          st0.x += x[i].x; st0.y += x[i].y; st0.z += x[i].z; st0.w += x[i].w;
          st1.x = fmaf(x[i].x, p.x - mu.x, st1.x); st1.y = fmaf(x[i].y, p.y - mu.y, st1.y); st1.z = fmaf(x[i].z, p.z - mu.z, st1.z); st1.w = fmaf(x[i].w, p.w - mu.w, st1.w);
        }
      }
    }
  }
  if (STATS != 0) {
    // the four lanes that share a column slot (lane, lane ^ 8, lane ^ 16, lane ^ 24) hold the block's 32 rows between them
#pragma unroll
    for (int o = 8; o <= 16; o <<= 1) {
      st0.x += __shfl_xor_sync(0xffffffffu, st0.x, o); st0.y += __shfl_xor_sync(0xffffffffu, st0.y, o);
      st0.z += __shfl_xor_sync(0xffffffffu, st0.z, o); st0.w += __shfl_xor_sync(0xffffffffu, st0.w, o);
      st1.x += __shfl_xor_sync(0xffffffffu, st1.x, o); st1.y += __shfl_xor_sync(0xffffffffu, st1.y, o);
      st1.z += __shfl_xor_sync(0xffffffffu, st1.z, o); st1.w += __shfl_xor_sync(0xffffffffu, st1.w, o);
    }
    const long long blk = row0 >> 5;
    if (lane < 8 && blk < e.stats_blocks) {
      float *dst = e.col_stats + blk * e.ldc + n;   // [block][N]: the result's pitch is N for the arrays that ask for this
      *reinterpret_cast<float4 *>(dst) = st0;
      *reinterpret_cast<float4 *>(dst + e.stats_blocks * e.ldc) = st1;
    }
  }
}

// The same block for arrays the vector path cannot take (bases or pitches that are not multiples of 16 bytes: the weight
// derivatives of LSTM layers land inside the reference's per-block parameter layout, whose row pitch is odd) and for the
// ragged right edge: staged through the same buffer, then lane l takes column col0 + l of one row after the other, so a
// warp's accesses still cover one contiguous row segment each.
__device__ __forceinline__ void epilogue_block32_rows(const Epilogue &e, float *tr, const float (&v)[32], int lane, long long row0, long long col0, int M, int N) {
  const long long n = col0 + lane;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    __syncwarp();
    if ((lane >> 4) == h) {
      float *dst = tr + (lane & 15) * TR_PITCH;
#pragma unroll
      for (int j = 0; j < 8; ++j) *reinterpret_cast<float4 *>(dst + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    __syncwarp();
    if (e.accumulate && e.bias == nullptr && e.addend == nullptr && e.deriv_af == 0u) {
      // C += product and nothing else (weight derivatives): the 16 old row segments are requested together - one after
      // the other, their latency (rows of an LSTM layer's weight derivatives lie a whole block apart) is what the
      // epilogue of a tile takes
      float old[16];
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const long long m = row0 + h * 16 + r;
        old[r] = (m < M && n < N) ? e.C[c_row(e, m) + n] : 0.f;
      }
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const long long m = row0 + h * 16 + r;
        if (m < M && n < N) e.C[c_row(e, m) + n] = tr[r * TR_PITCH + lane] + old[r];
      }
    } else {
#pragma unroll 4
      for (int r = 0; r < 16; ++r) {
        const long long m = row0 + h * 16 + r;
        if (m < M && n < N) e.C[c_row(e, m) + n] = epilogue_value(e, tr[r * TR_PITCH + lane], m, n);
      }
    }
  }
}

// Warp-collective: every lane of the warp calls it (row0, col0, M, N are the same for all of them).
__device__ __forceinline__ void epilogue_row32(const Epilogue &e, const float (&v)[32], long long row0, int lane, long long col0, int M, int N,
                                               bool vec_ok, int mode, float *tr) {
  if (col0 >= N) return;
  if (vec_ok && col0 + 32 <= N) {
    switch (mode) {
      case 0:
        if (e.stats_kind == 1) epilogue_block32<false, false, false, 1>(e, tr, v, lane, row0, col0, M);
        else epilogue_block32<false, false, false>(e, tr, v, lane, row0, col0, M);
        break;
      case 1:
        if (e.stats_kind == 2) epilogue_block32<false, true, false, 2>(e, tr, v, lane, row0, col0, M);
        else epilogue_block32<false, true, false>(e, tr, v, lane, row0, col0, M);
        break;
      case 2: epilogue_block32<false, false, true>(e, tr, v, lane, row0, col0, M); break;
      default: epilogue_block32<true, true, true>(e, tr, v, lane, row0, col0, M); break;
    }
  } else {
    epilogue_block32_rows(e, tr, v, lane, row0, col0, M, N);
  }
}

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + slack to align the base to 1024 bytes
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm3x_tf32_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
                           const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
                           const GemmDims dims, const Epilogue epi, int *error_flag) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + S::BAR_OFFSET);
  uint64_t *empty_bar = full_bar + STAGES;
  uint64_t *tmem_full_bar = empty_bar + STAGES;
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(tmem_full_bar + 1);

  // Accumulators in tensor memory (BN fp32 columns each): N_MAIN rotating ones for hi*hi and one for the two
  // cross terms.  The tensor core truncates when it adds into an accumulator, an error of up to one ulp of the
  // ACCUMULATOR per tcgen05.mma whatever the size of the addend; keeping the small terms apart and spreading the
  // dominant products over several accumulators cuts the number of truncating adds per accumulator (12 per stage
  // down to 4/N_MAIN) and with it the error of a long-K sum.  The epilogue adds them in fp32, round to nearest.
  constexpr int N_MAIN = (BN == 128) ? 3 : 1;
  constexpr int TMEM_COLS = 512;
  static_assert((N_MAIN + 1) * BN <= TMEM_COLS, "accumulators exceed tensor memory");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM;
  const int n0 = blockIdx.x * BN;
  const int num_kb = (dims.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    ptx::mbar_init(tmem_full_bar, 1);
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_holder, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  grid_dependency_wait();     // everything above touched no global memory
  grid_dependency_release();

  bool ok = true;
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = static_cast<uint32_t>(kb / STAGES) & 1u;
        if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u)) { ok = false; break; }
        uint8_t *st = smem + s * S::STAGE_BYTES;
        ptx::mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
        ptx::tma_load_2d(st, &tm_a_hi, &full_bar[s], kb * BK, m0);
        ptx::tma_load_2d(st + S::A_BYTES, &tm_a_lo, &full_bar[s], kb * BK, m0);
        ptx::tma_load_2d(st + 2 * S::A_BYTES, &tm_b_hi, &full_bar[s], kb * BK, n0);
        ptx::tma_load_2d(st + 2 * S::A_BYTES + S::B_BYTES, &tm_b_lo, &full_bar[s], kb * BK, n0);
      }
      if (!ok) atomicCAS(error_flag, 0, 101);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_tf32(BM, BN);
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = static_cast<uint32_t>(kb / STAGES) & 1u;
        if (!ptx::mbar_wait(&full_bar[s], ph)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t st = ptx::smem_u32(smem + s * S::STAGE_BYTES);
        const uint64_t a_hi = make_smem_desc(st);
        const uint64_t a_lo = make_smem_desc(st + S::A_BYTES);
        const uint64_t b_hi = make_smem_desc(st + 2 * S::A_BYTES);
        const uint64_t b_lo = make_smem_desc(st + 2 * S::A_BYTES + S::B_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t koff = static_cast<uint64_t>((k * UMMA_K * 4) >> 4);  // 32 bytes per K step, in 16-byte units
          const int step = kb * (BK / UMMA_K) + k;
          const int main_acc = step % N_MAIN;
          const uint32_t t_small = tmem_base + static_cast<uint32_t>(N_MAIN * BN);
          ptx::mma_bf16(t_small, a_lo + koff, b_lo + koff, make_idesc_bf16(BM, BN), step > 0 ? 1u : 0u);  // both cross terms
          ptx::mma_tf32(tmem_base + static_cast<uint32_t>(main_acc * BN), a_hi + koff, b_hi + koff, idesc,
                        step >= N_MAIN ? 1u : 0u);
        }
        ptx::tc_commit(&empty_bar[s]);  // the stage may be refilled once these MMAs have read it
      }
      ptx::tc_commit(tmem_full_bar);  // accumulator complete
      if (!ok) atomicCAS(error_flag, 0, 102);
    }
  } else {
    // ---------------- epilogue: warps 2..5, tensor-memory lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    if (!ptx::mbar_wait(tmem_full_bar, 0)) {
      ok = false;
      if (lane == 0) atomicCAS(error_flag, 0, 103);
    }
    ptx::tc_fence_after();
    if (ok && num_kb > 0) {
      const long long row_base = static_cast<long long>(m0) + q * 32;
      const bool vec_ok = epilogue_vector_ok(epi);
      const int mode = epilogue_mode(epi);
      // every MMA has completed, so the pipeline stages are free: the first bytes serve as the staging buffers
      float *tr = reinterpret_cast<float *>(smem) + (warp - 2) * TR_WARP_FLOATS;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        if (n0 + c >= dims.N) break;
        uint32_t r[32];
        float sum[32];
        const uint32_t t_chunk = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c);
        ptx::tmem_ld_32x32(t_chunk + static_cast<uint32_t>(N_MAIN * BN), r);  // cross terms first
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[j] = __uint_as_float(r[j]);
#pragma unroll
        for (int a = 0; a < N_MAIN; ++a) {
          ptx::tmem_ld_32x32(t_chunk + static_cast<uint32_t>(a * BN), r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[j] += __uint_as_float(r[j]);
        }
        epilogue_row32(epi, sum, row_base, lane, static_cast<long long>(n0) + c, dims.M, dims.N, vec_ok, mode, tr);
      }
    }
  }

  // drain: the producer makes sure none of its copies is still in flight before the CTA's shared memory goes away
  if (warp == 0 && lane == 0) {
    const int first = num_kb > STAGES ? num_kb - STAGES : 0;
    for (int kb = first; kb < num_kb; ++kb) {
      const int s = kb % STAGES;
      const uint32_t ph = static_cast<uint32_t>(kb / STAGES) & 1u;
      if (!ptx::mbar_wait(&full_bar[s], ph)) break;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster (two SMs) compute one 256 x 128 output tile with tcgen05.mma.cta_group::2
// (M = 256, N = 128, K = 8).  Each CTA stages only ITS 128 rows of A and ITS 64 rows of B (hi and lo: 48 KB per
// stage, 4 stages) and the tensor cores of the pair exchange the B halves themselves, so every SM writes 25 % fewer
// bytes into shared memory per product and the tensor core reads 6 KB instead of 8 KB of it per MMA: the 128 x 128
// single-CTA tile is bounded by shared-memory bandwidth at about 60 % of the tensor peak, this shape at about 80 %.
// The leader CTA (cluster rank 0) issues every MMA; completion bytes of both CTAs' TMA loads are counted on the
// leader's "full" barrier; tcgen05.commit multicasts the "empty" / "accumulator ready" arrivals to both CTAs.  Each CTA
// owns the accumulator rows of its half (tensor memory lanes 0-127, the same four 128-column accumulators) and runs
// its own epilogue.  No TMA multicast is used.
// ---------------------------------------------------------------------------------------------------------
constexpr int PAIR_STAGES = 4;
struct PairSmem {
  static constexpr int A_BYTES = BM * BK * 4;        // 128 rows
  static constexpr int B_BYTES = 64 * BK * 4;        // this CTA's half of the 128-row B tile
  static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  static constexpr int BAR_OFFSET = PAIR_STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm3x_tf32_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
                                const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
                                const GemmDims dims, const Epilogue epi, int *error_flag) {
  using S = PairSmem;
  constexpr int BN = 128, N_MAIN = 3, TMEM_COLS = 512, STAGES = PAIR_STAGES;
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared-memory window starts at the same offset in both CTAs, so aligned offsets match as well
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + S::BAR_OFFSET);
  uint64_t *empty_bar = full_bar + STAGES;
  uint64_t *tmem_full_bar = empty_bar + STAGES;
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(tmem_full_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = ptx::cluster_ctarank();  // 0 = leader
  const int m0 = (blockIdx.x >> 1) * 256 + static_cast<int>(cta_rank) * BM;  // this CTA's 128 rows (the pair sits along grid x)
  const int n0 = blockIdx.y * BN;
  const int nb0 = n0 + static_cast<int>(cta_rank) * 64;                       // this CTA's 64 rows of B
  const int num_kb = (dims.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);   // leader: its own arrive.expect_tx (bytes of both CTAs)
      ptx::mbar_init(&empty_bar[s], 1);  // one multicast commit
    }
    ptx::mbar_init(tmem_full_bar, 1);
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_holder, TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  bool ok = true;
  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = static_cast<uint32_t>(kb / STAGES) & 1u;
        if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u)) { ok = false; break; }
        uint8_t *st = smem + s * S::STAGE_BYTES;
        if (cta_rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * S::STAGE_BYTES);
        ptx::tma_load_2d_pair(st, &tm_a_hi, &full_bar[s], kb * BK, m0);
        ptx::tma_load_2d_pair(st + S::A_BYTES, &tm_a_lo, &full_bar[s], kb * BK, m0);
        ptx::tma_load_2d_pair(st + 2 * S::A_BYTES, &tm_b_hi, &full_bar[s], kb * BK, nb0);
        ptx::tma_load_2d_pair(st + 2 * S::A_BYTES + S::B_BYTES, &tm_b_lo, &full_bar[s], kb * BK, nb0);
      }
      if (!ok) atomicCAS(error_flag, 0, 201);
    }
  } else if (warp == 1) {
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_tf32(256, BN);
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = static_cast<uint32_t>(kb / STAGES) & 1u;
        if (!ptx::mbar_wait(&full_bar[s], ph)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t st = ptx::smem_u32(smem + s * S::STAGE_BYTES);
        const uint64_t a_hi = make_smem_desc(st);
        const uint64_t a_lo = make_smem_desc(st + S::A_BYTES);
        const uint64_t b_hi = make_smem_desc(st + 2 * S::A_BYTES);
        const uint64_t b_lo = make_smem_desc(st + 2 * S::A_BYTES + S::B_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t koff = static_cast<uint64_t>((k * UMMA_K * 4) >> 4);
          const int step = kb * (BK / UMMA_K) + k;
          const int main_acc = step % N_MAIN;
          const uint32_t t_small = tmem_base + static_cast<uint32_t>(N_MAIN * BN);
          ptx::mma_bf16_pair(t_small, a_lo + koff, b_lo + koff, make_idesc_bf16(256, BN), step > 0 ? 1u : 0u);  // both cross terms
          ptx::mma_tf32_pair(tmem_base + static_cast<uint32_t>(main_acc * BN), a_hi + koff, b_hi + koff, idesc, step >= N_MAIN ? 1u : 0u);
        }
        ptx::tc_commit_pair(&empty_bar[s]);
      }
      ptx::tc_commit_pair(tmem_full_bar);
      if (!ok) atomicCAS(error_flag, 0, 202);
    }
  } else {
    const int q = warp & 3;
    if (!ptx::mbar_wait(tmem_full_bar, 0)) {
      ok = false;
      if (lane == 0) atomicCAS(error_flag, 0, 203);
    }
    ptx::tc_fence_after();
    if (ok && num_kb > 0) {
      const long long row_base = static_cast<long long>(m0) + q * 32;
      const bool vec_ok = epilogue_vector_ok(epi);
      const int mode = epilogue_mode(epi);
      // every MMA has completed, so the pipeline stages are free: the first bytes serve as the staging buffers
      float *tr = reinterpret_cast<float *>(smem) + (warp - 2) * TR_WARP_FLOATS;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        if (n0 + c >= dims.N) break;
        uint32_t r[32];
        float sum[32];
        const uint32_t t_chunk = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c);
        ptx::tmem_ld_32x32(t_chunk + static_cast<uint32_t>(N_MAIN * BN), r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[j] = __uint_as_float(r[j]);
#pragma unroll
        for (int a = 0; a < N_MAIN; ++a) {
          ptx::tmem_ld_32x32(t_chunk + static_cast<uint32_t>(a * BN), r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[j] += __uint_as_float(r[j]);
        }
        epilogue_row32(epi, sum, row_base, lane, static_cast<long long>(n0) + c, dims.M, dims.N, vec_ok, mode, tr);
      }
    }
  }
  // the accumulator-ready arrival is the last thing the leader sends; once both CTAs have seen it (or given up) nobody
  // touches the peer's shared memory or barriers any more
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Operand preparation: fp32 matrix (either stride order) -> K-major hi / lo panels [rows][kp]
// ---------------------------------------------------------------------------------------------------------
// Wide CTA-pair variant, persistent: two SMs compute 256 x 256 output tiles (each CTA 128 rows x 256 columns) with
// tcgen05.mma.cta_group::2 (M = 256, N = 256).  Per 32 floats of K each CTA stages 64 KB (its 128 rows of A and its
// 128 rows of B, hi and cross panels; 3 stages) for 128 x 256 x 32 products: half the shared-memory and L2 traffic per
// product of the 128 x 128 tile, every MMA instruction carries twice the work, and the main loop runs at the tensor
// pipe's own pace (the 128 x 128 tile is held back by shared-memory reads: about 100 instead of 64 cycles per MMA).
// Tensor memory holds two 256-column accumulators, used as a ping-pong pair: all MMAs of one K chunk
// (WIDE_KC stages = 256 of K, 64 instructions) go into one buffer while the eight drain warps read the other into
// fp32 registers and add it, round to nearest, to the running sum.  A chain of truncating tensor-core adds is therefore
// never longer than 64 instructions, whatever K is (the 4-accumulator layout of the narrower kernels bounds it by K/24).
// The grid is one cluster per SM pair; each cluster walks tiles cluster, cluster + clusters, ... and the three roles
// (TMA producer, MMA issuer, drain warps) keep running stage / chunk counters across tiles, so the loads and MMAs of
// the next tile start while the drain warps, which hold the finished tile in registers, run its epilogue.
// 384 threads in three warpgroups: the role warps give registers back (setmaxnreg) and the eight drain warps take 232.
// Tiles are numbered in bands of 8 row tiles so that the tiles in flight at one time share operand panels in L2.
// ---------------------------------------------------------------------------------------------------------
constexpr int WIDE_STAGES = 3;
// Three warpgroups: warps 0-3 hold the two single-thread roles (warp 0 TMA, warp 1 MMA + tensor-memory allocation;
// warps 2-3 idle) and give most of their registers away; warps 4-11 drain and run the epilogue with 232 registers each
// (setmaxnreg), which is what keeps the 128-float running sum and the epilogue's loads out of local memory.
constexpr int WIDE_THREADS = 384;
constexpr int WIDE_DRAIN_WARP0 = 4;
constexpr int WIDE_KC = 8;
constexpr int WIDE_BAND = 8;
struct WideSmem {
  static constexpr int TILE_BYTES = 128 * BK * 4;           // 128 rows x 128 bytes
  static constexpr int STAGE_BYTES = 4 * TILE_BYTES;        // A hi, A cross, B hi, B cross
  static constexpr int BAR_OFFSET = WIDE_STAGES * STAGE_BYTES;
  static constexpr int TR_OFFSET = BAR_OFFSET + 512;        // epilogue staging: 8 warps x 16 x 36 floats (the stages stay busy)
  static constexpr int TOTAL = TR_OFFSET + 8 * TR_WARP_FLOATS * 4 + 1024;
};

// Work list of the wide kernel.  Tiles [0, dp_tiles) are computed whole, round-robin over the clusters.  The K chunks
// of the remaining tiles (the partial last wave, or every tile of a contraction with fewer tiles than clusters) form
// one sequence of sk_units chunks that is cut into equal runs of sk_chunks, one run per cluster ("stream-K"), so that
// the tail of the work list is spread over all SM pairs instead of leaving most of them idle.
struct WideWork {
  int tiles_m, tiles_n, num_tiles;
  int dp_tiles;
  int sk_chunks;           // chunks per cluster of the split part (0: nothing is split)
  int sk_units;            // (num_tiles - dp_tiles) * chunks per tile
  float *ws;               // partial sums of split tiles: [cluster][2][16 warp regions][32 float4 columns][32 lanes]
  unsigned int *counters;  // [split tile][16 warp regions] arrivals; the last arrival adds the partials up and resets it
};
constexpr int WIDE_REGION_FLOATS = 32 * 128;  // one drain warp's share of a tile: 32 rows x 128 columns

__device__ __forceinline__ void wide_tile_coords(const WideWork &w, int t, int &tm, int &tn) {
  const int per_band = WIDE_BAND * w.tiles_n;
  const int band = t / per_band;
  const int within = t - band * per_band;
  const int rows = min(WIDE_BAND, w.tiles_m - band * WIDE_BAND);
  tn = within / rows;
  tm = band * WIDE_BAND + (within - tn * rows);
}

// The segments (tile, chunk range) of one cluster, in the order every role of the kernel walks them.
struct WideSegments {
  int next_tile, stride, dp_tiles, num_chunks, u, u_end;
  int tile, c0, c1;  // the current segment
  __device__ __forceinline__ WideSegments(const WideWork &w, int cluster, int clusters, int chunks_per_tile)
      : next_tile(cluster), stride(clusters), dp_tiles(w.dp_tiles), num_chunks(chunks_per_tile) {
    u = min(cluster * w.sk_chunks, w.sk_units);
    u_end = min(u + w.sk_chunks, w.sk_units);
  }
  __device__ __forceinline__ bool next() {
    if (next_tile < dp_tiles) {
      tile = next_tile; c0 = 0; c1 = num_chunks;
      next_tile += stride;
      return true;
    }
    if (u < u_end) {
      const int ts = u / num_chunks;
      c0 = u - ts * num_chunks;
      if (c0 + (u_end - u) > num_chunks) {
        // The run crosses into the next tile (a run is shorter than a tile, so it touches two at most): the head of
        // the next tile goes first and the end of this tile after it.  Every cluster then walks K upwards from chunk 0
        // at the same time as the clusters on the neighbouring tiles, which read the same operand panels, and the
        // panels are fetched from DRAM once instead of once per tile.
        tile = dp_tiles + ts + 1;
        c0 = 0;
        c1 = u_end - (ts + 1) * num_chunks;
        u_end = (ts + 1) * num_chunks;
        return true;
      }
      c1 = min(num_chunks, c0 + (u_end - u));
      tile = dp_tiles + ts;
      u += c1 - c0;
      return true;
    }
    return false;
  }
};

// one operand's 128 rows of one stage: a K-major panel is one 2-D box per panel (32 floats of K x 128 rows), an
// MN-major panel one 3-D box (hi: 32 floats x 32 K rows x 4 chunks; cross: 64 bf16 x 64 K rows x 2 chunks)
template <bool MN>
__device__ __forceinline__ void wide_load_operand(uint8_t *dst_hi, uint8_t *dst_x, const CUtensorMap *m_hi, const CUtensorMap *m_x,
                                                  uint64_t *bar, int kb, int row0) {
  if (!MN) {
    ptx::tma_load_2d_pair(dst_hi, m_hi, bar, kb * BK, row0);
    ptx::tma_load_2d_pair(dst_x, m_x, bar, kb * BK, row0);
  } else {
    ptx::tma_load_3d_pair(dst_hi, m_hi, bar, 0, kb * BK, row0 >> 5);
    ptx::tma_load_3d_pair(dst_x, m_x, bar, 0, kb * 2 * BK, row0 >> 6);
  }
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(WIDE_THREADS, 1)
gemm3x_tf32_tcgen05_wide_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
                                const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
                                const GemmDims dims, const WideWork work, const Epilogue epi, int *error_flag) {
  using S = WideSmem;
  constexpr int STAGES = WIDE_STAGES, BN = 256, TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + S::BAR_OFFSET);
  uint64_t *empty_bar = full_bar + STAGES;
  uint64_t *acc_full_bar = empty_bar + STAGES;   // [2] a buffer holds a finished K chunk (multicast to both CTAs)
  uint64_t *acc_empty_bar = acc_full_bar + 2;    // [2] leader only: every drain warp of both CTAs has read the buffer
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(acc_empty_bar + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = ptx::cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  const int num_kb = (dims.K + BK - 1) / BK;
  const int num_chunks = (num_kb + WIDE_KC - 1) / WIDE_KC;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full_bar[b], 1);
      ptx::mbar_init(&acc_empty_bar[b], 16);  // one arrival per drain warp of the pair
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_holder, TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  grid_dependency_wait();     // everything above touched no global memory
  grid_dependency_release();

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    ptx::reg_release<40>();
    if (lane == 0) {
      bool ok = true;
      uint32_t it = 0;  // k-blocks staged so far, over all segments
      WideSegments seg(work, cluster_id, num_clusters, num_chunks);
      while (ok && seg.next()) {
        int tm, tn;
        wide_tile_coords(work, seg.tile, tm, tn);
        const int m0 = tm * 256 + static_cast<int>(cta_rank) * 128;
        const int nb0 = tn * BN + static_cast<int>(cta_rank) * 128;
        const int kb_end = min(num_kb, seg.c1 * WIDE_KC);
        for (int kb = seg.c0 * WIDE_KC; kb < kb_end; ++kb, ++it) {
          const int s = static_cast<int>(it % STAGES);
          const uint32_t ph = (it / STAGES) & 1u;
          if (!ptx::mbar_wait_or_abort(&empty_bar[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t *st = smem + s * S::STAGE_BYTES;
          if (cta_rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * S::STAGE_BYTES);
          wide_load_operand<A_MN>(st, st + S::TILE_BYTES, &tm_a_hi, &tm_a_lo, &full_bar[s], kb, m0);
          wide_load_operand<B_MN>(st + 2 * S::TILE_BYTES, st + 3 * S::TILE_BYTES, &tm_b_hi, &tm_b_lo, &full_bar[s], kb, nb0);
        }
      }
      if (!ok) atomicCAS(error_flag, 0, 301);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA) ----------------
    ptx::reg_release<40>();
    if (lane == 0 && cta_rank == 0) {
      bool ok = true;
      constexpr uint32_t idesc_main = make_idesc_tf32(256, BN, A_MN, B_MN);
      constexpr uint32_t idesc_cross = make_idesc_bf16(256, BN, A_MN, B_MN);
      // descriptor advance per K step of 8 (in 16-byte units): 32 bytes inside the swizzle row of a K-major tile; one
      // atom of 8 K rows (hi) or two (cross: 16 bf16 K rows) of an MN-major tile
      constexpr uint64_t a_step_hi = A_MN ? 64 : 2, a_step_x = A_MN ? 128 : 2;
      constexpr uint64_t b_step_hi = B_MN ? 64 : 2, b_step_x = B_MN ? 128 : 2;
      uint32_t it = 0;  // k-blocks consumed so far
      uint32_t g = 0;   // K chunks issued so far: chunk g goes into buffer g & 1
      WideSegments seg(work, cluster_id, num_clusters, num_chunks);
      while (ok && seg.next()) {
        for (int c = seg.c0; c < seg.c1 && ok; ++c, ++g) {
          const uint32_t b = g & 1u;
          if (g >= 2) {
            if (!ptx::mbar_wait_or_abort(&acc_empty_bar[b], ((g >> 1) - 1u) & 1u, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
          }
          const uint32_t acc = tmem_base + b * static_cast<uint32_t>(BN);
          const int kb_end = min(num_kb, (c + 1) * WIDE_KC);
          for (int kb = c * WIDE_KC; kb < kb_end; ++kb, ++it) {
            const int s = static_cast<int>(it % STAGES);
            const uint32_t ph = (it / STAGES) & 1u;
            if (!ptx::mbar_wait_or_abort(&full_bar[s], ph, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t st = ptx::smem_u32(smem + s * S::STAGE_BYTES);
            const uint64_t a_hi = A_MN ? make_smem_desc_mn(st, 4096, true) : make_smem_desc(st);
            const uint64_t a_x = A_MN ? make_smem_desc_mn(st + S::TILE_BYTES, 8192, false) : make_smem_desc(st + S::TILE_BYTES);
            const uint64_t b_hi = B_MN ? make_smem_desc_mn(st + 2 * S::TILE_BYTES, 4096, true) : make_smem_desc(st + 2 * S::TILE_BYTES);
            const uint64_t b_x = B_MN ? make_smem_desc_mn(st + 3 * S::TILE_BYTES, 8192, false) : make_smem_desc(st + 3 * S::TILE_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const bool first = (kb == c * WIDE_KC) && (k == 0);
              ptx::mma_bf16_pair(acc, a_x + k * a_step_x, b_x + k * b_step_x, idesc_cross, first ? 0u : 1u);  // lo*hi + hi*lo
              ptx::mma_tf32_pair(acc, a_hi + k * a_step_hi, b_hi + k * b_step_hi, idesc_main, 1u);          // hi*hi
            }
            ptx::tc_commit_pair(&empty_bar[s]);
          }
          if (ok) ptx::tc_commit_pair(&acc_full_bar[b]);
        }
      }
      if (!ok) atomicCAS(error_flag, 0, 302);
    }
  } else if (warp >= WIDE_DRAIN_WARP0) {
    // ---------------- drain + epilogue: 8 warps; lane quarter = warp % 4, column half = (warp - 4) / 4 ----------------
    ptx::reg_acquire<232>();
    const int q = warp & 3;
    const int half = (warp - WIDE_DRAIN_WARP0) >> 2;
    const int region = static_cast<int>(cta_rank) * 8 + (warp - WIDE_DRAIN_WARP0);  // this warp's 32 x 128 share of the pair's tile
    const bool vec_ok = epilogue_vector_ok(epi);
    const int mode = epilogue_mode(epi);
    float *tr = reinterpret_cast<float *>(smem + S::TR_OFFSET) + (warp - WIDE_DRAIN_WARP0) * TR_WARP_FLOATS;
    bool ok = true;
    uint32_t g = 0;
    WideSegments seg(work, cluster_id, num_clusters, num_chunks);
    while (ok && seg.next()) {
      float sum[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) sum[j] = 0.f;
      for (int c = seg.c0; c < seg.c1; ++c, ++g) {
        const uint32_t b = g & 1u;
        if (!ptx::mbar_wait_or_abort(&acc_full_bar[b], (g >> 1) & 1u, abort_flag)) {
          ok = false;
          if (lane == 0) atomicCAS(error_flag, 0, 303);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t tsrc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + b * static_cast<uint32_t>(BN) + static_cast<uint32_t>(half * 128);
#pragma unroll
        for (int jc = 0; jc < 4; ++jc) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(tsrc + static_cast<uint32_t>(jc * 32), r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[jc * 32 + j] += __uint_as_float(r[j]);
        }
        // this warp's reads of the buffer are complete: hand it back to the MMA issuer
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(&acc_empty_bar[b], 0);
      }
      if (!ok || num_kb <= 0) break;
      bool finish = true;  // this warp writes its share of the tile
      if (seg.c0 != 0 || seg.c1 != num_chunks) {
        // A split tile.  Every contributor leaves its partial sums in its own slot and counts itself in; the warp that
        // arrives last adds the slots up in cluster order (the same order whoever is last, so the result does not
        // depend on timing) and runs the epilogue.  Nobody waits for anybody.
        const int ts = seg.tile - work.dp_tiles;
        const int tile_u0 = ts * num_chunks;
        const int first = tile_u0 / work.sk_chunks;
        const int last = min((tile_u0 + num_chunks - 1) / work.sk_chunks, num_clusters - 1);
        const int my_slot = (cluster_id * work.sk_chunks >= tile_u0) ? 0 : 1;
        float4 *mine = reinterpret_cast<float4 *>(work.ws + (static_cast<size_t>(cluster_id * 2 + my_slot) * 16 + region) * WIDE_REGION_FLOATS);
#pragma unroll
        for (int j = 0; j < 32; ++j) __stcg(mine + j * 32 + lane, make_float4(sum[4 * j], sum[4 * j + 1], sum[4 * j + 2], sum[4 * j + 3]));
        __threadfence();
        __syncwarp();
        unsigned int arrived = 0;
        unsigned int *counter = work.counters + ts * 16 + region;
        if (lane == 0) arrived = atomicAdd(counter, 1u);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        finish = arrived == static_cast<unsigned int>(last - first);
        if (finish) {
          if (lane == 0) *counter = 0u;  // every contributor has arrived: ready for the next launch
          __threadfence();
          int tm, tn;
          wide_tile_coords(work, seg.tile, tm, tn);
          const long long row0 = static_cast<long long>(tm) * 256 + static_cast<long long>(cta_rank) * 128 + q * 32;
          const long long col_base = static_cast<long long>(tn) * BN + half * 128;
          if (last == first + 1) {
            // two contributors (the usual case): a + b is the same whichever of them is last, so the sum in registers
            // stays and only the other slot is read
            const int other = cluster_id == first ? last : first;
            const int slot = (other * work.sk_chunks >= tile_u0) ? 0 : 1;
            const float4 *theirs = reinterpret_cast<const float4 *>(work.ws + (static_cast<size_t>(other * 2 + slot) * 16 + region) * WIDE_REGION_FLOATS);
#pragma unroll
            for (int jb = 0; jb < 32; jb += 8) {
              float4 v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __ldcg(theirs + (jb + j) * 32 + lane);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                sum[4 * (jb + j)] += v[j].x; sum[4 * (jb + j) + 1] += v[j].y; sum[4 * (jb + j) + 2] += v[j].z; sum[4 * (jb + j) + 3] += v[j].w;
              }
            }
          } else {
            // more than two: every slot is added from zero in cluster order, 32 columns at a time with the loads of
            // four contributors in flight, and each 32 columns go straight to the epilogue
#pragma unroll 1
            for (int jc = 0; jc < 4; ++jc) {
              float acc[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) acc[j] = 0.f;
              for (int c4 = first; c4 <= last; c4 += 4) {
                float4 v[4][8];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const int cc = min(c4 + u, last);
                  const int slot = (cc * work.sk_chunks >= tile_u0) ? 0 : 1;
                  const float4 *theirs = reinterpret_cast<const float4 *>(work.ws + (static_cast<size_t>(cc * 2 + slot) * 16 + region) * WIDE_REGION_FLOATS);
#pragma unroll
                  for (int j = 0; j < 8; ++j) v[u][j] = __ldcg(theirs + (jc * 8 + j) * 32 + lane);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  if (c4 + u <= last) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                      acc[4 * j] += v[u][j].x; acc[4 * j + 1] += v[u][j].y; acc[4 * j + 2] += v[u][j].z; acc[4 * j + 3] += v[u][j].w;
                    }
                  }
                }
              }
              epilogue_row32(epi, acc, row0, lane, col_base + jc * 32, dims.M, dims.N, vec_ok, mode, tr);
            }
            finish = false;  // already written
          }
        }
      }
      if (finish) {
        int tm, tn;
        wide_tile_coords(work, seg.tile, tm, tn);
        const long long row0 = static_cast<long long>(tm) * 256 + static_cast<long long>(cta_rank) * 128 + q * 32;
        const long long col_base = static_cast<long long>(tn) * BN + half * 128;
#pragma unroll
        for (int jc = 0; jc < 4; ++jc) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = sum[jc * 32 + j];
          epilogue_row32(epi, v, row0, lane, col_base + jc * 32, dims.M, dims.N, vec_ok, mode, tr);
        }
      }
    }
  } else {
    ptx::reg_release<40>();  // warps 2-3: no role, but the whole warpgroup has to give its registers back
  }
  // every role leaves its loop only when its segments are done or a wait has given up; the pair stays together until
  // both CTAs are here, so nobody signals a barrier of a CTA that has exited
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Operand panels.  x = hi + lo with hi = x rounded to TF32 (round to nearest: truncation would bias every product the
// same way) and lo = x - hi (exact in fp32, at most 2^-11 |x|).  A product a*b is evaluated as
//     hi_a*hi_b                      one TF32 MMA (K = 8) into a "main" accumulator
//   + lo_a*hi_b + hi_a*lo_b          ONE BF16 MMA (K = 16) into the "cross" accumulator
// The cross terms are 2^-11 of the result, so 8 significant bits are enough for them (error 2^-19 of the result, below
// the fp32 accumulation noise of a long sum); packing both into one K = 16 instruction saves a third of the tensor work
// of the classical three-pass split.  Per 8 consecutive K elements the cross panel holds 16 bf16 (32 bytes, the same
// footprint as 8 fp32):  operand A: [lo x8 | hi x8],  operand B: [hi x8 | lo x8],  so that the K = 16 dot product of
// an A group with a B group is sum lo_a*hi_b + sum hi_a*lo_b.
// `raw` panels (FP32 FMA engine): hi = x unrounded, cross = 0.

// source already K-major (stride_k == 1); writes columns [0, round_up(k, 8)) of every panel row (pitch kp)
// With cross_mn != null the same pass also writes the cross panel of the source's OTHER reading, the one whose K runs
// along the source rows (MN-major operand, see gemm_prepare_shared): [2 * round_up(rows, 8)][kp] bf16, per 8 source
// rows 16 panel rows (role A: lo rows then hi rows; role B: hi rows then lo rows); source rows past `rows` are zero.
__global__ void split_rows_kernel(const float *__restrict__ src, long long stride_r, long long rows, long long k, long long kp,
                                  float *__restrict__ hi, float *__restrict__ cross, int role_b, int raw,
                                  uint16_t *__restrict__ cross_mn = nullptr, int role_mn_b = 0) {
  grid_dependency_wait();
  grid_dependency_release();
  const long long kg = (k + 7) >> 3;  // groups of 8 per panel row
  const long long rows_all = cross_mn != nullptr ? ((rows + 7) & ~7ll) : rows;
  const long long total = rows_all * kg;
  const bool vec = ((stride_r & 3) == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / kg;
    const long long c = (i - r * kg) << 3;
    float v[8];
    if (r >= rows) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    } else if (vec && c + 7 < k) {
      const float4 t = *reinterpret_cast<const float4 *>(src + r * stride_r + c);
      const float4 u = *reinterpret_cast<const float4 *>(src + r * stride_r + c + 4);
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; v[4] = u.x; v[5] = u.y; v[6] = u.z; v[7] = u.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (c + j < k) ? src[r * stride_r + c + j] : 0.f;
    }
    float h[8];
    uint32_t x[8];
    split_group(v, role_b, raw, h, x);
    if (r < rows) {
      float4 *ph = reinterpret_cast<float4 *>(hi + r * kp + c);
      ph[0] = make_float4(h[0], h[1], h[2], h[3]);
      ph[1] = make_float4(h[4], h[5], h[6], h[7]);
      if (cross != nullptr) {
        uint4 *px = reinterpret_cast<uint4 *>(cross + r * kp + c);
        px[0] = make_uint4(x[0], x[1], x[2], x[3]);
        px[1] = make_uint4(x[4], x[5], x[6], x[7]);
      }
    }
    if (cross_mn != nullptr) {
      // x[0..3] / x[4..7] are the packed lo and hi values of these 8 columns (in the order of role_b)
      const uint4 lo4 = role_b ? make_uint4(x[4], x[5], x[6], x[7]) : make_uint4(x[0], x[1], x[2], x[3]);
      const uint4 hi4 = role_b ? make_uint4(x[0], x[1], x[2], x[3]) : make_uint4(x[4], x[5], x[6], x[7]);
      const long long g16 = (r >> 3) * 16 + (r & 7);
      const long long row_lo = g16 + (role_mn_b ? 8 : 0), row_hi = g16 + (role_mn_b ? 0 : 8);
      *reinterpret_cast<uint4 *>(cross_mn + row_lo * kp + c) = lo4;
      *reinterpret_cast<uint4 *>(cross_mn + row_hi * kp + c) = hi4;
    }
  }
}

// source MN-major (stride_r == 1): tiled transposition, 32 (K) x 32 (rows) tile per block of 32 x 8 threads
__global__ void split_transpose_kernel(const float *__restrict__ src, long long stride_k, long long rows, long long k,
                                       long long kp, float *__restrict__ hi, float *__restrict__ cross, int role_b, int raw) {
  __shared__ float tile[32][33];
  const long long r0 = static_cast<long long>(blockIdx.x) * 32;  // panel rows (contiguous in the source)
  const long long k0 = static_cast<long long>(blockIdx.y) * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const long long kk = k0 + j, rr = r0 + threadIdx.x;
    tile[j][threadIdx.x] = (kk < k && rr < rows) ? src[kk * stride_k + rr] : 0.f;
  }
  __syncthreads();
  // thread x = word x of the row's 32 words: hi word = element x; cross word = bf16 pair (see the group layout above)
  const int g = threadIdx.x >> 3, q = threadIdx.x & 7;       // group of 8 within the 32, word within the group
  const int e = g * 8 + (q & 3) * 2;                         // first of the two source elements of this cross word
  const bool want_lo = role_b ? (q >= 4) : (q < 4);
  uint32_t *xw = reinterpret_cast<uint32_t *>(cross);
  for (int j = threadIdx.y; j < 32; j += 8) {
    const long long rr = r0 + j, kk = k0 + threadIdx.x;
    if (rr >= rows) continue;
    if (kk < ((k + 7) & ~7ll)) {
      const float x = tile[threadIdx.x][j];
      hi[rr * kp + kk] = raw ? x : round_tf32(x);
      const float x0 = tile[e][j], x1 = tile[e + 1][j];
      const float h0 = round_tf32(x0), h1 = round_tf32(x1);
      xw[rr * kp + kk] = raw ? 0u : (want_lo ? pack_bf16(x0 - h0, x1 - h1) : pack_bf16(h0, h1));
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// FP32 FMA engine: 64x64 tile, 16 of K per step, 256 threads x (4x4) outputs, arbitrary strides
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gemm_fp32_fma_kernel(const Operand A, const Operand B, const GemmDims dims, const Epilogue epi) {
  __shared__ float sa[16][64 + 4];
  __shared__ float sb[16][64 + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const long long m0 = static_cast<long long>(blockIdx.y) * 64, n0 = static_cast<long long>(blockIdx.x) * 64;
  float acc[4][4] = {};
  for (long long k0 = 0; k0 < dims.K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      int r, kk;
      if (A.stride_k == 1) { r = i >> 4; kk = i & 15; } else { kk = i >> 6; r = i & 63; }
      const long long m = m0 + r, k = k0 + kk;
      sa[kk][r] = (m < dims.M && k < dims.K) ? A.ptr[m * A.stride_r + k * A.stride_k] + (A.lo ? A.lo[m * A.stride_r + k * A.stride_k] : 0.f) : 0.f;
      if (B.stride_k == 1) { r = i >> 4; kk = i & 15; } else { kk = i >> 6; r = i & 63; }
      const long long n = n0 + r;
      sb[kk][r] = (n < dims.N && k0 + kk < dims.K) ? B.ptr[n * B.stride_r + (k0 + kk) * B.stride_k] + (B.lo ? B.lo[n * B.stride_r + (k0 + kk) * B.stride_k] : 0.f) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = sa[kk][ty * 4 + i]; b[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < dims.M && n < dims.N) epi.C[c_row(epi, m) + n] = epilogue_value(epi, acc[i][j], m, n);
    }
}

// ---------------------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  // function-local static: initialised once, by one thread, before any caller sees the pointer
  static const PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    return static_cast<PFN_cuTensorMapEncodeTiled_v12000>(nullptr);
  }();
  return fn;
}

// First-use set-up per (kernel, device): the opt-in to large dynamic shared memory is a per-device attribute of the
// kernel.  One table per kernel, indexed by the full device number and guarded, so that two host threads that drive
// two GPUs can make their first calls at the same time.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
  std::mutex mutex;
  int value[kMaxDevices] = {};  // 0 = not configured yet
  // returns the cached value (> 0) or the result of `configure` (<= 0 on failure, not cached)
  template <typename F> int get(int device, F configure) {
    if (device < 0 || device >= kMaxDevices) return 0;
    std::lock_guard<std::mutex> lock(mutex);
    if (value[device] == 0) {
      const int v = configure();
      if (v > 0) value[device] = v;
      return v;
    }
    return value[device];
  }
};

bool make_panel_map(CUtensorMap *map, const float *panel, long long rows, long long k, long long kp, int box_rows) {
  PFN_cuTensorMapEncodeTiled_v12000 fn = get_encode_fn();
  if (fn == nullptr) return false;
  // panels are zero-filled up to the next multiple of 8 along K and the cross panel is only meaningful in whole groups of 8
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>((k + 7) & ~7ll), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(kp) * 4};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(panel), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// MN-major panels (arrays [k][kp]): 3-D views (128 bytes of rows, K, 128-byte chunk) so that one box lands in shared
// memory chunk after chunk, each chunk K rows of 128 bytes.  hi: fp32, 32 K rows per stage; cross: bf16, 64 panel rows.
static bool make_panel_map_mn(CUtensorMap *map, const void *panel, bool cross, long long rows, long long k, long long kp) {
  PFN_cuTensorMapEncodeTiled_v12000 fn = get_encode_fn();
  if (fn == nullptr) return false;
  const long long elems = cross ? 64 : 32;                     // elements in 128 bytes
  const long long krows = cross ? 2 * ((k + 7) & ~7ll) : k;    // panel rows along K
  cuuint64_t gdim[3] = {static_cast<cuuint64_t>(elems), static_cast<cuuint64_t>(krows), static_cast<cuuint64_t>((rows + elems - 1) / elems)};
  cuuint64_t gstride[2] = {static_cast<cuuint64_t>(kp) * (cross ? 2 : 4), 128};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(elems), static_cast<cuuint32_t>(cross ? 2 * BK : BK), static_cast<cuuint32_t>(128 / elems)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, cross ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(panel), gdim, gstride,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, cross ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

static inline long long round_up(long long x, long long m) { return (x + m - 1) / m * m; }

size_t shared_panel_floats(long long R, long long C) {
  const long long pitch = round_up(C, 64), r8 = round_up(R, 8);
  return static_cast<size_t>(3 * r8 * pitch) + 64;  // hi, K-major cross, MN-major cross (2 * r8 rows of bf16)
}

void shared_panel_layout(float *mem, long long R, long long C, int role_rows, Panels *as_rows, int role_cols, Panels *as_cols, PanelSink *sink) {
  const long long pitch = round_up(C, 64), r8 = round_up(R, 8);
  float *hi = mem, *cross_k = mem + r8 * pitch;
  uint16_t *cross_mn = reinterpret_cast<uint16_t *>(mem + 2 * r8 * pitch);
  if (as_rows != nullptr) {
    *as_rows = Panels{};
    as_rows->hi = hi; as_rows->lo = cross_k; as_rows->rows = R; as_rows->k = C; as_rows->kp = pitch;
    as_rows->role = role_rows; as_rows->major = PANEL_K;
  }
  if (as_cols != nullptr) {
    *as_cols = Panels{};
    as_cols->hi = hi; as_cols->lo = reinterpret_cast<float *>(cross_mn); as_cols->rows = C; as_cols->k = R; as_cols->kp = pitch;
    as_cols->role = role_cols; as_cols->major = PANEL_MN;
  }
  if (sink != nullptr) {
    sink->hi = hi;
    sink->cross_k = as_rows != nullptr ? cross_k : nullptr;
    sink->cross_mn = as_cols != nullptr ? cross_mn : nullptr;
    sink->kp = pitch;
    sink->role_k = role_rows;
    sink->role_mn = role_cols;
  }
}

bool epilogue_takes_stats(const Context &ctx, const Epilogue &e, long long N) {
  if (ctx.gemm_engine != 0 || (N & 31) != 0 || e.ldc != N || e.addend != nullptr || e.accumulate || e.seg_rows != 0) return false;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(e.C) | reinterpret_cast<uintptr_t>(e.bias) | reinterpret_cast<uintptr_t>(e.aux_pre) |
                         reinterpret_cast<uintptr_t>(e.aux_y) | reinterpret_cast<uintptr_t>(e.col_scale) | reinterpret_cast<uintptr_t>(e.col_shift) |
                         reinterpret_cast<uintptr_t>(e.col_stats) | reinterpret_cast<uintptr_t>(e.col_mean);
  return (bits & 15) == 0 && ((e.ldc | e.ld_aux) & 3) == 0;
}

int gemm_prepare_shared(Context &ctx, const float *src, long long stride_r, long long R, long long C, float *mem, int role_rows,
                        Panels *as_rows, int role_cols, Panels *as_cols) {
  if (src == nullptr || mem == nullptr || R <= 0 || C <= 0 || (reinterpret_cast<uintptr_t>(mem) & 255) != 0) return MYEA_E_INVALID;
  const long long pitch = round_up(C, 64), r8 = round_up(R, 8);
  float *hi = mem, *cross_k = mem + r8 * pitch;
  uint16_t *cross_mn = reinterpret_cast<uint16_t *>(mem + 2 * r8 * pitch);
  shared_panel_layout(mem, R, C, role_rows, as_rows, role_cols, as_cols, nullptr);
  const int raw = ctx.gemm_engine == 1 ? 1 : 0;
  const long long total = r8 * ((C + 7) >> 3);
  int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
  if (blocks < 1) blocks = 1;
  ctx.begin(TC_SPLIT);
  launch_dependent(ctx, split_rows_kernel, dim3(blocks), dim3(256), 0, src, stride_r, R, C, pitch, hi, as_rows != nullptr ? cross_k : nullptr, role_rows,
                   raw, as_cols != nullptr ? cross_mn : nullptr, role_cols);
  ctx.end(TC_SPLIT);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

bool gemm_takes_mn_major(const Context &ctx, long long M, long long N) {
  if (ctx.gemm_engine == 1) return true;
  return ctx.gemm_bn == 0 ? (M > 128 && N > 128) : (ctx.gemm_bn == 3 || ctx.gemm_bn == 4);
}

size_t gemm_scratch_floats(long long M, long long N, long long K) {
  const long long kp = round_up(K, BK);
  return static_cast<size_t>(2 * (M + N) * kp) + 64;
}

size_t panel_floats(long long rows, long long k) { return static_cast<size_t>(2 * rows * round_up(k, BK)); }

Panels panels_at(float *mem, long long rows, long long k, int role) {
  Panels p;
  p.role = role;
  p.rows = rows;
  p.k = k;
  p.kp = round_up(k, BK);
  p.hi = mem;
  p.lo = mem + rows * p.kp;
  return p;
}

// Writes `op` (rows x k) into the region of `dst` that starts at (row_offset, k_offset): several sources can be
// fused into one panel set (the four LSTM gate matrices side by side, for instance).
int gemm_prepare_into(Context &ctx, const Operand &op, const Panels &dst, long long row_offset, long long k_offset) {
  // cross groups are 8 K elements wide: a fused source must start on a group boundary (its tail is zero-filled up to the
  // next boundary, so the following source may start there)
  if (op.rows <= 0 || op.k <= 0 || row_offset + op.rows > dst.rows || k_offset + op.k > dst.k || (k_offset & 7) != 0) return MYEA_E_INVALID;
  float *hi = dst.hi + row_offset * dst.kp + k_offset, *lo = dst.lo + row_offset * dst.kp + k_offset;
  const int raw = ctx.gemm_engine == 1 ? 1 : 0;
  ctx.begin(TC_SPLIT);
  if (op.stride_k == 1) {
    const long long total = op.rows * ((op.k + 7) >> 3);
    int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
    if (blocks < 1) blocks = 1;
    launch_dependent(ctx, split_rows_kernel, dim3(blocks), dim3(256), 0, op.ptr, op.stride_r, op.rows, op.k, dst.kp, hi, lo, dst.role, raw,
                     static_cast<uint16_t *>(nullptr), 0);
  } else {
    dim3 grid(static_cast<unsigned>((op.rows + 31) / 32), static_cast<unsigned>((op.k + 31) / 32));
    split_transpose_kernel<<<grid, dim3(32, 8), 0, ctx.stream>>>(op.ptr, op.stride_k, op.rows, op.k, dst.kp, hi, lo, dst.role, raw);
  }
  ctx.end(TC_SPLIT);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

int gemm_prepare_interleaved(Context &ctx, const Operand &op, const Panels &dst, long long row_offset, long long row_step) {
  if (op.rows <= 0 || op.k != dst.k || op.stride_k != 1 || row_step < 1 || row_offset + (op.rows - 1) * row_step >= dst.rows || dst.major != PANEL_K)
    return MYEA_E_INVALID;
  const int raw = ctx.gemm_engine == 1 ? 1 : 0;
  const long long total = op.rows * ((op.k + 7) >> 3);
  int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
  if (blocks < 1) blocks = 1;
  ctx.begin(TC_SPLIT);
  // the kernel only sees a wider pitch: source row r lands on panel row row_offset + r * row_step
  launch_dependent(ctx, split_rows_kernel, dim3(blocks), dim3(256), 0, op.ptr, op.stride_r, op.rows, op.k, dst.kp * row_step,
                   dst.hi + row_offset * dst.kp, dst.lo + row_offset * dst.kp, dst.role, raw, static_cast<uint16_t *>(nullptr), 0);
  ctx.end(TC_SPLIT);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

int gemm_prepare(Context &ctx, const Operand &op, float *mem, Panels *out, int role) {
  *out = panels_at(mem, op.rows, op.k, role);
  return gemm_prepare_into(ctx, op, *out, 0, 0);
}

template <int BN, int STAGES>
static int launch_tcgen05(Context &ctx, const CUtensorMap maps[4], const GemmDims &dims, const Epilogue &epi) {
  using S = GemmSmem<BN, STAGES>;
  static PerDeviceOnce once;
  if (once.get(ctx.device, [] {
        return cudaFuncSetAttribute(gemm3x_tf32_tcgen05_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL) == cudaSuccess ? 1 : 0;
      }) <= 0)
    return MYEA_E_CUDA;
  dim3 grid(static_cast<unsigned>((dims.N + BN - 1) / BN), static_cast<unsigned>((dims.M + BM - 1) / BM));
  launch_dependent(ctx, gemm3x_tf32_tcgen05_kernel<BN, STAGES>, grid, dim3(GEMM_THREADS), S::TOTAL, maps[0], maps[1], maps[2], maps[3], dims, epi,
                   ctx.d_error_flag);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

static int launch_tcgen05_pair(Context &ctx, const CUtensorMap maps[4], const GemmDims &dims, const Epilogue &epi) {
  static PerDeviceOnce once;
  if (once.get(ctx.device, [] {
        return cudaFuncSetAttribute(gemm3x_tf32_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL) == cudaSuccess ? 1 : 0;
      }) <= 0)
    return MYEA_E_CUDA;
  // the cluster shape (2, 1, 1) is a compile-time attribute of the kernel: the two CTAs of a pair are neighbours along
  // grid x and split the 256 rows of the tile; grid y walks the column tiles
  dim3 grid(static_cast<unsigned>(2 * ((dims.M + 255) / 256)), static_cast<unsigned>((dims.N + 127) / 128));
  gemm3x_tf32_tcgen05_pair_kernel<<<grid, GEMM_THREADS, PairSmem::TOTAL, ctx.stream>>>(maps[0], maps[1], maps[2], maps[3], dims, epi, ctx.d_error_flag);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// Workspace of the wide kernel's split tiles: two partial-sum slots of one 256 x 256 tile per cluster and one arrival
// counter per (split tile, warp region).  Without it the wide kernel computes whole tiles only.
int gemm_splitk_reserve(Context &ctx) {
  if (ctx.sk_ws != nullptr) return MYEA_OK;
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx.device) != cudaSuccess || sms < 2) return MYEA_E_CUDA;
  const int clusters = sms / 2;
  const size_t floats = static_cast<size_t>(clusters) * 2 * 16 * WIDE_REGION_FLOATS;
  if (cudaMalloc(&ctx.sk_ws, floats * sizeof(float)) != cudaSuccess) { ctx.sk_ws = nullptr; return MYEA_E_CUDA; }
  if (cudaMalloc(&ctx.sk_counters, static_cast<size_t>(clusters) * 16 * sizeof(unsigned int)) != cudaSuccess ||
      cudaMemset(ctx.sk_counters, 0, static_cast<size_t>(clusters) * 16 * sizeof(unsigned int)) != cudaSuccess) {
    cudaFree(ctx.sk_ws);
    ctx.sk_ws = nullptr;
    return MYEA_E_CUDA;
  }
  ctx.sk_clusters = clusters;
  return MYEA_OK;
}
void gemm_splitk_release(Context &ctx) {
  if (ctx.sk_ws != nullptr) cudaFree(ctx.sk_ws);
  if (ctx.sk_counters != nullptr) cudaFree(ctx.sk_counters);
  ctx.sk_ws = nullptr;
  ctx.sk_counters = nullptr;
  ctx.sk_clusters = 0;
}

template <bool A_MN, bool B_MN>
static int launch_tcgen05_wide(Context &ctx, const CUtensorMap maps[4], const GemmDims &dims, const Epilogue &epi) {
  auto kernel = gemm3x_tf32_tcgen05_wide_kernel<A_MN, B_MN>;
  static PerDeviceOnce once;  // value: clusters of two CTAs that can be resident at once on the device
  const int device = ctx.device;
  const int G = once.get(device, [kernel, device] {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WideSmem::TOTAL) != cudaSuccess) return 0;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 2) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1));
    cfg.blockDim = dim3(WIDE_THREADS);
    cfg.dynamicSmemBytes = WideSmem::TOTAL;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = sms / 2;
    }
    return n < sms / 2 ? n : sms / 2;
  });
  if (G <= 0) return MYEA_E_CUDA;
  const int num_kb = (dims.K + BK - 1) / BK;
  const int num_chunks = (num_kb + WIDE_KC - 1) / WIDE_KC;
  WideWork work = {};
  work.tiles_m = (dims.M + 255) / 256;
  work.tiles_n = (dims.N + 255) / 256;
  work.num_tiles = work.tiles_m * work.tiles_n;
  work.dp_tiles = work.num_tiles;
  int grid_clusters = work.num_tiles < G ? work.num_tiles : G;
  // stream-K for the partial last wave (gemm_bn 4 switches it off): needs the partial-sum workspace and more than one
  // K chunk per tile
  const int rem = work.num_tiles % G;
  if (ctx.gemm_bn != 4 && ctx.sk_ws != nullptr && ctx.sk_clusters >= G && rem != 0 && num_chunks >= 2) {
    const int units = rem * num_chunks;
    int per_cluster = (units + G - 1) / G;
    // at most 8 clusters share one tile: the cluster that arrives last adds up every other contributor's 256 KB of
    // partial sums, and past 8 that pass outweighs the shorter K walk (256 x 1024 x 4096, 4 tiles: 16-way split
    // 53.6 us, 8-way 47.2 us, 4-way 51.0 us per call with its split passes)
    constexpr int max_split = 8;
    per_cluster = std::max(per_cluster, (num_chunks + max_split - 1) / max_split);

    // splitting a tile costs about one chunk's time (partial sums through L2, one counter round trip, the second
    // pass of the warp that arrives last): worth it when it takes at least two chunks off the longest cluster
    if (num_chunks - per_cluster >= 2) {
      work.dp_tiles = work.num_tiles - rem;
      work.sk_units = units;
      work.sk_chunks = per_cluster;
      work.ws = ctx.sk_ws;
      work.counters = ctx.sk_counters;
      const int used = (units + per_cluster - 1) / per_cluster;
      grid_clusters = work.dp_tiles > 0 ? G : used;
    }
  }
  launch_dependent(ctx, kernel, dim3(static_cast<unsigned>(2 * grid_clusters)), dim3(WIDE_THREADS), WideSmem::TOTAL, maps[0], maps[1], maps[2],
                   maps[3], dims, work, epi, ctx.d_error_flag);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// C (+)= A * B^T on operands whose panels are already in place; (row0, rows) select a row range of each panel set.
int gemm_panels(Context &ctx, const Panels &A, long long a_row0, long long M, const Panels &B, long long b_row0, long long N,
                const Epilogue &epi) {
  if (A.k != B.k || M <= 0 || N <= 0 || A.k <= 0 || a_row0 < 0 || b_row0 < 0 || a_row0 + M > A.rows || b_row0 + N > B.rows) return MYEA_E_INVALID;
  if (A.role != PANEL_ROLE_A || B.role != PANEL_ROLE_B) return MYEA_E_INVALID;  // the cross panels of the two sides differ
  const bool a_mn = A.major == PANEL_MN, b_mn = B.major == PANEL_MN;
  // a row range of an MN-major operand starts on a multiple of 8 (16-byte TMA base) and its last 128-byte chunk must
  // stay inside the pitch
  if (a_mn && ((a_row0 & 7) != 0 || (A.kp & 63) != 0 || a_row0 + ((M + 63) & ~63ll) > A.kp)) return MYEA_E_INVALID;
  if (b_mn && ((b_row0 & 7) != 0 || (B.kp & 63) != 0 || b_row0 + ((N + 63) & ~63ll) > B.kp)) return MYEA_E_INVALID;
  GemmDims dims{static_cast<int>(M), static_cast<int>(N), static_cast<int>(A.k)};
  int rc;
  if (ctx.gemm_engine == 1) {
    // the FP32 FMA engine reads the (unrounded) hi panels by strides; their cross panels are zero
    Operand oa = a_mn ? Operand{A.hi + a_row0, M, A.k, 1, A.kp, nullptr} : Operand{A.hi + a_row0 * A.kp, M, A.k, A.kp, 1, A.lo + a_row0 * A.kp};
    Operand ob = b_mn ? Operand{B.hi + b_row0, N, B.k, 1, B.kp, nullptr} : Operand{B.hi + b_row0 * B.kp, N, B.k, B.kp, 1, B.lo + b_row0 * B.kp};
    ctx.begin(TC_GEMM);
    dim3 grid(static_cast<unsigned>((dims.N + 63) / 64), static_cast<unsigned>((dims.M + 63) / 64));
    gemm_fp32_fma_kernel<<<grid, 256, 0, ctx.stream>>>(oa, ob, dims, epi);
    ctx.end(TC_GEMM);
    rc = cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
  } else {
    // gemm_bn: 0 = heuristic, 3 = wide CTA pair (256 x 256), 4 = the same without stream-K, 2 = CTA pair (256 x 128),
    // 128 / 256 = single CTA
    // A short contraction whose 128 x 128 tiles fit one wave of CTAs runs on the single-CTA kernel: every tile walks
    // its whole K without a partial-sum hand-over, which on such shapes (a recurrent LSTM step, 256 x 4096 x 1024:
    // 16 wide tiles for 74 clusters) costs more than it saves.  Measured with K <= 1024 for 32 to 128 tiles: 3 to 7 us
    // less per launch; at K = 2048 the wide kernel with stream-K is ahead again.
    const long long tiles128 = ((M + 127) / 128) * ((N + 127) / 128);
    const bool one_wave = ctx.gemm_bn == 0 && !a_mn && !b_mn && M > 128 && N > 128 && A.k <= 1024 && tiles128 <= 148;
    const bool wide = gemm_takes_mn_major(ctx, M, N) && !one_wave;
    if ((a_mn || b_mn) && !wide) return MYEA_E_INVALID;
    const bool pair = !wide && !one_wave && (ctx.gemm_bn == 0 ? (M > 128) : (ctx.gemm_bn == 2));
    const int bn = ctx.gemm_bn == 256 ? 256 : 128;
    const int b_box = wide ? 128 : (pair ? 64 : bn);
    CUtensorMap maps[4];
    bool ok = true;
    if (a_mn) ok = ok && make_panel_map_mn(&maps[0], A.hi + a_row0, false, M, A.k, A.kp) &&
                  make_panel_map_mn(&maps[1], reinterpret_cast<const uint16_t *>(A.lo) + a_row0, true, M, A.k, A.kp);
    else ok = ok && make_panel_map(&maps[0], A.hi + a_row0 * A.kp, M, A.k, A.kp, BM) && make_panel_map(&maps[1], A.lo + a_row0 * A.kp, M, A.k, A.kp, BM);
    if (b_mn) ok = ok && make_panel_map_mn(&maps[2], B.hi + b_row0, false, N, B.k, B.kp) &&
                  make_panel_map_mn(&maps[3], reinterpret_cast<const uint16_t *>(B.lo) + b_row0, true, N, B.k, B.kp);
    else ok = ok && make_panel_map(&maps[2], B.hi + b_row0 * B.kp, N, B.k, B.kp, b_box) && make_panel_map(&maps[3], B.lo + b_row0 * B.kp, N, B.k, B.kp, b_box);
    if (!ok) return MYEA_E_CUDA;
    ctx.begin(TC_GEMM);
    if (wide) {
      if (a_mn) rc = b_mn ? launch_tcgen05_wide<true, true>(ctx, maps, dims, epi) : launch_tcgen05_wide<true, false>(ctx, maps, dims, epi);
      else rc = b_mn ? launch_tcgen05_wide<false, true>(ctx, maps, dims, epi) : launch_tcgen05_wide<false, false>(ctx, maps, dims, epi);
    } else if (pair) {
      rc = launch_tcgen05_pair(ctx, maps, dims, epi);
    } else {
      rc = (bn == 256) ? launch_tcgen05<256, 2>(ctx, maps, dims, epi) : launch_tcgen05<128, 3>(ctx, maps, dims, epi);
    }
    ctx.end(TC_GEMM);
  }
  ctx.gemm_flops += 2.0 * dims.M * dims.N * static_cast<double>(dims.K);
  return rc;
}

int gemm_nt(Context &ctx, const Operand &A, const Operand &B, const Epilogue &epi, const GemmScratch &scratch) {
  if (A.k != B.k || A.rows <= 0 || B.rows <= 0 || A.k <= 0) return MYEA_E_INVALID;
  if (ctx.gemm_engine == 1) {  // the FP32 FMA engine reads the fp32 sources directly
    GemmDims dims{static_cast<int>(A.rows), static_cast<int>(B.rows), static_cast<int>(A.k)};
    ctx.begin(TC_GEMM);
    dim3 grid(static_cast<unsigned>((dims.N + 63) / 64), static_cast<unsigned>((dims.M + 63) / 64));
    gemm_fp32_fma_kernel<<<grid, 256, 0, ctx.stream>>>(A, B, dims, epi);
    ctx.end(TC_GEMM);
    ctx.gemm_flops += 2.0 * dims.M * dims.N * static_cast<double>(dims.K);
    return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
  }
  if (scratch.base == nullptr || scratch.floats < gemm_scratch_floats(A.rows, B.rows, A.k)) return MYEA_E_INVALID;
  float *base = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(scratch.base) + 255) & ~static_cast<uintptr_t>(255));
  Panels pa, pb;
  int rc = gemm_prepare(ctx, A, base, &pa, PANEL_ROLE_A);
  if (rc == MYEA_OK) rc = gemm_prepare(ctx, B, base + panel_floats(A.rows, A.k), &pb, PANEL_ROLE_B);
  if (rc != MYEA_OK) return rc;
  return gemm_panels(ctx, pa, 0, A.rows, pb, 0, B.rows, epi);
}

}  // namespace myea
