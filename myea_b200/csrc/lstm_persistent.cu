// All time steps of one LSTM layer and direction in ONE launch.
//
// The reference walks time strictly serially: per step the recurrent products of the four gates, the gate / cell /
// peephole arithmetic, then the next step (forward: Neural_Network__Recurrent_Forward_Pass__OpenMP.cpp:448-471 with the
// gates at :859-1040; BPTT: Neural_Network__Recurrent_Backward_Pass__OpenMP.cpp:440-862 with :1130-1604).  Launching a
// contraction and a cell kernel per step leaves the GPU waiting on launches: a step is 2 GFLOP.  Here one kernel stays
// resident for the whole walk:
//
//   grid      one cluster of SPLIT CTAs per 128 x BN tile of the step's product; the CTAs of a cluster share the tile and
//             split its K range (forward: BN = 128 gate columns, K = cells in 2 slices; backward: BN = 64 cells, K = 4 x
//             cells in 4 slices: 8-CTA clusters would halve the weight traffic per SM, but a B200 holds only 15 of the 16
//             the benchmark layer needs), so that every SM streams a small share of the recurrent weights per step
//             (they do not fit shared memory; they stay in L2)
//   warp 0    TMA producer: waits until the operand panels of the previous step are complete (step barrier), then
//             loads its K slice of the step's operand (h of step s-1, or the gate errors of step s-1 of the walk) and
//             of the recurrent weight panels, 32 floats of K per stage, hi and cross panels
//   warp 1    one lane issues tcgen05.mma (TF32 hi*hi + one BF16 K=16 instruction for both cross terms) into tensor memory
//   warps 4-11 take the partial sums out of tensor memory and exchange them inside the cluster: every thread pushes the
//             columns that other CTAs finish into those CTAs' shared memory (distributed shared memory) and keeps its
//             own; the sums are added in slice order (bitwise repeatable).  Each thread then finishes 8 cells of one batch
//             row: gates, peepholes, cell state, zoneout keep (forward) or the gate errors (backward).  The operand
//             panels of the next step are stored before the step barrier; the layer's arrays, which only later kernels
//             read, after it.  What the cell needs from global memory is fetched before the wait for the tensor cores.
//   step barrier: every CTA of a row of tiles counts itself in on a global counter when its results of step s are
//             written; producers poll it before they load step s + 1.  Every wait in the kernel is bounded (about a
//             second of SM clock): a wait that runs out sets the handle's error flag and an abort word that makes all
//             other waits give up, the CTAs meet at their final barriers, free tensor memory and return.
// The launch needs all its CTAs resident at once (they wait for each other): lstm_persistent_plan checks the tile count
// against cudaOccupancyMaxActiveClusters and the layer falls back to one launch pair per step otherwise.
#include "lstm.cuh"
#include "panel_math.cuh"
#include "tcgen05.cuh"

#include <cudaTypedefs.h>

#include <algorithm>
#include <mutex>
#include <type_traits>

namespace myea {

// three warpgroups: warps 0-3 hold the two single-thread roles (warps 2-3 idle) and give most of their registers away
// (setmaxnreg); warps 4-11 exchange and run the cells with 232 registers each
constexpr int PS_THREADS = 384;
constexpr int PS_EPI_WARP0 = 4;
constexpr int PS_EPI_THREADS = 256;
constexpr int PS_TILE_BYTES = 128 * BK * 4;          // 128 operand rows x 128 bytes
// shapes of the two kernels: BN columns per tile, SPLIT K slices (= CTAs per cluster)
template <int KIND> struct PsShape;
template <> struct PsShape<1> { static constexpr int BN = 128, SPLIT = 2, STAGES = 3; };
template <> struct PsShape<2> { static constexpr int BN = 64, SPLIT = 4, STAGES = 4; };
template <int KIND> struct PsSmem {
  static constexpr int BN = PsShape<KIND>::BN, STAGES = PsShape<KIND>::STAGES;
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int STAGE_BYTES = 2 * PS_TILE_BYTES + 2 * B_BYTES;  // A hi, A cross, B hi, B cross
  static constexpr int RECV_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int RECV_BYTES = (PsShape<KIND>::SPLIT - 1) * 128 * (BN / PsShape<KIND>::SPLIT) * 4;  // one slot per peer
  static constexpr int BAR_OFFSET = RECV_OFFSET + RECV_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 512 + 1024;                // barriers, peepholes, slack to align the base
  // Accumulators in tensor memory, BN columns each, filled one after the other: every one takes the products of
  // ACC_KB K blocks (or more when the K slice is longer than MAX_ACC of them), hi*hi and cross terms alike.  The tensor
  // core truncates when it adds into an accumulator, so a chain of adds is kept to 64 instructions where the slice
  // allows; and the exchange warps read an accumulator while the tensor core fills the next one.
  static constexpr int TMEM_COLS = 512;
  static constexpr int MAX_ACC = TMEM_COLS / BN, ACC_KB = 8;
  static_assert(TOTAL <= 227 * 1024, "shared memory of one SM");
  static_assert(STAGE_BYTES % 1024 == 0 && B_BYTES % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
};

struct LstmSeq {
  int T = 0, B = 0, C = 0;
  int reverse = 0;              // the direction's time runs from T-1 down to 0
  int tiles_m = 0, tiles_n = 0;
  int split = 1;                // CTAs per cluster = K slices per tile
  int kb_per = 0, num_kb = 0;   // 32-float K blocks per slice / in all
  long long ldh = 0;            // pitch of the layer's output / error rows
  long long a_rows = 0;         // rows of one of the two operand-panel buffers (a multiple of 128)
  long long kpa = 0;            // pitch of the operand panels
  long long Cp = 0;
  float *a_hi = nullptr, *a_cross = nullptr;  // [2][a_rows][kpa]: step s reads buffer (s-1)&1 and writes buffer s&1
  const float *peep = nullptr;                // [3][C]
  const float *gates_in = nullptr;            // [T*B, 4C]
  float *act = nullptr, *cstate = nullptr, *cact = nullptr;
  float *values = nullptr;                    // layer outputs, this direction's columns, pitch ldh
  const uint8_t *zone_state = nullptr, *zone_output = nullptr;  // [T][C] or null
  float *deriv = nullptr;                     // error on the outputs, this direction's columns, pitch ldh
  float *dgates = nullptr, *dcstate = nullptr;
  unsigned int *sync = nullptr;               // [tiles_m] step counters, then one abort word
  int *error_flag = nullptr;
};

// the arrays of walk step s as the cell arithmetic wants them
template <int KIND>
__device__ __forceinline__ LstmStep step_view(const LstmSeq &q, int s) {
  LstmStep p;
  const long long B = q.B, C = q.C, T = q.T;
  p.C = C; p.ldh = q.ldh; p.kp = q.kpa; p.Cp = q.Cp;
  p.peep = q.peep;
  if (s + 1 < q.T) {
    p.p_hi = q.a_hi + static_cast<long long>(s & 1) * q.a_rows * q.kpa;
    p.p_cross = q.a_cross + static_cast<long long>(s & 1) * q.a_rows * q.kpa;
  }
  if (KIND == 1) {
    const long long t = q.reverse ? T - 1 - s : s, tp = q.reverse ? t + 1 : t - 1;
    p.gates_in = q.gates_in + t * B * 4 * C;
    p.c_prev = q.cstate + tp * B * C;
    p.h_prev = q.values + tp * B * q.ldh;
    p.act = q.act + t * B * 4 * C;
    p.cstate = q.cstate + t * B * C;
    p.cact = q.cact + t * B * C;
    p.h = q.values + t * B * q.ldh;
    p.zone_state = q.zone_state != nullptr ? q.zone_state + t * C : nullptr;
    p.zone_output = q.zone_output != nullptr ? q.zone_output + t * C : nullptr;
  } else {
    const long long t = q.reverse ? s : T - 1 - s;        // the walk goes against the direction
    const long long tn = q.reverse ? t - 1 : t + 1;       // the step after t in the layer's direction (done before)
    const long long tp = q.reverse ? t + 1 : t - 1;       // the step before t
    p.dh = q.deriv + t * B * q.ldh;
    p.b_act = q.act + t * B * 4 * C;
    p.b_cact = q.cact + t * B * C;
    p.b_c_prev = (tp >= 0 && tp < T) ? q.cstate + tp * B * C : nullptr;
    p.act_next = q.act + tn * B * 4 * C;
    p.dgates_next = q.dgates + tn * B * 4 * C;
    p.dc_next = q.dcstate + tn * B * C;
    p.dgates = q.dgates + t * B * 4 * C;
    p.dcstate = q.dcstate + t * B * C;
  }
  return p;
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_relaxed_gpu(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int *p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait for a step counter; gives up when any CTA has raised the abort word or after about a second.
__device__ __forceinline__ bool wait_step_counter(const unsigned int *counter, unsigned int target, const unsigned int *abort_word, volatile int *abort_flag) {
  if (*abort_flag) return false;
  if (ld_acquire_gpu(counter) >= target) return true;
  const long long t0 = clock64();
  for (;;) {
    if (ld_acquire_gpu(counter) >= target) return true;
    if (ld_relaxed_gpu(abort_word) != 0u || clock64() - t0 > (1ll << 31)) {
      *abort_flag = 1;
      return false;
    }
  }
}

template <int KIND>
__global__ void __launch_bounds__(PS_THREADS, 1)
lstm_persistent_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_x,
                       const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_x, const LstmSeq q) {
  using SM = PsSmem<KIND>;
  constexpr int STAGES = SM::STAGES, BN = SM::BN, S = PsShape<KIND>::SPLIT;
  constexpr int W = BN / S;   // columns of the tile this CTA finishes: 16 cells (x 4 gates forward)
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared-memory window starts at the same offset in every CTA of the cluster, so the aligned offsets
  // (and with them the addresses peers compute for each other's buffers and barriers) match as well
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  float *recv = reinterpret_cast<float *>(smem + SM::RECV_OFFSET);  // [S - 1 peers][128 rows][W]: partial sums pushed by the peers
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + SM::BAR_OFFSET);
  uint64_t *empty_bar = full_bar + STAGES;
  uint64_t *acc_full = empty_bar + STAGES;   // [MAX_ACC] accumulator a of the step is complete
  uint64_t *acc_empty = acc_full + SM::MAX_ACC;  // the 8 exchange warps have read tensor memory
  uint64_t *red_ready = acc_empty + 1;       // every exchange warp of every peer has pushed its partial sums for this CTA
  uint64_t *step_go = red_ready + 1;         // the producer has passed the step barrier
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(step_go + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
  float *peep_s = reinterpret_cast<float *>(smem + SM::BAR_OFFSET + 256);  // [3][16] peepholes of this CTA's cells

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int cluster_id = static_cast<int>(blockIdx.x) / S;
  const int tile_m = cluster_id / q.tiles_n, tile_n = cluster_id - tile_m * q.tiles_n;
  const int m0 = tile_m * 128, n0 = tile_n * BN;
  const int kb0 = min(static_cast<int>(rank) * q.kb_per, q.num_kb), kb1 = min(kb0 + q.kb_per, q.num_kb);
  const int my_kb = kb1 - kb0;
  const int acc_kb = max(SM::ACC_KB, (q.kb_per + SM::MAX_ACC - 1) / SM::MAX_ACC);  // K blocks per accumulator
  const int nacc = (my_kb + acc_kb - 1) / acc_kb;                                    // accumulators this CTA fills per step
  unsigned int *counter = q.sync + tile_m;
  unsigned int *abort_word = q.sync + q.tiles_m;
  const unsigned int per_step = static_cast<unsigned int>(q.tiles_n * S);  // CTAs that complete a row of tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < SM::MAX_ACC; ++a) ptx::mbar_init(&acc_full[a], 1);
    ptx::mbar_init(acc_empty, 8);
    ptx::mbar_init(red_ready, static_cast<uint32_t>(8 * (S - 1)));
    ptx::mbar_init(step_go, 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_holder, SM::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();  // every CTA's barriers exist before anyone signals across the cluster
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  uint32_t issued = 0;  // producer: K blocks staged so far (for the final drain)
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    ptx::reg_release<40>();
    if (lane == 0) {
      bool ok = true;
      for (int s = 1; s < q.T && ok; ++s) {
        // the panels this step reads: left by the kernels before this launch (s == 1) or by step s - 1 of this launch
        if (s > 1) {
          if (!wait_step_counter(counter, per_step * static_cast<unsigned int>(s - 1), abort_word, abort_flag)) { ok = false; break; }
          ptx::mbar_arrive_local(step_go);
        }
        ptx::fence_proxy_async_global();  // the other CTAs wrote them with ordinary stores; TMA reads through the async proxy
        const int a_row = ((s - 1) & 1) * static_cast<int>(q.a_rows) + m0;
        for (int kb = kb0; kb < kb1; ++kb, ++issued) {
          const int st = static_cast<int>(issued % STAGES);
          const uint32_t ph = (issued / STAGES) & 1u;
          if (!ptx::mbar_wait_or_abort(&empty_bar[st], ph ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t *dst = smem + st * SM::STAGE_BYTES;
          ptx::mbar_arrive_expect_tx(&full_bar[st], SM::STAGE_BYTES);
          ptx::tma_load_2d(dst, &tm_a_hi, &full_bar[st], kb * BK, a_row);
          ptx::tma_load_2d(dst + PS_TILE_BYTES, &tm_a_x, &full_bar[st], kb * BK, a_row);
          ptx::tma_load_2d(dst + 2 * PS_TILE_BYTES, &tm_b_hi, &full_bar[st], kb * BK, n0);
          ptx::tma_load_2d(dst + 2 * PS_TILE_BYTES + SM::B_BYTES, &tm_b_x, &full_bar[st], kb * BK, n0);
        }
      }
      if (!ok) {
        atomicCAS(q.error_flag, 0, 401);
        atomicExch(abort_word, 1u);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    ptx::reg_release<40>();
    if (lane == 0) {
      bool ok = true;
      constexpr uint32_t idesc_main = make_idesc_tf32(128, BN);
      constexpr uint32_t idesc_cross = make_idesc_bf16(128, BN);
      uint32_t it = 0;
      for (int s = 1; s < q.T && ok; ++s) {
        if (s > 1) {  // tensor memory still holds step s - 1 until the exchange warps have read it
          if (!ptx::mbar_wait_or_abort(acc_empty, static_cast<uint32_t>(s - 2) & 1u, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
        }
        int in_acc = 0, acc = 0;  // K blocks issued into the current accumulator, its index
        for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
          const int st = static_cast<int>(it % STAGES);
          const uint32_t ph = (it / STAGES) & 1u;
          if (!ptx::mbar_wait_or_abort(&full_bar[st], ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t base = ptx::smem_u32(smem + st * SM::STAGE_BYTES);
          const uint64_t a_hi = make_smem_desc(base), a_x = make_smem_desc(base + PS_TILE_BYTES);
          const uint64_t b_hi = make_smem_desc(base + 2 * PS_TILE_BYTES), b_x = make_smem_desc(base + 2 * PS_TILE_BYTES + SM::B_BYTES);
          const uint32_t t_acc = tmem_base + static_cast<uint32_t>(acc * BN);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t koff = static_cast<uint64_t>((k * UMMA_K * 4) >> 4);
            ptx::mma_bf16(t_acc, a_x + koff, b_x + koff, idesc_cross, (in_acc > 0 || k > 0) ? 1u : 0u);  // lo*hi + hi*lo
            ptx::mma_tf32(t_acc, a_hi + koff, b_hi + koff, idesc_main, 1u);                                  // hi*hi
          }
          ptx::tc_commit(&empty_bar[st]);
          if (++in_acc == acc_kb || kb + 1 == kb1) {
            ptx::tc_commit(&acc_full[acc]);
            ++acc;
            in_acc = 0;
          }
        }
      }
      if (!ok) {
        atomicCAS(q.error_flag, 0, 402);
        atomicExch(abort_word, 1u);
      }
    }
  } else if (warp >= PS_EPI_WARP0) {
    // ---------------- exchange + cell: 8 warps; tensor-memory lane quarter = warp % 4, half of the CTA's cells = (warp - 4) / 4 ----------------
    ptx::reg_acquire<232>();
    constexpr int HW = W / 2;   // this thread's columns of its CTA's share: 8 cells (x 4 gates forward)
    constexpr int CW = W / 4;   // 16-byte chunks per row of a receive slot
    static_assert((KIND == 1 ? BN / 4 : BN) / S == 16 && (HW == 32 || HW == 8), "16 cells per CTA, 8 per thread");
    const int qd = warp & 3, half = (warp - PS_EPI_WARP0) >> 2;
    const int row = qd * 32 + lane;
    const int swz = CW == 16 ? (row & 15) : ((row >> 1) & 3);  // chunk swizzle of the receive slots (bank conflicts)
    const long long b = static_cast<long long>(m0) + row;
    // a tile holds 32 cells x 4 gates (forward) or 64 cells (backward); this CTA finishes 16 of them, this thread 8
    const long long cta_cell0 = static_cast<long long>(tile_n) * (KIND == 1 ? BN / 4 : BN) + static_cast<long long>(rank) * 16;
    const long long cell0 = cta_cell0 + half * 8;
    const bool active = b < q.B && cell0 < q.C;
    const uint32_t recv_addr = ptx::smem_u32(recv);
    {  // the peepholes of this CTA's cells stay in shared memory for the whole walk
      const int i = static_cast<int>(threadIdx.x) - PS_EPI_WARP0 * 32;
      if (i < 48) {
        const long long cell = cta_cell0 + (i & 15);
        peep_s[i] = cell < q.C ? q.peep[static_cast<long long>(i >> 4) * q.C + cell] : 0.f;
      }
      ptx::named_barrier_sync(1, PS_EPI_THREADS);
    }
    using In = typename std::conditional<KIND == 1, LstmForwardIn, LstmBackwardIn>::type;
    using Out = typename std::conditional<KIND == 1, LstmForwardOut, LstmBackwardOut>::type;
    Out out;               // results of the step before; its arrays are written once the step barrier has been passed
    bool pending = false;
    auto store_arrays = [&](int step) {
      const LstmStep pp = step_view<KIND>(q, step);
      if constexpr (KIND == 1) lstm_forward_store_arrays8(pp, out, b, cell0);
      else lstm_backward_store_arrays8(pp, out, b, cell0);
    };
    for (int s = 1; s < q.T; ++s) {
      bool ok = true;
      const LstmStep p = step_view<KIND>(q, s);
      In in;
      if (active) {
        // what the cell needs from global memory goes out before any wait; what this thread computed itself in the step
        // before (and has not written yet) comes from its registers
        if (!pending) {
          if constexpr (KIND == 1) lstm_forward_load8<true, false>(p, in, b, cell0);
          else lstm_backward_load8<true, false>(p, in, b, cell0);
        } else {
          if constexpr (KIND == 1) {
            lstm_forward_load8<false, false>(p, in, b, cell0);
#pragma unroll
            for (int i = 0; i < 8; ++i) { in.cp[i] = out.cs[i]; in.hp[i] = out.h[i]; }
          } else {
            lstm_backward_load8<false, false>(p, in, b, cell0);
#pragma unroll
            for (int i = 0; i < 8; ++i) { in.dni[i] = out.di[i]; in.dnf[i] = out.df[i]; in.dcn[i] = out.dc[i]; }
          }
        }
      }
      if (pending) {
        // the arrays of step s - 1 (read by later kernels only) leave now, beside this step's operand stream, and not
        // while the step barrier is in flight: 128 CTAs storing at once slowed the barrier down by microseconds
        if (!ptx::mbar_wait_or_abort(step_go, static_cast<uint32_t>(s - 2) & 1u, abort_flag)) ok = false;
        if (ok && active) store_arrays(s - 1);
        pending = false;
      }
      // Partial sums of this CTA's K slice: for every CTA d of the cluster the columns of d's cells that belong to this
      // thread's (row, half), added up over the accumulators as the tensor core completes them (part[S - 1] is this
      // CTA's own share, the others go to the peers in the order rank + 1, rank + 2, ...)
      float part[S][HW];
#pragma unroll
      for (int dd = 0; dd < S; ++dd)
#pragma unroll
        for (int j = 0; j < HW; ++j) part[dd][j] = 0.f;
      for (int a = 0; a < nacc && ok; ++a) {
        if (!ptx::mbar_wait_or_abort(&acc_full[a], static_cast<uint32_t>(s - 1) & 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
#pragma unroll
        for (int dd = 1; dd <= S; ++dd) {
          const int d = (static_cast<int>(rank) + dd) % S;
          uint32_t r[HW];
          const uint32_t t0 = tmem_base + (static_cast<uint32_t>(qd * 32) << 16) + static_cast<uint32_t>(a * BN + d * W + half * HW);
          if constexpr (HW == 32) ptx::tmem_ld_32x32(t0, r);
          else ptx::tmem_ld_32x8(t0, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < HW; ++j) part[dd - 1][j] += __uint_as_float(r[j]);
        }
      }
      if (ok) {
        // the peers' shares are pushed into their receive slots, this CTA's own share stays in registers
#pragma unroll
        for (int dd = 1; dd < S; ++dd) {
          const int d = (static_cast<int>(rank) + dd) % S;
          const int slot = static_cast<int>(rank) < d ? static_cast<int>(rank) : static_cast<int>(rank) - 1;
          const uint32_t dst = ptx::map_to_cta(recv_addr + static_cast<uint32_t>((slot * 128 + row) * W * 4), static_cast<uint32_t>(d));
#pragma unroll
          for (int i = 0; i < HW / 4; ++i)
            ptx::st_cluster_f4(dst + (static_cast<uint32_t>((half * (HW / 4) + i) ^ swz) << 4),
                               make_float4(part[dd - 1][4 * i], part[dd - 1][4 * i + 1], part[dd - 1][4 * i + 2], part[dd - 1][4 * i + 3]));
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive_local(acc_empty);
#pragma unroll
          for (int dd = 1; dd < S; ++dd) ptx::mbar_arrive_release_cluster(red_ready, (rank + static_cast<uint32_t>(dd)) % S);
        }
        if (!ptx::mbar_wait_cluster_or_abort(red_ready, static_cast<uint32_t>(s - 1) & 1u, abort_flag)) ok = false;
      }
      if (ok) {
        // the sums over the K slices, added in slice order whichever CTA adds them (bitwise repeatable)
        float rec[HW];
#pragma unroll
        for (int i = 0; i < HW; ++i) rec[i] = 0.f;
#pragma unroll
        for (int j = 0; j < S; ++j) {
          if (j == static_cast<int>(rank)) {
#pragma unroll
            for (int i = 0; i < HW; ++i) rec[i] += part[S - 1][i];
          } else {
            const int slot = j < static_cast<int>(rank) ? j : j - 1;
            const float *src = recv + (slot * 128 + row) * W;
            float4 v[HW / 4];
#pragma unroll
            for (int i = 0; i < HW / 4; ++i) v[i] = *reinterpret_cast<const float4 *>(src + (((half * (HW / 4) + i) ^ swz) << 2));
#pragma unroll
            for (int i = 0; i < HW / 4; ++i) { rec[4 * i] += v[i].x; rec[4 * i + 1] += v[i].y; rec[4 * i + 2] += v[i].z; rec[4 * i + 3] += v[i].w; }
          }
        }
        if (active) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { in.pi[i] = peep_s[half * 8 + i]; in.pf[i] = peep_s[16 + half * 8 + i]; in.po[i] = peep_s[32 + half * 8 + i]; }
          // the cell; only what the NEXT step's contraction reads (the operand panels) leaves before the step barrier
          if constexpr (KIND == 1) {
            lstm_forward_compute8(in, rec, out);
            lstm_forward_store_panels8(p, out, b, cell0);
          } else {
            lstm_backward_compute8(in, rec, p.b_c_prev != nullptr, out);
            lstm_backward_store_panels8(p, out, b, cell0);
          }
        }
        // this thread's panel stores come before the TMA copies that the step barrier lets loose (generic -> async proxy)
        ptx::fence_proxy_async_global();
        pending = true;
      }
      if (!ok && lane == 0) {
        atomicCAS(q.error_flag, 0, 403);
        atomicExch(abort_word, 1u);
      }
      // the 8 warps stay in step and leave together: the barrier returns the OR of what each thread saw of the CTA's
      // abort flag (a warp that gave up has set it before it gets here), the same answer in every thread
      if (ptx::named_barrier_or(1, PS_EPI_THREADS, *abort_flag != 0)) { pending = false; break; }
      // the barrier above ordered every thread's panel stores before this thread; its release makes them visible to
      // the GPU together with the count
      if (warp == PS_EPI_WARP0 && lane == 0) red_release_gpu_add(counter, 1u);
    }
    if (pending && active) store_arrays(q.T - 1);
  } else {
    ptx::reg_release<40>();  // warps 2-3: no role, but the whole warpgroup has to give its registers back
  }

  // the producer makes sure none of its copies is still in flight before the CTA's shared memory goes away
  if (warp == 0 && lane == 0) {
    const uint32_t first = issued > static_cast<uint32_t>(STAGES) ? issued - STAGES : 0u;
    for (uint32_t i = first; i < issued; ++i) {
      if (!ptx::mbar_wait(&full_bar[i % STAGES], (i / STAGES) & 1u)) break;
    }
  }
  // peers may still be pushing into this CTA's receive slots or signalling its barriers: the cluster stays together until
  // everybody is here
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, SM::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
struct LstmPersistent {
  bool ready = false;
  int tiles_m = 0;
  long long a_rows = 0;
  unsigned int *sync = nullptr;  // [tiles_m + 1]
};

template <int KIND>
static int resident_clusters(int device) {
  constexpr int split = PsShape<KIND>::SPLIT;
  constexpr int PS_SMEM_TOTAL = PsSmem<KIND>::TOTAL;
  // clusters of `split` CTAs that fit the device at once; configured once per device (the shared-memory opt-in is a
  // per-device attribute of the kernel)
  static std::mutex mutex;
  static int cached[64] = {};
  if (device < 0 || device >= 64) return 0;
  std::lock_guard<std::mutex> lock(mutex);
  if (cached[device] != 0) return cached[device];
  auto kernel = lstm_persistent_kernel<KIND>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PS_SMEM_TOTAL) != cudaSuccess) { cudaGetLastError(); return 0; }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sms / split * split));
  cfg.blockDim = dim3(PS_THREADS);
  cfg.dynamicSmemBytes = PS_SMEM_TOTAL;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(split);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  cached[device] = n > 0 ? n : -1;
  return cached[device];
}

int lstm_persistent_plan(myea_b200_net *net, LayerPlan &L) {
  LstmPlan *P = L.lstm;
  P->persist = nullptr;
  if (!P->fuse || net->T < 2) return MYEA_OK;
  const long long B = net->B, C = P->C;
  const int tiles_m = static_cast<int>((B + 127) / 128);
  const long long fwd_clusters = tiles_m * ((4 * C + PsShape<1>::BN - 1) / PsShape<1>::BN), bwd_clusters = tiles_m * ((C + PsShape<2>::BN - 1) / PsShape<2>::BN);
  const int fit_f = resident_clusters<1>(net->ctx.device), fit_b = resident_clusters<2>(net->ctx.device);
  if (fwd_clusters > fit_f || bwd_clusters > fit_b) return MYEA_OK;  // the CTAs of a launch wait for each other: all of them have to fit
  LstmPersistent *ps = new LstmPersistent();
  ps->tiles_m = tiles_m;
  ps->a_rows = static_cast<long long>(tiles_m) * 128;
  void *q = nullptr;
  if (cudaMalloc(&q, (tiles_m + 1) * sizeof(unsigned int)) != cudaSuccess) { delete ps; net->ctx.error = "cudaMalloc failed (LSTM step counters)"; return MYEA_E_CUDA; }
  net->allocations.push_back(q);
  ps->sync = static_cast<unsigned int *>(q);
  ps->ready = true;
  P->persist = ps;
  return MYEA_OK;
}

void lstm_persistent_destroy(LstmPlan *P) {
  if (P != nullptr) { delete P->persist; P->persist = nullptr; }
}

bool lstm_persistent_ready(const LstmPlan *P) { return P != nullptr && P->persist != nullptr && P->persist->ready; }

template <int KIND>
static int launch(myea_b200_net *net, LstmSeq &q, const float *a_hi, const float *a_cross, long long K, const Panels &w) {
  Context &ctx = net->ctx;
  CUtensorMap maps[4];
  // operand panels: both ping-pong buffers in one map (row coordinate = buffer * a_rows + tile row); weights: one box of
  // 128 panel rows per tile of output columns
  if (!make_panel_map(&maps[0], a_hi, 2 * q.a_rows, K, q.kpa, 128) || !make_panel_map(&maps[1], a_cross, 2 * q.a_rows, K, q.kpa, 128) ||
      !make_panel_map(&maps[2], w.hi, w.rows, w.k, w.kp, PsShape<KIND>::BN) || !make_panel_map(&maps[3], w.lo, w.rows, w.k, w.kp, PsShape<KIND>::BN))
    return MYEA_E_CUDA;
  if (cudaMemsetAsync(q.sync, 0, (q.tiles_m + 1) * sizeof(unsigned int), ctx.stream) != cudaSuccess) return MYEA_E_CUDA;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(q.tiles_m * q.tiles_n * q.split));
  cfg.blockDim = dim3(PS_THREADS);
  cfg.dynamicSmemBytes = PsSmem<KIND>::TOTAL;
  cfg.stream = ctx.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(q.split);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  ctx.begin(TC_GEMM);
  const cudaError_t err = cudaLaunchKernelEx(&cfg, lstm_persistent_kernel<KIND>, maps[0], maps[1], maps[2], maps[3], q);
  ctx.end(TC_GEMM);
  ctx.gemm_flops += 2.0 * q.B * 4.0 * q.C * q.C * (q.T - 1);
  return err == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

int lstm_persistent_forward(myea_b200_net *net, LayerPlan &L, int dir, const Panels &w_rec_interleaved, const float *peep_compact, bool zoneout) {
  LstmPlan *P = L.lstm;
  if (!lstm_persistent_ready(P)) return MYEA_E_UNSUPPORTED;
  const LstmDir &D = P->d[dir];
  LstmSeq q;
  q.T = static_cast<int>(net->T); q.B = static_cast<int>(net->B); q.C = static_cast<int>(P->C);
  q.reverse = dir;
  q.tiles_m = P->persist->tiles_m;
  q.tiles_n = static_cast<int>((4 * P->C + PsShape<1>::BN - 1) / PsShape<1>::BN);
  q.split = PsShape<1>::SPLIT;
  q.num_kb = static_cast<int>((P->C + BK - 1) / BK);
  q.kb_per = (q.num_kb + q.split - 1) / q.split;
  q.ldh = L.n_out;
  q.a_rows = P->persist->a_rows;
  q.kpa = P->h_pan[0].kp;
  q.a_hi = P->h_pan[0].hi; q.a_cross = P->h_pan[0].lo;
  q.peep = peep_compact;
  q.gates_in = D.gates_in; q.act = D.act; q.cstate = D.cstate; q.cact = D.cact;
  q.values = L.values + dir * P->C;
  q.zone_state = zoneout ? D.zone_state : nullptr;
  q.zone_output = zoneout ? D.zone_output : nullptr;
  q.sync = P->persist->sync;
  q.error_flag = net->ctx.d_error_flag;
  return launch<1>(net, q, q.a_hi, q.a_cross, P->C, w_rec_interleaved);
}

int lstm_persistent_backward(myea_b200_net *net, LayerPlan &L, int dir, const Panels &w_rec_transposed, const float *peep_compact) {
  LstmPlan *P = L.lstm;
  if (!lstm_persistent_ready(P)) return MYEA_E_UNSUPPORTED;
  const LstmDir &D = P->d[dir];
  const long long Cp = (P->C + 7) & ~7ll;
  LstmSeq q;
  q.T = static_cast<int>(net->T); q.B = static_cast<int>(net->B); q.C = static_cast<int>(P->C);
  q.reverse = dir;
  q.tiles_m = P->persist->tiles_m;
  q.tiles_n = static_cast<int>((P->C + PsShape<2>::BN - 1) / PsShape<2>::BN);
  q.split = PsShape<2>::SPLIT;
  q.num_kb = static_cast<int>((4 * Cp + BK - 1) / BK);
  q.kb_per = (q.num_kb + q.split - 1) / q.split;
  q.ldh = L.n_out;
  q.a_rows = P->persist->a_rows;
  q.kpa = P->dg_pan[0].kp;
  q.Cp = Cp;
  q.a_hi = P->dg_pan[0].hi; q.a_cross = P->dg_pan[0].lo;
  q.peep = peep_compact;
  q.act = D.act; q.cstate = D.cstate; q.cact = D.cact;
  q.deriv = L.deriv + dir * P->C;
  q.dgates = D.dgates; q.dcstate = D.dcstate;
  q.sync = P->persist->sync;
  q.error_flag = net->ctx.d_error_flag;
  return launch<2>(net, q, q.a_hi, q.a_cross, 4 * Cp, w_rec_transposed);
}

}  // namespace myea

// Diagnostic (not part of the training interface): how many clusters of the two persistent kernels the device holds at
// once; a layer runs persistently when its tiles fit (see lstm_persistent_plan).
extern "C" int myea_b200_lstm_resident_clusters(int device, int *forward_pairs, int *backward_quads) {
  if (cudaSetDevice(device) != cudaSuccess) return MYEA_E_CUDA;
  if (forward_pairs) *forward_pairs = myea::resident_clusters<1>(device);
  if (backward_quads) *backward_quads = myea::resident_clusters<2>(device);
  return MYEA_OK;
}
