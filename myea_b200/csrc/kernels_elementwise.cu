// Bandwidth-bound kernels of the feed-forward training step: batch (re)normalization forward statistics and backward
// reductions, activation + dropout application, softmax, output error with loss / accuracy accumulation, column sums
// for the bias derivatives.  All of them stream [rows, H] row-major fp32 tensors with 128-bit accesses where the
// shape allows and reduce over rows with per-thread partial sums, a shared-memory tree and a second small pass.
#include "common.cuh"
#include "panel_math.cuh"

#include <algorithm>

namespace myea {

// ---------------------------------------------------------------------------------------------------------
// Column reductions over the rows of a [rows, H] tensor.
// grid = (column groups, row chunks); block = 32 column lanes x 8 row lanes; each column lane owns VEC adjacent
// columns.  Row chunk c of column j lands in partial[which][c][j]; a finalize kernel adds the chunks.
// ---------------------------------------------------------------------------------------------------------
enum ReduceKind { RK_SUM_SQ = 0, RK_NORM_BWD = 1, RK_SUM = 2 };

template <int VEC, int KIND>
__global__ void __launch_bounds__(256) column_reduce_kernel(const float *__restrict__ x, const float *__restrict__ y,
                                                            const float *__restrict__ mean, long long rows, long long H,
                                                            int chunks, float *__restrict__ partial) {
  __shared__ float s0[8][32 * VEC + 1];
  __shared__ float s1[8][32 * VEC + 1];
  const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const long long col = (static_cast<long long>(blockIdx.x) * 32 + cl) * VEC;
  const long long rows_per_chunk = (rows + chunks - 1) / chunks;
  const long long r_begin = blockIdx.y * rows_per_chunk;
  const long long r_end = min(rows, r_begin + rows_per_chunk);
  float a0[VEC], a1[VEC], mu[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) { a0[v] = 0.f; a1[v] = 0.f; mu[v] = 0.f; }
  const bool active = col < H;
  if (active && KIND == RK_NORM_BWD) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) mu[v] = mean[col + v];
  }
  if (active) {
    // four rows per trip so that four (eight with a second array) 16-byte loads are in flight per thread
#pragma unroll 4
    for (long long r = r_begin + rl; r < r_end; r += 8) {
      float xv[VEC], yv[VEC];
      if (VEC == 4) {
        const float4 t = *reinterpret_cast<const float4 *>(x + r * H + col);
        xv[0] = t.x; xv[1] = t.y; xv[2] = t.z; xv[3] = t.w;
        if (KIND == RK_NORM_BWD) {
          const float4 u = *reinterpret_cast<const float4 *>(y + r * H + col);
          yv[0] = u.x; yv[1] = u.y; yv[2] = u.z; yv[3] = u.w;
        }
      } else {
        xv[0] = x[r * H + col];
        if (KIND == RK_NORM_BWD) yv[0] = y[r * H + col];
      }
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        if (KIND == RK_SUM_SQ) { a0[v] += xv[v]; a1[v] = fmaf(xv[v], xv[v], a1[v]); }
        if (KIND == RK_NORM_BWD) { a0[v] += yv[v]; a1[v] = fmaf(yv[v], xv[v] - mu[v], a1[v]); }  // x = z, y = delta
        if (KIND == RK_SUM) { a0[v] += xv[v]; }
      }
    }
  }
#pragma unroll
  for (int v = 0; v < VEC; ++v) { s0[rl][cl * VEC + v] = a0[v]; s1[rl][cl * VEC + v] = a1[v]; }
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * VEC; i += 256) {
    const long long c = static_cast<long long>(blockIdx.x) * 32 * VEC + i;
    if (c < H) {
      float t0 = 0.f, t1 = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) { t0 += s0[r][i]; t1 += s1[r][i]; }
      partial[(0ll * chunks + blockIdx.y) * H + c] = t0;
      if (KIND != RK_SUM) partial[(1ll * chunks + blockIdx.y) * H + c] = t1;
    }
  }
}

static int pick_chunks(long long rows, long long H, int vec, int max_chunks) {
  const long long groups = (H + 32 * vec - 1) / (32 * vec);
  long long c = (148 * 4 + groups - 1) / groups;
  c = std::min<long long>(c, std::max<long long>(1, rows / 16));
  c = std::min<long long>(c, max_chunks);
  return static_cast<int>(std::max<long long>(1, c));
}

template <int KIND>
static void launch_column_reduce(Context &ctx, const float *x, const float *y, const float *mean, long long rows, long long H,
                                 int chunks, float *partial) {
  const bool vec4 = (H % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && (y == nullptr || (reinterpret_cast<uintptr_t>(y) & 15) == 0);
  if (vec4) {
    dim3 grid(static_cast<unsigned>((H + 127) / 128), chunks);
    column_reduce_kernel<4, KIND><<<grid, 256, 0, ctx.stream>>>(x, y, mean, rows, H, chunks, partial);
  } else {
    dim3 grid(static_cast<unsigned>((H + 31) / 32), chunks);
    column_reduce_kernel<1, KIND><<<grid, 256, 0, ctx.stream>>>(x, y, mean, rows, H, chunks, partial);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Normalization forward: statistics -> per-column affine map  y = z * col_scale + col_shift
// Forward_Pass__Batch_Normalization__Training / …Batch_Renormalization__Training
// (Neural_Network__Forward_Pass__OpenMP.cpp:4591-4701, 4703-4837), inference :4559-4589.
// The "variance" buffers of the reference hold the standard deviation sqrt(E[x^2] - mean^2 + eps); the running
// averages are exponential averages of mean and standard deviation; r and d use the ALREADY UPDATED averages.
// ---------------------------------------------------------------------------------------------------------
// The two column sums of partial[2][chunks][H] for column j = blockIdx.x * 32 + (threadIdx.x & 31): blocks of 256
// threads = 32 columns x 8 chunk lanes (the contractions' epilogues leave one chunk per 32 rows: 128 of them for a batch
// of 4096, too many for one thread per column to walk alone).  Valid in the threads with threadIdx.x < 32.
__device__ __forceinline__ void chunk_sums(const float *__restrict__ partial, int chunks, long long H, long long j, float &s, float &q) {
  __shared__ float sh[2][8][33];
  const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
  float a = 0.f, b = 0.f;
  if (j < H) {
#pragma unroll 4
    for (int c = rl; c < chunks; c += 8) { a += partial[(0ll * chunks + c) * H + j]; b += partial[(1ll * chunks + c) * H + j]; }
  }
  sh[0][rl][cl] = a;
  sh[1][rl][cl] = b;
  __syncthreads();
  s = 0.f; q = 0.f;
  if (rl == 0) {
#pragma unroll
    for (int r = 0; r < 8; ++r) { s += sh[0][r][cl]; q += sh[1][r][cl]; }
  }
}

// sums[2][H] = chunk sums of partial[2][chunks][H]: the message of the cross-GPU all-reduce
__global__ void __launch_bounds__(256) chunk_sum_kernel(const float *__restrict__ partial, int chunks, long long H, float *__restrict__ sums) {
  const long long j = blockIdx.x * 32ll + (threadIdx.x & 31);
  float s, q;
  chunk_sums(partial, chunks, H, j, s, q);
  if (threadIdx.x >= 32 || j >= H) return;
  sums[j] = s;
  sums[H + j] = q;
}

// `rows` is the batch the statistics are taken over: the global batch when the column sums were all-reduced (chunks == 1
// then, partial = the reduced [2][H] sums).
__global__ void __launch_bounds__(256) norm_stats_finalize_kernel(const float *__restrict__ partial, int chunks, long long rows, long long H,
                                                                  NormParams np, int training) {
  const long long j = blockIdx.x * 32ll + (threadIdx.x & 31);
  float s = 0.f, q = 0.f;
  if (training) chunk_sums(partial, chunks, H, j, s, q);
  if (threadIdx.x >= 32 || j >= H) return;
  float mean, sigma, r = 1.f, d = 0.f;
  if (training) {
    const float scale = 1.0f / static_cast<float>(rows);
    mean = s * scale;
    sigma = sqrtf(q * scale - mean * mean + np.epsilon);
    float ma = np.mean_avg[j], sa = np.sigma_avg[j];
    ma += np.momentum * (mean - ma);
    sa += np.momentum * (sigma - sa);
    np.mean_avg[j] = ma;
    np.sigma_avg[j] = sa;
    if (np.type == MYEA_NORM_BATCH_RENORMALIZATION) {
      r = fminf(fmaxf(sigma / sa, 1.0f / np.r_max), np.r_max);
      d = fminf(fmaxf((mean - ma) / sa, -np.d_max), np.d_max);
    }
    np.mean[j] = mean;
    np.sigma[j] = sigma;
    np.r[j] = r;
    np.d[j] = d;
  } else {
    mean = np.mean_avg[j];
    sigma = np.sigma_avg[j];
  }
  const float g = np.gamma[j], b = np.beta[j];
  const float k = r / sigma;
  np.col_scale[j] = g * k;
  np.col_shift[j] = b + g * (d - mean * k);
}

int norm_forward_stats(Context &ctx, const float *z, long long rows, long long H, const NormParams &np, int training,
                       const SumHook *hook, const OverlapWork *meanwhile, int fused_chunks) {
  ctx.begin(TC_NORM);
  int launches = 1;
  int chunks = 1;
  const float *sums = np.partial;
  long long rows_total = rows;
  if (training) {
    if (fused_chunks > 0) {
      chunks = fused_chunks;  // the contraction's epilogue has left the sums of every 32-row block in np.partial
    } else {
      chunks = pick_chunks(rows, H, (H % 4 == 0) ? 4 : 1, np.chunks);
      launch_column_reduce<RK_SUM_SQ>(ctx, z, nullptr, nullptr, rows, H, chunks, np.partial);
      ++launches;
    }
    if (hook != nullptr && hook->world > 1) {
      // sharded batch: sum the column sums over the ranks, then every rank finalizes the same global statistics
      float *g = np.partial + 2ll * np.chunks * H + 3 * H;
      chunk_sum_kernel<<<static_cast<unsigned>((H + 31) / 32), 256, 0, ctx.stream>>>(np.partial, chunks, H, g);
      ctx.end(TC_NORM, launches + 1);
      if (hook->begin != nullptr && hook->end != nullptr && meanwhile != nullptr && meanwhile->run != nullptr && !ctx.profiling) {
        // the exchange is pure latency (a few KB): queue the caller's independent work beside it
        if (hook->begin(hook->user, g, static_cast<size_t>(2 * H)) != MYEA_OK) return MYEA_E_COMM;
        const int rc = meanwhile->run(meanwhile->arg);
        if (hook->end(hook->user) != MYEA_OK) return MYEA_E_COMM;
        if (rc != MYEA_OK) return rc;
      } else if (hook->all_reduce(hook->user, g, static_cast<size_t>(2 * H)) != MYEA_OK) {
        return MYEA_E_COMM;
      }
      ctx.begin(TC_NORM);
      launches = 1;
      sums = g;
      chunks = 1;
      rows_total = rows * hook->world;
    }
  }
  norm_stats_finalize_kernel<<<static_cast<unsigned>((H + 31) / 32), 256, 0, ctx.stream>>>(sums, chunks, rows_total, H, np, training);
  ctx.end(TC_NORM, launches);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// ---------------------------------------------------------------------------------------------------------
// Activation (+ folded normalization) + dropout mask, one pass:  out = mask(f(z * col_scale + col_shift))
// Forward_Pass__FC_AF (…Forward_Pass__OpenMP.cpp:4839-4868), Forward_Pass__Dropout__Bernoulli__Inverted (:4907-4938)
// and …Bernoulli__Training (:4940-4966).  The mask holds one byte per UNIT and is shared by every row of the batch.
// ---------------------------------------------------------------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(256) activation_forward_kernel(const float *__restrict__ z, float *__restrict__ out, long long rows,
                                                                 long long H, uint32_t af, const float *__restrict__ col_scale,
                                                                 const float *__restrict__ col_shift,
                                                                 const uint8_t *__restrict__ mask, float keep_scale) {
  const long long hv = H / VEC;
  const long long total = rows * hv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / hv;
    const long long c = (i - r * hv) * VEC;
    float v[VEC];
    if (VEC == 4) {
      const float4 t = *reinterpret_cast<const float4 *>(z + r * H + c);
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
      v[0] = z[r * H + c];
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float pre = v[k];
      if (col_scale != nullptr) pre = pre * col_scale[c + k] + col_shift[c + k];
      float y = af_fire(af, pre);
      if (mask != nullptr) y = mask[c + k] ? y * keep_scale : 0.f;
      else if (keep_scale != 1.0f) y *= keep_scale;   // inference of plain Bernoulli dropout: every unit times p
      v[k] = y;
    }
    if (VEC == 4) {
      *reinterpret_cast<float4 *>(out + r * H + c) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      out[r * H + c] = v[0];
    }
  }
}

// The same for H a multiple of 4 and 16-byte aligned arrays: a thread keeps four COLUMNS (affine coefficients and mask
// bytes loaded once) and walks rows four at a time with the four loads in flight; the activation is a template
// argument, so no switch is left in the loop.  Grid: x = column groups of 1024, y = row walkers.
template <uint32_t AF>
__global__ void __launch_bounds__(256) activation_forward_cols_kernel(const float *__restrict__ z, float *__restrict__ out, long long rows,
                                                                      long long H, const float *__restrict__ col_scale,
                                                                      const float *__restrict__ col_shift, const uint8_t *__restrict__ mask,
                                                                      float keep_scale) {
  const long long c = (blockIdx.x * 256ll + threadIdx.x) * 4;
  if (c >= H) return;
  const bool affine = col_scale != nullptr;
  const float4 cs = affine ? *reinterpret_cast<const float4 *>(col_scale + c) : make_float4(1.f, 1.f, 1.f, 1.f);
  const float4 ch = affine ? *reinterpret_cast<const float4 *>(col_shift + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  const bool masked = mask != nullptr;
  const bool k0 = !masked || mask[c] != 0, k1 = !masked || mask[c + 1] != 0, k2 = !masked || mask[c + 2] != 0, k3 = !masked || mask[c + 3] != 0;
  const bool scale = masked || keep_scale != 1.0f;  // kept units of a training mask, or every unit at inference of plain Bernoulli dropout
  for (long long r0 = blockIdx.y * 4ll; r0 < rows; r0 += gridDim.y * 4ll) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (r0 + u < rows) v[u] = *reinterpret_cast<const float4 *>(z + (r0 + u) * H + c);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (r0 + u >= rows) break;
      float4 y;
      y.x = af_fire(AF, affine ? v[u].x * cs.x + ch.x : v[u].x);
      y.y = af_fire(AF, affine ? v[u].y * cs.y + ch.y : v[u].y);
      y.z = af_fire(AF, affine ? v[u].z * cs.z + ch.z : v[u].z);
      y.w = af_fire(AF, affine ? v[u].w * cs.w + ch.w : v[u].w);
      if (scale) { y.x *= keep_scale; y.y *= keep_scale; y.z *= keep_scale; y.w *= keep_scale; }
      if (!k0) y.x = 0.f;
      if (!k1) y.y = 0.f;
      if (!k2) y.z = 0.f;
      if (!k3) y.w = 0.f;
      *reinterpret_cast<float4 *>(out + (r0 + u) * H + c) = y;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Producers that also write their result as operand panels (see PanelSink): the contraction that reads the tensor next
// then needs no split pass of its own.  A thread keeps EIGHT columns (one group of the cross panels) and walks rows.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void write_panels8(const PanelSink &s, long long r, long long c, const float (&v)[8]) {
  float h[8];
  uint32_t x[8];
  split_group(v, s.role_k, 0, h, x);
  store8(s.hi + r * s.kp + c, h);
  if (s.cross_k != nullptr) {
    uint4 *px = reinterpret_cast<uint4 *>(s.cross_k + r * s.kp + c);
    px[0] = make_uint4(x[0], x[1], x[2], x[3]);
    px[1] = make_uint4(x[4], x[5], x[6], x[7]);
  }
  if (s.cross_mn != nullptr) {
    // x[0..3] / x[4..7] are the packed lo and hi values of these 8 columns in the order of role_k; the column reading
    // wants, per 8 source rows, 8 panel rows of lo and 8 of hi (role A) or hi then lo (role B)
    const uint4 lo4 = s.role_k ? make_uint4(x[4], x[5], x[6], x[7]) : make_uint4(x[0], x[1], x[2], x[3]);
    const uint4 hi4 = s.role_k ? make_uint4(x[0], x[1], x[2], x[3]) : make_uint4(x[4], x[5], x[6], x[7]);
    const long long g16 = (r >> 3) * 16 + (r & 7);
    const long long row_lo = g16 + (s.role_mn ? 8 : 0), row_hi = g16 + (s.role_mn ? 0 : 8);
    *reinterpret_cast<uint4 *>(s.cross_mn + row_lo * s.kp + c) = lo4;
    *reinterpret_cast<uint4 *>(s.cross_mn + row_hi * s.kp + c) = hi4;
  }
}

template <uint32_t AF>
__global__ void __launch_bounds__(256) activation_forward_panels_kernel(const float *__restrict__ z, float *__restrict__ out, long long rows,
                                                                        long long H, const float *__restrict__ col_scale,
                                                                        const float *__restrict__ col_shift, const uint8_t *__restrict__ mask,
                                                                        float keep_scale, const PanelSink sink) {
  const long long c = (blockIdx.x * 256ll + threadIdx.x) * 8;
  if (c >= H) return;
  const bool affine = col_scale != nullptr;
  float cs[8], ch[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) { cs[k] = affine ? col_scale[c + k] : 1.f; ch[k] = affine ? col_shift[c + k] : 0.f; }
  const bool masked = mask != nullptr;
  const unsigned long long keep = masked ? *reinterpret_cast<const unsigned long long *>(mask + c) : ~0ull;
  const bool scale = masked || keep_scale != 1.0f;
  for (long long r0 = blockIdx.y * 2ll; r0 < rows; r0 += gridDim.y * 2ll) {
    float v[2][8];
#pragma unroll
    for (int u = 0; u < 2; ++u)
      if (r0 + u < rows) load8(v[u], z + (r0 + u) * H + c);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (r0 + u >= rows) break;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float y = af_fire(AF, affine ? v[u][k] * cs[k] + ch[k] : v[u][k]);
        if (scale) y *= keep_scale;
        if (((keep >> (8 * k)) & 0xFFull) == 0ull) y = 0.f;
        v[u][k] = y;
      }
      store8(out + (r0 + u) * H + c, v[u]);
      write_panels8(sink, r0 + u, c, v[u]);
    }
  }
}

__global__ void __launch_bounds__(256) norm_backward_apply_panels_kernel(const float *__restrict__ z, const float *__restrict__ delta,
                                                                         float *__restrict__ out, long long rows, long long H,
                                                                         const float *__restrict__ mean, const float *__restrict__ coef,
                                                                         const PanelSink sink) {
  const long long c = (blockIdx.x * 256ll + threadIdx.x) * 8;
  if (c >= H) return;
  float mu[8], k0[8], k1[8], k2[8];
  load8(mu, mean + c); load8(k0, coef + c); load8(k1, coef + H + c); load8(k2, coef + 2 * H + c);
  for (long long r0 = blockIdx.y * 2ll; r0 < rows; r0 += gridDim.y * 2ll) {
    float t[2][8], u[2][8];
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (r0 + i < rows) { load8(t[i], z + (r0 + i) * H + c); load8(u[i], delta + (r0 + i) * H + c); }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (r0 + i >= rows) break;
      float d[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) d[k] = u[i][k] * k0[k] + (t[i][k] - mu[k]) * k1[k] + k2[k];
      store8(out + (r0 + i) * H + c, d);
      write_panels8(sink, r0 + i, c, d);
    }
  }
}

static dim3 column_walk_grid8(long long rows, long long H) {
  const unsigned gx = static_cast<unsigned>((H / 8 + 255) / 256);
  const long long walkers = std::max<long long>(1, (148 * 8) / gx);
  return dim3(gx, static_cast<unsigned>(std::max<long long>(1, std::min<long long>((rows + 1) / 2, walkers))));
}

static dim3 column_walk_grid(long long rows, long long H) {
  const unsigned gx = static_cast<unsigned>((H / 4 + 255) / 256);
  const long long walkers = std::max<long long>(1, (148 * 8) / gx);
  return dim3(gx, static_cast<unsigned>(std::max<long long>(1, std::min<long long>((rows + 3) / 4, walkers))));
}

// the functions whose kernel can also write the next contraction's operand panels
bool activation_writes_panels(uint32_t af) {
  switch (af) {
    case MYEA_AF_TANH: case MYEA_AF_SIGMOID: case MYEA_AF_RELU: case MYEA_AF_LEAKY_RELU: case MYEA_AF_ELU: case MYEA_AF_SELU: case MYEA_AF_LINEAR: return true;
    default: return false;
  }
}

int activation_forward(Context &ctx, const float *z, float *out, long long rows, long long H, uint32_t af, const float *col_scale,
                       const float *col_shift, const uint8_t *mask, float keep_scale, const PanelSink *sink) {
  ctx.begin(TC_ELEMENTWISE);
  const bool vec4 = (H % 4 == 0) && ((reinterpret_cast<uintptr_t>(z) & 15) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                    ((reinterpret_cast<uintptr_t>(col_scale) & 15) == 0) && ((reinterpret_cast<uintptr_t>(col_shift) & 15) == 0);
  if (sink != nullptr) {
    if (!vec4 || (H & 7) != 0 || (rows & 7) != 0) return MYEA_E_INVALID;
    const dim3 grid = column_walk_grid8(rows, H);
#define MYEA_AF_CASE(A) case A: activation_forward_panels_kernel<A><<<grid, 256, 0, ctx.stream>>>(z, out, rows, H, col_scale, col_shift, mask, keep_scale, *sink); break
    switch (af) {
      MYEA_AF_CASE(MYEA_AF_TANH);
      MYEA_AF_CASE(MYEA_AF_SIGMOID);
      MYEA_AF_CASE(MYEA_AF_RELU);
      MYEA_AF_CASE(MYEA_AF_LEAKY_RELU);
      MYEA_AF_CASE(MYEA_AF_ELU);
      MYEA_AF_CASE(MYEA_AF_SELU);
      case MYEA_AF_LINEAR: activation_forward_panels_kernel<MYEA_AF_LINEAR><<<grid, 256, 0, ctx.stream>>>(z, out, rows, H, col_scale, col_shift, mask, keep_scale, *sink); break;
      default: return MYEA_E_INVALID;  // activation_writes_panels(af) is false: the caller asks for plain arrays
    }
#undef MYEA_AF_CASE
    ctx.end(TC_ELEMENTWISE);
    return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
  }
  const long long total = rows * (vec4 ? H / 4 : H);
  const int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>((total + 255) / 256, 148 * 16)));
  if (vec4) {
    const dim3 grid = column_walk_grid(rows, H);
#define MYEA_AF_CASE(A) case A: activation_forward_cols_kernel<A><<<grid, 256, 0, ctx.stream>>>(z, out, rows, H, col_scale, col_shift, mask, keep_scale); break
    switch (af) {
      MYEA_AF_CASE(MYEA_AF_TANH);
      MYEA_AF_CASE(MYEA_AF_SIGMOID);
      MYEA_AF_CASE(MYEA_AF_RELU);
      MYEA_AF_CASE(MYEA_AF_LEAKY_RELU);
      MYEA_AF_CASE(MYEA_AF_ELU);
      MYEA_AF_CASE(MYEA_AF_SELU);
      default: activation_forward_kernel<4><<<blocks, 256, 0, ctx.stream>>>(z, out, rows, H, af, col_scale, col_shift, mask, keep_scale); break;
    }
#undef MYEA_AF_CASE
  } else
    activation_forward_kernel<1><<<blocks, 256, 0, ctx.stream>>>(z, out, rows, H, af, col_scale, col_shift, mask, keep_scale);
  ctx.end(TC_ELEMENTWISE);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// ---------------------------------------------------------------------------------------------------------
// Softmax over each row, max-subtracted (Forward_Pass__FC_AF__Softmax, …Forward_Pass__OpenMP.cpp:4870-4905)
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_reduce_max(float v, float *sh) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sh[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w) r = fmaxf(r, sh[w]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_reduce_sum(float v, float *sh) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) r += sh[w];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(128) softmax_forward_kernel(const float *__restrict__ z, float *__restrict__ out, long long H) {
  __shared__ float sh[4];
  const float *zr = z + blockIdx.x * H;
  float *orow = out + blockIdx.x * H;
  float mx = -3.402823466e+38f;
  for (long long j = threadIdx.x; j < H; j += blockDim.x) mx = fmaxf(mx, zr[j]);
  mx = block_reduce_max(mx, sh);
  float s = 0.f;
  for (long long j = threadIdx.x; j < H; j += blockDim.x) {
    const float e = expf(zr[j] - mx);
    orow[j] = e;
    s += e;
  }
  s = block_reduce_sum(s, sh);
  const float inv = 1.0f / s;
  for (long long j = threadIdx.x; j < H; j += blockDim.x) orow[j] *= inv;
}

// d[r][c] *= f'(z[r][c] * col_scale[c] + col_shift[c], y[r][c])   (Backward_Pass__FC__DF, Neural_Network__Backward_Pass__OpenMP.cpp:1225-1263)
__global__ void __launch_bounds__(256) activation_backward_kernel(float *__restrict__ d, const float *__restrict__ z, const float *__restrict__ y,
                                                                  long long rows, long long H, uint32_t af, const float *__restrict__ col_scale,
                                                                  const float *__restrict__ col_shift) {
  const long long total = rows * H;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long c = i % H;
    const float pre = col_scale != nullptr ? fmaf(z[i], col_scale[c], col_shift[c]) : z[i];
    d[i] *= af_derive(af, pre, y[i]);
  }
}

int activation_backward(Context &ctx, float *d, const float *z, const float *y, long long rows, long long H, uint32_t af, const float *col_scale,
                        const float *col_shift) {
  if (rows <= 0 || H <= 0) return MYEA_OK;
  ctx.begin(TC_ELEMENTWISE);
  const int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>((rows * H + 255) / 256, 148 * 16)));
  activation_backward_kernel<<<blocks, 256, 0, ctx.stream>>>(d, z, y, rows, H, af, col_scale, col_shift);
  ctx.end(TC_ELEMENTWISE);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

int softmax_forward(Context &ctx, const float *z, float *out, long long rows, long long H) {
  ctx.begin(TC_ELEMENTWISE);
  softmax_forward_kernel<<<static_cast<unsigned>(rows), 128, 0, ctx.stream>>>(z, out, H);
  ctx.end(TC_ELEMENTWISE);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// ---------------------------------------------------------------------------------------------------------
// Normalization backward. Backward_Pass__Batch_Normalization / …Batch_Renormalization
// (Neural_Network__Backward_Pass__OpenMP.cpp:1346-1467, 1586-1709).  With x_hat = (z-mean)/sigma*r + d and
// dh = delta*gamma the reference accumulates, per column,
//   d_gamma += sum delta*x_hat      d_beta += sum delta
//   d_mean   = sum dh * (-r/sigma)  d_sigma = sum dh * (z-mean) * (-r/sigma^2)
// and then writes dx = dh*r/sigma + d_sigma*(z-mean)/(B*sigma) + d_mean/B.  Everything follows from the two column
// sums S1 = sum delta and S2 = sum delta*(z-mean):  d_beta += S1, d_gamma += (r/sigma)*S2 + d*S1,
// d_mean = -gamma*(r/sigma)*S1, d_sigma = -gamma*(r/sigma^2)*S2, so one reduction pass and one apply pass suffice.
// r and d are constants of the backward pass, as in the reference.
// ---------------------------------------------------------------------------------------------------------
// `global` (may be null): the column sums added over all ranks of a sharded batch; d_gamma / d_beta take the LOCAL sums
// (the derivative buffers are summed over ranks later), d_mean / d_sigma and `rows` are those of the whole batch.
__global__ void __launch_bounds__(256) norm_backward_finalize_kernel(const float *__restrict__ partial, int chunks, const float *__restrict__ global,
                                                                     long long rows, long long H, NormParams np, float *__restrict__ coef) {
  const long long j = blockIdx.x * 32ll + (threadIdx.x & 31);
  float s1, s2;
  chunk_sums(partial, chunks, H, j, s1, s2);
  if (threadIdx.x >= 32 || j >= H) return;
  const float sigma = np.sigma[j], r = np.r[j], d = np.d[j], g = np.gamma[j];
  const float k = r / sigma;
  np.d_beta[j] += s1;
  np.d_gamma[j] += k * s2 + d * s1;
  if (global != nullptr) { s1 = global[j]; s2 = global[H + j]; }
  const float d_mean = -g * k * s1;
  const float d_sigma = -g * (r / (sigma * sigma)) * s2;
  const float inv_b = 1.0f / static_cast<float>(rows);
  coef[0 * H + j] = g * k;                                             // multiplies delta
  coef[1 * H + j] = d_sigma / (static_cast<float>(rows) * sigma);      // multiplies (z - mean)
  coef[2 * H + j] = d_mean * inv_b;                                    // constant
}

template <int VEC>
__global__ void __launch_bounds__(256) norm_backward_apply_kernel(const float *__restrict__ z, const float *__restrict__ delta,
                                                                  float *__restrict__ out, long long rows, long long H,
                                                                  const float *__restrict__ mean, const float *__restrict__ coef) {
  const long long hv = H / VEC;
  const long long total = rows * hv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / hv;
    const long long c = (i - r * hv) * VEC;
    float zv[VEC], dv[VEC];
    if (VEC == 4) {
      const float4 t = *reinterpret_cast<const float4 *>(z + r * H + c);
      const float4 u = *reinterpret_cast<const float4 *>(delta + r * H + c);
      zv[0] = t.x; zv[1] = t.y; zv[2] = t.z; zv[3] = t.w;
      dv[0] = u.x; dv[1] = u.y; dv[2] = u.z; dv[3] = u.w;
    } else {
      zv[0] = z[r * H + c];
      dv[0] = delta[r * H + c];
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k)
      dv[k] = dv[k] * coef[0 * H + c + k] + (zv[k] - mean[c + k]) * coef[1 * H + c + k] + coef[2 * H + c + k];
    if (VEC == 4)
      *reinterpret_cast<float4 *>(out + r * H + c) = make_float4(dv[0], dv[1], dv[2], dv[3]);
    else
      out[r * H + c] = dv[0];
  }
}

// vectorized form: a thread keeps four columns (mean and the three coefficients loaded once) and walks rows four at a time
__global__ void __launch_bounds__(256) norm_backward_apply_cols_kernel(const float *__restrict__ z, const float *__restrict__ delta,
                                                                       float *__restrict__ out, long long rows, long long H,
                                                                       const float *__restrict__ mean, const float *__restrict__ coef) {
  const long long c = (blockIdx.x * 256ll + threadIdx.x) * 4;
  if (c >= H) return;
  const float4 mu = *reinterpret_cast<const float4 *>(mean + c);
  const float4 k0 = *reinterpret_cast<const float4 *>(coef + c), k1 = *reinterpret_cast<const float4 *>(coef + H + c),
               k2 = *reinterpret_cast<const float4 *>(coef + 2 * H + c);
  for (long long r0 = blockIdx.y * 4ll; r0 < rows; r0 += gridDim.y * 4ll) {
    float4 t[4], u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (r0 + i < rows) {
        t[i] = *reinterpret_cast<const float4 *>(z + (r0 + i) * H + c);
        u[i] = *reinterpret_cast<const float4 *>(delta + (r0 + i) * H + c);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (r0 + i >= rows) break;
      float4 d;
      d.x = u[i].x * k0.x + (t[i].x - mu.x) * k1.x + k2.x;
      d.y = u[i].y * k0.y + (t[i].y - mu.y) * k1.y + k2.y;
      d.z = u[i].z * k0.z + (t[i].z - mu.z) * k1.z + k2.z;
      d.w = u[i].w * k0.w + (t[i].w - mu.w) * k1.w + k2.w;
      *reinterpret_cast<float4 *>(out + (r0 + i) * H + c) = d;
    }
  }
}

int norm_backward(Context &ctx, const float *z, const float *delta_af, float *delta_out, long long rows, long long H,
                  const NormParams &np, const SumHook *hook, int fused_chunks, const PanelSink *sink) {
  ctx.begin(TC_NORM);
  const int chunks = fused_chunks > 0 ? fused_chunks : pick_chunks(rows, H, (H % 4 == 0) ? 4 : 1, np.chunks);
  if (fused_chunks <= 0) launch_column_reduce<RK_NORM_BWD>(ctx, z, delta_af, np.mean, rows, H, chunks, np.partial);
  float *coef = np.partial + 2ll * np.chunks * H;  // [3][H] behind the partial sums
  const float *global = nullptr;
  long long rows_total = rows;
  if (hook != nullptr && hook->world > 1) {
    float *g = coef + 3 * H;
    chunk_sum_kernel<<<static_cast<unsigned>((H + 31) / 32), 256, 0, ctx.stream>>>(np.partial, chunks, H, g);
    ctx.end(TC_NORM, 2);
    if (hook->all_reduce(hook->user, g, static_cast<size_t>(2 * H)) != MYEA_OK) return MYEA_E_COMM;
    ctx.begin(TC_NORM);
    global = g;
    rows_total = rows * hook->world;
  }
  norm_backward_finalize_kernel<<<static_cast<unsigned>((H + 31) / 32), 256, 0, ctx.stream>>>(np.partial, chunks, global, rows_total, H, np, coef);
  const bool vec4 = (H % 4 == 0) && ((reinterpret_cast<uintptr_t>(z) & 15) == 0) && ((reinterpret_cast<uintptr_t>(delta_af) & 15) == 0) &&
                    ((reinterpret_cast<uintptr_t>(delta_out) & 15) == 0);
  const long long total = rows * (vec4 ? H / 4 : H);
  const int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>((total + 255) / 256, 148 * 16)));
  const bool cols_ok = vec4 && (reinterpret_cast<uintptr_t>(np.mean) & 15) == 0 && (reinterpret_cast<uintptr_t>(coef) & 15) == 0;
  if (sink != nullptr && !(cols_ok && (H & 7) == 0 && (rows & 7) == 0)) return MYEA_E_INVALID;
  if (sink != nullptr)
    norm_backward_apply_panels_kernel<<<column_walk_grid8(rows, H), 256, 0, ctx.stream>>>(z, delta_af, delta_out, rows, H, np.mean, coef, *sink);
  else if (cols_ok)
    norm_backward_apply_cols_kernel<<<column_walk_grid(rows, H), 256, 0, ctx.stream>>>(z, delta_af, delta_out, rows, H, np.mean, coef);
  else if (vec4)
    norm_backward_apply_kernel<4><<<blocks, 256, 0, ctx.stream>>>(z, delta_af, delta_out, rows, H, np.mean, coef);
  else
    norm_backward_apply_kernel<1><<<blocks, 256, 0, ctx.stream>>>(z, delta_af, delta_out, rows, H, np.mean, coef);
  ctx.end(TC_NORM, 3);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// ---------------------------------------------------------------------------------------------------------
// Output error and loss / accuracy accumulators: FF__Compute__Error (Neural_Network__Compute__Error__OpenMP.cpp:22-141),
// Update_Error (…Compute__Error__Loop.cpp:20-76).  delta = f'(pre, y) * (y - desired) whatever the loss function; the
// loss type only selects what is added to the loss accumulator.  One block per row.
// d_acc[0] += loss terms, d_acc[1] += accuracy hits, d_count[0] += number of loss terms.
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) output_error_kernel(const float *__restrict__ pre, const float *__restrict__ y,
                                                           const float *__restrict__ desired, float *__restrict__ delta, long long H,
                                                           uint32_t af, uint32_t loss, uint32_t accuracy, float accuracy_variance,
                                                           double *d_acc, unsigned long long *d_count) {
  __shared__ float sh[4];
  __shared__ int shi[4];
  __shared__ float shv[4];
  const long long base = blockIdx.x * H;
  float loss_sum = 0.f, hits = 0.f;
  // arg max of the prediction (the LAST maximum wins: the reference compares with >=) and first desired == 1
  float best = -3.402823466e+38f;
  int best_i = -1, want_i = 0x7fffffff;
  for (long long j = threadIdx.x; j < H; j += blockDim.x) {
    const float yv = y[base + j], t = desired[base + j];
    const float diff = yv - t;
    const float p = pre != nullptr ? pre[base + j] : 0.f;
    delta[base + j] = af_derive(af, p, yv) * diff;
    if (loss == MYEA_LOSS_MSE) {
      loss_sum += diff * diff;
    } else if (loss == MYEA_LOSS_CROSS_ENTROPY) {
      const float o = yv != 0.f ? yv : fmaxf(yv, 1e-6f);
      if (H == 1) loss_sum += -(t * logf(o) + (1.f - t) * logf(1.f - o));
      else loss_sum += -(t * logf(o));
    }
    if (accuracy == MYEA_ACCURACY_DISTANCE) hits += fabsf(diff) <= accuracy_variance ? 1.f : 0.f;
    if (accuracy == MYEA_ACCURACY_CROSS_ENTROPY) {
      if (yv >= best) { best = yv; best_i = static_cast<int>(j); }
      if (t == 1.0f && static_cast<int>(j) < want_i) want_i = static_cast<int>(j);
    }
  }
  loss_sum = block_reduce_sum(loss_sum, sh);
  hits = block_reduce_sum(hits, sh);
  if (accuracy == MYEA_ACCURACY_CROSS_ENTROPY) {
    // per-thread candidates are in increasing j; combine: larger value wins, ties go to the larger index
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      const int ow = __shfl_xor_sync(0xffffffffu, want_i, o);
      if (ob > best || (ob == best && oi > best_i)) { best = ob; best_i = oi; }
      want_i = min(want_i, ow);
    }
    if ((threadIdx.x & 31) == 0) { shv[threadIdx.x >> 5] = best; shi[threadIdx.x >> 5] = best_i; sh[threadIdx.x >> 5] = __int_as_float(want_i); }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < 4; ++w) {
        if (shv[w] > best || (shv[w] == best && shi[w] > best_i)) { best = shv[w]; best_i = shi[w]; }
        want_i = min(want_i, __float_as_int(sh[w]));
      }
      if (want_i == 0x7fffffff) want_i = static_cast<int>(H);  // no desired == 1: the reference's search runs off the end
      hits = (want_i == best_i) ? 1.f : 0.f;
    }
  }
  if (threadIdx.x == 0) {
    atomicAdd(&d_acc[0], static_cast<double>(loss_sum));
    atomicAdd(&d_acc[1], static_cast<double>(hits));
    atomicAdd(d_count, static_cast<unsigned long long>(H));
  }
}

int output_error(Context &ctx, const float *pre, const float *y, const float *desired, float *delta, long long rows, long long H,
                 uint32_t af, uint32_t loss, uint32_t accuracy, float accuracy_variance, double *d_acc, unsigned long long *d_count) {
  ctx.begin(TC_ELEMENTWISE);
  output_error_kernel<<<static_cast<unsigned>(rows), 128, 0, ctx.stream>>>(pre, y, desired, delta, H, af, loss, accuracy,
                                                                            accuracy_variance, d_acc, d_count);
  ctx.end(TC_ELEMENTWISE);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// ---------------------------------------------------------------------------------------------------------
// Bias derivative: out[j] (+)= sum over rows (Update_Derivative_Weight__Bias, …Update_Derivative_Weight__OpenMP.cpp:218-242)
// ---------------------------------------------------------------------------------------------------------
__global__ void column_sum_finalize_kernel(const float *__restrict__ partial, int chunks, long long H, float *__restrict__ out,
                                           int accumulate) {
  const long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (j >= H) return;
  float s = 0.f;
#pragma unroll 8
  for (int c = 0; c < chunks; ++c) s += partial[static_cast<long long>(c) * H + j];
  out[j] = accumulate ? out[j] + s : s;
}

int column_sum(Context &ctx, const float *in, long long rows, long long H, float *out, int accumulate, float *partial, int max_chunks) {
  ctx.begin(TC_ELEMENTWISE);
  const int chunks = pick_chunks(rows, H, (H % 4 == 0) ? 4 : 1, max_chunks);
  launch_column_reduce<RK_SUM>(ctx, in, nullptr, nullptr, rows, H, chunks, partial);
  column_sum_finalize_kernel<<<static_cast<unsigned>((H + 255) / 256), 256, 0, ctx.stream>>>(partial, chunks, H, out, accumulate);
  ctx.end(TC_ELEMENTWISE, 2);
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

int fill_zero(Context &ctx, float *p, size_t n) {
  return cudaMemsetAsync(p, 0, n * sizeof(float), ctx.stream) == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

}  // namespace myea
