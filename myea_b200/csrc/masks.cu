// Dropout, zoneout and ShakeDrop draws made on the device with a counter-based generator, so that an epoch needs no
// host-side mask generation and upload.  Replaces Dropout_Bernoulli (Neural_Network__Dropout__Bernoulli__Loop.cpp:70-90),
// Dropout_Zoneout (Neural_Network__Dropout__Zoneout__Loop.cpp:57-100) and the draws inside
// Forward_Pass__Dropout__ShakeDrop (Neural_Network__Forward_Pass__Loop.cpp:5016-5045) and
// Backward_Pass__Dropout__ShakeDrop (Neural_Network__Backward_Pass__OpenMP.cpp:1009-1042), which walk a std::mt19937
// per thread.  The streams here are statistically, not bit for bit, comparable to those; they are a pure function of
// (seed, step, layer, kind, element), the same on every GPU, which is what data-parallel ranks need for masks that are
// shared by the whole batch.
//
// Generator: Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11).
//   key     = (seed low, seed high)
//   counter = (element / 4, step low, step high, 8 * layer + kind)        element e uses word e % 4 of its block
//   u       = (word >> 8) * 2^-24 in [0, 1)
// Bernoulli keep mask: u < retention probability.  Zoneout: "compute" unless u < zoneout probability.  ShakeDrop: mask
// u < p per sample, alpha = 2u - 1, beta = u per (sample, unit).
#include "net.cuh"

namespace myea {

void lstm_zoneout_arrays(LayerPlan &L, int dir, uint8_t **state, uint8_t **output, long long *cells, int *dirs, float *p_state, float *p_output);

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

struct DrawStream {
  uint32_t seed_lo, seed_hi, step_lo, step_hi, stream;
};

__device__ __forceinline__ float draw_uniform(const DrawStream &s, unsigned long long element) {
  uint32_t c[4] = {static_cast<uint32_t>(element >> 2), s.step_lo, s.step_hi, s.stream};
  philox4x32_10(c, s.seed_lo, s.seed_hi);
  return static_cast<float>(c[element & 3ull] >> 8) * (1.0f / 16777216.0f);
}

// out[i] = u(element(i)) < p ? below : other;  element(i) = (i / inner) * outer_pitch + offset + i % inner lets one
// direction of a bidirectional layer ([T][C] on the device) take its elements from the [T][dirs * C] numbering
__global__ void draw_mask_kernel(uint8_t *__restrict__ out, long long n, float p, uint8_t below, uint8_t other, long long inner,
                                 long long outer_pitch, long long offset, const DrawStream s) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const long long e = (i / inner) * outer_pitch + offset + (i % inner);
  out[i] = draw_uniform(s, static_cast<unsigned long long>(e)) < p ? below : other;
}

__global__ void draw_coefficient_kernel(float *__restrict__ out, long long n, float scale, float shift, const DrawStream s) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  out[i] = __fmaf_rn(scale, draw_uniform(s, static_cast<unsigned long long>(i)), shift);
}

static unsigned blocks_for(long long n) { return static_cast<unsigned>((n + 255) / 256); }

}  // namespace myea

using namespace myea;

extern "C" int myea_b200_generate_masks(myea_handle net, uint64_t seed, uint64_t step) {
  if (net == nullptr) return MYEA_E_INVALID;
  if (cudaSetDevice(net->ctx.device) != cudaSuccess) return MYEA_E_CUDA;
  Context &ctx = net->ctx;
  DrawStream s;
  s.seed_lo = static_cast<uint32_t>(seed); s.seed_hi = static_cast<uint32_t>(seed >> 32);
  s.step_lo = static_cast<uint32_t>(step); s.step_hi = static_cast<uint32_t>(step >> 32);
  for (size_t l = 1; l < net->layers.size(); ++l) {
    LayerPlan &L = net->layers[l];
    if (L.mask_bernoulli != nullptr) {
      const long long n = net->T * L.n_out;
      s.stream = static_cast<uint32_t>(8 * l + MYEA_MASK_BERNOULLI);
      ctx.begin(TC_ELEMENTWISE);
      draw_mask_kernel<<<blocks_for(n), 256, 0, ctx.stream>>>(L.mask_bernoulli, n, L.desc.dropout_values[0], 1, 0, n, 0, 0, s);
      ctx.end(TC_ELEMENTWISE);
    }
    if (L.type == MYEA_LAYER_LSTM && L.desc.type_dropout == MYEA_DROPOUT_ZONEOUT) {
      for (int d = 0; d < (L.desc.use_bidirectional ? 2 : 1); ++d) {
        uint8_t *zs = nullptr, *zo = nullptr;
        long long cells = 0;
        int dirs = 1;
        float ps = 0.f, po = 0.f;
        lstm_zoneout_arrays(L, d, &zs, &zo, &cells, &dirs, &ps, &po);
        if (zs == nullptr) continue;
        const long long n = net->T * cells;
        ctx.begin(TC_ELEMENTWISE);
        s.stream = static_cast<uint32_t>(8 * l + MYEA_MASK_ZONEOUT_STATE);
        draw_mask_kernel<<<blocks_for(n), 256, 0, ctx.stream>>>(zs, n, ps, 0, 1, cells, dirs * cells, d * cells, s);
        s.stream = static_cast<uint32_t>(8 * l + MYEA_MASK_ZONEOUT_OUTPUT);
        draw_mask_kernel<<<blocks_for(n), 256, 0, ctx.stream>>>(zo, n, po, 0, 1, cells, dirs * cells, d * cells, s);
        ctx.end(TC_ELEMENTWISE, 2);
      }
    }
    if (L.shake_mask != nullptr) {
      const long long n = net->B * L.n_out;
      ctx.begin(TC_ELEMENTWISE);
      s.stream = static_cast<uint32_t>(8 * l + MYEA_MASK_SHAKEDROP);
      draw_mask_kernel<<<blocks_for(net->B), 256, 0, ctx.stream>>>(L.shake_mask, net->B, L.desc.dropout_values[0], 1, 0, net->B, 0, 0, s);
      s.stream = static_cast<uint32_t>(8 * l + MYEA_MASK_SHAKEDROP_ALPHA);
      draw_coefficient_kernel<<<blocks_for(n), 256, 0, ctx.stream>>>(L.shake_alpha, n, 2.0f, -1.0f, s);
      s.stream = static_cast<uint32_t>(8 * l + MYEA_MASK_SHAKEDROP_BETA);
      draw_coefficient_kernel<<<blocks_for(n), 256, 0, ctx.stream>>>(L.shake_beta, n, 1.0f, 0.0f, s);
      ctx.end(TC_ELEMENTWISE, 3);
    }
  }
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

extern "C" int myea_b200_download_mask(myea_handle net, uint32_t layer, int kind, void *host, uint64_t bytes) {
  if (net == nullptr || host == nullptr || layer >= net->layers.size()) return MYEA_E_INVALID;
  if (cudaSetDevice(net->ctx.device) != cudaSuccess) return MYEA_E_CUDA;
  LayerPlan &L = net->layers[layer];
  cudaStream_t st = net->ctx.stream;
  cudaError_t err = cudaSuccess;
  bool ok = false;
  switch (kind) {
    case MYEA_MASK_BERNOULLI:
      if (L.mask_bernoulli != nullptr && bytes == static_cast<uint64_t>(net->T * L.n_out)) {
        err = cudaMemcpyAsync(host, L.mask_bernoulli, bytes, cudaMemcpyDeviceToHost, st);
        ok = true;
      }
      break;
    case MYEA_MASK_ZONEOUT_STATE:
    case MYEA_MASK_ZONEOUT_OUTPUT:
      if (L.type == MYEA_LAYER_LSTM && L.desc.type_dropout == MYEA_DROPOUT_ZONEOUT) {
        const int nd = L.desc.use_bidirectional ? 2 : 1;
        for (int d = 0; d < nd && err == cudaSuccess; ++d) {
          uint8_t *zs = nullptr, *zo = nullptr;
          long long cells = 0;
          int dirs = 1;
          float ps, po;
          lstm_zoneout_arrays(L, d, &zs, &zo, &cells, &dirs, &ps, &po);
          if (zs == nullptr || bytes != static_cast<uint64_t>(net->T * dirs * cells)) break;
          ok = true;
          // device [T][C] per direction -> host [T][dirs * C]
          err = cudaMemcpy2DAsync(static_cast<uint8_t *>(host) + d * cells, dirs * cells, kind == MYEA_MASK_ZONEOUT_STATE ? zs : zo, cells, cells,
                                  net->T, cudaMemcpyDeviceToHost, st);
        }
      }
      break;
    case MYEA_MASK_SHAKEDROP:
      if (L.shake_mask != nullptr && bytes == static_cast<uint64_t>(net->B)) {
        err = cudaMemcpyAsync(host, L.shake_mask, bytes, cudaMemcpyDeviceToHost, st);
        ok = true;
      }
      break;
    case MYEA_MASK_SHAKEDROP_ALPHA:
    case MYEA_MASK_SHAKEDROP_BETA:
      if (L.shake_mask != nullptr && bytes == static_cast<uint64_t>(net->B * L.n_out) * sizeof(float)) {
        err = cudaMemcpyAsync(host, kind == MYEA_MASK_SHAKEDROP_ALPHA ? L.shake_alpha : L.shake_beta, bytes, cudaMemcpyDeviceToHost, st);
        ok = true;
      }
      break;
    default: break;
  }
  if (!ok) {
    net->ctx.error = "download_mask: the layer has no such array, or the size does not match";
    return MYEA_E_INVALID;
  }
  if (err != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) return MYEA_E_CUDA;
  return MYEA_OK;
}
