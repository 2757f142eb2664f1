// Stand-alone entry point of the dense contraction (host buffers in, host buffers out): used by kernel-level
// parity tests and by roofline timing of the GEMM alone.
#include "common.cuh"

#include <stdio.h>
#include <stdlib.h>
#include <vector>

using namespace myea;

extern "C" int myea_b200_gemm_nt(int device, int engine, uint64_t M, uint64_t N, uint64_t K, const float *A, const float *B,
                                 float *C, int accumulate, float *elapsed_ms, int repeats) {
  if (A == nullptr || B == nullptr || C == nullptr || M == 0 || N == 0 || K == 0) return MYEA_E_INVALID;
  if (cudaSetDevice(device) != cudaSuccess) return MYEA_E_CUDA;
  Context ctx;
  ctx.device = device;
  ctx.gemm_engine = engine & 1;
  ctx.gemm_bn = (engine >> 8) & 0x1FF;  // bits 8..16: forced tile shape (0 = heuristic, 3 = 256 x 256 CTA pair, 4 = the same without stream-K, 2 = 256 x 128 CTA pair, 128 / 256 = single-CTA N tile)
  int rc = MYEA_OK;
  float *dA = nullptr, *dB = nullptr, *dC = nullptr, *dS = nullptr, *dAux = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  // bits 17 / 18: A / B are handed over transposed ([K][M] / [K][N] row-major) and read as MN-major operands
  const bool a_t = (engine >> 17) & 1, b_t = (engine >> 18) & 1;
  const size_t a_floats = a_t ? shared_panel_floats(K, M) + 64 : panel_floats(M, K) + 64;
  const size_t scratch = (a_t || b_t) ? a_floats + (b_t ? shared_panel_floats(K, N) : panel_floats(N, K)) + 128 : gemm_scratch_floats(M, N, K);
  if (cudaStreamCreate(&ctx.stream) != cudaSuccess) return MYEA_E_CUDA;
  if (cudaMalloc(&dA, M * K * 4) != cudaSuccess || cudaMalloc(&dB, N * K * 4) != cudaSuccess ||
      cudaMalloc(&dC, M * N * 4) != cudaSuccess || cudaMalloc(&dS, scratch * 4) != cudaSuccess ||
      cudaMalloc(&ctx.d_error_flag, sizeof(int)) != cudaSuccess) {
    rc = MYEA_E_CUDA;
  }
  if (rc == MYEA_OK) rc = gemm_splitk_reserve(ctx);
  if (rc == MYEA_OK) {
    cudaMemsetAsync(ctx.d_error_flag, 0, sizeof(int), ctx.stream);
    cudaMemcpyAsync(dA, A, M * K * 4, cudaMemcpyHostToDevice, ctx.stream);
    cudaMemcpyAsync(dB, B, N * K * 4, cudaMemcpyHostToDevice, ctx.stream);
    cudaMemcpyAsync(dC, C, M * N * 4, cudaMemcpyHostToDevice, ctx.stream);
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    Operand oa{dA, (long long)M, (long long)K, (long long)K, 1};
    Operand ob{dB, (long long)N, (long long)K, (long long)K, 1};
    Epilogue epi;
    epi.C = dC;
    epi.ldc = (long long)N;
    epi.accumulate = accumulate;
    if ((engine >> 19) & 1) {
      // bit 19: the fused activation-derivative epilogue of the error-propagation product, for kernel-level tests:
      // C = (A * B^T) .* relu'(C_in), the incoming C serving as the pre-activation array
      if (cudaMalloc(&dAux, M * N * 4) != cudaSuccess) rc = MYEA_E_CUDA;
      else {
        cudaMemcpyAsync(dAux, C, M * N * 4, cudaMemcpyHostToDevice, ctx.stream);
        epi.deriv_af = ((engine >> 21) & 1) ? MYEA_AF_TANH : MYEA_AF_RELU;   // bits 20 / 21: timing variants (one array only)
        epi.aux_pre = ((engine >> 21) & 1) ? nullptr : dAux;
        epi.aux_y = ((engine >> 20) & 1) ? nullptr : dAux;
        epi.ld_aux = (long long)N;
        epi.accumulate = 0;
      }
    }
    GemmScratch gs{dS, scratch};
    auto run = [&]() -> int {
      if (!a_t && !b_t) return gemm_nt(ctx, oa, ob, epi, gs);
      if (!gemm_takes_mn_major(ctx, (long long)M, (long long)N)) return MYEA_E_INVALID;
      float *base = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(dS) + 255) & ~static_cast<uintptr_t>(255));
      float *mem_b = base + ((a_floats + 63) & ~static_cast<size_t>(63));
      Panels pa, pb;
      int r = a_t ? gemm_prepare_shared(ctx, dA, (long long)M, (long long)K, (long long)M, base, PANEL_ROLE_A, nullptr, PANEL_ROLE_A, &pa)
                  : gemm_prepare(ctx, oa, base, &pa, PANEL_ROLE_A);
      if (r != MYEA_OK) return r;
      r = b_t ? gemm_prepare_shared(ctx, dB, (long long)N, (long long)K, (long long)N, mem_b, PANEL_ROLE_B, nullptr, PANEL_ROLE_B, &pb)
              : gemm_prepare(ctx, ob, mem_b, &pb, PANEL_ROLE_B);
      if (r != MYEA_OK) return r;
      return gemm_panels(ctx, pa, 0, (long long)M, pb, 0, (long long)N, epi);
    };
    rc = run();  // the call whose result is returned
    if (rc == MYEA_OK && repeats > 0 && elapsed_ms != nullptr) {
      // timing passes write a second output buffer so that `accumulate` does not pile up in C
      float *dC2 = nullptr;
      if (cudaMalloc(&dC2, M * N * 4) == cudaSuccess) {
        epi.C = dC2;
        epi.accumulate = 0;
        run();
        cudaEventRecord(e0, ctx.stream);
        for (int i = 0; i < repeats && rc == MYEA_OK; ++i) rc = run();
        cudaEventRecord(e1, ctx.stream);
        cudaEventSynchronize(e1);
        cudaEventElapsedTime(elapsed_ms, e0, e1);
        *elapsed_ms /= (float)repeats;
        cudaFree(dC2);
      }
    }
    if (cudaMemcpyAsync(C, dC, M * N * 4, cudaMemcpyDeviceToHost, ctx.stream) != cudaSuccess) rc = MYEA_E_CUDA;
    int flag = 0;
    cudaMemcpyAsync(&flag, ctx.d_error_flag, sizeof(int), cudaMemcpyDeviceToHost, ctx.stream);
    if (cudaStreamSynchronize(ctx.stream) != cudaSuccess) rc = MYEA_E_CUDA;
    if (rc == MYEA_OK && flag != 0) rc = MYEA_E_KERNEL;
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(dA); cudaFree(dB); cudaFree(dC); cudaFree(dS); cudaFree(ctx.d_error_flag);
  if (dAux != nullptr) cudaFree(dAux);
  gemm_splitk_release(ctx);
  cudaStreamDestroy(ctx.stream);
  return rc;
}
