// Dense contraction for callers that must not allocate device memory.
//
// Who this is for: the reference library is driven tick by tick from a trading terminal through a DLL, and similar
// hosts (a process whose GPU memory was reserved up front by the embedding application, a latency-critical loop)
// cannot afford cudaMalloc in the call path: it synchronises the whole device, takes an unpredictable time and can
// fail at an arbitrary moment once memory is fragmented or spoken for.  Every other contraction of this library
// takes its operand-panel scratch from memory the handle allocated at creation; this entry point instead keeps the
// scratch in a fixed array that is part of the loaded library image, so the call path contains no cudaMalloc,
// cudaFree or allocating library routine at all.  Inputs and output stay the caller's (device pointers).
//
// Cost: every GPU that loads the library holds the array (MYEA_STATIC_SCRATCH_BYTES = 32 MiB, plus a 256-byte status
// word) until the process exits, whether or not this entry point is ever called.
// Limit: the hi/lo K-major panels of both operands must fit: 2 * (M + N) * round_up(K, 32) + 64 floats <= 8 Mi floats;
// larger problems are refused with MYEA_E_INVALID and a message, never truncated.
// Sharing: all calls on a device use the same array, which keeps whatever the previous call left in it.  Nothing in
// it has to start at zero except the status word, which each call clears first: a call rewrites columns
// [0, round_up(K, 8)) of every panel row it uses, and what an earlier, larger call left beyond that is never read,
// because the tensor maps the kernel loads through end at round_up(K, 8) and the hardware fills the rest of a tile
// with zeros.  Two calls that overlap on the GPU (different streams, or different host threads) would overwrite each
// other's panels: callers must serialise them.
// Set-up: the device address of the array is looked up once per device, on the first call for that device, with that
// device current.
// The call is synchronous: it waits for the result and reads the status word back, so it must never be made on a
// stream that is being captured (neither the first call nor a later one).
// Current device: the call makes `device` current for its own work and puts the caller's current device back before
// it returns.
#include "common.cuh"

#include <mutex>
#include <stdio.h>

namespace {

constexpr size_t kStaticScratchFloats = size_t(8) << 20;  // 32 MiB
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
static __device__ __align__(256) int g_static_status[64];

struct StaticSetup {
  bool ready = false;
  float *scratch = nullptr;  // DEVICE addresses of the two arrays above on this device
  int *status = nullptr;
};
StaticSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

void say(char *dst, size_t cap, const char *msg) {
  if (dst != nullptr && cap > 0) snprintf(dst, cap, "%s", msg);
}

}  // namespace

extern "C" int myea_b200_gemm_nt_static(int device, uint64_t M, uint64_t N, uint64_t K, const float *device_A,
                                        const float *device_B, float *device_C, int accumulate, void *stream,
                                        char *error_message, size_t error_capacity) {
  using namespace myea;
  if (device_A == nullptr || device_B == nullptr || device_C == nullptr || M == 0 || N == 0 || K == 0) {
    say(error_message, error_capacity, "gemm_nt_static: null operand or zero dimension");
    return MYEA_E_INVALID;
  }
  if (device < 0 || device >= kMaxDevices) {
    say(error_message, error_capacity, "gemm_nt_static: device index out of range");
    return MYEA_E_INVALID;
  }
  const size_t need = gemm_scratch_floats(static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(K));
  if (M > (1u << 30) || N > (1u << 30) || K > (1u << 30) || need > kStaticScratchFloats) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "gemm_nt_static: problem too large for the fixed scratch: 2*(M+N)*round_up(K,32)+64 = %zu floats, limit %zu "
             "(32 MiB); use a handle-based call instead",
             need, kStaticScratchFloats);
    say(error_message, error_capacity, msg);
    return MYEA_E_INVALID;
  }
  int previous_device = -1;
  if (cudaGetDevice(&previous_device) != cudaSuccess || cudaSetDevice(device) != cudaSuccess) {
    say(error_message, error_capacity, "gemm_nt_static: cudaSetDevice failed");
    return MYEA_E_CUDA;
  }
  // the caller's current device comes back on every way out of this function
  struct RestoreDevice {
    int device;
    ~RestoreDevice() { if (device >= 0) cudaSetDevice(device); }
  } restore{previous_device == device ? -1 : previous_device};
  StaticSetup &su = g_setup[device];
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!su.ready) {
      // In host code `g_static_scratch` names a host-side stand-in for the symbol, not device memory: a kernel handed
      // that name would read the wrong memory.  The device address on THIS device comes from the runtime.
      void *p = nullptr, *q = nullptr;
      if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || cudaGetSymbolAddress(&q, g_static_status) != cudaSuccess ||
          p == nullptr || q == nullptr) {
        say(error_message, error_capacity, "gemm_nt_static: cudaGetSymbolAddress failed (no sm_100a device image loaded?)");
        return MYEA_E_CUDA;
      }
      su.scratch = static_cast<float *>(p);
      su.status = static_cast<int *>(q);
      su.ready = true;
    }
  }
  Context ctx;
  ctx.device = device;
  ctx.stream = static_cast<cudaStream_t>(stream);
  ctx.d_error_flag = su.status;
  ctx.gemm_engine = 0;
  if (cudaMemsetAsync(su.status, 0, sizeof(int), ctx.stream) != cudaSuccess) {  // the one thing that must start at zero
    say(error_message, error_capacity, "gemm_nt_static: clearing the status word failed");
    return MYEA_E_CUDA;
  }
  Operand a{device_A, static_cast<long long>(M), static_cast<long long>(K), static_cast<long long>(K), 1};
  Operand b{device_B, static_cast<long long>(N), static_cast<long long>(K), static_cast<long long>(K), 1};
  Epilogue e;
  e.C = device_C;
  e.ldc = static_cast<long long>(N);
  e.accumulate = accumulate;
  GemmScratch gs{su.scratch, kStaticScratchFloats};
  int rc = gemm_nt(ctx, a, b, e, gs);
  if (rc != MYEA_OK) {
    say(error_message, error_capacity, "gemm_nt_static: kernel launch failed");
    return rc;
  }
  int flag = 0;
  if (cudaMemcpyAsync(&flag, su.status, sizeof(int), cudaMemcpyDeviceToHost, ctx.stream) != cudaSuccess ||
      cudaStreamSynchronize(ctx.stream) != cudaSuccess) {
    say(error_message, error_capacity, "gemm_nt_static: a CUDA call failed while waiting for the result");
    return MYEA_E_CUDA;
  }
  if (flag != 0) {
    say(error_message, error_capacity, "gemm_nt_static: the kernel gave up a bounded wait");
    return MYEA_E_KERNEL;
  }
  say(error_message, error_capacity, "");
  return MYEA_OK;
}
