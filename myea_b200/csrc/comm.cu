// Data-parallel plumbing: one handle per GPU, each on its shard of the batch, joined by an NCCL communicator.
//
// What is exchanged is exactly what the reference merges across its OpenMP threads: the per-thread derivative slices
// summed by Merge_Derivatives_Parameters (Neural_Network__Merge.cpp:20-50) become a sum over the ranks of the flat
// derivative buffer, issued in per-layer buckets on a second stream as soon as a layer's weight derivative is complete so
// that it overlaps the remaining layers.  A bucket whose size divides evenly is REDUCE-SCATTERED: every rank receives the
// sum of its 1/world slice only, runs the optimizer on that slice (the update is element by element) and the updated
// parameters are ALL-GATHERED - the same bytes on the wire as an all-reduce, 1/world of the optimizer's memory traffic
// per rank.  Other buckets (and every bucket when the max-norm constraint needs whole rows) are
// all-reduced and every rank updates all of them; the per-thread partial sums of the batch-normalization statistics
// (Neural_Network__Forward_Pass__OpenMP.cpp:4591-4701, …Backward_Pass__OpenMP.cpp:1346-1709) become small all-reduces of
// [2][H] column sums, so a sharded step computes the same statistics as the one-GPU step; the loss / accuracy
// accumulators (Merge__Post__Training, Neural_Network__Merge.cpp:52-98) are summed when they are read.
// Derivatives are sums over samples (never divided by the batch), so no rescaling is needed.
//
// NCCL is loaded at run time (dlopen) so that the library itself has no link-time dependency on it.
#include "net.cuh"

#include <algorithm>
#include <utility>
#include <vector>

#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <string.h>

namespace myea {

struct NcclApi {
  void *lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

// Loaded once; the function-local static's initialiser runs on one thread and every caller sees the finished table
// (two host threads, one per GPU, may make their first communicator calls at the same time).
static NcclApi *nccl_api() {
  static const NcclApi api = [] {
    NcclApi a;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
      a.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (a.lib != nullptr) break;
    }
    if (a.lib != nullptr) {
      a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(a.lib, "ncclGetUniqueId"));
      a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(a.lib, "ncclCommInitRank"));
      a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(a.lib, "ncclAllReduce"));
      a.ReduceScatter = reinterpret_cast<decltype(a.ReduceScatter)>(dlsym(a.lib, "ncclReduceScatter"));
      a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(a.lib, "ncclAllGather"));
      a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(a.lib, "ncclCommDestroy"));
      a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(a.lib, "ncclGetErrorString"));
      if (!a.GetUniqueId || !a.CommInitRank || !a.AllReduce || !a.ReduceScatter || !a.AllGather || !a.CommDestroy) a.lib = nullptr;
    }
    return a;
  }();
  return api.lib != nullptr ? const_cast<NcclApi *>(&api) : nullptr;
}

// One-shot sum of a small vector over the ranks through peer-mapped memory (the batch-normalization column sums of a
// sharded batch: 2 x H floats, 16 exchanges per step, each pure latency for a library all-reduce).  Every rank owns one
// allocation that all ranks map (CUDA IPC): [2 parities][world slots][capacity] floats followed by
// [2 parities][world][PEER_MAX_BLOCKS] arrival words.
constexpr int PEER_MAX_BLOCKS = 64;
// how long a rank waits for a peer's arrival word before it gives up and flags the handle: about two minutes of SM
// clocks - ranks may reach an exchange far apart (the first step, a rank that loads data), but it is a bound
constexpr long long PEER_WAIT_CYCLES = 1ll << 38;
constexpr int PEER_MAX_WORLD = 16;
struct PeerSum {
  bool ready = false;
  float *local = nullptr;            // this rank's allocation
  void *mapped[PEER_MAX_WORLD] = {}; // every rank's allocation in this process's address space ([rank] = local)
  float **mapped_d = nullptr;        // the same table on the device
  size_t capacity = 0;               // floats per slot
  unsigned int epoch = 0;            // exchanges so far; the same on every rank
};

// Block b of every rank handles the same 1024 floats.  It stores its floats into slot `rank` of EVERY rank's buffer
// (plain peer stores over NVLink), publishes them with one arrival word per peer, waits (bounded) for the arrival words of
// all ranks in its own buffer and adds the slots in rank order - the same order on every rank, so all ranks end with
// bitwise identical sums.  Two parities: exchange e + 2 can only start when every rank has finished e + 1, and a rank
// enters e + 1 only after it has read the slots of e.
__global__ void __launch_bounds__(256) peer_sum_kernel(float *__restrict__ data, int n, int rank, int world, float *const *__restrict__ bufs,
                                                       size_t capacity, unsigned int epoch, int *error_flag) {
  const int par = static_cast<int>(epoch & 1u);
  const size_t slots = static_cast<size_t>(2) * world * capacity;  // floats before the arrival words
  const int i = (static_cast<int>(blockIdx.x) * 256 + static_cast<int>(threadIdx.x)) * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (i + k < n) v[k] = data[i + k];
  if (i < n) {
    for (int r = 0; r < world; ++r) {
      float *dst = bufs[r] + (static_cast<size_t>(par) * world + rank) * capacity + i;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (i + k < n) dst[k] = v[k];
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < world) {
    const int r = static_cast<int>(threadIdx.x);
    // tell rank r that this rank's floats of this block are in its buffer
    unsigned int *theirs = reinterpret_cast<unsigned int *>(bufs[r] + slots) + (static_cast<size_t>(par) * world + rank) * PEER_MAX_BLOCKS + blockIdx.x;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    // and wait until rank r's floats are in this rank's buffer; the bound is generous (ranks may reach their first
    // exchange seconds apart) but it is a bound
    const unsigned int *mine = reinterpret_cast<const unsigned int *>(bufs[rank] + slots) + (static_cast<size_t>(par) * world + r) * PEER_MAX_BLOCKS + blockIdx.x;
    const long long t0 = clock64();
    for (;;) {
      unsigned int seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (static_cast<int>(seen - epoch) >= 0) break;
      if (clock64() - t0 > PEER_WAIT_CYCLES) { failed = 1; break; }
    }
  }
  __syncthreads();
  if (failed) {
    if (threadIdx.x == 0) atomicCAS(error_flag, 0, 501);
    return;
  }
  if (i < n) {
    float t[4] = {0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const volatile float *src = bufs[rank] + (static_cast<size_t>(par) * world + r) * capacity + i;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (i + k < n) t[k] += src[k];
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (i + k < n) data[i + k] = t[k];
  }
}

// Derivative buckets and updated parameters over peer memory, moved by the copy engines.  The library's reduce-scatter
// and all-gather run as kernels; beside the persistent contraction kernels, which hold every SM, those kernels start
// late and push contraction CTAs off their SMs, so neither side gets the overlap.  Copies between peer-mapped buffers
// need no SM at all.  Per bucket of n floats and rank r (count = n / world):
//   sum:    every rank copies, for each peer p, its derivative slice p into p's staging area (slot of the sender),
//           then sets p's arrival word; rank p waits for world - 1 words and adds the slots to its own slice in rank order
//           (the same order on every rank's slice, whoever arrives first);
//   gather: after the update every rank copies its parameter slice into every peer's parameter buffer and sets the
//           peers' arrival words; a reader of the parameters waits for the words of the buckets it reads.
// The staging area of a bucket is the bucket's own index range in a buffer as long as the parameter buffer; words carry
// the step number, so nothing is ever reset.  A rank cannot run ahead by a step: its next push of a bucket comes after
// its forward pass has waited for every peer's gather of that bucket, which the peer issues after it has added the slots.
constexpr int PEER_MAX_BUCKETS = 256;
struct PeerCopy {
  bool ready = false;
  float *stage = nullptr;                      // [total_parameters] receive area for derivative slices
  unsigned int *flags = nullptr;               // [2 kinds][PEER_MAX_BUCKETS][PEER_MAX_WORLD] arrival words
  void *params[PEER_MAX_WORLD] = {};           // every rank's parameter buffer, staging area and words in this address space
  void *stages[PEER_MAX_WORLD] = {};
  void *words[PEER_MAX_WORLD] = {};
  unsigned int **words_d = nullptr;            // `words` on the device
  unsigned int epoch = 0;                      // steps that issued buckets so far; the same on every rank
};
__host__ __device__ inline size_t peer_word(int kind, size_t bucket, int source) {
  return (static_cast<size_t>(kind) * PEER_MAX_BUCKETS + bucket) * PEER_MAX_WORLD + static_cast<size_t>(source);
}

// tells every peer that this rank's copies of (kind, bucket) are in its memory (same stream as the copies, behind them)
// (which: 0 every peer, 1 / 2 the peers an odd / even number of ranks ahead - the two halves travel on two streams)
__global__ void peer_signal_kernel(unsigned int *const *__restrict__ words, int kind, size_t bucket, int rank, int world, unsigned int epoch, int which) {
  const int r = static_cast<int>(threadIdx.x);
  if (r >= world || r == rank) return;
  const int ahead = (r - rank + world) % world;
  if ((which == 1 && (ahead & 1) == 0) || (which == 2 && (ahead & 1) == 1)) return;
  __threadfence_system();
  unsigned int *theirs = words[r] + peer_word(kind, bucket, rank);
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
}
// waits (bounded) until every peer's copies of (kind, bucket) of step `epoch` are in this rank's memory
__global__ void peer_wait_kernel(const unsigned int *__restrict__ mine, int kind, size_t bucket, int rank, int world, unsigned int epoch, int *error_flag) {
  const int r = static_cast<int>(threadIdx.x);
  if (r >= world || r == rank) return;
  const unsigned int *word = mine + peer_word(kind, bucket, r);
  const long long t0 = clock64();
  for (;;) {
    unsigned int seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(word) : "memory");
    if (static_cast<int>(seen - epoch) >= 0) return;
    if (clock64() - t0 > PEER_WAIT_CYCLES) {
      atomicCAS(error_flag, 0, 502 + kind);
      return;
    }
    __nanosleep(200);
  }
}
// slice[i] = sum over ranks in rank order of (r == rank ? slice[i] : slot of r), float4 at a time
__global__ void __launch_bounds__(256) peer_slices_sum_kernel(float4 *__restrict__ slice, const float4 *__restrict__ slots, size_t count4, int rank, int world) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < count4; i += static_cast<size_t>(gridDim.x) * 256) {
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = r == rank ? slice[i] : __ldcs(slots + static_cast<size_t>(r < rank ? r : r - 1) * count4 + i);
      t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
    }
    slice[i] = t;
  }
}

struct CommState {
  PeerSum peer;
  PeerCopy copy;
  ncclComm_t comm = nullptr;
  int world = 1, rank = 0;
  cudaStream_t stream = nullptr;   // bucket all-reduces run here, beside the compute stream
  cudaStream_t stream_aux = nullptr;    // peer copies: the peers an even number of ranks ahead (a second copy engine)
  cudaStream_t stream_small = nullptr;  // peer copies of small buckets (biases), so that they do not queue behind the large ones
  cudaStream_t stream_gather = nullptr, stream_gather_aux = nullptr;  // updated parameters: not behind the last derivative slices
  cudaEvent_t aux_done = nullptr;
  cudaEvent_t ready = nullptr;     // compute -> comm: the bucket is complete
  cudaEvent_t done = nullptr;      // comm -> compute: every bucket issued so far is reduced
  cudaEvent_t side_done = nullptr; // comm -> compute: the small sum started by comm_side_sum_begin has arrived
  bool pending = false;
  size_t reduced_weights = 0;      // how much of the weight range has been handed to the comm stream this step
  struct Bucket {
    size_t offset = 0, n = 0;
    bool scattered = false;          // reduce-scattered: only [offset + rank * n / world, + n / world) holds the sum
    cudaEvent_t reduced = nullptr;   // comm -> compute: the sum (or this rank's slice of it) has arrived
    cudaEvent_t updated = nullptr;   // compute -> comm: the optimizer has updated this rank's slice of the parameters
    cudaEvent_t gathered = nullptr;  // comm -> compute: every rank's slice of the updated parameters has landed
    bool gather_open = false;        // the gather was issued and the compute stream has not been told to wait for it yet
    bool by_copies = false;          // moved by peer copies and arrival words instead of the library's collectives
    size_t index = 0;                // position in this step's issue order (names the arrival words)
    unsigned int epoch = 0;          // the step whose words it waits for
  };
  std::vector<Bucket> buckets;     // the ranges issued this step, each with the event that says its sum has arrived
  size_t used = 0;
  bool scatter = false;            // this step's buckets may be reduce-scattered (set by update_derivative_weight's caller)
  std::vector<std::pair<size_t, size_t>> last_scattered;  // (offset, n) of the buckets the last update handled in slices
  bool gathers_open = false;       // some bucket's gather_open is set
};

static int nccl_fail(myea_b200_net *net, ncclResult_t r, const char *what) {
  NcclApi *api = nccl_api();
  char msg[256];
  snprintf(msg, sizeof(msg), "%s: %s", what, (api && api->GetErrorString) ? api->GetErrorString(r) : "NCCL error");
  net->ctx.error = msg;
  return MYEA_E_COMM;
}

int comm_world(const myea_b200_net *net) { return net->comm != nullptr ? net->comm->world : 1; }
int comm_rank(const myea_b200_net *net) { return net->comm != nullptr ? net->comm->rank : 0; }

// the peer-memory exchange when it is set up and the vector fits, on `stream`
static bool peer_sum(myea_b200_net *net, float *buf, size_t n, cudaStream_t stream) {
  CommState *c = net->comm;
  PeerSum &p = c->peer;
  const int blocks = static_cast<int>((n + 1023) / 1024);
  if (!p.ready || n > p.capacity || blocks > PEER_MAX_BLOCKS) return false;
  ++p.epoch;
  peer_sum_kernel<<<blocks, 256, 0, stream>>>(buf, static_cast<int>(n), c->rank, c->world, p.mapped_d, p.capacity, p.epoch, net->ctx.d_error_flag);
  return true;
}

// in-place sum over ranks on the COMPUTE stream (small, latency-bound messages: normalization sums, loss counters)
int comm_all_reduce_sum(myea_b200_net *net, float *buf, size_t n) {
  if (net->comm == nullptr || n == 0) return MYEA_OK;
  NcclApi *api = nccl_api();
  net->ctx.begin(TC_COMM);
  if (peer_sum(net, buf, n, net->ctx.stream)) {
    net->ctx.end(TC_COMM);
    return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
  }
  ncclResult_t r = api->AllReduce(buf, buf, n, ncclFloat, ncclSum, net->comm->comm, net->ctx.stream);
  net->ctx.end(TC_COMM);
  return r == ncclSuccess ? MYEA_OK : nccl_fail(net, r, "ncclAllReduce");
}

int comm_all_reduce_sum_f64(myea_b200_net *net, double *buf, size_t n) {
  if (net->comm == nullptr || n == 0) return MYEA_OK;
  NcclApi *api = nccl_api();
  ncclResult_t r = api->AllReduce(buf, buf, n, ncclDouble, ncclSum, net->comm->comm, net->ctx.stream);
  net->ctx.launches += 1;
  return r == ncclSuccess ? MYEA_OK : nccl_fail(net, r, "ncclAllReduce");
}

int comm_gather_join(myea_b200_net *net);

// Peer copies of one bucket: kind 0 sends peer p this rank's derivative slice p (into the sender's slot of p's staging
// area), kind 1 sends every peer this rank's slice of the updated parameters.  The copies start once `producer` (recorded
// on the compute stream) has passed; `finished` is recorded when all of them have left.  Rank r starts with rank r + 1, so
// at any moment every rank receives from one sender per stream.
static int peer_push(myea_b200_net *net, int kind, size_t index, unsigned int epoch, size_t offset, size_t count, cudaEvent_t producer,
                     cudaEvent_t finished) {
  CommState *c = net->comm;
  const int w = c->world;
  const bool small = count * sizeof(float) * static_cast<size_t>(w - 1) < (static_cast<size_t>(4) << 20);
  cudaStream_t main = small ? c->stream_small : (kind == 0 ? c->stream : c->stream_gather);
  cudaStream_t aux = (small || w < 4) ? nullptr : (kind == 0 ? c->stream_aux : c->stream_gather_aux);
  if (cudaStreamWaitEvent(main, producer, 0) != cudaSuccess) return MYEA_E_CUDA;
  if (aux != nullptr && cudaStreamWaitEvent(aux, producer, 0) != cudaSuccess) return MYEA_E_CUDA;
  for (int k = 1; k < w; ++k) {
    const int p = (c->rank + k) % w;
    const float *src;
    float *dst;
    if (kind == 0) {
      src = net->grads + offset + static_cast<size_t>(p) * count;
      dst = static_cast<float *>(c->copy.stages[p]) + offset + static_cast<size_t>(c->rank < p ? c->rank : c->rank - 1) * count;
    } else {
      src = net->params + offset + static_cast<size_t>(c->rank) * count;
      dst = static_cast<float *>(c->copy.params[p]) + offset + static_cast<size_t>(c->rank) * count;
    }
    if (cudaMemcpyAsync(dst, src, count * sizeof(float), cudaMemcpyDeviceToDevice, (aux != nullptr && (k & 1) == 0) ? aux : main) != cudaSuccess) return MYEA_E_CUDA;
  }
  peer_signal_kernel<<<1, 32, 0, main>>>(c->copy.words_d, kind, index, c->rank, w, epoch, aux != nullptr ? 1 : 0);
  if (aux != nullptr) {
    peer_signal_kernel<<<1, 32, 0, aux>>>(c->copy.words_d, kind, index, c->rank, w, epoch, 2);
    if (cudaEventRecord(c->aux_done, aux) != cudaSuccess || cudaStreamWaitEvent(main, c->aux_done, 0) != cudaSuccess) return MYEA_E_CUDA;
  }
  if (cudaGetLastError() != cudaSuccess || cudaEventRecord(finished, main) != cudaSuccess) return MYEA_E_CUDA;
  return MYEA_OK;
}

// Hands the derivative range [offset, offset + n) to the communication stream: it is summed over ranks while the compute
// stream carries on with the next layer.  Every rank issues the same buckets in the same order.
int comm_reduce_bucket_async(myea_b200_net *net, size_t offset, size_t n) {
  CommState *c = net->comm;
  if (c == nullptr || n == 0) return MYEA_OK;
  NcclApi *api = nccl_api();
  if (comm_gather_join(net) != MYEA_OK) return MYEA_E_CUDA;  // the bucket records are about to be reused
  // a slice starts on a 16-byte boundary (the update kernel reads float4) and all slices are equal
  const size_t w = static_cast<size_t>(c->world);
  const bool scattered = c->scatter && (n % (4 * w)) == 0 && (offset % 4) == 0;
  if (c->used == 0) ++c->copy.epoch;
  const bool by_copies = scattered && c->copy.ready && c->used < static_cast<size_t>(PEER_MAX_BUCKETS);
  ncclResult_t r = ncclSuccess;
  if (c->used == c->buckets.size()) {
    CommState::Bucket b;
    if (cudaEventCreateWithFlags(&b.reduced, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&b.updated, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&b.gathered, cudaEventDisableTiming) != cudaSuccess)
      return MYEA_E_CUDA;
    c->buckets.push_back(b);
  }
  if (cudaEventRecord(c->ready, net->ctx.stream) != cudaSuccess) return MYEA_E_CUDA;
  if (by_copies) {
    if (peer_push(net, 0, c->used, c->copy.epoch, offset, n / w, c->ready, c->buckets[c->used].reduced) != MYEA_OK) return MYEA_E_CUDA;
  } else if (cudaStreamWaitEvent(c->stream, c->ready, 0) != cudaSuccess) {
    return MYEA_E_CUDA;
  } else if (scattered) {
    const size_t count = n / w;
    r = api->ReduceScatter(net->grads + offset, net->grads + offset + static_cast<size_t>(c->rank) * count, count, ncclFloat, ncclSum, c->comm, c->stream);
  } else {
    r = api->AllReduce(net->grads + offset, net->grads + offset, n, ncclFloat, ncclSum, c->comm, c->stream);
  }
  if (r != ncclSuccess) return nccl_fail(net, r, scattered ? "ncclReduceScatter (bucket)" : "ncclAllReduce (bucket)");
  CommState::Bucket &b = c->buckets[c->used++];
  b.offset = offset;
  b.n = n;
  b.scattered = scattered;
  b.by_copies = by_copies;
  b.index = c->used - 1;
  b.epoch = c->copy.epoch;
  if (!by_copies && cudaEventRecord(b.reduced, c->stream) != cudaSuccess) return MYEA_E_CUDA;
  c->pending = true;
  net->ctx.launches += 1;
  net->ctx.class_launches[TC_COMM] += 1;
  return MYEA_OK;
}

// A small in-place sum over the ranks on the comm stream, beside whatever the compute stream is given next.
int comm_side_sum_begin(myea_b200_net *net, float *buf, size_t n) {
  CommState *c = net->comm;
  if (c == nullptr) return MYEA_E_INVALID;
  NcclApi *api = nccl_api();
  if (cudaEventRecord(c->ready, net->ctx.stream) != cudaSuccess || cudaStreamWaitEvent(c->stream, c->ready, 0) != cudaSuccess) return MYEA_E_CUDA;
  if (!peer_sum(net, buf, n, c->stream)) {
    ncclResult_t r = api->AllReduce(buf, buf, n, ncclFloat, ncclSum, c->comm, c->stream);
    if (r != ncclSuccess) return nccl_fail(net, r, "ncclAllReduce (side)");
  }
  if (cudaEventRecord(c->side_done, c->stream) != cudaSuccess) return MYEA_E_CUDA;
  net->ctx.launches += 1;
  net->ctx.class_launches[TC_COMM] += 1;
  return MYEA_OK;
}
int comm_side_sum_end(myea_b200_net *net) {
  CommState *c = net->comm;
  if (c == nullptr) return MYEA_E_INVALID;
  return cudaStreamWaitEvent(net->ctx.stream, c->side_done, 0) == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// Makes the compute stream wait until every bucket issued so far has been reduced.
int comm_join(myea_b200_net *net) {
  CommState *c = net->comm;
  if (c == nullptr || !c->pending) return MYEA_OK;
  for (size_t i = 0; i < c->used; ++i)  // (buckets may have travelled on several streams)
    if (cudaStreamWaitEvent(net->ctx.stream, c->buckets[i].reduced, 0) != cudaSuccess) return MYEA_E_CUDA;
  if (cudaEventRecord(c->done, c->stream) != cudaSuccess || cudaStreamWaitEvent(net->ctx.stream, c->done, 0) != cudaSuccess) return MYEA_E_CUDA;
  c->pending = false;
  c->used = 0;
  c->last_scattered.clear();  // every rank updates everything after a join
  return MYEA_OK;
}

// A bucket that travelled by peer copies: once every peer's slot has arrived, this rank's slice becomes the sum.
static int add_peer_slots(myea_b200_net *net, const CommState::Bucket &b) {
  CommState *c = net->comm;
  const size_t count = b.n / static_cast<size_t>(c->world), count4 = count / 4;
  net->ctx.begin(TC_COMM);
  peer_wait_kernel<<<1, 32, 0, net->ctx.stream>>>(c->copy.flags, 0, b.index, c->rank, c->world, b.epoch, net->ctx.d_error_flag);
  const unsigned blocks = static_cast<unsigned>(std::max<size_t>(1, std::min<size_t>((count4 + 255) / 256, 148 * 8)));
  peer_slices_sum_kernel<<<blocks, 256, 0, net->ctx.stream>>>(reinterpret_cast<float4 *>(net->grads + b.offset + static_cast<size_t>(c->rank) * count),
                                                              reinterpret_cast<const float4 *>(c->copy.stage + b.offset), count4, c->rank, c->world);
  net->ctx.end(TC_COMM);
  net->ctx.launches += 2;
  return cudaGetLastError() == cudaSuccess ? MYEA_OK : MYEA_E_CUDA;
}

// The ranges handed to the communicator this step, in the order their sums arrive.
size_t comm_bucket_count(const myea_b200_net *net) { return net->comm != nullptr ? net->comm->used : 0; }
// Makes the compute stream wait for bucket i only and says which range it covers; for a reduce-scattered bucket
// (slice_offset, slice_n) is the slice whose sum this rank holds (otherwise the whole bucket).
int comm_bucket_wait(myea_b200_net *net, size_t i, size_t *offset, size_t *n, size_t *slice_offset, size_t *slice_n) {
  CommState *c = net->comm;
  if (c == nullptr || i >= c->used) return MYEA_E_INVALID;
  const CommState::Bucket &b = c->buckets[i];
  if (cudaStreamWaitEvent(net->ctx.stream, b.reduced, 0) != cudaSuccess) return MYEA_E_CUDA;  // by copies: this rank's slices have left
  *offset = b.offset;
  *n = b.n;
  const size_t count = b.scattered ? b.n / static_cast<size_t>(c->world) : b.n;
  if (b.by_copies && add_peer_slots(net, b) != MYEA_OK) return MYEA_E_CUDA;
  *slice_offset = b.scattered ? b.offset + static_cast<size_t>(c->rank) * count : b.offset;
  *slice_n = count;
  return MYEA_OK;
}
// After the optimizer has updated this rank's slice of bucket i (queued on the compute stream): the slices of all ranks
// are gathered into every rank's parameter buffer on the communication stream.  A bucket that was all-reduced needs
// nothing.  The derivative slices of the OTHER ranks are cleared here (the optimizer clears its own).  Nobody waits for
// the gather here: whoever reads the parameters next asks with comm_wait_gathers (one range) or comm_gather_join (all).
int comm_bucket_gather(myea_b200_net *net, size_t i) {
  CommState *c = net->comm;
  if (c == nullptr || i >= c->used) return MYEA_E_INVALID;
  CommState::Bucket &b = c->buckets[i];
  if (!b.scattered) return MYEA_OK;
  NcclApi *api = nccl_api();
  const size_t count = b.n / static_cast<size_t>(c->world), mine = static_cast<size_t>(c->rank) * count;
  if (mine > 0 && cudaMemsetAsync(net->grads + b.offset, 0, mine * sizeof(float), net->ctx.stream) != cudaSuccess) return MYEA_E_CUDA;
  if (mine + count < b.n &&
      cudaMemsetAsync(net->grads + b.offset + mine + count, 0, (b.n - mine - count) * sizeof(float), net->ctx.stream) != cudaSuccess)
    return MYEA_E_CUDA;
  if (cudaEventRecord(b.updated, net->ctx.stream) != cudaSuccess) return MYEA_E_CUDA;
  if (b.by_copies) {
    if (peer_push(net, 1, b.index, b.epoch, b.offset, count, b.updated, b.gathered) != MYEA_OK) return MYEA_E_CUDA;
  } else {
    if (cudaStreamWaitEvent(c->stream, b.updated, 0) != cudaSuccess) return MYEA_E_CUDA;
    ncclResult_t r = api->AllGather(net->params + b.offset + mine, net->params + b.offset, count, ncclFloat, c->comm, c->stream);
    if (r != ncclSuccess) return nccl_fail(net, r, "ncclAllGather (bucket)");
    if (cudaEventRecord(b.gathered, c->stream) != cudaSuccess) return MYEA_E_CUDA;
  }
  b.gather_open = true;
  c->gathers_open = true;
  net->ctx.launches += 1;
  net->ctx.class_launches[TC_COMM] += 1;
  return MYEA_OK;
}
// The update turned out to need whole derivative buffers (a clip or a max-norm constraint was switched on after the
// buckets had been issued): the slices are gathered so that every rank holds every sum, as after an all-reduce.
int comm_unscatter(myea_b200_net *net) {
  CommState *c = net->comm;
  if (c == nullptr) return MYEA_OK;
  NcclApi *api = nccl_api();
  for (size_t i = 0; i < c->used; ++i) {
    CommState::Bucket &b = c->buckets[i];
    if (!b.scattered) continue;
    const size_t count = b.n / static_cast<size_t>(c->world), mine = static_cast<size_t>(c->rank) * count;
    if (b.by_copies) {  // the slots are added on the compute stream first
      if (cudaStreamWaitEvent(net->ctx.stream, b.reduced, 0) != cudaSuccess || add_peer_slots(net, b) != MYEA_OK ||
          cudaEventRecord(c->ready, net->ctx.stream) != cudaSuccess || cudaStreamWaitEvent(c->stream, c->ready, 0) != cudaSuccess)
        return MYEA_E_CUDA;
      b.by_copies = false;
    }
    ncclResult_t r = api->AllGather(net->grads + b.offset + mine, net->grads + b.offset, count, ncclFloat, c->comm, c->stream);
    if (r != ncclSuccess) return nccl_fail(net, r, "ncclAllGather (derivative slices)");
    if (cudaEventRecord(b.reduced, c->stream) != cudaSuccess) return MYEA_E_CUDA;
    b.scattered = false;
  }
  c->pending = true;
  return MYEA_OK;
}
// the compute stream waits until every rank's slice of the bucket's updated parameters is in this rank's buffer
static int gather_wait(myea_b200_net *net, const CommState::Bucket &b) {
  CommState *c = net->comm;
  if (cudaStreamWaitEvent(net->ctx.stream, b.gathered, 0) != cudaSuccess) return MYEA_E_CUDA;  // by copies: this rank's slice has left
  if (b.by_copies) {
    peer_wait_kernel<<<1, 32, 0, net->ctx.stream>>>(c->copy.flags, 1, b.index, c->rank, c->world, b.epoch, net->ctx.d_error_flag);
    if (cudaGetLastError() != cudaSuccess) return MYEA_E_CUDA;
    net->ctx.launches += 1;
  }
  return MYEA_OK;
}
// Makes the compute stream wait for the gathers of the buckets that overlap the parameter range [offset, offset + n):
// the forward pass asks layer by layer, so the gathers of the upper layers travel while the lower layers compute.
int comm_wait_gathers(myea_b200_net *net, size_t offset, size_t n) {
  CommState *c = net->comm;
  if (c == nullptr || !c->gathers_open) return MYEA_OK;
  bool any = false;
  for (auto &b : c->buckets) {
    if (!b.gather_open) continue;
    if (b.offset < offset + n && offset < b.offset + b.n) {
      if (gather_wait(net, b) != MYEA_OK) return MYEA_E_CUDA;
      b.gather_open = false;
    } else {
      any = true;
    }
  }
  c->gathers_open = any;
  return MYEA_OK;
}
// Makes the compute stream wait until every gather issued so far has landed.
int comm_gather_join(myea_b200_net *net) {
  CommState *c = net->comm;
  if (c == nullptr || !c->gathers_open) return MYEA_OK;
  for (auto &b : c->buckets) {
    if (!b.gather_open) continue;
    if (gather_wait(net, b) != MYEA_OK) return MYEA_E_CUDA;
    b.gather_open = false;
  }
  c->gathers_open = false;
  return MYEA_OK;
}
// Whether the buckets issued from now on may be reduce-scattered (the caller knows if the update needs whole buffers).
void comm_set_scatter(myea_b200_net *net, bool on) {
  if (net->comm != nullptr) net->comm->scatter = on;
}
bool comm_any_scattered(const myea_b200_net *net) {
  if (net->comm == nullptr) return false;
  for (size_t i = 0; i < net->comm->used; ++i)
    if (net->comm->buckets[i].scattered) return true;
  return false;
}
// The optimizer state of a sharded update lives in slices: before a buffer of it is read back, every rank's slice of
// every bucket that was scattered in the last step is gathered (collective: every rank has to ask).
int comm_gather_state(myea_b200_net *net, float *buf) {
  CommState *c = net->comm;
  if (c == nullptr || buf == nullptr) return MYEA_OK;
  NcclApi *api = nccl_api();
  for (const auto &b : c->last_scattered) {
    const size_t count = b.second / static_cast<size_t>(c->world), mine = static_cast<size_t>(c->rank) * count;
    ncclResult_t r = api->AllGather(buf + b.first + mine, buf + b.first, count, ncclFloat, c->comm, net->ctx.stream);
    if (r != ncclSuccess) return nccl_fail(net, r, "ncclAllGather (optimizer state)");
  }
  return MYEA_OK;
}
void comm_buckets_done(myea_b200_net *net) {
  CommState *c = net->comm;
  if (c == nullptr) return;
  c->last_scattered.clear();
  for (size_t i = 0; i < c->used; ++i)
    if (c->buckets[i].scattered) c->last_scattered.emplace_back(c->buckets[i].offset, c->buckets[i].n);
  c->used = 0;
  c->pending = false;
}

size_t &comm_reduced_weights(myea_b200_net *net) {
  static size_t none = 0;
  return net->comm != nullptr ? net->comm->reduced_weights : none;
}

// Maps one allocation of every rank into this process (CUDA IPC; the handles travel in an all-gather).  Every rank takes
// part in the gather even when its own side failed (a zero handle marks the failure); false when anything failed on
// this rank.
static bool ipc_map_all(CommState *c, void *local, bool local_ok, void **mapped) {
  NcclApi *api = nccl_api();
  unsigned char *stage = nullptr;
  std::vector<cudaIpcMemHandle_t> handles(c->world);
  cudaIpcMemHandle_t mine = {};
  bool ok = local_ok && local != nullptr && cudaIpcGetMemHandle(&mine, local) == cudaSuccess;
  if (!ok) memset(&mine, 0, sizeof(mine));
  const bool staged = cudaMalloc(&stage, c->world * sizeof(mine)) == cudaSuccess &&
                      cudaMemcpy(stage + c->rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice) == cudaSuccess;
  const bool gathered = staged && api->AllGather(stage + c->rank * sizeof(mine), stage, sizeof(mine), ncclChar, c->comm, c->stream) == ncclSuccess &&
                        cudaStreamSynchronize(c->stream) == cudaSuccess &&
                        cudaMemcpy(handles.data(), stage, c->world * sizeof(mine), cudaMemcpyDeviceToHost) == cudaSuccess;
  if (stage != nullptr) cudaFree(stage);
  ok = ok && gathered;
  const cudaIpcMemHandle_t zero = {};
  for (int r = 0; ok && r < c->world; ++r)
    if (memcmp(&handles[r], &zero, sizeof(zero)) == 0) ok = false;
  for (int r = 0; ok && r < c->world; ++r) {
    if (r == c->rank) { mapped[r] = local; continue; }
    if (cudaIpcOpenMemHandle(&mapped[r], handles[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { mapped[r] = nullptr; ok = false; }
  }
  cudaGetLastError();
  return ok;
}
// all ranks use a peer-memory path or none does: a rank that failed would otherwise wait for arrivals that never come
static bool all_ranks_agree(CommState *c, bool ok) {
  NcclApi *api = nccl_api();
  int *flag = nullptr;
  int all = 0;
  if (cudaMalloc(&flag, sizeof(int)) == cudaSuccess) {
    const int v = ok ? 1 : 0;
    cudaMemcpy(flag, &v, sizeof(int), cudaMemcpyHostToDevice);
    if (api->AllReduce(flag, flag, 1, ncclInt, ncclMin, c->comm, c->stream) == ncclSuccess && cudaStreamSynchronize(c->stream) == cudaSuccess)
      cudaMemcpy(&all, flag, sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(flag);
  }
  cudaGetLastError();
  return ok && all == 1;
}

// Sets the peer-memory paths up.  Any failure leaves a path off; the library's collectives then do its work.
static void peer_setup(myea_b200_net *net) {
  CommState *c = net->comm;
  if (c->world > PEER_MAX_WORLD) return;
  {  // the small sums of the normalization layers: [2 parities][world slots][capacity] floats + arrival words
    PeerSum &p = c->peer;
    long long widest = 0;
    for (const auto &L : net->layers)
      if (L.has_norm) widest = std::max(widest, L.n_out);
    p.capacity = static_cast<size_t>(2 * std::max<long long>(widest, 1) + 3) & ~static_cast<size_t>(3);
    const size_t bytes = static_cast<size_t>(2) * c->world * p.capacity * sizeof(float) + static_cast<size_t>(2) * c->world * PEER_MAX_BLOCKS * sizeof(unsigned int);
    bool ok = cudaMalloc(&p.local, bytes) == cudaSuccess && cudaMemset(p.local, 0, bytes) == cudaSuccess;
    ok = ipc_map_all(c, p.local, ok, p.mapped);
    ok = ok && cudaMalloc(&p.mapped_d, c->world * sizeof(float *)) == cudaSuccess &&
         cudaMemcpy(p.mapped_d, p.mapped, c->world * sizeof(float *), cudaMemcpyHostToDevice) == cudaSuccess;
    p.ready = all_ranks_agree(c, ok);
  }
  {  // derivative buckets and updated parameters by peer copies
    PeerCopy &q = c->copy;
    const size_t floats = net->total_parameters + 4;
    const size_t words = static_cast<size_t>(2) * PEER_MAX_BUCKETS * PEER_MAX_WORLD;
    bool ok = cudaMalloc(&q.stage, floats * sizeof(float)) == cudaSuccess && cudaMalloc(&q.flags, words * sizeof(unsigned int)) == cudaSuccess &&
              cudaMemset(q.flags, 0, words * sizeof(unsigned int)) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess;
    const bool a = ipc_map_all(c, net->params, ok, q.params);
    const bool b = ipc_map_all(c, q.stage, ok, q.stages);
    const bool d = ipc_map_all(c, q.flags, ok, q.words);
    ok = ok && a && b && d;
    ok = ok && cudaMalloc(&q.words_d, c->world * sizeof(unsigned int *)) == cudaSuccess &&
         cudaMemcpy(q.words_d, q.words, c->world * sizeof(unsigned int *), cudaMemcpyHostToDevice) == cudaSuccess;
    q.ready = all_ranks_agree(c, ok);
  }
  cudaGetLastError();
}

static void peer_teardown(CommState *c) {
  PeerSum &p = c->peer;
  PeerCopy &q = c->copy;
  for (int r = 0; r < c->world && r < PEER_MAX_WORLD; ++r) {
    if (r == c->rank) continue;
    if (p.mapped[r] != nullptr) cudaIpcCloseMemHandle(p.mapped[r]);
    if (q.params[r] != nullptr) cudaIpcCloseMemHandle(q.params[r]);
    if (q.stages[r] != nullptr) cudaIpcCloseMemHandle(q.stages[r]);
    if (q.words[r] != nullptr) cudaIpcCloseMemHandle(q.words[r]);
  }
  if (p.mapped_d != nullptr) cudaFree(p.mapped_d);
  if (p.local != nullptr) cudaFree(p.local);
  if (q.words_d != nullptr) cudaFree(q.words_d);
  if (q.stage != nullptr) cudaFree(q.stage);
  if (q.flags != nullptr) cudaFree(q.flags);
  p = PeerSum();
  q = PeerCopy();
}

void comm_destroy(myea_b200_net *net) {
  if (net->comm == nullptr) return;
  NcclApi *api = nccl_api();
  // Peers may still be copying into this rank's buffers: slices of a step whose update was never asked for, parameters
  // of the last update.  Their arrival words are waited for (bounded) before anything is unmapped or freed.
  CommState *c = net->comm;
  for (size_t i = 0; i < c->used; ++i) {
    const CommState::Bucket &b = c->buckets[i];
    if (b.by_copies) peer_wait_kernel<<<1, 32, 0, net->ctx.stream>>>(c->copy.flags, 0, b.index, c->rank, c->world, b.epoch, net->ctx.d_error_flag);
  }
  comm_gather_join(net);
  if (net->ctx.stream) cudaStreamSynchronize(net->ctx.stream);
  for (cudaStream_t st : {net->comm->stream, net->comm->stream_aux, net->comm->stream_small, net->comm->stream_gather, net->comm->stream_gather_aux})
    if (st) cudaStreamSynchronize(st);
  cudaGetLastError();
  peer_teardown(net->comm);
  if (api && net->comm->comm) api->CommDestroy(net->comm->comm);
  if (net->comm->ready) cudaEventDestroy(net->comm->ready);
  if (net->comm->done) cudaEventDestroy(net->comm->done);
  if (net->comm->side_done) cudaEventDestroy(net->comm->side_done);
  for (auto &b : net->comm->buckets) {
    if (b.reduced) cudaEventDestroy(b.reduced);
    if (b.updated) cudaEventDestroy(b.updated);
    if (b.gathered) cudaEventDestroy(b.gathered);
  }
  for (cudaStream_t st : {net->comm->stream, net->comm->stream_aux, net->comm->stream_small, net->comm->stream_gather, net->comm->stream_gather_aux})
    if (st) cudaStreamDestroy(st);
  if (net->comm->aux_done) cudaEventDestroy(net->comm->aux_done);
  delete net->comm;
  net->comm = nullptr;
}

}  // namespace myea

using namespace myea;

extern "C" int myea_b200_comm_unique_id(uint8_t id_out[128]) {
  if (id_out == nullptr) return MYEA_E_INVALID;
  NcclApi *api = nccl_api();
  if (api == nullptr) return MYEA_E_COMM;
  ncclUniqueId id;
  if (api->GetUniqueId(&id) != ncclSuccess) return MYEA_E_COMM;
  static_assert(sizeof(id) == 128, "ncclUniqueId is 128 bytes");
  memcpy(id_out, &id, 128);
  return MYEA_OK;
}

extern "C" int myea_b200_comm_init(myea_handle net, int world, int rank, const uint8_t unique_id[128]) {
  if (net == nullptr || unique_id == nullptr || world < 1 || rank < 0 || rank >= world) return MYEA_E_INVALID;
  if (net->comm != nullptr) { net->ctx.error = "a communicator is already attached"; return MYEA_E_INVALID; }
  if (world == 1) return MYEA_OK;
  NcclApi *api = nccl_api();
  if (api == nullptr) { net->ctx.error = "libnccl.so.2 could not be loaded"; return MYEA_E_COMM; }
  if (cudaSetDevice(net->ctx.device) != cudaSuccess) return MYEA_E_CUDA;
  CommState *c = new CommState();
  c->world = world;
  c->rank = rank;
  ncclUniqueId id;
  memcpy(&id, unique_id, 128);
  ncclResult_t r = api->CommInitRank(&c->comm, world, id, rank);
  if (r != ncclSuccess) { delete c; return nccl_fail(net, r, "ncclCommInitRank"); }
  if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&c->stream_aux, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&c->stream_small, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&c->stream_gather, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&c->stream_gather_aux, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&c->aux_done, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&c->ready, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&c->side_done, cudaEventDisableTiming) != cudaSuccess) {
    api->CommDestroy(c->comm);
    if (c->stream) cudaStreamDestroy(c->stream);
    if (c->stream_aux) cudaStreamDestroy(c->stream_aux);
    if (c->stream_small) cudaStreamDestroy(c->stream_small);
    if (c->stream_gather) cudaStreamDestroy(c->stream_gather);
    if (c->stream_gather_aux) cudaStreamDestroy(c->stream_gather_aux);
    if (c->aux_done) cudaEventDestroy(c->aux_done);
    if (c->ready) cudaEventDestroy(c->ready);
    if (c->done) cudaEventDestroy(c->done);
    if (c->side_done) cudaEventDestroy(c->side_done);
    delete c;
    net->ctx.error = "stream / event creation failed";
    return MYEA_E_CUDA;
  }
  net->comm = c;
  peer_setup(net);  // optional: without it the small sums go through the library
  net->hook.world = world;
  net->hook.user = net;
  net->hook.all_reduce = [](void *user, float *buf, size_t n) { return comm_all_reduce_sum(static_cast<myea_b200_net *>(user), buf, n); };
  net->hook.begin = [](void *user, float *buf, size_t n) { return comm_side_sum_begin(static_cast<myea_b200_net *>(user), buf, n); };
  net->hook.end = [](void *user) { return comm_side_sum_end(static_cast<myea_b200_net *>(user)); };
  return MYEA_OK;
}

// Diagnostic (not part of the training interface): 1 when the small cross-rank sums of this handle go through the
// peer-memory exchange kernel, 0 when they use the library's all-reduce.
extern "C" int myea_b200_comm_peer_sums(myea_handle net) { return (net != nullptr && net->comm != nullptr && net->comm->peer.ready) ? 1 : 0; }
// 1 when derivative buckets and updated parameters travel by peer copies, 0 when the library's collectives move them
extern "C" int myea_b200_comm_peer_copies(myea_handle net) { return (net != nullptr && net->comm != nullptr && net->comm->copy.ready) ? 1 : 0; }
