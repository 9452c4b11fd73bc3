// All-reduce of row-parallel partial outputs over the peers' memory (include/sage_b200_peer.h):
// push the partial rows into every peer's exchange over NVLink, publish an epoch flag, wait
// (bounded) for the peers' flags in local memory, sum in rank order.  One launch per rank.
//
// Exchange layout (one allocation per rank, mapped by all peers):
//   [0, 4096)            epochs[kPeerCtas]            calls made so far, per CTA (local use only)
//   [4096, 8192)         flags[world][kPeerCtas]      flags[r][c]: last epoch rank r's CTA c published
//   [8192, ...)          slots                        FP16 partials of both parities and all ranks, interleaved in
//                                                     512-byte blocks: block b of the data sits at
//                                                     ((b * 2 + parity) * world + rank) * 512 bytes, so a small
//                                                     message stays within a few pages however large the
//                                                     exchange is, and a warp still moves 512 contiguous bytes
//
// CTA c of every rank owns the same 16-byte chunks (c * 512 + t, stride 64 * 512), so the
// handshake is per CTA: no grid-wide step.  A call moves (world - 1) * 2 * elements bytes out of
// and into every GPU; for a decode row (a few KB) it is bound by one NVLink store latency plus one
// flag store, not by bandwidth.
#include <string.h>

#include "../../include/sage_b200.h"
#include "../../include/sage_b200_peer.h"
#include "sage_common.cuh"
#include "sage_kernels.h"

namespace sageb200 {
namespace {

constexpr int kPeerCtas = 64;  // (a decode row uses the first one or two; a chunk of prompt rows all of them)
constexpr int kPeerThreads = 512;
constexpr size_t kFlagOffset = 4096;
constexpr size_t kSlotOffset = 8192;
constexpr long long kPeerWaitNs = 2000000000ll;  // two seconds, then the time-out status
constexpr long long kPeerMaxCapacity = 1ll << 26;

struct PeerParams {
  unsigned char *exchange[SAGEB200_PEER_MAX_WORLD];
  uint4 *data;
  long long capacity;  // elements per slot
  int chunks;          // 16-byte chunks of `data`
  int world, rank;
  int *status;
};

__device__ __forceinline__ unsigned load_acquire_system(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_release_system(unsigned *p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void add_halves(float (&acc)[8], const uint4 &v) {
  const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 f = __half22float2(h[q]);
    acc[2 * q] += f.x;
    acc[2 * q + 1] += f.y;
  }
}

__global__ void __launch_bounds__(kPeerThreads) peer_all_reduce_kernel(const __grid_constant__ PeerParams p) {
  const int cta = blockIdx.x, tid = threadIdx.x;
  // The next kernel of the stream may be scheduled now (it runs its own prologue and then waits
  // for this grid to complete); this grid itself was scheduled while its producer still ran and
  // waits here for the producer's rows, and for the previous call's epoch update.
  pdl_launch_dependents();
  pdl_wait();
  if (cta * kPeerThreads >= p.chunks) return;  // (the same CTAs on every rank: same `chunks`)
  __shared__ unsigned epoch_shared;
  __shared__ int abort_shared;
  unsigned char *own = p.exchange[p.rank];
  if (tid == 0) {
    unsigned *epochs = reinterpret_cast<unsigned *>(own);
    const unsigned e = epochs[cta] + 1u;
    epochs[cta] = e;
    epoch_shared = e;
    abort_shared = 0;
  }
  __syncthreads();
  const unsigned epoch = epoch_shared;
  const unsigned parity = epoch & 1u;
  // 16-byte chunk i of rank r's partial, this call's parity (see the layout above)
  auto slot_index = [&](int i, int r) {
    return ((static_cast<size_t>(i >> 5) * 2 + parity) * p.world + r) * 32 + (i & 31);
  };

  // ---- push this rank's chunks into slot [parity][rank] of every peer
  for (int i = cta * kPeerThreads + tid; i < p.chunks; i += kPeerCtas * kPeerThreads) {
    const uint4 v = p.data[i];
    for (int w = 0; w < p.world; ++w) {
      if (w == p.rank) continue;
      uint4 *slots = reinterpret_cast<uint4 *>(p.exchange[w] + kSlotOffset);
      slots[slot_index(i, p.rank)] = v;
    }
  }
  __syncthreads();
  // ---- publish (the release orders the CTA's stores above, which the barrier made visible to
  //      this thread, before the flag), then wait for the peers' flags in local memory
  if (tid < p.world && tid != p.rank) {
    __threadfence_system();
    unsigned *peer_flags = reinterpret_cast<unsigned *>(p.exchange[tid] + kFlagOffset);
    store_release_system(peer_flags + p.rank * kPeerCtas + cta, epoch);
    const unsigned *flag = reinterpret_cast<const unsigned *>(own + kFlagOffset) + tid * kPeerCtas + cta;
    if (static_cast<int>(load_acquire_system(flag) - epoch) < 0) {
      const long long begin = global_nanoseconds();
      unsigned spins = 0;
      while (static_cast<int>(load_acquire_system(flag) - epoch) < 0) {
        if ((++spins & 63u) == 0 && global_nanoseconds() - begin > kPeerWaitNs) {
          if (p.status) atomicExch(p.status, SAGEB200_ERR_TIMEOUT);
          abort_shared = 1;
          break;
        }
      }
    }
  }
  __syncthreads();
  if (abort_shared) return;  // (the output keeps this rank's partial; the status word says so)

  // ---- reduce in rank order
  const uint4 *own_slots = reinterpret_cast<const uint4 *>(own + kSlotOffset);
  for (int i = cta * kPeerThreads + tid; i < p.chunks; i += kPeerCtas * kPeerThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < p.world; ++w) {
      const uint4 v = w == p.rank ? p.data[i] : __ldcg(own_slots + slot_index(i, w));
      add_halves(acc, v);
    }
    uint4 out;
    __half2 *h = reinterpret_cast<__half2 *>(&out);
#pragma unroll
    for (int q = 0; q < 4; ++q) h[q] = __floats2half2_rn(acc[2 * q], acc[2 * q + 1]);
    p.data[i] = out;
  }
}

bool exchange_arguments_ok(int world, long long capacity) {
  return world >= 2 && world <= SAGEB200_PEER_MAX_WORLD && capacity >= 8 && (capacity & 7) == 0 &&
         capacity <= kPeerMaxCapacity;
}

}  // namespace
}  // namespace sageb200

using namespace sageb200;

extern "C" {

size_t sageb200_peer_exchange_bytes(int world, long long capacity) {
  if (!exchange_arguments_ok(world, capacity)) return 0;
  const size_t padded = (static_cast<size_t>(capacity) + 255) / 256 * 256;  // whole 512-byte blocks
  return kSlotOffset + static_cast<size_t>(2) * world * padded * sizeof(__half);
}

int sageb200_peer_create(int world, long long capacity, void **exchange, unsigned char *handle) {
  if (!exchange || !handle) return SAGEB200_ERR_INVALID_ARGUMENT;
  const size_t bytes = sageb200_peer_exchange_bytes(world, capacity);
  if (bytes == 0) return SAGEB200_ERR_INVALID_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == SAGEB200_PEER_HANDLE_BYTES, "IPC handle size");
  void *memory = nullptr;
  if (cudaMalloc(&memory, bytes) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  cudaIpcMemHandle_t ipc;
  if (cudaMemset(memory, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
      cudaIpcGetMemHandle(&ipc, memory) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(memory);
    return SAGEB200_ERR_CUDA;
  }
  memcpy(handle, &ipc, sizeof(ipc));
  *exchange = memory;
  return SAGEB200_OK;
}

int sageb200_peer_open(const unsigned char *handle, void **exchange) {
  if (!handle || !exchange) return SAGEB200_ERR_INVALID_ARGUMENT;
  cudaIpcMemHandle_t ipc;
  memcpy(&ipc, handle, sizeof(ipc));
  void *memory = nullptr;
  if (cudaIpcOpenMemHandle(&memory, ipc, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  *exchange = memory;
  return SAGEB200_OK;
}

int sageb200_peer_close(void *peer_exchange) {
  if (!peer_exchange) return SAGEB200_ERR_INVALID_ARGUMENT;
  if (cudaIpcCloseMemHandle(peer_exchange) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  return SAGEB200_OK;
}

int sageb200_peer_destroy(void *own_exchange) {
  if (!own_exchange) return SAGEB200_ERR_INVALID_ARGUMENT;
  if (cudaFree(own_exchange) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  return SAGEB200_OK;
}

int sageb200_peer_all_reduce(void *const *exchanges, int world, int rank, long long capacity, void *data,
                             long long elements, void *stream) {
  if (!exchanges || !data || !exchange_arguments_ok(world, capacity) || rank < 0 || rank >= world ||
      elements <= 0 || (elements & 7) || elements > capacity)
    return SAGEB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(data) & 15) return SAGEB200_ERR_ALIGNMENT;
  PeerParams params = {};
  for (int r = 0; r < world; ++r) {
    if (!exchanges[r]) return SAGEB200_ERR_INVALID_ARGUMENT;
    params.exchange[r] = static_cast<unsigned char *>(exchanges[r]);
  }
  int *status_word = nullptr;
  int sm_count = 0;
  const int state = acquire_device(&status_word, &sm_count);
  if (state != SAGEB200_OK) return state;
  params.data = static_cast<uint4 *>(data);
  params.capacity = capacity;
  params.chunks = static_cast<int>(elements >> 3);
  params.world = world;
  params.rank = rank;
  params.status = status_word;
  if (launch_dependent<1>(peer_all_reduce_kernel, kPeerCtas, kPeerThreads, 0, static_cast<cudaStream_t>(stream),
                          params) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  count_launches(1);
  return SAGEB200_OK;
}

}  // extern "C"
