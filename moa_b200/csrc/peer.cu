// Buffers that the GPUs of one node write into directly, and a barrier across their ranks.
//
// With heads sharded over G GPUs, every rank's decode kernel stores its output rows straight into the
// (B, 1, H, D) gather buffer of every rank (plain stores over NVLink, moa_decode_gather_fwd), instead of
// an all-gather collective plus a permuting copy afterwards.  This file provides what that needs around
// the kernel: device buffers that other processes of the node can map (CUDA IPC), and a barrier kernel
// that orders "all ranks have stored" before "any rank reads" through flag words in those buffers.
//
// The barrier's wait is bounded like every wait in this library: when it runs out the kernel writes a
// status word and returns.  Nothing here loads bulk data from a peer and no multicast object is used.
#include <string.h>

#include "common.cuh"

namespace moa {
namespace {

constexpr int kMaxPeers = 8;

struct BarrierParams {
  uint32_t* flags[kMaxPeers];   // flags[g]: rank g's flag words (one per rank), mapped into this process
  int rank, world;
  uint32_t epoch;
  uint32_t* epoch_counter;      // this rank's call counter in device memory, or nullptr: `epoch` is used
  long long limit_cycles;
  int32_t* status;              // int32[4]: [0] = 21 when the wait ran out, [1] = the rank waited for, [2] = epoch
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Thread g tells rank g "rank `rank` has reached `epoch`" and waits until rank g has told this rank the same.
// Everything this rank's stream did before the barrier (the decode kernel's stores into the peers' buffers)
// is ordered before the release; everything after the barrier on this stream follows the acquires.
__global__ void peer_barrier_kernel(const BarrierParams p) {
  __shared__ uint32_t epoch_shared;
  const int g = threadIdx.x;
  if (g == 0) {
    // The call's number: given by the host, or counted on the device (the form a CUDA graph can replay).
    uint32_t e = p.epoch;
    if (p.epoch_counter != nullptr) {
      e = *p.epoch_counter + 1u;
      *p.epoch_counter = e;
    }
    epoch_shared = e;
  }
  __syncthreads();
  if (g >= p.world) return;
  const uint32_t epoch = epoch_shared;
  __threadfence_system();
  st_release_sys(p.flags[g] + p.rank, epoch);
  const uint32_t* mine = p.flags[p.rank] + g;
  const long long t0 = clock64();
  for (uint32_t spin = 1;; ++spin) {
    if ((int32_t)(ld_acquire_sys(mine) - epoch) >= 0) break;
    if ((spin & 63u) == 0 && clock64() - t0 > p.limit_cycles) {
      if (atomicCAS(&p.status[0], 0, 21) == 0) {
        p.status[1] = g;
        p.status[2] = (int32_t)epoch;
        p.status[3] = p.rank;
      }
      break;
    }
  }
  __threadfence_system();
}

}  // namespace
}  // namespace moa

extern "C" {

int moa_peer_alloc(void** ptr, int64_t bytes) {
  MOA_REQUIRE(ptr != nullptr && bytes > 0, "peer_alloc: bad arguments");
  MOA_CUDA_CHECK(cudaMalloc(ptr, (size_t)bytes));
  MOA_CUDA_CHECK(cudaMemset(*ptr, 0, (size_t)bytes));
  return MOA_OK;
}

int moa_peer_free(void* ptr) {
  if (ptr) MOA_CUDA_CHECK(cudaFree(ptr));
  return MOA_OK;
}

int moa_peer_export(void* ptr, void* handle) {
  MOA_REQUIRE(ptr && handle, "peer_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == MOA_PEER_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  MOA_CUDA_CHECK(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle, &h, sizeof(h));
  return MOA_OK;
}

int moa_peer_open(const void* handle, void** ptr) {
  MOA_REQUIRE(ptr && handle, "peer_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  MOA_CUDA_CHECK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return MOA_OK;
}

int moa_peer_close(void* ptr) {
  if (ptr) MOA_CUDA_CHECK(cudaIpcCloseMemHandle(ptr));
  return MOA_OK;
}

int moa_peer_barrier(void* const* flags, int rank, int world, uint32_t epoch, uint32_t* epoch_counter,
                     int64_t limit_cycles, int32_t* status, moa_stream_t stream) {
  using namespace moa;
  MOA_REQUIRE(flags && status, "peer_barrier: null pointer");
  MOA_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, "peer_barrier: 1..8 ranks");
  MOA_REQUIRE(limit_cycles > 0 && limit_cycles <= 20000000000ll, "peer_barrier: limit must be within (0, 2e10] cycles");
  BarrierParams p;
  for (int g = 0; g < kMaxPeers; ++g) p.flags[g] = g < world ? reinterpret_cast<uint32_t*>(flags[g]) : nullptr;
  for (int g = 0; g < world; ++g) MOA_REQUIRE(p.flags[g] != nullptr, "peer_barrier: null flag pointer");
  p.rank = rank; p.world = world; p.epoch = epoch; p.epoch_counter = epoch_counter;
  p.limit_cycles = (long long)limit_cycles; p.status = status;
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(p);
  MOA_CUDA_CHECK(cudaGetLastError());
  return MOA_OK;
}

}  // extern "C"
