// Peer-memory runtime: device allocations that other processes on the same NVLink domain can map, the
// handle export/import calls, and small cross-GPU signalling kernels (flag set / bounded flag wait).
// This is the plumbing under the fused weight-sync, reduce-scatter+AdamW and all-gather kernels; it plays
// the role that NCCL unique-id exchange + ncclSend/Recv plays in the reference
// (cosmos_rl/utils/pynccl.py:546-921, cosmos_rl/collective/collective.py:39-423): handles are exchanged
// through the controller's key/value store exactly like NCCL ids.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "api.h"
#include "sm100.cuh"

extern "C" {

// cudaMalloc'ed (not pool / not VMM) memory: the only kind legacy CUDA IPC can export.
int b200_peer_alloc(void** out, unsigned long long bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return B200_ERR_RUNTIME; }
  if (cudaMemset(p, 0, bytes) != cudaSuccess) { cudaGetLastError(); cudaFree(p); return B200_ERR_RUNTIME; }
  *out = p;
  return 0;
}

int b200_peer_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : B200_ERR_RUNTIME; }

// handle_out: 64 bytes
int b200_peer_export(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaGetLastError(); return B200_ERR_RUNTIME; }
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

int b200_peer_open(const void* handle_in, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_in, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return B200_ERR_RUNTIME;
  }
  *out = p;
  return 0;
}

int b200_peer_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : B200_ERR_RUNTIME; }

int b200_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) { cudaGetLastError(); return 0; }
  return ok;
}

}  // extern "C"

namespace {

__global__ void flag_set_kernel(volatile uint32_t* flag, uint32_t value) {
  __threadfence_system();
  *flag = value;
}

// Wait until *flag >= value, for at most WAIT_LIMIT_NS; on a timeout record ST_TIMEOUT_PEER_FLAG.
__global__ void flag_wait_kernel(volatile uint32_t* flag, uint32_t value, uint32_t* status,
                                 unsigned long long limit_ns) {
  const unsigned long long t0 = b200::globaltimer_ns();
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int32_t)(v - value) >= 0) return;
    if (b200::globaltimer_ns() - t0 > limit_ns) {
      atomicCAS(status, b200::ST_OK, b200::ST_TIMEOUT_PEER_FLAG);
      return;
    }
    __nanosleep(200);
  }
}

}  // namespace

extern "C" {

// Stream-ordered flag write (release, system scope): everything enqueued before it on `stream` is visible to
// a peer that observes the new value.
int b200_flag_set(uint32_t* flag, uint32_t value, cudaStream_t stream) {
  flag_set_kernel<<<1, 1, 0, stream>>>(flag, value);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

// Stream-ordered bounded wait on a (possibly remote) flag. Never launch this on the same GPU as the kernel
// that is supposed to set the flag unless that kernel was enqueued earlier on the same stream.
int b200_flag_wait(uint32_t* flag, uint32_t value, uint32_t* status, unsigned long long limit_ns,
                   cudaStream_t stream) {
  flag_wait_kernel<<<1, 1, 0, stream>>>(flag, value, status, limit_ns);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"
