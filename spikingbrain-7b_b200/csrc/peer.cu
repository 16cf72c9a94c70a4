// Peer memory for the head-sharded decode step: buffers that the other GPUs of one NVSwitch
// domain can store into, the flags they raise when a step's stores are complete, and the
// bounded wait on those flags.
//
// One process drives one GPU. A gathered-output buffer is plain device memory (cudaMalloc) of
// this process; its IPC handle is handed to the other processes by the host (the caller owns
// that exchange: any byte transport will do), which map it and get an address their kernels
// can store to through NVLink. Only plain stores and loads cross the link -- no multicast
// object is created and no copy engine or tensor-map load ever gets a peer address.
//
// Protocol of one step s (s grows by one per step, never reused):
//   writer r:   stores its head slice of every output row into each peer's buffer, then
//               fence (system scope) -> count finished CTAs -> the last one stores s into
//               flag[r] of each peer with release semantics        (sbk_swa_decode_gather)
//               (s = flag_value + *flag_base when a base word is given: a captured graph stores
//               the same relative value at every replay while the base counts the steps)
//   reader:     one thread per peer polls flag[peer] with acquire loads until it is >= s,
//               for at most `timeout_ms`; a wait that runs out raises SBK_ST_WAIT_TIMEOUT in
//               the status word and returns, the context stays usable; either way it then
//               adds `advance` to *flag_base                                (sbk_peer_wait)
// The wait is a kernel of its own in the reader's stream: whatever is enqueued behind it sees
// the complete [tokens, all heads, D] rows.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "sbk_common.cuh"

namespace sbk {

__global__ void peer_wait_kernel(const int32_t* flags, int n, int self, int32_t value, int32_t* flag_base,
                                 int32_t advance, uint64_t timeout_ns, int32_t* status) {
  const int p = threadIdx.x;
  const int32_t base = flag_base ? __ldcg(flag_base) : 0;
  const int32_t target = value + base;
  if (p < n && p != self) {
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool seen = false;
    // two limits: wall time on the device, and a poll count in case the timer does not advance
    for (uint32_t i = 0; i < (1u << 26); ++i) {
      int32_t v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + p) : "memory");
      if (v - target >= 0) { seen = true; break; }
      __nanosleep(100);
      uint64_t t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t - t0 > timeout_ns) break;
    }
    if (!seen) raise_status(status, SBK_ST_WAIT_TIMEOUT);
  }
  __syncwarp();
  // the step counter moves on whether or not the peers delivered: later steps keep their numbers
  if (p == 0 && flag_base && advance) *flag_base = base + advance;
}

__global__ void peer_signal_kernel(Int32PtrTable flags, int n, int32_t value, const int32_t* flag_base) {
  const int p = threadIdx.x;
  if (p >= n) return;
  const int32_t v = value + (flag_base ? __ldcg(flag_base) : 0);
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags.p[p]), "r"(v) : "memory");
}

}  // namespace sbk

extern "C" int sbk_peer_alloc(size_t bytes, void** ptr) {
  using namespace sbk;
  if (!ptr || bytes == 0) {
    set_error("sbk_peer_alloc: null result pointer or zero size");
    return SBK_E_ARG;
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    set_error("sbk_peer_alloc: %zu bytes: %s", bytes, cudaGetErrorString(e));
    (void)cudaGetLastError();
    return SBK_E_LAUNCH;
  }
  *ptr = p;
  return SBK_OK;
}

extern "C" int sbk_peer_free(void* ptr) {
  using namespace sbk;
  if (!ptr) return SBK_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) {
    set_error("sbk_peer_free: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return SBK_E_LAUNCH;
  }
  return SBK_OK;
}

extern "C" int sbk_peer_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

extern "C" int sbk_peer_export(const void* ptr, void* handle, int handle_bytes) {
  using namespace sbk;
  if (!ptr || !handle || handle_bytes != (int)sizeof(cudaIpcMemHandle_t)) {
    set_error("sbk_peer_export: null pointer or a handle buffer that is not %d bytes",
              (int)sizeof(cudaIpcMemHandle_t));
    return SBK_E_ARG;
  }
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
  if (e != cudaSuccess) {
    set_error("sbk_peer_export: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return SBK_E_LAUNCH;
  }
  memcpy(handle, &h, sizeof(h));
  return SBK_OK;
}

extern "C" int sbk_peer_open(const void* handle, int handle_bytes, void** ptr) {
  using namespace sbk;
  if (!ptr || !handle || handle_bytes != (int)sizeof(cudaIpcMemHandle_t)) {
    set_error("sbk_peer_open: null pointer or a handle that is not %d bytes", (int)sizeof(cudaIpcMemHandle_t));
    return SBK_E_ARG;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    set_error("sbk_peer_open: %s (the owner must be another process on a GPU with peer access to this one)",
              cudaGetErrorString(e));
    (void)cudaGetLastError();
    return SBK_E_LAUNCH;
  }
  *ptr = p;
  return SBK_OK;
}

extern "C" int sbk_peer_close(void* ptr) {
  using namespace sbk;
  if (!ptr) return SBK_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) {
    set_error("sbk_peer_close: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return SBK_E_LAUNCH;
  }
  return SBK_OK;
}

extern "C" int sbk_peer_wait(const int32_t* flags, int n, int self, int32_t value, int32_t* flag_base,
                             int32_t advance, int timeout_ms, int32_t* status, void* stream) {
  using namespace sbk;
  if (!flags || n < 1 || n > 32 || timeout_ms < 1 || timeout_ms > 60000) {
    set_error("sbk_peer_wait: need a flag array of 1..32 ranks and a timeout of 1..60000 ms (n=%d, %d ms)", n,
              timeout_ms);
    return SBK_E_ARG;
  }
  peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, n, self, value, flag_base, advance,
                                                      (uint64_t)timeout_ms * 1000000ull, status);
  return check_launch("sbk_peer_wait");
}

extern "C" int sbk_peer_signal(int32_t* const* peer_flag, int n_peer, int32_t value, const int32_t* flag_base,
                               void* stream) {
  using namespace sbk;
  if (n_peer < 0 || n_peer > kPeerTableSize || (n_peer > 0 && !peer_flag)) {
    set_error("sbk_peer_signal: n_peer=%d outside [0,%d] or null table", n_peer, kPeerTableSize);
    return SBK_E_ARG;
  }
  if (n_peer == 0) return SBK_OK;
  Int32PtrTable t;
  for (int p = 0; p < kPeerTableSize; ++p) t.p[p] = p < n_peer ? peer_flag[p] : nullptr;
  peer_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(t, n_peer, value, flag_base);
  return check_launch("sbk_peer_signal");
}
