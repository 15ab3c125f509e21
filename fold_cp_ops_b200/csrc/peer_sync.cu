// Rank-to-rank ordering for the two fused reshards: monotonically increasing counters in a small
// symmetric flag array on every rank.  After a kernel whose epilogue stored into the peers'
// buffers, `peer_signal` adds 1 to one counter slot on every rank of the cp group (release at
// system scope); before the kernel that reads what the peers stored, `peer_wait` polls the local
// slot (acquire at system scope) until it reaches the expected count.  Both are single-CTA
// launches on the caller's stream; there is no host synchronisation and no NCCL call.
// (Takes over `_A2ADeviceSignal` / `_DeviceSignalKernel` and the quiet + barrier_all drains of
//  fold_cp_ops/distributed/workflows/trimul_autotuned.py:322-560, 3272-3300.)
//
// The wait is bounded: after `timeout_ns` it records a status and returns, so a peer that never
// arrives costs one error report, not a hung GPU.
#include <stdarg.h>
#include <stdio.h>

#include "../../include/trimul_sm100.h"
#include "trimul_common.cuh"

namespace trimul {

__global__ void peer_signal_kernel(PeerPtrs flags, int cp, int slot) {
  const int r = threadIdx.x;
  if (r < cp) {
    unsigned long long* f = static_cast<unsigned long long*>(flags.ptr[r]) + slot;
    __threadfence_system();  // everything this stream stored before the launch is ordered first
    asm volatile("red.release.sys.global.add.u64 [%0], 1;" ::"l"(f) : "memory");
  }
}

__global__ void peer_wait_kernel(const unsigned long long* local_flags, int slot, unsigned long long expected,
                                 DeviceStatus* status, unsigned long long* timeline, uint64_t timeout_ns) {
  if (threadIdx.x != 0) return;
  const unsigned long long* f = local_flags + slot;
  const uint64_t t0 = sm100::globaltimer_ns();
  if (timeline != nullptr && slot < 3) timeline[kTlWaitBase + 2 * slot] = t0;
  unsigned long long v;
  uint32_t spins = 0;
  while (true) {
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(f) : "memory");
    if (v >= expected) break;
    if ((++spins & 0xff) == 0 && sm100::globaltimer_ns() - t0 > timeout_ns) {
      report_timeout(status, kKernelPeerSync, slot, static_cast<int>(v));
      break;
    }
    __nanosleep(64);
  }
  if (timeline != nullptr && slot < 3) timeline[kTlWaitBase + 2 * slot + 1] = sm100::globaltimer_ns();
}

}  // namespace trimul

extern "C" {

int trimul_sm100_peer_signal(void* const* flag_peers, int32_t cp, int32_t slot, trimul_stream_t stream) {
  if (flag_peers == nullptr || cp < 1 || cp > TRIMUL_MAX_PEERS || slot < 0 || slot >= 16) return TRIMUL_ERR_INVALID_ARGUMENT;
  trimul::PeerPtrs p;
  for (int i = 0; i < trimul::kMaxPeers; ++i) p.ptr[i] = (i < cp) ? flag_peers[i] : nullptr;
  for (int i = 0; i < cp; ++i)
    if (p.ptr[i] == nullptr) return TRIMUL_ERR_INVALID_ARGUMENT;
  trimul::peer_signal_kernel<<<1, 32, 0, stream>>>(p, cp, slot);
  return cudaGetLastError() == cudaSuccess ? TRIMUL_OK : TRIMUL_ERR_CUDA;
}

int trimul_sm100_peer_wait(const void* local_flags, int32_t slot, uint64_t expected, trimul_status_t* status,
                           uint64_t* timeline, uint64_t timeout_ns, trimul_stream_t stream) {
  if (local_flags == nullptr || slot < 0 || slot >= 16) return TRIMUL_ERR_INVALID_ARGUMENT;
  trimul::peer_wait_kernel<<<1, 32, 0, stream>>>(static_cast<const unsigned long long*>(local_flags), slot,
                                                 static_cast<unsigned long long>(expected),
                                                 reinterpret_cast<trimul::DeviceStatus*>(status),
                                                 reinterpret_cast<unsigned long long*>(timeline),
                                                 timeout_ns ? timeout_ns : 2000000000ull);
  return cudaGetLastError() == cudaSuccess ? TRIMUL_OK : TRIMUL_ERR_CUDA;
}

}  // extern "C"
