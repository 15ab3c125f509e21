// trimul_sm100_forward_static: the single-GPU TriMul forward for callers that must not allocate.
//
// Some hosts of this library cannot hand it freshly allocated device memory: an inference server
// whose own pool already owns the whole GPU, a plugin that runs inside a sandbox where allocation
// calls are off limits, or a latency-critical loop where cudaMalloc's implicit device
// synchronisation is unacceptable.  The regular entry point (trimul_sm100_forward) asks such a
// caller for three scratch buffers (the a|b operand planes, the contraction result and the output
// gate) that it has no way to provide.  This variant carries that scratch itself, in one
// statically sized array inside the library image: the caller passes only inputs, weights and the
// output.  Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
//
// Price and limits
//   * the array is kTrimulStaticScratchBytes (32 MiB) and every GPU that loads the library holds
//     it until the process exits, used or not;
//   * the scratch needs 8 * batch * n * n * d bytes, so shapes with batch*n*n*d > 4 Mi elements
//     (for example n > 128 at d = 256, batch = 1) are refused with TRIMUL_ERR_UNSUPPORTED_SHAPE;
//   * every call on a device uses the SAME array: two calls whose kernels overlap on the GPU (two
//     streams, two host threads) race on it and corrupt each other.  Issue them on one stream, or
//     order them yourself;
//   * the array keeps whatever the previous call left in it.  This forward overwrites every
//     element it later reads (all operand planes, the whole gate, the whole contraction result),
//     so nothing has to be cleared between calls and nothing is.
//   * the first call on each device resolves the array's device address (cudaGetSymbolAddress,
//     with that device current -- the device that owns `stream` must be the current device).  Make
//     that first call outside any stream capture; later calls on the same device reuse the cached
//     address.  The cache lives as long as the process: after a cudaDeviceReset the cached address
//     is stale and this entry point must not be used again in that process.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/trimul_sm100.h"

namespace {

constexpr size_t kTrimulStaticScratchBytes = TRIMUL_STATIC_SCRATCH_BYTES;  // the capacity the header promises

// File-scope device array.  In host code this NAME is only a handle for the runtime's symbol
// table, not a device pointer: it must never be passed to a kernel or used in pointer arithmetic.
// The device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_trimul_static_scratch[kTrimulStaticScratchBytes];

constexpr int kMaxDevices = 64;
// Per-device address of the array, resolved on first use.  Atomic slots: host threads may race on
// their first calls; every racer resolves the same address, so the last store wins harmlessly.
std::atomic<void*> g_scratch_addr[kMaxDevices];

// Device address of the scratch array on the CURRENT device (resolved once per device).
int scratch_base(unsigned char** out, char* msg, size_t msg_len) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(msg, msg_len, "forward_static: cannot identify the current device (%s)",
             cudaGetErrorString(e));
    return TRIMUL_ERR_CUDA;
  }
  void* ptr = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    e = cudaGetSymbolAddress(&ptr, g_trimul_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      snprintf(msg, msg_len, "forward_static: cudaGetSymbolAddress failed on device %d (%s)", dev,
               cudaGetErrorString(e));
      return TRIMUL_ERR_CUDA;
    }
    g_scratch_addr[dev].store(ptr, std::memory_order_release);
  }
  *out = static_cast<unsigned char*>(ptr);
  return TRIMUL_OK;
}

size_t round256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

namespace trimul {
void set_last_error(const char* msg);  // defined next to trimul_sm100_last_error
}

extern "C" {

int trimul_sm100_forward_static(const trimul_geom_t* geom, const void* x, const void* mask, int32_t mask_kind,
                                const float* ln_in_w, const float* ln_in_b, const void* w_packed,
                                const float* bias_packed, const void* w_fold, const float* cd, void* out,
                                trimul_status_t* status, uint64_t timeout_ns, trimul_stream_t stream) {
  char msg[384];
  trimul_workspace_t ws;
  int rc = trimul_sm100_workspace(geom, &ws);  // validates the geometry and leaves its own message on failure
  if (rc != TRIMUL_OK) return rc;
  if (geom->cp0 != 1 || geom->cp1 != 1) {
    trimul::set_last_error("forward_static: single-GPU only, the cp grid must be 1 x 1");
    return TRIMUL_ERR_INVALID_ARGUMENT;
  }
  const size_t ab_off = 0;
  const size_t tri_off = round256(ws.ab_bytes);
  const size_t gate_off = tri_off + round256(ws.tri_bytes);
  const size_t need = gate_off + round256(ws.gate_bytes);
  if (need > kTrimulStaticScratchBytes) {
    snprintf(msg, sizeof(msg),
             "forward_static: batch=%d n=%d d=%d needs %zu bytes of scratch but the built-in array holds %zu "
             "(8*batch*n*n*d bytes must fit); use trimul_sm100_forward with caller-provided buffers",
             geom->batch, geom->n, geom->d, need, kTrimulStaticScratchBytes);
    trimul::set_last_error(msg);
    return TRIMUL_ERR_UNSUPPORTED_SHAPE;
  }
  unsigned char* base = nullptr;
  rc = scratch_base(&base, msg, sizeof(msg));
  if (rc != TRIMUL_OK) {
    trimul::set_last_error(msg);
    return rc;
  }
  return trimul_sm100_forward(geom, x, mask, mask_kind, ln_in_w, ln_in_b, w_packed, bias_packed, w_fold, cd,
                              base + ab_off, base + tri_off, base + gate_off, out, status, timeout_ns, stream);
}

}  // extern "C"
