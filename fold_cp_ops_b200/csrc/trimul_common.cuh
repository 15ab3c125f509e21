// Shared definitions for the three TriMul kernels: status word, peer table, launch helpers.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace trimul {

constexpr int kMaxPeers = 8;  // one NVSwitch domain: up to 8 ranks in the cp group

// Kernel ids reported in the status word.
enum KernelId : int { kKernelGatedProj = 1, kKernelTriContract = 2, kKernelOutProj = 3, kKernelPeerSync = 4 };

// status[0] = 0 OK | 1 bounded wait expired ; [1] kernel id ; [2] block ; [3] role ; [4] detail
struct DeviceStatus {
  int code;
  int kernel;
  int block;
  int role;
  int detail;
  int pad[3];
};

__device__ __forceinline__ void report_timeout(DeviceStatus* st, int kernel, int role, int detail) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, 1) == 0) {
    st->kernel = kernel;
    st->block = static_cast<int>(blockIdx.x);
    st->role = role;
    st->detail = detail;
    __threadfence_system();
  }
}

// Optional device timeline of one forward: sixteen %globaltimer values (ns) per rank.  "First"
// slots are reduced with atomicMin over the CTAs of a kernel (the host presets them to all ones),
// "last" slots with atomicMax (preset 0); the flag waits write their entry and exit times.  One
// atomic per CTA per slot: free next to a kernel's run time.  A null pointer switches it off.
enum TimelineSlot : int {
  kTlFrontStart = 0,        // min: projection kernel, first CTA running
  kTlFrontFirstStore = 1,   // min: first a|b store issued (local or peer)
  kTlFrontLastStore = 2,    // max: last store of the kernel performed
  kTlContractStart = 3,     // min
  kTlContractLastStore = 4, // max
  kTlOutStart = 5,          // min
  kTlOutEnd = 6,            // max
  kTlWaitBase = 8,          // + 2 * flag slot: wait entry, + 1: wait exit (FRONT, BACK, CONSUMED)
  kTlSlots = 16,
};

__device__ __forceinline__ void timeline_min(unsigned long long* tl, int slot) {
  if (tl != nullptr) atomicMin(tl + slot, static_cast<unsigned long long>(sm100::globaltimer_ns()));
}
__device__ __forceinline__ void timeline_max(unsigned long long* tl, int slot) {
  if (tl != nullptr) atomicMax(tl + slot, static_cast<unsigned long long>(sm100::globaltimer_ns()));
}

// Order in which the contraction kernels walk the output tiles of one plane.  The plane's tile grid is cut
// into bands of `band_rows` tile rows; inside a band the walk is column by column.  The CTAs of one wave hold
// consecutive tiles, so a wave covers about band_rows x (wave / band_rows) tiles and streams that many A row
// strips and B row strips through L2 instead of a few A strips and ALL B strips (band_rows = 1, row-major).
// `rot_i` / `rot_j` shift where the walk starts (in tiles, modulo the grid): at cp > 1 every rank starts at the
// tiles whose result it owns itself, so that at any moment the ranks' stores go to different owners instead of
// all to the owner of the first rows.
__host__ __device__ __forceinline__ void tile_of(int r, int tiles_i, int tiles_j, int band_rows, int rot_i, int rot_j,
                                                 int& ti, int& tj) {
  const int band_tiles = band_rows * tiles_j;
  const int band = r / band_tiles;
  const int rem = r - band * band_tiles;
  const int left = tiles_i - band * band_rows;
  const int rows = band_rows < left ? band_rows : left;
  tj = rem / rows;
  ti = band * band_rows + (rem - tj * rows) + rot_i;
  tj += rot_j;
  if (ti >= tiles_i) ti -= tiles_i;
  if (tj >= tiles_j) tj -= tiles_j;
}

// Base pointers of one logical buffer on every rank of the cp group (index = flat cp rank).
// At cp=1 only ptr[0] is used and it is local memory.
struct PeerPtrs {
  void* ptr[kMaxPeers];
};

// Ring-buffer stage/phase bookkeeping for mbarrier pipelines.
struct PipeState {
  uint32_t stage;
  uint32_t phase;
  __device__ __forceinline__ void advance(uint32_t nstages) {
    if (++stage == nstages) {
      stage = 0;
      phase ^= 1;
    }
  }
};

}  // namespace trimul
