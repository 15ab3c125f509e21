// Triangle contraction on CTA PAIRS (tcgen05 cta_group::2): the same computation as
// tri_contract.cu,
//     T_l[i, j] = sum_k  A_l[i, k] * B_l[j, k]          (bf16 in, fp32 accumulate, bf16 out)
// with a 256 x 256 output tile per pair of CTAs on neighbouring SMs.  Each CTA loads its own 128
// rows of A and HALF of the 256 B rows; one thread of the pair's first CTA issues
// tcgen05.mma.cta_group::2 (M = 256), which reads A from each CTA's own shared memory and the two
// B halves from both, and leaves rows [128 r, 128 r + 128) of the tile in CTA r's TMEM.  Per FLOP
// that is two thirds of the L2 -> SM traffic and half of the B-operand shared-memory reads of the
// single-CTA 128 x 256 tile, and the smaller stages make the ring six deep.
//
// Barriers: every CTA waits only on barriers in its own shared memory.  The operand loads of
// both CTAs complete on the FIRST CTA's `full` barrier (cp.async.bulk.tensor .cta_group::2 lets a
// load signal the peer's barrier; no multicast load anywhere); tcgen05.commit releases a stage /
// publishes an accumulator in BOTH CTAs at once; the second CTA's epilogue warps hand the
// accumulator back with a remote arrive on the first CTA's `tmem_empty`.  All waits are bounded as
// in the single-CTA kernel.
#include "tri_contract_epilogue.cuh"

namespace trimul {

namespace {

constexpr int BM = 128;          // rows per CTA
constexpr int BN = 256;          // columns per pair
constexpr int BNH = BN / 2;      // B rows each CTA loads
constexpr int BK = 64;
constexpr int kStages = 6;
constexpr int kABytes = BM * BK * 2;    // 16 KB
constexpr int kBBytes = BNH * BK * 2;   // 16 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;
constexpr int kThreads = 192;  // warp 0 TMA, warp 1 MMA (first CTA) + TMEM alloc, warps 2..5 epilogue

struct SmemCtl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

constexpr int kSmemBytes = kStages * kStageBytes + tri::kOutStageBytes + 1024 /*align slack*/ + 256 /*ctl*/;

// Wave pacing (a performance hint, never a dependency).  Tiles that run at the same time share operand
// strips through L2 only while they move through K together; left alone, the pairs drift apart by a good
// part of a tile and most of that sharing is lost.  Before loading its n-th tile a pair's first producer
// counts itself in and waits -- for at most `pace_ns` -- until the other pairs have started their n-th tile
// too (while the pairs are in step that wait is far shorter than the six loaded stages cover).  A pair that is late never waits, an early pair gives up after
// pace_ns and loads anyway, so no result and no termination depends on the counter; the last pair out resets
// it.  [0]: tiles started, [1]: pairs finished.
__device__ unsigned int g_wave_pace[2];

}  // namespace

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
tri_contract_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ TriOutMaps out_maps, const TriContractArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = tiles + kStages * kStageBytes;
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(out_stage + tri::kOutStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = sm100::cluster_ctarank();          // 0: first CTA of the pair (issues the MMAs), 1: second
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int tiles_i = (p.n_i + 2 * BM - 1) / (2 * BM);
  const int tiles_j = (p.n_j + BN - 1) / BN;
  const int tiles_per_plane = tiles_i * tiles_j;
  const long total_tiles = static_cast<long>(tiles_per_plane) * p.planes;
  const int num_k = (p.n_k + BK - 1) / BK;
  const int rot_i = (p.rot_rows / (2 * BM)) % tiles_i;   // first tile row / column of this rank's own block
  const int rot_j = (p.rot_cols / BN) % tiles_j;

  if (threadIdx.x == 0) {
    timeline_min(p.timeline, kTlContractStart);
    for (int s = 0; s < kStages; ++s) {
      sm100::mbar_init(&ctl->full[s], 1);    // first CTA: its producer's arrive + the bytes of both CTAs' loads
      sm100::mbar_init(&ctl->empty[s], 1);   // tcgen05.commit, delivered to both CTAs
    }
    for (int a = 0; a < 2; ++a) {
      sm100::mbar_init(&ctl->tmem_full[a], 1);
      sm100::mbar_init(&ctl->tmem_empty[a], 8);  // four epilogue warps of each CTA (counted in the first CTA)
    }
    ctl->abort_flag = 0;
    sm100::fence_mbar_init_cluster();
  }
  if (warp == 1) {
    sm100::tmem_alloc_pair(&ctl->tmem_base, kTmemCols);
    sm100::tmem_relinquish_pair();
  }
  sm100::tcgen05_fence_before_sync();
  __syncthreads();
  sm100::cluster_sync_all();   // barriers of both CTAs are initialised before anyone signals the peer
  sm100::tcgen05_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  const uint64_t tmo = p.timeout_ns;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      sm100::tma_prefetch_desc(&tmA);
      sm100::tma_prefetch_desc(&tmB);
      PipeState ps{0, 0};
      long wave_end = num_pairs;   // tiles that have started once every pair has started its current one
      for (long t = pair; t < total_tiles; t += num_pairs, wave_end += num_pairs) {
        const int plane = static_cast<int>(t / tiles_per_plane);
        const int r = static_cast<int>(t - static_cast<long>(plane) * tiles_per_plane);
        int ti, tj;
        tile_of(r, tiles_i, tiles_j, p.band_rows, rot_i, rot_j, ti, tj);
        if (p.pace_ns != 0 && cta == 0) {
          const unsigned int target = static_cast<unsigned int>(wave_end < total_tiles ? wave_end : total_tiles);
          atomicAdd(&g_wave_pace[0], 1u);
          const uint64_t t0 = sm100::globaltimer_ns();
          while (*reinterpret_cast<volatile unsigned int*>(&g_wave_pace[0]) < target &&
                 sm100::globaltimer_ns() - t0 < p.pace_ns) {
          }
        }
        bool ok = true;
        for (int kc = 0; kc < num_k; ++kc) {
          if (!sm100::mbar_wait(&ctl->empty[ps.stage], ps.phase ^ 1, abort_flag, tmo)) {
            report_timeout(p.status, kKernelTriContract, 0, kc);
            ok = false;
            break;
          }
          uint8_t* sa = tiles + ps.stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          // both CTAs' bytes are counted on the first CTA's barrier
          const uint32_t bar = sm100::map_to_cta(sm100::smem_u32(&ctl->full[ps.stage]), 0);
          if (cta == 0) sm100::mbar_arrive_expect_tx(&ctl->full[ps.stage], 2 * kStageBytes);
          sm100::tma_load_3d_pair(sa, &tmA, bar, kc * BK, ti * 2 * BM + static_cast<int>(cta) * BM, plane);
          sm100::tma_load_3d_pair(sb, &tmB, bar, kc * BK, tj * BN + static_cast<int>(cta) * BNH, plane);
          ps.advance(kStages);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- UMMA issuer (first CTA only)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = sm100::umma_idesc_bf16_f32(2 * BM, BN);
      PipeState ps{0, 0};
      uint32_t acc = 0, acc_phase = 0;
      for (long t = pair; t < total_tiles; t += num_pairs) {
        bool ok = sm100::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1, abort_flag, tmo);
        if (!ok) {
          report_timeout(p.status, kKernelTriContract, 1, -1);
          break;
        }
        sm100::tcgen05_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kc = 0; kc < num_k; ++kc) {
          if (!sm100::mbar_wait(&ctl->full[ps.stage], ps.phase, abort_flag, tmo)) {
            report_timeout(p.status, kKernelTriContract, 1, kc);
            ok = false;
            break;
          }
          sm100::tcgen05_fence_after_sync();
          const uint32_t sa = sm100::smem_u32(tiles + ps.stage * kStageBytes);
          const uint64_t da = sm100::umma_desc_kmajor_sw128(sa);
          const uint64_t db = sm100::umma_desc_kmajor_sw128(sa + kABytes);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            sm100::umma_bf16_ss_pair(d_tmem, da + 2 * k4, db + 2 * k4, idesc, (kc | k4) != 0);
          }
          sm100::umma_commit_pair(&ctl->empty[ps.stage]);  // frees the stage in both CTAs when the MMAs retire
          ps.advance(kStages);
        }
        if (!ok) break;
        sm100::umma_commit_pair(&ctl->tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;
    uint32_t acc = 0, acc_phase = 0, out_par = 0;
    for (long t = pair; t < total_tiles; t += num_pairs) {
      const int plane = static_cast<int>(t / tiles_per_plane);
      const int r = static_cast<int>(t - static_cast<long>(plane) * tiles_per_plane);
      int ti, tj;
      tile_of(r, tiles_i, tiles_j, p.band_rows, rot_i, rot_j, ti, tj);
      bool ok = sm100::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort_flag, tmo);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        report_timeout(p.status, kKernelTriContract, 2, static_cast<int>(t));
        break;
      }
      sm100::tcgen05_fence_after_sync();
      const int i0w = ti * 2 * BM + static_cast<int>(cta) * BM + quarter * 32;  // first row of this warp's 32-row band
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      tri::store_band(p, out_maps, taddr_row, i0w, tj * BN, plane, out_stage + (warp - 2) * 2 * tri::kOutBufBytes,
                      out_par, lane);
      sm100::tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive_remote(sm100::map_to_cta(sm100::smem_u32(&ctl->tmem_empty[acc]), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) {
      sm100::tma_store_wait_all<0>();
      timeline_max(p.timeline, kTlContractLastStore);
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0) {
    // a wait expired: give loads still in flight (this CTA's and the peer's) time to land
    const uint64_t t0 = sm100::globaltimer_ns();
    while (sm100::globaltimer_ns() - t0 < 200000ull) {
    }
  }
  sm100::tcgen05_fence_before_sync();
  sm100::cluster_sync_all();   // neither CTA retires while the other may still signal it or read its operand half
  if (warp == 1) {
    sm100::tcgen05_fence_after_sync();
    sm100::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (p.pace_ns != 0 && cta == 0 && threadIdx.x == 0) {
    // the last pair to finish leaves the pacing counter at zero for the next launch
    if (atomicAdd(&g_wave_pace[1], 1u) == static_cast<unsigned int>(num_pairs) - 1u) {
      g_wave_pace[0] = 0u;
      g_wave_pace[1] = 0u;
      __threadfence();
    }
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
// The walk the kernel above makes over one plane's tile grid, evaluated on the host (same tile sizes, same
// arithmetic): position r of the walk is tile (ti[r], tj[r]).
void tri_contract_pair_walk(const TriContractArgs& args, int capacity, int* ti, int* tj, int* tiles_i_out,
                            int* tiles_j_out) {
  const int tiles_i = (args.n_i + 2 * BM - 1) / (2 * BM);
  const int tiles_j = (args.n_j + BN - 1) / BN;
  const int rot_i = (args.rot_rows / (2 * BM)) % tiles_i;
  const int rot_j = (args.rot_cols / BN) % tiles_j;
  *tiles_i_out = tiles_i;
  *tiles_j_out = tiles_j;
  for (int r = 0; r < tiles_i * tiles_j && r < capacity; ++r)
    tile_of(r, tiles_i, tiles_j, args.band_rows, rot_i, rot_j, ti[r], tj[r]);
}

cudaError_t launch_tri_contract_pair(const CUtensorMap& tmA, const CUtensorMap& tmBhalf, const TriOutMaps& out_maps,
                                     const TriContractArgs& args, int num_sms, cudaStream_t stream) {
  cudaError_t e =
      cudaFuncSetAttribute(tri_contract_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  const int tiles_i = (args.n_i + 2 * BM - 1) / (2 * BM);
  const int tiles_j = (args.n_j + BN - 1) / BN;
  const long total = static_cast<long>(tiles_i) * tiles_j * args.planes;
  if (total <= 0) return cudaSuccess;
  const long pairs = num_sms / 2;
  const int grid = 2 * static_cast<int>(total < pairs ? total : pairs);
  tri_contract_pair_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tmA, tmBhalf, out_maps, args);
  return cudaGetLastError();
}

}  // namespace trimul
