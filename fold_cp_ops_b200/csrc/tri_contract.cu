// Triangle contraction: for every channel plane l (l = d_loc * B + b)
//     T_l[i, j] = sum_k  A_l[i, k] * B_l[j, k]          (bf16 in, fp32 accumulate, bf16 out)
// A_l and B_l are row-major (rows x n_k) planes of the gated projections "a" and "b".  The
// outgoing update feeds a[i,k], b[j,k]; the incoming update feeds the transposed planes
// a^T[i,k] = a[k,i], b^T[j,k] = b[k,j], which the projection kernel writes directly, so this
// kernel only ever sees K-major operands.
// (Reference: the token-pair GEMM of fold_cp_ops/workflows/trimul_autotune.py:805-853 and the
//  back store of fold_cp_ops/distributed/gemm_sm90_a2a.py; reshard layout reshard.py:277-289.)
//
// One persistent CTA per SM, 128 x 256 output tile, 64-wide K chunks through a TMA->smem ring,
// tcgen05.mma (cta_group::1) into two 256-column TMEM accumulators so the epilogue of tile t
// overlaps the main loop of tile t+1.  The epilogue converts to bf16, stages 32-row x 64-column
// blocks (128-byte rows) in shared memory and sends them with TMA stores straight into the buffer
// of the rank that owns the (i, j) token block: the back all-to-all rides the store, in 128-byte
// row segments.  Ragged edges and blocks that straddle two owners fall back to 16-byte vector
// stores from registers.  At cp=1 the only owner is this GPU.
#include "tri_contract_epilogue.cuh"

namespace trimul {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;  // 16 KB
constexpr int kBBytes = BN * BK * 2;  // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;
constexpr int kThreads = 192;  // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue

struct SmemCtl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  volatile uint32_t armed[kStages];  // parity of the phase the producer last armed, 2 = none
};

constexpr int kSmemBytes = kStages * kStageBytes + tri::kOutStageBytes + 1024 /*align slack*/ + 256 /*ctl*/;

}  // namespace

__global__ void __launch_bounds__(kThreads, 1)
tri_contract_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ TriOutMaps out_maps, const TriContractArgs p) {
  extern __shared__ uint8_t smem_raw[];
  // SW128 tiles need 1024-byte alignment
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = tiles + kStages * kStageBytes;  // [4 warps][2][32 rows x 128 B], 128-byte swizzle
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(out_stage + tri::kOutStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_i = (p.n_i + BM - 1) / BM;
  const int tiles_j = (p.n_j + BN - 1) / BN;
  const int tiles_per_plane = tiles_i * tiles_j;
  const long total_tiles = static_cast<long>(tiles_per_plane) * p.planes;
  const int num_k = (p.n_k + BK - 1) / BK;
  const int rot_i = (p.rot_rows / BM) % tiles_i;   // first tile row / column of this rank's own block
  const int rot_j = (p.rot_cols / BN) % tiles_j;

  if (threadIdx.x == 0) {
    timeline_min(p.timeline, kTlContractStart);
    for (int s = 0; s < kStages; ++s) {
      sm100::mbar_init(&ctl->full[s], 1);
      sm100::mbar_init(&ctl->empty[s], 1);
      ctl->armed[s] = 2;
    }
    for (int a = 0; a < 2; ++a) {
      sm100::mbar_init(&ctl->tmem_full[a], 1);
      sm100::mbar_init(&ctl->tmem_empty[a], 4);  // one arrive per epilogue warp
    }
    ctl->abort_flag = 0;
    sm100::mbar_init_fence();
  }
  if (warp == 1) {
    sm100::tmem_alloc(&ctl->tmem_base, kTmemCols);
    sm100::tmem_relinquish();
  }
  sm100::tcgen05_fence_before_sync();
  __syncthreads();
  sm100::tcgen05_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  const uint64_t tmo = p.timeout_ns;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      sm100::tma_prefetch_desc(&tmA);
      sm100::tma_prefetch_desc(&tmB);
      PipeState ps{0, 0};
      for (long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        const int plane = static_cast<int>(t / tiles_per_plane);
        const int r = static_cast<int>(t - static_cast<long>(plane) * tiles_per_plane);
        int ti, tj;
        tile_of(r, tiles_i, tiles_j, p.band_rows, rot_i, rot_j, ti, tj);
        bool ok = true;
        for (int kc = 0; kc < num_k; ++kc) {
          if (!sm100::mbar_wait(&ctl->empty[ps.stage], ps.phase ^ 1, abort_flag, tmo)) {
            report_timeout(p.status, kKernelTriContract, 0, kc);
            ok = false;
            break;
          }
          uint8_t* sa = tiles + ps.stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          ctl->armed[ps.stage] = ps.phase;
          sm100::mbar_arrive_expect_tx(&ctl->full[ps.stage], kStageBytes);
          sm100::tma_load_3d(sa, &tmA, &ctl->full[ps.stage], kc * BK, ti * BM, plane);
          sm100::tma_load_3d(sb, &tmB, &ctl->full[ps.stage], kc * BK, tj * BN, plane);
          ps.advance(kStages);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- UMMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = sm100::umma_idesc_bf16_f32(BM, BN);
      PipeState ps{0, 0};
      uint32_t acc = 0, acc_phase = 0;
      for (long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
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
            // +32 bytes per 16-element K step inside the 128-byte swizzle row (>>4 => +2)
            sm100::umma_bf16_ss(d_tmem, da + 2 * k4, db + 2 * k4, idesc, (kc | k4) != 0);
          }
          sm100::umma_commit(&ctl->empty[ps.stage]);  // frees the smem stage when the MMAs retire
          ps.advance(kStages);
        }
        if (!ok) break;
        sm100::umma_commit(&ctl->tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t acc = 0, acc_phase = 0, out_par = 0;
    for (long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const int plane = static_cast<int>(t / tiles_per_plane);
      const int r = static_cast<int>(t - static_cast<long>(plane) * tiles_per_plane);
      int ti, tj;
      tile_of(r, tiles_i, tiles_j, p.band_rows, rot_i, rot_j, ti, tj);
      bool ok = sm100::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort_flag, tmo);
      ok = __all_sync(0xffffffffu, ok);  // the warp leaves together: tcgen05.ld is warp-collective
      if (!ok) {
        report_timeout(p.status, kKernelTriContract, 2, static_cast<int>(t));
        break;
      }
      sm100::tcgen05_fence_after_sync();
      const int i0w = ti * BM + quarter * 32;  // first row of this warp's 32-row band
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      tri::store_band(p, out_maps, taddr_row, i0w, tj * BN, plane, out_stage + (warp - 2) * 2 * tri::kOutBufBytes,
                      out_par, lane);
      sm100::tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&ctl->tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    // every store this thread issued must have been performed before the CTA exits
    if (lane == 0) {
      sm100::tma_store_wait_all<0>();
      timeline_max(p.timeline, kTlContractLastStore);
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();  // single-lane roles reconverge with their warp
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0) {
    // a wait expired somewhere: let TMA copies still in flight land before the CTA exits
    for (int s = 0; s < kStages; ++s) {
      const uint32_t ph = ctl->armed[s];
      if (ph != 2) {
        const uint64_t t0 = sm100::globaltimer_ns();
        while (!sm100::mbar_test(&ctl->full[s], ph) && sm100::globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  }
  __syncthreads();
  if (warp == 1) {
    sm100::tcgen05_fence_after_sync();
    sm100::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
int tri_contract_smem_bytes() { return kSmemBytes; }

// The walk the kernel above makes over one plane's tile grid, evaluated on the host (same tile sizes, same
// arithmetic): position r of the walk is tile (ti[r], tj[r]).
void tri_contract_walk(const TriContractArgs& args, int capacity, int* ti, int* tj, int* tiles_i_out, int* tiles_j_out) {
  const int tiles_i = (args.n_i + BM - 1) / BM;
  const int tiles_j = (args.n_j + BN - 1) / BN;
  const int rot_i = (args.rot_rows / BM) % tiles_i;
  const int rot_j = (args.rot_cols / BN) % tiles_j;
  *tiles_i_out = tiles_i;
  *tiles_j_out = tiles_j;
  for (int r = 0; r < tiles_i * tiles_j && r < capacity; ++r)
    tile_of(r, tiles_i, tiles_j, args.band_rows, rot_i, rot_j, ti[r], tj[r]);
}

cudaError_t launch_tri_contract(const CUtensorMap& tmA, const CUtensorMap& tmB, const TriOutMaps& out_maps,
                                const TriContractArgs& args, int num_sms, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(tri_contract_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  const int tiles_i = (args.n_i + BM - 1) / BM;
  const int tiles_j = (args.n_j + BN - 1) / BN;
  const long total = static_cast<long>(tiles_i) * tiles_j * args.planes;
  if (total <= 0) return cudaSuccess;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  tri_contract_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tmA, tmB, out_maps, args);
  return cudaGetLastError();
}

}  // namespace trimul
