// Output LayerNorm fused with the gated output projection:
//     out = gate * ( LayerNorm(tri) Wp^T + bp )
// with tri arriving CHANNEL-major (D planes of `rows` tokens, exactly as the contraction kernel
// stores it on the token-owning rank) and gate = sigmoid(xn Wo^T + bo) already computed by the
// projection kernel.  (Reference: ops 8-12 of trimul_ref,
// fold_cp_ops/workflows/trimul_autotune.py:1519-1525; fused consumer
// fold_cp_ops/kernels/layernorm_dual_gated_gemm.py:5342; recv layout reshard.py:347-363.)
//
// Persistent CTA, 128-token tiles.  Eight LayerNorm warps -- one per group of D/8 channels -- read
// the tile in two 64-token halves with coalesced 128-byte warp loads (two tokens per lane) into
// registers, double-buffered so the loads of the next half are in flight while the current one is
// reduced; per-token statistics of the eight channel groups are combined with Chan's formula
// through shared memory, and the normalised bf16 operand is written in the K-major
// 128-byte-swizzle layout.  W_out stays resident in shared memory for the life of the CTA (one TMA
// load).  One thread issues tcgen05.mma; eight epilogue warps prefetch their slice of the gate
// before the accumulator is ready, then apply bias and gate and store 16-byte vectors token-major.
#include "trimul_common.cuh"
#include "trimul_kernels.h"

namespace trimul {

namespace {

constexpr int BM = 128;
constexpr int HALF = 64;
// Five warpgroups: w0-3 control (w0: TMEM alloc, W load, MMA issue), w4-11 epilogue, w12-19 LayerNorm.
// The kernel launches at 96 registers per thread and rebalances with setmaxnreg: the control
// warpgroup shrinks to 40, the epilogue grows to 104 and the LayerNorm warps to 112
// (per SM sub-partition: (40 + 2*104 + 2*112) * 32 = 15104 <= 16384 registers).
constexpr int kThreads = 640;
constexpr int kEpiWarp0 = 4;
constexpr int kLnWarp0 = 12;
constexpr int kCtlWarp = 0;
constexpr int kGroups = 8;  // channel groups = LayerNorm warps

template <int D>
struct Cfg {
  static constexpr int KB = D / 64;
  static constexpr int CPT = D / kGroups;  // channels per LayerNorm thread
  static constexpr int kABytes = BM * D * 2;
  static constexpr int kKBlockBytes = BM * 128;
  static constexpr int kWBytes = D * D * 2;
  static constexpr int kWBlockBytes = D * 128;
  static constexpr int kABufs = (D == 256) ? 1 : 2;
  static constexpr int kTmemCols = (2 * D <= 256) ? 256 : 512;
  static constexpr int kTileBytes = kWBytes + kABufs * kABytes;
};

template <int D>
struct SmemCtl {
  uint64_t w_full;
  uint64_t a_ready[2];
  uint64_t a_empty[2];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t red_bar[2];  // LayerNorm warps: partial statistics of parity p are all written
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  float2 red[2][kGroups][HALF];  // [parity][channel group][token of the half] = (mean, M2) partials
  float gamma[D];
  float beta[D];
};

template <int D>
constexpr int smem_bytes() {
  return Cfg<D>::kTileBytes + 1024 + static_cast<int>(sizeof(SmemCtl<D>)) + 64;
}

__device__ __forceinline__ uint32_t ldg_nc_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

}  // namespace

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
out_proj_kernel(const __grid_constant__ CUtensorMap tmW, const OutProjArgs p) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* w_tiles = tiles;                 // KB blocks of (D rows x 64 k)
  uint8_t* a_tiles = tiles + C::kWBytes;    // kABufs operand tiles
  SmemCtl<D>* ctl = reinterpret_cast<SmemCtl<D>*>(tiles + C::kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long total_tiles = (p.rows + BM - 1) / BM;
  // tiles this CTA owns: blockIdx.x, blockIdx.x + gridDim.x, ...
  const long my_tiles = (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;

  if (threadIdx.x == 0) {
    sm100::mbar_init(&ctl->w_full, 1);
    for (int a = 0; a < 2; ++a) {
      sm100::mbar_init(&ctl->a_ready[a], kGroups);
      sm100::mbar_init(&ctl->a_empty[a], 1);
      sm100::mbar_init(&ctl->tmem_full[a], 1);
      sm100::mbar_init(&ctl->tmem_empty[a], 8);
      sm100::mbar_init(&ctl->red_bar[a], kGroups);
    }
    ctl->abort_flag = 0;
    sm100::mbar_init_fence();
  }
  for (int i = threadIdx.x; i < D; i += kThreads) {
    ctl->gamma[i] = p.ln_w[i];
    ctl->beta[i] = p.ln_b ? p.ln_b[i] : 0.0f;
  }
  if (warp == kCtlWarp) {
    sm100::tmem_alloc(&ctl->tmem_base, C::kTmemCols);
    sm100::tmem_relinquish();
  }
  sm100::tcgen05_fence_before_sync();
  __syncthreads();
  sm100::tcgen05_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  const uint64_t tmo = p.timeout_ns;
  bool w_armed = false;

  if (warp < kEpiWarp0) {
    sm100::setmaxnreg_dec<40>();
    if (warp == kCtlWarp && lane == 0 && my_tiles > 0) {
      // ---------------------------------------------------------- W_out: one TMA load, resident
      sm100::tma_prefetch_desc(&tmW);
      sm100::mbar_arrive_expect_tx(&ctl->w_full, C::kWBytes);
      for (int kb = 0; kb < C::KB; ++kb) {
        sm100::tma_load_2d(w_tiles + kb * C::kWBlockBytes, &tmW, &ctl->w_full, kb * 64, 0);
      }
      w_armed = true;
      // ---------------------------------------------------------- UMMA issuer
      constexpr uint32_t idesc = sm100::umma_idesc_bf16_f32(BM, D);
      uint32_t acc = 0, acc_phase = 0, buf = 0, buf_phase = 0;
      bool ok = sm100::mbar_wait(&ctl->w_full, 0, abort_flag, tmo);
      if (!ok) report_timeout(p.status, kKernelOutProj, 1, -3);
      const uint32_t w_addr = sm100::smem_u32(w_tiles);
      for (long it = 0; it < my_tiles && ok; ++it) {
        if (!sm100::mbar_wait(&ctl->a_ready[buf], buf_phase, abort_flag, tmo)) {
          report_timeout(p.status, kKernelOutProj, 1, -1);
          break;
        }
        if (!sm100::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1, abort_flag, tmo)) {
          report_timeout(p.status, kKernelOutProj, 1, -2);
          break;
        }
        sm100::tcgen05_fence_after_sync();
        const uint32_t a_addr = sm100::smem_u32(a_tiles + buf * C::kABytes);
        const uint32_t d_tmem = tmem_base + acc * D;
#pragma unroll
        for (int kb = 0; kb < C::KB; ++kb) {
          const uint64_t da = sm100::umma_desc_kmajor_sw128(a_addr + kb * C::kKBlockBytes);
          const uint64_t db = sm100::umma_desc_kmajor_sw128(w_addr + kb * C::kWBlockBytes);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            sm100::umma_bf16_ss(d_tmem, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
          }
        }
        sm100::umma_commit(&ctl->a_empty[buf]);
        sm100::umma_commit(&ctl->tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
        if (++buf == C::kABufs) {
          buf = 0;
          buf_phase ^= 1;
        }
      }
    }
  } else if (warp >= kLnWarp0) {
    // ------------------------------------------------------------ LayerNorm prologue (8 warps)
    sm100::setmaxnreg_inc<112>();
    constexpr int CPT = C::CPT;
    const int cg = warp - kLnWarp0;  // channel group of this warp
    const int r_in_half = 2 * lane;  // tokens 2*lane, 2*lane+1 of the half
    const uint8_t* tb = static_cast<const uint8_t*>(p.tri);
    uint32_t buf = 0, buf_phase = 0, par = 0, red_phase = 0;
    bool ok = true;
    const long total_halves = 2 * my_tiles;

    auto load_half = [&](uint32_t (&v)[CPT], long h) {
      const long t = blockIdx.x + (h >> 1) * gridDim.x;
      const long m0 = t * BM + (h & 1) * HALF + r_in_half;
      if (m0 < p.rows && !(p.debug_skip & 1)) {  // rows is even: the pair is valid or invalid together
        const uint8_t* q = tb + (static_cast<long>(cg * CPT) * p.rows + m0) * 2;
        const long plane_bytes = p.rows * 2;
#pragma unroll
        for (int e = 0; e < CPT; ++e) {
          v[e] = ldg_nc_u32(q);
          q += plane_bytes;
        }
      } else {
#pragma unroll
        for (int e = 0; e < CPT; ++e) v[e] = 0;
      }
    };

    auto process_half = [&](uint32_t (&v)[CPT], long h) {
      const int half = static_cast<int>(h & 1);
      // local statistics over this thread's CPT channels, per token
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int e = 0; e < CPT; ++e) {
        s0 += sm100::bf16_lo(v[e]);
        s1 += sm100::bf16_hi(v[e]);
      }
      const float lm0 = s0 * (1.0f / CPT), lm1 = s1 * (1.0f / CPT);
      float q0 = 0.f, q1 = 0.f;
#pragma unroll
      for (int e = 0; e < CPT; ++e) {
        const float d0 = sm100::bf16_lo(v[e]) - lm0;
        const float d1 = sm100::bf16_hi(v[e]) - lm1;
        q0 = fmaf(d0, d0, q0);
        q1 = fmaf(d1, d1, q1);
      }
      *reinterpret_cast<float4*>(&ctl->red[par][cg][r_in_half]) = make_float4(lm0, q0, lm1, q1);
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&ctl->red_bar[par]);
      ok = sm100::mbar_wait(&ctl->red_bar[par], (red_phase >> par) & 1, abort_flag, tmo);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        report_timeout(p.status, kKernelOutProj, 4, static_cast<int>(h));
        return;
      }
      red_phase ^= (1u << par);
      // combine the eight (mean, M2) partials; the partials are re-read for the second pass
      // instead of being kept live, which saves 32 registers against the two in-flight halves
      const float4* part = reinterpret_cast<const float4*>(&ctl->red[par][0][r_in_half]);
      constexpr int kPartStride = HALF / 2;  // float4 elements between channel groups
      float mean0 = 0.f, mean1 = 0.f;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        const float4 pg = part[g * kPartStride];
        mean0 += pg.x;
        mean1 += pg.z;
      }
      mean0 *= (1.0f / kGroups);
      mean1 *= (1.0f / kGroups);
      float m20 = 0.f, m21 = 0.f;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        const float4 pg = part[g * kPartStride];
        const float e0 = pg.x - mean0, e1 = pg.z - mean1;
        m20 += pg.y + CPT * e0 * e0;
        m21 += pg.w + CPT * e1 * e1;
      }
      const float rstd0 = rsqrtf(m20 * (1.0f / D) + p.eps);
      const float rstd1 = rsqrtf(m21 * (1.0f / D) + p.eps);
      const float nm0 = -mean0 * rstd0, nm1 = -mean1 * rstd1;
      par ^= 1;  // the next half uses the other partial buffer: no second barrier needed

      if (half == 0) {
        ok = sm100::mbar_wait(&ctl->a_empty[buf], buf_phase ^ 1, abort_flag, tmo);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          report_timeout(p.status, kKernelOutProj, 3, static_cast<int>(h));
          return;
        }
      }
      uint8_t* a_tile = a_tiles + buf * C::kABytes;
      const int r0 = half * HALF + r_in_half;
#pragma unroll
      for (int c8 = 0; c8 < CPT / 8; ++c8) {
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) {
          const int e = c8 * 8 + e2 * 2;
          const int d = cg * CPT + e;
          const float2 gm = *reinterpret_cast<const float2*>(&ctl->gamma[d]);
          const float2 bt = *reinterpret_cast<const float2*>(&ctl->beta[d]);
          const float x00 = fmaf(sm100::bf16_lo(v[e]), rstd0, nm0);
          const float x01 = fmaf(sm100::bf16_lo(v[e + 1]), rstd0, nm0);
          const float x10 = fmaf(sm100::bf16_hi(v[e]), rstd1, nm1);
          const float x11 = fmaf(sm100::bf16_hi(v[e + 1]), rstd1, nm1);
          lo[e2] = sm100::pack_bf16x2(fmaf(x00, gm.x, bt.x), fmaf(x01, gm.y, bt.y));
          hi[e2] = sm100::pack_bf16x2(fmaf(x10, gm.x, bt.x), fmaf(x11, gm.y, bt.y));
        }
        const int chunk = (cg * CPT) / 8 + c8;  // 16-byte chunk index along K
        const uint32_t kb_off = (chunk >> 3) * C::kKBlockBytes;
        const uint32_t o0 = kb_off + r0 * 128 + (((chunk & 7) ^ (r0 & 7)) << 4);
        const uint32_t o1 = kb_off + (r0 + 1) * 128 + (((chunk & 7) ^ ((r0 + 1) & 7)) << 4);
        *reinterpret_cast<uint4*>(a_tile + o0) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<uint4*>(a_tile + o1) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      }
      if (half == 1) {
        sm100::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&ctl->a_ready[buf]);
        if (++buf == C::kABufs) {
          buf = 0;
          buf_phase ^= 1;
        }
      }
    };

    uint32_t v0[CPT], v1[CPT];
    if (total_halves > 0) load_half(v0, 0);
    for (long h = 0; h < total_halves && ok; h += 2) {
      load_half(v1, h + 1);  // total_halves is even: h + 1 always exists
      process_half(v0, h);
      if (!ok) break;
      if (h + 2 < total_halves) load_half(v0, h + 2);
      process_half(v1, h + 1);
    }
  } else {
    // ------------------------------------------------------------ epilogue (8 warps)
    sm100::setmaxnreg_inc<104>();
    const int quarter = warp & 3;
    const int hh = (warp - kEpiWarp0) >> 2;  // which half of the output columns
    const int r = quarter * 32 + lane;
    constexpr int COLS = D / 2;          // columns this warp handles
    constexpr int NV = COLS / 8;         // 16-byte vectors of gate / out per thread
    uint32_t acc = 0, acc_phase = 0;
    for (long it = 0; it < my_tiles; ++it) {
      const long t = blockIdx.x + it * gridDim.x;
      const long m = t * BM + r;
      const bool valid = m < p.rows;
      // the gate slice is fetched before the accumulator is ready: its latency hides behind the wait
      uint4 gt[NV];
      if (valid && !(p.debug_skip & 2)) {
        const uint8_t* gp = static_cast<const uint8_t*>(p.gate) + (m * D + hh * COLS) * 2;
#pragma unroll
        for (int q = 0; q < NV; ++q) gt[q] = ldg_nc_v4(gp + q * 16);
      } else {
#pragma unroll
        for (int q = 0; q < NV; ++q) gt[q] = make_uint4(0, 0, 0, 0);
      }
      bool ok = sm100::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort_flag, tmo);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        report_timeout(p.status, kKernelOutProj, 2, static_cast<int>(t));
        break;
      }
      sm100::tcgen05_fence_after_sync();
      const uint32_t trow = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * D + hh * COLS;
      uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + m * D + hh * COLS);
#pragma unroll
      for (int g = 0; g < COLS / 16; ++g) {
        uint32_t pv[16];
        sm100::tmem_ld_32x32b_x16(trow + g * 16, pv);
        sm100::tmem_ld_wait();
        if (valid && !(p.debug_skip & 4)) {
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const uint4 gq = gt[g * 2 + q];
            const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
            uint32_t ow[4];
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              const int e = q * 8 + e2 * 2;
              float y0 = __uint_as_float(pv[e]);
              float y1 = __uint_as_float(pv[e + 1]);
              if (p.bias != nullptr) {
                y0 += __ldg(p.bias + hh * COLS + g * 16 + e);
                y1 += __ldg(p.bias + hh * COLS + g * 16 + e + 1);
              }
              ow[e2] = sm100::pack_bf16x2(y0 * sm100::bf16_lo(gw[e2]), y1 * sm100::bf16_hi(gw[e2]));
            }
            dst[g * 2 + q] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
        }
      }
      sm100::tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&ctl->tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();  // single-lane roles reconverge with their warp
  __syncthreads();
  if (warp == kCtlWarp && lane == 0 && w_armed) {
    // the weight load is the only TMA copy of this kernel; make sure it landed before exit
    const uint64_t t0 = sm100::globaltimer_ns();
    while (!sm100::mbar_test(&ctl->w_full, 0) && sm100::globaltimer_ns() - t0 < 2000000ull) {
    }
  }
  __syncthreads();
  if (warp == kCtlWarp) {
    sm100::tcgen05_fence_after_sync();
    sm100::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
int out_proj_smem_bytes(int D) {
  if (D == 128) return smem_bytes<128>();
  if (D == 256) return smem_bytes<256>();
  return -1;
}

template <int D>
static cudaError_t launch_t(const CUtensorMap& tmW, const OutProjArgs& args, int num_sms, cudaStream_t stream) {
  cudaError_t e =
      cudaFuncSetAttribute(out_proj_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<D>());
  if (e != cudaSuccess) return e;
  const long total = (args.rows + BM - 1) / BM;
  if (total <= 0) return cudaSuccess;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  out_proj_kernel<D><<<grid, kThreads, smem_bytes<D>(), stream>>>(tmW, args);
  return cudaGetLastError();
}

cudaError_t launch_out_proj(const CUtensorMap& tmW, const OutProjArgs& args, int num_sms, cudaStream_t stream) {
  if (args.D == 128) return launch_t<128>(tmW, args, num_sms, stream);
  if (args.D == 256) return launch_t<256>(tmW, args, num_sms, stream);
  return cudaErrorInvalidValue;
}

}  // namespace trimul
