// Output LayerNorm fused with the gated output projection:
//     out = gate * ( LayerNorm(tri) Wp^T + bp )
// with tri arriving CHANNEL-major (D planes of `rows` tokens, exactly as the contraction kernel
// stores it on the token-owning rank) and gate = sigmoid(xn Wo^T + bo) already computed by the
// projection kernel.  (Reference: ops 8-12 of trimul_ref,
// fold_cp_ops/workflows/trimul_autotune.py:1519-1525; fused consumer
// fold_cp_ops/kernels/layernorm_dual_gated_gemm.py:5342 -- its "alg_fold" form :41-43; recv
// layout reshard.py:347-363.)
//
// The LayerNorm is folded algebraically so the channel-major tile never has to be transposed or
// rewritten:   LN(x) W^T + b  =  rstd * ( x (gamma .* W)^T  -  mean * c )  +  d ,
//     c[n] = sum_k bf16(gamma_k W[n,k]),   d[n] = sum_k beta_k W[n,k] + b[n]        (packed once).
// The GEMM is issued transposed -- acc[n][m] = sum_k W'[n][k] tri[k][m] -- so that TMEM lanes are
// output CHANNELS and columns are tokens: an epilogue warp then touches 32 consecutive channels of
// one token per instruction (64 contiguous bytes of the token-major gate / out rows) instead of 32
// different rows.  The raw tile is the B operand exactly as it lies in memory: TMA brings
// (64 channels x 64 tokens) boxes with the 128-byte swizzle along TOKENS, and the tensor core
// reads them through an MN-major (token-major) shared-memory descriptor.  Eight statistics warps read the same staged boxes and
// reduce per-token mean / M2 (two-pass per 16 channels, Chan-merged), so the tile is fetched from
// HBM exactly once, asynchronously, through a 5..8 stage ring.  gamma .* W stays resident in
// shared memory.  Eight epilogue warps (one channel per lane) apply
// rstd[m] * acc + (-mean[m]*rstd[m]) * c[n] + d[n], multiply by the gate and store token-major.
#include "trimul_common.cuh"
#include "trimul_kernels.h"

namespace trimul {

namespace {

constexpr int BM = 128;
// Five warpgroups: w0-3 control (w0 TMA producer, w1 MMA issuer, w2 TMEM alloc), w4-11 epilogue,
// w12-19 statistics.
constexpr int kThreads = 640;
constexpr int kEpiWarp0 = 4;
constexpr int kStatWarp0 = 12;
constexpr int kStageBytes = 2 * 64 * 128;  // two token blocks x 64 channels x 128 B

template <int D>
struct Cfg {
  static constexpr int KB = D / 64;
  static constexpr int kWBytes = D * D * 2;
  static constexpr int kWBlockBytes = D * 128;
  static constexpr int kStages = (D == 256) ? 5 : 8;
  static constexpr int kTmemCols = (2 * D <= 256) ? 256 : 512;
  static constexpr int kTileBytes = kWBytes + kStages * kStageBytes;
};

template <int D>
struct SmemCtl {
  uint64_t w_full;
  uint64_t full[Cfg<D>::kStages];
  uint64_t empty[Cfg<D>::kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t red_bar[2];
  uint64_t stats_ready[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  volatile uint32_t armed[Cfg<D>::kStages];
  alignas(16) float2 red[2][4][BM];   // [tile parity][channel subgroup][token] = (mean, M2) over D/4 channels
  float2 stat[2][BM];     // [accumulator][token] = (rstd, -mean * rstd)
};

template <int D>
constexpr int smem_bytes() {
  return Cfg<D>::kTileBytes + 1024 + static_cast<int>(sizeof(SmemCtl<D>)) + 64;
}

__device__ __forceinline__ uint32_t ldg_nc_u16(const void* p) {
  uint32_t v;
  asm volatile("{\n\t.reg .b16 h;\n\tld.global.nc.u16 h, [%1];\n\tcvt.u32.u16 %0, h;\n\t}" : "=r"(v) : "l"(p));
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
out_proj_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmT,
                const OutProjArgs p) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* w_tiles = tiles;                 // KB blocks of (D rows x 64 k), K-major, resident
  uint8_t* ring = tiles + C::kWBytes;       // kStages x [2 token blocks][64 channels][128 B]
  SmemCtl<D>* ctl = reinterpret_cast<SmemCtl<D>*>(tiles + C::kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long total_tiles = (p.rows + BM - 1) / BM;
  const long my_tiles = (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;

  if (threadIdx.x == 0) {
    sm100::mbar_init(&ctl->w_full, 1);
    for (int s = 0; s < C::kStages; ++s) {
      sm100::mbar_init(&ctl->full[s], 1);
      sm100::mbar_init(&ctl->empty[s], 1 + 8);  // tcgen05.commit + one arrive per statistics warp
      ctl->armed[s] = 2;
    }
    for (int a = 0; a < 2; ++a) {
      sm100::mbar_init(&ctl->tmem_full[a], 1);
      sm100::mbar_init(&ctl->tmem_empty[a], 8);
      sm100::mbar_init(&ctl->red_bar[a], 8);
      sm100::mbar_init(&ctl->stats_ready[a], 2);
    }
    ctl->abort_flag = 0;
    sm100::mbar_init_fence();
  }
  if (warp == 2) {
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && my_tiles > 0) {
      sm100::tma_prefetch_desc(&tmW);
      sm100::tma_prefetch_desc(&tmT);
      sm100::mbar_arrive_expect_tx(&ctl->w_full, C::kWBytes);
      for (int kb = 0; kb < C::KB; ++kb) {
        sm100::tma_load_2d(w_tiles + kb * C::kWBlockBytes, &tmW, &ctl->w_full, kb * 64, 0);
      }
      w_armed = true;
      PipeState ps{0, 0};
      bool ok = true;
      for (long it = 0; it < my_tiles && ok; ++it) {
        const long m0 = (blockIdx.x + it * gridDim.x) * BM;
        for (int kb = 0; kb < C::KB; ++kb) {
          if (!sm100::mbar_wait(&ctl->empty[ps.stage], ps.phase ^ 1, abort_flag, tmo)) {
            report_timeout(p.status, kKernelOutProj, 0, kb);
            ok = false;
            break;
          }
          uint8_t* st = ring + ps.stage * kStageBytes;
          ctl->armed[ps.stage] = ps.phase;
          sm100::mbar_arrive_expect_tx(&ctl->full[ps.stage], kStageBytes);
          // (tokens, channels) boxes of 64 x 64; a block past the last token is zero-filled
          sm100::tma_load_2d(st, &tmT, &ctl->full[ps.stage], static_cast<int>(m0), kb * 64);
          sm100::tma_load_2d(st + kStageBytes / 2, &tmT, &ctl->full[ps.stage], static_cast<int>(m0 + 64), kb * 64);
          ps.advance(C::kStages);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    if (lane == 0 && my_tiles > 0) {
      // A: folded weights, K-major, one 128-channel M tile at a time; B: raw tile, token-major (MN-major)
      constexpr uint32_t idesc = sm100::umma_idesc_bf16_f32(128, BM) | (1u << 16);
      constexpr int MT = D / 128;  // M tiles (output channels / 128)
      PipeState ps{0, 0};
      uint32_t acc = 0, acc_phase = 0;
      bool ok = sm100::mbar_wait(&ctl->w_full, 0, abort_flag, tmo);
      if (!ok) report_timeout(p.status, kKernelOutProj, 1, -3);
      const uint32_t w_addr = sm100::smem_u32(w_tiles);
      // token blocks of 64 are kStageBytes/2 apart (leading offset); 8-channel groups 1024 B apart
      const uint32_t lbo = p.mn_swap ? 1024u : static_cast<uint32_t>(kStageBytes / 2);
      const uint32_t sbo = p.mn_swap ? static_cast<uint32_t>(kStageBytes / 2) : 1024u;
      for (long it = 0; it < my_tiles && ok; ++it) {
        if (!sm100::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1, abort_flag, tmo)) {
          report_timeout(p.status, kKernelOutProj, 1, -2);
          break;
        }
        sm100::tcgen05_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * D;
        for (int kb = 0; kb < C::KB; ++kb) {
          if (!sm100::mbar_wait(&ctl->full[ps.stage], ps.phase, abort_flag, tmo)) {
            report_timeout(p.status, kKernelOutProj, 1, kb);
            ok = false;
            break;
          }
          sm100::tcgen05_fence_after_sync();
          const uint32_t b_addr = sm100::smem_u32(ring + ps.stage * kStageBytes);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              // weights: 128 rows x 128 B per M tile inside the K block; tile: 16 channels per MMA = 2 KB
              const uint64_t da = sm100::umma_desc_kmajor_sw128(w_addr + kb * C::kWBlockBytes + mt * 128 * 128) + 2 * k4;
              const uint64_t db = sm100::umma_desc_mnmajor_sw128(b_addr + k4 * 2048, lbo, sbo);
              sm100::umma_bf16_ss(d_tmem + mt * BM, da, db, idesc, (kb | k4) != 0);
            }
          }
          sm100::umma_commit(&ctl->empty[ps.stage]);
          ps.advance(C::kStages);
        }
        if (!ok) break;
        sm100::umma_commit(&ctl->tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp >= kStatWarp0) {
    // ------------------------------------------------------------ statistics (8 warps)
    const int st_tid = threadIdx.x - kStatWarp0 * 32;  // 0..255
    const int pr = st_tid & 63;                        // token pair: tokens 2*pr, 2*pr+1
    const int cs = st_tid >> 6;                        // channel subgroup: 16 of every 64 channels
    const int t0 = 2 * pr;
    // byte offset of the pair inside a (64 channels x 64 tokens) box row, before the swizzle
    const uint32_t blk_off = (t0 >> 6) * (kStageBytes / 2);
    const uint32_t chunk16 = (t0 & 63) >> 3;
    const uint32_t in_chunk = (t0 & 7) * 2;
    PipeState ps{0, 0};
    uint32_t acc = 0, acc_phase = 0, par = 0, red_phase = 0;
    bool ok = true;
    for (long it = 0; it < my_tiles && ok; ++it) {
      float mean0 = 0.f, m20 = 0.f, mean1 = 0.f, m21 = 0.f;  // running (mean, M2) of the two tokens
      for (int kb = 0; kb < C::KB; ++kb) {
        ok = sm100::mbar_wait(&ctl->full[ps.stage], ps.phase, abort_flag, tmo);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          report_timeout(p.status, kKernelOutProj, 3, kb);
          break;
        }
        const uint8_t* st = ring + ps.stage * kStageBytes + blk_off;
        uint32_t v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const uint32_t d = cs * 16 + e;  // channel row inside the stage
          v[e] = *reinterpret_cast<const uint32_t*>(st + d * 128 + ((chunk16 ^ (d & 7)) << 4) + in_chunk);
        }
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&ctl->empty[ps.stage]);  // values are in registers
        ps.advance(C::kStages);
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          s0 += sm100::bf16_lo(v[e]);
          s1 += sm100::bf16_hi(v[e]);
        }
        const float lm0 = s0 * (1.0f / 16), lm1 = s1 * (1.0f / 16);
        float q0 = 0.f, q1 = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float d0 = sm100::bf16_lo(v[e]) - lm0;
          const float d1 = sm100::bf16_hi(v[e]) - lm1;
          q0 = fmaf(d0, d0, q0);
          q1 = fmaf(d1, d1, q1);
        }
        // Chan merge of (16 kb samples so far) with (16 new samples)
        const float na = 16.0f * kb, nb = 16.0f, nn = na + nb;
        const float dl0 = lm0 - mean0, dl1 = lm1 - mean1;
        mean0 += dl0 * (nb / nn);
        mean1 += dl1 * (nb / nn);
        m20 += q0 + dl0 * dl0 * (na * nb / nn);
        m21 += q1 + dl1 * dl1 * (na * nb / nn);
      }
      if (!ok) break;
      // combine the four channel subgroups (each D/4 channels)
      *reinterpret_cast<float4*>(&ctl->red[par][cs][t0]) = make_float4(mean0, m20, mean1, m21);
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&ctl->red_bar[par]);
      ok = sm100::mbar_wait(&ctl->red_bar[par], (red_phase >> par) & 1, abort_flag, tmo);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        report_timeout(p.status, kKernelOutProj, 4, static_cast<int>(it));
        break;
      }
      red_phase ^= (1u << par);
      if (cs == 0) {
        // the epilogue of the tile that last used stat[acc] must have finished reading it
        ok = sm100::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1, abort_flag, tmo);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          report_timeout(p.status, kKernelOutProj, 5, static_cast<int>(it));
          break;
        }
        constexpr float nq = D / 4;
        float mu0 = 0.f, mu1 = 0.f;
        float4 pp[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          pp[g] = *reinterpret_cast<const float4*>(&ctl->red[par][g][t0]);
          mu0 += pp[g].x;
          mu1 += pp[g].z;
        }
        mu0 *= 0.25f;
        mu1 *= 0.25f;
        float M0 = 0.f, M1 = 0.f;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const float e0 = pp[g].x - mu0, e1 = pp[g].z - mu1;
          M0 += pp[g].y + nq * e0 * e0;
          M1 += pp[g].w + nq * e1 * e1;
        }
        const float r0 = rsqrtf(M0 * (1.0f / D) + p.eps);
        const float r1 = rsqrtf(M1 * (1.0f / D) + p.eps);
        *reinterpret_cast<float4*>(&ctl->stat[acc][t0]) = make_float4(r0, -mu0 * r0, r1, -mu1 * r1);
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&ctl->stats_ready[acc]);
      }
      par ^= 1;
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------ epilogue (8 warps)
    // TMEM lane = output channel, column = token.  D = 256: warps 4-7 take channels 0-127, warps
    // 8-11 channels 128-255, all 128 tokens each.  D = 128: both sets take all channels and split
    // the tokens 64 / 64.
    const int quarter = warp & 3;
    const int set = (warp - kEpiWarp0) >> 2;
    constexpr int MT = D / 128;
    const int mt = (MT == 2) ? set : 0;
    constexpr int NTOK = (MT == 2) ? BM : BM / 2;     // tokens this warp handles
    const int tok0 = (MT == 2) ? 0 : set * NTOK;
    const int n = mt * 128 + quarter * 32 + lane;      // this lane's output channel
    const float2 cdn = reinterpret_cast<const float2*>(p.cd)[n];
    const __nv_bfloat16* gate = static_cast<const __nv_bfloat16*>(p.gate) + n;
    __nv_bfloat16* outp = static_cast<__nv_bfloat16*>(p.out) + n;
    const bool skip_ld = (p.debug_skip & 2) != 0, skip_st = (p.debug_skip & 4) != 0;
    uint32_t acc = 0, acc_phase = 0;
    for (long it = 0; it < my_tiles; ++it) {
      const long m0 = (blockIdx.x + it * gridDim.x) * BM + tok0;
      const int nvalid = static_cast<int>(p.rows - m0 < NTOK ? (p.rows - m0 > 0 ? p.rows - m0 : 0) : NTOK);
      // gate values of the first 16 tokens are requested before the accumulator is ready.  Loads are
      // unconditional (a token index past the end is clamped to the last valid one) so that all 16
      // are in flight together; only the stores are predicated.
      const int last = nvalid - 1;
      const bool do_ld = nvalid > 0 && !skip_ld;
      uint32_t gcur[16], gnext[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) gcur[e] = gnext[e] = 0;
      if (do_ld) {
#pragma unroll
        for (int e = 0; e < 16; ++e) gcur[e] = ldg_nc_u16(gate + (m0 + (e < last ? e : last)) * D);
      }
      bool ok = sm100::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort_flag, tmo);
      ok = ok && sm100::mbar_wait(&ctl->stats_ready[acc], acc_phase, abort_flag, tmo);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        report_timeout(p.status, kKernelOutProj, 2, static_cast<int>(it));
        break;
      }
      sm100::tcgen05_fence_after_sync();
      const uint32_t trow = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * D + mt * BM + tok0;
      const float2* stat = &ctl->stat[acc][tok0];
      // TMEM reads and gate loads are software-pipelined one 16-token group ahead
      if (!(p.debug_skip & 8)) {
        uint32_t pa[16], pb[16];
        sm100::tmem_ld_32x32b_x16(trow, pa);
#pragma unroll
        for (int g = 0; g < NTOK / 16; ++g) {
          sm100::tmem_ld_wait();
          if (g + 1 < NTOK / 16) {
            if ((g & 1) == 0) sm100::tmem_ld_32x32b_x16(trow + (g + 1) * 16, pb);
            else sm100::tmem_ld_32x32b_x16(trow + (g + 1) * 16, pa);
            if (do_ld) {
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const int m = (g + 1) * 16 + e;
                gnext[e] = ldg_nc_u16(gate + (m0 + (m < last ? m : last)) * D);
              }
            }
          }
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int m = g * 16 + e;
            const float2 rs = stat[m];  // (rstd, -mean * rstd), same address for every lane
            const float accv = __uint_as_float((g & 1) == 0 ? pa[e] : pb[e]);
            const float y = fmaf(accv, rs.x, fmaf(rs.y, cdn.x, cdn.y));
            const float gv = __uint_as_float(gcur[e] << 16);
            if (m < nvalid && !skip_st) outp[(m0 + m) * D] = __float2bfloat16_rn(y * gv);
          }
#pragma unroll
          for (int e = 0; e < 16; ++e) gcur[e] = gnext[e];
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
  if (warp == 0 && lane == 0 && w_armed) {
    // let TMA copies still in flight land before the CTA exits (only matters after an expired wait)
    const uint64_t t0 = sm100::globaltimer_ns();
    while (!sm100::mbar_test(&ctl->w_full, 0) && sm100::globaltimer_ns() - t0 < 2000000ull) {
    }
    if (*abort_flag != 0) {
      for (int s = 0; s < C::kStages; ++s) {
        const uint32_t ph = ctl->armed[s];
        if (ph != 2) {
          const uint64_t t1 = sm100::globaltimer_ns();
          while (!sm100::mbar_test(&ctl->full[s], ph) && sm100::globaltimer_ns() - t1 < 2000000ull) {
          }
        }
      }
    }
  }
  __syncthreads();
  if (warp == 2) {
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
static cudaError_t launch_t(const CUtensorMap& tmW, const CUtensorMap& tmT, const OutProjArgs& args, int num_sms,
                            cudaStream_t stream) {
  cudaError_t e =
      cudaFuncSetAttribute(out_proj_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<D>());
  if (e != cudaSuccess) return e;
  const long total = (args.rows + BM - 1) / BM;
  if (total <= 0) return cudaSuccess;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  out_proj_kernel<D><<<grid, kThreads, smem_bytes<D>(), stream>>>(tmW, tmT, args);
  return cudaGetLastError();
}

cudaError_t launch_out_proj(const CUtensorMap& tmW, const CUtensorMap& tmT, const OutProjArgs& args, int num_sms,
                            cudaStream_t stream) {
  if (args.D == 128) return launch_t<128>(tmW, tmT, args, num_sms, stream);
  if (args.D == 256) return launch_t<256>(tmW, tmT, args, num_sms, stream);
  return cudaErrorInvalidValue;
}

}  // namespace trimul
