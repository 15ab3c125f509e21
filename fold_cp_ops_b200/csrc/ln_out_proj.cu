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
// The raw tile is the A operand exactly as it lies in memory: TMA brings (64 channels x 64
// tokens) boxes with the 128-byte swizzle along TOKENS and the tensor core reads them through an
// MN-major shared-memory descriptor; the folded weights stream from L2 beside it (one ring stage
// = one 64-channel K block of both operands).  Eight statistics warps read the same staged boxes
// and reduce per-token mean / M2 (two-pass per 16 channels, Chan-merged), so the tile is fetched
// from HBM exactly once.
//
// Every byte of global traffic moves as a TMA box with 128-byte rows: the gate arrives as
// (128 token x 64 channel) boxes in a four-slot ring, eight epilogue warps (one token per thread)
// combine it IN PLACE with  rstd[m] * acc + (-mean[m]*rstd[m]) * c[n] + d[n]  from TMEM, and a
// forwarding thread sends each finished box to `out` and hands the slot back to the gate loader.
// No thread issues a global load or store.
#include "trimul_common.cuh"
#include "trimul_kernels.h"

namespace trimul {

namespace {

constexpr int BM = 128;
// Five warpgroups: w0-3 control (w0 operand TMA, w1 MMA issue, w2 TMEM alloc + forwarder,
// w3 gate TMA), w4-11 epilogue, w12-19 statistics.
constexpr int kThreads = 640;
constexpr int kEpiWarp0 = 4;
constexpr int kStatWarp0 = 12;
constexpr int kTriBytes = 2 * 64 * 128;   // one K block of the tile: two token blocks x 64 channels x 128 B
constexpr int kBoxBytes = BM * 128;       // gate / out box: 128 tokens x 64 channels
constexpr int kMaxBoxSlots = 4;

// D = 128 / 256: two accumulators (the epilogue of tile t overlaps the MMAs of tile t + 1), 3-4 ring stages.
// D = 384 / 512: one accumulator fills most of TMEM (D columns) and a K block of the folded weights is
// 48-64 KB, so the ring has two stages, the tiles are serialised on the single accumulator and every MMA
// step is issued in column chunks of at most 256.
template <int D>
struct Cfg {
  static constexpr int KB = D / 64;                // K blocks per tile
  static constexpr int NBT = D / 64;               // gate / out boxes per tile
  static constexpr int NBS = NBT / 2;              // boxes per channel half (one half per epilogue warp set)
  static constexpr int kWBytes = D * 128;          // one K block of the folded weights: D rows x 64 k
  static constexpr int kWBoxRows = (D <= 256) ? D : 128;  // rows one weight TMA box brings
  static constexpr int kStageBytes = kTriBytes + kWBytes;
  static constexpr int kStages = (D > 256) ? 2 : ((D == 256) ? 3 : 4);
  static constexpr int kAccs = (2 * D <= 512) ? 2 : 1;
  static constexpr int kTmemCols = (2 * D <= 256) ? 256 : 512;
  static constexpr int kBoxSlots = (D == 512) ? 3 : 4;
  static constexpr int kTileBytes = kStages * kStageBytes + kBoxSlots * kBoxBytes;
  // Boxes are loaded, combined and stored in the order the two channel halves consume them: the first
  // box of each half, then the second of each, ...; position j of that order holds box (j & 1) * NBS + j / 2.
  static constexpr __host__ __device__ int box_at(int j) { return (j & 1) * NBS + (j >> 1); }
  static constexpr __host__ __device__ int pos_of(int jb) { return 2 * (jb % NBS) + jb / NBS; }
};

template <int D>
struct SmemCtl {
  uint64_t full[Cfg<D>::kStages];
  uint64_t empty[Cfg<D>::kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t red_bar[2];
  uint64_t stats_ready[2];
  uint64_t g_full[kMaxBoxSlots];   // gate box landed (TMA transaction bytes)
  uint64_t o_full[kMaxBoxSlots];   // box overwritten with the result by the four warps that own it
  uint64_t g_free[kMaxBoxSlots];   // result read by its bulk store: the slot may be refilled
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  volatile uint32_t armed[Cfg<D>::kStages];
  volatile uint32_t g_armed[kMaxBoxSlots];
  alignas(16) float2 red[2][4][BM];   // [tile parity][channel subgroup][token] = (mean, M2) over D/4 channels
  float2 stat[2][BM];                 // [accumulator][token] = (rstd, -mean * rstd)
  float2 cd[D];                       // (c[n], d[n]) of the folded projection
};

template <int D>
constexpr int smem_bytes() {
  return Cfg<D>::kTileBytes + 1024 + static_cast<int>(sizeof(SmemCtl<D>)) + 64;
}

}  // namespace

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
out_proj_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmT,
                const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmO,
                const OutProjArgs p) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = tiles;                                   // kStages x [tri K block | weight K block]
  uint8_t* boxes = tiles + C::kStages * C::kStageBytes;    // kBoxSlots x kBoxBytes
  constexpr int kBoxSlots = C::kBoxSlots;
  SmemCtl<D>* ctl = reinterpret_cast<SmemCtl<D>*>(tiles + C::kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long total_tiles = (p.rows + BM - 1) / BM;
  const long my_tiles = (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;

  if (threadIdx.x == 0) {
    timeline_min(p.timeline, kTlOutStart);
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
    for (int s = 0; s < kBoxSlots; ++s) {
      sm100::mbar_init(&ctl->g_full[s], 1);
      sm100::mbar_init(&ctl->o_full[s], 4);
      sm100::mbar_init(&ctl->g_free[s], 1);
      ctl->g_armed[s] = 2;
    }
    ctl->abort_flag = 0;
    sm100::mbar_init_fence();
  }
  for (int n = threadIdx.x; n < D; n += kThreads) ctl->cd[n] = reinterpret_cast<const float2*>(p.cd)[n];
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

  if (warp == 0) {
    // ------------------------------------------------------------ operand producer (tri from HBM, weights from L2)
    if (lane == 0 && my_tiles > 0) {
      sm100::tma_prefetch_desc(&tmW);
      sm100::tma_prefetch_desc(&tmT);
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
          uint8_t* st = ring + ps.stage * C::kStageBytes;
          ctl->armed[ps.stage] = ps.phase;
          sm100::mbar_arrive_expect_tx(&ctl->full[ps.stage], C::kStageBytes);
          // (tokens, channels) boxes of 64 x 64; a block past the last token is zero-filled
          sm100::tma_load_2d(st, &tmT, &ctl->full[ps.stage], static_cast<int>(m0), kb * 64);
          sm100::tma_load_2d(st + kTriBytes / 2, &tmT, &ctl->full[ps.stage], static_cast<int>(m0 + 64), kb * 64);
#pragma unroll
          for (int n0 = 0; n0 < D; n0 += C::kWBoxRows)
            sm100::tma_load_2d(st + kTriBytes + n0 * 128, &tmW, &ctl->full[ps.stage], kb * 64, n0);
          ps.advance(C::kStages);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    if (lane == 0 && my_tiles > 0) {
      // A: raw tile, token-major (MN-major); B: folded weights, K-major, all D output channels
      constexpr int kN0 = D < 256 ? D : 256;   // column chunks of one MMA step: kN0 and, for D > 256, the rest
      constexpr int kN1 = D - kN0;
      constexpr uint32_t idesc = sm100::umma_idesc_bf16_f32(BM, kN0) | (1u << 15);
      constexpr uint32_t idesc1 = sm100::umma_idesc_bf16_f32(BM, kN1 > 0 ? kN1 : 16) | (1u << 15);
      PipeState ps{0, 0};
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
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
          const uint32_t a_addr = sm100::smem_u32(ring + ps.stage * C::kStageBytes);
          const uint64_t db = sm100::umma_desc_kmajor_sw128(a_addr + kTriBytes);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            // tile: 16 channels per MMA = 2 KB; token blocks of 64 are kTriBytes/2 apart, 8-channel groups 1024 B
            const uint64_t da = sm100::umma_desc_mnmajor_sw128(a_addr + k4 * 2048, kTriBytes / 2, 1024);
            sm100::umma_bf16_ss(d_tmem, da, db + 2 * k4, idesc, (kb | k4) != 0);
            if constexpr (kN1 > 0) {  // weight rows [256, D): 256 rows x 128 B further into the stage
              sm100::umma_bf16_ss(d_tmem + kN0, da, db + ((kN0 * 128) >> 4) + 2 * k4, idesc1, (kb | k4) != 0);
            }
          }
          sm100::umma_commit(&ctl->empty[ps.stage]);
          ps.advance(C::kStages);
        }
        if (!ok) break;
        sm100::umma_commit(&ctl->tmem_full[acc]);
        if (++acc == C::kAccs) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------ gate producer (HBM -> box ring)
    if (lane == 0 && my_tiles > 0) {
      sm100::tma_prefetch_desc(&tmG);
      uint32_t seq = 0;
      bool ok = true;
      for (long it = 0; it < my_tiles && ok; ++it) {
        const long m0 = (blockIdx.x + it * gridDim.x) * BM;
        for (int j = 0; j < C::NBT; ++j) {
          const int jb = C::box_at(j);
          const uint32_t sq = seq + j;
          const uint32_t slot = sq % kBoxSlots, ph = (sq / kBoxSlots) & 1;
          if (!sm100::mbar_wait(&ctl->g_free[slot], ph ^ 1, abort_flag, tmo)) {
            report_timeout(p.status, kKernelOutProj, 6, jb);
            ok = false;
            break;
          }
          ctl->g_armed[slot] = ph;
          sm100::mbar_arrive_expect_tx(&ctl->g_full[slot], kBoxBytes);
          sm100::tma_load_2d(boxes + slot * kBoxBytes, &tmG, &ctl->g_full[slot], jb * 64, static_cast<int>(m0));
        }
        seq += C::NBT;
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ forwarder (finished boxes -> out)
    if (lane == 0 && my_tiles > 0) {
      uint32_t seq = 0;
      bool ok = true;
      for (long it = 0; it < my_tiles && ok; ++it) {
        const long m0 = (blockIdx.x + it * gridDim.x) * BM;
        // the two channel halves finish their boxes side by side: take them in completion order
        for (int j = 0; j < C::NBT; ++j) {
          const int jb = C::box_at(j);
          const uint32_t sq = seq + j;
          const uint32_t slot = sq % kBoxSlots, ph = (sq / kBoxSlots) & 1;
          if (!sm100::mbar_wait(&ctl->o_full[slot], ph, abort_flag, tmo)) {
            report_timeout(p.status, kKernelOutProj, 7, jb);
            ok = false;
            break;
          }
          sm100::tma_store_2d(&tmO, boxes + slot * kBoxBytes, jb * 64, static_cast<int>(m0));
          sm100::tma_store_commit();
          sm100::tma_store_wait_read<0>();
          sm100::mbar_arrive(&ctl->g_free[slot]);
        }
        seq += C::NBT;
      }
      sm100::tma_store_wait_all<0>();
      timeline_max(p.timeline, kTlOutEnd);
    }
  } else if (warp >= kStatWarp0) {
    // ------------------------------------------------------------ statistics (8 warps)
    const int st_tid = threadIdx.x - kStatWarp0 * 32;  // 0..255
    const int pr = st_tid & 63;                        // token pair: tokens 2*pr, 2*pr+1
    const int cs = st_tid >> 6;                        // channel subgroup: 16 of every 64 channels
    const int t0 = 2 * pr;
    // byte offset of the pair inside a (64 channels x 64 tokens) box row, before the swizzle
    const uint32_t blk_off = (t0 >> 6) * (kTriBytes / 2);
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
        const uint8_t* st = ring + ps.stage * C::kStageBytes + blk_off;
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
      if (++acc == C::kAccs) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------ epilogue (8 warps)
    // TMEM lane = token, column = output channel.  Warps 4-7 take the first half of the boxes
    // (channels), warps 8-11 the second half; a warp owns the 32 token rows of its lane quarter.
    const int quarter = warp & 3;
    const int set = (warp - kEpiWarp0) >> 2;
    constexpr int NBS = C::NBT / 2;                 // boxes per channel half
    const int r = quarter * 32 + lane;              // token row inside the tile
    const int sw = r & 7;
    uint32_t acc = 0, acc_phase = 0, seq0 = 0;
    for (long it = 0; it < my_tiles; ++it) {
      bool ok = sm100::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort_flag, tmo);
      ok = ok && sm100::mbar_wait(&ctl->stats_ready[acc], acc_phase, abort_flag, tmo);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        report_timeout(p.status, kKernelOutProj, 2, static_cast<int>(it));
        break;
      }
      sm100::tcgen05_fence_after_sync();
      const float2 rs = ctl->stat[acc][r];  // (rstd, -mean * rstd) of this thread's token
      const uint32_t trow = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * D;
      // TMEM reads are software-pipelined one 16-channel group ahead, across the boxes of the half
      uint32_t pa[16], pb[16];
      sm100::tmem_ld_32x32b_x16(trow + set * NBS * 64, pa);
#pragma unroll
      for (int i = 0; i < NBS; ++i) {
        const int jb = set * NBS + i;
        const uint32_t sq = seq0 + C::pos_of(jb);
        const uint32_t slot = sq % kBoxSlots, ph = (sq / kBoxSlots) & 1;
        ok = sm100::mbar_wait(&ctl->g_full[slot], ph, abort_flag, tmo);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          report_timeout(p.status, kKernelOutProj, 8, jb);
          break;
        }
        uint8_t* row = boxes + slot * kBoxBytes + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int gi = i * 4 + g;
          sm100::tmem_ld_wait();
          if (gi + 1 < NBS * 4) {
            if ((gi & 1) == 0) sm100::tmem_ld_32x32b_x16(trow + set * NBS * 64 + (gi + 1) * 16, pb);
            else sm100::tmem_ld_32x32b_x16(trow + set * NBS * 64 + (gi + 1) * 16, pa);
          }
          const float2* cdp = &ctl->cd[jb * 64 + g * 16];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint4* slot_ptr = reinterpret_cast<uint4*>(row + (((2 * g + hh) ^ sw) << 4));
            const uint4 gt = *slot_ptr;
            const uint32_t gw[4] = {gt.x, gt.y, gt.z, gt.w};
            uint32_t ow[4];
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              const int e = hh * 8 + e2 * 2;
              const float4 cd2 = *reinterpret_cast<const float4*>(cdp + e);  // (c, d) of two channels, same for all lanes
              const float a0 = __uint_as_float((gi & 1) == 0 ? pa[e] : pb[e]);
              const float a1 = __uint_as_float((gi & 1) == 0 ? pa[e + 1] : pb[e + 1]);
              const float y0 = fmaf(a0, rs.x, fmaf(rs.y, cd2.x, cd2.y));
              const float y1 = fmaf(a1, rs.x, fmaf(rs.y, cd2.z, cd2.w));
              ow[e2] = sm100::pack_bf16x2(y0 * sm100::bf16_lo(gw[e2]), y1 * sm100::bf16_hi(gw[e2]));
            }
            *slot_ptr = make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
        }
        sm100::fence_proxy_async_smem();  // generic-proxy writes -> visible to the bulk store
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&ctl->o_full[slot]);
      }
      if (!ok) break;
      seq0 += C::NBT;
      sm100::tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&ctl->tmem_empty[acc]);
      if (++acc == C::kAccs) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();  // single-lane roles reconverge with their warp
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0) {
    // let TMA copies still in flight land before the CTA exits (only after an expired wait)
    for (int s = 0; s < C::kStages; ++s) {
      const uint32_t ph = ctl->armed[s];
      if (ph != 2) {
        const uint64_t t1 = sm100::globaltimer_ns();
        while (!sm100::mbar_test(&ctl->full[s], ph) && sm100::globaltimer_ns() - t1 < 2000000ull) {
        }
      }
    }
    for (int s = 0; s < kBoxSlots; ++s) {
      const uint32_t ph = ctl->g_armed[s];
      if (ph != 2) {
        const uint64_t t1 = sm100::globaltimer_ns();
        while (!sm100::mbar_test(&ctl->g_full[s], ph) && sm100::globaltimer_ns() - t1 < 2000000ull) {
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
  if (D == 384) return smem_bytes<384>();
  if (D == 512) return smem_bytes<512>();
  return -1;
}

template <int D>
static cudaError_t launch_t(const CUtensorMap& tmW, const CUtensorMap& tmT, const CUtensorMap& tmG,
                            const CUtensorMap& tmO, const OutProjArgs& args, int num_sms, cudaStream_t stream) {
  cudaError_t e =
      cudaFuncSetAttribute(out_proj_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<D>());
  if (e != cudaSuccess) return e;
  const long total = (args.rows + BM - 1) / BM;
  if (total <= 0) return cudaSuccess;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  out_proj_kernel<D><<<grid, kThreads, smem_bytes<D>(), stream>>>(tmW, tmT, tmG, tmO, args);
  return cudaGetLastError();
}

cudaError_t launch_out_proj(const CUtensorMap& tmW, const CUtensorMap& tmT, const CUtensorMap& tmG,
                            const CUtensorMap& tmO, const OutProjArgs& args, int num_sms, cudaStream_t stream) {
  if (args.D == 128) return launch_t<128>(tmW, tmT, tmG, tmO, args, num_sms, stream);
  if (args.D == 256) return launch_t<256>(tmW, tmT, tmG, tmO, args, num_sms, stream);
  if (args.D == 384) return launch_t<384>(tmW, tmT, tmG, tmO, args, num_sms, stream);
  if (args.D == 512) return launch_t<512>(tmW, tmT, tmG, tmO, args, num_sms, stream);
  return cudaErrorInvalidValue;
}

}  // namespace trimul
