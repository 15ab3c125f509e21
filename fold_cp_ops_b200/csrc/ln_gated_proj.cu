// Input LayerNorm fused into the gated dual projection:
//     xn   = LayerNorm(x) * gamma + beta                         (fp32 statistics, bf16 operand)
//     a|b  = (xn Wp^T + bp) * sigmoid(xn Wg^T + bg) * mask       (2D channels, bf16)
//     gate = sigmoid(xn Wo^T + bo)                               (D channels, bf16, stays local)
// The packed weights and biases arrive pre-scaled by 1/2 (exact in bf16), so with p' = p/2 and
// g' = g/2 the gated value is  p * sigmoid(g) = p' * tanh(g') + p'  -- one MUFU op and one FMA --
// and the output gate is  0.5 * tanh(go') + 0.5.
// (Reference: ops 1-5 and 10 of trimul_ref, fold_cp_ops/workflows/trimul_autotune.py:1505-1524;
//  front kernel fold_cp_ops/distributed/dual_gated_gemm_a2a.py:56-76; K1 kernels/layernorm.py:730.)
//
// Persistent CTA, 128-token tiles.  Eight LayerNorm warps pull token rows from HBM into
// registers, normalise them there (two-pass fp32 statistics), and write the bf16 operand tile into
// shared memory in the K-major 128-byte-swizzle layout once the tensor core has released it;
// weights stream through a TMA ring (they live in L2); one thread issues tcgen05.mma for the
// tile's column chunks (128 gated channels = 256 columns each, then the output gate) into two
// TMEM accumulators, every CTA starting the gated chunks at a different point so that the grid's
// stores are spread over all owner ranks; sixteen epilogue warps (four per TMEM lane quarter)
// apply bias / gate / mask.  The accumulator is token-per-lane but the operand planes are
// channel-major, so the gated chunks are read in the 16x256b fragment layout (tcgen05.ld), packed
// two channels to a bf16x2 register, and written with stmatrix.trans: one warp instruction stores
// 8 channels x 32 tokens as 16-byte rows of eight consecutive tokens -- the transpose costs no
// instruction of its own.  The CTA-wide staging tile is [token half][channel][64 tokens] with the
// 128-byte swizzle (double-buffered); when all sixteen warps have arrived, one forwarding thread
// sends it as TMA stores of 16 channels x 64 tokens into the channel-major operand plane of the
// rank that owns the channels (front all-to-all fused in the store; at cp=1 that rank is this GPU).
// The output gate leaves the same way, token-major.  No thread issues a global store: per-thread
// 16-byte stores cost this kernel 40 % of its time, and rows shorter than 128 bytes reach half of
// the HBM / NVLink write rate.
#include "trimul_common.cuh"
#include "trimul_kernels.h"

namespace trimul {

namespace {

// Role ablation for profiling builds only: -DTRIMUL_ABLATE=<bits> compiles a SEPARATE library in which a role
// of the projection kernel does no work (results are then wrong), so that the time each role adds can be
// measured.  bit 0: epilogue math and staging, 1: LayerNorm loads / math / tile write, 2: MMA issue,
// 3: a|b and gate stores, 4: weight loads after the first ring fill.  0 (the shipped library): every
// `if (kAblate & x)` below is dead code.
#ifndef TRIMUL_ABLATE
#define TRIMUL_ABLATE 0
#endif
constexpr int kAblate = TRIMUL_ABLATE;

constexpr int BM = 128;
// Seven warpgroups: w0-3 control (w0 weight TMA, w1 MMA issue, w2 TMEM alloc), w4-19 epilogue,
// w20-27 LayerNorm.  Launched at 72 registers per thread and rebalanced with setmaxnreg:
// control 40, epilogue 64, LayerNorm 104 ((40 + 4*64 + 2*104) * 32 = 16128 <= 16384 per SMSP).
constexpr int kEpiWarps = 16;
constexpr int kLnWarps = 8;
constexpr int kEpiWarp0 = 4;
constexpr int kLnWarp0 = kEpiWarp0 + kEpiWarps;
constexpr int kThreads = (kLnWarp0 + kLnWarps) * 32;
constexpr int kHalfTokens = 64;          // tokens per staged row: 128 bytes, the swizzle span
constexpr int kFwdWarp = 3;              // control warp whose lane 0 forwards staged tiles

// Column chunks of a tile.  A gated chunk always holds 128 channels of a (or b): 128 projection
// columns followed by the 128 gate columns of the same channels, N = 256 -- the MMA shape that
// keeps the tensor core off the shared-memory bandwidth limit (a 128 x 128 x 16 MMA reads as many
// operand bytes as it has clocks for).  D = 256: a_lo, a_hi, b_lo, b_hi, gate (N = 256);
// D = 128: a, b, gate (N = 128).  Wide rows (D = 384, 512): six / eight gated chunks and the output gate
// in chunks of 128 columns; the operand tile alone is 96 / 128 KB, so the weight ring has two stages, the
// tile is single-buffered and D = 512 has ONE staging buffer (each chunk's stores drain before the next
// chunk is staged) -- the same pipeline with less slack, not a different kernel.
template <int D>
struct Cfg {
  static constexpr bool kWide = D > 256;
  static constexpr int CH = 128;                // channels per gated chunk
  static constexpr int kChunkN = 2 * CH;        // columns of a gated chunk (also the accumulator stride in TMEM)
  static constexpr int kGated = 2 * D / CH;     // gated chunks per tile
  static constexpr int kPerHalf = kGated / 2;   // gated chunks of a (and of b)
  static constexpr int kGateN = kWide ? 128 : D;         // columns of one output-gate chunk
  static constexpr int kGateChunks = D / kGateN;         // output-gate chunks per tile
  static constexpr int kNumChunks = kGated + kGateChunks;
  static constexpr int KB = D / 64;             // 64-wide K blocks
  static constexpr int kABytes = BM * D * 2;    // one operand tile
  static constexpr int kKBlockBytes = BM * 128; // one K block of the operand tile
  static constexpr int kWBoxRows = kWide ? 128 : D;   // rows one weight TMA box brings (the packed matrix has 5 D rows)
  static constexpr int kWStageBytes = kChunkN * 128;  // one stage: up to 256 weight rows x 64 k
  static constexpr int kWStages = kWide ? 2 : 3;
  static constexpr int kABufs = (D == 128) ? 2 : 1;
  static constexpr int kTmemCols = 512;
  static constexpr int kHalfBytes = CH * 128;        // one token half of a staged a|b chunk: CH channel rows of 64 tokens
  static constexpr int kStageBuf = 2 * kHalfBytes;   // one staging buffer: CH channels x 128 tokens (a|b chunk), or two gate boxes
  static constexpr int kGateBoxBytes = BM * 128;     // gate box: 128 tokens x 64 channels, 128-byte swizzle
  static constexpr int kStBufs = (D == 512) ? 1 : 2; // staging buffers (two to four; more did not pay at D = 128)
  static constexpr int kBoxesPerBuf = kStageBuf / kGateBoxBytes;  // gate boxes one buffer holds
  static constexpr int kGateUses = (kGateN / 64) / kBoxesPerBuf;  // staging buffers one output-gate chunk fills
  static constexpr int kTileBytes = kABufs * kABytes + kWStages * kWStageBytes + kStBufs * kStageBuf;
  // first row of chunk c in the packed weight / bias arrays, and its number of columns
  static constexpr __host__ __device__ int chunk_row0(int c) { return c < kGated ? c * kChunkN : 4 * D + (c - kGated) * kGateN; }
  static constexpr __host__ __device__ int chunk_cols(int c) { return c < kGated ? kChunkN : kGateN; }
};

template <int D>
struct SmemCtl {
  uint64_t w_full[Cfg<D>::kWStages];
  uint64_t w_empty[Cfg<D>::kWStages];
  uint64_t xn_ready[2];
  uint64_t x_empty[2];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t st_full[4];   // staging buffer written by all sixteen epilogue warps (kStBufs of them are used)
  uint64_t st_free[4];   // ... and read completely by the forwarder's bulk stores
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  volatile uint32_t armed[Cfg<D>::kWStages];
};

template <int D>
constexpr int smem_bytes() {
  return Cfg<D>::kTileBytes + 1024 + static_cast<int>(sizeof(SmemCtl<D>)) + 64;
}

__device__ __forceinline__ float tanh_approx(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}

// Two neighbouring channels of one token of a gated chunk: (pa, pb) = p/2 and (ga, gb) = g/2
// accumulators; returns the pair as bf16x2 (even channel in the low half).
template <bool HAS_BIAS, bool HAS_MASK>
__device__ __forceinline__ uint32_t gate_pair(uint32_t pa, uint32_t pb, uint32_t ga, uint32_t gb, float2 bias_p,
                                              float2 bias_g, float mval) {
  float p0 = __uint_as_float(pa), p1 = __uint_as_float(pb);
  float g0 = __uint_as_float(ga), g1 = __uint_as_float(gb);
  if (HAS_BIAS) {
    p0 += bias_p.x;
    p1 += bias_p.y;
    g0 += bias_g.x;
    g1 += bias_g.y;
  }
  float v0 = fmaf(p0, tanh_approx(g0), p0);
  float v1 = fmaf(p1, tanh_approx(g1), p1);
  if (HAS_MASK) {
    v0 *= mval;
    v1 *= mval;
  }
  return sm100::pack_bf16x2(v0, v1);
}

// Sixteen channels x thirty-two tokens of a gated chunk, one warp.  pl / ph (gl / gh): projection
// (gate) accumulators of TMEM lanes 0-15 / 16-31 of the warp's quarter in the 16x256b fragment
// layout.  Each group of eight channels leaves as one stmatrix.x4.trans: tile j = tokens 8j..8j+7,
// memory row = channel.  `row_addr` is the shared-memory address this thread contributes for the
// first group (its row of its tile), `row_step` the distance to the same row of the second group;
// `m[j]` the mask of this thread's token in tile j.
template <bool HAS_BIAS, bool HAS_MASK>
__device__ __forceinline__ void gated16_to_stage(const uint32_t (&pl)[8], const uint32_t (&ph)[8],
                                                 const uint32_t (&gl)[8], const uint32_t (&gh)[8],
                                                 const float* bias_p, const float* bias_g, const float (&m)[4],
                                                 uint32_t row_addr0, uint32_t row_addr1, int tq) {
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    float2 bp = make_float2(0.f, 0.f), bg = make_float2(0.f, 0.f);
    if (HAS_BIAS) {
      bp = __ldg(reinterpret_cast<const float2*>(bias_p + k * 8 + 2 * tq));
      bg = __ldg(reinterpret_cast<const float2*>(bias_g + k * 8 + 2 * tq));
    }
    const uint32_t r0 = gate_pair<HAS_BIAS, HAS_MASK>(pl[4 * k], pl[4 * k + 1], gl[4 * k], gl[4 * k + 1], bp, bg, m[0]);
    const uint32_t r1 =
        gate_pair<HAS_BIAS, HAS_MASK>(pl[4 * k + 2], pl[4 * k + 3], gl[4 * k + 2], gl[4 * k + 3], bp, bg, m[1]);
    const uint32_t r2 = gate_pair<HAS_BIAS, HAS_MASK>(ph[4 * k], ph[4 * k + 1], gh[4 * k], gh[4 * k + 1], bp, bg, m[2]);
    const uint32_t r3 =
        gate_pair<HAS_BIAS, HAS_MASK>(ph[4 * k + 2], ph[4 * k + 3], gh[4 * k + 2], gh[4 * k + 3], bp, bg, m[3]);
    sm100::stmatrix_x4_trans(k == 0 ? row_addr0 : row_addr1, r0, r1, r2, r3);
  }
}

// Sixteen output-gate channels of this thread's token: sigmoid, bf16, written as two 16-byte slots
// (slot0, slot0 + 1) of the token's 128-byte row of a (128 token x 64 channel) gate box, in the
// 128-byte-swizzle layout the TMA store expects (slot ^ (row % 8)); conflict-free.
template <bool HAS_BIAS>
__device__ __forceinline__ void gate16_to_stage(const uint32_t (&gv)[16], const float* bias_g, uint8_t* box, int row,
                                                int slot0) {
  uint8_t* row_ptr = box + row * 128;
  const int sw = row & 7;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    float s[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float ga = __uint_as_float(gv[q * 8 + e]);
      if (HAS_BIAS) ga += __ldg(bias_g + q * 8 + e);
      s[e] = fmaf(0.5f, tanh_approx(ga), 0.5f);
    }
    uint4 pk;
    pk.x = sm100::pack_bf16x2(s[0], s[1]);
    pk.y = sm100::pack_bf16x2(s[2], s[3]);
    pk.z = sm100::pack_bf16x2(s[4], s[5]);
    pk.w = sm100::pack_bf16x2(s[6], s[7]);
    *reinterpret_cast<uint4*>(row_ptr + (((slot0 + q) ^ sw) << 4)) = pk;
  }
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Order in which a CTA walks the five column chunks of a tile.  The four gated chunks (a_lo, a_hi,
// b_lo, b_hi) belong to different owner ranks; CTAs start them at different points of the cycle so
// that, at any moment, the stores of the whole grid are spread over all owners (and all NVLink
// directions) instead of everyone sending to the same half of the ranks.  The gate chunks stay last.
template <int GATED>
__device__ __forceinline__ int chunk_at(int step, int rot) {
  return step < GATED ? (step + rot) % GATED : step;
}

struct TileCoord {
  int b, line, w0;
};

__device__ __forceinline__ TileCoord decode_tile(long t, int tiles_per_line, int n_lines) {
  const long lines = t / tiles_per_line;
  TileCoord c;
  c.w0 = static_cast<int>(t - lines * tiles_per_line) * BM;
  c.b = static_cast<int>(lines / n_lines);
  c.line = static_cast<int>(lines - static_cast<long>(c.b) * n_lines);
  return c;
}

}  // namespace

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
gated_proj_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ GatedOutMaps om,
                  const GatedProjArgs p) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_tiles = tiles;                              // kABufs x kABytes
  uint8_t* w_tiles = tiles + C::kABufs * C::kABytes;     // kWStages x kWStageBytes
  uint8_t* st_tiles = w_tiles + C::kWStages * C::kWStageBytes;  // kStBufs x kStageBuf
  SmemCtl<D>* ctl = reinterpret_cast<SmemCtl<D>*>(tiles + C::kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_per_line = (p.n_walk + BM - 1) / BM;
  const long total_tiles = static_cast<long>(p.batch) * p.n_lines * tiles_per_line;
  const int rot = p.rotate_chunks ? static_cast<int>(blockIdx.x % C::kGated) : 0;  // see chunk_at

  if (threadIdx.x == 0) {
    timeline_min(p.timeline, kTlFrontStart);
    for (int s = 0; s < C::kWStages; ++s) {
      sm100::mbar_init(&ctl->w_full[s], 1);
      sm100::mbar_init(&ctl->w_empty[s], 1);
      ctl->armed[s] = 2;
    }
    for (int a = 0; a < 2; ++a) {
      sm100::mbar_init(&ctl->xn_ready[a], kLnWarps);    // one arrive per LayerNorm warp
      sm100::mbar_init(&ctl->x_empty[a], 1);     // tcgen05.commit
      sm100::mbar_init(&ctl->tmem_full[a], 1);   // tcgen05.commit
      sm100::mbar_init(&ctl->tmem_empty[a], kEpiWarps);  // one arrive per epilogue warp
    }
    for (int b = 0; b < C::kStBufs; ++b) {
      sm100::mbar_init(&ctl->st_full[b], kEpiWarps);     // one arrive per epilogue warp
      sm100::mbar_init(&ctl->st_free[b], 1);             // the forwarder
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

  if (warp < kEpiWarp0) {
    sm100::setmaxnreg_dec<40>();
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------- weight producer (TMA from L2)
      sm100::tma_prefetch_desc(&tmW);
      PipeState ps{0, 0};
      bool ok = true;
      [[maybe_unused]] int n_loads = 0;
      for (long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        for (int ci = 0; ci < C::kNumChunks && ok; ++ci) {
          const int c = chunk_at<C::kGated>(ci, rot);
          for (int kb = 0; kb < C::KB; ++kb) {
            if (!sm100::mbar_wait(&ctl->w_empty[ps.stage], ps.phase ^ 1, abort_flag, tmo)) {
              report_timeout(p.status, kKernelGatedProj, 0, c * 16 + kb);
              ok = false;
              break;
            }
            if ((kAblate & 16) && n_loads++ >= C::kWStages) {
              sm100::mbar_arrive(&ctl->w_full[ps.stage]);  // stale stage: no weight traffic
              ps.advance(C::kWStages);
              continue;
            }
            // a gated chunk is rows [256 c, 256 c + 256) of the packed matrix, the gate chunks the last D rows
            const int rows = C::chunk_cols(c);
            ctl->armed[ps.stage] = ps.phase;
            sm100::mbar_arrive_expect_tx(&ctl->w_full[ps.stage], rows * 128);
            for (int r0 = 0; r0 < rows; r0 += C::kWBoxRows) {
              sm100::tma_load_2d(w_tiles + ps.stage * C::kWStageBytes + r0 * 128, &tmW, &ctl->w_full[ps.stage], kb * 64,
                                 C::chunk_row0(c) + r0);
            }
            ps.advance(C::kWStages);
          }
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------- UMMA issuer
      constexpr uint32_t idesc_gated = sm100::umma_idesc_bf16_f32(BM, C::kChunkN);
      constexpr uint32_t idesc_gate = sm100::umma_idesc_bf16_f32(BM, C::kGateN);
      PipeState ps{0, 0};
      uint32_t acc = 0, acc_phase = 0, buf = 0, buf_phase = 0;
      bool ok = true;
      for (long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        if (!sm100::mbar_wait(&ctl->xn_ready[buf], buf_phase, abort_flag, tmo)) {
          report_timeout(p.status, kKernelGatedProj, 1, -1);
          break;
        }
        sm100::tcgen05_fence_after_sync();
        const uint32_t a_addr = sm100::smem_u32(a_tiles + buf * C::kABytes);
        for (int ci = 0; ci < C::kNumChunks && ok; ++ci) {
          const int c = chunk_at<C::kGated>(ci, rot);
          if (!sm100::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1, abort_flag, tmo)) {
            report_timeout(p.status, kKernelGatedProj, 1, -2);
            ok = false;
            break;
          }
          sm100::tcgen05_fence_after_sync();
          const uint32_t d_tmem = tmem_base + acc * C::kChunkN;
          const uint32_t idesc = c < C::kGated ? idesc_gated : idesc_gate;
          for (int kb = 0; kb < C::KB; ++kb) {
            if (!sm100::mbar_wait(&ctl->w_full[ps.stage], ps.phase, abort_flag, tmo)) {
              report_timeout(p.status, kKernelGatedProj, 1, c * 16 + kb);
              ok = false;
              break;
            }
            sm100::tcgen05_fence_after_sync();
            const uint64_t da = sm100::umma_desc_kmajor_sw128(a_addr + kb * C::kKBlockBytes);
            const uint64_t db = sm100::umma_desc_kmajor_sw128(sm100::smem_u32(w_tiles + ps.stage * C::kWStageBytes));
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              if (!(kAblate & 4)) sm100::umma_bf16_ss(d_tmem, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
            }
            sm100::umma_commit(&ctl->w_empty[ps.stage]);
            ps.advance(C::kWStages);
          }
          if (!ok) break;
          sm100::umma_commit(&ctl->tmem_full[acc]);
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1;
          }
        }
        if (!ok) break;
        sm100::umma_commit(&ctl->x_empty[buf]);  // operand tile free once every MMA of the tile retired
        if (++buf == C::kABufs) {
          buf = 0;
          buf_phase ^= 1;
        }
      }
    } else if (warp == kFwdWarp && lane == 0) {
      // ---------------------------------------------------------- forwarder (TMA stores of staged tiles)
      // Buffer uses per tile: one per a|b chunk and kGateUses per output-gate chunk (D = 256: 4 + 2).
      // Use u lives in buffer u % kStBufs, phase (u / kStBufs) & 1; every use is one bulk group.  A
      // buffer is handed back when its group has been read; with more than two buffers the forwarder
      // waits only for the group kStBufs - 2 behind the newest, so it never stalls on its own last
      // stores.
      constexpr uint32_t NB = C::kStBufs;
      constexpr uint32_t kLag = NB >= 2 ? NB - 2 : 0;   // bulk groups that may still read their buffer
      const int d_loc_n = p.d_loc;
      const int sc = p.store_ch;   // channels one a|b store moves: the largest of 64 / 32 / 16 that divides D / cp
      uint32_t use = 0;
      bool ok = true, stamped = false;
      for (long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileCoord tc = decode_tile(t, tiles_per_line, p.n_lines);
        const int dst_x = p.dst_x0 + tc.w0;
        const int dst_y = p.dst_y0 + tc.line;
        for (int ci = 0; ci < C::kNumChunks && ok; ++ci) {
          const int c = chunk_at<C::kGated>(ci, rot);
          const int n_use = (c < C::kGated) ? 1 : C::kGateUses;
          for (int u = 0; u < n_use && ok; ++u, ++use) {
            const uint32_t b = use % NB, ph = (use / NB) & 1;
            if (!sm100::mbar_wait(&ctl->st_full[b], ph, abort_flag, tmo)) {
              report_timeout(p.status, kKernelGatedProj, 4, c);
              ok = false;
              break;
            }
            const uint8_t* src = st_tiles + b * C::kStageBuf;
            if (c < C::kGated) {
              const int h = c / C::kPerHalf;   // 0: a, 1: b
              if (!stamped) {
                timeline_min(p.timeline, kTlFrontFirstStore);
                stamped = true;
              }
#pragma unroll 1
              for (int k = 0; k < ((kAblate & 8) ? 0 : C::CH / sc); ++k) {
                const int d = (c % C::kPerHalf) * C::CH + k * sc;  // first channel of the group inside the a (or b) half
                const int owner = d / d_loc_n;
                const CUtensorMap* map = &om.ab[owner];
                const int plane = h * d_loc_n + (d - owner * d_loc_n);
                // `sc` channel rows of each token half: (64 tokens, sc channels) boxes, 128-byte rows
                sm100::tma_store_4d(map, src + k * sc * 128, dst_x, dst_y, tc.b, plane);
                sm100::tma_store_4d(map, src + C::kHalfBytes + k * sc * 128, dst_x + kHalfTokens, dst_y, tc.b, plane);
              }
            } else {
              const int cw = p.gate_walk_dim == 1 ? tc.w0 : tc.line;
              const int cl = p.gate_walk_dim == 1 ? tc.line : tc.w0;
#pragma unroll 1
              for (int j = 0; j < ((kAblate & 8) ? 0 : C::kBoxesPerBuf); ++j) {
                const int jb = (c - C::kGated) * (C::kGateN / 64) + u * C::kBoxesPerBuf + j;  // gate box: channels [64 jb, 64 jb + 64)
                sm100::tma_store_4d(&om.gate, src + j * C::kGateBoxBytes, jb * 64, cw, cl, tc.b);
              }
            }
            sm100::tma_store_commit();
            sm100::tma_store_wait_read<kLag>();  // every group but the newest kLag has read its buffer
            if (kLag == 0 || use >= kLag) sm100::mbar_arrive(&ctl->st_free[(use - kLag) % NB]);
          }
        }
      }
      sm100::tma_store_wait_all<0>();  // every bulk store has been performed before the CTA retires
      timeline_max(p.timeline, kTlFrontLastStore);
    }
  } else if (warp >= kLnWarp0) {
    // ------------------------------------------------------------ LayerNorm prologue (8 warps)
    sm100::setmaxnreg_inc<104>();
    const int lw = warp - kLnWarp0;
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);
    if constexpr (C::kWide) {
      // Rows of 768 / 1024 bytes: a lane owns the 16-byte chunks `lane` and `lane + 32` of a row (the second
      // one only exists for lane + 32 < D / 8), a warp normalises its sixteen rows in four batches of four.
      constexpr int CPR = D / 8;
      constexpr int ROWS_PER_WARP = 16, RB = 4;
      const int c0 = lane, c1 = lane + 32;
      const bool has1 = c1 < CPR;
      float gam[16], bet[16];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        gam[e] = p.ln_w[c0 * 8 + e];
        bet[e] = p.ln_b ? p.ln_b[c0 * 8 + e] : 0.0f;
        gam[8 + e] = has1 ? p.ln_w[c1 * 8 + e] : 0.0f;
        bet[8 + e] = (has1 && p.ln_b) ? p.ln_b[c1 * 8 + e] : 0.0f;
      }
      uint32_t buf_phase = 0;
      for (long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        const TileCoord tc = decode_tile(t, tiles_per_line, p.n_lines);
        const long row0 = tc.b * p.batch_rows + tc.line * p.line_rows;
        bool ok = true;
#pragma unroll 1
        for (int rb = 0; rb < ROWS_PER_WARP / RB && ok; ++rb) {
          uint4 raw[RB][2];
#pragma unroll
          for (int i = 0; i < RB; ++i) {
            const int w = tc.w0 + lw * ROWS_PER_WARP + rb * RB + i;
            const uint8_t* row = xb + (row0 + static_cast<long>(w) * p.walk_rows) * D * 2;
            const bool live = w < p.n_walk && !(kAblate & 2);
            raw[i][0] = live ? ldg_nc_v4(row + c0 * 16) : make_uint4(0, 0, 0, 0);
            raw[i][1] = (live && has1) ? ldg_nc_v4(row + c1 * 16) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int i = 0; i < RB; ++i) {
            float v[16];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              v[8 * h + 0] = sm100::bf16_lo(raw[i][h].x); v[8 * h + 1] = sm100::bf16_hi(raw[i][h].x);
              v[8 * h + 2] = sm100::bf16_lo(raw[i][h].y); v[8 * h + 3] = sm100::bf16_hi(raw[i][h].y);
              v[8 * h + 4] = sm100::bf16_lo(raw[i][h].z); v[8 * h + 5] = sm100::bf16_hi(raw[i][h].z);
              v[8 * h + 6] = sm100::bf16_lo(raw[i][h].w); v[8 * h + 7] = sm100::bf16_hi(raw[i][h].w);
            }
            float sum = 0.0f;
#pragma unroll
            for (int e = 0; e < 16; ++e) sum += v[e];
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const float mean = sum * (1.0f / D);
            float q = 0.0f;
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              v[e] -= mean;
              if (e < 8 || has1) q = fmaf(v[e], v[e], q);
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
            const float rstd = rsqrtf(q * (1.0f / D) + p.eps);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const float* g = gam + 8 * h;
              const float* bt = bet + 8 * h;
              const float* vv = v + 8 * h;
              raw[i][h].x = sm100::pack_bf16x2(fmaf(vv[0] * rstd, g[0], bt[0]), fmaf(vv[1] * rstd, g[1], bt[1]));
              raw[i][h].y = sm100::pack_bf16x2(fmaf(vv[2] * rstd, g[2], bt[2]), fmaf(vv[3] * rstd, g[3], bt[3]));
              raw[i][h].z = sm100::pack_bf16x2(fmaf(vv[4] * rstd, g[4], bt[4]), fmaf(vv[5] * rstd, g[5], bt[5]));
              raw[i][h].w = sm100::pack_bf16x2(fmaf(vv[6] * rstd, g[6], bt[6]), fmaf(vv[7] * rstd, g[7], bt[7]));
            }
          }
          if (rb == 0) {  // the tensor core must have released the (single) operand tile before the first write
            // That wait lasts most of a tile's MMA phase.  The rows of the three later batches are loaded only
            // after it (no registers to park them in): ask L2 for them now, so that those loads are L2 hits.
            if (!(kAblate & 2)) {
#pragma unroll
              for (int i = RB; i < ROWS_PER_WARP; ++i) {
                const int w = tc.w0 + lw * ROWS_PER_WARP + i;
                if (w < p.n_walk) {
                  const uint8_t* row = xb + (row0 + static_cast<long>(w) * p.walk_rows) * D * 2;
                  prefetch_l2(row + c0 * 16);
                  if (has1) prefetch_l2(row + c1 * 16);
                }
              }
            }
            ok = sm100::mbar_wait(&ctl->x_empty[0], buf_phase ^ 1, abort_flag, tmo);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
              report_timeout(p.status, kKernelGatedProj, 3, static_cast<int>(t));
              break;
            }
          }
          if (!(kAblate & 2)) {
#pragma unroll
            for (int i = 0; i < RB; ++i) {
              const int r = lw * ROWS_PER_WARP + rb * RB + i;
              // K-major, 128-byte swizzle: K block (chunk / 8), row r, 16-byte slot (chunk % 8) ^ (r % 8)
              *reinterpret_cast<uint4*>(a_tiles + (c0 >> 3) * C::kKBlockBytes + r * 128 + (((c0 & 7) ^ (r & 7)) << 4)) =
                  raw[i][0];
              if (has1)
                *reinterpret_cast<uint4*>(a_tiles + (c1 >> 3) * C::kKBlockBytes + r * 128 + (((c1 & 7) ^ (r & 7)) << 4)) =
                    raw[i][1];
            }
          }
        }
        if (!ok) break;
        sm100::fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&ctl->xn_ready[0]);
        buf_phase ^= 1;
      }
    } else {
      constexpr int CPR = D / 8;        // 16-byte chunks per row
      constexpr int RPP = 32 / CPR;     // rows one warp-wide load covers
      constexpr int ROWS_PER_WARP = 16;
      constexpr int PASSES = ROWS_PER_WARP / RPP;
      const int chunk = lane % CPR;
      const int sub = lane / CPR;
      float gam[8], bet[8];
  #pragma unroll
      for (int e = 0; e < 8; ++e) {
        gam[e] = p.ln_w[chunk * 8 + e];
        bet[e] = p.ln_b ? p.ln_b[chunk * 8 + e] : 0.0f;
      }
      // every row of this warp is requested before any is used: 16 rows in flight per warp
      auto request_rows = [&](long t, uint4 (&dst)[PASSES]) {
        const TileCoord tc = decode_tile(t, tiles_per_line, p.n_lines);
        const long row0 = tc.b * p.batch_rows + tc.line * p.line_rows;
  #pragma unroll
        for (int ps = 0; ps < PASSES; ++ps) {
          const int r = lw * ROWS_PER_WARP + ps * RPP + sub;
          const int w = tc.w0 + r;
          if (w < p.n_walk && !(kAblate & 2)) {
            dst[ps] = ldg_nc_v4(xb + ((row0 + w * p.walk_rows) * D + chunk * 8) * 2);
          } else {
            dst[ps] = make_uint4(0, 0, 0, 0);
          }
        }
      };
      // When a tile's rows fit in half of the register budget (D = 128: eight 16-byte loads per lane) the
      // rows of the NEXT tile are requested before this tile is written to shared memory, so the HBM latency
      // of a tile is hidden behind the normalisation and hand-off of the one before it; at D = 256 one tile
      // fills the registers, and the single operand buffer gives the loads a whole MMA phase anyway.
      constexpr bool kPrefetch = PASSES <= 8;
      uint4 raw[PASSES];
      uint4 ahead[kPrefetch ? PASSES : 1];
      bool have_rows = false;
      uint32_t buf = 0, buf_phase = 0;
      for (long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        if (!have_rows) request_rows(t, raw);
        // normalise in registers while the tensor core still reads the previous tile
  #pragma unroll
        for (int ps = 0; ps < ((kAblate & 2) ? 0 : PASSES); ++ps) {
          float v[8];
          v[0] = sm100::bf16_lo(raw[ps].x); v[1] = sm100::bf16_hi(raw[ps].x);
          v[2] = sm100::bf16_lo(raw[ps].y); v[3] = sm100::bf16_hi(raw[ps].y);
          v[4] = sm100::bf16_lo(raw[ps].z); v[5] = sm100::bf16_hi(raw[ps].z);
          v[6] = sm100::bf16_lo(raw[ps].w); v[7] = sm100::bf16_hi(raw[ps].w);
          float s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
  #pragma unroll
          for (int o = CPR / 2; o >= 1; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
          const float mean = s * (1.0f / D);
          float q = 0.0f;
  #pragma unroll
          for (int e = 0; e < 8; ++e) {
            v[e] -= mean;
            q = fmaf(v[e], v[e], q);
          }
  #pragma unroll
          for (int o = CPR / 2; o >= 1; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
          const float rstd = rsqrtf(q * (1.0f / D) + p.eps);
          raw[ps].x = sm100::pack_bf16x2(fmaf(v[0] * rstd, gam[0], bet[0]), fmaf(v[1] * rstd, gam[1], bet[1]));
          raw[ps].y = sm100::pack_bf16x2(fmaf(v[2] * rstd, gam[2], bet[2]), fmaf(v[3] * rstd, gam[3], bet[3]));
          raw[ps].z = sm100::pack_bf16x2(fmaf(v[4] * rstd, gam[4], bet[4]), fmaf(v[5] * rstd, gam[5], bet[5]));
          raw[ps].w = sm100::pack_bf16x2(fmaf(v[6] * rstd, gam[6], bet[6]), fmaf(v[7] * rstd, gam[7], bet[7]));
        }
        if constexpr (kPrefetch) {
          have_rows = t + gridDim.x < total_tiles;
          if (have_rows) request_rows(t + gridDim.x, ahead);
        }
        bool ok = sm100::mbar_wait(&ctl->x_empty[buf], buf_phase ^ 1, abort_flag, tmo);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          report_timeout(p.status, kKernelGatedProj, 3, static_cast<int>(t));
          break;
        }
        uint8_t* a_tile = a_tiles + buf * C::kABytes;
  #pragma unroll
        for (int ps = 0; ps < ((kAblate & 2) ? 0 : PASSES); ++ps) {
          const int r = lw * ROWS_PER_WARP + ps * RPP + sub;
          // K-major, 128-byte swizzle: K block (chunk/8), row r, 16-byte slot (chunk%8) ^ (r%8)
          const uint32_t off = (chunk >> 3) * C::kKBlockBytes + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(a_tile + off) = raw[ps];
        }
        sm100::fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&ctl->xn_ready[buf]);
        if constexpr (kPrefetch) {
          if (have_rows) {
  #pragma unroll
            for (int ps = 0; ps < PASSES; ++ps) raw[ps] = ahead[ps];
          }
        }
        if (++buf == C::kABufs) {
          buf = 0;
          buf_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (16 warps)
    sm100::setmaxnreg_dec<64>();
    const int ew = warp - kEpiWarp0;
    const int quarter = warp & 3;   // TMEM lane quarter this warp may read
    const int part = ew >> 2;       // which quarter of the chunk's columns
    const int r = quarter * 32 + lane;  // token row of this thread inside the tile (32x32b reads: the gate chunk)
    // 16x256b fragment reads of the gated chunks: this thread holds channel pair `tq` of tokens
    // quarter*32 + 8j + tr (j = 0..3); for stmatrix it addresses row `mr` of token tile `mj`
    const int tq = lane & 3, tr = lane >> 2;
    const int mj = lane >> 3, mr = lane & 7;
    uint32_t acc = 0, acc_phase = 0, use = 0;
    bool ok = true;
    for (long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const TileCoord tc = decode_tile(t, tiles_per_line, p.n_lines);
      float mval[4] = {1.0f, 1.0f, 1.0f, 1.0f};
      if (p.mask_kind != 0) {
        const long row0 = tc.b * p.batch_rows + tc.line * p.line_rows;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int w = tc.w0 + quarter * 32 + 8 * j + tr;
          if (w < p.n_walk) {
            const long srow = row0 + static_cast<long>(w) * p.walk_rows;
            if (p.mask_kind == 1) {
              mval[j] = __bfloat162float(static_cast<const __nv_bfloat16*>(p.mask)[srow]);
            } else if (p.mask_kind == 2) {
              mval[j] = static_cast<const float*>(p.mask)[srow];
            } else {
              mval[j] = static_cast<const uint8_t*>(p.mask)[srow] ? 1.0f : 0.0f;
            }
          }
        }
      }
      // a warp whose 32 tokens all carry mask 1 (the common case) skips the multiply: x * 1 is exact
      const bool warp_has_mask =
          p.mask_kind != 0 &&
          !__all_sync(0xffffffffu, mval[0] == 1.0f && mval[1] == 1.0f && mval[2] == 1.0f && mval[3] == 1.0f);
      for (int ci = 0; ci < C::kNumChunks; ++ci) {
        const int c = chunk_at<C::kGated>(ci, rot);
        ok = sm100::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort_flag, tmo);
        // the staging buffer(s) of this chunk must have been forwarded (two uses ago)
        constexpr uint32_t NB = C::kStBufs;
        const int n_use = (c < C::kGated) ? 1 : C::kGateUses;
        for (int u = 0; u < n_use; ++u) {
          const uint32_t b = (use + u) % NB, ph = ((use + u) / NB) & 1;
          ok = ok && sm100::mbar_wait(&ctl->st_free[b], ph ^ 1, abort_flag, tmo);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          report_timeout(p.status, kKernelGatedProj, 2, c);
          break;
        }
        sm100::tcgen05_fence_after_sync();
        const uint32_t trow = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * C::kChunkN;
        if (kAblate & 1) {
          // ablated: no TMEM reads, no math, nothing staged
        } else if (c < C::kGated) {
          // gated chunk: columns [0, CH) projection, [CH, 2CH) gate, same channel order
          constexpr int CW = C::CH / 4;   // channels of the chunk this warp handles
          constexpr int NS = CW / 16;     // in 16-channel sub-groups
          const int colw = part * CW;
          const float* bias_p0 = p.bias + C::chunk_row0(c) + colw;
          const uint32_t trow_hi = trow + (16u << 16);   // TMEM lanes 16-31 of the quarter
          // staged layout: token half (quarter / 2), channel row, 16-byte slot of eight tokens
          // (quarter % 2) * 4 + tile, XOR-swizzled with the row as the store descriptor expects
          const uint32_t half_addr =
              sm100::smem_u32(st_tiles + (use % NB) * C::kStageBuf + (quarter >> 1) * C::kHalfBytes);
          const int slot = (quarter & 1) * 4 + mj;
#pragma unroll
          for (int sg = 0; sg < NS; ++sg) {
            const int c0 = colw + sg * 16;
            uint32_t pl[8], ph[8], gl[8], gh[8];
            sm100::tmem_ld_16x256b_x2(trow + c0, pl);
            sm100::tmem_ld_16x256b_x2(trow_hi + c0, ph);
            sm100::tmem_ld_16x256b_x2(trow + C::CH + c0, gl);
            sm100::tmem_ld_16x256b_x2(trow_hi + C::CH + c0, gh);
            sm100::tmem_ld_wait();
            const int row_a = c0 + mr, row_b = c0 + 8 + mr;
            const uint32_t addr_a = half_addr + row_a * 128 + ((slot ^ (row_a & 7)) << 4);
            const uint32_t addr_b = half_addr + row_b * 128 + ((slot ^ (row_b & 7)) << 4);
            const float* bp = bias_p0 + sg * 16;
            if (p.has_bias) {
              if (warp_has_mask) gated16_to_stage<true, true>(pl, ph, gl, gh, bp, bp + C::CH, mval, addr_a, addr_b, tq);
              else gated16_to_stage<true, false>(pl, ph, gl, gh, bp, bp + C::CH, mval, addr_a, addr_b, tq);
            } else {
              if (warp_has_mask) gated16_to_stage<false, true>(pl, ph, gl, gh, bp, bp + C::CH, mval, addr_a, addr_b, tq);
              else gated16_to_stage<false, false>(pl, ph, gl, gh, bp, bp + C::CH, mval, addr_a, addr_b, tq);
            }
          }
        } else {
          // output-gate chunk: sigmoid only, token-major, into (128 token x 64 channel) boxes
          constexpr int GW = C::kGateN / 4;
          constexpr int NS = GW / 16;
          const int colw = part * GW;
          const float* bias_g0 = p.bias + C::chunk_row0(c) + colw;
          const int jb = colw >> 6;  // gate box of this warp's columns inside the chunk; boxes fill the chunk's buffers in order
          uint8_t* box = st_tiles + ((use + jb / C::kBoxesPerBuf) % NB) * C::kStageBuf +
                         (jb % C::kBoxesPerBuf) * C::kGateBoxBytes;
          const int slot_base = (colw & 63) >> 3;
#pragma unroll
          for (int sg = 0; sg < NS; ++sg) {
            uint32_t gv[16];
            sm100::tmem_ld_32x32b_x16(trow + colw + sg * 16, gv);
            sm100::tmem_ld_wait();
            if (p.has_bias) gate16_to_stage<true>(gv, bias_g0 + sg * 16, box, r, slot_base + sg * 2);
            else gate16_to_stage<false>(gv, bias_g0 + sg * 16, box, r, slot_base + sg * 2);
          }
        }
        // accumulator back to the tensor core, staged data over to the forwarder
        sm100::tcgen05_fence_before_sync();
        sm100::fence_proxy_async_smem();  // generic-proxy writes -> visible to the bulk stores
        __syncwarp();
        if (lane == 0) {
          sm100::mbar_arrive(&ctl->tmem_empty[acc]);
          for (int u = 0; u < n_use; ++u) sm100::mbar_arrive(&ctl->st_full[(use + u) % NB]);
        }
        use += n_use;
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();  // single-lane roles reconverge with their warp
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0) {
    for (int s = 0; s < C::kWStages; ++s) {
      const uint32_t ph = ctl->armed[s];
      if (ph != 2) {
        const uint64_t t0 = sm100::globaltimer_ns();
        while (!sm100::mbar_test(&ctl->w_full[s], ph) && sm100::globaltimer_ns() - t0 < 2000000ull) {
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
int gated_proj_smem_bytes(int D) {
  if (D == 128) return smem_bytes<128>();
  if (D == 256) return smem_bytes<256>();
  if (D == 384) return smem_bytes<384>();
  if (D == 512) return smem_bytes<512>();
  return -1;
}

template <int D>
static cudaError_t launch_t(const CUtensorMap& tmW, const GatedOutMaps& maps, const GatedProjArgs& args, int num_sms,
                            cudaStream_t stream) {
  cudaError_t e =
      cudaFuncSetAttribute(gated_proj_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<D>());
  if (e != cudaSuccess) return e;
  const int tiles_per_line = (args.n_walk + BM - 1) / BM;
  const long total = static_cast<long>(args.batch) * args.n_lines * tiles_per_line;
  if (total <= 0) return cudaSuccess;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  gated_proj_kernel<D><<<grid, kThreads, smem_bytes<D>(), stream>>>(tmW, maps, args);
  return cudaGetLastError();
}

cudaError_t launch_gated_proj(const CUtensorMap& tmW, const GatedOutMaps& maps, const GatedProjArgs& args, int num_sms,
                              cudaStream_t stream) {
  if (args.D == 128) return launch_t<128>(tmW, maps, args, num_sms, stream);
  if (args.D == 256) return launch_t<256>(tmW, maps, args, num_sms, stream);
  if (args.D == 384) return launch_t<384>(tmW, maps, args, num_sms, stream);
  if (args.D == 512) return launch_t<512>(tmW, maps, args, num_sms, stream);
  return cudaErrorInvalidValue;
}

}  // namespace trimul
