// Epilogue shared by the single-CTA and the CTA-pair contraction kernels: one warp converts its
// 32-row band of a 256-column accumulator to bf16 and sends it to the rank that owns the tokens.
#pragma once
#include "trimul_common.cuh"
#include "trimul_kernels.h"

namespace trimul {
namespace tri {

constexpr int kAccCols = 256;                      // accumulator columns (tile width)
constexpr int kOutCols = 64;                       // columns per output store (128-byte rows)
constexpr int kOutBufBytes = 32 * kOutCols * 2;    // 32 rows x 64 cols bf16 = 4 KB, one per warp and parity
constexpr int kOutStageBytes = 4 * 2 * kOutBufBytes;

// `i0w`: first row of the warp's band in the plane; `j_tile0`: first column of the tile;
// `taddr_row`: TMEM address of the band (lane quarter and accumulator already applied);
// `warp_stage`: the warp's two 4 KB staging buffers; `out_par`: running parity of their use.
// 32 x 64 blocks inside the matrix and inside one owner's token block go out as TMA stores of
// 128-byte rows (128-byte swizzle in the stage); ragged edges and blocks that straddle two owners
// fall back to 16-byte vector stores from registers.
__device__ __forceinline__ void store_band(const TriContractArgs& p, const TriOutMaps& out_maps, uint32_t taddr_row,
                                           int i0w, int j_tile0, int plane, uint8_t* warp_stage, uint32_t& out_par,
                                           int lane) {
  const long owner_plane_elems = static_cast<long>(p.ni_loc) * p.nj_loc;
  const int i = i0w + lane;
  const bool row_ok = i < p.n_i;
  const int i_blk = row_ok ? i / p.ni_loc : 0;
  const int i_l = i - i_blk * p.ni_loc;
  // the band can go out as TMA stores when it lies inside the matrix and inside one owner's row block
  const int iw_blk = i0w / p.ni_loc;
  const bool band_ok = (i0w + 31 < p.n_i) && ((i0w + 31) / p.ni_loc == iw_blk);
  // destination plane index on the owner: (chan_offset + d_loc) * B + b  == chan_offset*B + plane
  const long dst_plane = static_cast<long>(p.chan_offset) * p.batch + plane;
#pragma unroll 1
  for (int cc = 0; cc < kAccCols / kOutCols; ++cc) {
    uint32_t v[kOutCols];
    {
      uint32_t (&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&v[0]);
      uint32_t (&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&v[32]);
      sm100::tmem_ld_32x32b_x32(taddr_row + cc * kOutCols, lo);
      sm100::tmem_ld_32x32b_x32(taddr_row + cc * kOutCols + 32, hi);
    }
    const int j0 = j_tile0 + cc * kOutCols;
    const int jw_blk = j0 / p.nj_loc;
    const bool fast = band_ok && (j0 + kOutCols - 1 < p.n_j) && ((j0 + kOutCols - 1) / p.nj_loc == jw_blk);
    uint8_t* buf = warp_stage + (out_par & 1) * kOutBufBytes;
    if (fast) {
      // the store that last used this buffer (two chunks ago) must have finished reading it
      if (lane == 0) sm100::tma_store_wait_read<1>();
      __syncwarp();
    }
    sm100::tmem_ld_wait();
    if (fast) {
#pragma unroll
      for (int q = 0; q < kOutCols / 8; ++q) {
        uint4 pk;
        pk.x = sm100::pack_bf16x2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
        pk.y = sm100::pack_bf16x2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
        pk.z = sm100::pack_bf16x2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
        pk.w = sm100::pack_bf16x2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
        // row = lane, 16-byte chunk q, 128-byte swizzle (what the store descriptor expects)
        *reinterpret_cast<uint4*>(buf + lane * 128 + ((q ^ (lane & 7)) << 4)) = pk;
      }
      sm100::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        sm100::tma_store_3d(&out_maps.map[iw_blk * p.cp1 + jw_blk], buf, j0 - jw_blk * p.nj_loc,
                            i0w - iw_blk * p.ni_loc, static_cast<int>(dst_plane));
        sm100::tma_store_commit();
      }
      ++out_par;
    } else if (row_ok && j0 < p.n_j) {
#pragma unroll
      for (int q = 0; q < kOutCols / 8; ++q) {
        const int j = j0 + q * 8;
        if (j < p.n_j) {  // n_j % 8 == 0: a 16-byte vector never straddles the edge or an owner
          const int j_blk = j / p.nj_loc;
          const int j_l = j - j_blk * p.nj_loc;
          __nv_bfloat16* base = static_cast<__nv_bfloat16*>(p.out.ptr[i_blk * p.cp1 + j_blk]);
          uint4 pk;
          pk.x = sm100::pack_bf16x2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
          pk.y = sm100::pack_bf16x2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
          pk.z = sm100::pack_bf16x2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
          pk.w = sm100::pack_bf16x2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
          *reinterpret_cast<uint4*>(base + dst_plane * owner_plane_elems + static_cast<long>(i_l) * p.nj_loc + j_l) =
              pk;
        }
      }
    }
  }
}

}  // namespace tri
}  // namespace trimul
