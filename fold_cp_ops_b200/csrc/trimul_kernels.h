// Internal C++ interface between the C-ABI layer and the three kernels.  Plain structs only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "trimul_common.cuh"

namespace trimul {

// ---------------------------------------------------------------------------------------------
// K_A  LayerNorm + gated dual projection (+ output gate), front reshard fused in the store
// ---------------------------------------------------------------------------------------------
// Token walk: the local pair block is x[b, i, j, :] with row index (b*Ni + i)*Nj + j.  A tile is
// up to 128 tokens along the "walk" coordinate of one "line":
//     row(b, line, w) = b * batch_rows + line * line_rows + w * walk_rows
// outgoing: line = i, walk = j  (line_rows = Nj, walk_rows = 1)
// incoming: line = j, walk = i  (line_rows = 1,  walk_rows = Nj)
// so that the 128 tokens of a tile are consecutive along the CONTRACTION index k of the plane
// they land in, and the store to the channel-major operand plane is contiguous.
struct GatedProjArgs {
  const void* x;         // bf16 (rows, D)
  const void* mask;      // nullable; one scalar per row
  int mask_kind;         // 0 none, 1 bf16, 2 fp32, 3 uint8/bool
  const float* ln_w;     // (D,)
  const float* ln_b;     // (D,) or nullptr
  const float* bias;     // (5*D,) fp32 in PACKED row order, pre-scaled by 1/2 (zeros where the layer has no bias)
  int has_bias;          // 0: every packed bias is zero, the epilogue skips the loads
  float eps;
  int D;
  int batch;
  int n_lines;           // lines per batch plane
  int n_walk;            // tokens per line
  long batch_rows, line_rows, walk_rows;
  // destination of the a / b planes: ptr[s] = base of rank s's operand buffer laid out
  // (2, D_loc, B, plane_rows, plane_cols); this rank fills [dst_base + line*dst_line + w]
  PeerPtrs ab;
  int d_loc;             // D / cp: channels of a (and of b) each rank contracts
  int store_ch;          // channels per a|b store box (64, 32 or 16; divides d_loc, so a box has one owner)
  long plane_elems;      // plane_rows * plane_cols of the destination plane (global N*N)
  long dst_base;         // element offset of (line 0, w 0) inside a plane
  long dst_line;         // element stride between lines inside a plane
  int dst_x0, dst_y0;    // the same origin as tensor-map coordinates: dst_base = dst_y0 * dst_line + dst_x0
  int gate_walk_dim;     // which coordinate of the gate map the walk index is (1 or 2; the line index is the other)
  void* gate_out;        // bf16 (rows, D): sigmoid(xn * g_out^T + b), local, row index as x
  int rotate_chunks;     // 1: CTAs start the gated chunks at different points of the cycle (spreads the stores over the owners)
  unsigned long long* timeline;  // optional device timeline (TimelineSlot), nullptr = off
  DeviceStatus* status;
  uint64_t timeout_ns;
};

// Store-side tensor maps of the projection kernel.  ab[s]: rank s's operand buffer as
// (x, y, batch, 2*D_loc planes), box 64 tokens x store_ch planes, 128-byte swizzle; dim 0 is clipped at the end of
// this rank's walk so ragged tiles never touch a neighbour's tokens.  gate: the local gate buffer
// as (D, walk | line, line | walk, batch), box 64 channels x 128 tokens, 128-byte swizzle.
struct GatedOutMaps {
  CUtensorMap ab[kMaxPeers];
  CUtensorMap gate;
};

int gated_proj_smem_bytes(int D);
cudaError_t launch_gated_proj(const CUtensorMap& tmW, const GatedOutMaps& maps, const GatedProjArgs& args, int num_sms,
                              cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// K_B  per-channel N x N x N contraction, back reshard fused in the store
// ---------------------------------------------------------------------------------------------
struct TriContractArgs {
  int planes;       // D_loc * B, plane l = d_loc * B + b
  int batch;        // B
  int n_i, n_j, n_k;
  // destination: rank (i / ni_loc) * cp1 + (j / nj_loc) owns token block; its buffer is laid out
  // (D, B, ni_loc, nj_loc) and this rank fills channels [chan_offset, chan_offset + D_loc)
  PeerPtrs out;
  int ni_loc, nj_loc, cp1;
  int chan_offset;
  int band_rows;    // tile rows per band of the tile walk (>= 1; 1 = row-major)
  int rot_rows, rot_cols;  // the walk starts at the tile holding this result row / column (this rank's own block)
  unsigned int pace_ns;    // CTA-pair form: longest time a pair waits for the others before a tile (0 = no pacing)
  unsigned long long* timeline;  // optional device timeline, nullptr = off
  DeviceStatus* status;
  uint64_t timeout_ns;
};

// One store descriptor per destination rank: rank s's `tri` buffer as (nj_loc, ni_loc, D*B), box (64, 32, 1).
struct TriOutMaps {
  CUtensorMap map[kMaxPeers];
};

int tri_contract_smem_bytes();
cudaError_t launch_tri_contract(const CUtensorMap& tmA, const CUtensorMap& tmB, const TriOutMaps& out_maps,
                                const TriContractArgs& args, int num_sms, cudaStream_t stream);

// host-side evaluation of the kernels' tile walk over one plane (position r -> tile (ti[r], tj[r]))
void tri_contract_walk(const TriContractArgs& args, int capacity, int* ti, int* tj, int* tiles_i, int* tiles_j);
void tri_contract_pair_walk(const TriContractArgs& args, int capacity, int* ti, int* tj, int* tiles_i, int* tiles_j);

// CTA-pair form (tcgen05 cta_group::2, 256 x 256 tile per pair); tmBhalf has box (64, 128, 1)
cudaError_t launch_tri_contract_pair(const CUtensorMap& tmA, const CUtensorMap& tmBhalf, const TriOutMaps& out_maps,
                                     const TriContractArgs& args, int num_sms, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// K_C  output LayerNorm + output projection, gated
// ---------------------------------------------------------------------------------------------
struct OutProjArgs {
  const void* gate;      // bf16 (rows, D); read through tmG
  const float* cd;       // (D, 2) fp32: c[n] = sum_k bf16(gamma_k W[n,k]),  d[n] = sum_k beta_k W[n,k] + b[n]
  void* out;             // bf16 (rows, D)
  float eps;
  int D;
  long rows;
  unsigned long long* timeline;  // optional device timeline, nullptr = off
  DeviceStatus* status;
  uint64_t timeout_ns;
};

int out_proj_smem_bytes(int D);
// tmW: folded weights bf16 (D, D) K-major, box (64, D); tmT: tri as (tokens, channels), box (64, 64);
// tmG / tmO: gate and out as (D, rows), box (64 channels, 128 tokens), 128-byte swizzle
cudaError_t launch_out_proj(const CUtensorMap& tmW, const CUtensorMap& tmT, const CUtensorMap& tmG,
                            const CUtensorMap& tmO, const OutProjArgs& args, int num_sms, cudaStream_t stream);

}  // namespace trimul
