// C ABI of libtrimul_sm100.so (declared in include/trimul_sm100.h): argument checking, geometry
// derivation, TMA descriptor encoding, and the launches.  No allocation, no hidden streams.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>

#include "../../include/trimul_sm100.h"
#include "trimul_kernels.h"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* where) {
  return fail(TRIMUL_ERR_CUDA, "%s: %s", where, cudaGetErrorString(e));
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup: no link-time libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// bf16 tensor, innermost dim contiguous, 128-byte swizzle unless told otherwise, zero fill out of bounds.
int make_tmap(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
              const uint32_t* box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(TRIMUL_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim,
                  gstr, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TRIMUL_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TRIMUL_OK;
}

int num_sms_current() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) cached[dev] = n;
  }
  return cached[dev];
}

struct Derived {
  int cp, r0, r1, ni_loc, nj_loc, d_loc;
  long i_off, j_off, rows;
};

int check_geom(const trimul_geom_t* g, Derived* d) {
  if (g == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "geom is NULL");
  if (g->batch < 1 || g->n < 1) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "batch and n must be >= 1");
  if (g->d != 128 && g->d != 256 && g->d != 384 && g->d != 512)
    return fail(TRIMUL_ERR_UNSUPPORTED_SHAPE, "feature width d=%d is not supported (128, 256, 384 or 512)", g->d);
  if (g->cp0 < 1 || g->cp1 < 1 || g->cp0 * g->cp1 > TRIMUL_MAX_PEERS)
    return fail(TRIMUL_ERR_INVALID_ARGUMENT, "cp grid %d x %d must have 1..%d ranks", g->cp0, g->cp1,
                TRIMUL_MAX_PEERS);
  const int cp = g->cp0 * g->cp1;
  if (g->rank < 0 || g->rank >= cp) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "rank %d outside cp=%d", g->rank, cp);
  if (g->direction != TRIMUL_OUTGOING && g->direction != TRIMUL_INCOMING)
    return fail(TRIMUL_ERR_INVALID_ARGUMENT, "direction must be 0 (outgoing) or 1 (incoming)");
  if (g->n % 8 != 0) return fail(TRIMUL_ERR_UNSUPPORTED_SHAPE, "n=%d must be a multiple of 8", g->n);
  if (g->n % g->cp0 != 0 || g->n % g->cp1 != 0)
    return fail(TRIMUL_ERR_UNSUPPORTED_SHAPE, "n=%d must divide by each cp axis (%d, %d)", g->n, g->cp0, g->cp1);
  if (g->d % cp != 0) return fail(TRIMUL_ERR_UNSUPPORTED_SHAPE, "d=%d must divide by cp=%d", g->d, cp);
  d->cp = cp;
  d->r0 = g->rank / g->cp1;
  d->r1 = g->rank % g->cp1;
  d->ni_loc = g->n / g->cp0;
  d->nj_loc = g->n / g->cp1;
  if (cp > 1 && (d->ni_loc % 8 != 0 || d->nj_loc % 8 != 0))
    return fail(TRIMUL_ERR_UNSUPPORTED_SHAPE, "local token extents (%d, %d) must be multiples of 8", d->ni_loc,
                d->nj_loc);
  d->d_loc = g->d / cp;
  if (d->d_loc % 16 != 0)
    return fail(TRIMUL_ERR_UNSUPPORTED_SHAPE, "d/cp=%d must be a multiple of 16 (the reshard stores move 16 channels)", d->d_loc);
  d->i_off = static_cast<long>(d->r0) * d->ni_loc;
  d->j_off = static_cast<long>(d->r1) * d->nj_loc;
  d->rows = static_cast<long>(g->batch) * d->ni_loc * d->nj_loc;
  return TRIMUL_OK;
}


// Where this rank's tokens go in the front reshard and where contraction tiles go in the back one.
void derive_plan(const trimul_geom_t* g, const Derived& d, trimul_reshard_plan_t* p) {
  const long n = g->n;
  p->batch_rows = static_cast<long>(d.ni_loc) * d.nj_loc;
  if (g->direction == TRIMUL_OUTGOING) {
    if (g->cp1 == 1) {
      // rows (b, i, :) are contiguous in x and in the destination plane: walk the whole block
      p->n_lines = 1;
      p->n_walk = static_cast<int32_t>(static_cast<long>(d.ni_loc) * d.nj_loc);
      p->line_rows = 0;
      p->walk_rows = 1;
      p->dst_base = d.i_off * n;
      p->dst_line = 0;
    } else {
      p->n_lines = d.ni_loc;
      p->n_walk = d.nj_loc;
      p->line_rows = d.nj_loc;
      p->walk_rows = 1;
      p->dst_base = d.i_off * n + d.j_off;
      p->dst_line = n;
    }
  } else {
    p->n_lines = d.nj_loc;
    p->n_walk = d.ni_loc;
    p->line_rows = 1;
    p->walk_rows = d.nj_loc;
    p->dst_base = d.j_off * n + d.i_off;
    p->dst_line = n;
  }
  p->plane_elems = n * n;
  p->d_loc = d.d_loc;
  p->planes = d.d_loc * g->batch;
  p->ni_loc = d.ni_loc;
  p->nj_loc = d.nj_loc;
  p->chan_offset = g->rank * d.d_loc;
  p->rows = d.rows;
}

// ---------------------------------------------------------------------------------------------
// weight packing kernel (runs once per layer)
// ---------------------------------------------------------------------------------------------
__global__ void pack_weights_kernel(int d, const __nv_bfloat16* p_in, const __nv_bfloat16* g_in,
                                    const __nv_bfloat16* g_out, const float* p_in_b, const float* g_in_b,
                                    const float* g_out_b, __nv_bfloat16* w_packed, float* bias_packed) {
  const int row = blockIdx.x;  // packed row 0 .. 5d-1
  // rows [0, 4d): gated chunks of 256 rows = 128 projection rows followed by the 128 gate rows of the
  // same channels; chunk c covers rows [128 c, 128 c + 128) of the (2d, d) matrices (a first, then b).
  // rows [4d, 5d): the output gate.
  const __nv_bfloat16* src;
  float bias;
  if (row < 4 * d) {
    const int c = row / 256;
    const int rr = row - c * 256;
    const bool is_gate = rr >= 128;
    const int src_row = c * 128 + (rr & 127);
    src = (is_gate ? g_in : p_in) + static_cast<long>(src_row) * d;
    const float* b = is_gate ? g_in_b : p_in_b;
    bias = b ? b[src_row] : 0.0f;
  } else {
    const int rr = row - 4 * d;
    src = g_out + static_cast<long>(rr) * d;
    bias = g_out_b ? g_out_b[rr] : 0.0f;
  }
  // every packed row and bias carries a factor 1/2 (exact in bf16): the projection kernel turns
  // p * sigmoid(g) into (p/2) * tanh(g/2) + p/2 and sigmoid(go) into 0.5 * tanh(go/2) + 0.5
  for (int c = threadIdx.x; c < d; c += blockDim.x)
    w_packed[static_cast<long>(row) * d + c] = __float2bfloat16_rn(0.5f * __bfloat162float(src[c]));
  if (threadIdx.x == 0) bias_packed[row] = 0.5f * bias;
}


// Fold the output LayerNorm into the output projection (runs once per layer).  One block per
// output row n:  w_fold[n,k] = bf16(gamma_k * W[n,k]);  c[n] = sum_k w_fold[n,k];
// d[n] = sum_k beta_k * W[n,k] + b[n].
__global__ void pack_out_weights_kernel(int d, const __nv_bfloat16* w_out, const float* ln_w, const float* ln_b,
                                        const float* bias, __nv_bfloat16* w_fold, float* cd) {
  const int n = blockIdx.x;
  float c = 0.f, dd = 0.f;
  for (int k = threadIdx.x; k < d; k += blockDim.x) {
    const float w = __bfloat162float(w_out[static_cast<long>(n) * d + k]);
    const __nv_bfloat16 wf = __float2bfloat16_rn(ln_w[k] * w);
    w_fold[static_cast<long>(n) * d + k] = wf;
    c += __bfloat162float(wf);
    dd += (ln_b ? ln_b[k] : 0.f) * w;
  }
  __shared__ float sc[32], sd[32];
  for (int o = 16; o >= 1; o >>= 1) {
    c += __shfl_xor_sync(0xffffffffu, c, o);
    dd += __shfl_xor_sync(0xffffffffu, dd, o);
  }
  if ((threadIdx.x & 31) == 0) {
    sc[threadIdx.x >> 5] = c;
    sd[threadIdx.x >> 5] = dd;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float tc = 0.f, td = 0.f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) {
      tc += sc[w];
      td += sd[w];
    }
    cd[2 * n] = tc;
    cd[2 * n + 1] = td + (bias ? bias[n] : 0.f);
  }
}


// ---------------------------------------------------------------------------------------------
// the three launches, split into "encode once" (build_*) and "launch" (launch_*)
// ---------------------------------------------------------------------------------------------
struct FrontPart {
  CUtensorMap tmW;
  trimul::GatedOutMaps maps;
  trimul::GatedProjArgs args;
};

struct ContractPart {
  CUtensorMap tmA, tmB;
  trimul::TriOutMaps maps;
  trimul::TriContractArgs args;
  bool pair;
};

struct OutPart {
  CUtensorMap tmW, tmT, tmG, tmO;
  const void* tmO_for;  // the `out` pointer tmO was encoded for (re-encoded only when it changes)
  trimul::OutProjArgs args;
};

constexpr uint64_t kDefaultTimeoutNs = 2000000000ull;

int build_front(const trimul_geom_t* geom, const Derived& d, const trimul_tuning_t* tuning, const float* ln_w,
                const float* ln_b, const void* w_packed, const float* bias_packed, void* const* ab_peers, void* gate_out,
                trimul_status_t* status, uint64_t* timeline, uint64_t timeout_ns, FrontPart* out) {
  if (!ln_w || !w_packed || !ab_peers || !gate_out) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "ln_gated_proj: NULL pointer");
  const int D = geom->d;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(D), static_cast<uint64_t>(5 * D)};
    const uint64_t strides[1] = {static_cast<uint64_t>(D) * 2};
    const uint32_t box[2] = {64, static_cast<uint32_t>(D <= 256 ? D : 128)};  // wide rows: 128-row boxes
    int rc = make_tmap(&out->tmW, w_packed, 2, dims, strides, box);
    if (rc != TRIMUL_OK) return rc;
  }
  trimul::GatedProjArgs& a = out->args;
  memset(&a, 0, sizeof(a));
  a.ln_w = ln_w;
  a.ln_b = ln_b;
  a.bias = bias_packed;
  a.has_bias = bias_packed != nullptr ? 1 : 0;
  a.eps = geom->eps;
  a.D = D;
  a.batch = geom->batch;
  if (geom->direction == TRIMUL_OUTGOING && geom->cp1 == 1 && static_cast<long>(d.ni_loc) * d.nj_loc > 0x7fffffffL)
    return fail(TRIMUL_ERR_UNSUPPORTED_SHAPE, "local token block too large");
  trimul_reshard_plan_t plan;
  derive_plan(geom, d, &plan);
  a.batch_rows = plan.batch_rows;
  a.n_lines = plan.n_lines;
  a.n_walk = plan.n_walk;
  a.line_rows = plan.line_rows;
  a.walk_rows = plan.walk_rows;
  a.dst_base = plan.dst_base;
  a.dst_line = plan.dst_line;
  for (int s = 0; s < d.cp; ++s) {
    if (ab_peers[s] == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "ab_peers[%d] is NULL", s);
    a.ab.ptr[s] = ab_peers[s];
  }
  a.d_loc = d.d_loc;
  a.store_ch = (d.d_loc % 64 == 0) ? 64 : ((d.d_loc % 32 == 0) ? 32 : 16);
  a.plane_elems = plan.plane_elems;
  a.gate_out = gate_out;
  if (static_cast<long>(geom->n) * geom->n > 0x7fffffffL)
    return fail(TRIMUL_ERR_UNSUPPORTED_SHAPE, "n=%d: a plane must hold fewer than 2^31 tokens", geom->n);
  memset(&out->maps, 0, sizeof(out->maps));
  {
    // Store maps.  a|b: every owner's operand buffer as (x, y, batch, 2*D_loc planes); x is clipped
    // at the end of this rank's walk so a ragged tile cannot reach a neighbour's tokens.  Boxes are
    // 64 tokens x store_ch channel planes with the 128-byte swizzle (the layout stmatrix fills).
    const uint64_t n = static_cast<uint64_t>(geom->n);
    const bool flat = plan.dst_line == 0;  // whole block contiguous: one line, x runs over the plane
    a.dst_x0 = static_cast<int>(flat ? plan.dst_base : plan.dst_base % plan.dst_line);
    a.dst_y0 = static_cast<int>(flat ? 0 : plan.dst_base / plan.dst_line);
    const uint64_t dims[4] = {static_cast<uint64_t>(a.dst_x0) + static_cast<uint64_t>(plan.n_walk), flat ? 1 : n,
                              static_cast<uint64_t>(geom->batch), static_cast<uint64_t>(2 * d.d_loc)};
    const uint64_t strides[3] = {flat ? n * n * 2 : n * 2, n * n * 2, n * n * 2 * geom->batch};
    const uint32_t box[4] = {64, 1, 1, static_cast<uint32_t>(a.store_ch)};
    for (int s = 0; s < d.cp; ++s) {
      int rc = make_tmap(&out->maps.ab[s], ab_peers[s], 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc != TRIMUL_OK) return rc;
    }
    // gate: local (rows, D) buffer as (D, walk | line, line | walk, batch), the smaller row stride first
    const uint64_t row_b = static_cast<uint64_t>(D) * 2;
    const uint64_t line_stride =
        (plan.n_lines > 1 ? static_cast<uint64_t>(plan.line_rows) : static_cast<uint64_t>(plan.batch_rows)) * row_b;
    const uint64_t walk_stride = static_cast<uint64_t>(plan.walk_rows) * row_b;
    const uint64_t batch_stride = static_cast<uint64_t>(plan.batch_rows) * row_b;
    const bool walk_first = walk_stride <= line_stride;
    a.gate_walk_dim = walk_first ? 1 : 2;
    const uint64_t gdims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(walk_first ? plan.n_walk : plan.n_lines),
                               static_cast<uint64_t>(walk_first ? plan.n_lines : plan.n_walk),
                               static_cast<uint64_t>(geom->batch)};
    const uint64_t gstr[3] = {walk_first ? walk_stride : line_stride, walk_first ? line_stride : walk_stride, batch_stride};
    const uint32_t gbox[4] = {64, walk_first ? 128u : 1u, walk_first ? 1u : 128u, 1};
    int rc = make_tmap(&out->maps.gate, gate_out, 4, gdims, gstr, gbox, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TRIMUL_OK) return rc;
  }
  a.rotate_chunks = (tuning != nullptr && tuning->front_fixed_order) ? 0 : 1;
  a.timeline = reinterpret_cast<unsigned long long*>(timeline);
  a.status = reinterpret_cast<trimul::DeviceStatus*>(status);
  a.timeout_ns = timeout_ns ? timeout_ns : kDefaultTimeoutNs;
  return TRIMUL_OK;
}

int launch_front(FrontPart& part, const void* x, const void* mask, int32_t mask_kind, int num_sms, cudaStream_t stream) {
  if (x == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "ln_gated_proj: x is NULL");
  if (mask_kind < 0 || mask_kind > 3 || (mask_kind != 0 && mask == nullptr))
    return fail(TRIMUL_ERR_INVALID_ARGUMENT, "ln_gated_proj: bad mask_kind %d", mask_kind);
  part.args.x = x;
  part.args.mask = mask_kind ? mask : nullptr;
  part.args.mask_kind = mask_kind;
  cudaError_t e = trimul::launch_gated_proj(part.tmW, part.maps, part.args, num_sms, stream);
  if (e != cudaSuccess) return cuda_fail(e, "ln_gated_proj launch");
  return TRIMUL_OK;
}

// Tile rows per band of the contraction's tile walk when the caller leaves the choice to the library.
// Measured at n = 4096, 256 planes (one-pass DRAM counters of a whole launch): the row-major walk reads
// 86.9 GB, bands of 4 / 8 / 16 rows 61.8 / 58.8 / 63.2 GB (first touch is 17.2 GB); the kernel's time is the
// same within the run-to-run spread, so the choice is the one that moves the fewest bytes.
constexpr int kDefaultBandRows = 8;
// Longest wait of a CTA pair for the other pairs before a tile.  Alternating bounds inside full forwards in one
// process at n = 8192, 128 planes (a tile streams 8 MB; unpaced, the pairs' re-reads can ask more of DRAM than it
// has): unpaced 138-145 ms, 2 us 120 ms (single forwards 97-141), 5 us 106, 20 us 102 (97-110), 60 us 104; runs of
// one bound per process on other devices read 99-106 ms with and without pacing.  n = 4096, 256 planes: unpaced
// 25.3 ms, 2 / 5 / 20 us 25.6 / 25.6 / 24.8; DRAM reads 58.8 GB unpaced, 48.1 GB paced.  A bound of a few us pulls
// a pair that has drifted back by only that much per tile; 20 us re-locks it at once.
constexpr int kDefaultPaceNs = 20000;

// How the contraction walks a plane's tiles, from the tuning record: band height, where the walk starts, pacing.
int derive_walk(const Derived& d, const trimul_tuning_t* tuning, trimul::TriContractArgs* a) {
  const int band = tuning != nullptr ? tuning->contract_band_rows : 0;
  if (band < 0) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "tuning.contract_band_rows=%d must be >= 0", band);
  a->band_rows = band > 0 ? band : kDefaultBandRows;
  const int pace = tuning != nullptr ? tuning->contract_pace_ns : 0;
  if (pace > 100000) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "tuning.contract_pace_ns=%d must be <= 100000", pace);
  a->pace_ns = pace < 0 ? 0u : static_cast<unsigned int>(pace > 0 ? pace : kDefaultPaceNs);
  // every rank starts its walk at the block of the result it owns itself and all ranks advance alike, so at any
  // moment the ranks' stores go to different owners (a rotation of the ranks) instead of all to the same one
  const bool fixed_start = tuning != nullptr && tuning->contract_fixed_start != 0;
  a->rot_rows = fixed_start ? 0 : static_cast<int>(d.i_off);
  a->rot_cols = fixed_start ? 0 : static_cast<int>(d.j_off);
  return TRIMUL_OK;
}

int build_contract(const trimul_geom_t* geom, const Derived& d, const trimul_tuning_t* tuning, const void* ab_local,
                   void* const* tri_peers, trimul_status_t* status, uint64_t* timeline, uint64_t timeout_ns, int num_sms,
                   ContractPart* out) {
  if (!ab_local || !tri_peers) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "tri_contract: NULL pointer");
  const int form = tuning != nullptr ? tuning->contract_form : TRIMUL_CONTRACT_DEFAULT;
  if (form < TRIMUL_CONTRACT_DEFAULT || form > TRIMUL_CONTRACT_PAIR)
    return fail(TRIMUL_ERR_INVALID_ARGUMENT, "tuning.contract_form=%d is not one of TRIMUL_CONTRACT_*", form);
  // default: CTA pairs (256 x 256 tiles over two SMs) -- faster than 128 x 256 single-CTA tiles at
  // every shape measured -- unless the device has a single SM
  out->pair = form == TRIMUL_CONTRACT_PAIR || (form == TRIMUL_CONTRACT_DEFAULT && num_sms >= 2);
  if (out->pair && num_sms < 2) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "the CTA-pair contraction needs two SMs");
  const uint64_t n = static_cast<uint64_t>(geom->n);
  const uint64_t planes = static_cast<uint64_t>(d.d_loc) * geom->batch;
  {
    // A: 128-row boxes; B: 256-row boxes for the single-CTA form, two 128-row halves for a pair
    const uint64_t dims[3] = {n, n, planes};
    const uint64_t strides[2] = {n * 2, n * n * 2};
    const uint32_t boxA[3] = {64, 128, 1};
    const uint32_t boxB[3] = {64, out->pair ? 128u : 256u, 1};
    int rc = make_tmap(&out->tmA, ab_local, 3, dims, strides, boxA);
    if (rc != TRIMUL_OK) return rc;
    const uint8_t* b_base = static_cast<const uint8_t*>(ab_local) + planes * n * n * 2;
    rc = make_tmap(&out->tmB, b_base, 3, dims, strides, boxB);
    if (rc != TRIMUL_OK) return rc;
  }
  trimul::TriContractArgs& a = out->args;
  memset(&a, 0, sizeof(a));
  a.planes = static_cast<int>(planes);
  a.batch = geom->batch;
  a.n_i = a.n_j = a.n_k = geom->n;
  for (int s = 0; s < d.cp; ++s) {
    if (tri_peers[s] == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "tri_peers[%d] is NULL", s);
    a.out.ptr[s] = tri_peers[s];
  }
  a.ni_loc = d.ni_loc;
  a.nj_loc = d.nj_loc;
  a.cp1 = geom->cp1;
  a.chan_offset = geom->rank * d.d_loc;
  {
    int rc = derive_walk(d, tuning, &a);
    if (rc != TRIMUL_OK) return rc;
  }
  memset(&out->maps, 0, sizeof(out->maps));
  {
    // every owner's tri buffer as (columns, rows, channel planes of ALL D channels x batch)
    const uint64_t odims[3] = {static_cast<uint64_t>(d.nj_loc), static_cast<uint64_t>(d.ni_loc),
                               static_cast<uint64_t>(geom->d) * geom->batch};
    const uint64_t ostr[2] = {static_cast<uint64_t>(d.nj_loc) * 2, static_cast<uint64_t>(d.nj_loc) * d.ni_loc * 2};
    const uint32_t obox[3] = {64, 32, 1};
    for (int s = 0; s < d.cp; ++s) {
      int rc = make_tmap(&out->maps.map[s], tri_peers[s], 3, odims, ostr, obox);
      if (rc != TRIMUL_OK) return rc;
    }
  }
  a.timeline = reinterpret_cast<unsigned long long*>(timeline);
  a.status = reinterpret_cast<trimul::DeviceStatus*>(status);
  a.timeout_ns = timeout_ns ? timeout_ns : kDefaultTimeoutNs;
  return TRIMUL_OK;
}

int launch_contract(const ContractPart& part, int num_sms, cudaStream_t stream) {
  cudaError_t e = part.pair ? trimul::launch_tri_contract_pair(part.tmA, part.tmB, part.maps, part.args, num_sms, stream)
                            : trimul::launch_tri_contract(part.tmA, part.tmB, part.maps, part.args, num_sms, stream);
  if (e != cudaSuccess) return cuda_fail(e, "tri_contract launch");
  return TRIMUL_OK;
}

int encode_out_map(CUtensorMap* map, const void* base, int D, long rows) {
  // gate and out, token-major (rows, D): boxes of 64 channels x 128 tokens (128-byte rows)
  const uint64_t dims[2] = {static_cast<uint64_t>(D), static_cast<uint64_t>(rows)};
  const uint64_t strides[1] = {static_cast<uint64_t>(D) * 2};
  const uint32_t box[2] = {64, 128};
  return make_tmap(map, base, 2, dims, strides, box);
}

int build_out(const trimul_geom_t* geom, const Derived& d, const void* tri_local, const void* gate, const void* w_fold,
              const float* cd, trimul_status_t* status, uint64_t* timeline, uint64_t timeout_ns, OutPart* out) {
  if (!tri_local || !gate || !w_fold || !cd) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "ln_out_proj: NULL pointer");
  const int D = geom->d;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(D), static_cast<uint64_t>(D)};
    const uint64_t strides[1] = {static_cast<uint64_t>(D) * 2};
    const uint32_t box[2] = {64, static_cast<uint32_t>(D <= 256 ? D : 128)};  // wide rows: 128-row boxes
    int rc = make_tmap(&out->tmW, w_fold, 2, dims, strides, box);
    if (rc != TRIMUL_OK) return rc;
  }
  {
    // tri as (tokens contiguous, channels): the tile is consumed token-major exactly as stored
    const uint64_t dims[2] = {static_cast<uint64_t>(d.rows), static_cast<uint64_t>(D)};
    const uint64_t strides[1] = {static_cast<uint64_t>(d.rows) * 2};
    const uint32_t box[2] = {64, 64};
    int rc = make_tmap(&out->tmT, tri_local, 2, dims, strides, box);
    if (rc != TRIMUL_OK) return rc;
  }
  int rc = encode_out_map(&out->tmG, gate, D, d.rows);
  if (rc != TRIMUL_OK) return rc;
  out->tmO_for = nullptr;
  trimul::OutProjArgs& a = out->args;
  memset(&a, 0, sizeof(a));
  a.gate = gate;
  a.cd = cd;
  a.eps = geom->eps;
  a.D = D;
  a.rows = d.rows;
  a.timeline = reinterpret_cast<unsigned long long*>(timeline);
  a.status = reinterpret_cast<trimul::DeviceStatus*>(status);
  a.timeout_ns = timeout_ns ? timeout_ns : kDefaultTimeoutNs;
  return TRIMUL_OK;
}

int launch_out(OutPart& part, void* out, int num_sms, cudaStream_t stream) {
  if (out == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "ln_out_proj: out is NULL");
  if (part.tmO_for != out) {  // a caller that reuses its output buffer pays for this once
    int rc = encode_out_map(&part.tmO, out, part.args.D, part.args.rows);
    if (rc != TRIMUL_OK) return rc;
    part.tmO_for = out;
  }
  part.args.out = out;
  cudaError_t e = trimul::launch_out_proj(part.tmW, part.tmT, part.tmG, part.tmO, part.args, num_sms, stream);
  if (e != cudaSuccess) return cuda_fail(e, "ln_out_proj launch");
  return TRIMUL_OK;
}

}  // namespace

// The opaque plan of the C ABI: one rank's three launches for a fixed geometry and set of buffers.
struct trimul_plan {
  int device;
  int num_sms;
  FrontPart front;
  ContractPart contract;
  OutPart out;
};

namespace trimul {
// Lets other translation units of the library leave a message in the slot trimul_sm100_last_error reads.
void set_last_error(const char* msg) { fail(0, "%s", msg); }
}  // namespace trimul

extern "C" {

const char* trimul_sm100_last_error(void) { return g_err; }

#ifndef TRIMUL_BUILD_ID
#define TRIMUL_BUILD_ID "unknown"
#endif
const char* trimul_sm100_build_id(void) { return TRIMUL_BUILD_ID; }

int trimul_sm100_query(int device, trimul_caps_t* out) {
  if (out == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "caps is NULL");
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->num_sms = prop.multiProcessorCount;
  out->max_smem_per_block = static_cast<int32_t>(prop.sharedMemPerBlockOptin);
  out->supported = (prop.major == 10) ? 1 : 0;
  if (!out->supported)
    return fail(TRIMUL_ERR_UNSUPPORTED_ARCH,
                "fold-cp-ops (B200 build) requires SM100 (B200); got sm_%d%d. No other architecture has a code path.",
                prop.major, prop.minor);
  return TRIMUL_OK;
}

int trimul_sm100_workspace(const trimul_geom_t* geom, trimul_workspace_t* out) {
  Derived d;
  int rc = check_geom(geom, &d);
  if (rc != TRIMUL_OK) return rc;
  if (out == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "workspace is NULL");
  const uint64_t nn = static_cast<uint64_t>(geom->n) * geom->n;
  out->ab_bytes = 2ull * d.d_loc * geom->batch * nn * 2ull;
  out->tri_bytes = static_cast<uint64_t>(geom->d) * d.rows * 2ull;
  out->gate_bytes = static_cast<uint64_t>(d.rows) * geom->d * 2ull;
  return TRIMUL_OK;
}

int trimul_sm100_reshard_plan(const trimul_geom_t* geom, trimul_reshard_plan_t* out) {
  Derived d;
  int rc = check_geom(geom, &d);
  if (rc != TRIMUL_OK) return rc;
  if (out == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "plan is NULL");
  derive_plan(geom, d, out);
  return TRIMUL_OK;
}

int trimul_sm100_contract_walk(const trimul_geom_t* geom, const trimul_tuning_t* tuning, int32_t capacity,
                               int32_t* tile_row, int32_t* tile_col, int32_t* tiles_i, int32_t* tiles_j) {
  Derived d;
  int rc = check_geom(geom, &d);
  if (rc != TRIMUL_OK) return rc;
  if (!tiles_i || !tiles_j || capacity < 0 || (capacity > 0 && (!tile_row || !tile_col)))
    return fail(TRIMUL_ERR_INVALID_ARGUMENT, "contract_walk: NULL output or negative capacity");
  const int form = tuning != nullptr ? tuning->contract_form : TRIMUL_CONTRACT_DEFAULT;
  if (form < TRIMUL_CONTRACT_DEFAULT || form > TRIMUL_CONTRACT_PAIR)
    return fail(TRIMUL_ERR_INVALID_ARGUMENT, "tuning.contract_form=%d is not one of TRIMUL_CONTRACT_*", form);
  trimul::TriContractArgs a;
  memset(&a, 0, sizeof(a));
  a.n_i = a.n_j = a.n_k = geom->n;
  rc = derive_walk(d, tuning, &a);
  if (rc != TRIMUL_OK) return rc;
  int ti = 0, tj = 0;
  if (form == TRIMUL_CONTRACT_SINGLE) {
    trimul::tri_contract_walk(a, capacity, tile_row, tile_col, &ti, &tj);
  } else {
    trimul::tri_contract_pair_walk(a, capacity, tile_row, tile_col, &ti, &tj);
  }
  *tiles_i = ti;
  *tiles_j = tj;
  return TRIMUL_OK;
}

int trimul_sm100_pack_weights(int32_t d, const void* p_in_w, const void* g_in_w, const void* g_out_w,
                              const float* p_in_b, const float* g_in_b, const float* g_out_b, void* w_packed,
                              float* bias_packed, trimul_stream_t stream) {
  if (d != 128 && d != 256 && d != 384 && d != 512) return fail(TRIMUL_ERR_UNSUPPORTED_SHAPE, "feature width d=%d is not supported", d);
  if (!p_in_w || !g_in_w || !g_out_w || !w_packed || !bias_packed)
    return fail(TRIMUL_ERR_INVALID_ARGUMENT, "pack_weights: NULL weight pointer");
  pack_weights_kernel<<<5 * d, 128, 0, stream>>>(
      d, static_cast<const __nv_bfloat16*>(p_in_w), static_cast<const __nv_bfloat16*>(g_in_w),
      static_cast<const __nv_bfloat16*>(g_out_w), p_in_b, g_in_b, g_out_b, static_cast<__nv_bfloat16*>(w_packed),
      bias_packed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "pack_weights launch");
  return TRIMUL_OK;
}

int trimul_sm100_pack_out_weights(int32_t d, const void* w_out, const float* ln_w, const float* ln_b,
                                  const float* bias_out, void* w_fold, float* cd, trimul_stream_t stream) {
  if (d != 128 && d != 256 && d != 384 && d != 512) return fail(TRIMUL_ERR_UNSUPPORTED_SHAPE, "feature width d=%d is not supported", d);
  if (!w_out || !ln_w || !w_fold || !cd) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "pack_out_weights: NULL pointer");
  pack_out_weights_kernel<<<d, 128, 0, stream>>>(d, static_cast<const __nv_bfloat16*>(w_out), ln_w, ln_b, bias_out,
                                                 static_cast<__nv_bfloat16*>(w_fold), cd);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "pack_out_weights launch");
  return TRIMUL_OK;
}

int trimul_sm100_ln_gated_proj(const trimul_geom_t* geom, const trimul_tuning_t* tuning, const void* x, const void* mask,
                               int32_t mask_kind, const float* ln_w, const float* ln_b, const void* w_packed,
                               const float* bias_packed, void* const* ab_peers, void* gate_out,
                               trimul_status_t* status, uint64_t timeout_ns, trimul_stream_t stream) {
  Derived d;
  int rc = check_geom(geom, &d);
  if (rc != TRIMUL_OK) return rc;
  FrontPart part;
  rc = build_front(geom, d, tuning, ln_w, ln_b, w_packed, bias_packed, ab_peers, gate_out, status, nullptr, timeout_ns,
                   &part);
  if (rc != TRIMUL_OK) return rc;
  return launch_front(part, x, mask, mask_kind, num_sms_current(), stream);
}

int trimul_sm100_tri_contract(const trimul_geom_t* geom, const trimul_tuning_t* tuning, const void* ab_local,
                              void* const* tri_peers, trimul_status_t* status, uint64_t timeout_ns,
                              trimul_stream_t stream) {
  Derived d;
  int rc = check_geom(geom, &d);
  if (rc != TRIMUL_OK) return rc;
  ContractPart part;
  rc = build_contract(geom, d, tuning, ab_local, tri_peers, status, nullptr, timeout_ns, num_sms_current(), &part);
  if (rc != TRIMUL_OK) return rc;
  return launch_contract(part, num_sms_current(), stream);
}

int trimul_sm100_ln_out_proj(const trimul_geom_t* geom, const void* tri_local, const void* gate, const void* w_fold,
                             const float* cd, void* out, trimul_status_t* status, uint64_t timeout_ns,
                             trimul_stream_t stream) {
  Derived d;
  int rc = check_geom(geom, &d);
  if (rc != TRIMUL_OK) return rc;
  OutPart part;
  rc = build_out(geom, d, tri_local, gate, w_fold, cd, status, nullptr, timeout_ns, &part);
  if (rc != TRIMUL_OK) return rc;
  return launch_out(part, out, num_sms_current(), stream);
}

int trimul_sm100_forward(const trimul_geom_t* geom, const void* x, const void* mask, int32_t mask_kind,
                         const float* ln_in_w, const float* ln_in_b, const void* w_packed,
                         const float* bias_packed, const void* w_fold, const float* cd, void* ab, void* tri,
                         void* gate, void* out, trimul_status_t* status, uint64_t timeout_ns,
                         trimul_stream_t stream) {
  if (geom == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "geom is NULL");
  if (geom->cp0 != 1 || geom->cp1 != 1)
    return fail(TRIMUL_ERR_INVALID_ARGUMENT, "trimul_sm100_forward is the single-GPU chain; cp grid must be 1 x 1");
  void* ab_peers[1] = {ab};
  void* tri_peers[1] = {tri};
  int rc = trimul_sm100_ln_gated_proj(geom, nullptr, x, mask, mask_kind, ln_in_w, ln_in_b, w_packed, bias_packed,
                                      ab_peers, gate, status, timeout_ns, stream);
  if (rc != TRIMUL_OK) return rc;
  rc = trimul_sm100_tri_contract(geom, nullptr, ab, tri_peers, status, timeout_ns, stream);
  if (rc != TRIMUL_OK) return rc;
  return trimul_sm100_ln_out_proj(geom, tri, gate, w_fold, cd, out, status, timeout_ns, stream);
}

// ---------------------------------------------------------------------------------------------
// plans: the three launches of one (geometry, buffers) binding with every descriptor encoded once
// ---------------------------------------------------------------------------------------------
int trimul_sm100_plan_create(const trimul_plan_desc_t* desc, trimul_plan_t** out) {
  if (desc == nullptr || out == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "plan_create: NULL argument");
  *out = nullptr;
  Derived d;
  int rc = check_geom(&desc->geom, &d);
  if (rc != TRIMUL_OK) return rc;
  const int sms = num_sms_current();
  if (sms <= 0) return fail(TRIMUL_ERR_CUDA, "plan_create: cannot query the current device");
  trimul_plan* pl = new (std::nothrow) trimul_plan;
  if (pl == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "plan_create: out of host memory");
  pl->num_sms = sms;
  cudaGetDevice(&pl->device);
  void* const* abp = desc->ab_peers;
  void* const* trp = desc->tri_peers;
  rc = build_front(&desc->geom, d, &desc->tuning, desc->ln_in_w, desc->ln_in_b, desc->w_packed, desc->bias_packed, abp,
                   desc->gate, desc->status, desc->timeline, desc->timeout_ns, &pl->front);
  if (rc == TRIMUL_OK)
    rc = build_contract(&desc->geom, d, &desc->tuning, desc->ab_peers[desc->geom.rank], trp, desc->status, desc->timeline,
                        desc->timeout_ns, sms, &pl->contract);
  if (rc == TRIMUL_OK)
    rc = build_out(&desc->geom, d, desc->tri_peers[desc->geom.rank], desc->gate, desc->w_fold, desc->cd, desc->status,
                   desc->timeline, desc->timeout_ns, &pl->out);
  if (rc != TRIMUL_OK) {
    delete pl;
    return rc;
  }
  *out = pl;
  return TRIMUL_OK;
}

int trimul_sm100_plan_ln_gated_proj(trimul_plan_t* plan, const void* x, const void* mask, int32_t mask_kind,
                                    trimul_stream_t stream) {
  if (plan == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "plan is NULL");
  return launch_front(plan->front, x, mask, mask_kind, plan->num_sms, stream);
}

int trimul_sm100_plan_tri_contract(trimul_plan_t* plan, trimul_stream_t stream) {
  if (plan == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "plan is NULL");
  return launch_contract(plan->contract, plan->num_sms, stream);
}

int trimul_sm100_plan_ln_out_proj(trimul_plan_t* plan, void* out, trimul_stream_t stream) {
  if (plan == nullptr) return fail(TRIMUL_ERR_INVALID_ARGUMENT, "plan is NULL");
  return launch_out(plan->out, out, plan->num_sms, stream);
}

void trimul_sm100_plan_destroy(trimul_plan_t* plan) { delete plan; }

}  // extern "C"
