/*
 * trimul_sm100.h -- C ABI of libtrimul_sm100.so: the Blackwell (sm_100a) kernels behind the
 * context-parallel triangle multiplicative update ("TriMul") forward.
 *
 * The reference package (NVIDIA-BioNeMo/fold-cp-ops) has no native code: its kernels are CuTe-DSL
 * Python objects JIT-compiled for SM90 and launched from Python.  Each entry point below names the
 * reference Python interface whose job it takes over (path inside the reference project : line).
 *
 * Conventions
 *   - every function returns 0 on success or a negative TRIMUL_ERR_* code; nothing throws or exits;
 *   - every pointer is caller-owned DEVICE memory unless stated otherwise; no device memory is
 *     allocated or freed here (a plan is a small HOST object) and there are no hidden streams: work
 *     is enqueued on the stream that is passed;
 *   - all activations and weights are bf16, LayerNorm gains/biases and projection biases are fp32;
 *   - device-side waits are bounded: on expiry a kernel writes a trimul_status_t record and returns
 *     normally, so the CUDA context stays usable.  The caller owns the status record (8 x int32,
 *     zero it once) and reads it after synchronising the stream.
 */
#ifndef TRIMUL_SM100_H_
#define TRIMUL_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRIMUL_OK 0
#define TRIMUL_ERR_INVALID_ARGUMENT (-1)
#define TRIMUL_ERR_UNSUPPORTED_ARCH (-2)
#define TRIMUL_ERR_CUDA (-3)
#define TRIMUL_ERR_UNSUPPORTED_SHAPE (-4)

#define TRIMUL_MAX_PEERS 8

#define TRIMUL_MASK_NONE 0
#define TRIMUL_MASK_BF16 1
#define TRIMUL_MASK_FP32 2
#define TRIMUL_MASK_U8 3

#define TRIMUL_OUTGOING 0
#define TRIMUL_INCOMING 1

typedef struct CUstream_st* trimul_stream_t;

/* Device capabilities.  Mirrors the architecture gate of fold_cp_ops/_internal/arch.py:145-170
 * (`check_arch_supported`), inverted: this library needs compute capability 10.x. */
typedef struct trimul_caps {
  int32_t cc_major;
  int32_t cc_minor;
  int32_t num_sms;
  int32_t max_smem_per_block;
  int32_t supported; /* 1 when the kernels can run on this device */
} trimul_caps_t;

/* Geometry of one forward on one rank.  The global pair tensor is (batch, n, n, d), d in {128, 256, 384,
 * 512} (other widths: TRIMUL_ERR_UNSUPPORTED_SHAPE); the token grid
 * is split cp0 x cp1 (rows x columns) and this rank is flat cp rank `rank` = r0 * cp1 + r1, the
 * row-major peer order of fold_cp_ops/distributed/pe_map.py:265-283.  cp0 = cp1 = 1 is the
 * single-GPU case. */
typedef struct trimul_geom {
  int32_t batch;
  int32_t n;
  int32_t d;
  int32_t cp0;
  int32_t cp1;
  int32_t rank;
  int32_t direction; /* TRIMUL_OUTGOING | TRIMUL_INCOMING */
  float eps;
} trimul_geom_t;

/* Record a kernel leaves behind when a bounded wait expires. */
typedef struct trimul_status {
  int32_t code;   /* 0 = OK, 1 = a bounded wait expired */
  int32_t kernel; /* 1 gated projection, 2 contraction, 3 output projection, 4 peer sync */
  int32_t block;
  int32_t role;
  int32_t detail;
  int32_t pad[3];
} trimul_status_t;

/* Choices the sm_100a kernels leave open (0 in every field = the library's default).  Takes over the
 * typed knobs of `TriMulTuning` (fold_cp_ops/distributed/workflows/trimul_tuning.py:72-217), whose SM90
 * tile / cluster / drain settings have no meaning here. */
#define TRIMUL_CONTRACT_DEFAULT 0 /* CTA pairs when the device has at least two SMs */
#define TRIMUL_CONTRACT_SINGLE 1  /* one CTA per 128 x 256 output tile (tcgen05 cta_group::1) */
#define TRIMUL_CONTRACT_PAIR 2    /* two CTAs per 256 x 256 output tile (tcgen05 cta_group::2) */
typedef struct trimul_tuning {
  int32_t contract_form;     /* TRIMUL_CONTRACT_* */
  int32_t front_fixed_order; /* 1: every CTA of the projection kernel walks the gated chunks in the same
                                order; 0: CTAs start at different chunks so that, at cp > 1, the grid's
                                stores reach all owner ranks at any moment */
  int32_t contract_band_rows; /* tile rows per band of the contraction kernel's tile walk: inside a band
                                 the walk is column by column, so one wave of CTAs streams about as many A
                                 row strips as B row strips through L2.  0: the library's choice; 1: row-major */
  int32_t contract_fixed_start; /* 1: every rank walks the contraction's tiles from tile (0, 0); 0: each rank
                                   starts at the block of the result it owns, so that at cp > 1 the ranks' stores
                                   go to different owners at any moment */
  int32_t contract_pace_ns;     /* CTA-pair contraction: before each tile a pair waits at most this long (ns,
                                   <= 100000) for the other pairs to start theirs, so that tiles that share
                                   operand strips move through K together and share them in L2.  A hint only:
                                   no result and no termination depends on it.  0: the library's choice (20000);
                                   negative: off */
  int32_t reserved[3];
} trimul_tuning_t;

/* Optional device timeline of one forward: TRIMUL_TIMELINE_SLOTS x uint64 of %globaltimer (ns) on this
 * rank.  "first" slots are reduced with min over a kernel's CTAs -- preset them to UINT64_MAX -- and
 * "last" slots with max -- preset 0; a flag wait writes its entry and exit time.  Time spent in the
 * waits (exit - entry) is the all-to-all time this rank did NOT hide behind a kernel. */
#define TRIMUL_TIMELINE_SLOTS 16
#define TRIMUL_TL_FRONT_START 0        /* first: projection kernel running */
#define TRIMUL_TL_FRONT_FIRST_STORE 1  /* first: first a|b store issued */
#define TRIMUL_TL_FRONT_LAST_STORE 2   /* last: every store of the projection kernel performed */
#define TRIMUL_TL_CONTRACT_START 3     /* first */
#define TRIMUL_TL_CONTRACT_LAST_STORE 4 /* last */
#define TRIMUL_TL_OUT_START 5          /* first */
#define TRIMUL_TL_OUT_END 6            /* last */
#define TRIMUL_TL_WAIT_BASE 8          /* + 2 * flag slot: wait entry; + 1: wait exit (flag slots 0..2) */

/* Bytes of each buffer a rank needs for `geom` (all bf16):
 *   ab   : operand planes this rank contracts, (2, d/cp, batch, n, n)   -- written by every rank
 *   tri  : contraction result for this rank's tokens, (d, batch, n/cp0, n/cp1) -- written by every rank
 *   gate : output gate for this rank's tokens, (batch, n/cp0, n/cp1, d)  -- local only
 * Replaces the receive-buffer sizing of `ReshardLayout` (fold_cp_ops/distributed/reshard.py:63-289)
 * and `_symmetric_empty` (fold_cp_ops/distributed/workflows/trimul_autotuned.py:150). */
typedef struct trimul_workspace {
  uint64_t ab_bytes;
  uint64_t tri_bytes;
  uint64_t gate_bytes;
} trimul_workspace_t;

/* Index arithmetic of the two fused reshards for one rank (host-only; touches no device).
 * Front: local token (b, line, w) is row  b*batch_rows + line*line_rows + w*walk_rows  of x and lands
 * at element  ((h*d_loc + c)*batch + b)*plane_elems + dst_base + line*dst_line + w  of the `ab` buffer
 * of the rank owning channel h*d + s*d_loc + c (h = 0 for a, 1 for b; s = owner).  Back: element
 * (c, b, i, j) of this rank's contraction lands at  ((chan_offset + c)*batch + b)*ni_loc*nj_loc +
 * (i % ni_loc)*nj_loc + (j % nj_loc)  of the `tri` buffer of rank (i / ni_loc)*cp1 + (j / nj_loc).
 * Replaces the wire-layout description `ReshardLayout` (fold_cp_ops/distributed/reshard.py:63-377). */
typedef struct trimul_reshard_plan {
  int32_t n_lines;
  int32_t n_walk;
  int64_t batch_rows;
  int64_t line_rows;
  int64_t walk_rows;
  int64_t plane_elems;
  int64_t dst_base;
  int64_t dst_line;
  int32_t d_loc;
  int32_t planes;
  int32_t ni_loc;
  int32_t nj_loc;
  int32_t chan_offset;
  int32_t pad;
  int64_t rows;
} trimul_reshard_plan_t;

int trimul_sm100_query(int device, trimul_caps_t* out);
int trimul_sm100_reshard_plan(const trimul_geom_t* geom, trimul_reshard_plan_t* out);
int trimul_sm100_workspace(const trimul_geom_t* geom, trimul_workspace_t* out);
/* Host-only: the order in which the contraction kernel visits the tiles of one channel plane for this rank and
 * tuning (tuning->contract_form picks the tile height: 256 rows for CTA pairs -- also the default -- 128 for the
 * single-CTA form; tiles are 256 columns wide).  Writes the grid size to tiles_i / tiles_j and, for the first
 * min(capacity, tiles_i*tiles_j) positions r of the walk, the tile's row and column index to tile_row[r] /
 * tile_col[r].  Evaluates the same function the kernels call; touches no device.  Takes over what the reference
 * leaves to its persistent tile scheduler (fold_cp_ops/distributed/gemm_a2a_epi.py:78). */
int trimul_sm100_contract_walk(const trimul_geom_t* geom, const trimul_tuning_t* tuning /* nullable */, int32_t capacity,
                               int32_t* tile_row, int32_t* tile_col, int32_t* tiles_i, int32_t* tiles_j);
const char* trimul_sm100_last_error(void);
/* Digest of the sources this library was compiled from (set by the build script; "unknown" for a hand
 * build).  The Python loader compares it with the sources beside the library and refuses a stale one.
 * No counterpart in the reference, whose kernels are JIT-compiled from the installed sources. */
const char* trimul_sm100_build_id(void);

/* Pack the input-side weights once at construction: rows of p_in / g_in / g_out (each row-major
 * (out, in), bf16) are regrouped into 4d/256 gated chunks of 256 rows (128 projection rows of a --
 * then of b -- followed by the 128 matching gate rows) and the d rows of g_out; biases (fp32, any may
 * be NULL) are packed the same way.  Every packed row and bias is scaled by 1/2 (exact), which lets the kernel evaluate
 * p * sigmoid(g) as (p/2) * tanh(g/2) + p/2.  w_packed: (5d, d) bf16; bias_packed: (5d) fp32.
 * Replaces `interleave_dual_weights` (fold_cp_ops/kernels/dual_gated_gemm.py:958). */
int trimul_sm100_pack_weights(int32_t d, const void* p_in_w, const void* g_in_w, const void* g_out_w,
                              const float* p_in_b, const float* g_in_b, const float* g_out_b, void* w_packed,
                              float* bias_packed, trimul_stream_t stream);

/* Stage 1+2: input LayerNorm fused into the gated dual projection, front reshard fused in the
 * store.  x: this rank's (batch, n/cp0, n/cp1, d) block; mask: one scalar per local token or NULL;
 * ab_peers[s]: base of rank s's `ab` buffer (cp0*cp1 entries; entry `rank` is local memory);
 * gate_out: local `gate` buffer; bias_packed may be NULL when the layer has no projection bias.
 * Replaces `layernorm_fwd` (fold_cp_ops/kernels/layernorm.py:730) + `DualGatedGemmDistStore.run`
 * (fold_cp_ops/distributed/workflows/trimul_autotuned.py:1744) + the g_out half of
 * `layernorm_dual_gated_gemm` (fold_cp_ops/kernels/layernorm_dual_gated_gemm.py:5342). */
int trimul_sm100_ln_gated_proj(const trimul_geom_t* geom, const trimul_tuning_t* tuning /* nullable */, const void* x,
                               const void* mask, int32_t mask_kind, const float* ln_w, const float* ln_b,
                               const void* w_packed, const float* bias_packed, void* const* ab_peers, void* gate_out,
                               trimul_status_t* status, uint64_t timeout_ns, trimul_stream_t stream);

/* Stage 3: per-channel n x n x n contraction of this rank's `ab` planes, back reshard fused in the
 * store.  tri_peers[s]: base of rank s's `tri` buffer.
 * Replaces `GemmA2AStore.run` (fold_cp_ops/distributed/workflows/trimul_autotuned.py:2548) and the
 * cp=1 `_gemm1` (fold_cp_ops/workflows/trimul_autotune.py:805). */
int trimul_sm100_tri_contract(const trimul_geom_t* geom, const trimul_tuning_t* tuning /* nullable */,
                              const void* ab_local, void* const* tri_peers, trimul_status_t* status,
                              uint64_t timeout_ns, trimul_stream_t stream);

/* Fold the output LayerNorm into the output projection once at construction:
 *   w_fold[n,k] = bf16(ln_w[k] * w_out[n,k])            (d, d) bf16
 *   cd[n] = { sum_k w_fold[n,k],  sum_k ln_b[k] * w_out[n,k] + bias_out[n] }   (d, 2) fp32
 * so that LN(x) w_out^T + b = rstd * (x w_fold^T - mean * c) + d.  ln_b and bias_out may be NULL.
 * Replaces `_fold_precompute_kernel` (fold_cp_ops/kernels/layernorm_dual_gated_gemm.py:4617). */
int trimul_sm100_pack_out_weights(int32_t d, const void* w_out, const float* ln_w, const float* ln_b,
                                  const float* bias_out, void* w_fold, float* cd, trimul_stream_t stream);

/* Stage 4: output LayerNorm fused with the output projection, gated.  out: (batch, n/cp0, n/cp1, d).
 * w_fold / cd come from trimul_sm100_pack_out_weights.
 * Replaces `_consume` (fold_cp_ops/distributed/workflows/trimul_autotuned.py:3482-3550). */
int trimul_sm100_ln_out_proj(const trimul_geom_t* geom, const void* tri_local, const void* gate, const void* w_fold,
                             const float* cd, void* out, trimul_status_t* status, uint64_t timeout_ns,
                             trimul_stream_t stream);

/* The whole single-GPU forward (cp0 = cp1 = 1): stages 1-4 back to back on `stream`.
 * Replaces `trimul_autotuned` (fold_cp_ops/workflows/trimul_autotune.py:1531). */
int trimul_sm100_forward(const trimul_geom_t* geom, const void* x, const void* mask, int32_t mask_kind,
                         const float* ln_in_w, const float* ln_in_b, const void* w_packed,
                         const float* bias_packed, const void* w_fold, const float* cd, void* ab, void* tri,
                         void* gate, void* out, trimul_status_t* status, uint64_t timeout_ns,
                         trimul_stream_t stream);

/* A plan binds one geometry to one set of buffers and encodes every TMA descriptor of the three
 * launches once (the stateless entry points above encode cp + 2, cp + 3 and 4 descriptors on every
 * call).  It is a few KB of HOST memory; creating and destroying it touches no device memory.  Make the
 * device the buffers live on current when creating it.  `ab_peers[geom.rank]` / `tri_peers[geom.rank]`
 * are this rank's own buffers; `timeline` may be NULL.  The output descriptor is cached per `out`
 * pointer.  Not thread-safe: one plan, one caller thread at a time.
 * Takes over the construction half of `TriMulAutotuned.__init__` / `_rebind_runtime`
 * (fold_cp_ops/distributed/workflows/trimul_autotuned.py:2686-3244, 3553-3601), where the reference
 * compiles its kernels and builds its per-peer store descriptors. */
typedef struct trimul_plan trimul_plan_t;
typedef struct trimul_plan_desc {
  trimul_geom_t geom;
  trimul_tuning_t tuning;
  const float* ln_in_w;
  const float* ln_in_b; /* nullable */
  const void* w_packed;
  const float* bias_packed; /* nullable */
  const void* w_fold;
  const float* cd;
  void* ab_peers[TRIMUL_MAX_PEERS];
  void* tri_peers[TRIMUL_MAX_PEERS];
  void* gate;
  trimul_status_t* status;
  uint64_t* timeline; /* nullable; TRIMUL_TIMELINE_SLOTS x uint64 on the device */
  uint64_t timeout_ns;
} trimul_plan_desc_t;
int trimul_sm100_plan_create(const trimul_plan_desc_t* desc, trimul_plan_t** out);
int trimul_sm100_plan_ln_gated_proj(trimul_plan_t* plan, const void* x, const void* mask, int32_t mask_kind,
                                    trimul_stream_t stream);
int trimul_sm100_plan_tri_contract(trimul_plan_t* plan, trimul_stream_t stream);
int trimul_sm100_plan_ln_out_proj(trimul_plan_t* plan, void* out, trimul_stream_t stream);
void trimul_sm100_plan_destroy(trimul_plan_t* plan);

/* Single-GPU forward for callers that cannot allocate device memory (no counterpart in the
 * reference, which always allocates its own buffers).  Same arguments as trimul_sm100_forward minus
 * the three scratch buffers: the a|b planes, the contraction result and the gate live in a
 * TRIMUL_STATIC_SCRATCH_BYTES array built into the library, resident on every GPU that loads it.
 * Meant for hosts whose memory pool already owns the whole device, sandboxed plugins that may not call
 * allocation APIs, and latency-critical loops that cannot afford cudaMalloc's device synchronisation.
 * No cudaMalloc / cudaFree / allocating library call is made.  Limits: cp0 = cp1 = 1 and
 * 8 * batch * n * n * d <= TRIMUL_STATIC_SCRATCH_BYTES, otherwise TRIMUL_ERR_UNSUPPORTED_SHAPE with a
 * message in trimul_sm100_last_error().  All calls on a device share the one array: calls that overlap on
 * the GPU race.  The array keeps the previous call's contents; the forward overwrites everything it
 * reads, so nothing is cleared.  The first call on a device looks up the array's device address (with
 * that device current: the device that owns `stream` must be the current one) -- make it outside any
 * stream capture.  The address is cached per device for the life of the process; a cudaDeviceReset
 * invalidates it, after which this entry point must not be used again in that process.  Host threads
 * may make their first calls concurrently. */
#define TRIMUL_STATIC_SCRATCH_BYTES (32u << 20)
int trimul_sm100_forward_static(const trimul_geom_t* geom, const void* x, const void* mask, int32_t mask_kind,
                                const float* ln_in_w, const float* ln_in_b, const void* w_packed,
                                const float* bias_packed, const void* w_fold, const float* cd, void* out,
                                trimul_status_t* status, uint64_t timeout_ns, trimul_stream_t stream);

/* Rank-to-rank ordering of the fused reshards.  Every rank owns a symmetric array of 16 uint64
 * counters (zeroed once).  `peer_signal` adds 1 to counter `slot` on every rank listed in
 * flag_peers[0..cp) (release, system scope) and is enqueued after the kernel whose stores it
 * publishes; `peer_wait` is enqueued before the kernel that consumes them and polls this rank's
 * own counter until it reaches `expected`, giving up after timeout_ns with a status record; with a
 * timeline it records its entry and exit time in slots TRIMUL_TL_WAIT_BASE + 2 * slot (+ 1), slot < 3.
 * Replaces `_A2ADeviceSignal` and the `quiet` + `barrier_all` drains
 * (fold_cp_ops/distributed/workflows/trimul_autotuned.py:322-560, 3272-3300). */
int trimul_sm100_peer_signal(void* const* flag_peers, int32_t cp, int32_t slot, trimul_stream_t stream);
int trimul_sm100_peer_wait(const void* local_flags, int32_t slot, uint64_t expected, trimul_status_t* status,
                           uint64_t* timeline /* nullable */, uint64_t timeout_ns, trimul_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TRIMUL_SM100_H_ */
