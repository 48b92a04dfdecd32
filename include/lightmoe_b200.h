/*
 * C-ABI of the B200 (sm_100a) NVFP4 routed-expert inference kernels.
 *
 * Every entry point takes plain device pointers and sizes, launches on the
 * given CUDA stream, allocates nothing, never synchronises, and returns 0 on
 * success or a non-zero LM_ERR_* code (lm_last_error_string() then describes
 * the failure for the calling thread).  All checks happen on the host before
 * any launch.  Buffers are owned by the caller.
 *
 * The reference project has no C interface: its device code is generated from
 * Python (CuTe DSL) and launched through TVM-FFI.  Each entry point below
 * names the reference host function whose launch it replaces, by file:line in
 * the reference checkout (package `lightmoe`).
 *
 * Data formats
 *   q      E2M1 codes, two per byte, even contraction index in the low nibble
 *   sf     E4M3 scale factor per 16 contraction elements, stored in 512-byte
 *          atoms of 128 rows x 4 factors: byte (row%32)*16 + (row/32%4)*4 + k%4
 *   varlen scale factors: expert e starts at atom row  m_indptr[e]/128 + e
 */
#ifndef LIGHTMOE_B200_H
#define LIGHTMOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* lm_stream_t; /* cudaStream_t */

enum {
  LM_OK = 0,
  LM_ERR_INVALID = 1, /* bad argument (shape, alignment, null pointer) */
  LM_ERR_CUDA = 2,    /* a CUDA runtime or driver call failed */
  LM_ERR_LIMIT = 3    /* size beyond a stated maximum */
};

enum { LM_DTYPE_BF16 = 0, LM_DTYPE_F32 = 1 };

/* scale-factor placement of lm_quantize_rowwise */
enum {
  LM_SF_VARLEN = 0,  /* (1, ceil(rows/128)+E, K/64, 32,4,4), expert e at m_indptr[e]/128 + e */
  LM_SF_BATCHED = 1, /* (E, ceil(rows_per_group/128), K/64, 32,4,4), equal-sized groups   */
  LM_SF_LINEAR = 2   /* (rows, K/16) row-major bytes                                         */
};

enum {
  LM_ACT_NONE = 0,
  LM_ACT_SWIGLU = 1,
  LM_ACT_SWIGLU_OAI = 2,
  LM_ACT_GEGLU = 3,
  LM_ACT_REGLU = 4,
  LM_ACT_RELU2 = 5
};

enum { LM_OUT_BF16 = 0, LM_OUT_F32 = 1, LM_OUT_NVFP4 = 2 };

int lm_version(void);
const char* lm_last_error_string(void);

/* Number of SMs of the current device (used to size persistent grids). */
int lm_sm_count(int* out);

/* Kernel launches this process has made through the library so far (launches recorded into a
   CUDA graph count once, at capture).  For benchmarks that report how many kernels a step is. */
unsigned long long lm_launch_count(void);

/*
 * Device-side status word.  A kernel whose bounded wait ran out sets a bit here and returns
 * instead of hanging: bits 0-2 the GEMM's producer / MMA / epilogue roles (bit 3 unused),
 * LM_STATUS_EP_TIMEOUT a cross-rank signal that never arrived.  Synchronises the stream.
 * *out == 0 means no kernel has reported a problem since the last lm_device_status_clear().
 */
#define LM_STATUS_EP_TIMEOUT 16
#define LM_STATUS_EP_OVERFLOW 32 /* lm_ep_plan: a rank would have received more rows than its buffers hold */
int lm_device_status(uint32_t* out, lm_stream_t stream);
int lm_device_status_clear(lm_stream_t stream);

/*
 * Row-wise NVFP4 quantization, optionally of gathered rows.
 * Replaces nvfp4_quantize_rowwise (lightmoe/kernels/quantize/runtime.py:107-156,
 * kernel body lightmoe/kernels/quantize/kernel.py:807-971).
 *
 *   x            (src_rows, features) BF16 or FP32, row stride = features
 *   rows         number of output rows
 *   m_indptr     (experts+1) int32 prefix of rows per expert; LM_SF_VARLEN only
 *   rows_per_group  LM_SF_BATCHED only: every group has this many rows
 *   scale_pair   float[2] = {pts, 1/pts} on the device
 *   gather_idx   optional (rows) int32: output row r reads x[gather_idx[r]]
 *   q            (rows, features/2) bytes
 *   sf           scale factors in the layout named by sf_mode; within an atom
 *                row that holds valid rows, rows past the group end get 0
 *   te_math      0: sf = e4m3((amax/6)/pts), q = e2m1(x * ((1/pts)/sf))
 *                1: sf = e4m3(amax * ((1/pts) * (1/6))), q = e2m1(x * (1/(sf*pts)))
 * features must be a multiple of 64.
 */
int lm_quantize_rowwise(const void* x, int x_dtype, int64_t rows, int features,
                        const int32_t* m_indptr, int experts, int64_t rows_per_group,
                        const float* scale_pair, const int32_t* gather_idx, uint8_t* q,
                        uint8_t* sf, int sf_mode, int te_math, lm_stream_t stream);

/*
 * Decode quantization: each token row is quantized once (te math) and its
 * packed row and scale factors are written to every destination slot.
 * Replaces nvfp4_quantize_decode (lightmoe/kernels/quantize/decode.py:1108-1165).
 *   slots  (tokens*top_k) int32 destination rows, -1 = dropped
 *   sf     varlen atoms addressed through m_indptr like LM_SF_VARLEN
 */
int lm_quantize_decode(const void* x, int64_t tokens, int features, int top_k,
                       const int32_t* slots, const int32_t* topk_ids, const int32_t* m_indptr,
                       int experts, const float* scale_pair, uint8_t* q, uint8_t* sf,
                       lm_stream_t stream);

/*
 * Calibration: *out = max |act(preact)| over a BF16 first-projection result (rows, n), the
 * activation applied in FP32 with exact exp / tanh; gated activations read (gate, up) from
 * column pairs (2j, 2j+1).  Stands in for the torch chain of InferenceMoE.calibrate_routed
 * (lightmoe/inference.py:763-779); the hidden scale is *out / 2688.  n must be a multiple of 8.
 */
int lm_activation_amax(const void* preact, int64_t rows, int n, int activation, float clamp_limit,
                       float sigmoid_alpha, float up_bias, float* out, lm_stream_t stream);

/*
 * Scratch size, in int32 elements, that lm_dispatch needs for `rows`
 * assignments and `experts` experts.
 */
int64_t lm_dispatch_scratch_elems(int64_t rows, int experts);

/*
 * Stable expert-major permutation of (token, route) pairs.
 * Replaces moe_dispatch (lightmoe/kernels/routing/dispatch.py:368-397).
 *
 *   topk_ids      (tokens, top_k) int32 expert of each pair, values in [0, experts)
 *   topk_weights  (tokens, top_k) float
 *   gather        (rows) int32   out: source token of each expert-major row
 *   m_indptr      (experts+1)    out: prefix of rows per expert
 *   probs         (rows) float   out: routing weight of each expert-major row
 *   slots         (rows) int32   out: expert-major row of pair p = token*top_k + route
 *   padded_offsets (experts)     out: inclusive prefix of ceil(count/plan_tile_rows)*128
 *   scratch       int32 scratch of lm_dispatch_scratch_elems() elements; when
 *                 rows <= 1024 it also receives the decode plan:
 *                 scratch[0] = tile count, scratch[1+i] = expert + tile*experts,
 *                 scratch[scratch_elems-experts+e] = first atom row of expert e
 *   plan_tile_rows  rows per plan tile (8,16,32,64 or 128); the multi-block
 *                 path (rows > 1024) always pads to 128
 * experts <= 256.  rows = tokens*top_k <= 2^22.
 */
int lm_dispatch(const int32_t* topk_ids, const float* topk_weights, int64_t tokens, int top_k,
                int experts, int32_t* gather, int32_t* m_indptr, float* probs, int32_t* slots,
                int32_t* padded_offsets, int32_t* scratch, int64_t scratch_elems,
                int plan_tile_rows, lm_stream_t stream);

/*
 * Decode step preparation in one launch: lm_dispatch followed by lm_quantize_decode for at
 * most 1024 assignments.  Every CTA repeats the single-block dispatch in shared memory, so
 * the launch has no inter-CTA dependency.
 * Replaces nvfp4_dispatch_quantize_decode (lightmoe/kernels/quantize/decode.py:1168-1257).
 * Arguments as in lm_dispatch and lm_quantize_decode; x is (tokens, features) BF16.
 */
int lm_dispatch_quantize_decode(const void* x, const int32_t* topk_ids, const float* topk_weights,
                                int64_t tokens, int top_k, int experts, int features,
                                int32_t* gather, int32_t* m_indptr, float* probs, int32_t* slots,
                                int32_t* padded_offsets, int32_t* scratch, int64_t scratch_elems,
                                int plan_tile_rows, const float* scale_pair, uint8_t* q, uint8_t* sf,
                                lm_stream_t stream);

/*
 * Decode step preparation for ONE token in one launch, without scratch: the routing metadata
 * of lm_dispatch for its top_k routes and lm_quantize_decode of its row.
 * Replaces nvfp4_decode_prepare and nvfp4_direct_decode_prepare
 * (lightmoe/kernels/quantize/decode.py:946-1105, kernel :548-818).
 *   direct == 0  expert-major: gather / slots / probs (top_k), cu = m_indptr (experts+1),
 *                padded_offsets (experts); the row is written to each of its top_k
 *                expert-major rows, scale factors as varlen atoms (expert e in atom row e).
 *   direct != 0  route order is kept: slots[r] = r, cu[r] = expert of route r (top_k entries,
 *                what lm_gemm_args.direct_routes reads as its table), probs[r] = weight of route
 *                r; the row is quantized once into row 0 of q, scale factors into atom row 0.
 *                padded_offsets is not written.
 * x is (1, features) BF16; top_k <= min(experts, 32).
 */
int lm_decode_prepare(const void* x, const int32_t* topk_ids, const float* topk_weights, int top_k,
                      int experts, int features, int direct, int32_t* gather, int32_t* slots,
                      int32_t* cu, float* probs, int32_t* padded_offsets, const float* scale_pair,
                      uint8_t* q, uint8_t* sf, lm_stream_t stream);

/*
 * lm_dispatch for callers that have no device memory to give as scratch and
 * may not obtain any: a plugin inside a serving process whose memory pool
 * already owns the whole GPU, or a host runtime that forbids its extensions to
 * call the CUDA allocator.  This entry point has no counterpart in the
 * reference.  It computes exactly what lm_dispatch computes, but keeps the
 * per-chunk counts in a fixed array inside the library (128 KB of device
 * memory per GPU, held until the process exits) and calls no allocating
 * routine.
 *
 *   Limit: tokens * top_k <= lm_dispatch_static_max_rows() (131072) and
 *   experts <= 256; larger inputs return LM_ERR_LIMIT and launch nothing.
 *   plan_out / plan_elems: optional buffer for the decode plan that the
 *   single-block path (rows <= 1024) writes, laid out as lm_dispatch lays it
 *   out in its scratch; NULL to drop the plan.
 *
 * The first call on each device looks up the array's device address (with
 * that device current); make that first call before any stream capture
 * begins.  All calls on a device share the one array and nothing in it needs
 * to start at zero -- each call overwrites every entry it later reads -- but
 * two calls that overlap on the GPU (different streams) race on it: keep calls
 * on one device in stream order.
 */
int64_t lm_dispatch_static_max_rows(void);
int lm_dispatch_static(const int32_t* topk_ids, const float* topk_weights, int64_t tokens,
                       int top_k, int experts, int32_t* gather, int32_t* m_indptr, float* probs,
                       int32_t* slots, int32_t* padded_offsets, int32_t* plan_out,
                       int64_t plan_elems, int plan_tile_rows, lm_stream_t stream);

/*
 * Deterministic top-k combine: out[t] = bf16(sum_j f32(rows[slot]) * w[slot]),
 * j ascending, product rounded before the add, slot -1 skipped.
 * Replaces moe_finalize (lightmoe/kernels/routing/combine.py:231-281).
 *   routed_out (rows, hidden) BF16; slots (tokens*top_k); weights (rows) or NULL
 *   out (tokens, hidden) BF16.  hidden must be a multiple of 8.
 *   valid    optional device flag: when *valid == 0 the rows were not computed this step (an
 *            expert-parallel step that lm_ep_plan skipped) and out is written as zeros
 *   use_pdl  launch as a programmatic dependent of the previous kernel in the stream: the kernel
 *            reads slots and weights while that kernel may still run and waits for it before
 *            it reads routed_out, so slots, weights and valid must not be that kernel's output
 */
int lm_finalize(const void* routed_out, const int32_t* slots, const float* weights, void* out,
                int64_t tokens, int top_k, int hidden, int64_t routed_row_stride,
                int64_t out_row_stride, const int32_t* valid, int use_pdl, lm_stream_t stream);

/*
 * Grouped / dense block-scaled FP4 GEMM:  out[rows_e, :] = alpha_e * A_e @ B_e^T
 * with FP32 accumulation, optionally followed by a gated or unary activation
 * and NVFP4 requantization of the result.
 * Replaces GroupedNvfp4Gemm.prepare/launch
 * (lightmoe/kernels/grouped/runtime.py:325-589) and DenseNvfp4Gemm
 * (lightmoe/kernels/dense/runtime.py:54-143).
 */
typedef struct lm_gemm_args {
  int32_t experts;       /* 1 for a dense GEMM */
  int32_t n;             /* rows of each B_e (accumulator columns) */
  int32_t k;             /* contraction length, multiple of 64 */
  int32_t tile_m;        /* 128 */
  int32_t tile_n;        /* 64, 128 or 256 (NVFP4 output: 128) */
  int32_t out_kind;      /* LM_OUT_* */
  int32_t activation;    /* LM_ACT_*; requires out_kind == LM_OUT_NVFP4 */
  float clamp_limit;     /* 0 = no clamp */
  float sigmoid_alpha;
  float up_bias;
  int32_t alpha_per_expert; /* 0: alpha[0], 1: alpha[e] */
  int32_t dense;         /* 1: single group of `rows` rows, m_indptr ignored */
  int32_t sf_tile_rows;  /* rows per scale-factor atom row group: 128 */
  int32_t max_ctas;      /* 0 = one CTA per SM */
  int64_t rows;          /* rows of A and of out */
  const void* a;         /* (rows, k/2) bytes */
  const void* b;         /* (experts, n, k/2) bytes */
  void* out;             /* (rows, n) BF16/F32, or (rows, out_n/2) bytes */
  const int32_t* m_indptr; /* (experts+1) */
  const void* sfa;       /* varlen atoms, K/64 atom columns */
  const void* sfb;       /* (experts, ceil(n/128), k/64, 512) */
  const float* alpha;    /* (1) or (experts) */
  void* out_sf;          /* NVFP4 output: varlen atoms with out_n/64 atom columns */
  const float* out_scale; /* NVFP4 output: {pts, 1/pts} of the result */
  const uint64_t* out_row_ptrs; /* BF16 output, optional: device table (rows) of 16-byte aligned
                                   addresses, row i is written there instead of out + i*n; the
                                   addresses may point into a peer GPU's memory */
  /* Decode-shaped kernel (swap_ab of lightmoe/kernels/grouped/runtime.py:181-203, kernel
     lightmoe/kernels/grouped/kernel.py:155-221): the expert's weights take the 128-row side of
     the MMA and its few token rows the 8..64-column side; tile_m / tile_n are ignored, the
     result is bit-identical to the other tilings.  For steps with a handful of rows per expert. */
  int32_t swap_ab;
  /* swap_ab only (direct_routes / broadcast_a of the same constructor,
     lightmoe/inference.py:656-721): > 0 = the routes of ONE token without a dispatch.
     m_indptr then holds `direct_routes` expert ids; route r multiplies row r of a (row 0 with
     broadcast_a) -- its scale factors in atom row r (0), row 0 -- with expert m_indptr[r] and
     writes row r of out (NVFP4 output: scale factors in atom row r, row 0).  rows must equal
     direct_routes (<= 32).  An id outside [0, experts) computes nothing. */
  int32_t direct_routes;
  int32_t broadcast_a;
  /* Launch as a programmatic dependent of the previous kernel in the stream (use_pdl of the
     reference's constructor): the kernel sets itself up while that kernel may still run and
     waits for it before it reads m_indptr or an operand; its own dependents are released after
     that wait. */
  int32_t use_pdl;
  /* use_pdl only: read the routing table and start the weight stream before waiting for the
     previous kernel.  Allowed when m_indptr, b, sfb and alpha were complete before the previous
     kernel began, and that kernel either is a use_pdl launch of this library (it releases its
     dependents only after its own wait: the second projection after the first) or was launched
     the plain way and releases its dependents early (lm_decode_prepare before a first
     projection whose direct routes are read from the caller's topk_ids). */
  int32_t weights_ahead;
  /* With out_row_ptrs (BF16 output that returns to the ranks of an expert-parallel group): whole
     32-row blocks leave as one bulk tensor store each instead of row by row.  out_blocks is the
     table lm_ep_plan writes; return_bases is a HOST array of `return_world` addresses, the
     return buffer of every rank (return_rows rows of n BF16 values, 16-byte aligned).  Blocks
     the table marks -1 still go through out_row_ptrs. */
  const int32_t* out_blocks;
  const uint64_t* return_bases;
  int32_t return_world;
  int64_t return_rows;
} lm_gemm_args;

/* Caller-provided storage for a prepared GEMM (tensor maps + arguments). */
typedef struct lm_gemm_plan {
  uint64_t opaque[320];
} lm_gemm_plan;

/* Host only: validates `args` and encodes the TMA descriptors into `plan`. */
int lm_gemm_prepare(const lm_gemm_args* args, lm_gemm_plan* plan);
/* Launches a prepared GEMM.  Safe inside CUDA Graph capture. */
int lm_gemm_launch(const lm_gemm_plan* plan, lm_stream_t stream);
/* What a prepared plan will launch: kernel 0 = 128 x 128 tiles, 1 = 128 x 256 tiles, 2 = 256 x 256
   tiles on CTA pairs, 3 = the decode-shaped kernel; its grid; the depth of its operand ring
   (the `stages` the reference's plans report, lightmoe/kernels/dense/runtime.py:88). */
int lm_gemm_plan_info(const lm_gemm_plan* plan, int32_t* kernel, int32_t* grid, int32_t* ring_stages);

/*
 * Router step in front of lm_dispatch: softmax over the experts, top-k, renormalise, as the
 * reference's tests and benchmarks prepare their routing inputs with torch
 * (tests/test_training_gpu.py:23-27, benchmarks/moe.py: softmax -> topk -> divide by the sum).
 * The reference leaves this step to the host framework and keeps it out of its timings
 * (BENCHMARKS.md:15).
 *   logits        (tokens, experts) BF16 or FP32 (LM_DTYPE_*), experts <= 256
 *   topk_ids      (tokens, top_k) int32, larger probability first, lower id on a tie
 *   topk_weights  (tokens, top_k) FP32, summing to 1 per token
 */
int lm_route_topk(const void* logits, int logits_dtype, int64_t tokens, int experts, int top_k,
                  int32_t* topk_ids, float* topk_weights, lm_stream_t stream);

/* ---------------------------------------------------------------- expert parallel
 * The reference has no communication code (README.md:227-228 leaves expert-parallel
 * exchange to the host framework); these two entry points are that exchange for one
 * NVLink domain, over peer pointers.  Rank r of `world` owns experts
 * [r*experts/world, (r+1)*experts/world).
 */
#define LM_EP_MAX_RANKS 8

/*
 * Route plan, from the gathered row counts of all ranks, entirely on the device.
 *   counts_all   (world, experts) int32, row g = rows rank g routed to every expert
 *   return_base  HOST array (world) of the address of every rank's return buffer
 *                (rows of `row_bytes` bytes in that rank's own expert-major order)
 *   own_indptr   (experts/world + 1) bounds of the rows this rank receives, expert-major,
 *                within an expert by source rank
 *   dest_base    (experts) row on the owner where this rank's rows of expert e begin
 *   owner_start  (experts) row on the owner where expert e begins
 *   row_ptrs     (max_rows) address each received row's result goes to (lm_gemm_args.out_row_ptrs)
 *   out_blocks   optional ((max_rows/128 + experts/world) * 4, 2) int32 for lm_gemm_args.out_blocks:
 *                per 32-row block of every 128-row tile (atom row of the tile, quarter) the source
 *                rank and the first row in that rank's return buffer when the block is 32 whole
 *                rows of one (expert, source) segment, else -1
 *   valid        1, or 0 when some rank would receive more than max_rows rows: then own_indptr
 *                is all zero (the GEMMs compute nothing) and lm_ep_quantize_send sends nothing
 */
int lm_ep_plan(const int32_t* counts_all, int world, int rank, int experts, int64_t max_rows,
               int64_t row_bytes, const uint64_t* return_base, int32_t* own_indptr,
               int32_t* dest_base, int32_t* owner_start, uint64_t* row_ptrs, int32_t* out_blocks,
               int32_t* valid, lm_stream_t stream);

/*
 * lm_quantize_decode whose destinations are the owners' operand buffers: each token is
 * quantized once and its packed row and scale factors are stored, through peer pointers, at
 * the rows lm_ep_plan assigned.
 *   slots, topk_ids, src_indptr  this rank's lm_dispatch outputs over the global experts
 *   q_base, sf_base  HOST arrays (world) of the addresses of every rank's packed-row buffer
 *                    (rows of features/2 bytes) and row-major scale factors (rows of
 *                    features/16 bytes); the owner turns the latter into atoms with
 *                    lm_ep_sf_swizzle once every source has finished
 */
int lm_ep_quantize_send(const void* x, int64_t tokens, int features, int top_k, int world,
                        int experts, const int32_t* slots, const int32_t* topk_ids,
                        const int32_t* src_indptr, const int32_t* dest_base,
                        const int32_t* owner_start, const int32_t* valid, const float* scale_pair,
                        const uint64_t* q_base, const uint64_t* sf_base, lm_stream_t stream);

/*
 * Cross-rank signal, one launch of one CTA per rank; the ranks must run on different GPUs.
 * With m_indptr: first stores this rank's per-expert row counts (m_indptr[e+1] - m_indptr[e])
 * as row `rank` of every rank's (world, experts) table.  Then every rank tells every rank that
 * it has made one more signal call and waits until all of them have; stores this rank made to
 * peer memory in earlier launches of the stream are ordered before the signal.  Every rank
 * must make the same sequence of calls.  The call count lives on the device (word `world` of
 * the rank's own pad), so a captured CUDA graph of a step can be replayed.  The wait gives up
 * after timeout_ms (0 = ten seconds; counted in SM cycles at a nominal 2 GHz) and sets
 * LM_STATUS_EP_TIMEOUT.
 *   counts_all_base, signal_base  HOST arrays (world) of the addresses of every rank's count
 *                                 table and signal pad (world + 1 uint32 words, zero at start)
 */
int lm_ep_signal(const int32_t* m_indptr, int experts, int world, int rank,
                 const uint64_t* counts_all_base, const uint64_t* signal_base, int timeout_ms,
                 lm_stream_t stream);

/*
 * Row-major scale factors (max_rows, features/16) -> varlen atoms as LM_SF_VARLEN lays them
 * out (expert e starts at atom row m_indptr[e]/128 + e).  Rows past an expert's last row in
 * its last tile are written as zero.  features must be a multiple of 256.
 */
int lm_ep_sf_swizzle(const uint8_t* linear, int64_t max_rows, int features, const int32_t* m_indptr,
                     int experts, uint8_t* atoms, lm_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LIGHTMOE_B200_H */
