// Stable expert-major dispatch of (token, route) pairs: a counting sort with
// no data-dependent atomics in the placement, so the permutation is bit-stable.
//
// rows <= 1024: one CTA ranks, scans and scatters, and also writes the decode
//               tile plan.
// rows  > 1024: kernel 1 counts pairs per (1024-pair chunk, expert); kernel 2
//               gives each chunk its stable base (prefix over experts, then over
//               earlier chunks) and scatters.
#include <atomic>

#include "common.cuh"
#include "quantize_math.cuh"

namespace lm {
namespace {

constexpr int kThreads = 256;
constexpr int kChunk = 1024;
constexpr int kPerThread = kChunk / kThreads;  // 4
constexpr int kSegments = kChunk / 32;         // warp-sized segments per chunk
constexpr int kMaxExperts = 256;

struct DispatchParams {
  const int32_t* ids;
  const float* weights;
  int64_t rows;
  int top_k;
  int experts;
  int32_t* gather;
  int32_t* m_indptr;
  float* probs;
  int32_t* slots;
  int32_t* padded;
  int32_t* scratch;
  int64_t scratch_elems;
  int plan_tile_rows;
  int chunks;
};

__global__ void __launch_bounds__(kThreads) dispatch_count_kernel(DispatchParams p) {
  __shared__ int s_count[kMaxExperts];
  const int tid = threadIdx.x;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kChunk;
  for (int e = tid; e < p.experts; e += kThreads) s_count[e] = 0;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    int64_t pos = base + tid + i * kThreads;
    if (pos < p.rows) {
      int e = __ldg(p.ids + pos);
      if (e >= 0 && e < p.experts) atomicAdd(&s_count[e], 1);  // out-of-range ids are dropped
    }
  }
  __syncthreads();
  for (int e = tid; e < p.experts; e += kThreads)
    p.scratch[static_cast<int64_t>(blockIdx.x) * p.experts + e] = s_count[e];
}

// Block-wide inclusive scan of one int per thread (256 threads).
__device__ __forceinline__ int block_inclusive_scan(int v, int* s_warp) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int t = __shfl_up_sync(0xFFFFFFFFu, v, d);
    if (lane >= d) v += t;
  }
  if (lane == 31) s_warp[warp] = v;
  __syncthreads();
  int add = 0;
  for (int w = 0; w < warp; ++w) add += s_warp[w];
  __syncthreads();
  return v + add;
}

// Places the pairs of one 1024-pair chunk.  s_seg [kSegments][experts], s_chunk [kChunk],
// s_base [kMaxExperts] and s_warp [3][8] are shared-memory work areas; on return s_chunk
// holds each pair's expert (-1 = dropped), s_base each expert's first row for this chunk
// and, when s_slot is given, s_slot each pair's destination row (-1 = dropped).  Global
// outputs are written only when write_global is set.
template <bool kSingle>
__device__ __forceinline__ void dispatch_chunk(const DispatchParams& p, int chunk, bool write_global,
                                               int* s_seg, int* s_chunk, int* s_base,
                                               int (*s_warp)[kThreads / 32], int* s_slot) {
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int64_t chunk_base = static_cast<int64_t>(chunk) * kChunk;
  const int E = p.experts;

  for (int i = tid; i < kSegments * E; i += kThreads) s_seg[i] = 0;
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    int j = tid + i * kThreads;
    int64_t pos = chunk_base + j;
    int e = pos < p.rows ? __ldg(p.ids + pos) : -1;
    s_chunk[j] = (e >= 0 && e < E) ? e : -1;
  }
  __syncthreads();

  // ---- rank of every pair among equal experts inside its warp segment
  int rank[kPerThread];
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    int value = s_chunk[tid + i * kThreads];
    unsigned peers = __match_any_sync(0xFFFFFFFFu, value);
    rank[i] = __popc(peers & ((1u << lane) - 1u));
    if (value >= 0 && rank[i] == 0) s_seg[(i * (kThreads / 32) + warp) * E + value] = __popc(peers);
  }
  __syncthreads();

  // ---- per expert: exclusive prefix over segments, chunk total
  int in_chunk = 0;
  int total = 0;
  int before = 0;
  if (tid < E) {
    for (int s = 0; s < kSegments; ++s) {
      int c = s_seg[s * E + tid];
      s_seg[s * E + tid] = in_chunk;
      in_chunk += c;
    }
    if (kSingle) {
      total = in_chunk;
    } else {
      // sixteen independent loads in flight per round trip to L2
      for (int b0 = 0; b0 < p.chunks; b0 += 16) {
        int c[16];
#pragma unroll
        for (int j = 0; j < 16; ++j)
          c[j] = b0 + j < p.chunks ? __ldg(p.scratch + static_cast<int64_t>(b0 + j) * E + tid) : 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          total += c[j];
          if (b0 + j < chunk) before += c[j];
        }
      }
    }
  }
  const int tile_rows = kSingle ? p.plan_tile_rows : 128;
  const int tiles = (total + tile_rows - 1) / tile_rows;
  const int incl_rows = block_inclusive_scan(total, s_warp[0]);
  const int incl_pad = block_inclusive_scan(tiles * 128, s_warp[1]);
  const int incl_tiles = block_inclusive_scan(tiles, s_warp[2]);
  if (tid < E) {
    s_base[tid] = incl_rows - total + before;
    if (chunk == 0 && write_global) {
      p.m_indptr[tid + 1] = incl_rows;
      p.padded[tid] = incl_pad;
      if (tid == 0) p.m_indptr[0] = 0;
      if (kSingle) {
        int first = incl_tiles - tiles;
        for (int t = 0; t < tiles; ++t) p.scratch[1 + first + t] = tid + t * E;
        p.scratch[p.scratch_elems - E + tid] = first;
        if (tid == E - 1) p.scratch[0] = incl_tiles;
      }
    }
  }
  __syncthreads();

  // ---- scatter
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    int j = tid + i * kThreads;
    int64_t pos = chunk_base + j;
    int e = s_chunk[j];
    int dst = -1;
    if (pos < p.rows && e >= 0) dst = s_base[e] + s_seg[(i * (kThreads / 32) + warp) * E + e] + rank[i];
    if (s_slot != nullptr) s_slot[j] = dst;
    if (!write_global || pos >= p.rows) continue;
    p.slots[pos] = dst;  // -1 for a dropped pair: the combine skips it
    if (dst >= 0) {
      p.gather[dst] = static_cast<int32_t>(pos / p.top_k);
      p.probs[dst] = __ldg(p.weights + pos);
    }
  }
}

template <bool kSingle>
__global__ void __launch_bounds__(kThreads) dispatch_scatter_kernel(DispatchParams p) {
  extern __shared__ int s_dyn[];
  int* s_seg = s_dyn;                            // [kSegments][experts]
  int* s_chunk = s_seg + kSegments * p.experts;  // [kChunk]
  __shared__ int s_base[kMaxExperts];
  __shared__ int s_warp[3][kThreads / 32];
  dispatch_chunk<kSingle>(p, blockIdx.x, true, s_seg, s_chunk, s_base, s_warp, nullptr);
}

// ------------------------------------------------ decode: dispatch + quantize, one launch
// For at most 1024 pairs.  Every CTA repeats the (tiny) single-chunk dispatch in its own
// shared memory, so no CTA waits for another; CTA (0,0) alone writes the routing outputs.
// Then each warp quantizes one (token, 512-feature slice) once and writes codes and scale
// factors to all of the token's rows, as the stand-alone quantize-scatter kernel does.
struct DecodePrepareParams {
  DispatchParams d;
  const __nv_bfloat16* x;
  int features;
  const float* scale_pair;
  uint8_t* q;
  uint8_t* sf;
};

__global__ void __launch_bounds__(kThreads) dispatch_quantize_decode_kernel(DecodePrepareParams p) {
  // the first projection, launched as a programmatic dependent, may set itself up meanwhile
  // (it waits for this kernel to finish before it reads anything)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  extern __shared__ int s_dyn[];
  const int E = p.d.experts;
  int* s_seg = s_dyn;
  int* s_chunk = s_seg + kSegments * E;
  int* s_slot = s_chunk + kChunk;
  __shared__ int s_base[kMaxExperts];
  __shared__ int s_warp[3][kThreads / 32];
  dispatch_chunk<true>(p.d, 0, blockIdx.x == 0 && blockIdx.y == 0, s_seg, s_chunk, s_base, s_warp, s_slot);
  __syncthreads();

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int top_k = p.d.top_k;
  const int64_t tokens = p.d.rows / top_k;
  const int64_t token = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + warp;
  if (token >= tokens) return;
  const int col = blockIdx.y * 512 + lane * 16;
  const bool col_ok = col < p.features;
  int my_slot = -1, my_atom_row = 0, my_r = 0;
  if (lane < top_k) {
    const int pair = static_cast<int>(token) * top_k + lane;
    my_slot = s_slot[pair];
    if (my_slot >= 0) {
      const int e = s_chunk[pair];
      const int lo = s_base[e];
      const int local = my_slot - lo;
      my_atom_row = lo / 128 + e + local / 128;
      my_r = local % 128;
    }
  }
  const float pts = __ldg(p.scale_pair);
  const float inv_pts = __ldg(p.scale_pair + 1);
  Slice<__nv_bfloat16> v;
  uint2 packed = make_uint2(0, 0);
  uint32_t sf_byte = 0;
  if (col_ok) {
    v.load(p.x + token * p.features + col);
    sf_byte = quantize_group(v, pts, inv_pts, true, &packed);
  }
  uint32_t word = sf_byte;
  word |= __shfl_down_sync(0xFFFFFFFFu, sf_byte, 1) << 8;
  word |= __shfl_down_sync(0xFFFFFFFFu, sf_byte, 2) << 16;
  word |= __shfl_down_sync(0xFFFFFFFFu, sf_byte, 3) << 24;
  const int atom_cols = p.features >> 6;
  for (int j = 0; j < top_k; ++j) {
    const int slot = __shfl_sync(0xFFFFFFFFu, my_slot, j);
    const int atom_row = __shfl_sync(0xFFFFFFFFu, my_atom_row, j);
    const int r = __shfl_sync(0xFFFFFFFFu, my_r, j);
    if (slot < 0 || !col_ok) continue;
    *reinterpret_cast<uint2*>(p.q + static_cast<int64_t>(slot) * (p.features >> 1) + (col >> 1)) = packed;
    if ((lane & 3) == 0) {
      uint8_t* dst = p.sf + (static_cast<int64_t>(atom_row) * atom_cols + (col >> 6)) * 512 +
                     (r & 31) * 16 + (r >> 5) * 4;
      *reinterpret_cast<uint32_t*>(dst) = word;
    }
  }
}

// ------------------------------------------------ one token: routing metadata + quantize, one launch
// No sort is needed for the k <= 32 routes of a single token: thread r counts the routes that
// come before route r in expert-major order.  `direct` keeps the routes in their own order
// instead: the token is quantized once into row 0 and a table of expert ids replaces m_indptr.
struct OneTokenParams {
  const __nv_bfloat16* x;
  const int32_t* topk_ids;
  const float* topk_weights;
  int top_k;
  int experts;
  int features;
  int direct;
  int32_t* gather;
  int32_t* slots;
  int32_t* cu;  // m_indptr (experts + 1), or with `direct` the expert id of every route (top_k)
  float* probs;
  int32_t* padded_offsets;
  const float* scale_pair;
  uint8_t* q;
  uint8_t* sf;
};

__global__ void __launch_bounds__(kThreads) decode_prepare_one_kernel(OneTokenParams p) {
  // the first projection, launched as a programmatic dependent, may set itself up meanwhile
  // (it waits for this kernel to finish before it reads anything)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ int s_ids[32];
  __shared__ int s_dst[32];   // expert-major row of route r
  __shared__ int s_rank[32];  // its place among the routes of the same expert
  const int k = p.top_k;
  if (threadIdx.x < k) s_ids[threadIdx.x] = __ldg(p.topk_ids + threadIdx.x);
  __syncthreads();
  if (threadIdx.x < k) {
    const int r = threadIdx.x, e = s_ids[r];
    int dst = 0, rank = 0;
    for (int o = 0; o < k; ++o) {
      const int eo = s_ids[o];
      dst += (eo < e) || (eo == e && o < r);
      rank += (eo == e && o < r);
    }
    s_dst[r] = p.direct ? r : dst;
    s_rank[r] = p.direct ? 0 : rank;
    if (blockIdx.x == 0) {
      const int row = s_dst[r];
      p.slots[r] = row;
      p.gather[row] = 0;
      p.probs[row] = __ldg(p.topk_weights + r);
      if (p.direct) p.cu[r] = e;
    }
  }
  if (blockIdx.x == 0 && !p.direct) {
    // m_indptr[e] = routes of experts below e; padded_offsets[e] = 128 x experts up to e with a route
    for (int e = threadIdx.x; e <= p.experts; e += kThreads) {
      int below = 0, used = 0;
      for (int o = 0; o < k; ++o) {
        const int eo = s_ids[o];
        below += eo < e;
        bool first = eo <= e;
        for (int q = 0; q < o; ++q) first = first && s_ids[q] != eo;
        used += first;
      }
      p.cu[e] = below;
      if (e < p.experts) p.padded_offsets[e] = used * 128;
    }
  }
  __syncthreads();
  // quantize: each warp one 512-feature slice, written to every row of the token (row 0 only
  // with `direct`); the scale factors of expert-major row d of expert e sit in atom row e
  // (fewer than 128 rows in all), row `rank`
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = (blockIdx.x * (kThreads / 32) + warp) * 512 + lane * 16;
  if (col - lane * 16 >= p.features) return;
  const bool col_ok = col < p.features;
  const float pts = __ldg(p.scale_pair);
  const float inv_pts = __ldg(p.scale_pair + 1);
  Slice<__nv_bfloat16> v;
  uint2 packed = make_uint2(0, 0);
  uint32_t sf_byte = 0;
  if (col_ok) {
    v.load(p.x + col);
    sf_byte = quantize_group(v, pts, inv_pts, true, &packed);
  }
  uint32_t word = sf_byte;
  word |= __shfl_down_sync(0xFFFFFFFFu, sf_byte, 1) << 8;
  word |= __shfl_down_sync(0xFFFFFFFFu, sf_byte, 2) << 16;
  word |= __shfl_down_sync(0xFFFFFFFFu, sf_byte, 3) << 24;
  if (!col_ok) return;
  const int atom_cols = p.features >> 6;
  const int copies = p.direct ? 1 : k;
  for (int r = 0; r < copies; ++r) {
    const int row = p.direct ? 0 : s_dst[r];
    const int atom_row = p.direct ? 0 : s_ids[r];
    const int in_tile = p.direct ? 0 : s_rank[r];
    *reinterpret_cast<uint2*>(p.q + static_cast<int64_t>(row) * (p.features >> 1) + (col >> 1)) = packed;
    if ((lane & 3) == 0)
      *reinterpret_cast<uint32_t*>(p.sf + (static_cast<int64_t>(atom_row) * atom_cols + (col >> 6)) * 512 +
                                   (in_tile & 31) * 16 + (in_tile >> 5) * 4) = word;
  }
}

// Scratch of the entry point that allocates nothing: room for the per-chunk
// counts of 128 chunks x 256 experts (131072 assignments).  Every GPU that loads
// the library holds these 128 KB until the process exits.
constexpr int kStaticChunks = 128;
constexpr int64_t kStaticElems = static_cast<int64_t>(kStaticChunks) * kMaxExperts;
static __device__ __align__(256) int32_t g_static_scratch[kStaticElems];

// In host code the array's name is only a handle; the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_ptr(int32_t** out) {
  // two host threads may make the first call on a device at once: both look the address up and
  // store the same value, through atomics so that neither reads a torn pointer
  static std::atomic<int32_t*> cached[64];
  int device = 0;
  LM_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= 64) return set_error(LM_ERR_LIMIT, "dispatch_static: device index out of range");
  int32_t* ptr = cached[device].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    LM_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch));
    cached[device].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return LM_OK;
}

}  // namespace
}  // namespace lm

extern "C" int64_t lm_dispatch_scratch_elems(int64_t rows, int experts) {
  int64_t chunks = (rows + lm::kChunk - 1) / lm::kChunk;
  if (chunks < 128) chunks = 128;
  return chunks * experts;
}

extern "C" int lm_dispatch(const int32_t* topk_ids, const float* topk_weights, int64_t tokens,
                           int top_k, int experts, int32_t* gather, int32_t* m_indptr, float* probs,
                           int32_t* slots, int32_t* padded_offsets, int32_t* scratch,
                           int64_t scratch_elems, int plan_tile_rows, lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(topk_ids && topk_weights && gather && m_indptr && probs && slots && padded_offsets && scratch,
             "dispatch: null pointer");
  LM_REQUIRE(experts > 0 && experts <= kMaxExperts, "dispatch: at most 256 experts");
  LM_REQUIRE(top_k > 0 && tokens > 0, "dispatch: empty routing");
  LM_REQUIRE(plan_tile_rows > 0 && 128 % plan_tile_rows == 0, "dispatch: plan_tile_rows must divide 128");
  const int64_t rows = tokens * top_k;
  if (rows > (1ll << 22)) return set_error(LM_ERR_LIMIT, "dispatch: more than 2^22 assignments");
  const int chunks = static_cast<int>((rows + kChunk - 1) / kChunk);
  DispatchParams p{topk_ids, topk_weights, rows,    top_k,         experts,        gather, m_indptr,
                   probs,    slots,        padded_offsets, scratch, scratch_elems, plan_tile_rows, chunks};
  const size_t smem = sizeof(int) * (static_cast<size_t>(kSegments) * experts + kChunk);
  cudaStream_t s = as_stream(stream);
  if (chunks == 1) {
    int64_t plan_need = 1 + (rows + plan_tile_rows - 1) / plan_tile_rows + experts + experts;
    LM_REQUIRE(scratch_elems >= plan_need, "dispatch: scratch too small for the decode plan");
    dispatch_scatter_kernel<true><<<1, kThreads, smem, s>>>(p);
    note_launch();
  } else {
    LM_REQUIRE(scratch_elems >= static_cast<int64_t>(chunks) * experts, "dispatch: scratch too small");
    dispatch_count_kernel<<<chunks, kThreads, 0, s>>>(p);
    note_launch();
    LM_CUDA(cudaGetLastError());
    dispatch_scatter_kernel<false><<<chunks, kThreads, smem, s>>>(p);
    note_launch();
  }
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}

extern "C" int64_t lm_dispatch_static_max_rows(void) {
  return static_cast<int64_t>(lm::kStaticChunks) * lm::kChunk;
}

extern "C" int lm_dispatch_static(const int32_t* topk_ids, const float* topk_weights, int64_t tokens,
                                  int top_k, int experts, int32_t* gather, int32_t* m_indptr,
                                  float* probs, int32_t* slots, int32_t* padded_offsets,
                                  int32_t* plan_out, int64_t plan_elems, int plan_tile_rows,
                                  lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(topk_ids && topk_weights && gather && m_indptr && probs && slots && padded_offsets,
             "dispatch_static: null pointer");
  LM_REQUIRE(experts > 0 && experts <= kMaxExperts, "dispatch_static: at most 256 experts");
  LM_REQUIRE(top_k > 0 && tokens > 0, "dispatch_static: empty routing");
  LM_REQUIRE(plan_tile_rows > 0 && 128 % plan_tile_rows == 0,
             "dispatch_static: plan_tile_rows must divide 128");
  const int64_t rows = tokens * top_k;
  if (rows > lm_dispatch_static_max_rows())
    return set_error(LM_ERR_LIMIT, "dispatch_static: %lld assignments exceed the built-in scratch (%lld)",
                     static_cast<long long>(rows), static_cast<long long>(lm_dispatch_static_max_rows()));
  int32_t* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc != LM_OK) return rc;
  const int chunks = static_cast<int>((rows + kChunk - 1) / kChunk);
  DispatchParams p{topk_ids, topk_weights, rows,    top_k,         experts,      gather, m_indptr,
                   probs,    slots,        padded_offsets, scratch, kStaticElems, plan_tile_rows, chunks};
  const size_t smem = sizeof(int) * (static_cast<size_t>(kSegments) * experts + kChunk);
  cudaStream_t s = as_stream(stream);
  if (chunks == 1) {
    // the single-block path writes the decode plan where the scratch pointer says
    if (plan_out != nullptr) {
      int64_t plan_need = 1 + (rows + plan_tile_rows - 1) / plan_tile_rows + experts + experts;
      LM_REQUIRE(plan_elems >= plan_need, "dispatch_static: plan_out too small for the decode plan");
      p.scratch = plan_out;
      p.scratch_elems = plan_elems;
    }
    dispatch_scatter_kernel<true><<<1, kThreads, smem, s>>>(p);
    note_launch();
  } else {
    dispatch_count_kernel<<<chunks, kThreads, 0, s>>>(p);
    note_launch();
    LM_CUDA(cudaGetLastError());
    dispatch_scatter_kernel<false><<<chunks, kThreads, smem, s>>>(p);
    note_launch();
  }
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}

extern "C" int lm_decode_prepare(const void* x, const int32_t* topk_ids, const float* topk_weights, int top_k,
                                 int experts, int features, int direct, int32_t* gather, int32_t* slots,
                                 int32_t* cu, float* probs, int32_t* padded_offsets, const float* scale_pair,
                                 uint8_t* q, uint8_t* sf, lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(x && topk_ids && topk_weights && gather && slots && cu && probs && scale_pair && q && sf,
             "decode_prepare: null pointer");
  LM_REQUIRE(direct || padded_offsets, "decode_prepare: null pointer");
  LM_REQUIRE(experts > 0 && experts <= kMaxExperts, "decode_prepare: 1..256 experts");
  LM_REQUIRE(top_k > 0 && top_k <= 32 && top_k <= experts, "decode_prepare: top_k must be 1..min(experts, 32)");
  LM_REQUIRE(features > 0 && features % 64 == 0, "decode_prepare: features must be a multiple of 64");
  OneTokenParams p{static_cast<const __nv_bfloat16*>(x), topk_ids, topk_weights, top_k, experts, features,
                   direct ? 1 : 0, gather, slots, cu, probs, padded_offsets, scale_pair, q, sf};
  const int slices = (features + 511) / 512;
  const int grid = (slices + kThreads / 32 - 1) / (kThreads / 32);
  decode_prepare_one_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(p);
  note_launch();
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}

extern "C" int lm_dispatch_quantize_decode(const void* x, const int32_t* topk_ids,
                                           const float* topk_weights, int64_t tokens, int top_k,
                                           int experts, int features, int32_t* gather,
                                           int32_t* m_indptr, float* probs, int32_t* slots,
                                           int32_t* padded_offsets, int32_t* scratch,
                                           int64_t scratch_elems, int plan_tile_rows,
                                           const float* scale_pair, uint8_t* q, uint8_t* sf,
                                           lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(x && topk_ids && topk_weights && gather && m_indptr && probs && slots && padded_offsets &&
                 scratch && scale_pair && q && sf,
             "dispatch_quantize_decode: null pointer");
  LM_REQUIRE(experts > 0 && experts <= kMaxExperts, "dispatch_quantize_decode: at most 256 experts");
  LM_REQUIRE(top_k > 0 && top_k <= 32 && tokens > 0, "dispatch_quantize_decode: bad routing sizes");
  LM_REQUIRE(features > 0 && features % 64 == 0, "dispatch_quantize_decode: features must be a multiple of 64");
  LM_REQUIRE(plan_tile_rows > 0 && 128 % plan_tile_rows == 0,
             "dispatch_quantize_decode: plan_tile_rows must divide 128");
  const int64_t rows = tokens * top_k;
  if (rows > kChunk) return set_error(LM_ERR_LIMIT, "dispatch_quantize_decode: at most 1024 assignments");
  int64_t plan_need = 1 + (rows + plan_tile_rows - 1) / plan_tile_rows + experts + experts;
  LM_REQUIRE(scratch_elems >= plan_need, "dispatch_quantize_decode: scratch too small for the decode plan");
  DecodePrepareParams p{};
  p.d = DispatchParams{topk_ids, topk_weights, rows,    top_k,         experts,        gather, m_indptr,
                       probs,    slots,        padded_offsets, scratch, scratch_elems, plan_tile_rows, 1};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.features = features;
  p.scale_pair = scale_pair;
  p.q = q;
  p.sf = sf;
  const size_t smem = sizeof(int) * (static_cast<size_t>(kSegments) * experts + 2 * kChunk);
  dim3 grid(static_cast<unsigned>((tokens + kThreads / 32 - 1) / (kThreads / 32)), (features + 511) / 512);
  dispatch_quantize_decode_kernel<<<grid, kThreads, smem, as_stream(stream)>>>(p);
  note_launch();
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}
