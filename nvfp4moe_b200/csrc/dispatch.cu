// Stable expert-major dispatch of (token, route) pairs: a counting sort with
// no data-dependent atomics in the placement, so the permutation is bit-stable.
//
// rows <= 1024: one CTA ranks, scans and scatters, and also writes the decode
//               tile plan.
// rows  > 1024: kernel 1 counts pairs per (1024-pair chunk, expert); kernel 2
//               gives each chunk its stable base (prefix over experts, then over
//               earlier chunks) and scatters.
#include "common.cuh"

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

template <bool kSingle>
__global__ void __launch_bounds__(kThreads) dispatch_scatter_kernel(DispatchParams p) {
  extern __shared__ int s_dyn[];
  int* s_seg = s_dyn;                        // [kSegments][experts]
  int* s_chunk = s_seg + kSegments * p.experts;  // [kChunk]
  __shared__ int s_base[kMaxExperts];
  __shared__ int s_warp[3][kThreads / 32];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int chunk = blockIdx.x;
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
#pragma unroll 8
      for (int b = 0; b < p.chunks; ++b) {
        int c = __ldg(p.scratch + static_cast<int64_t>(b) * E + tid);
        total += c;
        if (b < chunk) before += c;
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
    if (chunk == 0) {
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
    if (pos < p.rows && e < 0) p.slots[pos] = -1;  // dropped pair: the combine skips it
    if (pos < p.rows && e >= 0) {
      int dst = s_base[e] + s_seg[(i * (kThreads / 32) + warp) * E + e] + rank[i];
      p.gather[dst] = static_cast<int32_t>(pos / p.top_k);
      p.probs[dst] = __ldg(p.weights + pos);
      p.slots[pos] = dst;
    }
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
  static int32_t* cached[64] = {nullptr};
  int device = 0;
  LM_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= 64) return set_error(LM_ERR_LIMIT, "dispatch_static: device index out of range");
  if (cached[device] == nullptr) {
    int32_t* ptr = nullptr;
    LM_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch));
    cached[device] = ptr;
  }
  *out = cached[device];
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
  } else {
    LM_REQUIRE(scratch_elems >= static_cast<int64_t>(chunks) * experts, "dispatch: scratch too small");
    dispatch_count_kernel<<<chunks, kThreads, 0, s>>>(p);
    LM_CUDA(cudaGetLastError());
    dispatch_scatter_kernel<false><<<chunks, kThreads, smem, s>>>(p);
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
  } else {
    dispatch_count_kernel<<<chunks, kThreads, 0, s>>>(p);
    LM_CUDA(cudaGetLastError());
    dispatch_scatter_kernel<false><<<chunks, kThreads, smem, s>>>(p);
  }
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}
