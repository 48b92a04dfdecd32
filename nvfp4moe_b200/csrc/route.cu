// Router step in front of the dispatch: softmax over the experts, top-k, renormalise.
//
// One warp per token.  Each lane keeps experts lane, lane+32, ... in registers (at most eight:
// experts <= 256); the k winners are picked by k rounds of a warp arg-max (larger probability
// first, lower expert id on a tie: the order torch.topk returns for distinct values).  The
// weight of winner i is exp(l_i - max) / sum over the winners of exp(l_j - max): the softmax
// denominator cancels in the renormalisation, so it is never formed.
#include "common.cuh"

namespace lm {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kPerLane = 8;

struct RouteParams {
  const void* logits;  // (tokens, experts) FP32 or BF16
  int64_t tokens;
  int experts;
  int top_k;
  int32_t* ids;        // (tokens, top_k)
  float* weights;      // (tokens, top_k)
};

template <typename In>
__device__ __forceinline__ float load_logit(const In* p);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p) {
  return __ldg(p);
}
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

template <typename In>
__global__ void __launch_bounds__(kThreads) route_topk_kernel(RouteParams p) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t token = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (token >= p.tokens) return;
  const In* row = static_cast<const In*>(p.logits) + token * p.experts;
  float v[kPerLane];
  float best = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < p.experts ? load_logit<In>(row + e) : -INFINITY;
    best = fmaxf(best, v[i]);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) best = fmaxf(best, __shfl_xor_sync(0xFFFFFFFFu, best, d));
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) v[i] = lane + 32 * i < p.experts ? expf(v[i] - best) : -1.0f;

  float sum = 0.0f;
  float my_value = 0.0f;  // lane j keeps winner j
  int my_id = 0;
  for (int j = 0; j < p.top_k; ++j) {
    // this lane's best remaining expert
    float cand = -1.0f;
    int cand_i = 0;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i)
      if (v[i] > cand) {  // strict: the lower expert id wins a tie inside the lane
        cand = v[i];
        cand_i = i;
      }
    int cand_e = lane + 32 * cand_i;
    float top = cand;
    int top_e = cand_e;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float other = __shfl_xor_sync(0xFFFFFFFFu, top, d);
      const int other_e = __shfl_xor_sync(0xFFFFFFFFu, top_e, d);
      if (other > top || (other == top && other_e < top_e)) {
        top = other;
        top_e = other_e;
      }
    }
    if (top_e == cand_e) {  // the owner retires the winner
#pragma unroll
      for (int i = 0; i < kPerLane; ++i)
        if (i == cand_i) v[i] = -1.0f;
    }
    sum += top;
    if (lane == j) {
      my_value = top;
      my_id = top_e;
    }
  }
  if (lane < p.top_k) {
    p.ids[token * p.top_k + lane] = my_id;
    p.weights[token * p.top_k + lane] = __fdiv_rn(my_value, sum);
  }
}

}  // namespace
}  // namespace lm

extern "C" int lm_route_topk(const void* logits, int logits_dtype, int64_t tokens, int experts, int top_k,
                             int32_t* topk_ids, float* topk_weights, lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(logits && topk_ids && topk_weights, "route_topk: null pointer");
  LM_REQUIRE(logits_dtype == LM_DTYPE_BF16 || logits_dtype == LM_DTYPE_F32, "route_topk: logits must be BF16 or FP32");
  LM_REQUIRE(experts > 0 && experts <= 32 * kPerLane, "route_topk: 1..256 experts");
  LM_REQUIRE(top_k > 0 && top_k <= 32 && top_k <= experts, "route_topk: top_k must be in 1..min(32, experts)");
  LM_REQUIRE(tokens >= 0, "route_topk: negative token count");
  if (tokens == 0) return LM_OK;
  RouteParams p{logits, tokens, experts, top_k, topk_ids, topk_weights};
  const unsigned grid = static_cast<unsigned>((tokens + kWarps - 1) / kWarps);
  if (logits_dtype == LM_DTYPE_F32) {
    route_topk_kernel<float><<<grid, kThreads, 0, as_stream(stream)>>>(p);
    note_launch();
  } else {
    route_topk_kernel<__nv_bfloat16><<<grid, kThreads, 0, as_stream(stream)>>>(p);
    note_launch();
  }
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}
