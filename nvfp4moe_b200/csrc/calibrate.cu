// Calibration helper: the largest post-activation magnitude of a first-projection result.
//
// The hidden-activation scale of a layer is amax(act(fc1 output)) / 2688.  The fc1 result of the
// calibration batch is kept as BF16 (rows x N, gate/up interleaved for the gated activations);
// this kernel applies the activation in FP32 with exact exp / tanh and reduces |value| to one
// float, so the host needs neither FP32 copies of the matrix nor a synchronisation.
#include "common.cuh"

namespace lm {
namespace {

constexpr int kThreads = 256;

struct AmaxParams {
  const __nv_bfloat16* preact;
  int64_t elements;  // rows * n
  int activation;
  float clamp_limit;
  float sigmoid_alpha;
  float up_bias;
  float* out;  // non-negative floats order like their bit patterns: atomicMax on the bits
};

__device__ __forceinline__ float post_activation(float g, float u, const AmaxParams& p) {
  if (p.activation == LM_ACT_RELU2) {
    const float x = fmaxf(g, 0.0f);
    return x * x;
  }
  if (p.clamp_limit > 0.0f) {
    g = fminf(g, p.clamp_limit);
    u = fmaxf(fminf(u, p.clamp_limit), -p.clamp_limit);
  }
  switch (p.activation) {
    case LM_ACT_SWIGLU:
    case LM_ACT_SWIGLU_OAI:
      return g * (1.0f / (1.0f + expf(-p.sigmoid_alpha * g))) * (u + p.up_bias);
    case LM_ACT_GEGLU: {
      const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
      return 0.5f * g * (1.0f + tanhf(inner)) * u;
    }
    default:  // reglu
      return fmaxf(g, 0.0f) * u;
  }
}

__global__ void __launch_bounds__(kThreads) activation_amax_kernel(AmaxParams p) {
  // eight BF16 values (four gate/up pairs, or eight unary inputs) per thread and step
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads * 8;
  float best = 0.0f;
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) * 8; i < p.elements; i += stride) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p.preact + i));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
      if (p.activation == LM_ACT_RELU2) {
        best = fmaxf(best, fmaxf(post_activation(lo, 0.0f, p), post_activation(hi, 0.0f, p)));
      } else {
        best = fmaxf(best, fabsf(post_activation(lo, hi, p)));
      }
    }
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) best = fmaxf(best, __shfl_xor_sync(0xFFFFFFFFu, best, d));
  __shared__ float s_best[kThreads / 32];
  if ((threadIdx.x & 31) == 0) s_best[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kThreads / 32; ++i) best = fmaxf(best, s_best[i]);
    atomicMax(reinterpret_cast<unsigned int*>(p.out), __float_as_uint(best));
  }
}

}  // namespace
}  // namespace lm

extern "C" int lm_activation_amax(const void* preact, int64_t rows, int n, int activation, float clamp_limit,
                                  float sigmoid_alpha, float up_bias, float* out, lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(preact && out, "activation_amax: null pointer");
  LM_REQUIRE(activation >= LM_ACT_SWIGLU && activation <= LM_ACT_RELU2, "activation_amax: unknown activation");
  LM_REQUIRE(rows >= 0 && n > 0 && n % 8 == 0, "activation_amax: N must be a multiple of 8");
  LM_REQUIRE((reinterpret_cast<uintptr_t>(preact) & 15) == 0, "activation_amax: the matrix must be 16-byte aligned");
  LM_CUDA(cudaMemsetAsync(out, 0, sizeof(float), as_stream(stream)));
  if (rows == 0) return LM_OK;
  AmaxParams p{static_cast<const __nv_bfloat16*>(preact), rows * n, activation, clamp_limit, sigmoid_alpha,
               up_bias, out};
  const int64_t steps = (p.elements / 8 + kThreads - 1) / kThreads;
  const int sms = sm_count();
  const int grid = static_cast<int>(steps < 8ll * sms ? (steps > 0 ? steps : 1) : 8ll * sms);
  activation_amax_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(p);
  note_launch();
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}
