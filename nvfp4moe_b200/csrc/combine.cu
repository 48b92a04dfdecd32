// Deterministic top-k combine (HBM-bound gather-reduce).
//
// One thread owns eight BF16 columns (16 bytes) of one token: it loads the
// token's rows eight routes at a time, adds them in route order to an FP32 sum in
// registers and stores the BF16 result once.  The product with the routing weight is rounded before the
// add (mul.rn then add.rn, never fused), so the result is independent of the
// launch shape and bit-identical from run to run.
#include "common.cuh"

namespace lm {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxTopK = 32;

struct CombineParams {
  const __nv_bfloat16* rows;
  const int32_t* slots;
  const float* weights;
  __nv_bfloat16* out;
  int64_t tokens;
  int top_k;
  int hidden;
  int64_t row_stride;
  int64_t out_stride;
  int vec_per_row;
  const int32_t* valid;  // optional: 0 = the rows were not computed this step, write zeros
};

template <bool kWeighted>
__global__ void __launch_bounds__(kThreads) combine_kernel(CombineParams p) {
  // As a programmatic dependent the kernel may start while its predecessor drains.  The routed
  // rows are that kernel's output and are read after the wait below; slots and weights are older
  // (the dispatch wrote them before the GEMMs began) and are read while it still runs.
  const int64_t token = blockIdx.x;
  const int vec = blockIdx.y * kThreads + threadIdx.x;
  if (vec >= p.vec_per_row) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    return;
  }
  const bool live = p.valid == nullptr || __ldg(p.valid) != 0;
  const int col = vec * 8;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

  const int32_t* slot_ptr = p.slots + token * p.top_k;
  // Eight routes at a time: their slots, then their rows and weights, are loaded together and
  // summed in route order afterwards, so a token costs two memory round trips per eight routes
  // instead of two per route (a decode step is a handful of tokens: nothing else hides them).
  constexpr int kBatch = 8;
  for (int j0 = 0; j0 < p.top_k; j0 += kBatch) {
    int slot[kBatch];
    uint4 row[kBatch];
    float w[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) slot[j] = (live && j0 + j < p.top_k) ? __ldg(slot_ptr + j0 + j) : -1;
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      w[j] = 0.0f;
      if (kWeighted && slot[j] >= 0) w[j] = __ldg(p.weights + slot[j]);
    }
    if (j0 == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
    // Plain loads in volatile asm, not __ldg: a load the compiler knows as invariant may be
    // hoisted above the wait now that its address (the slot) is known before it, and would
    // then read rows the previous kernel has not written yet.
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      row[j] = make_uint4(0, 0, 0, 0);
      if (slot[j] >= 0)
        asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(row[j].x), "=r"(row[j].y), "=r"(row[j].z), "=r"(row[j].w)
                     : "l"(p.rows + slot[j] * p.row_stride + col)
                     : "memory");
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (slot[j] < 0) continue;
      const uint32_t words[4] = {row[j].x, row[j].y, row[j].z, row[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float lo = __uint_as_float(words[i] << 16);
        float hi = __uint_as_float(words[i] & 0xFFFF0000u);
        if (kWeighted) {
          lo = __fmul_rn(lo, w[j]);
          hi = __fmul_rn(hi, w[j]);
        }
        acc[2 * i] = __fadd_rn(acc[2 * i], lo);
        acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], hi);
      }
    }
  }
  uint4 packed;
  uint32_t* pw = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    pw[i] = *reinterpret_cast<uint32_t*>(&v);
  }
  *reinterpret_cast<uint4*>(p.out + token * p.out_stride + col) = packed;
}

}  // namespace
}  // namespace lm

extern "C" int lm_finalize(const void* routed_out, const int32_t* slots, const float* weights,
                           void* out, int64_t tokens, int top_k, int hidden,
                           int64_t routed_row_stride, int64_t out_row_stride, const int32_t* valid,
                           int use_pdl, lm_stream_t stream) {
  using namespace lm;
  LM_REQUIRE(routed_out && slots && out, "finalize: null pointer");
  LM_REQUIRE(hidden > 0 && hidden % 8 == 0, "finalize: hidden must be a multiple of 8");
  LM_REQUIRE(routed_row_stride % 8 == 0 && out_row_stride % 8 == 0,
             "finalize: row strides must keep 16-byte alignment");
  LM_REQUIRE(top_k > 0 && top_k <= kMaxTopK, "finalize: top_k must be in 1..32");
  LM_REQUIRE(tokens >= 0 && tokens < (1ll << 31), "finalize: bad token count");
  if (tokens == 0) return LM_OK;
  CombineParams p{static_cast<const __nv_bfloat16*>(routed_out), slots, weights,
                  static_cast<__nv_bfloat16*>(out), tokens, top_k, hidden,
                  routed_row_stride, out_row_stride, hidden / 8, valid};
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(tokens), (p.vec_per_row + kThreads - 1) / kThreads);
  config.blockDim = dim3(kThreads);
  config.stream = as_stream(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = use_pdl ? 1 : 0;
  if (weights != nullptr) {
    LM_CUDA(cudaLaunchKernelEx(&config, combine_kernel<true>, p));
  } else {
    LM_CUDA(cudaLaunchKernelEx(&config, combine_kernel<false>, p));
  }
  note_launch();
  LM_CUDA(cudaGetLastError());
  return LM_OK;
}
