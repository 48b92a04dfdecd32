// Per-group NVFP4 quantization math shared by the row-wise quantizer and the fused
// decode dispatch + quantize kernel.
#pragma once

#include "common.cuh"

namespace lm {

// Sixteen consecutive inputs of one row, kept as loaded (8 registers for BF16).
template <typename In>
struct Slice;

template <>
struct Slice<__nv_bfloat16> {
  static constexpr int kUnroll = 4;
  uint32_t w[8];
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    const uint4* src = reinterpret_cast<const uint4*>(p);
    uint4 a = __ldg(src);
    uint4 b = __ldg(src + 1);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
  }
  // max |x|: comparisons in BF16 pick one of the inputs unchanged, so the result is exact
  __device__ __forceinline__ float amax() const {
    uint32_t m[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = w[i] & 0x7FFF7FFFu;
#pragma unroll
    for (int d = 4; d >= 1; d >>= 1)
#pragma unroll
      for (int i = 0; i < d; ++i)
        asm("max.bf16x2 %0, %1, %2;" : "=r"(m[i]) : "r"(m[i]), "r"(m[i + d]));
    return fmaxf(__uint_as_float(m[0] << 16), __uint_as_float(m[0] & 0xFFFF0000u));
  }
  __device__ __forceinline__ float lo(int pair) const { return __uint_as_float(w[pair] << 16); }
  __device__ __forceinline__ float hi(int pair) const { return __uint_as_float(w[pair] & 0xFFFF0000u); }
};

template <>
struct Slice<float> {
  static constexpr int kUnroll = 2;
  float v[16];
  __device__ __forceinline__ void load(const float* p) {
    const float4* src = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 t = __ldg(src + i);
      v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
  }
  __device__ __forceinline__ float amax() const {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
    return m;
  }
  __device__ __forceinline__ float lo(int pair) const { return v[2 * pair]; }
  __device__ __forceinline__ float hi(int pair) const { return v[2 * pair + 1]; }
};

// Quantize one 16-element group.  Returns the scale-factor byte; writes the
// eight packed bytes to `packed`.
template <typename In>
__device__ __forceinline__ uint32_t quantize_group(const Slice<In>& x, float pts, float inv_pts,
                                                   bool te_math, uint2* packed) {
  const float amax = x.amax();
  float scaled;
  if (te_math) {
    scaled = __fmul_rn(amax, __fmul_rn(inv_pts, inv6()));
  } else {
    scaled = __fdiv_rn(__fdiv_rn(amax, kF4Max), pts);
  }
  scaled = fmaxf(fminf(scaled, kE4M3Max), kE4M3MinSf);
  uint32_t sf_byte = f32_to_e4m3(scaled);
  float sf_value = e4m3_to_f32(sf_byte);
  float factor = te_math ? __fdiv_rn(1.0f, __fmul_rn(sf_value, pts)) : __fdiv_rn(inv_pts, sf_value);
  float s[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s[2 * i] = __fmul_rn(x.lo(i), factor);
    s[2 * i + 1] = __fmul_rn(x.hi(i), factor);
  }
  packed->x = f32x8_to_e2m1(s);
  packed->y = f32x8_to_e2m1(s + 8);
  return sf_byte;
}

}  // namespace lm
