// Shared helpers of the sm_100a NVFP4 kernels: error reporting, format
// conversions and the scale-factor atom addressing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/lightmoe_b200.h"

namespace lm {

// ---------------------------------------------------------------- host errors
int set_error(int code, const char* fmt, ...);

#define LM_REQUIRE(cond, ...)                                   \
  do {                                                          \
    if (!(cond)) return lm::set_error(LM_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define LM_CUDA(call)                                                          \
  do {                                                                         \
    cudaError_t err__ = (call);                                                \
    if (err__ != cudaSuccess)                                                  \
      return lm::set_error(LM_ERR_CUDA, "%s failed: %s", #call,                \
                           cudaGetErrorString(err__));                         \
  } while (0)

inline cudaStream_t as_stream(lm_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

int sm_count();
// Counts one kernel launch of this library (lm_launch_count reports the total).
void note_launch();
// status word of the expert-parallel kernels (expert_parallel.cu)
int ep_status_read(uint32_t* out);
int ep_status_clear();

// ------------------------------------------------------------- device helpers
constexpr float kF4Max = 6.0f;
constexpr float kE4M3Max = 448.0f;
constexpr float kE4M3MinSf = 0.001953125f;  // 2^-9
constexpr float kFltMax = 3.4028234663852886e38f;

// 1/6 rounded to FP32, as the reference's multiply chain uses it.
__device__ __forceinline__ float inv6() { return __fdiv_rn(1.0f, 6.0f); }

// FP32 -> E4M3 byte, round-to-nearest-even, saturating to +-448.
__device__ __forceinline__ uint32_t f32_to_e4m3(float v) {
  uint16_t packed;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(0.0f), "f"(v));
  return packed & 0xFFu;
}

// E4M3 byte -> FP32 (exact).
__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
  uint32_t h2;
  asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}"
      : "=r"(h2)
      : "r"(byte & 0xFFu));
  __half lo = __ushort_as_half(static_cast<unsigned short>(h2 & 0xFFFFu));
  return __half2float(lo);
}

// Two FP32 -> one byte of E2M1 codes (lo in the low nibble), RN-even, saturating.
__device__ __forceinline__ uint32_t f32x2_to_e2m1(float lo, float hi) {
  uint32_t out;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}"
      : "=r"(out)
      : "f"(hi), "f"(lo));
  return out;
}

// Eight FP32 -> 32 bits of E2M1 codes (v[0] in the lowest nibble): four conversions whose
// bytes are packed by one register move.
__device__ __forceinline__ uint32_t f32x8_to_e2m1(const float* v) {
  uint32_t out;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(out)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return out;
}

// Byte offset of (row, k_group) inside a scale-factor buffer whose atom rows
// have `atom_cols` = K/64 atoms; `atom_row` is the 128-row tile index.
__device__ __forceinline__ int64_t sf_offset(int64_t atom_row, int atom_cols, int row_in_tile,
                                             int k_group) {
  return (atom_row * atom_cols + (k_group >> 2)) * 512 + (row_in_tile & 31) * 16 +
         ((row_in_tile >> 5) & 3) * 4 + (k_group & 3);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

}  // namespace lm
