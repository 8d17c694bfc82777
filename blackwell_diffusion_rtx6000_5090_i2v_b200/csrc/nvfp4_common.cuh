// Shared device/host helpers for the sm_100a NVFP4 kernels.
#pragma once

#include <cfloat>
#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../../include/nvfp4_b200.h"

namespace nvfp4 {

constexpr int kBlock = 16;          // elements per scale block
constexpr int kSfAtomBytes = 512;   // 128 rows x 4 K-blocks
constexpr int kSfRowPad = 256;      // swizzled scale rows are padded to this
constexpr int kSfKbPad = 16;        // and K-blocks to this (= 256 elements)

// 128-row tiles and 4-block K atoms of the swizzled scale buffer.
__host__ __device__ inline int64_t sf_row_tiles(int64_t rows) {
  return (rows + kSfRowPad - 1) / kSfRowPad * (kSfRowPad / 128);
}
__host__ __device__ inline int64_t sf_k_atoms(int64_t cols) {
  return ((cols / kBlock) + kSfKbPad - 1) / kSfKbPad * (kSfKbPad / 4);
}
__host__ __device__ inline int64_t sf_swizzled_bytes(int64_t rows, int64_t cols) {
  return sf_row_tiles(rows) * sf_k_atoms(cols) * kSfAtomBytes;
}
// Byte offset of the scale of (row, K-block kb): atoms are [row tile][k atom],
// each atom is [32 rows][4 row groups][4 K-blocks].
__host__ __device__ inline int64_t sf_swizzled_offset(int64_t row, int64_t kb, int64_t k_atoms) {
  return ((row >> 7) * k_atoms + (kb >> 2)) * kSfAtomBytes + (row & 31) * 16 +
         ((row >> 5) & 3) * 4 + (kb & 3);
}

#ifdef __CUDACC__

// S_enc = min(448*6/amax, FLT_MAX); 1 when amax == 0 or the result is 0.
// IEEE division: the value must match the CPU restatement bit for bit.
__device__ __forceinline__ float global_encode_scale(float amax) {
  float s = __fdiv_rn(448.0f * 6.0f, amax);
  s = fminf(s, FLT_MAX);
  if (amax == 0.0f || s == 0.0f) return 1.0f;
  return s;
}

// x / 6, bit-identical to the IEEE quotient: one multiply by fl(1/6) and one residual
// correction (two FMAs).  The residual of a tiny quotient is itself inexact and that of an
// infinite one is NaN, so very small, very large and non-finite x take the division.  Checked
// against x / 6.0f for every bf16 x in the fast range and two million fp32 values.
__device__ __forceinline__ float div_by_6(float x) {
  const float c = 0x1.555556p-3f;
  const float q0 = __fmul_rn(x, c);
  const float q = __fmaf_rn(__fmaf_rn(-6.0f, q0, x), c, q0);
  return (x >= 1e-30f && x <= 1e37f) ? q : __fdiv_rn(x, 6.0f);
}

// E4M3 block scale: rn_satfinite( min( (amax_b / 6) * S_enc, FLT_MAX ) ).
__device__ __forceinline__ uint8_t block_scale_e4m3(float amax_b, float s_enc) {
  float d = __fmul_rn(__fdiv_rn(amax_b, 6.0f), s_enc);
  d = fminf(d, FLT_MAX);
  return (uint8_t)__nv_cvt_float_to_fp8(d, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(__half(h));
}

// Element encode scale: min( 1 / (float(sf) * (1/S_enc)), FLT_MAX ).
__device__ __forceinline__ float block_encode_scale(uint8_t sf, float s_dec) {
  return fminf(__fdiv_rn(1.0f, __fmul_rn(e4m3_to_f32(sf), s_dec)), FLT_MAX);
}

// Eight floats -> eight E2M1 codes in one 32-bit word, element 0 in the low
// nibble of byte 0 (round to nearest even, saturate to +-6).
__device__ __forceinline__ uint32_t f32x8_to_e2m1x8(float v0, float v1, float v2, float v3,
                                                    float v4, float v5, float v6, float v7) {
  uint32_t out;
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t"
      "}"
      : "=r"(out)
      : "f"(v0), "f"(v1), "f"(v2), "f"(v3), "f"(v4), "f"(v5), "f"(v6), "f"(v7));
  return out;
}

__device__ __forceinline__ float bf16lo_to_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t w) {
  return __uint_as_float(w & 0xFFFF0000u);
}

// Two fp32 lanes per instruction (sm_100): each lane is rounded exactly like the scalar
// op, the pair costs one issue slot.
__device__ __forceinline__ float2 f2_add(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 f2_sub(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "sub.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 f2_mul(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 f2_fma(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\tfma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 bf16x2_to_f2(uint32_t w) {
  return make_float2(bf16lo_to_f32(w), bf16hi_to_f32(w));
}
// (lo, hi) -> packed bf16x2, round to nearest even: one instruction for the pair
__device__ __forceinline__ uint32_t f2_to_bf16x2(float2 v) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(v.y), "f"(v.x));
  return d;
}
// max(acc, |v|) per bf16 lane (inputs finite)
__device__ __forceinline__ uint32_t bf16x2_max_abs(uint32_t acc, uint32_t v) {
  uint32_t d;
  asm("{\n\t.reg .b32 t;\n\tabs.bf16x2 t, %2;\n\tmax.bf16x2 %0, %1, t;\n\t}"
      : "=r"(d) : "r"(acc), "r"(v));
  return d;
}

#endif  // __CUDACC__

// Host helpers shared by the entry points.
int check_device_sm100();                 // NVFP4_OK or NVFP4_ERR_UNSUPPORTED_ARCH (cached per device)
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int sm_count();                           // SMs of the current device (cached per device)

}  // namespace nvfp4
