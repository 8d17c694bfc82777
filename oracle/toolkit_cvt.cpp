// TEST INFRASTRUCTURE ONLY.  Host-side wrappers over the CUDA toolkit's own
// software converters (cuda_fp8.h, cuda_fp4.h).  The reference casts block
// scales through __nv_fp8_e4m3 (fx/src/s4/nvfp4/quantization_te.cu:51) and
// names the E2M1 conversion of cuda_fp4.h (quantization_te_clean.cu:66-85);
// the oracle's hand-written converters are checked exhaustively against
// these.  Built by oracle/Makefile; no GPU is needed to call them.
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cstdint>

extern "C" {

uint8_t tk_f32_to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

float tk_e4m3_to_f32(uint8_t b) {
  __nv_fp8_e4m3 v;
  v.__x = b;
  return static_cast<float>(v);
}

uint8_t tk_f32_to_e2m1(float x) {
  return (uint8_t)__nv_cvt_float_to_fp4(x, __NV_E2M1, cudaRoundNearest);
}

// {x -> low nibble, y -> high nibble}
uint8_t tk_f32x2_to_e2m1x2(float x, float y) {
  float2 v;
  v.x = x;
  v.y = y;
  return (uint8_t)__nv_cvt_float2_to_fp4x2(v, __NV_E2M1, cudaRoundNearest);
}

void tk_f32_to_e4m3_many(const float* x, uint8_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = tk_f32_to_e4m3(x[i]);
}

void tk_f32_to_e2m1_many(const float* x, uint8_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = tk_f32_to_e2m1(x[i]);
}
}
