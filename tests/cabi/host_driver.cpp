// C++ host driver of the C ABI (include/nvfp4_b200.h), built and run by tests/test_cabi_cpp_gpu.py.
//
// What a C++ caller of the reference's launchers would do, with plain CUDA runtime calls and no
// torch: the cases mirror the reference's Catch2 tests -- round-trip mean relative error of the
// block-1D quantizer below 0.3 on [128,256] and [1024,1024] inputs and zeros in, zeros out
// (fx/src/s4/nvfp4/test_quantization.cpp:86-87,111-112,250-252), a custom stream (:295-328),
// n = 0 (:347-358), GEMM against an fp32 matmul of the bf16 operands below 0.3 for 128^3 and
// 512^3 (fx/src/s4/nvfp4/test_gemm.cpp:81-82,96-97), and argument errors returned, not thrown.
// Prints one line per check; exit code 0 only if all pass.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "nvfp4_b200.h"

static int failures = 0;
#define CHECK(cond, ...)                                                  \
  do {                                                                    \
    const bool ok_ = (cond);                                              \
    std::printf("%s  ", ok_ ? "ok  " : "FAIL");                           \
    std::printf(__VA_ARGS__);                                             \
    std::printf("\n");                                                    \
    if (!ok_) ++failures;                                                 \
  } while (0)

static float bf16_to_float(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
static uint16_t float_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
// seeded normal-ish values (sum of uniforms), like the fixtures' randn * scale
static std::vector<uint16_t> make_input(int64_t n, uint32_t seed, float scale) {
  std::vector<uint16_t> v((size_t)n);
  uint32_t s = seed * 2654435761u + 12345u;
  for (int64_t i = 0; i < n; ++i) {
    float acc = 0.f;
    for (int j = 0; j < 4; ++j) {
      s = s * 1664525u + 1013904223u;
      acc += (float)(s >> 8) * (1.0f / 16777216.0f);
    }
    v[(size_t)i] = float_to_bf16((acc - 2.0f) * 1.7320508f * scale);
  }
  return v;
}
template <typename T> static T* dev_alloc(size_t n) {
  void* p = nullptr;
  if (cudaMalloc(&p, n * sizeof(T) + 16) != cudaSuccess) std::exit(3);
  return static_cast<T*>(p);
}

struct Packed {
  uint8_t *data, *scales, *scales_swz;
  float *amax, *gscale;
};
static Packed quantize(const uint16_t* x_dev, int64_t rows, int64_t cols, cudaStream_t st, int* rc_out) {
  Packed p;
  p.data = dev_alloc<uint8_t>((size_t)(rows * cols / 2));
  p.scales = dev_alloc<uint8_t>((size_t)(rows * cols / 16));
  p.scales_swz = dev_alloc<uint8_t>((size_t)nvfp4_swizzled_scale_bytes(rows, cols));
  p.amax = dev_alloc<float>(1);
  p.gscale = dev_alloc<float>(1);
  int rc = nvfp4_amax_bf16(x_dev, rows * cols, p.amax, st);
  if (rc == NVFP4_OK)
    rc = nvfp4_quantize_bf16(x_dev, rows, cols, p.amax, p.data, p.scales, p.scales_swz, p.gscale, st);
  *rc_out = rc;
  return p;
}

static float roundtrip_error(int64_t rows, int64_t cols, uint32_t seed, float scale, cudaStream_t st) {
  const int64_t n = rows * cols;
  std::vector<uint16_t> x = make_input(n, seed, scale);
  uint16_t* xd = dev_alloc<uint16_t>((size_t)n);
  cudaMemcpy(xd, x.data(), (size_t)n * 2, cudaMemcpyHostToDevice);
  int rc;
  Packed p = quantize(xd, rows, cols, st, &rc);
  if (rc != NVFP4_OK) return 1e9f;
  uint16_t* yd = dev_alloc<uint16_t>((size_t)n);
  if (nvfp4_dequantize_bf16(p.data, p.scales, rows, cols, p.amax, yd, st) != NVFP4_OK) return 1e9f;
  cudaStreamSynchronize(st);
  std::vector<uint16_t> y((size_t)n);
  cudaMemcpy(y.data(), yd, (size_t)n * 2, cudaMemcpyDeviceToHost);
  double num = 0, den = 0;
  for (int64_t i = 0; i < n; ++i) {
    num += std::fabs(bf16_to_float(y[(size_t)i]) - bf16_to_float(x[(size_t)i]));
    den += std::fabs(bf16_to_float(x[(size_t)i]));
  }
  return (float)(num / den);
}

static float gemm_error(int64_t M, int64_t N, int64_t K) {
  std::vector<uint16_t> a = make_input(M * K, 7, 0.1f), b = make_input(N * K, 8, 0.1f);
  uint16_t* ad = dev_alloc<uint16_t>((size_t)(M * K));
  uint16_t* bd = dev_alloc<uint16_t>((size_t)(N * K));
  cudaMemcpy(ad, a.data(), (size_t)(M * K) * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(bd, b.data(), (size_t)(N * K) * 2, cudaMemcpyHostToDevice);
  int rc;
  Packed pa = quantize(ad, M, K, nullptr, &rc);
  if (rc != NVFP4_OK) return 1e9f;
  Packed pb = quantize(bd, N, K, nullptr, &rc);
  if (rc != NVFP4_OK) return 1e9f;
  uint16_t* dd = dev_alloc<uint16_t>((size_t)(M * N));
  int* status = dev_alloc<int>(1);
  cudaMemset(status, 0, sizeof(int));
  rc = nvfp4_gemm(pa.data, pb.data, pa.scales_swz, pb.scales_swz, pa.gscale, pb.gscale, M, N, K, 1.0f,
                  0.0f, nullptr, nullptr, nullptr, NVFP4_ACT_NONE, dd, nullptr, status, nullptr);
  if (rc != NVFP4_OK) return 1e9f;
  cudaDeviceSynchronize();
  int st_host = -1;
  cudaMemcpy(&st_host, status, sizeof(int), cudaMemcpyDeviceToHost);
  if (st_host != 0) return 1e9f;
  std::vector<uint16_t> d((size_t)(M * N));
  cudaMemcpy(d.data(), dd, (size_t)(M * N) * 2, cudaMemcpyDeviceToHost);
  double num = 0, den = 0;
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      float acc = 0.f;
      for (int64_t k = 0; k < K; ++k) acc += bf16_to_float(a[(size_t)(m * K + k)]) * bf16_to_float(b[(size_t)(n * K + k)]);
      num += std::fabs(bf16_to_float(d[(size_t)(m * N + n)]) - acc);
      den += std::fabs(acc);
    }
  return (float)(num / den);
}

int main() {
  int major = 0, minor = 0;
  const int rc_init = nvfp4_init(0, &major, &minor);
  CHECK(rc_init == NVFP4_OK, "nvfp4_init on compute capability %d.%d -> %s", major, minor,
        nvfp4_status_string(rc_init));
  if (rc_init != NVFP4_OK) return 2;
  cudaSetDevice(0);

  float e = roundtrip_error(128, 256, 42, 1.0f, nullptr);
  CHECK(e < 0.3f, "block-1D round trip [128,256]: mean relative error %.4f < 0.3", e);
  e = roundtrip_error(1024, 1024, 42, 1.0f, nullptr);
  CHECK(e < 0.3f, "block-1D round trip [1024,1024]: mean relative error %.4f < 0.3", e);
  cudaStream_t st;
  cudaStreamCreate(&st);
  e = roundtrip_error(64, 128, 123, 10.0f, st);
  CHECK(e < 0.3f, "round trip on a caller's stream: %.4f < 0.3", e);

  {  // zeros in, zeros out
    const int64_t n = 64 * 64;
    uint16_t* xd = dev_alloc<uint16_t>((size_t)n);
    cudaMemset(xd, 0, (size_t)n * 2);
    int rc;
    Packed p = quantize(xd, 64, 64, nullptr, &rc);
    uint16_t* yd = dev_alloc<uint16_t>((size_t)n);
    rc = rc == NVFP4_OK ? nvfp4_dequantize_bf16(p.data, p.scales, 64, 64, p.amax, yd, nullptr) : rc;
    cudaDeviceSynchronize();
    std::vector<uint16_t> y((size_t)n);
    cudaMemcpy(y.data(), yd, (size_t)n * 2, cudaMemcpyDeviceToHost);
    float worst = 0.f;
    for (uint16_t h : y) worst = std::fmax(worst, std::fabs(bf16_to_float(h)));
    CHECK(rc == NVFP4_OK && worst < 1e-6f, "zeros stay zeros (max |out| %.2g)", worst);
  }

  // empty input is a no-op; bad arguments come back as status codes
  CHECK(nvfp4_quantize_bf16(nullptr, 0, 64, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr) == NVFP4_OK,
        "n = 0 is accepted");
  CHECK(nvfp4_quantize_bf16(nullptr, 4, 24, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr) ==
            NVFP4_ERR_BAD_ARG, "cols %% 16 != 0 -> bad argument");
  CHECK(nvfp4_gemm(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 8, 12, 64, 1.f, 0.f, nullptr,
                   nullptr, nullptr, 0, nullptr, nullptr, nullptr, nullptr) == NVFP4_ERR_BAD_ARG,
        "GEMM with N %% 8 != 0 -> bad argument");

  e = gemm_error(128, 128, 128);
  CHECK(e < 0.3f, "GEMM 128^3 vs fp32 matmul of the bf16 operands: %.4f < 0.3", e);
  e = gemm_error(512, 512, 512);
  CHECK(e < 0.3f, "GEMM 512^3: %.4f < 0.3", e);
  e = gemm_error(100, 200, 96);     // the reference needs multiples of 128 here (kernel.cu:39)
  CHECK(e < 0.3f, "GEMM 100x200x96 (no padding needed): %.4f < 0.3", e);

  std::printf("%d failure(s)\n", failures);
  return failures == 0 ? 0 : 1;
}
