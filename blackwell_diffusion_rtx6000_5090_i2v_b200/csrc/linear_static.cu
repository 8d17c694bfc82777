// A whole NVFP4 linear (quantize the bf16 activation, block-scaled FP4 GEMM,
// fused bias / activation) that allocates nothing, for callers that cannot.
//
// The other entry points leave intermediate storage to the caller: the packed
// activation, its swizzled scales, the amax slot and the tensor scale are
// device buffers the caller allocates.  Some callers have no allocator to ask:
// code running inside a stream capture or another region where cudaMalloc is
// forbidden, real-time loops with a fixed memory budget, plug-ins that only
// receive input and output pointers from their host application.  For them the
// intermediates live in a fixed device array inside this library.
#include <mutex>

#include "nvfp4_common.cuh"

namespace nvfp4 {

// Largest activation the fixed scratch holds: 8 Mi elements (for example 2048 tokens of
// width 4096).  Footprint on every GPU that loads the library: 4 MiB of packed nibbles,
// 1 MiB of swizzled scales (room for row/K padding) and two fp32 slots.
constexpr int64_t kMaxElems = 8ll << 20;
constexpr int64_t kPackedBytes = kMaxElems / 2;
constexpr int64_t kScaleBytes = 2 * (kMaxElems / kBlock);
constexpr int64_t kSlotOffset = kPackedBytes + kScaleBytes;   // amax at +0, tensor scale at +4
constexpr int64_t kScratchBytes = kSlotOffset + 256;

// In host code this name is only a handle for cudaGetSymbolAddress, not a device address.
static __device__ __align__(256) uint8_t g_linear_scratch[kScratchBytes];

// Keeps the array in the module although no shipped kernel names it (never launched).
__global__ void linear_scratch_anchor(uint8_t* out) {
  if (out) *out = g_linear_scratch[0];
}

namespace {

std::mutex g_mu;
uint8_t* g_scratch_ptr[64];   // per device ordinal, resolved on first use

// Device address of the scratch array on the current device (null on failure).
uint8_t* scratch_for_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_linear_scratch) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    g_scratch_ptr[dev] = static_cast<uint8_t*>(p);
  }
  return g_scratch_ptr[dev];
}

}  // namespace
}  // namespace nvfp4

using namespace nvfp4;

extern "C" {

int64_t nvfp4_linear_bf16_static_max_elements(void) { return kMaxElems; }

int nvfp4_linear_bf16_static(const void* x_bf16, int64_t M, int64_t K, const uint8_t* w_packed,
                             const uint8_t* w_scales_swizzled, const float* w_global_scale_dev,
                             int64_t N, const void* bias_bf16, int act, void* y_bf16,
                             int* status_dev, void* stream) {
  if (M < 0 || K < 0 || N < 0 || K % 32 != 0 || N % 8 != 0) return NVFP4_ERR_BAD_ARG;
  // each extent on its own first, so that the products below cannot wrap
  if (M > kMaxElems || K > kMaxElems || N > (1 << 30)) return NVFP4_ERR_BAD_ARG;
  // The fixed scratch bounds the activation: M*K elements of nibbles, and the swizzled
  // scales, whose rows pad to 256 and K to 256 elements (so a very skinny activation can
  // exceed the scale area well below the element limit).  Larger problems must use the
  // caller-allocated path.
  if (M * K > kMaxElems || sf_swizzled_bytes(M, K) > kScaleBytes) return NVFP4_ERR_BAD_ARG;
  if (M == 0 || N == 0) return NVFP4_OK;
  if (K == 0 || !x_bf16 || !w_packed || !w_scales_swizzled || !y_bf16) return NVFP4_ERR_BAD_ARG;
  int rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
  uint8_t* s = scratch_for_current_device();
  if (!s) return NVFP4_ERR_LAUNCH_FAILED;
  uint8_t* packed = s;
  uint8_t* scales = s + kPackedBytes;
  float* amax = reinterpret_cast<float*>(s + kSlotOffset);
  float* gscale = amax + 1;
  // amax zeroes its slot and quantize zeroes the scale padding: nothing of the previous
  // call's contents is read
  rc = nvfp4_amax_bf16(x_bf16, M * K, amax, stream);
  if (rc != NVFP4_OK) return rc;
  rc = nvfp4_quantize_bf16(x_bf16, M, K, amax, packed, nullptr, scales, gscale, stream);
  if (rc != NVFP4_OK) return rc;
  return nvfp4_gemm(packed, w_packed, scales, w_scales_swizzled, gscale, w_global_scale_dev, M, N,
                    K, 1.0f, 0.0f, nullptr, bias_bf16, nullptr, act, y_bf16, nullptr, status_dev, stream);
}

}  // extern "C"
