// NVFP4 quantizer family for sm_100a: tensor amax, bf16 -> (E2M1 nibbles,
// E4M3 block scales, FP32 tensor scale), dequantize, scale re-layout.
//
// All kernels are HBM-bound byte movers: 128-bit loads, one 16-element scale
// block per thread so that the block amax needs no cross-lane traffic, and
// 64-bit packed stores.  Algorithmic bytes per element: 2 (bf16 in) + 0.5
// (nibbles) + 0.0625 (scale) = 2.5625.
#include "nvfp4_common.cuh"

namespace nvfp4 {

namespace {

constexpr int kThreads = 256;
constexpr int kBlocksPerThread = 2;  // two 16-element scale blocks (64 B of input) per thread

// ---------------------------------------------------------------- amax ----

__global__ void __launch_bounds__(kThreads) amax_bf16_kernel(const uint4* __restrict__ x,
                                                             int64_t n_vec,
                                                             const __nv_bfloat16* __restrict__ tail,
                                                             int n_tail, unsigned* __restrict__ out) {
  __nv_bfloat162 m2[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) m2[j] = __nv_bfloat162(__float2bfloat16(0.f), __float2bfloat16(0.f));
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  // four independent 16-byte loads in flight per thread
  for (; i + 3 * stride < n_vec; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __ldg(x + i + j * stride);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
      for (int k = 0; k < 4; ++k) m2[k] = __hmax2(m2[k], __habs2(p[k]));
    }
  }
  for (; i < n_vec; i += stride) {
    uint4 v = __ldg(x + i);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) m2[k] = __hmax2(m2[k], __habs2(p[k]));
  }
  __nv_bfloat162 m = __hmax2(__hmax2(m2[0], m2[1]), __hmax2(m2[2], m2[3]));
  float a = fmaxf(__bfloat162float(m.x), __bfloat162float(m.y));
  if (blockIdx.x == 0 && threadIdx.x < n_tail)
    a = fmaxf(a, fabsf(__bfloat162float(tail[threadIdx.x])));
  // non-negative floats order like their bit patterns
  unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(a));
  __shared__ unsigned warp_max[kThreads / 32];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = bits;
  __syncthreads();
  if (threadIdx.x < 32) {
    unsigned b = threadIdx.x < kThreads / 32 ? warp_max[threadIdx.x] : 0u;
    b = __reduce_max_sync(0xffffffffu, b);
    if (threadIdx.x == 0 && b != 0u) atomicMax(out, b);
  }
}

// ------------------------------------------------------------ quantize ----

// One thread quantizes kBlocksPerThread scale blocks.  Blocks are assigned so
// that in each of the j passes a warp reads 1 KiB of contiguous input.
__global__ void __launch_bounds__(kThreads)
quantize_bf16_kernel(const uint4* __restrict__ x, uint32_t n_blocks, uint32_t kb_per_row,
                     const float* __restrict__ amax_ptr, float amax_val,
                     uint2* __restrict__ packed, uint8_t* __restrict__ sf_lin,
                     uint8_t* __restrict__ sf_swz, uint32_t k_atoms,
                     float* __restrict__ global_scale_out) {
  const float amax_g = amax_ptr ? __ldg(amax_ptr) : amax_val;
  const float s_enc = global_encode_scale(amax_g);
  const float s_dec = __fdiv_rn(1.0f, s_enc);
  if (global_scale_out && blockIdx.x == 0 && threadIdx.x == 0) *global_scale_out = s_dec;

  // CTAs start at the END of the tensor: the amax pass that ran just before walked it
  // forwards, so its tail is what is still in L2 (126 MB) when this kernel begins
  const uint32_t base = (gridDim.x - 1u - blockIdx.x) * (kThreads * kBlocksPerThread) + threadIdx.x;
  uint4 v[kBlocksPerThread][2];
#pragma unroll
  for (int j = 0; j < kBlocksPerThread; ++j) {
    const uint32_t b = base + j * kThreads;
    if (b < n_blocks) {
      v[j][0] = __ldcs(x + 2 * (size_t)b);
      v[j][1] = __ldcs(x + 2 * (size_t)b + 1);
    } else {
      v[j][0] = make_uint4(0, 0, 0, 0);
      v[j][1] = make_uint4(0, 0, 0, 0);
    }
  }
  uint32_t row = 0, kb = 0;
  if (sf_swz) {
    row = base / kb_per_row;
    kb = base - row * kb_per_row;
  }
#pragma unroll
  for (int j = 0; j < kBlocksPerThread; ++j) {
    const uint32_t b = base + j * kThreads;
    const uint32_t w[8] = {v[j][0].x, v[j][0].y, v[j][0].z, v[j][0].w,
                           v[j][1].x, v[j][1].y, v[j][1].z, v[j][1].w};
    // block amax on the packed pairs (exact: the values are bf16), then widen once
    uint32_t a2 = 0u;
#pragma unroll
    for (int k = 0; k < 8; ++k) a2 = bf16x2_max_abs(a2, w[k]);
    const float amax_b = fmaxf(bf16lo_to_f32(a2), bf16hi_to_f32(a2));
    // (amax_b / 6) * S_enc -> E4M3; 1 / (float(sf) * S_dec): both quotients IEEE-rounded
    float d = __fmul_rn(div_by_6(amax_b), s_enc);
    d = fminf(d, FLT_MAX);
    const uint8_t sf = (uint8_t)__nv_cvt_float_to_fp8(d, __NV_SATFINITE, __NV_E4M3);
    const float enc = fminf(__frcp_rn(__fmul_rn(e4m3_to_f32(sf), s_dec)), FLT_MAX);
    const float2 enc2 = make_float2(enc, enc);
    float2 q[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) q[k] = f2_mul(bf16x2_to_f2(w[k]), enc2);
    uint2 out;
    out.x = f32x8_to_e2m1x8(q[0].x, q[0].y, q[1].x, q[1].y, q[2].x, q[2].y, q[3].x, q[3].y);
    out.y = f32x8_to_e2m1x8(q[4].x, q[4].y, q[5].x, q[5].y, q[6].x, q[6].y, q[7].x, q[7].y);
    if (b < n_blocks) {
      __stcs(packed + b, out);
      if (sf_lin) sf_lin[b] = sf;
      if (sf_swz) sf_swz[sf_swizzled_offset(row, kb, k_atoms)] = sf;
    }
    if (sf_swz) {  // advance (row, kb) by kThreads blocks
      kb += kThreads;
      while (kb >= kb_per_row) {
        kb -= kb_per_row;
        ++row;
      }
    }
  }
}

// ---------------------------------------------------------- dequantize ----

// One thread per 8 elements (4 packed bytes): x = e2m1 * (float(sf) / S_enc),
// S_enc derived from the tensor amax (device slot or by value).  IEEE
// division, so the bits match the CPU restatement of the reference formula.
__global__ void __launch_bounds__(kThreads)
dequantize_bf16_kernel(const uint32_t* __restrict__ packed, const uint8_t* __restrict__ sf_lin,
                       int64_t n_vec, const float* __restrict__ amax_ptr, float amax_val,
                       uint4* __restrict__ out) {
  const float s_enc = global_encode_scale(amax_ptr ? __ldg(amax_ptr) : amax_val);
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= n_vec) return;
  const uint32_t p = __ldg(packed + i);
  const float sf = e4m3_to_f32(__ldg(sf_lin + (i >> 1)));
  const float d = __fdiv_rn(sf, s_enc);
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t byte = (p >> (8 * k)) & 0xFFu;
    float lo, hi;
    {
      const uint32_t n0 = byte & 0xF, n1 = byte >> 4;
      // E2M1 magnitude: exponent e = bits 2:1, mantissa m = bit 0
      const uint32_t e0 = (n0 >> 1) & 3, m0 = n0 & 1, e1 = (n1 >> 1) & 3, m1 = n1 & 1;
      float a0 = e0 == 0 ? 0.5f * m0 : (float)(2 + m0) * (float)(1u << (e0 - 1)) * 0.5f;
      float a1 = e1 == 0 ? 0.5f * m1 : (float)(2 + m1) * (float)(1u << (e1 - 1)) * 0.5f;
      lo = (n0 & 8) ? -a0 : a0;
      hi = (n1 & 8) ? -a1 : a1;
    }
    __nv_bfloat162 r = __floats2bfloat162_rn(__fmul_rn(lo, d), __fmul_rn(hi, d));
    o[k] = *reinterpret_cast<uint32_t*>(&r);
  }
  out[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

// -------------------------------------------------------------- swizzle ----

__global__ void __launch_bounds__(kThreads)
swizzle_scales_kernel(const uint8_t* __restrict__ lin, int64_t n_sf, uint32_t kb_per_row,
                      uint32_t k_atoms, uint8_t* __restrict__ swz) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= n_sf) return;
  const int64_t row = i / kb_per_row;
  const int64_t kb = i - row * kb_per_row;
  swz[sf_swizzled_offset(row, kb, k_atoms)] = lin[i];
}

int launch_status() {
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}

// Zero the pad region of a swizzled scale buffer so that padded rows / K-blocks
// decode to 0 (a pad byte of 0x7F would be NaN and poison the accumulators).
int zero_swizzle_padding(uint8_t* swz, int64_t rows, int64_t cols, cudaStream_t st) {
  const int64_t kb = cols / kBlock;
  const int64_t total = sf_swizzled_bytes(rows, cols);
  if (kb % kSfKbPad != 0) {
    return cudaMemsetAsync(swz, 0, (size_t)total, st) == cudaSuccess ? NVFP4_OK
                                                                      : NVFP4_ERR_LAUNCH_FAILED;
  }
  if (rows % 128 != 0 || sf_row_tiles(rows) * 128 != (rows + 127) / 128 * 128) {
    const int64_t first = (rows / 128) * sf_k_atoms(cols) * kSfAtomBytes;  // first partial tile
    return cudaMemsetAsync(swz + first, 0, (size_t)(total - first), st) == cudaSuccess
               ? NVFP4_OK
               : NVFP4_ERR_LAUNCH_FAILED;
  }
  return NVFP4_OK;
}

int quantize_impl(const void* x, int64_t rows, int64_t cols, const float* amax_dev, float amax_val,
                  uint8_t* packed, uint8_t* sf_lin, uint8_t* sf_swz, float* gscale, void* stream) {
  if (rows < 0 || cols < 0 || cols % kBlock != 0) return NVFP4_ERR_BAD_ARG;
  // each extent first, so that the product cannot wrap; then at most 2^31 - 1 scale blocks
  if (rows >= ((int64_t)1 << 31) || cols >= ((int64_t)1 << 31)) return NVFP4_ERR_BAD_ARG;
  const int64_t n_blocks = rows * cols / kBlock;
  if (n_blocks >= (int64_t)1 << 31) return NVFP4_ERR_BAD_ARG;
  if (n_blocks == 0) return NVFP4_OK;
  if (!x || !packed) return NVFP4_ERR_BAD_ARG;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(packed) & 7u)) return NVFP4_ERR_BAD_ALIGN;
  int rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (sf_swz) {
    rc = zero_swizzle_padding(sf_swz, rows, cols, st);
    if (rc != NVFP4_OK) return rc;
  }
  const int per_cta = kThreads * kBlocksPerThread;
  const unsigned grid = (unsigned)((n_blocks + per_cta - 1) / per_cta);
  quantize_bf16_kernel<<<grid, kThreads, 0, st>>>(
      reinterpret_cast<const uint4*>(x), (uint32_t)n_blocks, (uint32_t)(cols / kBlock), amax_dev,
      amax_val, reinterpret_cast<uint2*>(packed), sf_lin, sf_swz, (uint32_t)sf_k_atoms(cols),
      gscale);
  return launch_status();
}

}  // namespace

}  // namespace nvfp4

using namespace nvfp4;

extern "C" {

int nvfp4_amax_bf16(const void* x, int64_t n, float* amax_dev, void* stream) {
  if (n < 0 || !amax_dev) return NVFP4_ERR_BAD_ARG;
  int rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(amax_dev, 0, sizeof(float), st) != cudaSuccess)
    return NVFP4_ERR_LAUNCH_FAILED;
  if (n == 0) return NVFP4_OK;
  if (!x) return NVFP4_ERR_BAD_ARG;
  if (!aligned16(x)) return NVFP4_ERR_BAD_ALIGN;
  const int64_t n_vec = n / 8;
  const int n_tail = (int)(n - n_vec * 8);
  int64_t want = (n_vec + kThreads * 4 - 1) / (kThreads * 4);
  const unsigned grid = (unsigned)(want < 1 ? 1 : (want > 148 * 8 ? 148 * 8 : want));
  amax_bf16_kernel<<<grid, kThreads, 0, st>>>(
      reinterpret_cast<const uint4*>(x), n_vec,
      reinterpret_cast<const __nv_bfloat16*>(x) + n_vec * 8, n_tail,
      reinterpret_cast<unsigned*>(amax_dev));
  return launch_status();
}

int64_t nvfp4_swizzled_scale_bytes(int64_t rows, int64_t cols) {
  return sf_swizzled_bytes(rows, cols);
}

int nvfp4_quantize_bf16(const void* x, int64_t rows, int64_t cols, const float* amax_dev,
                        uint8_t* packed, uint8_t* scales_linear, uint8_t* scales_swizzled,
                        float* global_scale_dev, void* stream) {
  // an empty tensor reads nothing, not even the amax slot
  if (!amax_dev && rows > 0 && cols > 0) return NVFP4_ERR_BAD_ARG;
  return quantize_impl(x, rows, cols, amax_dev, 0.0f, packed, scales_linear, scales_swizzled,
                       global_scale_dev, stream);
}

int nvfp4_quantize_bf16_amax(const void* x, uint8_t* packed, uint8_t* scales, int64_t n,
                             float global_amax, void* stream) {
  if (n < 0 || n % kBlock != 0) return NVFP4_ERR_BAD_ARG;
  if (n > 0 && !scales) return NVFP4_ERR_BAD_ARG;
  return quantize_impl(x, 1, n, nullptr, global_amax, packed, scales, nullptr, nullptr, stream);
}

static int dequantize_impl(const uint8_t* packed, const uint8_t* scales, int64_t n,
                           const float* amax_dev, float amax_val, void* out, void* stream) {
  if (n < 0 || n % kBlock != 0 || n / kBlock >= ((int64_t)1 << 31)) return NVFP4_ERR_BAD_ARG;
  if (n == 0) return NVFP4_OK;
  if (!packed || !scales || !out) return NVFP4_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(packed) & 3u) || !aligned16(out)) return NVFP4_ERR_BAD_ALIGN;
  int rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
  const int64_t n_vec = n / 8;
  const unsigned grid = (unsigned)((n_vec + kThreads - 1) / kThreads);
  dequantize_bf16_kernel<<<grid, kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(packed), scales, n_vec, amax_dev, amax_val,
      reinterpret_cast<uint4*>(out));
  return launch_status();
}

int nvfp4_dequantize_bf16(const uint8_t* packed, const uint8_t* scales_linear, int64_t rows,
                          int64_t cols, const float* amax_dev, void* out_bf16, void* stream) {
  if (rows < 0 || cols < 0 || cols % kBlock != 0 || !amax_dev) return NVFP4_ERR_BAD_ARG;
  if (rows >= ((int64_t)1 << 31) || cols >= ((int64_t)1 << 31)) return NVFP4_ERR_BAD_ARG;
  return dequantize_impl(packed, scales_linear, rows * cols, amax_dev, 0.0f, out_bf16,
                         stream);
}

int nvfp4_dequantize_bf16_amax(const uint8_t* packed, const uint8_t* scales, void* out_bf16,
                               int64_t n, float global_amax, void* stream) {
  return dequantize_impl(packed, scales, n, nullptr, global_amax, out_bf16, stream);
}

int nvfp4_swizzle_scales(const uint8_t* scales_linear, int64_t rows, int64_t cols,
                         uint8_t* scales_swizzled, void* stream) {
  if (rows < 0 || cols < 0 || cols % kBlock != 0) return NVFP4_ERR_BAD_ARG;
  if (rows >= ((int64_t)1 << 31) || cols >= ((int64_t)1 << 31)) return NVFP4_ERR_BAD_ARG;
  const int64_t n_sf = rows * cols / kBlock;
  if (n_sf >= (int64_t)1 << 32) return NVFP4_ERR_BAD_ARG;      // the grid would not fit
  if (n_sf == 0) return NVFP4_OK;
  if (!scales_linear || !scales_swizzled) return NVFP4_ERR_BAD_ARG;
  int rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  rc = zero_swizzle_padding(scales_swizzled, rows, cols, st);
  if (rc != NVFP4_OK) return rc;
  const unsigned grid = (unsigned)((n_sf + kThreads - 1) / kThreads);
  swizzle_scales_kernel<<<grid, kThreads, 0, st>>>(scales_linear, n_sf, (uint32_t)(cols / kBlock),
                                                   (uint32_t)sf_k_atoms(cols), scales_swizzled);
  return launch_status();
}

}  // extern "C"
