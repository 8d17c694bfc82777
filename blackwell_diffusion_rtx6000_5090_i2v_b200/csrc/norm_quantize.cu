// LayerNorm / RMSNorm + adaLN modulation fused with the NVFP4 quantizer.
//
//   h = bf16( ((x - mean) * rstd * w + b) * (1 + scale) + shift )      (fp32 math)
//   h -> packed E2M1 + E4M3 block scales + FP32 tensor scale
//
// replaces, for the inputs of the DiT block's QKV / Q / FFN-up linears, the
// chain norm -> modulation -> cast -> amax -> quantize
// (fx/src/s4/models/wan22/wan_transformer.py:204-206, 210, 218-220).  The
// per-tensor amax forces two sweeps; both read only x (2 B/element each) and
// recompute h, so h itself never travels: 4 + 0.5625 bytes per element moved
// against 2 + 2 + 2 + 2 + 0.5625 for the unfused chain.
//
// One CTA of 128 threads per row; a thread keeps its 16-byte vectors of the
// row in registers (cols <= 16384).  Sweep 1 leaves mean and rstd per row in a
// small stats buffer so that sweep 2 repeats exactly the same arithmetic.
#include "nvfp4_common.cuh"

namespace nvfp4 {
namespace {

constexpr int kThreads = 128;
constexpr int kMaxVec = 16;   // 16 vectors x 8 elements x 128 threads = 16384 columns

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();   // red may still be read from the previous reduction
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return (red[0] + red[1]) + (red[2] + red[3]);
}

// h for the 8 elements of one vector, rounded to bf16 and widened again (the quantizer's
// input is the bf16 tensor the unfused model would have produced).
__device__ __forceinline__ void modulate8(const uint4& xv, int col, float mean, float rstd,
                                          const float* __restrict__ w, const float* __restrict__ b,
                                          const float* __restrict__ scale,
                                          const float* __restrict__ shift, float (&h)[8]) {
  const uint32_t u[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float x = (e & 1) ? bf16hi_to_f32(u[e >> 1]) : bf16lo_to_f32(u[e >> 1]);
    float y = __fmul_rn(__fsub_rn(x, mean), rstd);
    if (w) y = __fmul_rn(y, __ldg(w + col + e));
    if (b) y = __fadd_rn(y, __ldg(b + col + e));
    if (scale) y = __fmul_rn(y, __fadd_rn(1.0f, __ldg(scale + col + e)));
    if (shift) y = __fadd_rn(y, __ldg(shift + col + e));
    h[e] = __bfloat162float(__float2bfloat16_rn(y));
  }
}

template <bool kQuantize, int kJ>   // kJ: 16-byte vectors of the row held per thread
__global__ void __launch_bounds__(kThreads)
norm_mod_kernel(const uint4* __restrict__ x, int cols, const float* __restrict__ w,
                const float* __restrict__ b, const float* __restrict__ scale,
                const float* __restrict__ shift, int rms, float eps, float* __restrict__ stats,
                unsigned* __restrict__ amax_out, uint4* __restrict__ h_out,
                const float* __restrict__ amax_in, uint32_t* __restrict__ packed,
                uint8_t* __restrict__ sf_lin, uint8_t* __restrict__ sf_swz, uint32_t k_atoms,
                float* __restrict__ gscale_out) {
  __shared__ float red[4];
  const int row = blockIdx.x;
  const int nvec = cols / 8;
  const uint4* xr = x + (size_t)row * nvec;
  uint4 v[kJ];
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int i = threadIdx.x + j * kThreads;
    v[j] = i < nvec ? __ldcs(xr + i) : make_uint4(0, 0, 0, 0);
  }
  float mean, rstd;
  if (!kQuantize) {
    // sweep 1: two-pass statistics in registers, then amax of h
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      const uint32_t u[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) s += bf16lo_to_f32(u[e]) + bf16hi_to_f32(u[e]);
    }
    mean = rms ? 0.0f : block_sum(s, red) / (float)cols;
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      if (threadIdx.x + j * kThreads < nvec) {
        const uint32_t u[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float a = bf16lo_to_f32(u[e]) - mean, c = bf16hi_to_f32(u[e]) - mean;
          ss += a * a + c * c;
        }
      }
    }
    rstd = rsqrtf(block_sum(ss, red) / (float)cols + eps);
    if (threadIdx.x == 0) {
      stats[2 * (size_t)row] = mean;
      stats[2 * (size_t)row + 1] = rstd;
    }
  } else {
    mean = __ldg(stats + 2 * (size_t)row);
    rstd = __ldg(stats + 2 * (size_t)row + 1);
  }

  float s_enc = 0.0f, s_dec = 0.0f;
  if (kQuantize) {
    s_enc = global_encode_scale(__ldg(amax_in));
    s_dec = __fdiv_rn(1.0f, s_enc);
    if (gscale_out && row == 0 && threadIdx.x == 0) *gscale_out = s_dec;
  }
  float amax_t = 0.0f;
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int i = threadIdx.x + j * kThreads;   // vector index in the row; lanes 2k, 2k+1 share a block
    const bool live = i < nvec;                 // nvec is even: a pair of lanes is live together
    // initialised even for lanes past the end of the row: left indeterminate, the optimiser
    // was free to (and did) feed the pack instruction garbage
    float h[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    float a8 = 0.0f;
    if (live) {
      modulate8(v[j], i * 8, mean, rstd, w, b, scale, shift, h);
#pragma unroll
      for (int e = 0; e < 8; ++e) a8 = fmaxf(a8, fabsf(h[e]));
    }
    if (!kQuantize) {
      amax_t = fmaxf(amax_t, a8);
      if (live && h_out) {
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 p2 = __floats2bfloat162_rn(h[2 * e], h[2 * e + 1]);
          o[e] = *reinterpret_cast<uint32_t*>(&p2);
        }
        h_out[(size_t)row * nvec + i] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    } else {
      // the partner lane holds the other half of the 16-element block
      const float amax_b = fmaxf(a8, __shfl_xor_sync(0xffffffffu, a8, 1));
      if (live) {
        const uint8_t sf = block_scale_e4m3(amax_b, s_enc);
        const float enc = block_encode_scale(sf, s_dec);
#pragma unroll
        for (int e = 0; e < 8; ++e) h[e] = __fmul_rn(h[e], enc);
        packed[(size_t)row * nvec + i] =
            f32x8_to_e2m1x8(h[0], h[1], h[2], h[3], h[4], h[5], h[6], h[7]);
        if ((i & 1) == 0) {
          const int kb = i >> 1;
          if (sf_lin) sf_lin[(size_t)row * (nvec / 2) + kb] = sf;
          if (sf_swz) sf_swz[sf_swizzled_offset(row, kb, k_atoms)] = sf;
        }
      }
    }
  }
  if (!kQuantize) {
    unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(amax_t));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = __uint_as_float(bits);
    __syncthreads();
    if (threadIdx.x == 0) {
      const float m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
      if (m > 0.0f) atomicMax(amax_out, __float_as_uint(m));
    }
  }
}

int check_args(const void* x, int64_t rows, int64_t cols) {
  if (rows < 0 || cols <= 0 || cols % kBlock != 0 || cols > kMaxVec * 8 * kThreads ||
      rows >= ((int64_t)1 << 31))
    return NVFP4_ERR_BAD_ARG;
  if (rows > 0 && !x) return NVFP4_ERR_BAD_ARG;
  if (!aligned16(x)) return NVFP4_ERR_BAD_ALIGN;
  return check_device_sm100();
}

}  // namespace
}  // namespace nvfp4

using namespace nvfp4;

extern "C" {

int nvfp4_norm_mod_amax_bf16(const void* x_bf16, int64_t rows, int64_t cols, const float* weight,
                             const float* bias, const float* scale, const float* shift, int rms,
                             float eps, float* row_stats, float* amax_dev, void* h_out_bf16,
                             void* stream) {
  int rc = check_args(x_bf16, rows, cols);
  if (rc != NVFP4_OK) return rc;
  if (!row_stats || !amax_dev) return NVFP4_ERR_BAD_ARG;
  if (!aligned16(h_out_bf16)) return NVFP4_ERR_BAD_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(amax_dev, 0, sizeof(float), st) != cudaSuccess) return NVFP4_ERR_LAUNCH_FAILED;
  if (rows == 0) return NVFP4_OK;
  const int need = (int)((cols / 8 + kThreads - 1) / kThreads);
#define NVFP4_LAUNCH_NORM_AMAX(J)                                                                \
  norm_mod_kernel<false, J><<<(unsigned)rows, kThreads, 0, st>>>(                                \
      reinterpret_cast<const uint4*>(x_bf16), (int)cols, weight, bias, scale, shift, rms, eps,   \
      row_stats, reinterpret_cast<unsigned*>(amax_dev), reinterpret_cast<uint4*>(h_out_bf16),    \
      nullptr, nullptr, nullptr, nullptr, 0u, nullptr)
  if (need <= 4) NVFP4_LAUNCH_NORM_AMAX(4);
  else if (need <= 8) NVFP4_LAUNCH_NORM_AMAX(8);
  else NVFP4_LAUNCH_NORM_AMAX(16);
#undef NVFP4_LAUNCH_NORM_AMAX
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}

int nvfp4_norm_mod_quantize_bf16(const void* x_bf16, int64_t rows, int64_t cols,
                                 const float* weight, const float* bias, const float* scale,
                                 const float* shift, const float* row_stats,
                                 const float* amax_dev, uint8_t* packed, uint8_t* scales_linear,
                                 uint8_t* scales_swizzled, float* global_scale_dev, void* stream) {
  int rc = check_args(x_bf16, rows, cols);
  if (rc != NVFP4_OK) return rc;
  if (!row_stats || !amax_dev || (rows > 0 && !packed)) return NVFP4_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(packed) & 3u) return NVFP4_ERR_BAD_ALIGN;
  if (rows == 0) return NVFP4_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (scales_swizzled) {
    // pad rows / K-blocks of the swizzled buffer must decode to zero
    const int64_t total = sf_swizzled_bytes(rows, cols);
    const bool k_pad = (cols / kBlock) % kSfKbPad != 0;
    const int64_t first = k_pad ? 0 : (rows / 128) * sf_k_atoms(cols) * kSfAtomBytes;
    if (first < total &&
        cudaMemsetAsync(scales_swizzled + first, 0, (size_t)(total - first), st) != cudaSuccess)
      return NVFP4_ERR_LAUNCH_FAILED;
  }
  const int need = (int)((cols / 8 + kThreads - 1) / kThreads);
#define NVFP4_LAUNCH_NORM_QUANT(J)                                                               \
  norm_mod_kernel<true, J><<<(unsigned)rows, kThreads, 0, st>>>(                                 \
      reinterpret_cast<const uint4*>(x_bf16), (int)cols, weight, bias, scale, shift, 0, 0.0f,    \
      const_cast<float*>(row_stats), nullptr, nullptr, amax_dev,                                 \
      reinterpret_cast<uint32_t*>(packed), scales_linear, scales_swizzled,                       \
      (uint32_t)sf_k_atoms(cols), global_scale_dev)
  if (need <= 4) NVFP4_LAUNCH_NORM_QUANT(4);
  else if (need <= 8) NVFP4_LAUNCH_NORM_QUANT(8);
  else NVFP4_LAUNCH_NORM_QUANT(16);
#undef NVFP4_LAUNCH_NORM_QUANT
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}

}  // extern "C"
