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
// Work split.  A CTA of T threads covers one row with kJ 16-byte vectors per thread
// (T * kJ * 8 >= cols) and walks over many groups of kR consecutive rows.  A group is one
// contiguous piece of x, fetched by a single bulk copy into a ring of kStages shared-memory
// slots that completes an mbarrier; kStages - 1 groups are always in flight per CTA, which is
// what keeps HBM busy -- no register holds data that is still on its way.  A thread sees the
// same columns in every row, so its slice of the per-column vectors (w, b, 1 + scale, shift)
// is loaded once into registers and costs nothing per row.  Row statistics are two-pass (sum,
// then squared deviations from the mean) over the registers; the two CTA-wide reductions per
// group serve kR rows each.  Sweep 1 leaves mean and rstd per row in a small stats buffer so
// that sweep 2, which needs no reduction at all, repeats exactly the same arithmetic.
//
// Sweep 1 walks the groups forwards and sweep 2 walks them backwards with an evict-first
// hint: the tail of x that sweep 1 left in L2 (126 MB) is what sweep 2 reads first.
#include "nvfp4_common.cuh"

namespace nvfp4 {
namespace {

constexpr int kMaxThreads = 512;
constexpr int kMaxJ = 4;          // 4 vectors x 8 elements x 512 threads = 16384 columns
constexpr int kMaxWarps = kMaxThreads / 32;
constexpr int kStages = 3;
constexpr long long kWaitCycles = 4000000000LL;   // about two seconds; then give up
constexpr int kErrCopyTimeout = 0x900;            // status code: a row group never arrived

// rows per group: at most 32 KB per slot (cols <= 4096 * kJ)
template <int kJ> struct RowsPerIter { static constexpr int value = kJ == 1 ? 4 : (kJ == 2 ? 2 : 1); };

struct NormArgs {
  const uint4* x;
  int64_t rows;
  int cols;
  const float* w;
  const float* b;
  const float* scale;
  const float* shift;
  int rms;
  float eps;
  float* stats;              // [rows][2] mean, rstd: written by sweep 1, read by sweep 2
  unsigned* amax_out;        // sweep 1
  uint4* h_out;              // sweep 1, optional
  const float* amax_in;      // sweep 2
  uint32_t* packed;          // sweep 2
  uint8_t* sf_lin;
  uint8_t* sf_swz;
  uint32_t k_atoms;
  float* gscale_out;
  int* status;               // nullable; receives kErrCopyTimeout
};

__device__ __forceinline__ void load8(const float* p, float (&d)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 c = __ldg(reinterpret_cast<const float4*>(p) + 1);
  d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w;
  d[4] = c.x; d[5] = c.y; d[6] = c.z; d[7] = c.w;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Contiguous global -> this CTA's shared memory, bytes reported to `bar`.  One destination,
// nothing broadcast.  Addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                          bool evict_first) {
  if (evict_first) {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
  }
}

// Bounded wait for a row group.  On expiry (or once any thread of the CTA has given up) the
// caller carries on without the data: every later barrier is still reached by all threads,
// the outputs of this CTA are then meaningless and the status word says so.
__device__ __forceinline__ void wait_group(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                           int* status) {
  if (mbar_try_wait(bar, parity)) return;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return;
    if ((it & 255u) == 0) {
      if (*abort_flag) return;
      if (clock64() - t0 > kWaitCycles) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, kErrCopyTimeout);
        return;
      }
    }
  }
}

// Sum over the CTA of kR values per thread; every thread gets all kR totals, added in a fixed
// order.  `red` is one of two buffers used alternately, which makes one barrier per reduction
// enough: a buffer is rewritten only after the barrier of the reduction in between.
template <int kR>
__device__ __forceinline__ void cta_sum(float (&v)[kR], float (*red)[kMaxWarps], int warps) {
#pragma unroll
  for (int r = 0; r < kR; ++r) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[r] += __shfl_xor_sync(0xffffffffu, v[r], o);
  }
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int r = 0; r < kR; ++r) red[r][threadIdx.x >> 5] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kR; ++r) {
    float t = 0.0f;
    for (int w4 = 0; w4 < warps; w4 += 4) {
      const float4 q = *reinterpret_cast<const float4*>(&red[r][w4]);   // unused slots hold 0
      t += (q.x + q.y) + (q.z + q.w);
    }
    v[r] = t;
  }
}

template <bool kQuantize, int kJ, bool kAffine, bool kMod>
__global__ void __launch_bounds__(kMaxThreads)
norm_mod_kernel(const NormArgs p) {
  constexpr int kR = RowsPerIter<kJ>::value;
  extern __shared__ __align__(128) uint8_t ring[];          // kStages slots of kR rows
  __shared__ __align__(16) float red[2][kR][kMaxWarps];
  __shared__ float red_max[kMaxWarps];
  __shared__ __align__(8) uint64_t full[kStages];
  __shared__ int abort_flag;
  const int T = blockDim.x;
  const int warps = T >> 5;
  const int nvec = p.cols >> 3;
  const uint32_t row_bytes = (uint32_t)p.cols * 2u;
  const uint32_t slot_bytes = row_bytes * kR;
  const int64_t groups = (p.rows + kR - 1) / kR;

  // group g of this CTA's walk -> first row and byte count (sweep 2 mirrors the order)
  auto group_base = [&](int64_t g) { return (kQuantize ? groups - 1 - g : g) * kR; };
  auto issue = [&](int64_t g, int slot) {
    const int64_t base = group_base(g);
    const int64_t n = p.rows - base < kR ? p.rows - base : kR;
    const uint32_t bytes = (uint32_t)n * row_bytes;
    const uint32_t bar = smem_u32(&full[slot]);
    mbar_expect_tx(bar, bytes);
    bulk_load(smem_u32(ring + (size_t)slot * slot_bytes),
              reinterpret_cast<const uint8_t*>(p.x) + base * row_bytes, bytes, bar, kQuantize);
  };

  if (threadIdx.x == 0) {
    abort_flag = 0;
#pragma unroll
    for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(&full[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < 2 * kR * kMaxWarps; i += T) (&red[0][0][0])[i] = 0.0f;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      const int64_t g = (int64_t)blockIdx.x + (int64_t)s * gridDim.x;
      if (g < groups) issue(g, s);
    }
  }

  // this thread's columns and its slice of the per-column vectors
  bool live[kJ];
  float cw[kAffine ? kJ : 1][8], cb[kAffine ? kJ : 1][8];
  float cs[kMod ? kJ : 1][8], ct[kMod ? kJ : 1][8];
  bool has_w = false, has_b = false, has_s = false, has_t = false;
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int i = threadIdx.x + j * T;
    live[j] = i < nvec;
    const int col = live[j] ? i * 8 : 0;
    if (kAffine) {
      has_w = p.w != nullptr; has_b = p.b != nullptr;
      if (has_w) load8(p.w + col, cw[j]);
      if (has_b) load8(p.b + col, cb[j]);
    }
    if (kMod) {
      has_s = p.scale != nullptr; has_t = p.shift != nullptr;
      if (has_s) {
        load8(p.scale + col, cs[j]);
#pragma unroll
        for (int e = 0; e < 8; ++e) cs[j][e] = __fadd_rn(1.0f, cs[j][e]);
      }
      if (has_t) load8(p.shift + col, ct[j]);
    }
  }

  float s_enc = 0.0f, s_dec = 0.0f;
  if (kQuantize) {
    s_enc = global_encode_scale(__ldg(p.amax_in));
    s_dec = __fdiv_rn(1.0f, s_enc);
    if (p.gscale_out && blockIdx.x == 0 && threadIdx.x == 0) *p.gscale_out = s_dec;
  }
  float amax_t = 0.0f;
  const float cols_f = (float)p.cols;

  int slot = 0;
  uint32_t phase = 0;
  for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
    const int64_t base = group_base(g);
    wait_group(smem_u32(&full[slot]), phase, &abort_flag, p.status);
    const uint4* src = reinterpret_cast<const uint4*>(ring + (size_t)slot * slot_bytes);
    bool row_ok[kR];
    uint4 v[kR][kJ];
#pragma unroll
    for (int r = 0; r < kR; ++r) {
      row_ok[r] = base + r < p.rows;
#pragma unroll
      for (int j = 0; j < kJ; ++j)
        v[r][j] = (live[j] && row_ok[r]) ? src[r * nvec + threadIdx.x + j * T]
                                         : make_uint4(0, 0, 0, 0);
    }
    float mean[kR], rstd[kR];
    bool refilled = false;
    // once every thread holds its vectors the slot can take the group kStages ahead
    auto refill = [&]() {
      const int64_t gn = g + (int64_t)kStages * gridDim.x;
      if (threadIdx.x == 0 && gn < groups) issue(gn, slot);
      refilled = true;
    };
    if (!kQuantize) {
      float s[kR];
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        s[r] = 0.0f;
#pragma unroll
        for (int j = 0; j < kJ; ++j) {
          const uint32_t u[4] = {v[r][j].x, v[r][j].y, v[r][j].z, v[r][j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) s[r] += bf16lo_to_f32(u[e]) + bf16hi_to_f32(u[e]);
        }
      }
      if (!p.rms) {
        cta_sum<kR>(s, red[0], warps);
        refill();
      }
#pragma unroll
      for (int r = 0; r < kR; ++r) mean[r] = p.rms ? 0.0f : s[r] / cols_f;
      float ss[kR];
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        ss[r] = 0.0f;
#pragma unroll
        for (int j = 0; j < kJ; ++j) {
          if (live[j]) {
            const uint32_t u[4] = {v[r][j].x, v[r][j].y, v[r][j].z, v[r][j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float a = bf16lo_to_f32(u[e]) - mean[r], c = bf16hi_to_f32(u[e]) - mean[r];
              ss[r] += a * a + c * c;
            }
          }
        }
      }
      cta_sum<kR>(ss, red[1], warps);
      if (!refilled) refill();
      if (p.rms) __syncthreads();   // red[1] is then the only buffer: keep groups apart
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        rstd[r] = rsqrtf(ss[r] / cols_f + p.eps);
        if (threadIdx.x == 0 && row_ok[r]) {
          p.stats[2 * (base + r)] = mean[r];
          p.stats[2 * (base + r) + 1] = rstd[r];
        }
      }
    } else {
      __syncthreads();
      refill();
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        const int64_t rr = row_ok[r] ? base + r : base;
        mean[r] = __ldg(p.stats + 2 * rr);
        rstd[r] = __ldg(p.stats + 2 * rr + 1);
      }
    }

#pragma unroll
    for (int r = 0; r < kR; ++r) {
      const int64_t row = base + r;
#pragma unroll
      for (int j = 0; j < kJ; ++j) {
        const int i = threadIdx.x + j * T;       // lanes 2k, 2k+1 hold the halves of one block
        const bool on = live[j] && row_ok[r];    // nvec and T are even: a pair is on together
        float h[8];
        float a8 = 0.0f;
        const uint32_t u[4] = {v[r][j].x, v[r][j].y, v[r][j].z, v[r][j].w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float x = (e & 1) ? bf16hi_to_f32(u[e >> 1]) : bf16lo_to_f32(u[e >> 1]);
          float y = __fmul_rn(__fsub_rn(x, mean[r]), rstd[r]);
          if (kAffine) {
            if (has_w) y = __fmul_rn(y, cw[j][e]);
            if (has_b) y = __fadd_rn(y, cb[j][e]);
          }
          if (kMod) {
            if (has_s) y = __fmul_rn(y, cs[j][e]);
            if (has_t) y = __fadd_rn(y, ct[j][e]);
          }
          // the quantizer's input is the bf16 tensor the unfused model would have produced
          h[e] = on ? __bfloat162float(__float2bfloat16_rn(y)) : 0.0f;
          a8 = fmaxf(a8, fabsf(h[e]));
        }
        if (!kQuantize) {
          amax_t = fmaxf(amax_t, a8);
          if (on && p.h_out) {
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 p2 = __floats2bfloat162_rn(h[2 * e], h[2 * e + 1]);
              o[e] = *reinterpret_cast<uint32_t*>(&p2);
            }
            p.h_out[row * nvec + i] = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
          const float amax_b = fmaxf(a8, __shfl_xor_sync(0xffffffffu, a8, 1));
          if (on) {
            const uint8_t sf = block_scale_e4m3(amax_b, s_enc);
            const float enc = block_encode_scale(sf, s_dec);
#pragma unroll
            for (int e = 0; e < 8; ++e) h[e] = __fmul_rn(h[e], enc);
            __stcs(p.packed + row * nvec + i,
                   f32x8_to_e2m1x8(h[0], h[1], h[2], h[3], h[4], h[5], h[6], h[7]));
            if ((i & 1) == 0) {
              const int kb = i >> 1;
              if (p.sf_lin) p.sf_lin[row * (nvec / 2) + kb] = sf;
              if (p.sf_swz) p.sf_swz[sf_swizzled_offset(row, kb, p.k_atoms)] = sf;
            }
          }
        }
      }
    }
    if (++slot == kStages) {
      slot = 0;
      phase ^= 1u;
    }
  }

  if (!kQuantize) {
    const unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(amax_t));
    if ((threadIdx.x & 31) == 0) red_max[threadIdx.x >> 5] = __uint_as_float(bits);
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = 0.0f;
      for (int w = 0; w < warps; ++w) m = fmaxf(m, red_max[w]);
      if (m > 0.0f) atomicMax(p.amax_out, __float_as_uint(m));
    }
  }
  // Every copy this CTA issued has been waited for (each group issued is a group consumed),
  // unless a wait expired: then give copies still in flight time to land before the shared
  // memory is handed to another CTA.
  if (abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
  }
}

int check_args(const void* x, int64_t rows, int64_t cols) {
  if (rows < 0 || cols <= 0 || cols % kBlock != 0 || cols > kMaxJ * 8 * kMaxThreads ||
      rows >= ((int64_t)1 << 31))
    return NVFP4_ERR_BAD_ARG;
  if (rows > 0 && !x) return NVFP4_ERR_BAD_ARG;
  if (!aligned16(x)) return NVFP4_ERR_BAD_ALIGN;
  return check_device_sm100();
}

bool vec_ok(const float* p) { return aligned16(p); }

// Vectors per thread (1, 2 or 4) and threads per CTA (a multiple of 32) for a row of nvec
// 16-byte vectors: the smallest kJ that fits 512 threads, then as few threads as cover it.
void shape_for(int nvec, int* j, int* threads) {
  int J = 1;
  while (J < kMaxJ && nvec > J * kMaxThreads) J *= 2;
  const int per = (nvec + J - 1) / J;
  *j = J;
  *threads = ((per + 31) / 32) * 32;
}

template <bool kQuantize, int kJ, bool kAffine, bool kMod>
int launch_variant(const NormArgs& a, int threads, cudaStream_t st) {
  auto kernel = norm_mod_kernel<kQuantize, kJ, kAffine, kMod>;
  constexpr int kR = RowsPerIter<kJ>::value;
  const size_t smem = (size_t)kStages * kR * a.cols * 2;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return NVFP4_ERR_LAUNCH_FAILED;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess ||
      per_sm < 1)
    return NVFP4_ERR_LAUNCH_FAILED;
  const int64_t groups = (a.rows + kR - 1) / kR;
  const int64_t resident = (int64_t)sm_count() * per_sm;
  const unsigned grid = (unsigned)(groups < resident ? groups : resident);
  kernel<<<grid, threads, smem, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}

template <bool kQuantize>
int launch(const NormArgs& a, cudaStream_t st) {
  int J, threads;
  shape_for(a.cols / 8, &J, &threads);
  const bool affine = a.w || a.b, mod = a.scale || a.shift;
#define NVFP4_NORM_CASE(JJ)                                                           \
  if (J == JJ) {                                                                      \
    if (affine && mod) return launch_variant<kQuantize, JJ, true, true>(a, threads, st);   \
    if (affine) return launch_variant<kQuantize, JJ, true, false>(a, threads, st);    \
    if (mod) return launch_variant<kQuantize, JJ, false, true>(a, threads, st);       \
    return launch_variant<kQuantize, JJ, false, false>(a, threads, st);               \
  }
  NVFP4_NORM_CASE(1)
  NVFP4_NORM_CASE(2)
  NVFP4_NORM_CASE(4)
#undef NVFP4_NORM_CASE
  return NVFP4_ERR_BAD_ARG;
}

}  // namespace
}  // namespace nvfp4

using namespace nvfp4;

extern "C" {

int nvfp4_norm_mod_amax_bf16(const void* x_bf16, int64_t rows, int64_t cols, const float* weight,
                             const float* bias, const float* scale, const float* shift, int rms,
                             float eps, float* row_stats, float* amax_dev, void* h_out_bf16,
                             int* status_dev, void* stream) {
  int rc = check_args(x_bf16, rows, cols);
  if (rc != NVFP4_OK) return rc;
  if (!row_stats || !amax_dev) return NVFP4_ERR_BAD_ARG;
  if (!aligned16(h_out_bf16) || !vec_ok(weight) || !vec_ok(bias) || !vec_ok(scale) || !vec_ok(shift))
    return NVFP4_ERR_BAD_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(amax_dev, 0, sizeof(float), st) != cudaSuccess) return NVFP4_ERR_LAUNCH_FAILED;
  if (rows == 0) return NVFP4_OK;
  NormArgs a{};
  a.x = reinterpret_cast<const uint4*>(x_bf16);
  a.rows = rows; a.cols = (int)cols;
  a.w = weight; a.b = bias; a.scale = scale; a.shift = shift;
  a.rms = rms; a.eps = eps;
  a.stats = row_stats;
  a.amax_out = reinterpret_cast<unsigned*>(amax_dev);
  a.h_out = reinterpret_cast<uint4*>(h_out_bf16);
  a.status = status_dev;
  return launch<false>(a, st);
}

int nvfp4_norm_mod_quantize_bf16(const void* x_bf16, int64_t rows, int64_t cols,
                                 const float* weight, const float* bias, const float* scale,
                                 const float* shift, const float* row_stats,
                                 const float* amax_dev, uint8_t* packed, uint8_t* scales_linear,
                                 uint8_t* scales_swizzled, float* global_scale_dev,
                                 int* status_dev, void* stream) {
  int rc = check_args(x_bf16, rows, cols);
  if (rc != NVFP4_OK) return rc;
  if (!row_stats || !amax_dev || (rows > 0 && !packed)) return NVFP4_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(packed) & 3u) || !vec_ok(weight) || !vec_ok(bias) ||
      !vec_ok(scale) || !vec_ok(shift))
    return NVFP4_ERR_BAD_ALIGN;
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
  NormArgs a{};
  a.x = reinterpret_cast<const uint4*>(x_bf16);
  a.rows = rows; a.cols = (int)cols;
  a.w = weight; a.b = bias; a.scale = scale; a.shift = shift;
  a.stats = const_cast<float*>(row_stats);
  a.amax_in = amax_dev;
  a.packed = reinterpret_cast<uint32_t*>(packed);
  a.sf_lin = scales_linear; a.sf_swz = scales_swizzled;
  a.k_atoms = (uint32_t)sf_k_atoms(cols);
  a.gscale_out = global_scale_dev;
  a.status = status_dev;
  return launch<true>(a, st);
}

}  // extern "C"
