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
// Work split.  A thread owns whole 16-element scale blocks: kJ of them per row
// (T * kJ * 16 >= cols for a CTA of T threads), the same columns in every row, so its slice of
// the per-column vectors (w, b, 1 + scale, shift) is loaded once into registers and costs
// nothing per row, and a block's scale needs no exchange between threads.  A CTA walks over
// many groups of kR consecutive rows.  A group is one contiguous piece of x, fetched by a
// single bulk copy into a ring of kStages shared-memory slots that completes an mbarrier;
// kStages - 1 groups are always in flight per CTA, which is what keeps HBM busy -- no register
// holds data that is still on its way.
//
// Instruction count is what limits a kernel like this once the copies are off the critical
// path (an earlier form spent 25 instructions per element and ran at a third of HBM speed), so:
// fp32 math runs two lanes per instruction (f32x2) with each lane rounded as the scalar op;
// the bf16 rounding, |h| and its maximum are packed bf16x2 ops; the row statistics take one
// pass and ONE CTA-wide reduction per group (sums of x - pivot and its square, the pivot
// being the row's first element, which keeps S2/n - (S1/n)^2 away from cancellation), whose
// warp stage folds the 2 kR values instead of reducing them one by one; the divisions of
// the quantizer are gone (x/6 by an exact three-operation form, the encode scale from a
// 128-entry table per tensor); scale offsets split into a per-row and a per-thread part.
// Sweep 1 leaves mean and rstd per row in a small stats buffer so that sweep 2, which needs
// no reduction at all, repeats exactly the same arithmetic.
//
// Sweep 1 walks the groups forwards and sweep 2 walks them backwards with an evict-first
// hint: the tail of x that sweep 1 left in L2 (126 MB) is what sweep 2 reads first.
#include "nvfp4_common.cuh"

namespace nvfp4 {
namespace {

constexpr int kMaxThreads = 512;
constexpr int kMaxJ = 2;          // 2 blocks x 16 elements x 512 threads = 16384 columns
constexpr int kMaxWarps = kMaxThreads / 32;
#ifndef NVFP4_NORM_STAGES
#define NVFP4_NORM_STAGES 3
#endif
constexpr int kStages = NVFP4_NORM_STAGES;
constexpr long long kWaitCycles = 4000000000LL;   // about two seconds; then give up
constexpr int kErrCopyTimeout = 0x900;            // status code: a row group never arrived

#ifndef NVFP4_NORM_R1
#define NVFP4_NORM_R1 2
#endif
// rows per group: a slot is at most 64 KB (cols <= 8192 * kJ)
template <int kJ> struct RowsPerIter { static constexpr int value = kJ == 1 ? NVFP4_NORM_R1 : 2; };

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

__device__ __forceinline__ void load16(const float* p, float2 (&d)[8]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p) + q);
    d[2 * q] = make_float2(a.x, a.y);
    d[2 * q + 1] = make_float2(a.z, a.w);
  }
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
                                          int hint) {
  if (hint != 0) {
    uint64_t policy;
    if (hint == 1) {
      asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    } else {
      asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    }
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

// One fold step of the multi-value warp sum: a lane hands kHalf of its 2*kHalf values to the
// partner across `mask` and keeps the sums of the other kHalf.
template <int kHalf>
__device__ __forceinline__ void fold_step(float* v, bool upper, int mask) {
#pragma unroll
  for (int i = 0; i < kHalf; ++i) {
    const float keep = upper ? v[i + kHalf] : v[i];
    const float give = upper ? v[i] : v[i + kHalf];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, give, mask);
  }
}

// Sum over the CTA of kV values per thread; every thread gets all kV totals, added in a
// fixed order.  Inside a warp the values are folded (kV + 2 shuffles for kV = 8 instead of
// 40).  `red` is one of two buffers used alternately, which makes one barrier per reduction
// enough: a buffer is rewritten only after the barrier of the reduction in between.
template <int kV>
__device__ __forceinline__ void cta_sum(float (&v)[kV], float (*red)[kMaxWarps], int warps) {
  static_assert(kV == 1 || kV == 2 || kV == 4 || kV == 8, "fold needs a power of two <= 8");
  constexpr int n0 = kV, n1 = n0 > 1 ? n0 / 2 : 1, n2 = n1 > 1 ? n1 / 2 : 1;
  const int lane = threadIdx.x & 31;
  int idx = 0;      // which of the kV values this lane ends up holding
  int mask = 16;
  if constexpr (n0 > 1) {
    const bool up = (lane & mask) != 0;
    fold_step<n0 / 2>(v, up, mask);
    idx += up ? n0 / 2 : 0;
    mask >>= 1;
  }
  if constexpr (n1 > 1) {
    const bool up = (lane & mask) != 0;
    fold_step<n1 / 2>(v, up, mask);
    idx += up ? n1 / 2 : 0;
    mask >>= 1;
  }
  if constexpr (n2 > 1) {
    const bool up = (lane & mask) != 0;
    fold_step<n2 / 2>(v, up, mask);
    idx += up ? n2 / 2 : 0;
    mask >>= 1;
  }
  for (int o = mask; o > 0; o >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
  if ((lane & (2 * mask - 1)) == 0) red[idx][threadIdx.x >> 5] = v[0];
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kV; ++r) {
    float t = 0.0f;
    for (int w4 = 0; w4 < warps; w4 += 4) {
      const float4 q = *reinterpret_cast<const float4*>(&red[r][w4]);   // unused slots hold 0
      t += (q.x + q.y) + (q.z + q.w);
    }
    v[r] = t;
  }
}

// h for one 16-element block as 8 packed bf16 pairs, and the running bf16x2 max of |h|.
template <bool kAffine, bool kMod>
__device__ __forceinline__ uint32_t normalize16(const uint32_t (&xp)[8], float2 m2, float2 r2,
                                                const float2 (&cw)[8], const float2 (&cb)[8],
                                                const float2 (&cs)[8], const float2 (&ct)[8],
                                                bool has_w, bool has_b, bool has_s, bool has_t,
                                                uint32_t (&hp)[8]) {
  uint32_t a2 = 0u;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float2 y = f2_mul(f2_sub(bf16x2_to_f2(xp[e]), m2), r2);
    if (kAffine) {
      if (has_w) y = f2_mul(y, cw[e]);
      if (has_b) y = f2_add(y, cb[e]);
    }
    if (kMod) {
      if (has_s) y = f2_mul(y, cs[e]);
      if (has_t) y = f2_add(y, ct[e]);
    }
    // the quantizer's input is the bf16 tensor the unfused model would have produced
    hp[e] = f2_to_bf16x2(y);
    a2 = bf16x2_max_abs(a2, hp[e]);
  }
  return a2;
}

template <bool kQuantize, int kJ, bool kAffine, bool kMod>
__global__ void __launch_bounds__(kMaxThreads)
norm_mod_kernel(const NormArgs p) {
  constexpr int kR = RowsPerIter<kJ>::value;
  constexpr int kV = 2 * kR;                                // (sum, sum of squares) per row
  extern __shared__ __align__(128) uint8_t ring[];          // kStages slots of kR rows
  __shared__ __align__(16) float red[2][kV][kMaxWarps];
  __shared__ float red_max[kMaxWarps];
  __shared__ float enc_tab[128];                            // sweep 2: encode scale per scale byte
  __shared__ __align__(8) uint64_t full[kStages];
  __shared__ int abort_flag;
  const int T = blockDim.x;
  const int warps = T >> 5;
  const int units = p.cols >> 4;                            // 16-element blocks per row
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
#ifdef NVFP4_NORM_TAIL_MB
    const int64_t tail_rows = ((int64_t)NVFP4_NORM_TAIL_MB << 20) / row_bytes;
    const int hint = kQuantize ? 1 : (base >= p.rows - tail_rows ? 2 : 1);
#else
    const int hint = kQuantize ? 1 : 0;
#endif
    bulk_load(smem_u32(ring + (size_t)slot * slot_bytes),
              reinterpret_cast<const uint8_t*>(p.x) + base * row_bytes, bytes, bar, hint);
  };

  if (threadIdx.x == 0) {
    abort_flag = 0;
#pragma unroll
    for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(&full[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < 2 * kV * kMaxWarps; i += T) (&red[0][0][0])[i] = 0.0f;
  float s_enc = 0.0f;
  if (kQuantize) {
    s_enc = global_encode_scale(__ldg(p.amax_in));
    const float s_dec = __fdiv_rn(1.0f, s_enc);
    if (p.gscale_out && blockIdx.x == 0 && threadIdx.x == 0) *p.gscale_out = s_dec;
    // the encode scale depends on the block only through its scale byte: tabulate it
    for (int b = threadIdx.x; b < 128; b += T) enc_tab[b] = block_encode_scale((uint8_t)b, s_dec);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      const int64_t g = (int64_t)blockIdx.x + (int64_t)s * gridDim.x;
      if (g < groups) issue(g, s);
    }
  }

  // this thread's blocks and its slice of the per-column vectors, as pairs of fp32 lanes
  bool live[kJ];
  float2 cw[kAffine ? kJ : 1][8], cb[kAffine ? kJ : 1][8];
  float2 cs[kMod ? kJ : 1][8], ct[kMod ? kJ : 1][8];
  int64_t swz_kb[kJ];                      // K-block part of the swizzled scale offset
  bool has_w = false, has_b = false, has_s = false, has_t = false;
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
    const int u = threadIdx.x + j * T;
    live[j] = u < units;
    const int col = live[j] ? u * 16 : 0;
    swz_kb[j] = (int64_t)(u >> 2) * kSfAtomBytes + (u & 3);
    if (kAffine) {
      has_w = p.w != nullptr; has_b = p.b != nullptr;
      if (has_w) load16(p.w + col, cw[j]);
      if (has_b) load16(p.b + col, cb[j]);
    }
    if (kMod) {
      has_s = p.scale != nullptr; has_t = p.shift != nullptr;
      if (has_s) {
        load16(p.scale + col, cs[j]);
#pragma unroll
        for (int e = 0; e < 8; ++e) cs[j][e] = f2_add(make_float2(1.0f, 1.0f), cs[j][e]);
      }
      if (has_t) load16(p.shift + col, ct[j]);
    }
  }

  uint32_t amax_t = 0u;                 // bf16x2 running max of |h| (sweep 1)
  const float cols_f = (float)p.cols;

  // sweep 2 asks for a group's row statistics one group ahead: the load would otherwise sit
  // at the head of every group's dependency chain
  float mean_n[kR], rstd_n[kR];
  auto fetch_stats = [&](int64_t g) {
    const int64_t base = group_base(g);
#pragma unroll
    for (int r = 0; r < kR; ++r) {
      const int64_t rr = base + r < p.rows ? base + r : base;
      const float2 st = __ldg(reinterpret_cast<const float2*>(p.stats) + rr);
      mean_n[r] = st.x;
      rstd_n[r] = st.y;
    }
  };
  if (kQuantize && (int64_t)blockIdx.x < groups) fetch_stats(blockIdx.x);

  int slot = 0;
  uint32_t phase = 0;
  int parity = 0;                        // which reduction buffer this group uses
  for (int64_t g = blockIdx.x; g < groups; g += gridDim.x, parity ^= 1) {
    const int64_t base = group_base(g);
    wait_group(smem_u32(&full[slot]), phase, &abort_flag, p.status);
    const uint8_t* slot_ptr = ring + (size_t)slot * slot_bytes;
    bool row_ok[kR];
    uint32_t xp[kR][kJ][8];             // the rows' blocks, still packed bf16 pairs
    float pivot[kR];                    // first element of the row
#pragma unroll
    for (int r = 0; r < kR; ++r) {
      row_ok[r] = base + r < p.rows;
      const uint4* src = reinterpret_cast<const uint4*>(slot_ptr + (size_t)r * row_bytes);
      pivot[r] = (!kQuantize && !p.rms && row_ok[r])
                     ? bf16lo_to_f32(*reinterpret_cast<const uint32_t*>(src)) : 0.0f;
#pragma unroll
      for (int j = 0; j < kJ; ++j) {
        const bool on = live[j] && row_ok[r];
        const int u = threadIdx.x + j * T;
        const uint4 a = on ? src[2 * u] : make_uint4(0, 0, 0, 0);
        const uint4 b = on ? src[2 * u + 1] : make_uint4(0, 0, 0, 0);
        xp[r][j][0] = a.x; xp[r][j][1] = a.y; xp[r][j][2] = a.z; xp[r][j][3] = a.w;
        xp[r][j][4] = b.x; xp[r][j][5] = b.y; xp[r][j][6] = b.z; xp[r][j][7] = b.w;
      }
    }
    float mean[kR], rstd[kR];
    // once every thread holds its blocks the slot can take the group kStages ahead
    auto refill = [&]() {
      const int64_t gn = g + (int64_t)kStages * gridDim.x;
      if (threadIdx.x == 0 && gn < groups) issue(gn, slot);
    };
    if (!kQuantize) {
      // one pass: sums of d = x - pivot and of d^2 (the pivot, a sample of the row, keeps the
      // variance formula S2/n - (S1/n)^2 away from cancellation); RMSNorm needs S2 of x only
      float acc[kV];
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        const float2 p2 = make_float2(pivot[r], pivot[r]);
        float2 s1 = make_float2(0.0f, 0.0f), s2 = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < kJ; ++j) {
          if (live[j] && row_ok[r]) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float2 d = f2_sub(bf16x2_to_f2(xp[r][j][e]), p2);
              s1 = f2_add(s1, d);
              s2 = f2_fma(d, d, s2);
            }
          }
        }
        acc[2 * r] = s1.x + s1.y;
        acc[2 * r + 1] = s2.x + s2.y;
      }
      cta_sum<kV>(acc, red[parity], warps);
      refill();
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        const float m1 = acc[2 * r] / cols_f;
        const float var = fmaxf(acc[2 * r + 1] / cols_f - m1 * m1, 0.0f);
        mean[r] = p.rms ? 0.0f : pivot[r] + m1;
        rstd[r] = rsqrtf((p.rms ? acc[2 * r + 1] / cols_f : var) + p.eps);
        if (threadIdx.x == 0 && row_ok[r])
          reinterpret_cast<float2*>(p.stats)[base + r] = make_float2(mean[r], rstd[r]);
      }
    } else {
      __syncthreads();
      refill();
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        mean[r] = mean_n[r];
        rstd[r] = rstd_n[r];
      }
      if (g + gridDim.x < groups) fetch_stats(g + gridDim.x);
    }

#pragma unroll
    for (int r = 0; r < kR; ++r) {
      const int64_t row = base + r;
      const float2 m2 = make_float2(mean[r], mean[r]);
      const float2 r2 = make_float2(rstd[r], rstd[r]);
      // row part of the swizzled scale offset (the K-block part is per thread)
      const int64_t swz_row = (row >> 7) * (int64_t)p.k_atoms * kSfAtomBytes + (row & 31) * 16 +
                              ((row >> 5) & 3) * 4;
#pragma unroll
      for (int j = 0; j < kJ; ++j) {
        const int u = threadIdx.x + j * T;
        const bool on = live[j] && row_ok[r];
        uint32_t hp[8];
        const uint32_t a2 = normalize16<kAffine, kMod>(
            xp[r][j], m2, r2, cw[kAffine ? j : 0], cb[kAffine ? j : 0], cs[kMod ? j : 0],
            ct[kMod ? j : 0], has_w, has_b, has_s, has_t, hp);
        if (!kQuantize) {
          if (on) {
            amax_t = bf16x2_max_abs(amax_t, a2);
            if (p.h_out) {
              uint4* dst = p.h_out + (row * units + u) * 2;
              dst[0] = make_uint4(hp[0], hp[1], hp[2], hp[3]);
              dst[1] = make_uint4(hp[4], hp[5], hp[6], hp[7]);
            }
          }
        } else if (on) {
          const float amax_b = fmaxf(bf16lo_to_f32(a2), bf16hi_to_f32(a2));
          float d = __fmul_rn(div_by_6(amax_b), s_enc);
          d = fminf(d, FLT_MAX);
          const uint8_t sf = (uint8_t)__nv_cvt_float_to_fp8(d, __NV_SATFINITE, __NV_E4M3);
          const float enc = enc_tab[sf & 127];
          const float2 enc2 = make_float2(enc, enc);
          float2 q[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) q[e] = f2_mul(bf16x2_to_f2(hp[e]), enc2);
          uint2 out;
          out.x = f32x8_to_e2m1x8(q[0].x, q[0].y, q[1].x, q[1].y, q[2].x, q[2].y, q[3].x, q[3].y);
          out.y = f32x8_to_e2m1x8(q[4].x, q[4].y, q[5].x, q[5].y, q[6].x, q[6].y, q[7].x, q[7].y);
          __stcs(reinterpret_cast<uint2*>(p.packed) + row * units + u, out);
          if (p.sf_lin) p.sf_lin[row * units + u] = sf;
          if (p.sf_swz) p.sf_swz[swz_row + swz_kb[j]] = sf;
        }
      }
    }
    if (++slot == kStages) {
      slot = 0;
      phase ^= 1u;
    }
  }

  if (!kQuantize) {
    const float amax_f = fmaxf(bf16lo_to_f32(amax_t), bf16hi_to_f32(amax_t));
    const unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(amax_f));
    __syncthreads();
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
  if (rows < 0 || cols <= 0 || cols % kBlock != 0 || cols > kMaxJ * 16 * kMaxThreads ||
      rows >= ((int64_t)1 << 31))
    return NVFP4_ERR_BAD_ARG;
  if (rows > 0 && !x) return NVFP4_ERR_BAD_ARG;
  if (!aligned16(x)) return NVFP4_ERR_BAD_ALIGN;
  return NVFP4_OK;     // the device is checked last: bad arguments are refused on any machine
}

bool vec_ok(const float* p) { return aligned16(p); }

// Blocks per thread (1 or 2) and threads per CTA (a multiple of 32) for a row of `units`
// 16-element blocks.
void shape_for(int units, int* j, int* threads) {
  int J = 1;
  while (J < kMaxJ && units > J * kMaxThreads) J *= 2;
  // two blocks per thread whenever the row is long enough for two warps: the per-row
  // bookkeeping is then shared by 32 elements instead of 16 (measured 17-20 % faster)
#ifndef NVFP4_NORM_FORCE_J1
  if (units % 2 == 0 && units / 2 >= 64) J = 2;
#endif
  const int per = (units + J - 1) / J;
  *j = J;
  *threads = ((per + 31) / 32) * 32;
}

template <bool kQuantize, int kJ, bool kAffine, bool kMod>
int launch_variant(const NormArgs& a, int threads, cudaStream_t st) {
  auto kernel = norm_mod_kernel<kQuantize, kJ, kAffine, kMod>;
  constexpr int kR = RowsPerIter<kJ>::value;
  const size_t smem = (size_t)kStages * kR * a.cols * 2;
  // (dynamic shared memory limit, CTAs per SM) of the last geometry this variant saw on each
  // device: a model calls it with one row width over and over
  struct Geometry { size_t smem; int threads; int per_sm; };
  static Geometry cached[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  Geometry& c = cached[dev];
  if (c.per_sm < 1 || c.smem != smem || c.threads != threads) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return NVFP4_ERR_LAUNCH_FAILED;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem) != cudaSuccess ||
        n < 1)
      return NVFP4_ERR_LAUNCH_FAILED;
    c = Geometry{smem, threads, n};
  }
  const int per_sm = c.per_sm;
  const int64_t groups = (a.rows + kR - 1) / kR;
  const int64_t resident = (int64_t)sm_count() * per_sm;
  const unsigned grid = (unsigned)(groups < resident ? groups : resident);
  kernel<<<grid, threads, smem, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}

template <bool kQuantize>
int launch(const NormArgs& a, cudaStream_t st) {
  int J, threads;
  shape_for(a.cols / 16, &J, &threads);
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
  rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
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
  // the kernel stores 8-byte words of nibbles
  if ((reinterpret_cast<uintptr_t>(packed) & 7u) || !vec_ok(weight) || !vec_ok(bias) ||
      !vec_ok(scale) || !vec_ok(shift))
    return NVFP4_ERR_BAD_ALIGN;
  rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
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
