// Block-scaled FP4 (NVFP4) GEMM for sm_100a, hand-written on tcgen05:
//
//   D[M,N] bf16 = beta*C + gate[n] * act( alpha*ga*gb * sum_k (a*sfa)(b*sfb) + bias[n] )
//
// One persistent CTA per SM walks 128x256 output tiles.  Roles by warp:
//   warp 0     producer: TMA loads of the packed A/B tiles (128-byte swizzle) and
//              bulk copies of the pre-swizzled scale atoms into a 4-stage ring
//   warp 1     tensor-core issuer: tcgen05.mma kind::mxf4nvf4 (16-element blocks,
//              UE4M3 scales) accumulates fp32 in tensor memory
//   warps 2-5  epilogue: tcgen05.ld of the accumulator, fused scale / bias /
//              GELU-tanh / gate / residual, bf16 stores
//   warps 6-9  scale-factor movers: read a stage's scale atoms from shared
//              memory and write them into tensor memory with tcgen05.st
//
// The scale factors go through registers and tcgen05.st rather than
// tcgen05.cp: measured on B200, every tcgen05.cp costs the tensor pipe about
// 45 cycles whatever its size, and a 128x256 tile needs three per MMA, which
// capped the kernel near 3.4 PFLOP/s; tcgen05.st runs beside the MMAs.
//
// Tensor memory (512 columns): two 256-column accumulators at columns 0 and
// 160 that overlap in [160,256), and two 48-column scale-factor buffers at
// 416 and 464.  The epilogue drains the overlapping 96 columns first and then
// lets the issuer start the next tile in the other accumulator, so the rest
// of the epilogue runs under the next tile's main loop.
//
// Every wait is bounded: when a wait gives up the kernel records where in
// *status, raises a CTA-wide abort flag, and every role leaves its loop so
// that tensor memory is released and the CTA exits.
#include <cuda.h>

#include "nvfp4_common.cuh"

namespace nvfp4 {
namespace gemm {

constexpr int BM = 128;                  // tile rows (= TMEM lanes)
constexpr int BN = 256;                  // tile columns (= one MMA N)
constexpr int BK = 256;                  // K elements per stage (128 bytes: one swizzle row)
constexpr int kStages = 4;
constexpr int kABytes = BM * BK / 2;     // 16384
constexpr int kBBytes = BN * BK / 2;     // 32768
constexpr int kSfaBytes = (BM / 128) * (BK / 64) * kSfAtomBytes;  // 2048
constexpr int kSfbBytes = (BN / 128) * (BK / 64) * kSfAtomBytes;  // 4096
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/;
constexpr int kThreads = 320;
constexpr int kEpiThreads = 128;
constexpr int kSfThreads = 128;
constexpr int kTmemCols = 512;
constexpr int kAccCol1 = 160;            // second accumulator's first column
constexpr int kSfCol0 = 416;             // scale factors live in [416,512)
constexpr int kSfUnitKb = 2;             // K-blocks (MMAs) per scale-factor hand-over unit
constexpr int kSfUnitCols = 12 * kSfUnitKb;   // per K-block: 4 columns of SFA + 8 of SFB
constexpr int kSfRing = 96 / kSfUnitCols;     // units resident in tensor memory
constexpr int kSfUnitsPerStage = (BK / 64) / kSfUnitKb;
static_assert(kSfUnitKb == 1 || kSfUnitKb == 2 || kSfUnitKb == 4, "unit must divide a stage");
constexpr int kEpiChunk = 32;            // accumulator columns per epilogue step
constexpr int kOverlapChunks = (256 - kAccCol1) / kEpiChunk;  // chunks shared by both accumulators
constexpr long long kWaitCycles = 4000000000LL;  // ~2 s at 2 GHz

static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB per-CTA shared memory limit");

// ----------------------------------------------------------- PTX wrappers --

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false (after raising the abort flag and recording
// `where`) when the barrier does not flip within kWaitCycles, or when another
// role has already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, where);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint32_t bar, uint32_t dst,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X"
      " [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
        "r"(sfb_tmem)
      : "memory");
}

// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread.
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x N columns <- N registers per thread (scale factors into tensor memory).
template <int N>
__device__ __forceinline__ void tc_st_sf(uint32_t taddr, const uint32_t* v);
template <>
__device__ __forceinline__ void tc_st_sf<4>(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3])
               : "memory");
}
template <>
__device__ __forceinline__ void tc_st_sf<8>(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
template <>
__device__ __forceinline__ void tc_st_sf<16>(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
               : "memory");
}
template <>
__device__ __forceinline__ void tc_st_sf<32>(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
               : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major operand rows of 128 bytes with the
// 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO), descriptor
// version 1, layout code 2.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::mxf4nvf4: A and B E2M1 (code 1) both K-major,
// N at bits 17-22 in units of 8, UE4M3 scales (bit 23 clear), M at bits 24-28
// in units of 16, scale-factor ids 0, K = 64 (bit 31 clear).
constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                            ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ float gelu_tanh(float x) {
  // 0.5 x (1 + tanh(u)) = x * sigmoid(2u), u = sqrt(2/pi) (x + 0.044715 x^3)
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return __fdividef(x, 1.0f + __expf(-2.0f * u));
}

struct Params {
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* ga;
  const float* gb;
  const __nv_bfloat16* c;
  const __nv_bfloat16* bias;
  const float* gate;
  __nv_bfloat16* d;
  int* status;
  float alpha, beta;
  int M, N, K;
  int m_tiles, n_tiles, k_tiles, k_atoms;
  int act;
};

__global__ void __launch_bounds__(kThreads, 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                  const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  // stage s: [A 16K][B 32K][SFA 2K][SFB 4K]; A and B start on 1024-byte boundaries
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kStages * kStageBytes + 240);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + kStages * kStageBytes + 244);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
  const uint32_t acc_empty_bar = bar_base + 8u * (2 * kStages + 2);
  auto sf_full_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 3 + b); };
  auto sf_empty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 3 + kSfRing + b); };
  static_assert(8 * (2 * kStages + 3 + 2 * kSfRing) <= 240, "barriers overrun their area");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full_bar(0), 1);
    mbar_init(acc_full_bar(1), 1);
    mbar_init(acc_empty_bar, kEpiThreads);
    for (int b = 0; b < kSfRing; ++b) {
      mbar_init(sf_full_bar(b), kSfThreads);
      mbar_init(sf_empty_bar(b), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------- producer ----
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int mt = tile % p.m_tiles;
        const int nt = tile / p.m_tiles;
        const uint8_t* sfa_row = p.sfa + (size_t)mt * p.k_atoms * kSfAtomBytes;
        const uint8_t* sfb_row0 = p.sfb + (size_t)(2 * nt) * p.k_atoms * kSfAtomBytes;
        const uint8_t* sfb_row1 = sfb_row0 + (size_t)p.k_atoms * kSfAtomBytes;
        for (int kt = 0; kt < p.k_tiles; ++kt) {
          ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, 0x100 + s);
          if (!ok) break;
          const uint32_t st = smem_base + s * kStageBytes;
          mbar_expect_tx(full_bar(s), kStageBytes);
          tma_load_2d(&map_a, full_bar(s), st, kt * (BK / 2), mt * BM);
          tma_load_2d(&map_b, full_bar(s), st + kABytes, kt * (BK / 2), nt * BN);
          const size_t koff = (size_t)kt * (BK / 64) * kSfAtomBytes;
          bulk_load(st + kABytes + kBBytes, sfa_row + koff, kSfaBytes, full_bar(s));
          bulk_load(st + kABytes + kBBytes + kSfaBytes, sfb_row0 + koff, kSfbBytes / 2,
                    full_bar(s));
          bulk_load(st + kABytes + kBBytes + kSfaBytes + kSfbBytes / 2, sfb_row1 + koff,
                    kSfbBytes / 2, full_bar(s));
          if (++s == kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      if (!ok) {
        // let copies already in flight land before the CTA's memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------- tensor-core issuer ----
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int t = 0;
      uint32_t un = 0;  // scale-factor units consumed so far: ring slot un % kSfRing
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++t) {
        const uint32_t acc = tmem_base + ((t & 1) ? kAccCol1 : 0);
        if (t > 0) {
          ok = mbar_wait(acc_empty_bar, (uint32_t)(t - 1) & 1u, abort_flag, p.status, 0x300);
          if (!ok) break;
          tc_fence_after();
        }
        for (int kt = 0; kt < p.k_tiles; ++kt) {
          ok = mbar_wait(full_bar(s), ph, abort_flag, p.status, 0x200 + s);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = smem_base + s * kStageBytes;
          const uint64_t da = desc_sw128(st);
          const uint64_t db = desc_sw128(st + kABytes);
#pragma unroll
          for (int u = 0; u < kSfUnitsPerStage; ++u, ++un) {
            const uint32_t slot = un % kSfRing;
            ok = mbar_wait(sf_full_bar(slot), (un / kSfRing) & 1u, abort_flag, p.status,
                           0x600 + slot);
            if (!ok) break;
            tc_fence_after();
            // unit layout: SFA of its K-block i at +4i, SFB at +4*kSfUnitKb + 8i
            const uint32_t sf_t = tmem_base + kSfCol0 + slot * kSfUnitCols;
#pragma unroll
            for (int i = 0; i < kSfUnitKb; ++i) {
              const int j = u * kSfUnitKb + i;
              // 64 elements = 32 bytes along K inside the swizzled row: +2 in 16-byte units
              tc_mma_nvf4(acc, da + 2 * j, db + 2 * j, kIdesc, sf_t + 4 * i,
                          sf_t + 4 * kSfUnitKb + 8 * i, (kt | j) != 0);
            }
            tc_commit(sf_empty_bar(slot));
          }
          if (!ok) break;
          tc_commit(empty_bar(s));
          if (++s == kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(acc_full_bar(t & 1));
      }
    }
  } else if (warp >= 6) {
    // --------------------------------------------- scale-factor movers ----
    // Lane l of every lane quarter holds, per 512-byte atom, the 16 bytes of rows
    // l, l+32, l+64, l+96 (4 K-blocks each): exactly four tensor-memory columns.
    const int q = warp & 3;
    int s = 0;
    uint32_t ph = 0, un = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      for (int kt = 0; kt < p.k_tiles; ++kt) {
        ok = mbar_wait(full_bar(s), ph, abort_flag, p.status, 0x500 + s);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint8_t* sf_s = smem_gen + s * kStageBytes + kABytes + kBBytes;
        uint32_t v[12 * (BK / 64)];  // unit u, K-block i: SFA at 4i, SFB at 4*kSfUnitKb + 8i
#pragma unroll
        for (int j = 0; j < BK / 64; ++j) {
          const uint4 a4 = *reinterpret_cast<const uint4*>(sf_s + j * kSfAtomBytes + lane * 16);
          const uint4 b0 = *reinterpret_cast<const uint4*>(sf_s + kSfaBytes + j * kSfAtomBytes +
                                                           lane * 16);
          const uint4 b1 = *reinterpret_cast<const uint4*>(sf_s + kSfaBytes + kSfbBytes / 2 +
                                                           j * kSfAtomBytes + lane * 16);
          const int ua = (j / kSfUnitKb) * kSfUnitCols + 4 * (j % kSfUnitKb);
          const int ub = (j / kSfUnitKb) * kSfUnitCols + 4 * kSfUnitKb + 8 * (j % kSfUnitKb);
          v[ua] = a4.x; v[ua + 1] = a4.y; v[ua + 2] = a4.z; v[ua + 3] = a4.w;
          v[ub] = b0.x; v[ub + 1] = b0.y; v[ub + 2] = b0.z; v[ub + 3] = b0.w;
          v[ub + 4] = b1.x; v[ub + 5] = b1.y; v[ub + 6] = b1.z; v[ub + 7] = b1.w;
        }
#pragma unroll
        for (int u = 0; u < kSfUnitsPerStage; ++u, ++un) {
          const uint32_t slot = un % kSfRing;
          ok = mbar_wait(sf_empty_bar(slot), ((un / kSfRing) & 1u) ^ 1u, abort_flag, p.status,
                         0x700 + slot);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + kSfCol0 + slot * kSfUnitCols;
          tc_st_sf<4 * kSfUnitKb>(ta, v + u * kSfUnitCols);
          tc_st_sf<8 * kSfUnitKb>(ta + 4 * kSfUnitKb, v + u * kSfUnitCols + 4 * kSfUnitKb);
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(sf_full_bar(slot));
        }
        if (!ok) break;
        if (++s == kStages) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------- epilogue ----
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    const float scale = p.alpha * (p.ga ? __ldg(p.ga) : 1.0f) * (p.gb ? __ldg(p.gb) : 1.0f);
    bool ok = true;
    int t = 0;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++t) {
      const int mt = tile % p.m_tiles;
      const int nt = tile / p.m_tiles;
      const int buf = t & 1;
      ok = mbar_wait(acc_full_bar(buf), (uint32_t)(t >> 1) & 1u, abort_flag, p.status, 0x400 + buf);
      // the whole warp must agree before the .sync.aligned loads below
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = mt * BM + q * 32 + lane;
      const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16) + (buf ? kAccCol1 : 0);
      // The chunks both accumulators share are read into registers first, and the issuer is
      // released before any of them is processed.
      constexpr int kChunks = BN / kEpiChunk;
      uint32_t ro[kOverlapChunks][kEpiChunk];
#pragma unroll
      for (int ci = 0; ci < kOverlapChunks; ++ci)
        tc_ld_32x32(acc + (buf ? ci : ci + kChunks - kOverlapChunks) * kEpiChunk, ro[ci]);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(acc_empty_bar);
#pragma unroll
      for (int ci = 0; ci < kChunks; ++ci) {
        // accumulator 0 shares its last kOverlapChunks chunks with the other accumulator,
        // accumulator 1 its first ones
        const int c = buf ? ci : (ci + kChunks - kOverlapChunks) % kChunks;
        uint32_t r[kEpiChunk];
        if (ci < kOverlapChunks) {
#pragma unroll
          for (int e = 0; e < kEpiChunk; ++e) r[e] = ro[ci][e];
        } else {
          tc_ld_32x32(acc + c * kEpiChunk, r);
          tc_wait_ld();
        }
        const int col0 = nt * BN + c * kEpiChunk;
        if (row < p.M) {
          __nv_bfloat16* drow = p.d + (size_t)row * p.N + col0;
          const __nv_bfloat16* crow = p.c ? p.c + (size_t)row * p.N + col0 : nullptr;
#pragma unroll
          for (int g = 0; g < kEpiChunk / 8; ++g) {
            if (col0 + g * 8 < p.N) {
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[g * 8 + e]) * scale;
              if (p.bias) {
                const uint4 bb = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + g * 8));
                const uint32_t bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  v[2 * e] += bf16lo_to_f32(bw[e]);
                  v[2 * e + 1] += bf16hi_to_f32(bw[e]);
                }
              }
              if (p.act == NVFP4_ACT_GELU_TANH) {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]);
              }
              if (p.gate) {
                const float4 g0 = __ldg(reinterpret_cast<const float4*>(p.gate + col0 + g * 8));
                const float4 g1 = __ldg(reinterpret_cast<const float4*>(p.gate + col0 + g * 8 + 4));
                v[0] *= g0.x; v[1] *= g0.y; v[2] *= g0.z; v[3] *= g0.w;
                v[4] *= g1.x; v[5] *= g1.y; v[6] *= g1.z; v[7] *= g1.w;
              }
              if (crow) {
                const uint4 cc = __ldg(reinterpret_cast<const uint4*>(crow + g * 8));
                const uint32_t cw[4] = {cc.x, cc.y, cc.z, cc.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  v[2 * e] += p.beta * bf16lo_to_f32(cw[e]);
                  v[2 * e + 1] += p.beta * bf16hi_to_f32(cw[e]);
                }
              }
              uint32_t o[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
                o[e] = *reinterpret_cast<uint32_t*>(&h);
              }
              *reinterpret_cast<uint4*>(drow + g * 8) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

// ------------------------------------------------------------- host side ----

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault,
                                         &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// Tensor map over a packed FP4 matrix seen as bytes: [rows][K/2], box of
// 128 bytes x box_rows, 128-byte swizzle, out-of-range rows/bytes read as 0.
static bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k_bytes,
                     int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)k_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k_bytes};
  cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1u, 1u};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int sm_count() {
  static int cached[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

}  // namespace gemm
}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_gemm(const uint8_t* a_packed, const uint8_t* b_packed,
                          const uint8_t* a_scales_swizzled, const uint8_t* b_scales_swizzled,
                          const float* a_global_scale_dev, const float* b_global_scale_dev,
                          int64_t M, int64_t N, int64_t K, float alpha, float beta,
                          const void* c_bf16, const void* bias_bf16, const float* gate_f32, int act,
                          void* d_bf16, int* status_dev, void* stream) {
  if (M < 0 || N < 0 || K < 0 || N % 8 != 0 || K % 32 != 0) return NVFP4_ERR_BAD_ARG;
  if (act != NVFP4_ACT_NONE && act != NVFP4_ACT_GELU_TANH) return NVFP4_ERR_BAD_ARG;
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return NVFP4_ERR_BAD_ARG;
  if (M == 0 || N == 0) return NVFP4_OK;
  if (K == 0) return NVFP4_ERR_BAD_ARG;
  if (!a_packed || !b_packed || !a_scales_swizzled || !b_scales_swizzled || !d_bf16)
    return NVFP4_ERR_BAD_ARG;
  if (!aligned16(a_packed) || !aligned16(b_packed) || !aligned16(a_scales_swizzled) ||
      !aligned16(b_scales_swizzled) || !aligned16(d_bf16) || !aligned16(c_bf16) ||
      !aligned16(bias_bf16) || !aligned16(gate_f32))
    return NVFP4_ERR_BAD_ALIGN;
  int rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;

  CUtensorMap map_a, map_b;
  if (!gemm::make_map(&map_a, a_packed, M, K / 2, gemm::BM) ||
      !gemm::make_map(&map_b, b_packed, N, K / 2, gemm::BN))
    return NVFP4_ERR_LAUNCH_FAILED;

  gemm::Params p;
  p.sfa = a_scales_swizzled;
  p.sfb = b_scales_swizzled;
  p.ga = a_global_scale_dev;
  p.gb = b_global_scale_dev;
  p.c = reinterpret_cast<const __nv_bfloat16*>(c_bf16);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias_bf16);
  p.gate = gate_f32;
  p.d = reinterpret_cast<__nv_bfloat16*>(d_bf16);
  p.status = status_dev;
  p.alpha = alpha;
  p.beta = beta;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.m_tiles = (int)((M + gemm::BM - 1) / gemm::BM);
  p.n_tiles = (int)((N + gemm::BN - 1) / gemm::BN);
  p.k_tiles = (int)((K + gemm::BK - 1) / gemm::BK);
  p.k_atoms = (int)sf_k_atoms(K);
  p.act = act;

  static bool attr_set[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm::nvfp4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             gemm::kSmemBytes) != cudaSuccess)
      return NVFP4_ERR_LAUNCH_FAILED;
    attr_set[dev] = true;
  }
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
  const int sms = gemm::sm_count();
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  gemm::nvfp4_gemm_kernel<<<grid, gemm::kThreads, gemm::kSmemBytes,
                            reinterpret_cast<cudaStream_t>(stream)>>>(map_a, map_b, p);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}
