// Non-causal bf16 attention for sm_100a, head dimension 128, with the maximum |o| of the
// output folded into the kernel (the NVFP4 quantizer in front of the attention-out linear
// then needs no amax pass of its own).  Replaces the library attention at the reference's call
// sites fx/src/s4/models/wan22/wan_transformer_fast.py:47-58 (flash_attn_qkvpacked_func) and
// fx/src/s4/models/wan22/wan_transformer.py:126-129,164-167 (scaled_dot_product_attention).
//
// One CTA owns 256 query rows of one head as two 128-row tiles, and walks the keys 128 at a
// time.  Per key tile and query tile:
//     S = Q K^T           tcgen05.mma, both operands from shared memory, S in tensor memory
//     P = exp2(S*c - m)   two threads per query row (64 keys each): tcgen05.ld, row max (the
//                         halves meet through shared memory), exp2, row sum, bf16 P written
//                         back over S with tcgen05.st
//     O += P V            tcgen05.mma with P read from tensor memory and V (keys x d, d
//                         contiguous: an MN-major operand) from shared memory
// The two query tiles alternate on the tensor pipe: while the threads of one tile run the
// softmax, the MMAs of the other tile execute.  The running maximum is only raised when the new
// row maximum exceeds it by more than 2^8 (exp2 domain); O is then rescaled in place by the
// softmax threads themselves, which is safe because the S tile they hold was committed after
// the previous P V product of the same query tile had completed.
//
// Tensor memory (512 columns): S0/P0 at 0, S1/P1 at 128, O0 at 256, O1 at 384.
// Shared memory: Q0, Q1 (32 KiB each), a ring of four 32 KiB K/V tiles (K0 V0 K1 V1 ...),
// every tile as two 128-row x 128-byte halves in the 128-byte swizzle that TMA writes.
//
// Warps 0-7: softmax + epilogue of query tile 0 (warp & 3 = the 32-lane quarter of tensor memory
// it may touch, bit 2 = which 64 keys); 8-15: of tile 1; 16: TMA loads; 17: MMA issue; 18-19
// idle (they complete the fifth warpgroup, which hands its registers to the softmax warps).
// Two warps per scheduler and tile matter: one warp alone issues in order and leaves the FMA,
// ALU and special-function pipes waiting on each other (measured: 1730 cycles per tile with
// four warps per tile against a tensor-pipe budget of 1024).
// Every wait is bounded: when one runs out the kernel records where in *status, raises a
// CTA-wide flag so that every role leaves its loop, and releases its tensor memory.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "nvfp4_common.cuh"

namespace nvfp4 {
namespace attn {

constexpr int kD = 128;                   // head dimension
constexpr int kBQ = 128;                  // query rows per tile (= tensor-memory lanes)
constexpr int kBKV = 128;                 // keys per tile
constexpr int kQTiles = 2;                // query tiles per CTA
constexpr int kHalfBytes = 128 * 128;     // 128 rows x 64 bf16
constexpr int kTileBytes = 2 * kHalfBytes;
constexpr int kKvSlots = 4;
constexpr int kDataBytes = (kQTiles + kKvSlots) * kTileBytes;
constexpr int kSmemBytes = kDataBytes + 1024 /*align slack*/ + 256 /*barriers*/ + 4096 /*row exchange*/;
constexpr int kSoftmaxWarps = 16;         // eight per query tile
constexpr int kLoaderWarp = 16, kIssuerWarp = 17;
constexpr int kThreads = 640;             // five warpgroups
constexpr int kRegsSoftmax = 104, kRegsHelper = 56;
constexpr int kXchgBytes = kQTiles * 2 * 2 * kBQ * 4;   // [tile][parity][half][row] floats
constexpr int kTmemCols = 512;
constexpr int kColS = 0, kColO = 256;     // + 128 * tile
constexpr float kRescaleStep = 8.f;       // raise the running maximum only past 2^8
#ifndef NVFP4_ATTN_FMA_EXP_EVERY
#define NVFP4_ATTN_FMA_EXP_EVERY 4
#endif
// Every kFmaExpEvery-th element pair takes 2^x on the FMA pipe (0: none), spread evenly so that
// the special-function unit works through its pairs while the FMA pipe works through these.
constexpr int kFmaExpEvery = NVFP4_ATTN_FMA_EXP_EVERY;
constexpr long long kWaitCycles = 4000000000LL;  // ~2 s at 2 GHz
constexpr int kErrBase = 0xA00;

static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB per-CTA shared memory limit");

struct Params {
  int64_t q_len, kv_len;
  int kv_tiles;
  float scale_log2;              // softmax scale * log2(e)
  uint8_t* o;                    // bf16 [q_len][heads][128], strided
  int64_t o_row_bytes, o_head_bytes;
  unsigned* amax;                // max |o| as float bits (atomicMax), or null
  int* status;
};

// ----------------------------------------------------------- PTX wrappers --

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t e;
  asm volatile(
      "{\n\t.reg .pred P;\n\t.reg .b32 r;\n\t"
      "elect.sync r|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(e));
  return e;
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
      "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}"
      ::"r"(bar), "r"(bytes), "r"(on)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cta.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false (after raising the abort flag and recording `where`) when the barrier
// does not flip within kWaitCycles or another role has already given up.
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
// One 128-row x 64-column bf16 box of a [tokens][heads][128] tensor into shared memory.
__device__ __forceinline__ void tma_load_3d(const CUtensorMap* map, uint32_t bar, uint32_t dst, int x,
                                            int y, int z, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %6, 0;\n\t"
      "@q cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];\n\t}"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(on)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on `bar` once this thread's earlier tcgen05 operations have completed.
__device__ __forceinline__ void tc_commit(uint32_t bar, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar), "r"(on)
      : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(on)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(on)
      : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns <-> 32 registers per thread.
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
        "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};"
               ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x for a pair, x <= 8, on the FMA pipe instead of the special-function unit (which is the
// scarcer resource here: 16 results per clock per SM against 128 FMA lanes).  x = i + f with
// f in [-0.5, 0.5] by magic-number rounding, a cubic for 2^f (relative error 7.5e-5, a fiftieth
// of a bf16 rounding step), and i added into the exponent field.  x is clamped at -126, where
// the result (1e-38) is already nothing next to the row's largest term.
__device__ __forceinline__ float2 exp2_fma(float2 x) {
  const float kMagic = 12582912.f;   // 1.5 * 2^23: the sum's low mantissa bits hold round(x)
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 magic = make_float2(kMagic, kMagic);
  const float2 r = f2_add(x, magic);
  const float2 f = f2_sub(x, f2_sub(r, magic));
  float2 y = f2_fma(f, make_float2(0.0551716685f, 0.0551716685f), make_float2(0.242611125f, 0.242611125f));
  y = f2_fma(y, f, make_float2(0.693260968f, 0.693260968f));
  y = f2_fma(y, f, make_float2(0.999928057f, 0.999928057f));
  y.x = __int_as_float(__float_as_int(y.x) + (__float_as_int(r.x) << 23));
  y.y = __int_as_float(__float_as_int(y.y) + (__float_as_int(r.y) << 23));
  return y;
}

// Shared-memory matrix descriptors, 128-byte swizzle (layout code 2, descriptor version 1).
// K-major operand (Q, K: rows of 64 contraction elements = 128 bytes): 8-row groups 1024 bytes
// apart (stride offset); the leading offset is unused.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand (V: each key is a row of 64 output-dimension elements = 128 bytes): groups of
// 8 keys 1024 bytes apart (stride offset), the second 64 output dimensions one half tile further
// (leading offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(kHalfBytes >> 4) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: fp32 accumulate (bit 4), A and B bf16 (code 1 at bits 7
// and 10), B MN-major when `b_mn` (bit 16), N = 128 at bits 17-22 in units of 8, M = 128 at
// bits 24-28 in units of 16.
__device__ __forceinline__ uint32_t make_idesc(bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(128 >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}

// ------------------------------------------------------------------ kernel --

__global__ void __launch_bounds__(kThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kDataBytes;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kDataBytes + 248);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + kDataBytes + 252);
  auto q_smem = [&](int t) { return smem_base + (uint32_t)t * kTileBytes; };
  auto kv_smem = [&](int s) { return smem_base + (uint32_t)(kQTiles + s) * kTileBytes; };
  auto q_full = [&]() { return bar_base; };
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + kKvSlots + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (1 + 2 * kKvSlots + t); };
  auto p_full = [&](int t) { return bar_base + 8u * (3 + 2 * kKvSlots + t); };
  auto o_full = [&](int t) { return bar_base + 8u * (5 + 2 * kKvSlots + t); };
  static_assert(8 * (7 + 2 * kKvSlots) <= 248, "barriers overrun their area");
  float* xchg = reinterpret_cast<float*>(smem_gen + kDataBytes + 256);
  static_assert(kXchgBytes <= 4096, "row exchange overruns its area");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int64_t q0 = (int64_t)blockIdx.x * (kQTiles * kBQ);
  const int n = p.kv_tiles;

  if (threadIdx.x == 0) {
    mbar_init(q_full(), 1);
    for (int s = 0; s < kKvSlots; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int t = 0; t < kQTiles; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), 2 * kBQ);     // every softmax thread of the tile arrives
      mbar_init(o_full(t), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == kIssuerWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= kSoftmaxWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsHelper));
  }
  if (warp == kLoaderWarp) {
    // ----------------------------------------------------------- loader ----
    const uint32_t on = elect_one();
    bool ok = true;
    mbar_expect_tx(q_full(), kQTiles * kTileBytes, on);
    for (int t = 0; t < kQTiles; ++t)
      for (int h = 0; h < 2; ++h)
        tma_load_3d(&map_q, q_full(), q_smem(t) + h * kHalfBytes, h * 64, head,
                    (int)(q0 + t * kBQ), on);
    for (int i = 0; i < 2 * n; ++i) {
      const int s = i & (kKvSlots - 1);
      if (i >= kKvSlots) {
        ok = mbar_wait(kv_empty(s), (uint32_t)((i / kKvSlots) + 1) & 1u, abort_flag, p.status,
                       kErrBase + 0x30 + s);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      const CUtensorMap* map = (i & 1) ? &map_v : &map_k;
      mbar_expect_tx(kv_full(s), kTileBytes, on);
      for (int h = 0; h < 2; ++h)
        tma_load_3d(map, kv_full(s), kv_smem(s) + h * kHalfBytes, h * 64, head, (i >> 1) * kBKV, on);
    }
    if (!ok) {
      // let copies already in flight land before the CTA's memory is released
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) {
      }
    }
  } else if (warp == kIssuerWarp) {
    // ------------------------------------------------------- MMA issuer ----
    const uint32_t on = elect_one();
    const uint32_t idesc_s = make_idesc(false);
    const uint32_t idesc_pv = make_idesc(true);
    auto issue_s = [&](int t, int slot) {
      // S_t = Q_t K^T: eight steps of 16 contraction elements (32 bytes inside the swizzled row,
      // the second 64 elements one half tile further)
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) {
        const uint32_t off = (uint32_t)(ks >> 2) * kHalfBytes + (uint32_t)(ks & 3) * 32u;
        tc_mma_ss(tmem_base + kColS + t * 128, desc_kmajor(q_smem(t) + off),
                  desc_kmajor(kv_smem(slot) + off), idesc_s, ks > 0, on);
      }
      tc_commit(s_full(t), on);
    };
    bool ok = mbar_wait(q_full(), 0, abort_flag, p.status, kErrBase + 0x10);
    if (ok) ok = mbar_wait(kv_full(0), 0, abort_flag, p.status, kErrBase + 0x20);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      issue_s(0, 0);
      issue_s(1, 0);
      tc_commit(kv_empty(0), on);
    }
    for (int j = 0; ok && j < n; ++j) {
      const int iv = 2 * j + 1, ik = 2 * j + 2;
      const int sv = iv & (kKvSlots - 1), sk = ik & (kKvSlots - 1);
      const bool has_next = j + 1 < n;
      ok = mbar_wait(kv_full(sv), (uint32_t)(iv / kKvSlots) & 1u, abort_flag, p.status,
                     kErrBase + 0x20 + sv);
      if (ok && has_next)
        ok = mbar_wait(kv_full(sk), (uint32_t)(ik / kKvSlots) & 1u, abort_flag, p.status,
                       kErrBase + 0x20 + sk);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      for (int t = 0; t < kQTiles; ++t) {
        ok = mbar_wait(p_full(t), (uint32_t)j & 1u, abort_flag, p.status, kErrBase + 0x50 + t);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // O_t += P_t V: sixteen keys per step = eight 32-bit columns of P, two 8-key groups of V
#pragma unroll
        for (int ks = 0; ks < kBKV / 16; ++ks)
          tc_mma_ts(tmem_base + kColO + t * 128, tmem_base + kColS + t * 128 + ks * 8,
                    desc_mnmajor(kv_smem(sv) + (uint32_t)ks * 2048u), idesc_pv, (j > 0 || ks > 0), on);
        if (has_next)
          issue_s(t, sk);
        else
          tc_commit(o_full(t), on);
      }
      if (!ok) break;
      tc_commit(kv_empty(sv), on);
      if (has_next) tc_commit(kv_empty(sk), on);
    }
  } else if (warp < kSoftmaxWarps) {
    // ----------------------------------------------- softmax + epilogue ----
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int t = warp >> 3;
    const int half = (warp >> 2) & 1;          // which 64 keys of the tile / 64 columns of O
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;         // row in the tile
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + kColS + t * 128 + half * 64;
    const uint32_t p_addr = tmem_base + lane_addr + kColS + t * 128 + half * 32;
    const uint32_t o_addr = tmem_base + lane_addr + kColO + t * 128 + half * 64;
    const int64_t row = q0 + t * kBQ + r;
    const int pair_bar = 1 + t * 4 + quarter;  // named barrier of the two warps that share these rows
    auto xslot = [&](int parity, int h) { return xchg + ((t * 2 + parity) * 2 + h) * kBQ + r; };
    const float c = p.scale_log2;
    float m_ref = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      ok = mbar_wait(s_full(t), (uint32_t)j & 1u, abort_flag, p.status, kErrBase + 0x40 + t);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        // The partner warp may have seen this barrier flip a moment before the abort flag went
        // up and be on its way to this key tile's meeting point, which has no time limit of its
        // own: arrive there without waiting, so that it gets through.  It cannot reach the next
        // meeting point: the next S needs this warp's probabilities, which never come.
        asm volatile("bar.arrive %0, %1;" ::"r"(pair_bar), "n"(64) : "memory");
        break;
      }
      tc_fence_after();
      uint32_t s[64];
      tc_ld32(s_addr, s);
      tc_ld32(s_addr + 32, s + 32);
      tc_wait_ld();
      if (j == n - 1) {
        // keys past the end of the sequence (their K rows were read as zeros) get no weight
        const int valid = (int)(p.kv_len - (int64_t)j * kBKV) - half * 64;
        if (valid < 64) {
#pragma unroll
          for (int e = 0; e < 64; ++e)
            if (e >= valid) s[e] = 0xFF800000u;   // -inf
        }
      }
      float mx0 = max3(__uint_as_float(s[0]), __uint_as_float(s[1]), __uint_as_float(s[2]));
      float mx1 = max3(__uint_as_float(s[3]), __uint_as_float(s[4]), __uint_as_float(s[5]));
      float mx2 = fmaxf(__uint_as_float(s[6]), __uint_as_float(s[7]));
      float mx3 = -INFINITY;
#pragma unroll
      for (int e = 8; e < 64; e += 8) {
        mx0 = max3(mx0, __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
        mx1 = max3(mx1, __uint_as_float(s[e + 2]), __uint_as_float(s[e + 3]));
        mx2 = max3(mx2, __uint_as_float(s[e + 4]), __uint_as_float(s[e + 5]));
        mx3 = max3(mx3, __uint_as_float(s[e + 6]), __uint_as_float(s[e + 7]));
      }
      // the two halves of a row meet: after this barrier both warps that own these 32 rows have
      // finished reading S, so the probabilities may go over it
      float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      *xslot(j & 1, half) = mx;
      asm volatile("bar.sync %0, %1;" ::"r"(pair_bar), "n"(64) : "memory");
      mx = fmaxf(mx, *xslot(j & 1, half ^ 1));
      const float mc = mx * c;
      if (j == 0) {
        m_ref = mc;
      } else {
        const bool raise = mc - m_ref > kRescaleStep;
        if (__any_sync(0xffffffffu, raise)) {
          // the previous P V of this tile completed before this S was committed: O is at rest
          const float alpha = raise ? ex2(m_ref - mc) : 1.f;
          if (raise) m_ref = mc;
          l *= alpha;
#pragma unroll 1
          for (int g = 0; g < 64 / 8; ++g) {
            uint32_t o[8];
            tc_ld8(o_addr + g * 8, o);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tc_st8(o_addr + g * 8, o);
          }
        }
      }
      // p = exp2(s*c - m); the row sum in fp32 before the rounding to bf16; bf16 pairs go back
      // over S (32 packed columns per thread)
      const float2 c2 = make_float2(c, c);
      const float2 nm2 = make_float2(-m_ref, -m_ref);
      float2 sum0 = make_float2(0.f, 0.f), sum1 = make_float2(0.f, 0.f);
      // three sweeps rather than one loop, so that consecutive exponentials do not depend on one
      // another's results: the special-function unit takes one warp instruction every 8 cycles
      // and a sum or a pack right behind each would stall on it
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float2 x = f2_fma(make_float2(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1])), c2, nm2);
        s[2 * e] = __float_as_uint(x.x);
        s[2 * e + 1] = __float_as_uint(x.y);
      }
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        float2 x = make_float2(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1]));
        if (kFmaExpEvery > 0 && e % (kFmaExpEvery > 0 ? kFmaExpEvery : 1) == 0) {
          x = exp2_fma(x);
        } else {
          x.x = ex2(x.x);
          x.y = ex2(x.y);
        }
        s[2 * e] = __float_as_uint(x.x);
        s[2 * e + 1] = __float_as_uint(x.y);
      }
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float2 x = make_float2(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1]));
        if (e & 1) sum1 = f2_add(sum1, x); else sum0 = f2_add(sum0, x);
        s[e] = f2_to_bf16x2(x);      // s[e] is dead by now: 2e, 2e+1 >= e
      }
      l += (sum0.x + sum0.y) + (sum1.x + sum1.y);
      tc_st32(p_addr, s);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_full(t));
    }
    if (ok) {
      ok = mbar_wait(o_full(t), 0, abort_flag, p.status, kErrBase + 0x60 + t);
      ok = __all_sync(0xffffffffu, ok);
      // as above: the partner may be on its way to the meeting point of the row sums
      if (!ok) asm volatile("bar.arrive %0, %1;" ::"r"(pair_bar), "n"(64) : "memory");
    }
    if (ok) {
      tc_fence_after();
      // the row sum of both halves (the slots of parity n & 1 were last used two tiles ago)
      *xslot(n & 1, half) = l;
      asm volatile("bar.sync %0, %1;" ::"r"(pair_bar), "n"(64) : "memory");
      l += *xslot(n & 1, half ^ 1);
      const float inv = 1.f / l;
      const bool live = row < p.q_len;
      uint8_t* dst = p.o + (live ? row : 0) * p.o_row_bytes + (int64_t)head * p.o_head_bytes + half * 128;
      uint32_t amax2 = 0u;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        uint32_t o[32];
        tc_ld32(o_addr + g * 32, o);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          o[e] = f2_to_bf16x2(make_float2(__uint_as_float(o[2 * e]) * inv, __uint_as_float(o[2 * e + 1]) * inv));
          if (live) amax2 = bf16x2_max_abs(amax2, o[e]);
        }
        if (live) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            reinterpret_cast<uint4*>(dst + g * 64)[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
        }
      }
      if (p.amax) {
        // non-negative floats order like their bit patterns: one atomic per warp
        const float a = fmaxf(bf16lo_to_f32(amax2), bf16hi_to_f32(amax2));
        const unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(a));
        if (lane == 0 && bits != 0u) atomicMax(p.amax, bits);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kIssuerWarp) {
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

// Tensor map over bf16 [tokens][heads][128] with the given element strides: boxes of 128 tokens x
// one head x 64 elements (128 bytes), 128-byte swizzle, tokens past the end read as zeros.
static bool make_map(CUtensorMap* map, const void* base, int64_t tokens, int heads, int64_t row_stride,
                     int64_t head_stride) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)head_stride * 2u, (cuuint64_t)row_stride * 2u};
  cuuint32_t box[3] = {64u, 1u, (cuuint32_t)kBKV};
  cuuint32_t elem[3] = {1u, 1u, 1u};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace attn
}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_attention_bf16(const void* q, int64_t q_row_stride, int64_t q_head_stride,
                                    const void* k, int64_t k_row_stride, int64_t k_head_stride,
                                    const void* v, int64_t v_row_stride, int64_t v_head_stride,
                                    int64_t q_len, int64_t kv_len, int heads, int head_dim,
                                    float softmax_scale, void* o, int64_t o_row_stride,
                                    int64_t o_head_stride, float* amax_dev, int* status_dev,
                                    void* stream) {
  if (q_len < 0 || kv_len < 1 || heads < 1 || heads > 65535 || head_dim != attn::kD ||
      q_len >= ((int64_t)1 << 31) || kv_len >= ((int64_t)1 << 31) || !(softmax_scale > 0.f))
    return NVFP4_ERR_BAD_ARG;
  if (q_len == 0) return NVFP4_OK;
  if (!q || !k || !v || !o) return NVFP4_ERR_BAD_ARG;
  const int64_t strides[8] = {q_row_stride, q_head_stride, k_row_stride, k_head_stride,
                              v_row_stride, v_head_stride, o_row_stride, o_head_stride};
  for (int64_t s : strides) {
    if (s < attn::kD || s >= ((int64_t)1 << 38)) return NVFP4_ERR_BAD_ARG;
    if (s % 8 != 0) return NVFP4_ERR_BAD_ALIGN;
  }
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return NVFP4_ERR_BAD_ALIGN;
  int rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;

  CUtensorMap map_q, map_k, map_v;
  if (!attn::make_map(&map_q, q, q_len, heads, q_row_stride, q_head_stride) ||
      !attn::make_map(&map_k, k, kv_len, heads, k_row_stride, k_head_stride) ||
      !attn::make_map(&map_v, v, kv_len, heads, v_row_stride, v_head_stride))
    return NVFP4_ERR_BAD_ARG;

  attn::Params p{};
  p.q_len = q_len;
  p.kv_len = kv_len;
  p.kv_tiles = (int)((kv_len + attn::kBKV - 1) / attn::kBKV);
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.o = static_cast<uint8_t*>(o);
  p.o_row_bytes = o_row_stride * 2;
  p.o_head_bytes = o_head_stride * 2;
  p.amax = reinterpret_cast<unsigned*>(amax_dev);
  p.status = status_dev;

  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return NVFP4_ERR_BAD_ARG;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(attn::attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             attn::kSmemBytes) != cudaSuccess)
      return NVFP4_ERR_LAUNCH_FAILED;
    attr_set[dev] = true;
  }
  const int64_t q_blocks = (q_len + attn::kQTiles * attn::kBQ - 1) / (attn::kQTiles * attn::kBQ);
  dim3 grid((unsigned)q_blocks, (unsigned)heads);
  attn::attention_kernel<<<grid, attn::kThreads, attn::kSmemBytes, reinterpret_cast<cudaStream_t>(stream)>>>(
      map_q, map_k, map_v, p);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}
