// Block-scaled FP4 (NVFP4) GEMM for sm_100a, hand-written on tcgen05:
//
//   D[M,N] bf16 = beta*C + gate[n] * act( alpha*ga*gb * sum_k (a*sfa)(b*sfb) + bias[n] )
//
// CTA pairs (clusters of two, one CTA per SM) walk 256x256 output tiles with
// tcgen05.mma.cta_group::2: each CTA holds 128 rows of A, half of the B tile's
// rows and 128 rows of the accumulator, so shared memory takes in 38 KiB and
// feeds 32 KiB per stage instead of 54 and 48 for a lone 128x256 CTA.  Roles by
// warp, in both CTAs unless noted:
//   warp 0     producer: five TMA loads per stage (this CTA's A rows, B half, A
//              scale atoms, both halves of the B scale atoms; 128-byte swizzle
//              for A/B, one destination CTA per copy) into a 5-stage ring whose
//              "full" barrier lives in the leader CTA
//   warp 1     leader CTA only: per stage twelve tcgen05.cp.cta_group::2 of the
//              scale atoms (each CTA copies from its own shared memory into its
//              own tensor memory), four tcgen05.mma kind::mxf4nvf4 (16-element
//              blocks, UE4M3 scales, fp32 accumulators in tensor memory) and one
//              tcgen05.commit to both CTAs
//   warps 2-5  epilogue: tcgen05.ld of the accumulator, fused scale / bias /
//              GELU-tanh / gate / residual, bf16 stores
//
// Producer and issuer run as whole converged warps with one elected lane
// enabled per instruction.  Measured on B200: from a one-lane divergent branch
// a tcgen05.cp costs the thread ~46 cycles and 12 copies + 4 MMAs take 801
// cycles; from converged code a copy costs ~8 and the same stage takes 511,
// the time of the four MMAs alone.
//
// Two tilings of N share the kernel body (template parameter kAlt):
//   uniform     256-wide tiles.  Tensor memory (512 columns): two 256-column
//               accumulators at columns 0 and 192 that overlap in [192,256), scale factors
//               at [448,496).  The epilogue reads the overlapping 64 columns into registers
//               first and then lets the issuer start the next tile in the other accumulator,
//               so the rest of the epilogue runs under the next tile's main loop; what stays
//               exposed per tile is that hand-off (about 1300 cycles).
//   alternating N is cut into 448-column pairs of a 256-wide and a 192-wide tile and every CTA
//               pair takes wide and narrow tiles in turn: the wide accumulator sits at columns
//               [0,256), the narrow one at [256,448), scale factors at [448,496) -- no shared
//               columns, so the issuer goes straight on to the next tile and an accumulator
//               is handed back only two tiles later.  Costs 7 % more operand bytes per flop;
//               pays when the main loop is short (K up to a few thousand).  In odd pairs the
//               narrow tile comes first so that every tile starts 0 or 64 rows into a 128-row
//               scale atom and two atoms always cover it.
//
// Every wait is bounded: when a wait gives up the kernel records where in
// *status, raises a CTA-wide abort flag, and every role leaves its loop so
// that tensor memory is released and the CTA exits.
#include <cuda.h>

#include "nvfp4_common.cuh"

namespace nvfp4 {
namespace gemm {

constexpr int BM = 128;                  // rows per CTA (= TMEM lanes); a CTA pair covers 2*BM
constexpr int BN = 256;                  // tile columns (= one MMA N)
constexpr int BK = 256;                  // K elements per stage (128 bytes: one swizzle row)
constexpr int kStages = 5;
constexpr int kABytes = BM * BK / 2;        // 16384: this CTA's 128 rows of A
constexpr int kBBytes = (BN / 2) * BK / 2;  // 16384: this CTA's half of the B tile's rows
constexpr int kSfaBytes = (BM / 128) * (BK / 64) * kSfAtomBytes;  // 2048
constexpr int kSfbBytes = (BN / 128) * (BK / 64) * kSfAtomBytes;  // 4096: all 256 columns
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
constexpr int kEpiSlabBytes = 32 * 128;    // 32 rows x 64 bf16 columns, one TMA store
constexpr int kEpiWarps = 8;
constexpr int kEpiBytes = kEpiWarps * kEpiSlabBytes;  // one slab per epilogue warp
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*align slack*/ + 256 /*barriers*/;
constexpr int kThreads = 320;          // producer, issuer, eight epilogue warps
constexpr int kTmemCols = 512;
constexpr int kAccCol1 = 192;            // uniform tiling: second accumulator's first column
constexpr int kAltPair = 448;            // alternating tiling: a 256-wide plus a 192-wide tile
constexpr int kAltNarrow = 192;
constexpr int kAltAccCol1 = 256;         // alternating tiling: the narrow accumulator's first column
constexpr int kBBytesNarrow = (kAltNarrow / 2) * BK / 2;   // 12288: a CTA's 96 rows of B
constexpr int kSfCol = 448;              // scale factors of one stage: 16 columns of SFA, 32 of SFB
constexpr long long kWaitCycles = 4000000000LL;  // ~2 s at 2 GHz

static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB per-CTA shared memory limit");

// ----------------------------------------------------------- PTX wrappers --

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// The asynchronous-unit instructions below take a predicate `on` instead of sitting in a
// one-lane branch: issued from converged warp code with one elected lane enabled they cost
// the warp ~8 cycles each, issued from a divergent single-lane branch ~45-75 (measured).
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
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// ---- CTA-pair (cluster of two) helpers ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of this CTA's shared-memory offset `addr` inside CTA `rank`
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// Arrive on a barrier given by its shared::cluster address (this CTA's or the peer's).
// Release semantics are required even though no shared or global data is published: with a
// relaxed arrive the issuer now and then (a few launches in a hundred at M = 27280) started the
// next tile's MMAs before a CTA's epilogue warps had read the shared accumulator columns --
// one tile's 128 x 64 piece wrong, found by comparing repeated launches bit for bit.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
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

// Tiled load into this CTA's shared memory whose byte count is reported to a barrier that
// may live in either CTA of the pair (`bar` is a shared::cluster address).  One destination
// CTA per copy: nothing is broadcast.
// `policy` is an L2 eviction policy from l2_policy_evict_last/first().
__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint32_t bar, uint32_t dst,
                                            int x, int y, uint64_t policy, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %6;\n\t}"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(on), "l"(policy)
      : "memory");
}
// Operands are re-read from L2 by many CTAs (keep them), the output is written once (let it
// go first): without these hints the 500 MB output stream evicts the operands and a quarter
// of the operand sectors miss in L2.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
// Tiled load into this CTA's own shared memory, bytes reported to one of its own barriers
// (the residual tile of the epilogue).  One destination, nothing broadcast.
__device__ __forceinline__ void tma_load_2d_local(const CUtensorMap* map, uint32_t bar, uint32_t dst,
                                                  int x, int y, uint64_t policy, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %6;\n\t}"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(on), "l"(policy)
      : "memory");
}
// Tiled store of a shared-memory slab to global memory (clipped at the tensor's edges).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y,
                                             uint64_t policy, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %4, 0;\n\t"
      "@q cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint"
      " [%0, {%2, %3}], [%1], %5;\n\t}"
      ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(on), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive, once this thread's earlier tcgen05 operations (in both CTAs of the pair) have
// completed, on the barrier at offset `bar` in the CTAs selected by `cta_mask`
// (bit 0 = leader, bit 1 = peer).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;\n\t}"
      ::"r"(bar), "h"(cta_mask), "r"(on)
      : "memory");
}
// One 512-byte scale atom (32 rows x 16 bytes) from shared to tensor memory, replicated
// to the four lane quarters, in BOTH CTAs of the pair: each copies from its own shared
// memory at the descriptor's offset into its own tensor memory.
__device__ __forceinline__ void tc_cp_sf_pair(uint32_t taddr, uint64_t sdesc, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
      "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;\n\t}"
      ::"r"(taddr), "l"(sdesc), "r"(on)
      : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                            uint32_t accumulate, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %7, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X"
      " [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
        "r"(sfb_tmem), "r"(on)
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
// Descriptor of one scale atom for tcgen05.cp: 32 rows of 16 bytes, no swizzle, 8-row
// groups 128 bytes apart.
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
// Instruction descriptor, kind::mxf4nvf4: A and B E2M1 (code 1) both K-major,
// N at bits 17-22 in units of 8, UE4M3 scales (bit 23 clear), M at bits 24-28
// in units of 16, scale-factor ids 0, K = 64 (bit 31 clear).
__device__ __forceinline__ uint32_t make_idesc(int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)((2 * BM) >> 4) << 24);  // M = 256 across the CTA pair
}

__device__ __forceinline__ float gelu_tanh(float x) {
  // 0.5 x (1 + tanh(u)) = x / (1 + exp(-2u)), u = sqrt(2/pi) (x + 0.044715 x^3): one ex2 and
  // one reciprocal, both accurate to about 1e-7 relative, so the bf16 result is the correctly
  // rounded one except in rare near-tie cases.  (The hardware tanh is one op cheaper but
  // its 5e-4 absolute error moves a quarter of the bf16 roundings, and the FP4 re-quantization
  // of the FFN hidden amplifies that to a percent-level difference downstream.)  exp overflow
  // gives 1/inf = 0, the right limit.
  const float z = x * (-2.302208198144325f + -0.1029432395800235f * x * x);   // -2 u log2(e)
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

// The same on a pair of lanes (the polynomial as f32x2 ops in the scalar form's order; the two
// special-function ops stay per lane).
__device__ __forceinline__ float2 gelu_tanh2(float2 x) {
  const float2 c1 = make_float2(-2.302208198144325f, -2.302208198144325f);
  const float2 c2 = make_float2(-0.1029432395800235f, -0.1029432395800235f);
  const float2 z = f2_mul(x, f2_fma(f2_mul(c2, x), x, c1));   // -2 u log2(e)
  float ex, ey, rx, ry;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(z.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ey) : "f"(z.y));
  const float2 d = f2_add(make_float2(ex, ey), make_float2(1.0f, 1.0f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rx) : "f"(d.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(ry) : "f"(d.y));
  return f2_mul(x, make_float2(rx, ry));
}

// Tile order.  Tiles are numbered so that the pairs running at one time (consecutive
// numbers) cover a block of kRasterM tile rows by several tile columns: each A row block is
// then swept over all columns while it is hot in L2 instead of once per column with the whole
// of A in between (A is 195 MB at K = 14336, more than L2).
constexpr int kRasterM = 4;
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int per_group = kRasterM * n_tiles;
  const int group = tile / per_group;
  const int rem = tile - group * per_group;
  const int first = group * kRasterM;
  const int rows = min(kRasterM, m_tiles - first);
  nt = rem / rows;
  mt = first + (rem - nt * rows);
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
  unsigned* d_amax;   // optional: max |D| (as stored, bf16) accumulated by atomicMax on the bits
  int* status;
  float alpha, beta;
  int M, N, K;
  int m_tiles, k_tiles, k_atoms;
  int n_a, n_b;       // uniform tiling: 256-wide tile columns, 0; alternating: wide, narrow columns
  int gb_group;       // 0: gb is one scalar; else gb[n / gb_group] (weights of several tensors
                      // stacked along N, each with its own tensor scale)
  int act;
};

// One output tile as every role sees it.
struct Tile {
  int mt;       // 256-row tile index
  int n0;       // first column
  int w;        // columns the MMA computes: 256 (uniform); 64..256 in steps of 64 (alternating)
  int buf;      // accumulator: uniform 0/1 by turns; alternating 0 = wide, 1 = narrow
};

// The sequence of tiles of one CTA pair; producer, issuer and epilogue each walk their own copy.
// Alternating tiling: wide and narrow tiles form two lists numbered like the uniform tiles
// (tile_coords over the list's columns); pair q takes items q, q + Q, ... of each list, wide
// on its even turns and narrow on its odd ones, and finishes whichever list is left over.
template <bool kAlt>
struct TileWalk {
  int m_tiles, N, stride, n_a, n_b, i_a, i_b, t;
  __device__ TileWalk(const Params& p, int pair, int num_pairs)
      : m_tiles(p.m_tiles), N(p.N), stride(num_pairs), n_a(p.n_a), n_b(p.n_b), i_a(pair),
        i_b(pair), t(0) {}
  __device__ __forceinline__ bool next(Tile& o) {
    if (!kAlt) {
      if (i_a >= m_tiles * n_a) return false;
      int nt;
      tile_coords(i_a, m_tiles, n_a, o.mt, nt);
      o.n0 = nt * BN;
      o.w = BN;
      o.buf = t & 1;
      i_a += stride;
      ++t;
      return true;
    }
    const bool a_left = i_a < m_tiles * n_a, b_left = i_b < m_tiles * n_b;
    if (!a_left && !b_left) return false;
    const bool wide = a_left && (!(t & 1) || !b_left);
    int j;   // column slot = index of the 448-column pair
    if (wide) {
      tile_coords(i_a, m_tiles, n_a, o.mt, j);
      o.n0 = kAltPair * j + ((j & 1) ? kAltNarrow : 0);
      i_a += stride;
    } else {
      tile_coords(i_b, m_tiles, n_b, o.mt, j);
      o.n0 = kAltPair * j + ((j & 1) ? 0 : BN);
      i_b += stride;
    }
    const int full = wide ? BN : kAltNarrow;
    const int left = (N - o.n0 + 63) & ~63;       // what is left of N, in whole 64-column groups
    o.w = left < full ? left : full;
    o.buf = wide ? 0 : 1;
    ++t;
    return true;
  }
};

template <bool kAlt>
__global__ void __launch_bounds__(kThreads, 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                  const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_b_narrow,
                  const __grid_constant__ CUtensorMap map_sfa,
                  const __grid_constant__ CUtensorMap map_sfb,
                  const __grid_constant__ CUtensorMap map_d,
                  const __grid_constant__ CUtensorMap map_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  // stage s: [A 16K][B half 16K][SFA 2K][SFB 4K]; A and B start on 1024-byte boundaries
  // then the epilogue slabs (32 KiB, 1024-byte aligned), then the barriers
  const uint32_t bar_base = smem_base + kStages * kStageBytes + kEpiBytes;
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem_gen + kStages * kStageBytes + kEpiBytes + 248);
  uint32_t* tmem_slot =
      reinterpret_cast<uint32_t*>(smem_gen + kStages * kStageBytes + kEpiBytes + 252);
  // Barriers sit at the same offsets in both CTAs.  "leader" = waited on in CTA 0 only and
  // fed by both CTAs; "local" = waited on in each CTA.
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                      // leader: the stage landed in both CTAs
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };         // local: the stage's MMAs are done
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };  // local
  // leader.  Uniform tiling: slot 0 = the shared columns of the previous tile have been read.
  // Alternating tiling: slot b = every epilogue warp has finished reading accumulator b.
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
  auto c_bar = [&](int w) { return bar_base + 8u * (2 * kStages + 4 + w); };     // local: epilogue warp w's residual tile landed
  // leader, uniform tiling: the column groups of accumulator b that do NOT gate the next tile
  // have been read
  auto acc_rest_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 4 + kEpiWarps + b); };
  static_assert(8 * (2 * kStages + 4 + kEpiWarps + 2) <= 248, "barriers overrun their area");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0 = leader of the pair
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);    // armed by the leader's producer with the bytes of BOTH CTAs
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full_bar(0), 1);
    mbar_init(acc_full_bar(1), 1);
    // uniform: one arrival per warp that drains the shared columns; alternating: one per
    // epilogue warp of either CTA
    mbar_init(acc_empty_bar(0), kAlt ? 2 * kEpiWarps : 2 * 4);
    mbar_init(acc_empty_bar(1), kAlt ? 2 * kEpiWarps : 2 * 4);
    for (int w = 0; w < kEpiWarps; ++w) mbar_init(c_bar(w), 1);
    mbar_init(acc_rest_bar(0), 2 * 4);   // one arrival per warp that reads the other two groups
    mbar_init(acc_rest_bar(1), 2 * 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // first tensor-memory column of accumulator b
  auto acc_col = [&](int b) -> uint32_t { return b ? (kAlt ? kAltAccCol1 : kAccCol1) : 0; };

  if (warp == 0) {
    // ------------------------------------------------------- producer ----
    // The whole warp walks the loop; one elected lane is enabled on each copy.
    const uint32_t on = elect_one();
    const uint64_t keep = l2_policy_evict_last();
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    TileWalk<kAlt> walk(p, pair, num_pairs);
    Tile tl;
    while (ok && walk.next(tl)) {
      // first scale atom of this CTA's A rows / of the two 128-row atoms that cover the tile's
      // columns (a tile starts 0 or 64 rows into its first atom)
      const int sfa_atom = (2 * tl.mt + (int)rank) * p.k_atoms;
      const int sfb_atom0 = (tl.n0 >> 7) * p.k_atoms;
      const int sfb_atom1 = sfb_atom0 + p.k_atoms;
      // this CTA's half of the tile's B rows; the narrow tiles use a 96-row box
      const bool narrow = kAlt && tl.buf == 1;
      const int b_row = tl.n0 + (int)rank * (tl.w >> 1);
      const CUtensorMap* mb = narrow ? &map_b_narrow : &map_b;
      const uint32_t stage_tx = 2u * (uint32_t)(kStageBytes - (narrow ? kBBytes - kBBytesNarrow : 0));
      for (int kt = 0; kt < p.k_tiles; ++kt) {
        ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, 0x100 + s);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t st = smem_base + s * kStageBytes;
        // Everything both CTAs load for this stage completes the leader's barrier, which the
        // leader alone arms (a remote arrive per stage stalls the issuing thread for
        // thousands of cycles).
        const uint32_t lead_full = mapa_u32(full_bar(s), 0);
        mbar_expect_tx(full_bar(s), stage_tx, rank == 0 ? on : 0u);
        tma_load_2d(&map_a, lead_full, st, kt * (BK / 2), (2 * tl.mt + (int)rank) * BM, keep, on);
        tma_load_2d(mb, lead_full, st + kABytes, kt * (BK / 2), b_row, keep, on);
        tma_load_2d(&map_sfa, lead_full, st + kABytes + kBBytes, 0, sfa_atom + kt * (BK / 64), keep,
                    on);
        tma_load_2d(&map_sfb, lead_full, st + kABytes + kBBytes + kSfaBytes, 0,
                    sfb_atom0 + kt * (BK / 64), keep, on);
        tma_load_2d(&map_sfb, lead_full, st + kABytes + kBBytes + kSfaBytes + kSfbBytes / 2, 0,
                    sfb_atom1 + kt * (BK / 64), keep, on);
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
  } else if (warp == 1) {
    // ---------------- tensor-core issuer (leader CTA; the peer's warp idles) ----
    // Per stage: twelve scale-atom copies and four MMAs for the pair, then one commit.
    // Copies and MMAs of one thread execute in issue order, so the single scale buffer
    // needs no barrier of its own.
    if (rank == 0) {
      const uint32_t on = elect_one();
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int uses0 = 0, uses1 = 0;                         // tiles each accumulator has held
      const uint32_t sfa_t = tmem_base + kSfCol;        // SFA of K-block j at +4j
      const uint32_t sfb_t = tmem_base + kSfCol + 16;   // SFB of K-block j at +8j (two atoms)
      TileWalk<kAlt> walk(p, pair, num_pairs);
      Tile tl;
      while (ok && walk.next(tl)) {
        const int t = walk.t - 1;                       // ordinal of this tile
        const uint32_t acc = tmem_base + acc_col(tl.buf);
        const uint32_t idesc = make_idesc(tl.w);
        // the tile's first column inside its first scale atom, in 32-row column units
        const uint32_t sfb_off = (uint32_t)(tl.n0 & 127) >> 5;
        for (int kt = 0; kt < p.k_tiles; ++kt) {
          ok = mbar_wait(full_bar(s), ph, abort_flag, p.status, 0x200 + s);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = smem_base + s * kStageBytes;
          const uint32_t sfa_s = st + kABytes + kBBytes;
          const uint32_t sfb_s = sfa_s + kSfaBytes;
#pragma unroll
          for (int j = 0; j < BK / 64; ++j) {
            tc_cp_sf_pair(sfa_t + 4 * j, desc_sf(sfa_s + j * kSfAtomBytes), on);
            tc_cp_sf_pair(sfb_t + 8 * j, desc_sf(sfb_s + j * kSfAtomBytes), on);
            tc_cp_sf_pair(sfb_t + 8 * j + 4, desc_sf(sfb_s + kSfbBytes / 2 + j * kSfAtomBytes), on);
          }
          if (kt == 0) {
            // Only the MMAs need the accumulator; the scale copies above went ahead of these
            // waits (they follow the previous tile's MMAs in issue order, which is all the
            // single scale buffer needs).
            if (kAlt) {
              // the epilogue of this accumulator's previous tile (two tiles back when wide and
              // narrow alternate) has read all of it
              const int used = tl.buf ? uses1 : uses0;
              if (used > 0) {
                ok = mbar_wait(acc_empty_bar(tl.buf), (uint32_t)(used - 1) & 1u, abort_flag,
                               p.status, 0x300 + tl.buf);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
              }
            } else if (t > 0) {
              // the previous tile's shared accumulator columns have been drained
              ok = mbar_wait(acc_empty_bar(0), (uint32_t)(t - 1) & 1u, abort_flag, p.status, 0x300);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
              if (t >= 2) {
                // This accumulator was last used two tiles ago.  The warps that own its shared
                // group have been through it (they arrived above for the tile in between); the
                // warps that own its other two groups are tracked here.  They are normally a
                // whole main loop ahead, so this wait costs nothing; without it a short K and a
                // slow residual load could let these MMAs overwrite columns not yet read.
                ok = mbar_wait(acc_rest_bar(t & 1), (uint32_t)((t >> 1) - 1) & 1u, abort_flag,
                               p.status, 0x310);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
              }
            }
            tc_fence_after();
          }
          const uint64_t da = desc_sw128(st);
          const uint64_t db = desc_sw128(st + kABytes);
#pragma unroll
          for (int j = 0; j < BK / 64; ++j) {
            // 64 elements = 32 bytes along K inside the swizzled row: +2 in 16-byte units
            tc_mma_nvf4(acc, da + 2 * j, db + 2 * j, idesc, sfa_t + 4 * j, sfb_t + 8 * j + sfb_off,
                        (kt | j) != 0, on);
          }
          tc_commit_pair(empty_bar(s), 3, on);   // both CTAs' producers may refill the stage
          if (++s == kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit_pair(acc_full_bar(tl.buf), 3, on);
        if (tl.buf) ++uses1; else ++uses0;
      }
    }
  } else {
    // ------------------------------------------------------- epilogue ----
    // Eight warps: warp w reads tensor-memory lanes 32*(w%4).. (rows of this CTA), warps 2-5
    // take the first two 64-column groups in processing order, warps 6-9 the other two (a
    // narrow tile has three groups or fewer: the warps without one only pass the barriers).
    // A group goes through the warp's 32 x 128-byte shared-memory slab (128-byte swizzle, so
    // that the lane-per-row writes spread over the banks) and leaves with one TMA store, which
    // also clips at M and N.
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    const float scale_a = p.alpha * (p.ga ? __ldg(p.ga) : 1.0f);
    const float scale_ab = scale_a * ((p.gb && p.gb_group == 0) ? __ldg(p.gb) : 1.0f);
    const uint32_t lead_acc_empty0 = mapa_u32(acc_empty_bar(0), 0);
    const uint32_t lead_acc_empty1 = mapa_u32(acc_empty_bar(1), 0);
    const uint32_t on = elect_one();
    const uint64_t stream_out = l2_policy_evict_first();
    uint32_t amax2 = 0u;                 // running max |D| of this thread, as a bf16 pair
    uint8_t* slab = smem_gen + kStages * kStageBytes + (warp - 2) * kEpiSlabBytes;
    const int g_first = warp >= 6 ? 2 : 0;   // this warp's groups: g_first, g_first + 1
    bool ok = true;
    uint32_t c_phase = 0;                // parity of this warp's residual-tile barrier
    int uses0 = 0, uses1 = 0;
    TileWalk<kAlt> walk(p, pair, num_pairs);
    Tile tl;
    while (ok && walk.next(tl)) {
      const int buf = tl.buf;
      const uint32_t lead_acc_empty = buf ? lead_acc_empty1 : lead_acc_empty0;
      ok = mbar_wait(acc_full_bar(buf), (uint32_t)(buf ? uses1 : uses0) & 1u, abort_flag, p.status,
                     0x400 + buf);
      if (buf) ++uses1; else ++uses0;
      // the whole warp must agree before the .sync.aligned loads below
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row0 = (2 * tl.mt + (int)rank) * BM + q * 32;
      const int row = row0 + lane;
      const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16) + acc_col(buf);
      constexpr int kGroups = BN / 64;   // uniform tiling: the first group processed is the one
                                         // both accumulators share
      static_assert(256 - kAccCol1 == 64, "the shared columns must be exactly one group");
      const int n_groups = tl.w >> 6;
      // alternating tiling: the last group this warp reads (-1: none)
      const int last_gi = g_first >= n_groups ? -1 : (g_first + 1 < n_groups ? g_first + 1 : n_groups - 1);
      if (kAlt && last_gi < 0) {
        // nothing of this tile is ours; the accumulator's barrier still counts every warp
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_acc_empty);
        continue;
      }
      uint32_t x[64];
#pragma unroll 1
      for (int gj = 0; gj < 2; ++gj) {
        const int gi = g_first + gj;
        if (kAlt && gi > last_gi) break;
        // tensor-memory column group: the uniform tiling walks them so that the shared group
        // comes first
        const int cg = kAlt ? gi : (buf ? gi : (gi + kGroups - 1) % kGroups);
        const int col0 = tl.n0 + cg * 64;
        // tensor-memory loads first (they are asynchronous until the wait below): for the
        // shared group they sit on the path to the next tile's first MMA
        tc_ld_32x32(acc + cg * 64, *reinterpret_cast<uint32_t(*)[32]>(&x[0]));
        tc_ld_32x32(acc + cg * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&x[32]));
        // The residual tile (32 rows x 64 columns of C) comes into the slab by one TMA load, in
        // the layout the result will leave in, while tensor memory is being read: as per-lane
        // row-strided 16-byte loads it put sixteen exposed global-memory latencies per tile on
        // this warp and made a K = 3072 GEMM with a residual epilogue-bound (half speed).
        if (p.c) {
          // the previous store must have finished reading the slab
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
          mbar_expect_tx(c_bar(warp - 2), kEpiSlabBytes, on);
          tma_load_2d_local(&map_c, c_bar(warp - 2), smem_u32(slab), col0, row0, stream_out, on);
        }
        tc_wait_ld();
        if (kAlt) {
          if (gi == last_gi) {
            // this warp is done with the accumulator
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_acc_empty);
          }
        } else if (gi == 0) {
          // the shared columns are in registers: the issuer may start the next tile
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(lead_acc_empty0);
        } else if (gi == kGroups - 1) {
          // the last of the other groups is in registers: this accumulator may be reused
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(mapa_u32(acc_rest_bar(buf), 0));
        }
        // per-column operands of the whole group first, so that their loads overlap
        uint4 bb[8];
        if (p.bias) {
#pragma unroll
          for (int g = 0; g < 8; ++g)
            bb[g] = col0 + g * 8 < p.N
                        ? __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + g * 8))
                        : make_uint4(0, 0, 0, 0);
        }
        // stacked weights: the tensor scale of the weight this group's columns belong to
        const float scale = (p.gb_group > 0 && col0 < p.N)
                                ? scale_a * __ldg(p.gb + col0 / p.gb_group) : scale_ab;
        if (!p.c) {
          // the previous store must have finished reading the slab
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
        } else {
          ok = mbar_wait(c_bar(warp - 2), c_phase, abort_flag, p.status, 0x800 + (warp - 2));
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          c_phase ^= 1u;
        }
        // Two fp32 lanes per instruction from here to the bf16 pack: at K = 3072 the eight
        // epilogue warps have about as many issue slots per tile as the main loop has cycles.
        const float2 scale2 = make_float2(scale, scale);
        const float2 beta2 = make_float2(p.beta, p.beta);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          float2 v[4];
          const bool in_n = col0 + g * 8 < p.N;
          if (p.bias) {
            const uint32_t bw[4] = {bb[g].x, bb[g].y, bb[g].z, bb[g].w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
              v[e] = f2_fma(make_float2(__uint_as_float(x[g * 8 + 2 * e]),
                                        __uint_as_float(x[g * 8 + 2 * e + 1])),
                            scale2, bf16x2_to_f2(bw[e]));
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              v[e] = f2_mul(make_float2(__uint_as_float(x[g * 8 + 2 * e]),
                                        __uint_as_float(x[g * 8 + 2 * e + 1])), scale2);
          }
          if (p.act == NVFP4_ACT_GELU_TANH) {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = gelu_tanh2(v[e]);
          }
          if (p.gate && in_n) {
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(p.gate + col0 + g * 8));
            const float4 g1 = __ldg(reinterpret_cast<const float4*>(p.gate + col0 + g * 8 + 4));
            v[0] = f2_mul(v[0], make_float2(g0.x, g0.y));
            v[1] = f2_mul(v[1], make_float2(g0.z, g0.w));
            v[2] = f2_mul(v[2], make_float2(g1.x, g1.y));
            v[3] = f2_mul(v[3], make_float2(g1.z, g1.w));
          }
          if (p.c) {   // rows past M and columns past N were zero-filled by the load
            const uint4 cc = *reinterpret_cast<const uint4*>(slab + lane * 128 + ((g ^ (lane & 7)) << 4));
            const uint32_t cw[4] = {cc.x, cc.y, cc.z, cc.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = f2_fma(beta2, bf16x2_to_f2(cw[e]), v[e]);
          }
          uint32_t o[4];
          const bool counted = p.d_amax && row < p.M && in_n;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            o[e] = f2_to_bf16x2(v[e]);
            if (counted) amax2 = bf16x2_max_abs(amax2, o[e]);
          }
          // row `lane` of the slab, 16-byte chunk g, at its 128-byte-swizzle position
          *reinterpret_cast<uint4*>(slab + lane * 128 + ((g ^ (lane & 7)) << 4)) =
              make_uint4(o[0], o[1], o[2], o[3]);
        }
        // make the slab visible to the TMA unit, then one lane sends it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        tma_store_2d(&map_d, smem_u32(slab), col0, row0, stream_out,
                     (row0 < p.M && col0 < p.N) ? on : 0u);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
    // the CTA's shared memory must outlive the stores that read it
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    if (p.d_amax) {
      // non-negative floats order like their bit patterns: one atomic per warp per launch
      const float a = fmaxf(bf16lo_to_f32(amax2), bf16hi_to_f32(amax2));
      const unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(a));
      if (lane == 0 && bits != 0u) atomicMax(p.d_amax, bits);
    }
  }

  // Both CTAs of the pair must be done with each other's barriers and with the shared
  // tensor-memory allocation before either releases it.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
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

// Tensor map over a swizzled scale buffer seen as [atoms][128 x u32]: box of four atoms
// (one pipeline stage of one 128-row tile, 2048 contiguous bytes), no swizzle.
static bool make_sf_map(CUtensorMap* map, const void* base, int64_t atoms) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {128u, (cuuint64_t)atoms};
  cuuint64_t strides[1] = {(cuuint64_t)kSfAtomBytes};
  cuuint32_t box[2] = {128u, (cuuint32_t)(BK / 64)};
  cuuint32_t elem[2] = {1u, 1u};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box,
            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor map over the bf16 output [M][N]: box of 64 columns x 32 rows (one epilogue slab),
// 128-byte swizzle.
static bool make_d_map(CUtensorMap* map, void* base, int64_t M, int64_t N) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  cuuint64_t strides[1] = {(cuuint64_t)N * 2u};
  cuuint32_t box[2] = {64u, 32u};
  cuuint32_t elem[2] = {1u, 1u};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace gemm
}  // namespace nvfp4

using namespace nvfp4;

namespace {

// 0 = choose per shape, 1 = uniform 256-wide tiles, 2 = alternating 256/192-wide tiles
int g_tiling_mode = 0;
// The alternating tiling removes the per-tile accumulator hand-off and adds 8 % to the bytes an
// SM takes in per flop (the narrow tiles reuse A less).  Measured on B200 the kernel is bound
// by that intake, not by the hand-off: alternating is 3 % slower at K = 3072 and 8 % slower at
// K = 14336 than uniform on the Wan 2.2 shapes, so the automatic choice is uniform for every
// shape and the alternating tiling stays a selectable variant (bit-identical results).
constexpr int kAltMaxK = 0;

template <bool kAlt>
int launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_b_narrow,
                const CUtensorMap& map_sfa, const CUtensorMap& map_sfb, const CUtensorMap& map_d,
                const CUtensorMap& map_c, const gemm::Params& p, int64_t tiles, cudaStream_t stream) {
  static bool attr_set[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm::nvfp4_gemm_kernel<kAlt>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             gemm::kSmemBytes) != cudaSuccess)
      return NVFP4_ERR_LAUNCH_FAILED;
    attr_set[dev] = true;
  }
  // one CTA pair (cluster of two) per pair of SMs, each pair walking its tiles
  const int max_pairs = sm_count() / 2;
  const unsigned pairs = (unsigned)(tiles < max_pairs ? tiles : max_pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(gemm::kThreads, 1, 1);
  cfg.dynamicSmemBytes = gemm::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm::nvfp4_gemm_kernel<kAlt>, map_a, map_b, map_b_narrow, map_sfa,
                         map_sfb, map_d, map_c, p) != cudaSuccess) {
    cudaGetLastError();
    return NVFP4_ERR_LAUNCH_FAILED;
  }
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}

int gemm_impl(const uint8_t* a_packed, const uint8_t* b_packed, const uint8_t* a_scales_swizzled,
              const uint8_t* b_scales_swizzled, const float* a_global_scale_dev,
              const float* b_global_scale_dev, int64_t b_group_rows, int64_t M, int64_t N,
              int64_t K, float alpha, float beta, const void* c_bf16, const void* bias_bf16,
              const float* gate_f32, int act, void* d_bf16, float* d_amax_dev, int* status_dev,
              void* stream) {
  if (M < 0 || N < 0 || K < 0 || N % 8 != 0 || K % 32 != 0) return NVFP4_ERR_BAD_ARG;
  if (act != NVFP4_ACT_NONE && act != NVFP4_ACT_GELU_TANH) return NVFP4_ERR_BAD_ARG;
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return NVFP4_ERR_BAD_ARG;
  // stacked weights: whole 64-column groups per weight, and a scale array to index
  if (b_group_rows < 0 || b_group_rows % 64 != 0 || (b_group_rows > 0 && !b_global_scale_dev))
    return NVFP4_ERR_BAD_ARG;
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

  CUtensorMap map_a, map_b, map_b_narrow, map_sfa, map_sfb, map_d, map_c;
  if (!gemm::make_map(&map_a, a_packed, M, K / 2, gemm::BM) ||
      !gemm::make_map(&map_b, b_packed, N, K / 2, gemm::BN / 2) ||
      !gemm::make_map(&map_b_narrow, b_packed, N, K / 2, gemm::kAltNarrow / 2) ||
      !gemm::make_sf_map(&map_sfa, a_scales_swizzled, sf_row_tiles(M) * sf_k_atoms(K)) ||
      !gemm::make_sf_map(&map_sfb, b_scales_swizzled, sf_row_tiles(N) * sf_k_atoms(K)) ||
      !gemm::make_d_map(&map_d, d_bf16, M, N))
    return NVFP4_ERR_LAUNCH_FAILED;
  // beta == 0 means C is not read at all (BLAS convention): a NaN in it cannot reach D
  if (beta == 0.0f) c_bf16 = nullptr;
  if (c_bf16) {
    // same geometry as the output: the epilogue loads residual tiles into its output slabs
    if (!gemm::make_d_map(&map_c, const_cast<void*>(c_bf16), M, N)) return NVFP4_ERR_LAUNCH_FAILED;
  } else {
    map_c = map_d;   // never dereferenced
  }

  gemm::Params p;
  p.sfa = a_scales_swizzled;
  p.sfb = b_scales_swizzled;
  p.ga = a_global_scale_dev;
  p.gb = b_global_scale_dev;
  p.c = reinterpret_cast<const __nv_bfloat16*>(c_bf16);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias_bf16);
  p.gate = gate_f32;
  p.d = reinterpret_cast<__nv_bfloat16*>(d_bf16);
  p.d_amax = reinterpret_cast<unsigned*>(d_amax_dev);
  p.status = status_dev;
  p.alpha = alpha;
  p.beta = beta;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.m_tiles = (int)((M + 2 * gemm::BM - 1) / (2 * gemm::BM));  // 256-row pair tiles
  p.k_tiles = (int)((K + gemm::BK - 1) / gemm::BK);
  p.k_atoms = (int)sf_k_atoms(K);
  p.gb_group = (int)b_group_rows;
  p.act = act;

  const bool alt = g_tiling_mode == 2 || (g_tiling_mode == 0 && K <= kAltMaxK && N > gemm::BN);
  if (alt) {
    // 448-column pairs of a wide and a narrow tile; in odd pairs the narrow one comes first
    const int full = (int)(N / gemm::kAltPair), rem = (int)(N % gemm::kAltPair);
    if ((full & 1) == 0) {
      p.n_a = full + (rem > 0);
      p.n_b = full + (rem > gemm::BN);
    } else {
      p.n_b = full + (rem > 0);
      p.n_a = full + (rem > gemm::kAltNarrow);
    }
  } else {
    p.n_a = (int)((N + gemm::BN - 1) / gemm::BN);
    p.n_b = 0;
  }

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (d_amax_dev && cudaMemsetAsync(d_amax_dev, 0, sizeof(float), st) != cudaSuccess)
    return NVFP4_ERR_LAUNCH_FAILED;
  const int64_t tiles = (int64_t)p.m_tiles * (p.n_a > p.n_b ? p.n_a : p.n_b);
  return alt ? launch_gemm<true>(map_a, map_b, map_b_narrow, map_sfa, map_sfb, map_d, map_c, p,
                                 tiles, st)
             : launch_gemm<false>(map_a, map_b, map_b_narrow, map_sfa, map_sfb, map_d, map_c, p,
                                  tiles, st);
}

}  // namespace

extern "C" int nvfp4_gemm_set_tiling(int mode) {
  if (mode < 0 || mode > 2) return NVFP4_ERR_BAD_ARG;
  g_tiling_mode = mode;
  return NVFP4_OK;
}

extern "C" int nvfp4_gemm(const uint8_t* a_packed, const uint8_t* b_packed,
                          const uint8_t* a_scales_swizzled, const uint8_t* b_scales_swizzled,
                          const float* a_global_scale_dev, const float* b_global_scale_dev,
                          int64_t M, int64_t N, int64_t K, float alpha, float beta,
                          const void* c_bf16, const void* bias_bf16, const float* gate_f32, int act,
                          void* d_bf16, float* d_amax_dev, int* status_dev, void* stream) {
  return gemm_impl(a_packed, b_packed, a_scales_swizzled, b_scales_swizzled, a_global_scale_dev,
                   b_global_scale_dev, 0, M, N, K, alpha, beta, c_bf16, bias_bf16, gate_f32, act,
                   d_bf16, d_amax_dev, status_dev, stream);
}

extern "C" int nvfp4_gemm_stacked(const uint8_t* a_packed, const uint8_t* b_packed,
                                  const uint8_t* a_scales_swizzled,
                                  const uint8_t* b_scales_swizzled,
                                  const float* a_global_scale_dev,
                                  const float* b_global_scales_dev, int64_t b_rows_per_weight,
                                  int64_t M, int64_t N, int64_t K, const void* bias_bf16,
                                  void* d_bf16, int* status_dev, void* stream) {
  if (b_rows_per_weight <= 0 || b_rows_per_weight % 256 != 0 || N % b_rows_per_weight != 0)
    return NVFP4_ERR_BAD_ARG;
  return gemm_impl(a_packed, b_packed, a_scales_swizzled, b_scales_swizzled, a_global_scale_dev,
                   b_global_scales_dev, b_rows_per_weight, M, N, K, 1.0f, 0.0f, nullptr, bias_bf16,
                   nullptr, NVFP4_ACT_NONE, d_bf16, nullptr, status_dev, stream);
}
