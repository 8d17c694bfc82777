// Flag signalling between the ranks of a sequence-parallel step, in memory every rank maps.
//
// Each rank owns one "sync block" (kSyncBytes of symmetric memory, zeroed once before use).
// A producer kernel on rank r, after ALL its CTAs have stored their data into the peers'
// buffers, writes its epoch into word flag[kind][r] of every peer's block; the consumer rank
// waits (nvfp4_exchange_wait) until the flags of all ranks have reached its own epoch.  The
// epochs live in device memory and advance by one per use, so a step recorded once can be
// replayed.  Plain loads and stores with system-scope fences only: no multicast mapping.
#pragma once

#include <cstdint>

namespace nvfp4 {
namespace xsync {

constexpr int kMaxRanks = 8;
constexpr int kKinds = 2;             // 0: q|k|v pieces before attention, 1: attention output after it
// word offsets inside a sync block
constexpr int kFlag = 0;                              // [kKinds][kMaxRanks] written by the peers
constexpr int kAmaxPart = kFlag + kKinds * kMaxRanks; // [kMaxRanks] fp32 bits, written by the peers
constexpr int kSent = kAmaxPart + kMaxRanks;          // [kKinds] epochs this rank has signalled
constexpr int kWaited = kSent + kKinds;               // [kKinds] epochs this rank has waited for
constexpr int kCtasDone = kWaited + kKinds;           // [kKinds] CTAs of the running producer that are done
constexpr int kAmaxWork = kCtasDone + kKinds;         // [kMaxRanks] running max per destination (producer-local)
constexpr int kWords = kAmaxWork + kMaxRanks;
constexpr int kSyncBytes = 256;
static_assert(kWords * 4 <= kSyncBytes, "sync block overruns its size");

struct Peers {
  int* sync[kMaxRanks];     // every rank's sync block as mapped here (own block at [rank])
  int world;
  int rank;
};

#ifdef __CUDACC__

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Called by every thread of every CTA at the end of a producer kernel (all of the CTA's
// stores issued).  The CTA that finishes last publishes, for every destination rank, this
// rank's partial amax (when `with_amax`) and then the new epoch.  Ordering: each CTA's stores
// -> its system fence -> its count; the last CTA sees all counts -> its system fence -> the
// flags.  `total_ctas` = CTAs of the whole grid.
__device__ __forceinline__ void signal_when_grid_done(const Peers& peers, int kind, unsigned total_ctas,
                                                      bool with_amax) {
  __syncthreads();
  if (threadIdx.x != 0) return;
  int* mine = peers.sync[peers.rank];
  __threadfence_system();
  const unsigned done = atomicAdd(reinterpret_cast<unsigned*>(mine + kCtasDone + kind), 1u) + 1u;
  if (done != total_ctas) return;
  __threadfence_system();
  mine[kCtasDone + kind] = 0;                        // the next launch counts from zero again
  const int epoch = mine[kSent + kind] + 1;
  mine[kSent + kind] = epoch;
  if (with_amax) {
    for (int r = 0; r < peers.world; ++r) {
      // atomicExch: reads the other CTAs' atomicMax results where they live and clears the slot
      const unsigned bits = atomicExch(reinterpret_cast<unsigned*>(mine + kAmaxWork + r), 0u);
      peers.sync[r][kAmaxPart + peers.rank] = (int)bits;
    }
    __threadfence_system();
  }
  for (int r = 0; r < peers.world; ++r) st_release_sys(peers.sync[r] + kFlag + kind * kMaxRanks + peers.rank, epoch);
}

#endif  // __CUDACC__

}  // namespace xsync
}  // namespace nvfp4
