// The head -> sequence return exchange of sequence-parallel attention and the flag waits that
// order the exchanges (no reference counterpart: the reference has no distributed code; its
// attention call sites are fx/src/s4/models/wan22/wan_transformer.py:126-129 and
// wan_transformer_fast.py:47-58).
//
// After attention a rank holds the output of ITS heads for ALL tokens, [tokens, heads/P, D];
// the attention-out linear needs all heads of the rank's OWN tokens, [tokens/P, heads, D].
// attn_return_kernel does that move in one pass over the attention output: every 16-byte
// piece is loaded once, folded into the running max |o| of its destination, and stored into
// the destination rank's buffer -- this GPU's memory or a peer's over NVLink, plain stores.
// The last CTA then publishes the per-destination maxima and raises the flags
// (exchange_sync.cuh).  The destination's wait kernel combines the maxima of all sources into
// the tensor amax of its assembled buffer, so the quantizer in front of the attention-out
// linear needs no amax pass of its own and no separate exchange phase remains.
//
// Every wait is bounded by a caller-given time; when it runs out the kernel records which
// rank was missing in the status word and returns normally.
#include "exchange_sync.cuh"
#include "nvfp4_common.cuh"

namespace nvfp4 {
namespace {

using xsync::Peers;

constexpr int kReturnThreads = 256;
constexpr int kReturnUnroll = 4;          // 16-byte pieces in flight per thread
constexpr int kErrFlagTimeout = 0xB00;    // status code: + the rank whose flag never came

struct ReturnArgs {
  const uint8_t* o;            // [tokens_total][heads_local][head_dim] bf16, strided
  int64_t row_bytes;           // distance between tokens of o
  int64_t head_bytes;          // distance between heads of o
  int64_t tokens_per_rank;
  int heads_local;
  int head_dim;
  uint8_t* out[xsync::kMaxRanks];   // rank s's [tokens_per_rank][heads_local*world][head_dim] buffer
  Peers peers;
};

__global__ void __launch_bounds__(kReturnThreads)
attn_return_kernel(const ReturnArgs p) {
  // CTA b serves destination (b + rank) % world, so that at any moment every rank's stores are
  // spread over all destinations (and every destination hears from all sources) instead of
  // all sources hammering one GPU's links at a time.
  const int world = p.peers.world;
  const int dest = (int)((blockIdx.x + (unsigned)p.peers.rank) % (unsigned)world);
  const unsigned lane_cta = blockIdx.x / (unsigned)world;     // this CTA among the destination's
  const unsigned ctas = gridDim.x / (unsigned)world;
  const int chunks_per_head = p.head_dim >> 3;                // 16-byte pieces
  const int chunks_per_token = p.heads_local * chunks_per_head;
  const int64_t total = p.tokens_per_rank * chunks_per_token;
  const int64_t out_row_bytes = (int64_t)p.heads_local * world * p.head_dim * 2;
  const uint8_t* src0 = p.o + (int64_t)dest * p.tokens_per_rank * p.row_bytes;
  uint8_t* dst0 = p.out[dest] + (int64_t)p.peers.rank * p.heads_local * p.head_dim * 2;

  uint32_t amax2 = 0u;                                        // bf16x2 running max |o|
  const int64_t stride = (int64_t)ctas * kReturnThreads;
  for (int64_t i0 = (int64_t)lane_cta * kReturnThreads + threadIdx.x; i0 < total;
       i0 += stride * kReturnUnroll) {
    uint4 v[kReturnUnroll];
    int64_t dst_off[kReturnUnroll];
#pragma unroll
    for (int u = 0; u < kReturnUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      dst_off[u] = -1;
      if (i < total) {
        const int64_t tok = i / chunks_per_token;
        const int rem = (int)(i - tok * chunks_per_token);
        const int head = rem / chunks_per_head;
        const int c = rem - head * chunks_per_head;
        v[u] = __ldcs(reinterpret_cast<const uint4*>(src0 + tok * p.row_bytes + head * p.head_bytes) + c);
        dst_off[u] = tok * out_row_bytes + (int64_t)rem * 16;
      }
    }
#pragma unroll
    for (int u = 0; u < kReturnUnroll; ++u) {
      if (dst_off[u] < 0) continue;
      amax2 = bf16x2_max_abs(bf16x2_max_abs(amax2, v[u].x), v[u].y);
      amax2 = bf16x2_max_abs(bf16x2_max_abs(amax2, v[u].z), v[u].w);
      *reinterpret_cast<uint4*>(dst0 + dst_off[u]) = v[u];
    }
  }
  // one atomic per warp: non-negative floats order like their bit patterns
  const float a = fmaxf(bf16lo_to_f32(amax2), bf16hi_to_f32(amax2));
  const unsigned bits = __reduce_max_sync(0xffffffffu, __float_as_uint(a));
  if ((threadIdx.x & 31) == 0 && bits != 0u)
    atomicMax(reinterpret_cast<unsigned*>(p.peers.sync[p.peers.rank] + xsync::kAmaxWork + dest), bits);
  xsync::signal_when_grid_done(p.peers, 1, gridDim.x, true);
}

// One warp: lane r waits for rank r's flag of `kind` to reach this rank's next epoch.
__global__ void exchange_wait_kernel(int* sync, int kind, int world, long long limit_ns,
                                     float* amax_out, int* status) {
  const int lane = threadIdx.x;
  const int epoch = sync[xsync::kWaited + kind] + 1;
  bool ok = true;
  // Once a wait has run out (the status word is set and nobody has cleared it) later waits do
  // not spin again: a step with a missing rank costs one time limit, not one per exchange.
  const bool failed_before = status != nullptr && *reinterpret_cast<volatile int*>(status) != 0;
  if (lane < world && !failed_before) {
    const int* flag = sync + xsync::kFlag + kind * xsync::kMaxRanks + lane;
    if (xsync::ld_acquire_sys(flag) - epoch < 0) {
      unsigned long long t0, t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
      for (;;) {
        if (xsync::ld_acquire_sys(flag) - epoch >= 0) break;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if ((long long)(t - t0) > limit_ns) {
          ok = false;
          if (status) atomicCAS(status, 0, kErrFlagTimeout + lane);
          break;
        }
        __nanosleep(200);
      }
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (amax_out) {
    // the tensor amax of the assembled buffer = max over the sources' maxima
    const unsigned part = lane < world ? (unsigned)xsync::ld_acquire_sys(sync + xsync::kAmaxPart + lane) : 0u;
    const unsigned bits = __reduce_max_sync(0xffffffffu, part);
    if (lane == 0) *amax_out = __uint_as_float(bits);
  }
  // the epoch advances even after a timeout, so that later waits stay aligned with the peers
  if (lane == 0) sync[xsync::kWaited + kind] = epoch;
  (void)ok;
}

int fill_peers(Peers& peers, void* const* sync_blocks, int world, int rank) {
  if (world < 1 || world > xsync::kMaxRanks || rank < 0 || rank >= world || !sync_blocks)
    return NVFP4_ERR_BAD_ARG;
  peers.world = world;
  peers.rank = rank;
  for (int r = 0; r < xsync::kMaxRanks; ++r) peers.sync[r] = nullptr;
  for (int r = 0; r < world; ++r) {
    if (!sync_blocks[r]) return NVFP4_ERR_BAD_ARG;
    if (!aligned16(sync_blocks[r])) return NVFP4_ERR_BAD_ALIGN;
    peers.sync[r] = static_cast<int*>(sync_blocks[r]);
  }
  return NVFP4_OK;
}

}  // namespace

// used by qk_norm_rope.cu
int exchange_fill_peers(xsync::Peers& peers, void* const* sync_blocks, int world, int rank) {
  return fill_peers(peers, sync_blocks, world, rank);
}

}  // namespace nvfp4

using namespace nvfp4;

extern "C" {

int64_t nvfp4_exchange_sync_bytes(void) { return xsync::kSyncBytes; }

int nvfp4_exchange_wait(void* sync_block, int kind, int world, int64_t limit_ns, float* amax_out_dev,
                        int* status_dev, void* stream) {
  if (!sync_block || kind < 0 || kind >= xsync::kKinds || world < 1 || world > xsync::kMaxRanks ||
      limit_ns <= 0)
    return NVFP4_ERR_BAD_ARG;
  if (!aligned16(sync_block)) return NVFP4_ERR_BAD_ALIGN;
  int rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
  exchange_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<int*>(sync_block), kind, world, (long long)limit_ns, amax_out_dev, status_dev);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}

int nvfp4_attn_return_exchange_bf16(const void* o_bf16, int64_t o_row_stride, int64_t o_head_stride,
                                    int64_t tokens_total, int heads_local, int head_dim,
                                    void* const* rank_buffers, void* const* sync_blocks, int world,
                                    int rank, void* stream) {
  if (tokens_total < 0 || heads_local <= 0 || head_dim <= 0 || head_dim % 8 != 0 ||
      o_head_stride < head_dim || o_row_stride < head_dim || o_row_stride % 8 != 0 ||
      o_head_stride % 8 != 0 || !rank_buffers)
    return NVFP4_ERR_BAD_ARG;
  ReturnArgs a{};
  int rc = fill_peers(a.peers, sync_blocks, world, rank);
  if (rc != NVFP4_OK) return rc;
  if (tokens_total % world != 0) return NVFP4_ERR_BAD_ARG;
  if (tokens_total > 0 && !o_bf16) return NVFP4_ERR_BAD_ARG;
  if (!aligned16(o_bf16)) return NVFP4_ERR_BAD_ALIGN;
  for (int r = 0; r < world; ++r) {
    if (!rank_buffers[r]) return NVFP4_ERR_BAD_ARG;
    if (!aligned16(rank_buffers[r])) return NVFP4_ERR_BAD_ALIGN;
    a.out[r] = static_cast<uint8_t*>(rank_buffers[r]);
  }
  rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
  a.o = static_cast<const uint8_t*>(o_bf16);
  a.row_bytes = o_row_stride * 2;
  a.head_bytes = o_head_stride * 2;
  a.tokens_per_rank = tokens_total / world;
  a.heads_local = heads_local;
  a.head_dim = head_dim;
  // enough CTAs to fill the GPU several times over, a whole number per destination; an empty
  // input still launches one round so that the flags advance
  const int64_t pieces = a.tokens_per_rank * heads_local * (head_dim / 8);
  int64_t per_dest = (pieces + (int64_t)kReturnThreads * kReturnUnroll - 1) /
                     ((int64_t)kReturnThreads * kReturnUnroll);
  const int64_t cap = ((int64_t)sm_count() * 8 + world - 1) / world;
  if (per_dest > cap) per_dest = cap;
  if (per_dest < 1) per_dest = 1;
  attn_return_kernel<<<(unsigned)(per_dest * world), kReturnThreads, 0,
                       reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}

}  // extern "C"
