// q/k RMSNorm across heads + rotary embedding, one pass over the QKV GEMM's output.
//
//   n = bf16( (x * rsqrt(mean(x^2) + eps)) * gain )            per token, over all heads
//   o[2i]   = bf16( n[2i] * c_i - n[2i+1] * s_i )              per head, pair i of head_dim/2
//   o[2i+1] = bf16( n[2i] * s_i + n[2i+1] * c_i )
//
// which is what the DiT block does between its QKV linear and attention
// (fx/src/s4/models/wan22/wan_transformer.py:91-92,114-115 for the norms, :61-75 for the
// rotation), there as about twenty elementwise torch kernels with fp32 round trips.  Every
// product and sum is rounded separately in fp32, as the unfused ops round them.  The value
// tensor can be carried along untouched so that q, k and v land in one packed
// [tokens, heads, 3 * head_dim] buffer ready for a head/sequence exchange.
//
// Layout of the work follows the fused norm + quantize kernel: a thread owns the same columns
// of every row (kC 8-element chunks a CTA width apart; its gains stay in registers), a CTA
// walks over groups of kR tokens that bulk copies stage in a ring of shared-memory slots, one
// CTA-wide reduction per group.
// blockIdx.y selects the tensor: 0 = q, 1 = k, 2 = v (copy only).
#include "exchange_sync.cuh"
#include "nvfp4_common.cuh"

namespace nvfp4 {

int exchange_fill_peers(xsync::Peers& peers, void* const* sync_blocks, int world, int rank);  // exchange.cu

namespace {

constexpr int kMaxThreads = 512;
constexpr int kMaxWarps = kMaxThreads / 32;
constexpr int kStages = 3;
constexpr int kR = 2;                              // tokens per group
#ifndef NVFP4_ROPE_CHUNKS
#define NVFP4_ROPE_CHUNKS 4
#endif
constexpr int kC = NVFP4_ROPE_CHUNKS;              // 8-element chunks per thread and row
constexpr long long kWaitCycles = 4000000000LL;    // about two seconds; then give up
constexpr int kErrCopyTimeout = 0xA00;             // status code: a token group never arrived

struct RopeArgs {
  const uint8_t* in[3];        // q, k, v: first element of row 0 (v may be null)
  int64_t in_row_bytes;        // distance between rows of an input
  int64_t rows;
  int dim;                     // heads * head_dim
  int head_dim;
  const float* gain[2];        // nullable: unit gain
  float eps;
  const float2* cos_sin;       // [rows][head_dim / 2] (cos of pair i, sin of pair i)
  uint8_t* out[3];
  int64_t out_row_bytes;
  int64_t out_head_bytes;
  int* status;
  // exchange form: heads are dealt out to `world` ranks, each of which receives its heads of
  // ALL tokens in a packed [tokens_total, heads_per_rank, 3 * head_dim] buffer
  uint8_t* peer[8];            // that buffer on every rank (this rank's own included)
  int heads_per_rank;          // 0: plain form
  int64_t row_offset;          // this rank's first token in the global order
  int signal;                  // exchange form: raise the peers' flags once the whole grid is done
  xsync::Peers peers;
};

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
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Bounded wait; on expiry the CTA carries on without the data (all barriers are still
// reached by all threads) and the status word says that its output is meaningless.
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

__global__ void __launch_bounds__(kMaxThreads)
qk_norm_rope_kernel(const RopeArgs p) {
  extern __shared__ __align__(128) uint8_t ring[];          // kStages slots of kR rows
  __shared__ __align__(16) float red[2][kR][kMaxWarps];
  __shared__ __align__(8) uint64_t full[kStages];
  __shared__ int abort_flag;
  const int which = blockIdx.y;                             // 0 q, 1 k, 2 v
  const int T = blockDim.x;
  const int warps = T >> 5;
  const uint32_t row_bytes = (uint32_t)p.dim * 2u;
  const uint32_t slot_bytes = row_bytes * kR;
  const int64_t groups = (p.rows + kR - 1) / kR;
  const uint8_t* in = which == 0 ? p.in[0] : (which == 1 ? p.in[1] : p.in[2]);
  uint8_t* out = which == 0 ? p.out[0] : (which == 1 ? p.out[1] : p.out[2]);   // plain form
  const float* gain_ptr = which == 0 ? p.gain[0] : (which == 1 ? p.gain[1] : nullptr);

  auto issue = [&](int64_t g, int slot) {
    const int64_t base = g * kR;
    const int n = (int)(p.rows - base < kR ? p.rows - base : kR);
    const uint32_t bar = smem_u32(&full[slot]);
    mbar_expect_tx(bar, (uint32_t)n * row_bytes);
    for (int r = 0; r < n; ++r)
      bulk_load(smem_u32(ring + (size_t)slot * slot_bytes + (size_t)r * row_bytes),
                in + (base + r) * p.in_row_bytes, row_bytes, bar);
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

  // This thread's kC 8-element chunks of every row: chunks t, t + T, ..., so that a warp's
  // shared-memory reads and global stores are each one contiguous 512 bytes.  A rotated pair
  // never straddles a chunk.  Per chunk: head, offset in the head, destination, gains.
  const int chunks = p.dim >> 3;
  bool live[kC];
  int d0[kC];
  uint8_t* dst_base[kC];
  int64_t out_off[kC];
  float2 gain[kC][4];
#pragma unroll
  for (int c = 0; c < kC; ++c) {
    const int ch = threadIdx.x + c * T;
    live[c] = ch < chunks;
    const int col = live[c] ? ch * 8 : 0;
    const int head = col / p.head_dim;
    d0[c] = col - head * p.head_dim;
    dst_base[c] = out;
    out_off[c] = (int64_t)head * p.out_head_bytes + (int64_t)d0[c] * 2;
    if (p.heads_per_rank > 0) {
      // plain stores into the owner rank's buffer (its own memory or a peer's over NVLink)
      const int dst = head / p.heads_per_rank;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r == dst) dst_base[c] = p.peer[r];
      out_off[c] = p.row_offset * p.out_row_bytes +
                   (int64_t)(head - dst * p.heads_per_rank) * p.out_head_bytes +
                   (int64_t)(which * p.head_dim + d0[c]) * 2;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) gain[c][e] = make_float2(1.0f, 1.0f);
    if (gain_ptr) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(gain_ptr + col) + q);
        gain[c][2 * q] = make_float2(a.x, a.y);
        gain[c][2 * q + 1] = make_float2(a.z, a.w);
      }
    }
  }
  const float dim_f = (float)p.dim;
  const int half_hd = p.head_dim >> 1;
  const bool rotate = which < 2 && p.cos_sin != nullptr;

  int slot = 0;
  uint32_t phase = 0;
  int parity = 0;
  for (int64_t g = blockIdx.x; g < groups; g += gridDim.x, parity ^= 1) {
    const int64_t base = g * kR;
    wait_group(smem_u32(&full[slot]), phase, &abort_flag, p.status);
    const uint8_t* slot_ptr = ring + (size_t)slot * slot_bytes;
    uint32_t xp[kR][kC][4];
    bool row_ok[kR];
#pragma unroll
    for (int r = 0; r < kR; ++r) {
      row_ok[r] = base + r < p.rows;
      const uint4* src = reinterpret_cast<const uint4*>(slot_ptr + (size_t)r * row_bytes);
#pragma unroll
      for (int c = 0; c < kC; ++c) {
        const uint4 a = live[c] ? src[threadIdx.x + c * T] : make_uint4(0, 0, 0, 0);
        xp[r][c][0] = a.x; xp[r][c][1] = a.y; xp[r][c][2] = a.z; xp[r][c][3] = a.w;
      }
    }
    float rstd[kR];
    if (which < 2) {
      float acc[kR];
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        float2 s2 = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int c = 0; c < kC; ++c) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 x = bf16x2_to_f2(xp[r][c][e]);
            s2 = f2_fma(x, x, s2);
          }
        }
        acc[r] = row_ok[r] ? s2.x + s2.y : 0.0f;      // chunks past the row hold zeros
      }
      // warp stage: fold the two values across lane bit 4, finish over the other bits
      {
        static_assert(kR == 2, "the fold below is written for two rows per group");
        const int lane = threadIdx.x & 31;
        const bool up = (lane & 16) != 0;
        const float keep = up ? acc[1] : acc[0], give = up ? acc[0] : acc[1];
        float v = keep + __shfl_xor_sync(0xffffffffu, give, 16);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        if ((lane & 15) == 0) red[parity][up ? 1 : 0][threadIdx.x >> 5] = v;
      }
      __syncthreads();
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        float t = 0.0f;
        for (int w4 = 0; w4 < warps; w4 += 4) {
          const float4 q = *reinterpret_cast<const float4*>(&red[parity][r][w4]);
          t += (q.x + q.y) + (q.z + q.w);
        }
        rstd[r] = rsqrtf(t / dim_f + p.eps);
      }
    } else {
      __syncthreads();
    }
    // every thread holds its chunks: the slot can take the group kStages ahead
    {
      const int64_t gn = g + (int64_t)kStages * gridDim.x;
      if (threadIdx.x == 0 && gn < groups) issue(gn, slot);
    }

#pragma unroll
    for (int r = 0; r < kR; ++r) {
      if (!row_ok[r]) continue;
      const float2 r2 = make_float2(rstd[r], rstd[r]);
      const float2 sign = make_float2(-1.0f, 1.0f);
#pragma unroll
      for (int c = 0; c < kC; ++c) {
        if (!live[c]) continue;
        uint32_t o[4];
        if (which < 2) {
          // this token's rotation table entries for the chunk's four pairs (L1 / L2 hits: every
          // head of the token reads the same 512 bytes)
          float4 cs[2];
          if (rotate) {
            const float4* t = reinterpret_cast<const float4*>(p.cos_sin + (base + r) * half_hd + (d0[c] >> 1));
            cs[0] = __ldg(t);
            cs[1] = __ldg(t + 1);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // normalized pair, rounded to bf16 as the unfused model rounds it
            const uint32_t nb = f2_to_bf16x2(f2_mul(f2_mul(bf16x2_to_f2(xp[r][c][e]), r2), gain[c][e]));
            if (!rotate) {
              o[e] = nb;
              continue;
            }
            const float2 n = bf16x2_to_f2(nb);
            const float4 t4 = cs[e >> 1];
            const float cc = (e & 1) ? t4.z : t4.x, ss = (e & 1) ? t4.w : t4.y;
            const float2 nc = f2_mul(n, make_float2(cc, cc));                      // (x1 c, x2 c)
            const float2 ns = f2_mul(make_float2(n.y, n.x), make_float2(ss, ss));  // (x2 s, x1 s)
            o[e] = f2_to_bf16x2(f2_fma(ns, sign, nc));   // (x1 c - x2 s, x2 c + x1 s), +-1 exact
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] = xp[r][c][e];
        }
        *reinterpret_cast<uint4*>(dst_base[c] + (base + r) * p.out_row_bytes + out_off[c]) =
            make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    if (++slot == kStages) {
      slot = 0;
      phase ^= 1u;
    }
  }
  if (abort_flag) {
    // a wait expired: give copies still in flight time to land before the shared memory is
    // handed to another CTA
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
  }
  // exchange form: the CTA that finishes last tells every rank that this rank's pieces are in
  // place (flags of kind 0)
  if (p.signal) xsync::signal_when_grid_done(p.peers, 0, gridDim.x * gridDim.y, false);
}

int launch_rope(RopeArgs& a, int tensors, cudaStream_t st) {
  // enough threads for every 8-element chunk of a row, kC chunks per thread, whole warps
  const int threads = ((a.dim / 8 + kC - 1) / kC + 31) / 32 * 32;
  const size_t smem = (size_t)kStages * kR * a.dim * 2;
  // (dynamic shared memory limit, CTAs per SM) of the last geometry seen on each device:
  // the model calls this with one row width over and over
  struct Geometry { size_t smem; int threads; int per_sm; };
  static Geometry cached[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  Geometry& c = cached[dev];
  if (c.per_sm < 1 || c.smem != smem || c.threads != threads) {
    if (cudaFuncSetAttribute(qk_norm_rope_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return NVFP4_ERR_LAUNCH_FAILED;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, qk_norm_rope_kernel, threads, smem) !=
            cudaSuccess || n < 1)
      return NVFP4_ERR_LAUNCH_FAILED;
    c = Geometry{smem, threads, n};
  }
  const int per_sm = c.per_sm;
  const int64_t groups = (a.rows + kR - 1) / kR;
  int64_t gx = ((int64_t)sm_count() * per_sm + tensors - 1) / tensors;
  if (gx > groups) gx = groups;
  if (gx < 1) gx = 1;
  qk_norm_rope_kernel<<<dim3((unsigned)gx, (unsigned)tensors), threads, smem, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH_FAILED;
}

}  // namespace
}  // namespace nvfp4

using namespace nvfp4;

extern "C" NVFP4_API int nvfp4_qk_norm_rope_bf16(const void* q_in, const void* k_in, const void* v_in,
                                       int64_t in_row_stride, int64_t rows, int heads, int head_dim,
                                       const float* gain_q, const float* gain_k, float eps,
                                       const float* cos_sin, void* q_out, void* k_out, void* v_out,
                                       int64_t out_row_stride, int64_t out_head_stride,
                                       int* status_dev, void* stream) {
  const int64_t dim = (int64_t)heads * head_dim;
  if (rows < 0 || heads <= 0 || head_dim <= 0 || head_dim % 16 != 0 || dim > 8 * kC * kMaxThreads ||
      in_row_stride < dim || out_head_stride < head_dim || in_row_stride % 8 != 0 ||
      out_row_stride % 8 != 0 || out_head_stride % 8 != 0)
    return NVFP4_ERR_BAD_ARG;
  if (rows > 0 && (!q_in || !q_out)) return NVFP4_ERR_BAD_ARG;
  if ((k_in == nullptr) != (k_out == nullptr) || (v_in == nullptr) != (v_out == nullptr) ||
      (v_in && !k_in))
    return NVFP4_ERR_BAD_ARG;
  if (!aligned16(q_in) || !aligned16(k_in) || !aligned16(v_in) || !aligned16(q_out) ||
      !aligned16(k_out) || !aligned16(v_out) || !aligned16(gain_q) || !aligned16(gain_k) ||
      !aligned16(cos_sin))
    return NVFP4_ERR_BAD_ALIGN;
  int rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
  if (rows == 0) return NVFP4_OK;
  RopeArgs a{};
  a.in[0] = static_cast<const uint8_t*>(q_in);
  a.in[1] = static_cast<const uint8_t*>(k_in);
  a.in[2] = static_cast<const uint8_t*>(v_in);
  a.in_row_bytes = in_row_stride * 2;
  a.rows = rows;
  a.dim = (int)dim;
  a.head_dim = head_dim;
  a.gain[0] = gain_q;
  a.gain[1] = gain_k;
  a.eps = eps;
  a.cos_sin = reinterpret_cast<const float2*>(cos_sin);
  a.out[0] = static_cast<uint8_t*>(q_out);
  a.out[1] = static_cast<uint8_t*>(k_out);
  a.out[2] = static_cast<uint8_t*>(v_out);
  a.out_row_bytes = out_row_stride * 2;
  a.out_head_bytes = out_head_stride * 2;
  a.status = status_dev;
  return launch_rope(a, v_in ? 3 : (k_in ? 2 : 1), reinterpret_cast<cudaStream_t>(stream));
}

extern "C" NVFP4_API int nvfp4_qk_norm_rope_exchange_bf16(
    const void* q_in, const void* k_in, const void* v_in, int64_t in_row_stride, int64_t rows,
    int heads, int head_dim, const float* gain_q, const float* gain_k, float eps,
    const float* cos_sin, void* const* rank_buffers, int world, int64_t row_offset,
    void* const* sync_blocks, int rank, int* status_dev, void* stream) {
  const int64_t dim = (int64_t)heads * head_dim;
  if (rows < 0 || heads <= 0 || head_dim <= 0 || head_dim % 16 != 0 || dim > 8 * kC * kMaxThreads ||
      in_row_stride < dim || in_row_stride % 8 != 0 || world < 1 || world > 8 ||
      heads % world != 0 || row_offset < 0 || !rank_buffers)
    return NVFP4_ERR_BAD_ARG;
  if (rows > 0 && (!q_in || !k_in || !v_in)) return NVFP4_ERR_BAD_ARG;
  if (!aligned16(q_in) || !aligned16(k_in) || !aligned16(v_in) || !aligned16(gain_q) ||
      !aligned16(gain_k) || !aligned16(cos_sin))
    return NVFP4_ERR_BAD_ALIGN;
  for (int r = 0; r < world; ++r) {
    if (!rank_buffers[r]) return NVFP4_ERR_BAD_ARG;
    if (!aligned16(rank_buffers[r])) return NVFP4_ERR_BAD_ALIGN;
  }
  RopeArgs a{};
  if (sync_blocks) {
    // a rank with nothing to send would raise no flag and leave its peers waiting
    if (rows == 0) return NVFP4_ERR_BAD_ARG;
    const int prc = exchange_fill_peers(a.peers, sync_blocks, world, rank);
    if (prc != NVFP4_OK) return prc;
    a.signal = 1;
  }
  int rc = check_device_sm100();
  if (rc != NVFP4_OK) return rc;
  if (rows == 0) return NVFP4_OK;
  a.in[0] = static_cast<const uint8_t*>(q_in);
  a.in[1] = static_cast<const uint8_t*>(k_in);
  a.in[2] = static_cast<const uint8_t*>(v_in);
  a.in_row_bytes = in_row_stride * 2;
  a.rows = rows;
  a.dim = (int)dim;
  a.head_dim = head_dim;
  a.gain[0] = gain_q;
  a.gain[1] = gain_k;
  a.eps = eps;
  a.cos_sin = reinterpret_cast<const float2*>(cos_sin);
  a.heads_per_rank = heads / world;
  a.out_head_bytes = (int64_t)3 * head_dim * 2;
  a.out_row_bytes = (int64_t)a.heads_per_rank * a.out_head_bytes;
  a.row_offset = row_offset;
  for (int r = 0; r < world; ++r) a.peer[r] = static_cast<uint8_t*>(rank_buffers[r]);
  a.status = status_dev;
  return launch_rope(a, 3, reinterpret_cast<cudaStream_t>(stream));
}
