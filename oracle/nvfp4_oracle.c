/*
 * NVFP4 CPU oracle -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's NVFP4 recipe: bf16 -> packed E2M1
 * nibbles + one FP8-E4M3 scale per 16-element K-block + one FP32 per-tensor
 * scale, the matching dequantizer, and the dequantize-then-matmul linear.
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may link
 * or call this file; the shipped CUDA path never does.
 *
 * Parity status.  The reference holds no golden vectors for packed bytes or
 * scales (its tests are statistical bounds only), so byte/scale parity is
 * pinned as follows instead of by reference fixtures:
 *   - scale bytes: against the reference's own kernel
 *     block_1d_quantization_kernel_te (fx/src/s4/nvfp4/quantization_te.cu:92)
 *     compiled from the reference tree by oracle/Makefile into oracle/_ref and
 *     run on a B200: its scale bytes for the golden cases are committed as
 *     tests/golden/ref_te_scales.npz (written by tests/golden/make_ref_scales.py)
 *     and compared with this file's on CPU and with the shipped kernel's on the
 *     GPU; where oracle/_ref is present the kernel is also run live.
 *   - E4M3 / E2M1 converters: exhaustively against the CUDA toolkit's host
 *     converters (cuda_fp8.h / cuda_fp4.h), which are the types the reference
 *     casts through (quantization_te.cu:51, quantization_te_clean.cu:70-79).
 *   - element nibbles: parity unpinned by the reference (its only E2M1 path is
 *     compiled out); they follow the PTX cvt.rn.satfinite.e2m1x2.f32 semantics
 *     that the reference's dead code names.
 *
 * Every function cites the reference lines it follows (paths relative to the
 * reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Threads the parallel loops below use (the benchmark's CPU-baseline leg sets it to the host's
 * core count explicitly: launchers such as torchrun export OMP_NUM_THREADS=1).  Returns the
 * number in effect. */
int nvfp4_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

#define NVFP4_BLOCK 16

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Round-to-nearest-even float -> bf16, the behaviour of __float2bfloat16
 * (fx/src/s4/nvfp4/quantization_te.cu:164). NaN maps to 0x7FFF. */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7FFFu + lsb;
  return (uint16_t)(u >> 16);
}

/* FP8 E4M3 (finite-only "fn" flavour: max 448, 0x7F = NaN), round to nearest
 * even, saturate to +-448: the behaviour of static_cast<__nv_fp8_e4m3>(float)
 * used at fx/src/s4/nvfp4/quantization_te.cu:51. */
uint8_t nvfp4_oracle_f32_to_e4m3(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint8_t sign = (uint8_t)((u >> 31) << 7);
  float a = fabsf(f);
  if (a != a) return 0x7F; /* any NaN -> canonical positive NaN */
  if (a >= 448.0f) return (uint8_t)(sign | 0x7E);
  if (a < 0.015625f) { /* below 2^-6: subnormal grid of 2^-9 */
    float q = nearbyintf(a * 512.0f); /* exact scaling, RN-even */
    return (uint8_t)(sign | (uint8_t)q); /* q == 8 is the smallest normal */
  }
  int e;
  float m = frexpf(a, &e); /* a = m * 2^e, m in [0.5,1) */
  m *= 2.0f;
  e -= 1; /* a = m * 2^e, m in [1,2) */
  float q = nearbyintf((m - 1.0f) * 8.0f);
  int mi = (int)q;
  if (mi == 8) {
    mi = 0;
    e += 1;
  }
  int code = ((e + 7) << 3) | mi;
  if (code > 0x7E) code = 0x7E;
  return (uint8_t)(sign | (uint8_t)code);
}

float nvfp4_oracle_e4m3_to_f32(uint8_t b) {
  int e = (b >> 3) & 0xF;
  int m = b & 7;
  float v;
  if (e == 0xF && m == 7)
    v = NAN;
  else if (e == 0)
    v = ldexpf((float)m, -9);
  else
    v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return (b & 0x80) ? -v : v;
}

/* FP4 E2M1 (sign | 2-bit exponent | 1-bit mantissa; magnitudes
 * {0,.5,1,1.5,2,3,4,6}), round to nearest even, saturate, NaN -> +6: the
 * semantics of cvt.rn.satfinite.e2m1x2.f32 which the reference intends at
 * fx/src/s4/nvfp4/quantization_te_clean.cu:70-79. */
uint8_t nvfp4_oracle_f32_to_e2m1(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint8_t sign = (uint8_t)((u >> 31) << 3);
  float a = fabsf(f);
  uint8_t code;
  if (a != a) return 0x7;
  if (a <= 0.25f)
    code = 0;
  else if (a < 0.75f)
    code = 1;
  else if (a <= 1.25f)
    code = 2;
  else if (a < 1.75f)
    code = 3;
  else if (a <= 2.5f)
    code = 4;
  else if (a < 3.5f)
    code = 5;
  else if (a <= 5.0f)
    code = 6;
  else
    code = 7;
  return (uint8_t)(sign | code);
}

static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* fx/src/s4/nvfp4/linear/nvfp4_linear.cpp:24 (table of E2M1 magnitudes). */
float nvfp4_oracle_e2m1_to_f32(uint8_t nib) {
  float v = kE2M1[nib & 7];
  return (nib & 8) ? -v : v;
}

/* Tensor-wide max |x| (fx/src/s4/nvfp4/tensor.cpp:54,
 * fx/src/s4/nvfp4/linear/nvfp4_linear.cpp:79). */
float nvfp4_oracle_amax_bf16(const uint16_t* x, int64_t n) {
  float amax = 0.0f;
#pragma omp parallel for reduction(max : amax)
  for (int64_t i = 0; i < n; ++i) {
    float v = fabsf(bf16_to_f32(x[i]));
    if (v > amax) amax = v;
  }
  return amax;
}

/* ComputeGlobalEncodeScaleFP4, fx/src/s4/nvfp4/quantization_te.cu:61-72. */
float nvfp4_oracle_global_encode_scale(float global_amax) {
  float s = 448.0f * 6.0f / global_amax;
  s = fminf(s, FLT_MAX);
  if (global_amax == 0.0f || s == 0.0f) return 1.0f;
  return s;
}

/* The FP32 per-tensor (decode) scale the packed tensor carries:
 * 1 / S_enc, the value the reference passes as global_decode_scale at
 * fx/src/s4/nvfp4/quantization_te.cu:113. */
float nvfp4_oracle_global_decode_scale(float global_amax) {
  return 1.0f / nvfp4_oracle_global_encode_scale(global_amax);
}

/* ComputeDecodeScaleFP4, fx/src/s4/nvfp4/quantization_te.cu:45-52. */
static inline uint8_t block_scale_e4m3(float amax_b, float s_enc) {
  float d = amax_b / 6.0f;
  d = d * s_enc;
  d = fminf(d, FLT_MAX);
  return nvfp4_oracle_f32_to_e4m3(d);
}

/* ComputeEncodeScaleFP4, fx/src/s4/nvfp4/quantization_te.cu:54-59. */
static inline float block_encode_scale(uint8_t sf, float global_decode_scale) {
  float denom = nvfp4_oracle_e4m3_to_f32(sf) * global_decode_scale;
  return fminf(1.0f / denom, FLT_MAX);
}

/* Quantize a row-major [rows, cols] bf16 matrix (cols % 16 == 0) given the
 * tensor amax.  Block loop of fx/src/s4/nvfp4/quantization_te.cu:92-135 with
 * the element conversion replaced by true E2M1 (see header); pack order
 * (odd << 4) | even per quantization_te.cu:133.  Scales are linear row-major
 * [rows, cols/16] per fx/src/s4/nvfp4/tensor.cpp:15. */
void nvfp4_oracle_quantize(const uint16_t* x, int64_t rows, int64_t cols, float global_amax,
                           uint8_t* packed, uint8_t* scales) {
  const float s_enc = nvfp4_oracle_global_encode_scale(global_amax);
  const float s_dec = 1.0f / s_enc;
  const int64_t nblk = rows * cols / NVFP4_BLOCK;
#pragma omp parallel for
  for (int64_t b = 0; b < nblk; ++b) {
    const uint16_t* xb = x + b * NVFP4_BLOCK;
    float amax = 0.0f;
    for (int i = 0; i < NVFP4_BLOCK; ++i) amax = fmaxf(amax, fabsf(bf16_to_f32(xb[i])));
    uint8_t sf = block_scale_e4m3(amax, s_enc);
    float enc = block_encode_scale(sf, s_dec);
    scales[b] = sf;
    for (int i = 0; i < NVFP4_BLOCK; i += 2) {
      uint8_t lo = nvfp4_oracle_f32_to_e2m1(bf16_to_f32(xb[i]) * enc);
      uint8_t hi = nvfp4_oracle_f32_to_e2m1(bf16_to_f32(xb[i + 1]) * enc);
      packed[(b * NVFP4_BLOCK + i) / 2] = (uint8_t)((hi << 4) | lo);
    }
  }
}

/* Dequantize to fp32: e2m1 * (float(sf) / S_enc), the scale expression of
 * fx/src/s4/nvfp4/quantization_te.cu:149-160 with the true E2M1 table. */
void nvfp4_oracle_dequantize_f32(const uint8_t* packed, const uint8_t* scales, int64_t rows,
                                 int64_t cols, float global_amax, float* out) {
  const float s_enc = nvfp4_oracle_global_encode_scale(global_amax);
  const int64_t n = rows * cols;
#pragma omp parallel for
  for (int64_t b = 0; b < n / NVFP4_BLOCK; ++b) {
    float d = nvfp4_oracle_e4m3_to_f32(scales[b]) / s_enc;
    for (int i = 0; i < NVFP4_BLOCK; ++i) {
      int64_t e = b * NVFP4_BLOCK + i;
      uint8_t byte = packed[e / 2];
      uint8_t nib = (e & 1) ? (byte >> 4) : (byte & 0xF);
      out[e] = nvfp4_oracle_e2m1_to_f32(nib) * d;
    }
  }
}

/* Same, rounded to bf16 as the reference kernel stores it
 * (fx/src/s4/nvfp4/quantization_te.cu:164-167). */
void nvfp4_oracle_dequantize_bf16(const uint8_t* packed, const uint8_t* scales, int64_t rows,
                                  int64_t cols, float global_amax, uint16_t* out) {
  const float s_enc = nvfp4_oracle_global_encode_scale(global_amax);
  const int64_t n = rows * cols;
#pragma omp parallel for
  for (int64_t b = 0; b < n / NVFP4_BLOCK; ++b) {
    float d = nvfp4_oracle_e4m3_to_f32(scales[b]) / s_enc;
    for (int i = 0; i < NVFP4_BLOCK; ++i) {
      int64_t e = b * NVFP4_BLOCK + i;
      uint8_t byte = packed[e / 2];
      uint8_t nib = (e & 1) ? (byte >> 4) : (byte & 0xF);
      out[e] = f32_to_bf16(nvfp4_oracle_e2m1_to_f32(nib) * d);
    }
  }
}

/* Size in bytes of the 128x4-interleaved scale buffer the tensor-core GEMM
 * reads (rows padded to 256, K-blocks padded to 16). */
int64_t nvfp4_oracle_swizzled_scale_bytes(int64_t rows, int64_t cols) {
  int64_t rt = (rows + 255) / 256 * 2;           /* 128-row tiles */
  int64_t kt = ((cols / 16) + 15) / 16 * 4;      /* 4-block k-atoms */
  return rt * kt * 512;
}

/* Re-order linear [rows, cols/16] scales into 512-byte atoms of 128 rows x 4
 * K-blocks laid out [32][4][4]: the SF layout the reference's GEMM asks
 * CUTLASS for at fx/src/s4/nvfp4/kernel.cu:91-96 (tile_atom_to_shape_SFA).
 * Padding bytes are zero. */
void nvfp4_oracle_swizzle_scales(const uint8_t* linear, int64_t rows, int64_t cols,
                                 uint8_t* swz) {
  int64_t kb = cols / 16;
  int64_t kt = (kb + 15) / 16 * 4;
  memset(swz, 0, (size_t)nvfp4_oracle_swizzled_scale_bytes(rows, cols));
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t k = 0; k < kb; ++k) {
      int64_t off = ((r / 128) * kt + k / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + k % 4;
      swz[off] = linear[r * kb + k];
    }
}

/* tanh-approximated GELU as the DiT feed-forward uses it
 * (fx/src/s4/models/wan22/wan_transformer.py:185, approximate="tanh"). */
static inline float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}

/* Reference linear: Y = bf16( sum_k xhat*what (fp32) + bias ), operands being
 * the fp32 dequantized values (fx/src/s4/nvfp4/linear/nvfp4_gemm_kernel.cu:
 * 137-142).  xq/wq are fp32 dequantized matrices [M,K], [N,K].  Optional
 * epilogue terms mirror the fused GEMM epilogue: act (0 none, 1 GELU-tanh),
 * gate[N] (fp32) and residual[M,N] (bf16): y = res + gate * act(acc + bias). */
void nvfp4_oracle_matmul_nt(const float* xq, const float* wq, const uint16_t* bias, int64_t M,
                            int64_t N, int64_t K, int act, const float* gate,
                            const uint16_t* residual, uint16_t* y_bf16, float* y_f32) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    const float* xr = xq + m * K;
    for (int64_t n = 0; n < N; ++n) {
      const float* wr = wq + n * K;
      /* eight independent partial sums keep the loop vectorisable while the
       * order stays fixed and compiler-independent */
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      int64_t k = 0;
      for (; k + 8 <= K; k += 8)
        for (int j = 0; j < 8; ++j) acc[j] += xr[k + j] * wr[k + j];
      float s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
      for (; k < K; ++k) s += xr[k] * wr[k];
      if (bias) s += bf16_to_f32(bias[n]);
      if (act == 1) s = gelu_tanh(s);
      if (gate) s *= gate[n];
      if (residual) s += bf16_to_f32(residual[m * N + n]);
      if (y_f32) y_f32[m * N + n] = s;
      if (y_bf16) y_bf16[m * N + n] = f32_to_bf16(s);
    }
  }
}

/* Whole CPU linear on bf16 inputs: quantize X and W (each with its own tensor
 * amax), dequantize, matmul, bias.  This is the reference's CPU arithmetic
 * for the path (host fake-quantizer + matmul,
 * fx/src/s4/nvfp4/linear/nvfp4_linear.cpp:61-152) restated with the true
 * NVFP4 codes; it is what the benchmark's cpu_baseline leg times.
 * Returns 0, or -1 when scratch memory cannot be allocated. */
int nvfp4_oracle_linear(const uint16_t* x, const uint16_t* w, const uint16_t* bias, int64_t M,
                        int64_t N, int64_t K, int act, uint16_t* y_bf16) {
  uint8_t* xp = malloc((size_t)(M * K / 2));
  uint8_t* xs = malloc((size_t)(M * K / 16));
  uint8_t* wp = malloc((size_t)(N * K / 2));
  uint8_t* ws = malloc((size_t)(N * K / 16));
  float* xq = malloc((size_t)(M * K) * 4);
  float* wq = malloc((size_t)(N * K) * 4);
  int rc = -1;
  if (xp && xs && wp && ws && xq && wq) {
    float ax = nvfp4_oracle_amax_bf16(x, M * K);
    float aw = nvfp4_oracle_amax_bf16(w, N * K);
    nvfp4_oracle_quantize(x, M, K, ax, xp, xs);
    nvfp4_oracle_quantize(w, N, K, aw, wp, ws);
    nvfp4_oracle_dequantize_f32(xp, xs, M, K, ax, xq);
    nvfp4_oracle_dequantize_f32(wp, ws, N, K, aw, wq);
    nvfp4_oracle_matmul_nt(xq, wq, bias, M, N, K, act, NULL, NULL, y_bf16, NULL);
    rc = 0;
  }
  free(xp); free(xs); free(wp); free(ws); free(xq); free(wq);
  return rc;
}

/* Check of a device-side shortcut, not part of the restated algorithm: the kernels form x / 6
 * as q0 = x * fl(1/6), q = fma(fma(-6, q0, x), fl(1/6), q0) inside [1e-30, 1e37] and by IEEE
 * division outside.  Returns the number of inputs among the n given for which that differs
 * from x / 6.0f (the tests feed every bf16 value and a few million fp32 values: expect 0). */
int64_t nvfp4_oracle_div6_mismatches(const float* x, int64_t n) {
  const float c = 1.0f / 6.0f;
  int64_t bad = 0;
  for (int64_t i = 0; i < n; ++i) {
    volatile float ref = x[i] / 6.0f;
    float q;
    if (x[i] >= 1e-30f && x[i] <= 1e37f) {
      const float q0 = x[i] * c;
      q = fmaf(fmaf(-6.0f, q0, x[i]), c, q0);
    } else {
      q = x[i] / 6.0f;
    }
    const float r = ref;
    if (memcmp(&q, &r, sizeof q) != 0 && !(q != q && r != r)) ++bad;
  }
  return bad;
}

