// TEST INFRASTRUCTURE ONLY.  C-ABI shim over the reference's own launchers in
// fx/src/s4/nvfp4/quantization_te.cu (declared at quantization.cuh:52-58), so
// that tests can run the reference kernel on a GPU and compare its E4M3 block
// scales byte-for-byte with the oracle and with the shipped kernel.  The
// reference source is compiled from where it lies (see oracle/Makefile); no
// reference code is copied here.
#include <cstdint>
#include <cuda_runtime.h>

#include "quantization.cuh"

extern "C" {

int ref_te_quantize(const void* x_bf16, uint8_t* packed, uint8_t* scales, int64_t n,
                    float global_amax, void* stream) {
  s4::nvfp4::launch_block_1d_quantization_cuda_te(
      reinterpret_cast<const at::BFloat16*>(x_bf16), packed, scales, n, global_amax,
      reinterpret_cast<cudaStream_t>(stream));
  return (int)cudaGetLastError();
}

int ref_te_dequantize(const uint8_t* packed, const uint8_t* scales, void* out_bf16, int64_t n,
                      float global_amax, void* stream) {
  s4::nvfp4::launch_block_1d_dequantization_cuda_te(
      packed, scales, reinterpret_cast<at::BFloat16*>(out_bf16), n, global_amax,
      reinterpret_cast<cudaStream_t>(stream));
  return (int)cudaGetLastError();
}
}
