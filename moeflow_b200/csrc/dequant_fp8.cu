// Block-scaled e4m3 weights -> bf16, one pass over the tensor.
//
// Used by the long-prefill path of layers that hold e4m3 experts: from 256-row token tiles on, the bf16 grouped
// GEMMs (two accumulators of 256 columns, no per-K-block promotion) are faster than the block-scaled ones, so the
// layer expands the experts of the current forward into a bf16 scratch first (three times the e4m3 bytes of HBM
// traffic, a few percent of a compute-bound forward) and runs the bf16 kernels on it.
//
// Layout: w8 [rows, K] e4m3, scale [rows / 128, K / 128] fp32 (the checkpoint's weight_scale_inv, experts
// concatenated along the rows), out [rows, K] bf16.  value = float(e4m3) * scale, rounded once to bf16.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "moeflow_b200.h"

namespace mf {

__global__ void __launch_bounds__(256) dequant_block_fp8_kernel(const uint8_t* w8, const float* scale, __nv_bfloat16* out,
                                                                long long rows, int K) {
  grid_dep_wait_cta();
  grid_dep_launch();
  const int chunks_per_row = K / 16;  // 16 e4m3 values per thread and step
  const int k_blocks = K / 128;
  const long long total = rows * chunks_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / chunks_per_row;
    const int c = (int)(i - r * chunks_per_row);
    const uint4 q = __ldcs(reinterpret_cast<const uint4*>(w8 + r * K) + c);  // streamed once
    const float s = __ldg(scale + (r >> 7) * k_blocks + (c >> 3));
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[8];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __nv_fp8x2_storage_t pair = (__nv_fp8x2_storage_t)((words[w] >> (16 * h)) & 0xffffu);
        const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
        const __nv_bfloat162 b = __floats2bfloat162_rn(f.x * s, f.y * s);
        o[2 * w + h] = *reinterpret_cast<const uint32_t*>(&b);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + r * K + (long long)c * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

}  // namespace mf

// rows % 128 == 0, K % 128 == 0; pointers 16-byte aligned.  Returns 0, a negative code for bad arguments, or the
// CUDA error of the launch.
extern "C" int mf_dequant_block_fp8(const void* w8, const float* scale, void* out_bf16, long long rows, int K,
                                    void* stream) {
  if (w8 == nullptr || scale == nullptr || out_bf16 == nullptr) return -1;
  if (rows <= 0 || K <= 0 || rows % 128 != 0 || K % 128 != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(w8) | reinterpret_cast<uintptr_t>(out_bf16)) & 15) return -3;
  const long long total = rows * (K / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)mf::launch_kernel(mf::dequant_block_fp8_kernel, dim3((unsigned)blocks), dim3(256), 0,
                                static_cast<cudaStream_t>(stream), true, static_cast<const uint8_t*>(w8), scale,
                                static_cast<__nv_bfloat16*>(out_bf16), rows, K);
}
