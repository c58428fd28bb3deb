// int8 -> f16 operand construction shared by the decode and prefill kernels.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace bp {

// Two k-slices of B = K^T from one word of four int8. DENORM: x + 128 placed in
// the low byte of an f16 is the subnormal (x + 128) * 2^-24, exact, and the
// +128 is removed later with the block sums of Q. Otherwise the byte is placed
// under 0x64 (1024 + x + 128) and 1152 is subtracted.
template <bool DENORM>
__device__ __forceinline__ void k_pair(uint32_t w, uint32_t& b0, uint32_t& b1) {
  const uint32_t x = w ^ 0x80808080u;
  if (DENORM) {
    b0 = x & 0x00ff00ffu;
    b1 = (x >> 8) & 0x00ff00ffu;
  } else {
    const __half2 bias = __half2half2(__ushort_as_half(0x6480));  // 1152
    uint32_t e = (x & 0x00ff00ffu) | 0x64006400u;
    uint32_t o = ((x >> 8) & 0x00ff00ffu) | 0x64006400u;
    __half2 eh = __hsub2(*reinterpret_cast<__half2*>(&e), bias);
    __half2 oh = __hsub2(*reinterpret_cast<__half2*>(&o), bias);
    b0 = *reinterpret_cast<uint32_t*>(&eh);
    b1 = *reinterpret_cast<uint32_t*>(&oh);
  }
}

template <bool DENORM>
__device__ __forceinline__ uint32_t v_fix(uint32_t a) {
  if (DENORM) return a;
  const __half2 bias = __half2half2(__ushort_as_half(0x6480));
  __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), bias);
  return *reinterpret_cast<uint32_t*>(&r);
}


}  // namespace bp
