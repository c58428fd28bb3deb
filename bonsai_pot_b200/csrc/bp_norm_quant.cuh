// Device functions shared by the write-back / Q kernels and the fused decode kernel: RMS-norm +
// weight + NEOX rotation of one head held by one warp (lane l = dims 4l..4l+3), and the block-32
// absmax quantiser. Every step uses explicitly rounded intrinsics (never contracted) and a fixed
// reduction tree, so that all callers produce the same bits as the CPU oracle.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace bp {

constexpr unsigned NRQ_FULL = 0xffffffffu;

struct Rot4 {
  float v[4];
};

// f16 load, RMS-norm, weight, NEOX rotation of R heads held by one warp at once. The R rows start at
// x, x + row_stride, ...; they sit at the same position (one rope_row) and share the norm weight w
// ([128] f16; rope_row: [64][2] f16). Every step runs over the R rows before the next step starts, so
// the rows' dependency chains (shuffles, the division, the reciprocal square root) overlap instead of
// queueing up. total / 128 is written as a multiplication by 2^-7, which rounds identically.
template <int R>
__device__ __forceinline__ void norm_rope_rows(const __half* x, size_t row_stride, const __half* w,
                                               const __half* rope_row, float eps, int lane, Rot4 (&out)[R]) {
  const uint2 wr = *reinterpret_cast<const uint2*>(w + 4 * lane);
  const uint4 rr = *reinterpret_cast<const uint4*>(rope_row + 8 * (lane & 15));
  const __half2* wh = reinterpret_cast<const __half2*>(&wr);
  const __half2* rh = reinterpret_cast<const __half2*>(&rr);
  float wt[4];
  {
    const float2 c = __half22float2(wh[0]), d = __half22float2(wh[1]);
    wt[0] = c.x; wt[1] = c.y; wt[2] = d.x; wt[3] = d.y;
  }
  float raw[R][4], sq[R][4];
#pragma unroll
  for (int r = 0; r < R; r++) {
    const uint2 xr = *reinterpret_cast<const uint2*>(x + r * row_stride + 4 * lane);
    const __half2* xh = reinterpret_cast<const __half2*>(&xr);
    const float2 a = __half22float2(xh[0]), b = __half22float2(xh[1]);
    raw[r][0] = a.x; raw[r][1] = a.y; raw[r][2] = b.x; raw[r][3] = b.y;
#pragma unroll
    for (int c = 0; c < 4; c++) sq[r][c] = __fmul_rn(raw[r][c], raw[r][c]);
  }
#pragma unroll
  for (int off = 4; off >= 1; off >>= 1) {
#pragma unroll
    for (int r = 0; r < R; r++) {
#pragma unroll
      for (int c = 0; c < 4; c++) sq[r][c] = __fadd_rn(sq[r][c], __shfl_xor_sync(NRQ_FULL, sq[r][c], off));
    }
  }
  float w32[R], inv_h[R];
#pragma unroll
  for (int r = 0; r < R; r++) w32[r] = __fadd_rn(__fadd_rn(sq[r][0], sq[r][2]), __fadd_rn(sq[r][1], sq[r][3]));
#pragma unroll
  for (int r = 0; r < R; r++) w32[r] = __fadd_rn(w32[r], __shfl_xor_sync(NRQ_FULL, w32[r], 8));
#pragma unroll
  for (int r = 0; r < R; r++) {
    const float total = __fadd_rn(w32[r], __shfl_xor_sync(NRQ_FULL, w32[r], 16));
    inv_h[r] = __frsqrt_rn(__fadd_rn(__fmul_rn(total, 0.0078125f), eps));
  }
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const float2 cs = __half22float2(rh[c]);  // (cos, sin) of j = dim mod 64
    // Lower half: x cos - partner sin; upper half: partner sin + x cos. One code path for both:
    // a - b == a + (-b) and (-p) s == -(p s) hold exactly in IEEE arithmetic, and + commutes.
    const float sn = lane < 16 ? -cs.y : cs.y;
#pragma unroll
    for (int r = 0; r < R; r++) {
      const float xn = __fmul_rn(__fmul_rn(raw[r][c], inv_h[r]), wt[c]);
      const float partner = __shfl_xor_sync(NRQ_FULL, xn, 16);
      out[r].v[c] = __fadd_rn(__fmul_rn(xn, cs.x), __fmul_rn(partner, sn));
    }
  }
}

// One head.
__device__ __forceinline__ Rot4 norm_rope(const __half* x, const __half* w, const __half* rope_row, float eps, int lane) {
  Rot4 out[1];
  norm_rope_rows<1>(x, 0, w, rope_row, eps, lane, out);
  return out[0];
}

// Block-32 absmax quantiser over 8 lanes x 4 values. Returns the packed int8
// word of this lane; *d_out is the block scale (same in all 8 lanes).
__device__ __forceinline__ uint32_t quant4(const float* x, float* d_out) {
  float a = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
  a = fmaxf(a, __shfl_xor_sync(NRQ_FULL, a, 1));
  a = fmaxf(a, __shfl_xor_sync(NRQ_FULL, a, 2));
  a = fmaxf(a, __shfl_xor_sync(NRQ_FULL, a, 4));
  const float d = __fdiv_rn(a, 127.0f);
  const float inv = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
  uint32_t packed = 0;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    float r = rintf(__fmul_rn(x[c], inv));
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    packed |= (static_cast<uint32_t>(static_cast<int>(r)) & 0xffu) << (8 * c);
  }
  *d_out = d;
  return packed;
}


}  // namespace bp
