// The non-attention operators of one decode / prefill layer on Q1_0 weights: what the reference's
// matvec_q1_0*.wgsl, rms_norm.wgsl, silu_mul.wgsl, embed.wgsl, quantize_q8_0.wgsl,
// matmul_q1_0_q8_0.wgsl and topk_reduce.wgsl compute, with the same operation ORDER, so that the
// f16 / f32 results are the reference's bit for bit under the evaluation rules the CPU restatement
// states (f16 operations rounded one by one, no FMA contraction, correctly rounded division and
// reciprocal square root, a fixed exp): every rounded operation below is an explicit intrinsic.
//
// Matvec family (one token): a row is reduced by 8 lanes, lane tx taking the 128-weight blocks
// b = tx (mod 8) in order, as the shaders do (matvec_q1_0.wgsl:84-133). Inside a block the four f16
// accumulators of the shader's vec4<f16> are two half2 registers; a weight's sign is applied by
// flipping the activation's sign bit. The sign bits are re-laid out once at load (bp_q1_relayout)
// so that the xor mask of a half2 is ONE shift and ONE and: word 0 / 1 of a block hold, for the
// groups g = 0..15 / 16..31, the flip bit of element 4 g at bit 15 - g and of element 4 g + 1 at
// bit 31 - g; words 2 / 3 the same for elements 4 g + 2, 4 g + 3. A lane works on four rows at
// once (the activations it reads from shared memory serve all four).
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <math.h>

#include "bp_common.cuh"
#include "bp_ptx.cuh"
#include "bp_q1_ops.cuh"

namespace {

using namespace bp;
namespace cg = cooperative_groups;
constexpr unsigned FULL = 0xffffffffu;
constexpr uint32_t MV_THREADS = 128;          // the invocation count of the fused shader: its sum of squares is per invocation
// rows per lane (R): 4 for tall tensors (the activations a lane reads serve all of them), fewer for the
// 4096-row ones, which would otherwise give the device only 64 CTAs
constexpr uint32_t XB_STRIDE = 128 + 8;       // halves per staged block: 16 bytes of padding keep the 8 lanes of a row off each other's banks

__device__ __forceinline__ float exp_det(float x) {  // the restatement's orc_exp_det, operation for operation
  x = fminf(fmaxf(x, -87.3f), 88.7f);
  const float n = rintf(__fmul_rn(x, 1.44269504088896341f));
  float r = __fmaf_rn(n, -0.693359375f, x);
  r = __fmaf_rn(n, 2.12194440e-4f, r);
  float p = __fmaf_rn(r, 1.0f / 720.0f, 1.0f / 120.0f);
  p = __fmaf_rn(r, p, 1.0f / 24.0f);
  p = __fmaf_rn(r, p, 1.0f / 6.0f);
  p = __fmaf_rn(r, p, 0.5f);
  p = __fmaf_rn(r, p, 1.0f);
  p = __fmaf_rn(r, p, 1.0f);
  return ldexpf(p, static_cast<int>(n));
}

// f16(g / (1 + exp(-g))) * up, in f16 (silu_mul.wgsl:22-26)
__device__ __forceinline__ __half silu_times_up(__half gate, __half up) {
  const float g = __half2float(gate);
  const float s = __fdiv_rn(g, __fadd_rn(1.0f, exp_det(-g)));
  return __hmul(__float2half_rn(s), up);
}

// subgroupAdd of a 32-lane subgroup: xor butterfly 16, 8, 4, 2, 1
__device__ __forceinline__ float butterfly32(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(FULL, v, off));
  return v;
}

// Workgroup sum of rms_norm.wgsl:62-78 / matvec_q1_0_fused_normed.wgsl:131-146 for a CTA of NW warps:
// per-warp butterfly, partial of warp s into lane s of warp 0 (zero elsewhere), butterfly again.
template <uint32_t NW>
__device__ __forceinline__ float workgroup_sum(float v, float* part /* shared, 32 floats */) {
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float s = butterfly32(v);
  if (lane == 0) part[warp] = s;
  __syncthreads();
  if (warp == 0) {
    const float c = lane < NW ? part[lane] : 0.0f;
    const float f = butterfly32(c);
    if (lane == 0) part[0] = f;
  }
  __syncthreads();
  const float total = part[0];
  __syncthreads();
  return total;
}

struct MvRange {
  const __half* d;        // block scales [n][nb]
  const uint4* bits;      // re-laid-out sign words [n][nb]
  __half* out;
  uint32_t n;
};
struct MvParams {
  MvRange r[3];
  uint32_t n_ranges, n_total, k;
  const __half* x;        // input activations (MODE 0, 1) or gate (MODE 2)
  const __half* aux;      // norm weight (MODE 1) or up (MODE 2)
  float eps;
  uint32_t accumulate;
};

// MODE 0: y (+)= W x (matvec_q1_0.wgsl); 1: W (rms_norm(x) * w), scales times inv_rms
// (matvec_q1_0_fused_normed.wgsl); 2: y (+)= W (silu(gate) * up) (matvec_q1_0_silu.wgsl);
// 3: MODE 1 over two tensors of equal height (gate, up) with silu_mul.wgsl applied to the pair of results:
// a lane computes row i of both (MV_ROWS_PER_LANE = 2 is the tensor index) and writes
// silu(f16(gate_i)) * f16(up_i), what the two dispatches of the reference leave in the buffer that feeds
// the down projection.
constexpr uint32_t MV_PF = 4;  // blocks of a lane in flight
// KB != 0: an instance for tensors of exactly 1024 KB inputs (KB blocks per lane: 4 and 12 at the 8B shape). With
// the block count a constant the loop bounds, the reload conditions and most of the address arithmetic of the
// general code fold away (about a tenth of the instructions of a call).
template <int MODE, uint32_t MV_ROWS_PER_LANE, uint32_t KB = 0>
__global__ void __launch_bounds__(MV_THREADS) matvec_q1_kernel(const MvParams p) {
  static_assert(MODE != 3 || MV_ROWS_PER_LANE == 2, "the paired mode computes one row of each of two tensors per lane");
  constexpr uint32_t MV_ROWS_PER_CTA = (MV_THREADS / 8) * (MODE == 3 ? 1 : MV_ROWS_PER_LANE);
  extern __shared__ __align__(16) uint8_t mv_smem[];
  __shared__ float part[32];
  __half* xs = reinterpret_cast<__half*>(mv_smem);
  pdl_launch_dependents();
  const uint32_t k_in = KB != 0 ? 1024u * KB : p.k;
  const uint32_t tid = threadIdx.x, nb = k_in / 128u;
  // ---- rows: lane = (row slot rs = lane / 8, tx = lane % 8); a lane owns rows base + rs + 4 j ----
  const uint32_t warp = tid >> 5, lane = tid & 31, tx = lane & 7, rs = lane >> 3;
  const uint32_t row0 = blockIdx.x * MV_ROWS_PER_CTA + warp * (4 * (MODE == 3 ? 1 : MV_ROWS_PER_LANE)) + rs;
  const __half* d_row[MV_ROWS_PER_LANE];
  const uint4* b_row[MV_ROWS_PER_LANE];
  __half* out_ptr[MV_ROWS_PER_LANE];
  bool valid[MV_ROWS_PER_LANE];
#pragma unroll
  for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++) {
    uint32_t row = MODE == 3 ? row0 : row0 + 4u * j;
    valid[j] = row < (MODE == 3 ? p.r[0].n : p.n_total);
    if (!valid[j]) row = 0;
    uint32_t ri = MODE == 3 ? j : 0;
    if (MODE != 3 && p.n_ranges > 1 && row >= p.r[0].n) {
      row -= p.r[0].n;
      ri = 1;
      if (p.n_ranges > 2 && row >= p.r[1].n) {
        row -= p.r[1].n;
        ri = 2;
      }
    }
    d_row[j] = p.r[ri].d + static_cast<size_t>(row) * nb;
    b_row[j] = p.r[ri].bits + static_cast<size_t>(row) * nb;
    out_ptr[j] = p.r[ri].out + row;
  }
  float acc[MV_ROWS_PER_LANE];
#pragma unroll
  for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++) acc[j] = 0.0f;
  const __half2 zero2 = __float2half2_rn(0.0f);
  // A lane works through its blocks tx, tx + 8, ... in order, and a block's sign words and scale are
  // requested MV_PF blocks ahead: with one block ahead a call was a chain of k / 1024 memory latencies
  // (8.9 us for 4096 x 12288 weights). The weights are constants: the first MV_PF blocks are on their way to
  // registers, and the others to L2, while the kernel before this one, which produces the activations, is
  // still running.
  uint4 w_q[MV_PF][MV_ROWS_PER_LANE];
  __half d_q[MV_PF][MV_ROWS_PER_LANE];
#pragma unroll
  for (uint32_t u = 0; u < MV_PF; u++) {
    if (tx + 8 * u < nb) {
#pragma unroll
      for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++) {
        w_q[u][j] = __ldg(b_row[j] + tx + 8 * u);
        d_q[u][j] = __ldg(d_row[j] + tx + 8 * u);
      }
    }
  }
  for (uint32_t b = tx + 8 * MV_PF; b < nb; b += 8) {
#pragma unroll
    for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++) prefetch_l2(b_row[j] + b);
  }
  if (tx == 0) {
#pragma unroll
    for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++)
      for (uint32_t b = 64; b < nb; b += 64) prefetch_l2(d_row[j] + b);  // scales: 64 per 128-byte line
  }
  pdl_wait();  // the activations come from the kernel before this one
  float inv_rms = 1.0f;
  // ---- stage the activations: block b at xs + b * XB_STRIDE ----
  // Loads of a batch are all requested before the first is used: one load per loop iteration made the
  // staging a chain of k / 512 L2 latencies (24 of them for the 12288-wide down projection).
  if (MODE == 1 || MODE == 3) {
    float ssq = 0.0f;
    constexpr uint32_t SB = 8;  // 4-element units of a thread per batch
    for (uint32_t v0 = tid; v0 < k_in / 4u; v0 += MV_THREADS * SB) {
      uint2 raw_q[SB], wr_q[SB];
#pragma unroll
      for (uint32_t u = 0; u < SB; u++) {
        const uint32_t v = v0 + u * MV_THREADS;
        if (v < k_in / 4u) {
          raw_q[u] = *reinterpret_cast<const uint2*>(p.x + 4u * v);
          wr_q[u] = __ldg(reinterpret_cast<const uint2*>(p.aux + 4u * v));
        }
      }
#pragma unroll
      for (uint32_t u = 0; u < SB; u++) {
        const uint32_t v = v0 + u * MV_THREADS;
        if (v >= k_in / 4u) break;
        const uint2 raw = raw_q[u], wr = wr_q[u];
        const __half2 x01 = *reinterpret_cast<const __half2*>(&raw.x), x23 = *reinterpret_cast<const __half2*>(&raw.y);
        const float2 f01 = __half22float2(x01), f23 = __half22float2(x23);
        ssq = __fadd_rn(ssq, __fmul_rn(f01.x, f01.x));
        ssq = __fadd_rn(ssq, __fmul_rn(f01.y, f01.y));
        ssq = __fadd_rn(ssq, __fmul_rn(f23.x, f23.x));
        ssq = __fadd_rn(ssq, __fmul_rn(f23.y, f23.y));
        const __half2 y01 = __hmul2(x01, *reinterpret_cast<const __half2*>(&wr.x));
        const __half2 y23 = __hmul2(x23, *reinterpret_cast<const __half2*>(&wr.y));
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&y01);
        o.y = *reinterpret_cast<const uint32_t*>(&y23);
        *reinterpret_cast<uint2*>(xs + (v >> 5) * XB_STRIDE + 4u * (v & 31u)) = o;
      }
    }
    const float total = workgroup_sum<MV_THREADS / 32>(ssq, part);
    inv_rms = __frsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(k_in)), p.eps));
  } else if (MODE == 0) {
    constexpr uint32_t SB = 6;  // 8-element units of a thread per batch
    for (uint32_t v0 = tid; v0 < k_in / 8u; v0 += MV_THREADS * SB) {
      uint4 raw_q[SB];
#pragma unroll
      for (uint32_t u = 0; u < SB; u++) {
        const uint32_t v = v0 + u * MV_THREADS;
        if (v < k_in / 8u) raw_q[u] = *reinterpret_cast<const uint4*>(p.x + 8u * v);
      }
#pragma unroll
      for (uint32_t u = 0; u < SB; u++) {
        const uint32_t v = v0 + u * MV_THREADS;
        if (v < k_in / 8u) *reinterpret_cast<uint4*>(xs + (v >> 4) * XB_STRIDE + 8u * (v & 15u)) = raw_q[u];
      }
    }
    __syncthreads();
  } else {
    for (uint32_t v = tid; v < k_in / 4u; v += MV_THREADS) {
      uint2 o = *reinterpret_cast<const uint2*>(p.x + 4u * v);
      const uint2 u = *reinterpret_cast<const uint2*>(p.aux + 4u * v);
      const __half* g4 = reinterpret_cast<const __half*>(&o);
      const __half* u4 = reinterpret_cast<const __half*>(&u);
      __half y[4];
#pragma unroll
      for (int c = 0; c < 4; c++) y[c] = silu_times_up(g4[c], u4[c]);
      o = *reinterpret_cast<const uint2*>(y);
      *reinterpret_cast<uint2*>(xs + (v >> 5) * XB_STRIDE + 4u * (v & 31u)) = o;
    }
    __syncthreads();
  }

  for (uint32_t b0 = tx; b0 < nb; b0 += 8 * MV_PF) {
#pragma unroll
  for (uint32_t u = 0; u < MV_PF; u++) {
    const uint32_t b = b0 + 8 * u;
    if (b >= nb) break;
    uint4 w[MV_ROWS_PER_LANE];
    __half dh[MV_ROWS_PER_LANE];
#pragma unroll
    for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++) {
      w[j] = w_q[u][j];
      dh[j] = d_q[u][j];
    }
    if (b + 8 * MV_PF < nb) {
#pragma unroll
      for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++) {
        w_q[u][j] = __ldg(b_row[j] + b + 8 * MV_PF);
        d_q[u][j] = __ldg(d_row[j] + b + 8 * MV_PF);
      }
    }
    __half2 a01[MV_ROWS_PER_LANE], a23[MV_ROWS_PER_LANE];
#pragma unroll
    for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++) a01[j] = a23[j] = zero2;
    const uint4* xb = reinterpret_cast<const uint4*>(xs + b * XB_STRIDE);
#pragma unroll
    for (uint32_t half = 0; half < 2; half++) {  // groups 0..15, then 16..31
#pragma unroll
      for (uint32_t g2 = 0; g2 < 8; g2++) {      // two groups per 16-byte read
        const uint4 xv = xb[half * 8 + g2];
#pragma unroll
        for (uint32_t gg = 0; gg < 2; gg++) {
          const uint32_t g = 2 * g2 + gg;
          const uint32_t x01 = gg ? xv.z : xv.x, x23 = gg ? xv.w : xv.y;
#pragma unroll
          for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++) {
            const uint32_t w01 = half ? w[j].y : w[j].x, w23 = half ? w[j].w : w[j].z;
            const uint32_t s01 = x01 ^ ((w01 << g) & 0x80008000u);
            const uint32_t s23 = x23 ^ ((w23 << g) & 0x80008000u);
            a01[j] = __hadd2(a01[j], *reinterpret_cast<const __half2*>(&s01));
            a23[j] = __hadd2(a23[j], *reinterpret_cast<const __half2*>(&s23));
          }
        }
      }
    }
#pragma unroll
    for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++) {
      const __half ls = __hadd(__hadd(__hadd(__low2half(a01[j]), __high2half(a01[j])), __low2half(a23[j])), __high2half(a23[j]));
      float d = __half2float(dh[j]);
      if (MODE == 1 || MODE == 3) d = __fmul_rn(d, inv_rms);
      acc[j] = __fadd_rn(acc[j], __fmul_rn(d, __half2float(ls)));
    }
  }
  }
  float total[MV_ROWS_PER_LANE];
#pragma unroll
  for (uint32_t j = 0; j < MV_ROWS_PER_LANE; j++) {
    float a = acc[j];
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 1));
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 2));
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 4));
    total[j] = a;
    if (MODE != 3 && tx == 0 && valid[j]) {
      if (MODE != 1 && p.accumulate) a = __fadd_rn(__half2float(*out_ptr[j]), a);
      *out_ptr[j] = __float2half_rn(a);
    }
  }
  if (MODE == 3 && tx == 0 && valid[0])
    *out_ptr[0] = silu_times_up(__float2half_rn(total[0]), __float2half_rn(total[MV_ROWS_PER_LANE - 1]));
}

// rms_norm.wgsl:41-85: one CTA of 512 threads per group.
__global__ void __launch_bounds__(512) rms_norm_kernel(const __half* in, __half* out, const __half* w, uint32_t n, float eps) {
  __shared__ float part[32];
  pdl_launch_dependents();
  pdl_wait();
  const __half* src = in + static_cast<size_t>(blockIdx.x) * n;
  __half* dst = out + static_cast<size_t>(blockIdx.x) * n;
  float s = 0.0f;
  for (uint32_t i = threadIdx.x; i < n; i += 512) {
    const float v = __half2float(src[i]);
    s = __fadd_rn(s, __fmul_rn(v, v));
  }
  const float total = workgroup_sum<16>(s, part);
  const __half inv_h = __float2half_rn(__frsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(n)), eps)));
  for (uint32_t i = threadIdx.x; i < n; i += 512) dst[i] = __hmul(__hmul(src[i], inv_h), w[i]);
}

// silu_mul.wgsl:18-27
// A thread takes eight values (16-byte loads and stores) where the buffers allow it, else one.
template <bool VEC8>
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* gate, const __half* up, __half* out, uint64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (VEC8) {
    if (8u * i >= n) return;
    const uint4 g = *reinterpret_cast<const uint4*>(gate + 8u * i), u = *reinterpret_cast<const uint4*>(up + 8u * i);
    const __half* g8 = reinterpret_cast<const __half*>(&g);
    const __half* u8 = reinterpret_cast<const __half*>(&u);
    __half y[8];
#pragma unroll
    for (int c = 0; c < 8; c++) y[c] = silu_times_up(g8[c], u8[c]);
    *reinterpret_cast<uint4*>(out + 8u * i) = *reinterpret_cast<const uint4*>(y);
  } else {
    if (i < n) out[i] = silu_times_up(gate[i], up[i]);
  }
}

// embed.wgsl:37-52: thread = one 16-byte unit (8 weights) of an output row
__global__ void __launch_bounds__(256) embed_kernel(const __half* d, const uint8_t* qs, uint32_t k, const uint32_t* tokens,
                                                    uint32_t m, __half* x) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t units = k / 8u;
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= static_cast<uint64_t>(m) * units) return;
  const uint32_t t = static_cast<uint32_t>(idx / units), u = static_cast<uint32_t>(idx % units);
  const uint64_t row = tokens[t];
  const uint32_t nb = k / 128u, b = u / 16u;
  const __half dp = d[row * nb + b], dn = __hneg(dp);
  const uint32_t byte = qs[(row * nb + b) * 16u + (u & 15u)];
  __half o[8];
#pragma unroll
  for (int bit = 0; bit < 8; bit++) o[bit] = (byte >> bit) & 1u ? dp : dn;
  *reinterpret_cast<uint4*>(x + static_cast<size_t>(t) * k + 8u * u) = *reinterpret_cast<const uint4*>(o);
}

// quantize_q8_0.wgsl:49-106. The shader reduces |x| over a block of 32 with a workgroup tree; the maximum does
// not depend on the order, so here a THREAD owns a block: 64 bytes in, the two divisions once per block instead
// of once per value, 32 bytes and one scale out (a warp per block spent 50 instructions per 32 values).
__global__ void __launch_bounds__(256) quantize_q8_kernel(const __half* x, uint64_t n_blocks, float* d_out, int8_t* qs_out) {
  pdl_launch_dependents();
  pdl_wait();
  const uint64_t blk = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (blk >= n_blocks) return;
  uint4 raw[4];
#pragma unroll
  for (int c = 0; c < 4; c++) raw[c] = *reinterpret_cast<const uint4*>(x + blk * 32u + 8u * c);
  const __half* h = reinterpret_cast<const __half*>(raw);
  float v[32];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; i++) {
    v[i] = __half2float(h[i]);
    amax = fmaxf(amax, fabsf(v[i]));
  }
  const float d = __fdiv_rn(amax, 127.0f);
  const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
  uint32_t q[8];
#pragma unroll
  for (int w = 0; w < 8; w++) {
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float r = fminf(fmaxf(rintf(__fmul_rn(v[4 * w + e], id)), -127.0f), 127.0f);
      word |= (static_cast<uint32_t>(static_cast<int>(r)) & 0xFFu) << (8 * e);
    }
    q[w] = word;
  }
  uint4* dst = reinterpret_cast<uint4*>(qs_out + blk * 32u);
  dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
  dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
  d_out[blk] = d;
}

// matmul_q1_0_q8_0.wgsl:57-293: y[m][n] (+)= sum_b sum_s (a_d[m][4 b + s] * w_d[n][b]) * f32(sumi), in that
// order. A CTA owns 64 x 64 outputs, a thread 4 (m) x 4 (n); the integer dot of 32 signs with 32 int8 values
// is 2 * dot(a, bit) - sum(a), eight dp4a each.
constexpr uint32_t MM_T = 64;
__global__ void __launch_bounds__(256) matmul_q1_q8_kernel(const __half* w_d, const uint8_t* w_qs, uint32_t k, uint32_t n, uint32_t m,
                                                           const float* a_d, const int8_t* a_qs, __half* y, uint32_t accumulate) {
  __shared__ float s_wd[MM_T];
  __shared__ uint32_t s_wb[MM_T][4 + 1];     // sign words of the block, one row per weight row
  __shared__ float s_ad[MM_T][4];
  __shared__ uint32_t s_aq[MM_T][32 + 1];    // 128 int8 of the block per token
  __shared__ int s_asum[MM_T][4];
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t tid = threadIdx.x, lx = tid & 15, ly = tid >> 4;
  const uint32_t n_base = blockIdx.x * MM_T, m_base = blockIdx.y * MM_T;
  const uint32_t nb1 = k / 128u, nb8 = k / 32u;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
  for (uint32_t b = 0; b < nb1; b++) {
    if (tid < MM_T) {
      const uint32_t ni = n_base + tid;
      s_wd[tid] = ni < n ? __half2float(w_d[static_cast<size_t>(ni) * nb1 + b]) : 0.0f;
    }
    {
      const uint32_t nl = tid >> 2, s = tid & 3, ni = n_base + nl;
      s_wb[nl][s] = ni < n ? *reinterpret_cast<const uint32_t*>(w_qs + (static_cast<size_t>(ni) * nb1 + b) * 16u + 4u * s) : 0u;
      const uint32_t ml = tid >> 2, mi = m_base + ml;
      s_ad[ml][s] = mi < m ? a_d[static_cast<size_t>(mi) * nb8 + 4u * b + s] : 0.0f;
    }
    for (uint32_t li = 0; li < 8; li++) {
      const uint32_t idx = li * 256 + tid, ml = idx >> 5, su = idx & 31, mi = m_base + ml;
      s_aq[ml][su] = mi < m ? *reinterpret_cast<const uint32_t*>(a_qs + static_cast<size_t>(mi) * k + 128u * b + 4u * su) : 0u;
    }
    __syncthreads();
    {
      const uint32_t ml = tid >> 2, s = tid & 3;
      int t = 0;
#pragma unroll
      for (int u = 0; u < 8; u++) t = __dp4a(static_cast<int>(s_aq[ml][8 * s + u]), 0x01010101, t);
      s_asum[ml][s] = t;
    }
    __syncthreads();
#pragma unroll
    for (uint32_t s = 0; s < 4; s++) {
      uint32_t spread[4][8];  // per weight row: 8 words whose bytes are 1 where the sign bit is set
#pragma unroll
      for (int tn = 0; tn < 4; tn++) {
        const uint32_t bw = s_wb[lx * 4 + tn][s];
#pragma unroll
        for (int u = 0; u < 8; u++) {
          const uint32_t bits = (bw >> (4 * u)) & 0xFu;
          spread[tn][u] = (bits & 1u) | ((bits & 2u) << 7) | ((bits & 4u) << 14) | ((bits & 8u) << 21);
        }
      }
#pragma unroll
      for (int tm = 0; tm < 4; tm++) {
        const uint32_t ml = ly * 4 + tm;
        const float ad = s_ad[ml][s];
        const int asum = s_asum[ml][s];
        int pos[4] = {0, 0, 0, 0};
#pragma unroll
        for (int u = 0; u < 8; u++) {
          const int a = static_cast<int>(s_aq[ml][8 * s + u]);
#pragma unroll
          for (int tn = 0; tn < 4; tn++) pos[tn] = __dp4a(a, static_cast<int>(spread[tn][u]), pos[tn]);
        }
#pragma unroll
        for (int tn = 0; tn < 4; tn++) {
          const float scale = __fmul_rn(ad, s_wd[lx * 4 + tn]);
          acc[tm][tn] = __fadd_rn(acc[tm][tn], __fmul_rn(scale, static_cast<float>(2 * pos[tn] - asum)));
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int tm = 0; tm < 4; tm++) {
    const uint32_t mi = m_base + ly * 4 + tm;
    if (mi >= m) continue;
#pragma unroll
    for (int tn = 0; tn < 4; tn++) {
      const uint32_t ni = n_base + lx * 4 + tn;
      if (ni >= n) continue;
      __half* dst = y + static_cast<size_t>(mi) * n + ni;
      const float v = accumulate ? __fadd_rn(__half2float(*dst), acc[tm][tn]) : acc[tm][tn];
      *dst = __float2half_rn(v);
    }
  }
}

// The same product with warp-level MMAs (mma.sync m16n8k32, int8 x int8 -> int32), for batches of more than
// MMA_MIN_M tokens: the integer dot of a sub-block of 32 is one MMA of the int8 activations with the weights
// as +1 / -1 bytes. What the reference does in floating point, y += (a_d * w_d) * f32(sumi) per sub-block
// in ascending order, is done in the same order by the thread that holds the MMA's accumulator, so the result
// has the same bits. A CTA of 16 warps owns 128 tokens x 128 weight rows, a warp 32 x 32 (2 x 4 MMA tiles
// of m16 n8). Per block of 128 inputs the CTA stages the activations [128][128] and the weights as +-1
// bytes [128][128] in shared memory (16-byte chunks xor-swizzled by the row, read back with ldmatrix); the
// next block's global loads are in flight while the current one is multiplied.
constexpr uint32_t MMA_MIN_M = 32;
constexpr uint32_t MT = 128;                        // tile edge, tokens and weight rows
constexpr uint32_t MMA_TILE_B = MT * 128;           // one operand tile: 128 rows of 128 int8
constexpr uint32_t MMA_SMEM = 4 * MMA_TILE_B + 2 * (MT * 4 + MT) * 4 + 64;  // A, B double-buffered, scales, sign table

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// d = a b + Q1_I2F_BIAS: the accumulator starts at the bit pattern of 1.5 * 2^23, so that the exact integer dot
// comes out as bits of the float 12582912 + dot, one subtraction away from float(dot) (exact for |dot| < 2^22;
// a sub-block's is below 2^12) with no conversion and no integer addition on the CUDA cores.
constexpr int Q1_I2F_BIAS = 0x4B400000;
__device__ __forceinline__ void mma_s8_s32(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(Q1_I2F_BIAS));
}
// Packed FP32 pairs (sm_100): one instruction rounds two products, or two sums, each exactly as the scalar
// instruction does (checked bit for bit on 32 million random operand pairs per operation). The assembler has
// been seen to contract a packed multiply into a packed add that consumes it, rounding modifiers or not, so a
// packed product is never fed to a packed add here: the accumulation uses the scalar add.
__device__ __forceinline__ void q1_mul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void q1_add2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// acc0 += (ad * w0) * float(dot0), acc1 += (ad * w1) * float(dot1), every product and sum rounded once, in that
// order (the shader's): five instructions for the two outputs instead of eight.
__device__ __forceinline__ void q1_accumulate2(float& acc0, float& acc1, float ad, float w0, float w1, int biased0, int biased1) {
  float f0, f1, p0, p1, q0, q1;
  q1_add2(f0, f1, __int_as_float(biased0), __int_as_float(biased1), -12582912.0f, -12582912.0f);
  q1_mul2(p0, p1, ad, ad, w0, w1);
  q1_mul2(q0, q1, p0, p1, f0, f1);
  acc0 = __fadd_rn(acc0, q0);
  acc1 = __fadd_rn(acc1, q1);
}
// four int8 -> four f16, exactly: bias to unsigned, 0x6400 | byte = 1024 + byte, minus 1152
__device__ __forceinline__ uint2 s8x4_to_f16x4(uint32_t x) {
  x ^= 0x80808080u;
  uint32_t lo = __byte_perm(x, 0x64646464u, 0x4140), hi = __byte_perm(x, 0x64646464u, 0x4342);
  const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));
  __half2 l = __hsub2(*reinterpret_cast<__half2*>(&lo), bias), h = __hsub2(*reinterpret_cast<__half2*>(&hi), bias);
  return make_uint2(*reinterpret_cast<uint32_t*>(&l), *reinterpret_cast<uint32_t*>(&h));
}

constexpr uint32_t MMA_THREADS = 512;   // 16 warps: 4 along the tokens x 4 along the weight rows
constexpr uint32_t MMA_SEG = MT * 128 / MMA_THREADS;  // inputs of one row that a thread stages: 32

// Up to three weight tensors over the same activations in one launch (Q, K and V of a layer: the K and V
// projections alone would fill a fifth of the device each): tile blockIdx.x belongs to the tensor whose
// range of tiles contains it.
struct MmaTensors {
  const __half* w_d[3];
  const uint8_t* w_qs[3];
  __half* y[3];
  uint32_t n[3];
  uint32_t tile_end[3];  // running total of 128-row tiles
  uint32_t tile0;        // the launch covers the tiles from this one on (blockIdx.x counts from it)
};

// MMA_MT_W m16 tiles per warp: 2 = tiles of 128 tokens, 1 = tiles of 64 tokens (every warp half the outputs, the
// weight tile staged as before), for launches whose 128-token tiles would leave most of the device idle in
// their last wave (Q, K and V at 512 tokens: 192 tiles on 148 SMs).
template <uint32_t MMA_MT_W>
__global__ void __launch_bounds__(MMA_THREADS, 1) matmul_q1_q8_mma_kernel(const MmaTensors tensors, uint32_t k, uint32_t m,
                                                                  const float* __restrict__ a_d, const int8_t* __restrict__ a_qs,
                                                                  uint32_t accumulate) {
  constexpr uint32_t TM = 64 * MMA_MT_W;  // tokens of a tile
  const uint32_t tile = blockIdx.x + tensors.tile0;
  const uint32_t which = tile < tensors.tile_end[0] ? 0u : tile < tensors.tile_end[1] ? 1u : 2u;
  const __half* __restrict__ w_d = tensors.w_d[which];
  const uint8_t* __restrict__ w_qs = tensors.w_qs[which];
  __half* y = tensors.y[which];
  const uint32_t n = tensors.n[which];
  extern __shared__ __align__(1024) uint8_t mm_smem[];
  uint8_t* sA = mm_smem;                                   // [2][128 tokens][128 int8]
  uint8_t* sB = mm_smem + 2 * MMA_TILE_B;                  // [2][128 weight rows][128 bytes of +1 / -1]
  float* s_ad = reinterpret_cast<float*>(mm_smem + 4 * MMA_TILE_B);      // [2][128][4]
  float* s_wd = s_ad + 2 * MT * 4;                                        // [2][128]
  uint32_t* s_sign = reinterpret_cast<uint32_t*>(s_wd + 2 * MT);         // nibble of sign bits -> four bytes of +-1
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t n_base = (tile - (which == 0 ? 0u : tensors.tile_end[which - 1])) * MT, m_base = blockIdx.y * TM;
  const uint32_t nb1 = k / 128u, nb8 = k / 32u;
  if (tid < 16) {
    uint32_t v = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) v |= ((tid >> e) & 1u ? 0x01u : 0xFFu) << (8 * e);  // bit set: +1, clear: -1
    s_sign[tid] = v;
  }
  // staging: thread -> (row, a segment of MMA_SEG of the row's 128 inputs)
  constexpr uint32_t SEGS = 128 / MMA_SEG, A_LD = MMA_SEG / 16, B_BYTES = MMA_SEG / 8;
  static_assert(B_BYTES == 4, "a thread stages one 32-bit word of sign bits");
  const uint32_t srow = tid / SEGS, sseg = tid % SEGS;
  const bool a_ok = srow < TM && m_base + srow < m, b_ok = n_base + srow < n;
  const int8_t* a_src = a_qs + static_cast<size_t>(m_base + srow) * k + MMA_SEG * sseg;
  const uint8_t* b_src = w_qs + static_cast<size_t>(n_base + srow) * nb1 * 16u + B_BYTES * sseg;
  uint4 ra[A_LD];
  uint32_t rb;
  float4 rad;
  float rwd;
  auto fetch = [&](uint32_t b) {
#pragma unroll
    for (uint32_t c = 0; c < A_LD; c++) ra[c] = a_ok ? *reinterpret_cast<const uint4*>(a_src + 128u * b + 16u * c) : make_uint4(0, 0, 0, 0);
    rb = b_ok ? *reinterpret_cast<const uint32_t*>(b_src + 16u * b) : 0u;
    if (tid < MT) {
      rad = tid < TM && m_base + tid < m ? *reinterpret_cast<const float4*>(a_d + static_cast<size_t>(m_base + tid) * nb8 + 4u * b)
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
    } else if (tid < 2 * MT) {
      const uint32_t ni = n_base + tid - MT;
      rwd = ni < n ? __half2float(w_d[static_cast<size_t>(ni) * nb1 + b]) : 0.0f;
    }
  };
  auto stage = [&](uint32_t buf) {
    uint8_t* arow = sA + buf * MMA_TILE_B + srow * 128u;
    uint8_t* brow = sB + buf * MMA_TILE_B + srow * 128u;
#pragma unroll
    for (uint32_t c = 0; c < A_LD; c++)  // a chunk of 16 int8 as it is
      *reinterpret_cast<uint4*>(arow + (((sseg * A_LD + c) ^ (srow & 7u)) << 4)) = ra[c];
#pragma unroll
    for (uint32_t j = 0; j < B_BYTES; j += 2) {  // two bytes of signs -> one chunk of 16 bytes
      const uint32_t b0 = (rb >> (8 * j)) & 0xFFu, b1 = (rb >> (8 * j + 8)) & 0xFFu;
      *reinterpret_cast<uint4*>(brow + (((sseg * (B_BYTES / 2) + (j >> 1)) ^ (srow & 7u)) << 4)) =
          make_uint4(s_sign[b0 & 15u], s_sign[b0 >> 4], s_sign[b1 & 15u], s_sign[b1 >> 4]);
    }
    if (tid < MT) {
      *reinterpret_cast<float4*>(s_ad + buf * MT * 4 + tid * 4) = rad;
    } else if (tid < 2 * MT) {
      s_wd[buf * MT + tid - MT] = rwd;
    }
  };
  const uint32_t wm = warp >> 2, wn = warp & 3, g = lane >> 2, t = lane & 3;
  float acc[MMA_MT_W][4][4];
#pragma unroll
  for (uint32_t i = 0; i < MMA_MT_W; i++)
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[i][j][e] = 0.0f;
  // ldmatrix row addresses of this lane: matrix lane >> 3, row lane & 7
  const uint32_t lm = lane >> 3, lr = lane & 7;
  const uint32_t a_row0 = wm * (16u * MMA_MT_W) + (lm & 1u) * 8u + lr, a_chunk0 = lm >> 1;  // + 16 per m tile; chunk + 2 per sub-block
  const uint32_t b_row0 = wn * 32u + (lm >> 1) * 8u + lr, b_chunk0 = lm & 1u;        // + 16 per pair of n tiles
  const uint32_t sA_u = static_cast<uint32_t>(__cvta_generic_to_shared(sA)), sB_u = static_cast<uint32_t>(__cvta_generic_to_shared(sB));

  __syncthreads();  // the sign table
  fetch(0);
  stage(0);
  __syncthreads();
  for (uint32_t b = 0; b < nb1; b++) {
    const uint32_t buf = b & 1u;
    if (b + 1 < nb1) fetch(b + 1);
    const float* ad = s_ad + buf * MT * 4;
    const float* wd = s_wd + buf * MT;
    float wdv[4][2];
#pragma unroll
    for (int nt = 0; nt < 4; nt++) {
      wdv[nt][0] = wd[wn * 32u + nt * 8u + 2u * t];
      wdv[nt][1] = wd[wn * 32u + nt * 8u + 2u * t + 1u];
    }
#pragma unroll 1
    for (uint32_t s = 0; s < 4; s++) {
      uint32_t bf[4][2];  // [n tile][register]
#pragma unroll
      for (uint32_t jp = 0; jp < 2; jp++) {
        const uint32_t row = b_row0 + jp * 16u, chunk = s * 2u + b_chunk0;
        ldmatrix_x4(sB_u + buf * MMA_TILE_B + row * 128u + ((chunk ^ (row & 7u)) << 4), bf[2 * jp][0], bf[2 * jp][1], bf[2 * jp + 1][0],
                    bf[2 * jp + 1][1]);
      }
#pragma unroll
      for (uint32_t mt = 0; mt < MMA_MT_W; mt++) {
        uint32_t af[4];
        {
          const uint32_t row = a_row0 + mt * 16u, chunk = s * 2u + a_chunk0;
          ldmatrix_x4(sA_u + buf * MMA_TILE_B + row * 128u + ((chunk ^ (row & 7u)) << 4), af[0], af[1], af[2], af[3]);
        }
        const float ad_lo = ad[(wm * (16u * MMA_MT_W) + mt * 16u + g) * 4u + s], ad_hi = ad[(wm * (16u * MMA_MT_W) + mt * 16u + g + 8u) * 4u + s];
#pragma unroll
        for (uint32_t nt = 0; nt < 4; nt++) {
          int d[4];
          mma_s8_s32(d, af, bf[nt][0], bf[nt][1]);
          q1_accumulate2(acc[mt][nt][0], acc[mt][nt][1], ad_lo, wdv[nt][0], wdv[nt][1], d[0], d[1]);
          q1_accumulate2(acc[mt][nt][2], acc[mt][nt][3], ad_hi, wdv[nt][0], wdv[nt][1], d[2], d[3]);
        }
      }
    }
    if (b + 1 < nb1) stage(buf ^ 1u);
    __syncthreads();
  }
#pragma unroll
  for (uint32_t mt = 0; mt < MMA_MT_W; mt++)
#pragma unroll
    for (uint32_t nt = 0; nt < 4; nt++)
#pragma unroll
      for (uint32_t e = 0; e < 4; e++) {
        const uint32_t mi = m_base + wm * (16u * MMA_MT_W) + mt * 16u + g + (e >> 1) * 8u, ni = n_base + wn * 32u + nt * 8u + 2u * t + (e & 1u);
        if (mi >= m || ni >= n) continue;
        __half* dst = y + static_cast<size_t>(mi) * n + ni;
        const float v = accumulate ? __fadd_rn(__half2float(*dst), acc[mt][nt][e]) : acc[mt][nt][e];
        *dst = __float2half_rn(v);
      }
}

// The same product on the 5th-generation tensor cores (tcgen05); selectable (variant 3), not the default.
// The arithmetic that has to stay on the CUDA cores, three roundings per output and sub-block, is what
// bounds it; the integer dots cost nothing on the tensor pipe. They are computed as f16 MMAs with FP32
// accumulation: every operand is an integer below 2^11 and every partial sum an integer below 2^13, so
// the result is the exact integer whatever the order of the additions, already in FP32 (no conversion).
// A CTA owns 128 tokens x 128 weight rows. Per half block (64 inputs = two sub-blocks):
//   16 worker warps   stage the half block two steps ahead (thread = 16 inputs of a row: int8 -> f16 for
//                     the activations, sign bits -> f16 +-1 for the weights) into a ring of K-major
//                     128-byte-swizzled operand tiles, then take the finished half block out of TMEM:
//                     thread = token = TMEM lane, 32 weight rows: y += (a_d * w_d) * sumi in the
//                     reference's order, accumulated in registers over all blocks
//   warp 0, lane 0    per sub-block two tcgen05.mma kind::f16 (M 128, N 128, K 16) into one of two TMEM
//                     buffers of 2 x 128 columns, one step ahead of the workers
// Every wait is bounded; a wait that gives up stores a code in the error word and the CTA winds down.
constexpr uint32_t UM_STAGES = 4, UM_TILE_B = 16384, UM_STAGE_B = 2 * UM_TILE_B;
constexpr uint32_t UM_EPI_WARPS = 16;
constexpr uint32_t UM_THREADS = (1 + UM_EPI_WARPS) * 32;
constexpr uint32_t UM_SMEM = UM_STAGES * UM_STAGE_B + 1024;
static __device__ uint32_t g_q1_err;  // error word of launches that were given none

__global__ void __launch_bounds__(UM_THREADS, 1) matmul_q1_q8_umma_kernel(const __half* __restrict__ w_d, const uint8_t* __restrict__ w_qs,
                                                                          uint32_t k, uint32_t n, uint32_t m, const float* __restrict__ a_d,
                                                                          const int8_t* __restrict__ a_qs, __half* y, uint32_t accumulate,
                                                                          uint32_t* err, uint32_t wait_limit) {
  extern __shared__ uint8_t um_raw[];
  __shared__ __align__(8) uint64_t full[UM_STAGES], empty[UM_STAGES], d_full[2], d_empty[2];
  __shared__ uint2 s_sign[16];
  __shared__ __align__(16) float s_wd[UM_EPI_WARPS][32];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile uint32_t abort_s;
  const uint32_t smem_base = (smem_u32(um_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = um_raw + (smem_base - smem_u32(um_raw));
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t n_base = blockIdx.x * MT, m_base = blockIdx.y * MT;
  const uint32_t nb1 = k / 128u, nb8 = k / 32u, n_stages = 2u * nb1;
  if (err == nullptr) err = &g_q1_err;
  if (tid == 0) {
    for (uint32_t i = 0; i < UM_STAGES; i++) {
      mbar_init(smem_u32(&full[i]), UM_EPI_WARPS);
      mbar_init(smem_u32(&empty[i]), 1);
    }
    for (uint32_t i = 0; i < 2; i++) {
      mbar_init(smem_u32(&d_full[i]), 1);
      mbar_init(smem_u32(&d_empty[i]), UM_EPI_WARPS);
    }
    abort_s = 0;
    fence_barrier_init();
  }
  if (tid < 16) {
    uint32_t h[4];
#pragma unroll
    for (int e = 0; e < 4; e++) h[e] = (tid >> e) & 1u ? 0x3C00u : 0xBC00u;  // bit set: +1, clear: -1
    s_sign[tid] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
  }
  if (warp == 0) tmem_alloc(smem_u32(&tmem_base_s), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  if (tid == 0) pdl_launch_dependents();
  pdl_wait();
  // try_wait with a suspend-time hint: sixteen warps polling at full rate would take issue slots from
  // the warps that are computing
  auto waitb = [&](uint64_t* bar, uint32_t parity) {
    if (abort_s) return;
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < wait_limit; i++) {
      uint32_t ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(addr), "r"(parity), "r"(2000u)
          : "memory");
      if (ok) return;
    }
    abort_s = 1;
    atomicExch(err, 6u);
  };

  if (warp == 0) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t IDESC = umma_idesc(1, 0, 0, 0, 0, 128, 128);  // f32 = f16 (K-major) x f16 (K-major)
      const uint64_t dk = umma_desc_sw128(0, 16, 1024);
      for (uint32_t j = 0; j < n_stages && !abort_s; j++) {
        const uint32_t slot = j % UM_STAGES, pb = j & 1u;
        waitb(&full[slot], (j / UM_STAGES) & 1u);
        if (j >= 2) waitb(&d_empty[pb], ((j >> 1) - 1u) & 1u);
        tc_fence_after();
        const uint64_t ad = dk + ((smem_base + slot * UM_STAGE_B) >> 4), bd = ad + (UM_TILE_B >> 4);
#pragma unroll
        for (uint32_t sb = 0; sb < 2; sb++)      // sub-block: 32 inputs = 64 bytes along the row
#pragma unroll
          for (uint32_t ks = 0; ks < 2; ks++)    // 16 inputs per MMA
            umma_f16(tmem + pb * 256u + sb * 128u, ad + sb * 4u + ks * 2u, bd + sb * 4u + ks * 2u, IDESC, ks);
        umma_commit(smem_u32(&empty[slot]));
        umma_commit(smem_u32(&d_full[pb]));
      }
    }
  } else {
    // ---------------- workers ----------------
    // staging: thread = 16 inputs (quarter q of the half block) of row srow, of A and of B
    const uint32_t wt = tid - 32u, srow = wt >> 2, sq = wt & 3u;
    const bool a_ok = m_base + srow < m, b_ok = n_base + srow < n;
    const int8_t* a_src = a_qs + static_cast<size_t>(m_base + srow) * k + 16u * sq;
    const uint8_t* b_src = w_qs + static_cast<size_t>(n_base + srow) * nb1 * 16u + 2u * sq;
    uint4 ra, ra2 = make_uint4(0, 0, 0, 0);   // the data of the step after next, and of the one after that
    uint32_t rb, rb2 = 0;
    auto fetch = [&](uint32_t h) {
      ra = ra2;
      rb = rb2;
      ra2 = a_ok ? *reinterpret_cast<const uint4*>(a_src + 64u * h) : make_uint4(0, 0, 0, 0);
      rb2 = b_ok ? *reinterpret_cast<const uint16_t*>(b_src + 8u * h) : 0u;
    };
    auto store = [&](uint32_t h) {
      const uint32_t slot = h % UM_STAGES;
      if (h >= UM_STAGES) waitb(&empty[slot], ((h / UM_STAGES) - 1u) & 1u);
      uint8_t* arow = smem_gen + slot * UM_STAGE_B + srow * 128u;
      uint8_t* brow = arow + UM_TILE_B;
      const uint2 h0 = s8x4_to_f16x4(ra.x), h1 = s8x4_to_f16x4(ra.y), h2 = s8x4_to_f16x4(ra.z), h3 = s8x4_to_f16x4(ra.w);
      *reinterpret_cast<uint4*>(arow + (((2u * sq) ^ (srow & 7u)) << 4)) = make_uint4(h0.x, h0.y, h1.x, h1.y);
      *reinterpret_cast<uint4*>(arow + (((2u * sq + 1u) ^ (srow & 7u)) << 4)) = make_uint4(h2.x, h2.y, h3.x, h3.y);
#pragma unroll
      for (uint32_t jb = 0; jb < 2; jb++) {  // one byte of signs -> one chunk of 8 halves; zeros beyond the last weight row
        const uint32_t byte = (rb >> (8u * jb)) & 0xFFu;
        const uint2 lo = s_sign[byte & 15u], hi = s_sign[byte >> 4];
        *reinterpret_cast<uint4*>(brow + (((2u * sq + jb) ^ (srow & 7u)) << 4)) = b_ok ? make_uint4(lo.x, lo.y, hi.x, hi.y) : make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&full[slot]));
    };
    // epilogue: thread = token (TMEM lane), 32 weight rows
    const uint32_t quad = warp & 3u, ew = warp - 1u, cg = ew >> 2;  // TMEM lane quarter; columns 32 cg ..
    const uint32_t row = quad * 32u + lane, mi = m_base + row;
    const uint32_t t_addr = tmem + ((quad * 32u) << 16) + cg * 32u;
    const bool row_ok = mi < m;
    const uint32_t my_col = n_base + cg * 32u + lane;  // the weight row whose scale this lane fetches for its warp
    const float* ad_src = a_d + static_cast<size_t>(mi) * nb8;
    const __half* wd_src = w_d + static_cast<size_t>(my_col) * nb1;
    float acc[32];
#pragma unroll
    for (int c = 0; c < 32; c++) acc[c] = 0.0f;
    float4 ad_next = row_ok ? *reinterpret_cast<const float4*>(ad_src) : make_float4(0.f, 0.f, 0.f, 0.f);
    float wd_next = my_col < n ? __half2float(wd_src[0]) : 0.0f;
    float adv[4] = {0.f, 0.f, 0.f, 0.f};
    // the first two steps, and the third one's data on its way
    // fetch(h) requests step h and makes step h - 1, requested one call earlier, the one that store() writes
    fetch(0);
    fetch(1);
    store(0);
    fetch(n_stages > 2 ? 2 : 1);
    store(1);
    fetch(n_stages > 3 ? 3 : 1);  // now: step 2 ready to be stored, step 3 on its way
    for (uint32_t j = 0; j < n_stages && !abort_s; j++) {
      const uint32_t pb = j & 1u, b = j >> 1;
      if (j + 2 < n_stages) {
        store(j + 2);
        fetch(j + 4 < n_stages ? j + 4 : j + 2);  // (past the end: any valid step, never stored)
      }
      if (pb == 0) {  // a new block: its scales, and the next block's on their way
        adv[0] = ad_next.x; adv[1] = ad_next.y; adv[2] = ad_next.z; adv[3] = ad_next.w;
        __syncwarp();
        s_wd[ew][lane] = wd_next;
        __syncwarp();
        if (b + 1 < nb1) {
          if (row_ok) ad_next = *reinterpret_cast<const float4*>(ad_src + 4u * (b + 1u));
          if (my_col < n) wd_next = __half2float(wd_src[b + 1u]);
        }
      }
      waitb(&d_full[pb], (j >> 1) & 1u);
      tc_fence_after();
      // The half block's 2 x 32 columns in four loads of 16, each in flight while the previous one's
      // sixteen outputs are scaled and added (all workers reach this point together: without the overlap
      // every load's latency would be exposed on all of them at once).
      uint32_t d[2][16];
      tmem_ld16(t_addr + pb * 256u, d[0]);
#pragma unroll
      for (uint32_t q = 0; q < 4; q++) {  // quarter q: sub-block q / 2, columns 16 (q % 2) ..
        tmem_ld_wait();
        if (q < 3) {
          tmem_ld16(t_addr + pb * 256u + ((q + 1u) >> 1) * 128u + ((q + 1u) & 1u) * 16u, d[(q + 1u) & 1u]);
        } else {  // the whole half block is in registers: the buffer may take the MMAs of the step after next
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&d_empty[pb]));
        }
        const float ad_s = adv[2u * pb + (q >> 1)];
        const uint32_t c0 = (q & 1u) * 16u;
#pragma unroll
        for (int c4 = 0; c4 < 4; c4++) {
          const float4 w4 = *reinterpret_cast<const float4*>(&s_wd[ew][c0 + 4 * c4]);
          const uint32_t* dq = d[q & 1u] + 4 * c4;
          float* a4 = acc + c0 + 4 * c4;
          a4[0] = __fadd_rn(a4[0], __fmul_rn(__fmul_rn(ad_s, w4.x), __uint_as_float(dq[0])));
          a4[1] = __fadd_rn(a4[1], __fmul_rn(__fmul_rn(ad_s, w4.y), __uint_as_float(dq[1])));
          a4[2] = __fadd_rn(a4[2], __fmul_rn(__fmul_rn(ad_s, w4.z), __uint_as_float(dq[2])));
          a4[3] = __fadd_rn(a4[3], __fmul_rn(__fmul_rn(ad_s, w4.w), __uint_as_float(dq[3])));
        }
      }
    }
    if (row_ok && !abort_s) {
      __half* dst = y + static_cast<size_t>(mi) * n + n_base + cg * 32u;
#pragma unroll
      for (int c = 0; c < 32; c++) {
        if (n_base + cg * 32u + c >= n) break;
        const float v = accumulate ? __fadd_rn(__half2float(dst[c]), acc[c]) : acc[c];
        dst[c] = __float2half_rn(v);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// topk_reduce.wgsl:59-196, the same steps on the same lists (256 per-invocation min-heaps of 32, heapsort,
// then log2(256) bitonic merge rounds), so that ties fall exactly where the shader's comparisons put them.
// What differs is only how the steps are scheduled:
//   - list j's element i sits at [i][slot of j] in shared memory as one 8-byte (value, index) pair;
//   - a sift moves the inserted element down a chain of holes instead of swapping at every level (the same
//     comparisons, hence the same final array);
//   - a list is scanned from a chunk of logits staged in shared memory, and the lanes of a warp are not held
//     in step: per chunk a lane first marks, in one straight-line pass, the elements above its heap's root,
//     then walks its marks (see the loop);
//   - for the merge rounds each list is moved to a row of its own (33 entries apart: consecutive lanes then
//     read consecutive entries of ONE list, as the shader's layout has it).
constexpr uint32_t TK_WG = 256, TK_K = 32, TK_CHUNK = 32;  // chunk: words (two logits) per list and stage
constexpr uint32_t TK_ROW = TK_K + 1;                      // entries between the rows of the merge rounds
// The kernel runs as one cluster of TK_CTAS CTAs of TK_THREADS threads, TK_WG / TK_CTAS lists per CTA, one lane per
// list: 16 CTAs with two lists per warp where the device forms clusters of 16 (88 us at 151936 logits), else the
// portable 8 with four lists per warp (98 us).
constexpr uint32_t TK_THREADS = TK_WG;  // the merge rounds of the first CTA run on the shader's 256 invocations
struct __align__(8) TkEntry { float v; uint32_t i; };
constexpr size_t tk_smem_bytes(uint32_t ctas) {
  return (TK_WG * TK_ROW + TK_K * (TK_WG / ctas)) * sizeof(TkEntry) + TK_CHUNK * (TK_WG / ctas) * sizeof(__half2);
}
// heap[0] of list j is being replaced by e: walk down while a child is smaller (topk_reduce.wgsl:35-50).
// The shader compares e with the left child, then the smaller of the two with the right child: it moves to the
// smaller child (the left one on a tie) if that child is below e, and stops otherwise. Which child is the smaller
// one does not depend on e, so the walk is written that way round: the chain from one level to the next is
// load, compare the children, select, and the comparison with e only decides where the walk ends (half the
// dependent instructions per level of the shader's order; the same moves, hence the same array).
// Returns the value left at the root.
template <uint32_t TK_LISTS>
__device__ __forceinline__ float tk_sift_hole(TkEntry* heap, uint32_t j, uint32_t limit, TkEntry e) {
  uint32_t i = 0;
  float root = e.v;
  for (;;) {
    const uint32_t l = 2 * i + 1, r = l + 1;
    if (l >= limit) break;
    const TkEntry cl = heap[l * TK_LISTS + j];
    const TkEntry cr = heap[(r < limit ? r : l) * TK_LISTS + j];
    const bool right = r < limit && cr.v < cl.v;
    const TkEntry m = right ? cr : cl;
    if (!(m.v < e.v)) break;
    heap[i * TK_LISTS + j] = m;
    if (i == 0) root = m.v;
    i = right ? r : l;
  }
  heap[i * TK_LISTS + j] = e;
  return root;
}
// The same walk on a FULL heap of TK_K = 32 entries (every insertion of the scan): the levels are unrolled, no
// slot has to be checked against a limit above the last level (only slot 15 has a child there, slot 31), and
// the four grandchildren of a node (slots 4 i + 3 .. 4 i + 6) are requested before its children are compared:
// a level of the walk is then compare, select, compare instead of address, load, compare, select, compare.
template <uint32_t TK_LISTS>
__device__ __forceinline__ float tk_sift_full(TkEntry* heap, uint32_t j, TkEntry e) {
  static_assert(TK_K == 32, "levels and slots below are those of a heap of 32");
  TkEntry* E = heap + j;
  uint32_t i = 0;
  float root = e.v;
  TkEntry cl = E[1 * TK_LISTS], cr = E[2 * TK_LISTS];
#pragma unroll
  for (uint32_t lvl = 0; lvl < 4; lvl++) {
    TkEntry g0 = {}, g1 = {}, g2 = {}, g3 = {};
    if (lvl < 3) {
      const TkEntry* G = E + (4 * i + 3) * TK_LISTS;
      g0 = G[0];
      g1 = G[TK_LISTS];
      g2 = G[2 * TK_LISTS];
      g3 = G[3 * TK_LISTS];
    }
    const bool right = cr.v < cl.v;
    const TkEntry m = right ? cr : cl;
    if (!(m.v < e.v)) {
      E[i * TK_LISTS] = e;
      return root;
    }
    E[i * TK_LISTS] = m;
    if (lvl == 0) root = m.v;
    i = 2 * i + 1 + (right ? 1u : 0u);
    if (lvl < 3) {
      cl = right ? g2 : g0;
      cr = right ? g3 : g1;
    }
  }
  if (i == 15) {  // the one slot of the fourth level with a child
    const TkEntry c = E[31 * TK_LISTS];
    if (c.v < e.v) {
      E[15 * TK_LISTS] = c;
      i = 31;
    }
  }
  E[i * TK_LISTS] = e;
  return root;
}
__device__ __forceinline__ void tk_merge_sync() { asm volatile("bar.sync 1, %0;" ::"n"(TK_WG) : "memory"); }  // the merging threads only
// One cluster of TK_CTAS CTAs. The 256 lists of the shader are independent until its merge rounds, and what
// a list costs is a chain of about 130 dependent sifts (375 us per call at 151936 logits with 32 lists per
// warp held in step, 176 us with the marks below, on ONE SM): so the lists are spread over the cluster, four
// to a warp, each CTA hands its sorted lists to the first CTA's shared memory, and that CTA runs the merge
// rounds on the shader's 256 invocations.
template <uint32_t TK_CTAS>
__global__ void __launch_bounds__(TK_THREADS) topk_kernel(const __half* logits, uint32_t n, uint32_t k, float* out_val, uint32_t* out_idx) {
  constexpr uint32_t TK_LISTS = TK_WG / TK_CTAS;              // lists per CTA
  constexpr uint32_t TK_LPW = TK_LISTS / (TK_THREADS / 32);   // lists per warp (one lane each; the other lanes load and copy)
  static_assert(TK_LPW >= 1 && TK_LPW * (TK_THREADS / 32) == TK_LISTS, "every list has a lane");
  extern __shared__ __align__(16) uint8_t tk_smem[];
  TkEntry* rows = reinterpret_cast<TkEntry*>(tk_smem);        // [TK_WG][TK_ROW], used in the first CTA only
  TkEntry* heap = rows + TK_WG * TK_ROW;                      // [TK_K][TK_LISTS]
  __half2* stage_all = reinterpret_cast<__half2*>(heap + TK_K * TK_LISTS);
  cg::cluster_group cluster = cg::this_cluster();
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool owner = lane < TK_LPW;                           // this lane scans a list
  const uint32_t jl = warp * TK_LPW + (owner ? lane : 0);     // the list's slot in this CTA
  const uint32_t j0 = cluster.block_rank() * TK_LISTS + warp * TK_LPW;  // the warp's first list
  const uint32_t j = j0 + (owner ? lane : 0);                 // the shader's invocation index of the list
  __half2* stage = stage_all + warp * (TK_CHUNK * TK_LPW);    // [TK_CHUNK][TK_LPW], this warp's
  if (owner)
    for (uint32_t i = 0; i < TK_K; i++) heap[i * TK_LISTS + jl] = TkEntry{-1e30f, 0u};
  const uint32_t n_words = (n + 1) >> 1;
  float cur_min = -1e30f;  // mirrors the root of this lane's heap
  // lane c fetches word c of the chunk for each of the warp's lists (adjacent words)
  __half2 nxt[TK_LPW];
  auto fetch = [&](uint32_t w_base) {
#pragma unroll
    for (uint32_t jj = 0; jj < TK_LPW; jj++) {
      const uint32_t w = w_base + lane * TK_WG + j0 + jj;
      nxt[jj] = w < n_words ? __ldg(reinterpret_cast<const __half2*>(logits + 2 * w)) : __half2();
    }
  };
  fetch(0);
  for (uint32_t w_base = 0; w_base < n_words; w_base += TK_CHUNK * TK_WG) {
    __syncwarp();  // the previous chunk has been consumed
#pragma unroll
    for (uint32_t jj = 0; jj < TK_LPW; jj++) stage[lane * TK_LPW + jj] = nxt[jj];
    if (w_base + TK_CHUNK * TK_WG < n_words) fetch(w_base + TK_CHUNK * TK_WG);  // in flight under this chunk's sifts
    __syncwarp();
    // this lane's elements of the chunk, in the shader's order: word c (low half, then high half) = bit 2 c, 2 c + 1
    const uint32_t words_here = owner && w_base + j < n_words ? min(TK_CHUNK, (n_words - w_base - j + TK_WG - 1) / TK_WG) : 0;
    unsigned long long marks = 0;
    if (owner) {
#pragma unroll
      for (uint32_t c = 0; c < TK_CHUNK; c++) {
        const __half2 pair = stage[c * TK_LPW + lane];
        const uint32_t i0 = 2 * (w_base + c * TK_WG + j);
        const bool m0 = c < words_here && __low2float(pair) > cur_min;
        const bool m1 = c < words_here && i0 + 1 < n && __high2float(pair) > cur_min;
        marks |= (static_cast<unsigned long long>(m0) << (2 * c)) | (static_cast<unsigned long long>(m1) << (2 * c + 1));
      }
    }
    // Only the elements above the heap's root at the start of the chunk can enter (the root only rises): every
    // lane skips to its next mark that still beats its root, and the lanes that have one sift together.
    for (;;) {
      float v = 0.f;
      uint32_t idx = 0;
      bool have = false;
      while (marks != 0) {
        const uint32_t pos = __ffsll(static_cast<long long>(marks)) - 1;
        marks &= marks - 1;
        const __half2 pair = stage[(pos >> 1) * TK_LPW + lane];
        v = (pos & 1) ? __high2float(pair) : __low2float(pair);
        idx = 2 * (w_base + (pos >> 1) * TK_WG + j) + (pos & 1);
        if (v > cur_min) {
          have = true;
          break;
        }
      }
      if (!__any_sync(FULL, have)) break;
      if (have) {
        cur_min = tk_sift_full<TK_LISTS>(heap, jl, TkEntry{v, idx});
      }
    }
  }
  // heapsort to descending order (topk_reduce.wgsl:106-126): swap the root with the last active slot, sift
  if (owner) {
    for (uint32_t active = TK_K - 1; active > 0; active--) {
      const TkEntry root = heap[jl], last = heap[active * TK_LISTS + jl];
      heap[active * TK_LISTS + jl] = root;
      tk_sift_hole<TK_LISTS>(heap, jl, active, last);
    }
  }
  __syncwarp();
  {  // every list to a row of its own in the first CTA: rows[j * TK_ROW + i]; lane i carries entry i
    TkEntry* rows0 = cluster.map_shared_rank(rows, 0);
#pragma unroll
    for (uint32_t jj = 0; jj < TK_LPW; jj++) rows0[(j0 + jj) * TK_ROW + lane] = heap[lane * TK_LISTS + warp * TK_LPW + jj];
  }
  cluster.sync();  // the rows are in the first CTA's shared memory; the other CTAs are done
  if (cluster.block_rank() != 0 || tid >= TK_WG) return;
  for (uint32_t s = TK_WG / 2; s > 0; s >>= 1) {
    for (uint32_t kk = tid; kk < s * TK_K; kk += TK_WG) {
      const uint32_t pair = kk / TK_K, i = kk % TK_K, bi = TK_K - 1 - i;
      const TkEntry a = rows[pair * TK_ROW + i], b = rows[(pair + s) * TK_ROW + bi];
      if (b.v > a.v) rows[pair * TK_ROW + i] = b;
    }
    tk_merge_sync();
    for (uint32_t stride = TK_K / 2; stride > 0; stride >>= 1) {
      for (uint32_t kk = tid; kk < s * (TK_K / 2); kk += TK_WG) {
        const uint32_t pair = kk / (TK_K / 2), local = kk % (TK_K / 2);
        const uint32_t lo = ((local & ~(stride - 1)) << 1) | (local & (stride - 1)), hi = lo | stride;
        const TkEntry a = rows[pair * TK_ROW + lo], b = rows[pair * TK_ROW + hi];
        if (b.v > a.v) {
          rows[pair * TK_ROW + lo] = b;
          rows[pair * TK_ROW + hi] = a;
        }
      }
      tk_merge_sync();
    }
  }
  const uint32_t kk = k < TK_K ? k : TK_K;
  if (tid < kk) {
    out_val[tid] = rows[tid].v;
    out_idx[tid] = rows[tid].i;
  }
}

// Sign bits of one Q1_0 tensor -> the matvec kernels' layout (see the file header). Thread = block.
__global__ void __launch_bounds__(256) relayout_kernel(const uint8_t* qs, uint4* out, uint64_t n_blocks) {
  const uint64_t blk = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (blk >= n_blocks) return;
  const uint4 src = *reinterpret_cast<const uint4*>(qs + blk * 16u);
  const uint32_t sw[4] = {src.x, src.y, src.z, src.w};
  uint32_t o[4] = {0, 0, 0, 0};
  for (uint32_t g = 0; g < 32; g++) {
    const uint32_t nib = (~(sw[g >> 3] >> (4 * (g & 7)))) & 0xFu;  // flip bits of elements 4 g .. 4 g + 3
    const uint32_t sh = 15 - (g & 15), hi = g >> 4;
    o[hi] |= ((nib & 1u) << sh) | (((nib >> 1) & 1u) << (sh + 16));
    o[2 + hi] |= (((nib >> 2) & 1u) << sh) | (((nib >> 3) & 1u) << (sh + 16));
  }
  out[blk] = make_uint4(o[0], o[1], o[2], o[3]);
}

size_t mv_smem_bytes(uint32_t k) { return static_cast<size_t>(k / 128u) * XB_STRIDE * sizeof(__half); }

template <int MODE, uint32_t R, uint32_t KB = 0>
cudaError_t launch_mv_r(bool pdl, cudaStream_t s, const MvParams& p) {
  const size_t smem = mv_smem_bytes(p.k);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(matvec_q1_kernel<MODE, R, KB>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    configured = smem;
  }
  const uint32_t rows_per_cta = (MV_THREADS / 8) * R;
  const uint32_t ctas = (p.n_total + rows_per_cta - 1) / rows_per_cta;
  return bp_launch(pdl, matvec_q1_kernel<MODE, R, KB>, dim3(ctas), dim3(MV_THREADS), smem, s, p);
}

uint32_t g_mv_rows_override = 0;  // tuning aid (bp_op_set_matvec_rows): 0 = by tensor height
bool g_mv_const_k = true;         // tuning aid: use the constant-block-count instances where one exists

template <int MODE>
cudaError_t launch_mv(bool pdl, cudaStream_t s, const MvParams& p) {
  uint32_t r = g_mv_rows_override;
  // measured at Bonsai-8B shapes (us per call, R = 1 / 2 / 4): 4096 rows 4.9 / 5.9 / 9.2, 6144 rows 5.8 / 6.9 / 7.6,
  // 24576 rows 12.9 / 10.6 / 10.9, 151936 rows 50 / 45 / 54
  if (r == 0) r = p.n_total >= 16384 ? 2 : 1;
  if (r >= 4) return launch_mv_r<MODE, 4>(pdl, s, p);
  // the instances with a constant block count: the tensors of a one-token step at the 8B shape
  // (measured: the two-rows-per-lane instances gain, LM head 47 -> 43 us; the one-row ones do not: Wo 3.7 -> 4.4 us)
  if (g_mv_const_k && (MODE == 0 || MODE == 1) && r == 2 && p.k == 4096) return launch_mv_r<MODE, 2, 4>(pdl, s, p);
  if (r == 2) return launch_mv_r<MODE, 2>(pdl, s, p);
  return launch_mv_r<MODE, 1>(pdl, s, p);
}

}  // namespace

void bp_q1_set_matvec_rows(uint32_t rows_per_lane) {
  g_mv_rows_override = rows_per_lane & 7u;
  g_mv_const_k = (rows_per_lane & 8u) == 0;  // + 8: the general instances only
}

cudaError_t bp_q1_relayout(cudaStream_t s, const uint8_t* qs, void* out, uint64_t n_blocks) {
  relayout_kernel<<<static_cast<unsigned>((n_blocks + 255) / 256), 256, 0, s>>>(qs, static_cast<uint4*>(out), n_blocks);
  return cudaGetLastError();
}

cudaError_t bp_q1_matvec(bool pdl, cudaStream_t s, const bp_q1_tensor& w, const __half* x, __half* y, bool accumulate) {
  MvParams p = {};
  p.r[0] = {w.d, static_cast<const uint4*>(w.bits), y, w.n};
  p.n_ranges = 1;
  p.n_total = w.n;
  p.k = w.k;
  p.x = x;
  p.accumulate = accumulate ? 1u : 0u;
  if (reinterpret_cast<uintptr_t>(x) % 16u != 0) return cudaErrorMisalignedAddress;  // the activations are staged 16 bytes at a time
  return launch_mv<0>(pdl, s, p);
}

cudaError_t bp_q1_matvec_normed(bool pdl, cudaStream_t s, const bp_q1_tensor* w, __half* const* out, uint32_t n_ranges,
                                const __half* x, const __half* w_norm, float eps) {
  if (n_ranges == 0 || n_ranges > 3) return cudaErrorInvalidValue;
  MvParams p = {};
  p.n_ranges = n_ranges;
  for (uint32_t r = 0; r < n_ranges; r++) {
    if (w[r].k != w[0].k || w[r].n % 16u != 0) return cudaErrorInvalidValue;  // the shader's range rule (ROWS_PER_WG = 16)
    p.r[r] = {w[r].d, static_cast<const uint4*>(w[r].bits), out[r], w[r].n};
    p.n_total += w[r].n;
  }
  p.k = w[0].k;
  p.x = x;
  p.aux = w_norm;
  p.eps = eps;
  return launch_mv<1>(pdl, s, p);
}

// out[i] = silu(f16(W_gate rms_norm(x))_i) * f16(W_up rms_norm(x))_i: matvec_q1_0_fused_normed over (gate, up)
// followed by silu_mul, in one launch.
cudaError_t bp_q1_matvec_normed_silu(bool pdl, cudaStream_t s, const bp_q1_tensor& w_gate, const bp_q1_tensor& w_up, __half* out,
                                     const __half* x, const __half* w_norm, float eps) {
  if (w_gate.k != w_up.k || w_gate.n != w_up.n) return cudaErrorInvalidValue;
  MvParams p = {};
  p.n_ranges = 2;
  p.r[0] = {w_gate.d, static_cast<const uint4*>(w_gate.bits), out, w_gate.n};
  p.r[1] = {w_up.d, static_cast<const uint4*>(w_up.bits), out, w_up.n};
  p.n_total = w_gate.n;
  p.k = w_gate.k;
  p.x = x;
  p.aux = w_norm;
  p.eps = eps;
  const size_t smem = mv_smem_bytes(p.k);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(matvec_q1_kernel<3, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    configured = smem;
  }
  const uint32_t rows_per_cta = MV_THREADS / 8;
  const dim3 grid((p.n_total + rows_per_cta - 1) / rows_per_cta);
  if (g_mv_const_k && p.k == 4096) return bp_launch(pdl, matvec_q1_kernel<3, 2, 4>, grid, dim3(MV_THREADS), smem, s, p);
  return bp_launch(pdl, matvec_q1_kernel<3, 2>, grid, dim3(MV_THREADS), smem, s, p);
}

cudaError_t bp_q1_matvec_silu(bool pdl, cudaStream_t s, const bp_q1_tensor& w, const __half* gate, const __half* up, __half* y,
                              bool accumulate) {
  MvParams p = {};
  p.r[0] = {w.d, static_cast<const uint4*>(w.bits), y, w.n};
  p.n_ranges = 1;
  p.n_total = w.n;
  p.k = w.k;
  p.x = gate;
  p.aux = up;
  p.accumulate = accumulate ? 1u : 0u;
  return launch_mv<2>(pdl, s, p);
}

cudaError_t bp_q1_rms_norm(bool pdl, cudaStream_t s, const __half* in, __half* out, const __half* w, uint32_t group_size,
                           uint32_t n_groups, float eps) {
  return bp_launch(pdl, rms_norm_kernel, dim3(n_groups), dim3(512), 0, s, in, out, w, group_size, eps);
}

cudaError_t bp_q1_silu_mul(bool pdl, cudaStream_t s, const __half* gate, const __half* up, __half* out, uint64_t n) {
  const bool vec8 = n % 8u == 0 && (reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(out)) % 16u == 0;
  if (vec8) return bp_launch(pdl, silu_mul_kernel<true>, dim3(static_cast<unsigned>((n / 8u + 255) / 256)), dim3(256), 0, s, gate, up, out, n);
  return bp_launch(pdl, silu_mul_kernel<false>, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s, gate, up, out, n);
}

cudaError_t bp_q1_embed(bool pdl, cudaStream_t s, const bp_q1_tensor& w, const uint32_t* tokens, uint32_t m, __half* x) {
  const uint64_t units = static_cast<uint64_t>(m) * (w.k / 8u);
  return bp_launch(pdl, embed_kernel, dim3(static_cast<unsigned>((units + 255) / 256)), dim3(256), 0, s, w.d, w.qs, w.k, tokens, m, x);
}

cudaError_t bp_q1_quantize_q8(bool pdl, cudaStream_t s, const __half* x, uint32_t k, uint32_t m, float* d_out, int8_t* qs_out) {
  const uint64_t n_blocks = static_cast<uint64_t>(m) * (k / 32u);
  if (reinterpret_cast<uintptr_t>(x) % 16u != 0 || reinterpret_cast<uintptr_t>(qs_out) % 16u != 0) return cudaErrorMisalignedAddress;
  return bp_launch(pdl, quantize_q8_kernel, dim3(static_cast<unsigned>((n_blocks + 255) / 256)), dim3(256), 0, s, x, n_blocks, d_out, qs_out);
}

static uint32_t g_matmul_variant = 0;  // 0 = by batch size; 1 dp4a, 2 mma.sync, 3 tcgen05; 4 / 5 = mma.sync with 64- / 128-token tiles only

static cudaError_t launch_mma(bool pdl, cudaStream_t s, const bp_q1_tensor* w, __half* const* y, uint32_t n_w, uint32_t m, const float* a_d,
                              const int8_t* a_qs, uint32_t acc) {
  MmaTensors t;
  uint32_t tiles = 0;
  for (uint32_t i = 0; i < 3; i++) {
    const uint32_t j = i < n_w ? i : n_w - 1;  // unused entries repeat the last tensor; their tile range is empty
    t.w_d[i] = w[j].d;
    t.w_qs[i] = w[j].qs;
    t.y[i] = y[j];
    t.n[i] = w[j].n;
    if (i < n_w) tiles += (w[i].n + MT - 1) / MT;
    t.tile_end[i] = tiles;
  }
  // Tiles of 128 tokens, of 64 tokens (0.62 of the time of a full one, measured: the weight tile is staged all
  // the same), or full tiles for as many whole waves of one CTA per SM as there are and half tiles for the rest
  // in a second launch (gate + up at 512 tokens: 768 full tiles are 5.2 waves; 740 full tiles and 56 half tiles
  // are 5 waves and a short one): whichever needs the least time.
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 1;
  }
  const uint32_t n_sm = static_cast<uint32_t>(sms), m_full = (m + 127) / 128, m_half = (m + 63) / 64;
  auto waves = [&](uint32_t ctas) { return static_cast<float>((ctas + n_sm - 1) / n_sm); };
  constexpr float HALF_COST = 0.62f;
  const float t_full = waves(tiles * m_full), t_half = HALF_COST * waves(tiles * m_half);
  const uint32_t n_a = (tiles * m_full / n_sm) * n_sm / m_full;  // column tiles that make whole waves of full tiles
  const float t_mixed = n_a == 0 || n_a == tiles ? 1e30f : waves(n_a * m_full) + HALF_COST * waves((tiles - n_a) * m_half) + 0.03f;
  auto launch = [&](bool half_tiles, uint32_t t0, uint32_t t1, bool dep) {
    t.tile0 = t0;
    if (half_tiles) return bp_launch(dep, matmul_q1_q8_mma_kernel<1>, dim3(t1 - t0, m_half), dim3(MMA_THREADS), MMA_SMEM, s, t, w[0].k, m, a_d, a_qs, acc);
    return bp_launch(dep, matmul_q1_q8_mma_kernel<2>, dim3(t1 - t0, m_full), dim3(MMA_THREADS), MMA_SMEM, s, t, w[0].k, m, a_d, a_qs, acc);
  };
  if (g_matmul_variant == 4) return launch(true, 0, tiles, pdl);
  if (g_matmul_variant == 5) return launch(false, 0, tiles, pdl);
  if (t_mixed < t_full && t_mixed < t_half) {
    cudaError_t e = launch(false, 0, n_a, pdl);
    if (e != cudaSuccess) return e;
    return launch(true, n_a, tiles, pdl);  // other outputs, the same inputs: it only has to follow in the stream
  }
  return t_half < t_full ? launch(true, 0, tiles, pdl) : launch(false, 0, tiles, pdl);
}

void bp_q1_set_matmul_variant(uint32_t v) { g_matmul_variant = v <= 5 ? v : 0; }

cudaError_t bp_q1_take_error(uint32_t* code) {
  cudaError_t e = cudaMemcpyFromSymbol(code, g_q1_err, sizeof(uint32_t));
  if (e != cudaSuccess || *code == 0) return e;
  const uint32_t zero = 0;
  return cudaMemcpyToSymbol(g_q1_err, &zero, sizeof zero);
}

// Batches of up to MMA_MIN_M tokens: CUDA cores (64 x 64 tiles fit them better than a 128-row MMA tile);
// larger ones: the mma.sync kernel, which measured faster than the tcgen05 one (254 against 323 us for
// 512 tokens x 4096 rows x 12288 inputs: both are bound by instruction issue, and what the tcgen05 kernel
// saves on the arithmetic, 3 instead of 5 instructions per output and sub-block, it spends on staging f16
// operands and on its barriers). Variant 1, 2, 3 forces dp4a, mma.sync, tcgen05 (tuning and tests: all
// three give the same bits).
cudaError_t bp_q1_matmul(bool pdl, cudaStream_t s, const bp_q1_tensor& w, uint32_t m, const float* a_d, const int8_t* a_qs, __half* y,
                         bool accumulate, uint32_t* err, uint32_t wait_limit) {
  const uint32_t variant = g_matmul_variant >= 4 ? 2u : g_matmul_variant != 0 ? g_matmul_variant : (m > MMA_MIN_M ? 2u : 1u);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(matmul_q1_q8_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(MMA_SMEM));
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(matmul_q1_q8_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(MMA_SMEM));
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(matmul_q1_q8_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(UM_SMEM));
    if (e != cudaSuccess) return e;
    configured = true;
  }
  if (m == 0) return cudaSuccess;
  const uint32_t acc = accumulate ? 1u : 0u;
  if (variant == 3) {
    dim3 grid((w.n + MT - 1) / MT, (m + MT - 1) / MT);
    return bp_launch(pdl, matmul_q1_q8_umma_kernel, grid, dim3(UM_THREADS), UM_SMEM, s, w.d, w.qs, w.k, w.n, m, a_d, a_qs, y, acc, err,
                     wait_limit != 0 ? wait_limit : (1u << 22));
  }
  if (variant == 2) {
    const bp_q1_tensor* one = &w;
    __half* out = y;
    return launch_mma(pdl, s, one, &out, 1, m, a_d, a_qs, acc);
  }
  dim3 grid((w.n + MM_T - 1) / MM_T, (m + MM_T - 1) / MM_T);
  return bp_launch(pdl, matmul_q1_q8_kernel, grid, dim3(256), 0, s, w.d, w.qs, w.k, w.n, m, a_d, a_qs, y, acc);
}

// The same activations through up to three weight tensors of equal k: one launch where the kernel allows.
cudaError_t bp_q1_matmul_multi(bool pdl, cudaStream_t s, const bp_q1_tensor* w, __half* const* y, uint32_t n_w, uint32_t m, const float* a_d,
                               const int8_t* a_qs, bool accumulate, uint32_t* err, uint32_t wait_limit) {
  const uint32_t variant = g_matmul_variant >= 4 ? 2u : g_matmul_variant != 0 ? g_matmul_variant : (m > MMA_MIN_M ? 2u : 1u);
  bool same_k = n_w >= 1 && n_w <= 3;
  for (uint32_t i = 1; i < n_w && same_k; i++) same_k = w[i].k == w[0].k;
  if (variant == 2 && same_k && n_w > 1) {
    cudaError_t e = bp_q1_matmul(pdl, s, w[0], 0, a_d, a_qs, y[0], accumulate, err, wait_limit);  // (m = 0: configures the kernels only)
    if (e != cudaSuccess) return e;
    return launch_mma(pdl, s, w, y, n_w, m, a_d, a_qs, accumulate ? 1u : 0u);
  }
  for (uint32_t i = 0; i < n_w; i++) {
    cudaError_t e = bp_q1_matmul(pdl, s, w[i], m, a_d, a_qs, y[i], accumulate, err, wait_limit);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

template <uint32_t CTAS>
static cudaError_t topk_launch(bool pdl, cudaStream_t s, const __half* logits, uint32_t n, uint32_t k, float* out_val, uint32_t* out_idx) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(CTAS);
  cfg.blockDim = dim3(TK_THREADS);
  cfg.dynamicSmemBytes = tk_smem_bytes(CTAS);
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, topk_kernel<CTAS>, logits, n, k, out_val, out_idx);
}

cudaError_t bp_q1_topk(bool pdl, cudaStream_t s, const __half* logits, uint32_t n, uint32_t k, float* out_val, uint32_t* out_idx) {
  // Per device, once: 16 CTAs per cluster (beyond the portable 8) if the device can hold such a cluster.
  static int ctas_of_device[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (ctas_of_device[dev] == 0) {
    e = cudaFuncSetAttribute(topk_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(tk_smem_bytes(8)));
    if (e != cudaSuccess) return e;
    int chosen = 8;
    if (cudaFuncSetAttribute(topk_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(tk_smem_bytes(16))) == cudaSuccess &&
        cudaFuncSetAttribute(topk_kernel<16>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(16);
      cfg.blockDim = dim3(TK_THREADS);
      cfg.dynamicSmemBytes = tk_smem_bytes(16);
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 16;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, topk_kernel<16>, &cfg) == cudaSuccess && clusters >= 1) chosen = 16;
    }
    (void)cudaGetLastError();  // a device without clusters of 16 is not an error of this call
    ctas_of_device[dev] = chosen;
  }
  return ctas_of_device[dev] == 16 ? topk_launch<16>(pdl, s, logits, n, k, out_val, out_idx) : topk_launch<8>(pdl, s, logits, n, k, out_val, out_idx);
}
