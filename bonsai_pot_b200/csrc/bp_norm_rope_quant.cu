// K-side norm + RoPE + Q8_0 quantise + cache write, V-side quantise + write,
// and the Q-side norm + RoPE. Replaces kv_writeback_fused.wgsl and
// q_norm_rope_fused.wgsl of the reference.
//
// One warp owns one (token, head): lane l holds dims 4l..4l+3, so a Q8_0 block
// of 32 dims is 8 consecutive lanes and the NEOX partner (dim +-64) is lane
// l ^ 16. Both kernels move 16 bytes or less per lane and are bound by HBM.
//
// Results are bit-exact against the CPU oracle, which fixes what WGSL leaves
// to the driver: binary32, round to nearest even, no FMA contraction,
// correctly rounded 1/sqrt and division, ties-to-even round(), and the sum of
// 128 squares as an xor butterfly (offsets 16, 8, 4, 2, 1) inside each aligned
// group of 32 dims followed by (w0 + w1) + (w2 + w3). Every arithmetic step
// below therefore uses the explicitly rounded intrinsics, which the compiler
// never contracts, and reproduces that tree: the dim offsets 16, 8, 4 are lane
// offsets 4, 2, 1, and the dim offsets 2, 1 are the in-lane sum
// (s0 + s2) + (s1 + s3).
#include "bp_common.cuh"
#include "bp_ptx.cuh"

namespace {

constexpr unsigned FULL = 0xffffffffu;

struct Rot4 {
  float v[4];
};

// Steps shared by both kernels: f16 load, RMS-norm, weight, NEOX rotation.
// x: the head's 128 f16 values; w: norm weight [128]; rope_row: [64][2] f16.
__device__ __forceinline__ Rot4 norm_rope(const __half* x, const __half* w, const __half* rope_row,
                                          float eps, int lane) {
  const uint2 xr = *reinterpret_cast<const uint2*>(x + 4 * lane);
  const uint2 wr = *reinterpret_cast<const uint2*>(w + 4 * lane);
  const uint4 rr = *reinterpret_cast<const uint4*>(rope_row + 8 * (lane & 15));
  const __half2* xh = reinterpret_cast<const __half2*>(&xr);
  const __half2* wh = reinterpret_cast<const __half2*>(&wr);
  const __half2* rh = reinterpret_cast<const __half2*>(&rr);
  float raw[4], wt[4], sq[4];
  {
    float2 a = __half22float2(xh[0]), b = __half22float2(xh[1]);
    raw[0] = a.x; raw[1] = a.y; raw[2] = b.x; raw[3] = b.y;
    float2 c = __half22float2(wh[0]), d = __half22float2(wh[1]);
    wt[0] = c.x; wt[1] = c.y; wt[2] = d.x; wt[3] = d.y;
  }
#pragma unroll
  for (int c = 0; c < 4; c++) sq[c] = __fmul_rn(raw[c], raw[c]);
#pragma unroll
  for (int off = 4; off >= 1; off >>= 1) {
#pragma unroll
    for (int c = 0; c < 4; c++) sq[c] = __fadd_rn(sq[c], __shfl_xor_sync(FULL, sq[c], off));
  }
  float w32 = __fadd_rn(__fadd_rn(sq[0], sq[2]), __fadd_rn(sq[1], sq[3]));
  w32 = __fadd_rn(w32, __shfl_xor_sync(FULL, w32, 8));
  const float total = __fadd_rn(w32, __shfl_xor_sync(FULL, w32, 16));
  const float inv_h = __frsqrt_rn(__fadd_rn(__fdiv_rn(total, 128.0f), eps));

  Rot4 out;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const float xn = __fmul_rn(__fmul_rn(raw[c], inv_h), wt[c]);
    const float partner = __shfl_xor_sync(FULL, xn, 16);
    const float2 cs = __half22float2(rh[c]);  // (cos, sin) of j = dim mod 64
    if (lane < 16) {
      out.v[c] = __fsub_rn(__fmul_rn(xn, cs.x), __fmul_rn(partner, cs.y));
    } else {
      out.v[c] = __fadd_rn(__fmul_rn(partner, cs.y), __fmul_rn(xn, cs.x));
    }
  }
  return out;
}

// Block-32 absmax quantiser over 8 lanes x 4 values. Returns the packed int8
// word of this lane; *d_out is the block scale (same in all 8 lanes).
__device__ __forceinline__ uint32_t quant4(const float* x, float* d_out) {
  float a = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
  a = fmaxf(a, __shfl_xor_sync(FULL, a, 1));
  a = fmaxf(a, __shfl_xor_sync(FULL, a, 2));
  a = fmaxf(a, __shfl_xor_sync(FULL, a, 4));
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

__global__ void __launch_bounds__(256)
kv_writeback_kernel(const __half* __restrict__ k_cur, const __half* __restrict__ v_cur,
                    const __half* __restrict__ w_k_norm, const __half* __restrict__ rope,
                    float* __restrict__ k_d, uint32_t* __restrict__ k_qs, float* __restrict__ v_d,
                    uint32_t* __restrict__ v_qs, uint32_t n_kv_head, uint32_t pos_base, uint32_t m,
                    float eps) {
  bp::pdl_launch_dependents();
  bp::pdl_wait();  // k_cur / v_cur come from the previous kernel; the cache rows may still be read by it
  const int lane = threadIdx.x & 31;
  const uint32_t unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= m * n_kv_head) return;  // whole warp leaves together
  const uint32_t tok = unit / n_kv_head, head = unit % n_kv_head;
  const uint32_t kv_dim = n_kv_head * BP_HEAD_DIM, nb = kv_dim / BP_QK8;
  const uint32_t pos = pos_base + tok;
  const size_t src = static_cast<size_t>(tok) * kv_dim + head * BP_HEAD_DIM;

  const Rot4 kp = norm_rope(k_cur + src, w_k_norm, rope + static_cast<size_t>(pos) * BP_HEAD_DIM,
                            eps, lane);
  const uint2 vr = *reinterpret_cast<const uint2*>(v_cur + src + 4 * lane);
  const __half2* vh = reinterpret_cast<const __half2*>(&vr);
  const float2 v01 = __half22float2(vh[0]), v23 = __half22float2(vh[1]);
  const float vraw[4] = {v01.x, v01.y, v23.x, v23.y};

  float dk, dv;
  const uint32_t pk = quant4(kp.v, &dk);
  const uint32_t pv = quant4(vraw, &dv);

  const size_t word = (static_cast<size_t>(pos) * kv_dim + head * BP_HEAD_DIM) / 4 + lane;
  k_qs[word] = pk;
  v_qs[word] = pv;
  if ((lane & 7) == 0) {
    const size_t blk = static_cast<size_t>(pos) * nb + head * 4 + (lane >> 3);
    k_d[blk] = dk;
    v_d[blk] = dv;
  }
}

__global__ void __launch_bounds__(256)
q_norm_rope_kernel(__half* __restrict__ q, const __half* __restrict__ w_q_norm,
                   const __half* __restrict__ rope, uint32_t n_head, uint32_t pos_base, uint32_t m,
                   uint32_t pos_step, float eps) {
  bp::pdl_launch_dependents();
  bp::pdl_wait();  // q comes from the previous kernel
  const int lane = threadIdx.x & 31;
  const uint32_t unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= m * n_head) return;
  const uint32_t tok = (unit / n_head) * pos_step;  // pos_step 0: every row is at pos_base
  __half* row = q + static_cast<size_t>(unit) * BP_HEAD_DIM;  // [m][n_head][128] is dense
  const Rot4 qp =
      norm_rope(row, w_q_norm, rope + static_cast<size_t>(pos_base + tok) * BP_HEAD_DIM, eps, lane);
  uint2 o;
  __half2 lo = __floats2half2_rn(qp.v[0], qp.v[1]);
  __half2 hi = __floats2half2_rn(qp.v[2], qp.v[3]);
  o.x = *reinterpret_cast<uint32_t*>(&lo);
  o.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(row + 4 * lane) = o;
}

}  // namespace

cudaError_t bp_launch_q_norm_rope(bp_attn_ctx* c, cudaStream_t s, __half* q, const __half* w,
                                  uint32_t pos_base, uint32_t m, uint32_t* launches) {
  const uint32_t units = m * c->cfg.n_head;
  *launches += 1;
  return bp_launch(c->opt_pdl != 0, q_norm_rope_kernel, dim3((units + 7) / 8), dim3(256), 0, s, q, w, c->rope, c->cfg.n_head,
                   pos_base, m, 1u, c->cfg.rms_eps);
}

cudaError_t bp_launch_q_norm_rope_rows(bp_attn_ctx* c, cudaStream_t s, __half* q, const __half* w,
                                       uint32_t pos, uint32_t rows, uint32_t* launches) {
  const uint32_t units = rows * c->cfg.n_head;
  *launches += 1;
  return bp_launch(c->opt_pdl != 0, q_norm_rope_kernel, dim3((units + 7) / 8), dim3(256), 0, s, q, w, c->rope, c->cfg.n_head,
                   pos, rows, 0u, c->cfg.rms_eps);
}

cudaError_t bp_launch_kv_writeback(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* k,
                                   const __half* v, const __half* w, uint32_t pos_base, uint32_t m,
                                   uint32_t* launches) {
  const uint32_t units = m * c->cfg.n_kv_head;
  float* k_d = reinterpret_cast<float*>(c->kv[0] + bp_d_off(c, layer));
  float* v_d = reinterpret_cast<float*>(c->kv[1] + bp_d_off(c, layer));
  uint32_t* k_qs = reinterpret_cast<uint32_t*>(c->kv[0] + bp_qs_off(c, layer));
  uint32_t* v_qs = reinterpret_cast<uint32_t*>(c->kv[1] + bp_qs_off(c, layer));
  *launches += 1;
  return bp_launch(c->opt_pdl != 0, kv_writeback_kernel, dim3((units + 7) / 8), dim3(256), 0, s, k, v, w, c->rope, k_d, k_qs, v_d,
                   v_qs, c->cfg.n_kv_head, pos_base, m, c->cfg.rms_eps);
}
