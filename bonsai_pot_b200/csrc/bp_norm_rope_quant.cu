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
#include "bp_norm_quant.cuh"

namespace {

using bp::Rot4;
using bp::norm_rope_rows;
using bp::quant4;

// R consecutive KV heads of one token per warp.
template <int R>
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
  const uint32_t per_tok = n_kv_head / R;
  if (unit >= m * per_tok) return;  // whole warp leaves together
  const uint32_t tok = unit / per_tok, head0 = (unit % per_tok) * R;
  const uint32_t kv_dim = n_kv_head * BP_HEAD_DIM, nb = kv_dim / BP_QK8;
  const uint32_t pos = pos_base + tok;
  const size_t src = static_cast<size_t>(tok) * kv_dim + head0 * BP_HEAD_DIM;

  Rot4 kp[R];
  norm_rope_rows<R>(k_cur + src, BP_HEAD_DIM, w_k_norm, rope + static_cast<size_t>(pos) * BP_HEAD_DIM, eps, lane, kp);
  float dk[R], dv[R];
  uint32_t pk[R], pv[R];
#pragma unroll
  for (int r = 0; r < R; r++) {
    const uint2 vr = *reinterpret_cast<const uint2*>(v_cur + src + r * BP_HEAD_DIM + 4 * lane);
    const __half2* vh = reinterpret_cast<const __half2*>(&vr);
    const float2 v01 = __half22float2(vh[0]), v23 = __half22float2(vh[1]);
    const float vraw[4] = {v01.x, v01.y, v23.x, v23.y};
    pk[r] = quant4(kp[r].v, &dk[r]);
    pv[r] = quant4(vraw, &dv[r]);
  }
#pragma unroll
  for (int r = 0; r < R; r++) {
    const size_t word = (static_cast<size_t>(pos) * kv_dim + (head0 + r) * BP_HEAD_DIM) / 4 + lane;
    k_qs[word] = pk[r];
    v_qs[word] = pv[r];
    if ((lane & 7) == 0) {
      const size_t blk = static_cast<size_t>(pos) * nb + (head0 + r) * 4 + (lane >> 3);
      k_d[blk] = dk[r];
      v_d[blk] = dv[r];
    }
  }
}

// R consecutive query heads of one token per warp (rows of q are dense: [m][n_head][128]).
template <int R>
__global__ void __launch_bounds__(256)
q_norm_rope_kernel(__half* __restrict__ q, const __half* __restrict__ w_q_norm,
                   const __half* __restrict__ rope, uint32_t n_head, uint32_t pos_base, uint32_t m,
                   uint32_t pos_step, float eps) {
  bp::pdl_launch_dependents();
  bp::pdl_wait();  // q comes from the previous kernel
  const int lane = threadIdx.x & 31;
  const uint32_t unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint32_t per_tok = n_head / R;
  if (unit >= m * per_tok) return;
  const uint32_t tok = (unit / per_tok) * pos_step;  // pos_step 0: every row is at pos_base
  __half* row = q + static_cast<size_t>(unit) * R * BP_HEAD_DIM;
  Rot4 qp[R];
  norm_rope_rows<R>(row, BP_HEAD_DIM, w_q_norm, rope + static_cast<size_t>(pos_base + tok) * BP_HEAD_DIM, eps, lane, qp);
#pragma unroll
  for (int r = 0; r < R; r++) {
    uint2 o;
    __half2 lo = __floats2half2_rn(qp[r].v[0], qp[r].v[1]);
    __half2 hi = __floats2half2_rn(qp[r].v[2], qp[r].v[3]);
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(row + r * BP_HEAD_DIM + 4 * lane) = o;
  }
}

template <int R>
cudaError_t launch_q(bp_attn_ctx* c, cudaStream_t s, __half* q, const __half* w, uint32_t pos, uint32_t rows, uint32_t pos_step) {
  const uint32_t units = rows * (c->cfg.n_head / R);
  return bp_launch(c->opt_pdl != 0, q_norm_rope_kernel<R>, dim3((units + 7) / 8), dim3(256), 0, s, q, w, c->rope, c->cfg.n_head,
                   pos, rows, pos_step, c->cfg.rms_eps);
}

}  // namespace

// Heads per warp: for a batch of rows as many (4, 2 or 1) as divide the head count: more rows per warp
// overlap the rows' dependency chains and share the weight / RoPE loads. A decode step has only a
// few rows and wants the shortest chain per warp instead.
cudaError_t bp_launch_q_norm_rope(bp_attn_ctx* c, cudaStream_t s, __half* q, const __half* w,
                                  uint32_t pos_base, uint32_t m, uint32_t* launches) {
  *launches += 1;
  const bool big = static_cast<uint64_t>(m) * c->cfg.n_head >= 8192;  // a decode step's few rows want the shortest chain
  if (big && c->cfg.n_head % 4 == 0) return launch_q<4>(c, s, q, w, pos_base, m, 1u);
  if (big && c->cfg.n_head % 2 == 0) return launch_q<2>(c, s, q, w, pos_base, m, 1u);
  return launch_q<1>(c, s, q, w, pos_base, m, 1u);
}

cudaError_t bp_launch_q_norm_rope_rows(bp_attn_ctx* c, cudaStream_t s, __half* q, const __half* w,
                                       uint32_t pos, uint32_t rows, uint32_t* launches) {
  *launches += 1;
  const bool big = static_cast<uint64_t>(rows) * c->cfg.n_head >= 8192;
  if (big && c->cfg.n_head % 4 == 0) return launch_q<4>(c, s, q, w, pos, rows, 0u);
  if (big && c->cfg.n_head % 2 == 0) return launch_q<2>(c, s, q, w, pos, rows, 0u);
  return launch_q<1>(c, s, q, w, pos, rows, 0u);
}

template <int R>
static cudaError_t launch_kv(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* k, const __half* v, const __half* w,
                             uint32_t pos_base, uint32_t m) {
  const uint32_t units = m * (c->cfg.n_kv_head / R);
  float* k_d = reinterpret_cast<float*>(c->kv[0] + bp_d_off(c, layer));
  float* v_d = reinterpret_cast<float*>(c->kv[1] + bp_d_off(c, layer));
  uint32_t* k_qs = reinterpret_cast<uint32_t*>(c->kv[0] + bp_qs_off(c, layer));
  uint32_t* v_qs = reinterpret_cast<uint32_t*>(c->kv[1] + bp_qs_off(c, layer));
  return bp_launch(c->opt_pdl != 0, kv_writeback_kernel<R>, dim3((units + 7) / 8), dim3(256), 0, s, k, v, w, c->rope, k_d, k_qs, v_d,
                   v_qs, c->cfg.n_kv_head, pos_base, m, c->cfg.rms_eps);
}

cudaError_t bp_launch_kv_writeback(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* k,
                                   const __half* v, const __half* w, uint32_t pos_base, uint32_t m,
                                   uint32_t* launches) {
  *launches += 1;
  bp_note_row_write(c, layer, pos_base);
  if (static_cast<uint64_t>(m) * c->cfg.n_kv_head >= 4096 && c->cfg.n_kv_head % 2 == 0)
    return launch_kv<2>(c, s, layer, k, v, w, pos_base, m);
  return launch_kv<1>(c, s, layer, k, v, w, pos_base, m);
}
