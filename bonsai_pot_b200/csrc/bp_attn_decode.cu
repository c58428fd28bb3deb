// Single-token GQA decode attention over the Q8_0 KV cache: split-KV partial
// pass + log-sum-exp combine. Replaces attention_split.wgsl and
// attention_merge.wgsl of the reference (src/forward.rs:822-856).
//
// Production kernel (decode_mma_kernel), HBM-bound by design:
//   * One CTA owns a contiguous token range (a "split") for ALL KV heads of the
//     context, so the CTA streams whole cache rows: HBM sees long sequential
//     reads of the qs-section and of the d-section.
//   * A producer warp moves the rows into shared memory with tiled TMA loads
//     (128-byte swizzle, completion on mbarriers, a ring of stages); no load
//     uses cluster multicast.
//   * Each compute warp owns one KV head and a 16-token sub-tile per stage and
//     computes on the tensor cores with warp-level MMA: S = Q K^T with the
//     (<= 8) query heads of the group padded to M = 16, O^T = V^T P^T with the
//     head dims on M. int8 is expanded to f16 bit patterns with two logic ops
//     per pair (see k_pair / v_pairs); the Q8_0 block scales stay in f32 and
//     multiply the per-block accumulators (K) or fold into P (V).
//   * Softmax runs in the exp2 domain with the running max shared by the four
//     lanes of a quad (warp shuffles), rescaling O only when a max moves.
//   * Partials (o[128], m, l per head and split) go to the context's scratch and
//     a second small kernel combines them; with one split the kernel writes the
//     f16 output itself.
//
// A plain CUDA-core kernel (attn_scalar_kernel) is kept as an on-device
// cross-check (variant 1); it is also the first-generation prefill kernel.
#include "bp_common.cuh"
#include "bp_ptx.cuh"
#include "bp_q8.cuh"

namespace {

using namespace bp;

constexpr unsigned FULL = 0xffffffffu;
constexpr float NEG_BIG = -1e30f;  // the reference's initial running max

// ------------------------------------------------------------------------
// Cross-check kernel: one block per (split, query head, token); 4 warps take
// tokens round-robin, lane l holds dims 4l..4l+3. f32 throughout, dequantising
// as scale * f32(int8) like load_k / load_v (attention_split.wgsl:87-109).
// ------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
attn_scalar_kernel(const __half* __restrict__ q, const float* __restrict__ k_d,
                   const uint32_t* __restrict__ k_qs, const float* __restrict__ v_d,
                   const uint32_t* __restrict__ v_qs, float* __restrict__ partials,
                   __half* __restrict__ out, uint32_t n_head, uint32_t n_kv_head, uint32_t cur_pos,
                   uint32_t tps, uint32_t is_prefill, float scale) {
  const uint32_t split = blockIdx.x, h = blockIdx.y, tok = blockIdx.z;
  const uint32_t n_splits = gridDim.x;
  const uint32_t g = h / (n_head / n_kv_head);
  const uint32_t kv_dim = n_kv_head * BP_HEAD_DIM, nb = kv_dim / BP_QK8;
  const uint32_t n_keys = is_prefill ? tok + 1 : cur_pos;
  const uint32_t t0 = split * tps;
  const uint32_t t1 = min(t0 + tps, n_keys);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  const __half* qrow = q + (static_cast<size_t>(tok) * n_head + h) * BP_HEAD_DIM;
  float qf[4];
  {
    const uint2 qr = *reinterpret_cast<const uint2*>(qrow + 4 * lane);
    const __half2* qh = reinterpret_cast<const __half2*>(&qr);
    const float2 a = __half22float2(qh[0]), b = __half22float2(qh[1]);
    qf[0] = a.x; qf[1] = a.y; qf[2] = b.x; qf[3] = b.y;
  }
  float m_run = NEG_BIG, l_run = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
  for (uint32_t t = t0 + warp; t < t1; t += 4) {
    const size_t word = (static_cast<size_t>(t) * kv_dim + g * BP_HEAD_DIM) / 4 + lane;
    const size_t blk = static_cast<size_t>(t) * nb + g * 4 + (lane >> 3);
    const uint32_t kw = k_qs[word], vw = v_qs[word];
    const float ks = k_d[blk], vs = v_d[blk];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < 4; c++) {
      const float kf = ks * static_cast<float>(static_cast<int8_t>(kw >> (8 * c)));
      dot += kf * qf[c];
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) dot += __shfl_xor_sync(FULL, dot, off);
    const float s = dot * scale;
    const float m_new = fmaxf(m_run, s);
    const float corr = __expf(m_run - m_new), w = __expf(s - m_new);
    l_run = l_run * corr + w;
    m_run = m_new;
#pragma unroll
    for (int c = 0; c < 4; c++) {
      const float vf = vs * static_cast<float>(static_cast<int8_t>(vw >> (8 * c)));
      o[c] = o[c] * corr + w * vf;
    }
  }
  __shared__ float sm_o[4][BP_HEAD_DIM];
  __shared__ float sm_m[4], sm_l[4];
#pragma unroll
  for (int c = 0; c < 4; c++) sm_o[warp][4 * lane + c] = o[c];
  if (lane == 0) { sm_m[warp] = m_run; sm_l[warp] = l_run; }
  __syncthreads();
  const int d = threadIdx.x;
  const float m_all = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
  float oo = 0.f, ll = 0.f;
#pragma unroll
  for (int w = 0; w < 4; w++) {
    const float e = __expf(sm_m[w] - m_all);
    oo += sm_o[w][d] * e;
    ll += sm_l[w] * e;
  }
  if (n_splits == 1) {
    out[(static_cast<size_t>(tok) * n_head + h) * BP_HEAD_DIM + d] = __float2half_rn(oo * (1.0f / ll));
  } else {
    float* dst = partials + ((static_cast<size_t>(tok) * n_splits + split) * n_head + h) * BP_PART_STRIDE;
    dst[d] = oo;
    if (d == 0) { dst[128] = m_all * 1.4426950408889634f; dst[129] = ll; }  // m kept in log2 units
  }
}

// Log-sum-exp combine over splits (attention_merge.wgsl:70-130). One block per
// query head, 4 groups of 128 threads: group k takes splits k, k+4, ... so that
// many independent loads are in flight; thread d of a group owns output dim d.
// m is stored in log2 units. n_splits <= COMBINE_MAX_SPLITS.
constexpr uint32_t COMBINE_MAX_SPLITS = 256;
constexpr uint32_t COMBINE_GROUPS = 4;

__global__ void __launch_bounds__(128 * COMBINE_GROUPS)
attn_combine_kernel(const float* __restrict__ partials, __half* __restrict__ out, uint32_t n_head,
                    uint32_t n_splits) {
  pdl_launch_dependents();
  pdl_wait();  // the partials come from the kernel before this one
  __shared__ float w_sh[COMBINE_MAX_SPLITS];
  __shared__ float red[16];
  __shared__ float o_sh[COMBINE_GROUPS][BP_HEAD_DIM];
  const uint32_t h = blockIdx.x, tid = threadIdx.x, d = tid & 127, grp = tid >> 7;
  const int lane = tid & 31, warp = tid >> 5;
  const float* base = partials + static_cast<size_t>(h) * BP_PART_STRIDE;
  const size_t stride = static_cast<size_t>(n_head) * BP_PART_STRIDE;

  float m_s = NEG_BIG, l_s = 0.f;
  if (tid < n_splits) {
    m_s = base[tid * stride + 128];
    l_s = base[tid * stride + 129];
  }
  float m_all = m_s;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) m_all = fmaxf(m_all, __shfl_xor_sync(FULL, m_all, off));
  if (lane == 0) red[warp] = m_all;
  __syncthreads();
  m_all = red[0];
#pragma unroll
  for (int w = 1; w < 16; w++) m_all = fmaxf(m_all, red[w]);
  __syncthreads();
  const float wgt = ex2(m_s - m_all);
  if (tid < n_splits) w_sh[tid] = wgt;
  float l = l_s * wgt;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) l += __shfl_xor_sync(FULL, l, off);
  if (lane == 0) red[warp] = l;
  __syncthreads();
  l = 0.f;
#pragma unroll
  for (int w = 0; w < 16; w++) l += red[w];

  float o = 0.f;
#pragma unroll 8
  for (uint32_t s = grp; s < n_splits; s += COMBINE_GROUPS) o = fmaf(base[s * stride + d], w_sh[s], o);
  o_sh[grp][d] = o;
  __syncthreads();
  if (grp == 0) {
    o = (o_sh[0][d] + o_sh[1][d]) + (o_sh[2][d] + o_sh[3][d]);
    out[static_cast<size_t>(h) * BP_HEAD_DIM + d] = __float2half_rn(o * (1.0f / l));
  }
}

// ------------------------------------------------------------------------
// Production kernel.
// ------------------------------------------------------------------------
constexpr int MAX_STAGES = 5;
constexpr uint32_t SUBTILE = 16;  // tokens per warp per stage
constexpr uint32_t SMEM_LIMIT = 227 * 1024;

template <int NW_>
struct Geo {
  static constexpr uint32_t STAGE_QS = NW_ * SUBTILE * 128;  // bytes of K (or V) quants per stage
  static constexpr uint32_t STAGE_D = NW_ * SUBTILE * 16;    // bytes of K (or V) scales per stage
  static constexpr uint32_t STAGE_BYTES = 2 * STAGE_QS + 2 * STAGE_D;
  static constexpr uint32_t MERGE_BYTES = NW_ * 8 * BP_HEAD_DIM * 4 + NW_ * 8 * 8;
  static constexpr uint32_t max_stages() {
    uint32_t n = (SMEM_LIMIT - MERGE_BYTES - 1024) / STAGE_BYTES;
    return n > MAX_STAGES ? MAX_STAGES : n;
  }
};

struct DecodeParams {
  const __half* q;
  __half* out;
  float* partials;
  uint32_t* err;       // device word: set non-zero when a bounded wait gives up
  uint32_t row_base;   // layer * max_seq
  uint32_t cur_pos;
  uint32_t tps;        // tokens per split, a multiple of the stage size
  uint32_t n_stages;
  uint32_t n_head;     // query heads of the context
  uint32_t hpc;        // KV heads per CTA (blockIdx.y selects the group of heads)
  uint32_t qpg;
  uint32_t d_swz;      // 1 when the scale tiles are 128 B wide and swizzled
  float sm_scale_log2; // softmax scale * log2(e)
};

// Running state of one compute warp: softmax statistics of head `lane / 4`,
// and O^T accumulators (dims on rows, heads 2*quad, 2*quad+1 on columns).
struct WarpAcc {
  float m_run, l_run;
  float oacc[4][2][4];
  float pacc[4][4];  // DENORM only: sum of P' per block, from an all-ones A operand
};

// One 16-token sub-tile of one KV head. ktile/vtile: 16 x 128 B swizzled int8
// tiles; kd/vd: this warp's rows of the scale tiles. koff/voff/soff are
// per-lane byte offsets computed once per kernel (block b adds an xor of b<<5).
template <bool DENORM, bool TAIL>
__device__ __forceinline__ void process_tile(WarpAcc& w, uint32_t ktile, uint32_t vtile, uint32_t kd, uint32_t vd,
                                             const uint32_t (&koff)[2], const uint32_t (&voff)[4],
                                             const uint32_t (&soff)[4], const uint32_t (&qa0)[4][2],
                                             const uint32_t (&qa2)[4][2], const float (&qcorr)[4], float s_mul,
                                             uint32_t valid, int qd) {
  // ---- S = Q K^T, one accumulator per (token tile, Q8_0 block) ----
  float acc[2][4][4];
#pragma unroll
  for (int t = 0; t < 2; t++) {
#pragma unroll
    for (int b = 0; b < 4; b++) {
#pragma unroll
      for (int c = 0; c < 4; c++) acc[t][b][c] = 0.f;
      const uint2 kw = lds64(ktile + (koff[t] ^ (b << 5)));
      uint32_t b0, b1;
      k_pair<DENORM>(kw.x, b0, b1);
      mma_16816(acc[t][b], qa0[b][0], 0u, qa2[b][0], 0u, b0, b1);
      k_pair<DENORM>(kw.y, b0, b1);
      mma_16816(acc[t][b], qa0[b][1], 0u, qa2[b][1], 0u, b0, b1);
    }
  }
  // ---- scores of this lane: head lane/4, token slots j = 0..3 ----
  float sc[4];
  float4 sv[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const float4 sk = lds128f(kd + soff[j]);
    sv[j] = lds128f(vd + soff[j]);
    const int t = j & 1, c = j >> 1;
    float sj = sk.x * (acc[t][0][c] - qcorr[0]);
    sj = fmaf(sk.y, acc[t][1][c] - qcorr[1], sj);
    sj = fmaf(sk.z, acc[t][2][c] - qcorr[2], sj);
    sj = fmaf(sk.w, acc[t][3][c] - qcorr[3], sj);
    sc[j] = sj * s_mul;
    if (TAIL) {
      const uint32_t rowj = 4 * qd + (j ^ (qd & 2));
      if (rowj >= valid) {
        sc[j] = NEG_BIG;
        sv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  }
  float m_loc = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
  m_loc = fmaxf(m_loc, __shfl_xor_sync(FULL, m_loc, 1));
  m_loc = fmaxf(m_loc, __shfl_xor_sync(FULL, m_loc, 2));
  const float m_new = fmaxf(w.m_run, m_loc);
  const float corr = ex2(w.m_run - m_new);
  const bool moved = m_new > w.m_run;
  w.m_run = m_new;
  float pj[4];
#pragma unroll
  for (int j = 0; j < 4; j++) pj[j] = ex2(sc[j] - m_new);
  w.l_run = w.l_run * corr + ((pj[0] + pj[1]) + (pj[2] + pj[3]));

  if (__any_sync(FULL, moved)) {
    const float ca = __shfl_sync(FULL, corr, 8 * qd);
    const float cb = __shfl_sync(FULL, corr, 8 * qd + 4);
#pragma unroll
    for (int b = 0; b < 4; b++) {
#pragma unroll
      for (int t = 0; t < 2; t++) {
        w.oacc[b][t][0] *= ca; w.oacc[b][t][1] *= cb;
        w.oacc[b][t][2] *= ca; w.oacc[b][t][3] *= cb;
      }
      if (DENORM) {
        w.pacc[b][0] *= ca; w.pacc[b][1] *= cb;
        w.pacc[b][2] *= ca; w.pacc[b][3] *= cb;
      }
    }
  }

  // ---- O^T += V^T P'^T, P' = p * (V block scale), per Q8_0 block ----
#pragma unroll
  for (int b = 0; b < 4; b++) {
    const float sb0 = b == 0 ? sv[0].x : b == 1 ? sv[0].y : b == 2 ? sv[0].z : sv[0].w;
    const float sb1 = b == 0 ? sv[1].x : b == 1 ? sv[1].y : b == 2 ? sv[1].z : sv[1].w;
    const float sb2 = b == 0 ? sv[2].x : b == 1 ? sv[2].y : b == 2 ? sv[2].z : sv[2].w;
    const float sb3 = b == 0 ? sv[3].x : b == 1 ? sv[3].y : b == 2 ? sv[3].z : sv[3].w;
    __half2 h01 = __floats2half2_rn(pj[0] * sb0, pj[1] * sb1);
    __half2 h23 = __floats2half2_rn(pj[2] * sb2, pj[3] * sb3);
    const uint32_t pb0 = *reinterpret_cast<uint32_t*>(&h01);
    const uint32_t pb1 = *reinterpret_cast<uint32_t*>(&h23);
    // With an A operand of all ones (2^-24 each) the tensor core itself sums the
    // rounded P' of the 16 tokens: the +128 of the V bytes then cancels exactly.
    if (DENORM) mma_16816(w.pacc[b], 0x00010001u, 0x00010001u, 0x00010001u, 0x00010001u, pb0, pb1);

    uint32_t e[4], o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint32_t x = lds32(vtile + (voff[j] ^ (b << 5))) ^ 0x80808080u;
      e[j] = x & 0x00ff00ffu;
      o[j] = x & 0xff00ff00u;
      if (!DENORM) { e[j] |= 0x64006400u; o[j] |= 0x00640064u; }
    }
    // dims 32b + 4r + {0 (row r), 2 (row r+8)}
    mma_16816(w.oacc[b][0], v_fix<DENORM>(prmt(e[0], e[1], 0x5410)), v_fix<DENORM>(prmt(e[0], e[1], 0x7632)),
              v_fix<DENORM>(prmt(e[2], e[3], 0x5410)), v_fix<DENORM>(prmt(e[2], e[3], 0x7632)), pb0, pb1);
    // dims 32b + 4r + {1 (row r), 3 (row r+8)}
    mma_16816(w.oacc[b][1], v_fix<DENORM>(prmt(o[0], o[1], 0x4501)), v_fix<DENORM>(prmt(o[0], o[1], 0x6723)),
              v_fix<DENORM>(prmt(o[2], o[3], 0x4501)), v_fix<DENORM>(prmt(o[2], o[3], 0x6723)), pb0, pb1);
  }
}

template <int NW_, bool DENORM>
__global__ void __launch_bounds__((NW_ + 1) * 32, 1)
decode_mma_kernel(const __grid_constant__ CUtensorMap map_kq, const __grid_constant__ CUtensorMap map_kd,
                  const __grid_constant__ CUtensorMap map_vq, const __grid_constant__ CUtensorMap map_vd,
                  const DecodeParams p) {
  using G = Geo<NW_>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t hpc = p.hpc, wph = NW_ / hpc, st_tok = SUBTILE * wph;
  const uint32_t ns = p.n_stages;
  const uint32_t g0 = blockIdx.y * hpc;  // first KV head of this CTA

  const uint32_t split = blockIdx.x, n_splits = gridDim.x;
  const uint32_t tok_begin = split * p.tps;
  const uint32_t tok_end = min(tok_begin + p.tps, p.cur_pos);
  const uint32_t n_iter = (tok_end - tok_begin + st_tok - 1) / st_tok;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < ns; s++) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), NW_);
    }
    fence_barrier_init();
  }
  __syncthreads();

  if (warp == NW_) {
    // ---------------- producer ----------------
    if (lane == 0) {
      prefetch_tensormap(&map_kq);
      prefetch_tensormap(&map_vq);
      prefetch_tensormap(&map_kd);
      prefetch_tensormap(&map_vd);
      bool ok = true;
      for (uint32_t it = 0; it < n_iter && ok; it++) {
        const uint32_t s = it % ns, use = it / ns;
        if (use > 0) ok = mbar_wait(smem_u32(&empty_bar[s]), (use - 1) & 1);
        if (!ok) break;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t stage = smem_base + s * G::STAGE_BYTES;
        const int row = static_cast<int>(p.row_base + tok_begin + it * st_tok);
        mbar_arrive_expect_tx(bar, G::STAGE_BYTES);
        tma_load_2d(stage + 2 * G::STAGE_QS, &map_kd, bar, static_cast<int>(g0 * 16), row);
        for (uint32_t g = 0; g < hpc; g++)
          tma_load_3d(stage + g * (st_tok * 128), &map_kq, bar, 0, static_cast<int>(g0 + g), row);
        tma_load_2d(stage + 2 * G::STAGE_QS + G::STAGE_D, &map_vd, bar, static_cast<int>(g0 * 16), row);
        for (uint32_t g = 0; g < hpc; g++)
          tma_load_3d(stage + G::STAGE_QS + g * (st_tok * 128), &map_vq, bar, 0, static_cast<int>(g0 + g), row);
      }
      if (!ok) atomicExch(p.err, 1u);
    }
  } else {
    // ---------------- compute ----------------
    const int r = lane >> 2, qd = lane & 3;
    const uint32_t g = warp % hpc, slot = warp / hpc;
    const bool row_valid = static_cast<uint32_t>(r) < p.qpg;

    // A fragments of Q for the 8 k-slices (block b, half s): slice (b, s) covers
    // dims 32b + 8*quad + 4s + {0,1,2,3}; a0 = (dim+0, dim+2), a2 = (dim+1, dim+3)
    // to match the byte order k_pair produces. Rows >= qpg are zero.
    uint32_t qa0[4][2], qa2[4][2];
    float qcorr[4];
    {
      const __half* qrow = p.q + (static_cast<size_t>(g0 + g) * p.qpg + (row_valid ? r : 0)) * BP_HEAD_DIM;
#pragma unroll
      for (int b = 0; b < 4; b++) {
        float bsum = 0.f;
#pragma unroll
        for (int s = 0; s < 2; s++) {
          uint2 hv = make_uint2(0u, 0u);
          if (row_valid) hv = *reinterpret_cast<const uint2*>(qrow + 32 * b + 8 * qd + 4 * s);
          qa0[b][s] = prmt(hv.x, hv.y, 0x5410);  // (h0, h2)
          qa2[b][s] = prmt(hv.x, hv.y, 0x7632);  // (h1, h3)
          const float2 f0 = __half22float2(*reinterpret_cast<__half2*>(&hv.x));
          const float2 f1 = __half22float2(*reinterpret_cast<__half2*>(&hv.y));
          bsum += (f0.x + f0.y) + (f1.x + f1.y);
        }
        bsum += __shfl_xor_sync(FULL, bsum, 1);
        bsum += __shfl_xor_sync(FULL, bsum, 2);
        qcorr[b] = DENORM ? bsum * (128.0f / 16777216.0f) : 0.f;
      }
    }
    // In the DENORM path accumulators carry a factor 2^-24.
    const float s_mul = p.sm_scale_log2 * (DENORM ? 16777216.0f : 1.0f);

    // Per-lane byte offsets inside a sub-tile (block b is an xor with b << 5).
    // K (B operand): lane (r, quad) reads token row 2*(r ^ (r>>2)) + t, 8 bytes of block 0.
    // V (A operand) and scales: quad owns token rows 4*quad + (j ^ (quad & 2)).
    uint32_t koff[2], voff[4], soff[4];
    const uint32_t rb = 16 * hpc;
#pragma unroll
    for (int t = 0; t < 2; t++) {
      const uint32_t row = 2 * (r ^ (r >> 2)) + t;
      koff[t] = row * 128 + ((((qd >> 1)) ^ (row & 7)) << 4) + ((qd & 1) << 3);
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint32_t rowj = 4 * qd + (j ^ (qd & 2));
      voff[j] = rowj * 128 + ((((r >> 2)) ^ (rowj & 7)) << 4) + ((r & 3) << 2);
      const uint32_t o = (slot * SUBTILE + rowj) * rb + g * 16;
      soff[j] = p.d_swz ? swz128(o) : o;
    }

    WarpAcc w;
    w.m_run = NEG_BIG;
    w.l_run = 0.f;
#pragma unroll
    for (int b = 0; b < 4; b++) {
#pragma unroll
      for (int c = 0; c < 4; c++) { w.oacc[b][0][c] = 0.f; w.oacc[b][1][c] = 0.f; w.pacc[b][c] = 0.f; }
    }

    bool ok = true;
    for (uint32_t it = 0; it < n_iter; it++) {
      const uint32_t s = it % ns, use = it / ns;
      ok = mbar_wait(smem_u32(&full_bar[s]), use & 1);
      if (!ok) break;
      const uint32_t stage = smem_base + s * G::STAGE_BYTES;
      const uint32_t tile_tok0 = tok_begin + it * st_tok + slot * SUBTILE;
      if (tile_tok0 < tok_end) {
        const uint32_t ktile = stage + g * (st_tok * 128) + slot * (SUBTILE * 128);
        const uint32_t vtile = ktile + G::STAGE_QS;
        const uint32_t kd_tile = stage + 2 * G::STAGE_QS;
        const uint32_t vd_tile = kd_tile + G::STAGE_D;
        if (tile_tok0 + SUBTILE <= tok_end) {
          process_tile<DENORM, false>(w, ktile, vtile, kd_tile, vd_tile, koff, voff, soff, qa0, qa2, qcorr, s_mul, 16u, qd);
        } else {
          process_tile<DENORM, true>(w, ktile, vtile, kd_tile, vd_tile, koff, voff, soff, qa0, qa2, qcorr, s_mul,
                                     tok_end - tile_tok0, qd);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
    }
    if (!ok && lane == 0) atomicExch(p.err, 1u);

    // ---- warp result -> merge buffer (placed after the stage ring) ----
    float l_run = w.l_run;
    l_run += __shfl_xor_sync(FULL, l_run, 1);
    l_run += __shfl_xor_sync(FULL, l_run, 2);
    float* mo = reinterpret_cast<float*>(smem_gen + ns * G::STAGE_BYTES);
    float* mm = mo + NW_ * 8 * BP_HEAD_DIM;
    float* ml = mm + NW_ * 8;
    const float os = DENORM ? 16777216.0f : 1.0f;
#pragma unroll
    for (int b = 0; b < 4; b++) {
      const int dim = 32 * b + 4 * r;
      const float pa = DENORM ? w.pacc[b][0] * 128.0f : 0.f;  // head 2*quad
      const float pb = DENORM ? w.pacc[b][1] * 128.0f : 0.f;  // head 2*quad + 1
      if (static_cast<uint32_t>(2 * qd) < p.qpg) {
        float4 v = make_float4((w.oacc[b][0][0] - pa) * os, (w.oacc[b][1][0] - pa) * os,
                               (w.oacc[b][0][2] - pa) * os, (w.oacc[b][1][2] - pa) * os);
        *reinterpret_cast<float4*>(mo + (warp * 8 + 2 * qd) * BP_HEAD_DIM + dim) = v;
      }
      if (static_cast<uint32_t>(2 * qd + 1) < p.qpg) {
        float4 v = make_float4((w.oacc[b][0][1] - pb) * os, (w.oacc[b][1][1] - pb) * os,
                               (w.oacc[b][0][3] - pb) * os, (w.oacc[b][1][3] - pb) * os);
        *reinterpret_cast<float4*>(mo + (warp * 8 + 2 * qd + 1) * BP_HEAD_DIM + dim) = v;
      }
    }
    if (qd == 0 && row_valid) {
      mm[warp * 8 + r] = w.m_run;
      ml[warp * 8 + r] = l_run;
    }
  }
  __syncthreads();

  // ---- merge the warps of each KV head, write the split's partial ----
  {
    const float* mo = reinterpret_cast<const float*>(smem_gen + ns * G::STAGE_BYTES);
    const float* mm = mo + NW_ * 8 * BP_HEAD_DIM;
    const float* ml = mm + NW_ * 8;
    const uint32_t total = hpc * p.qpg * BP_HEAD_DIM;  // outputs of this CTA
    for (uint32_t idx = threadIdx.x; idx < total; idx += blockDim.x) {
      const uint32_t hl = idx >> 7, d = idx & 127;
      const uint32_t g = hl / p.qpg, hq = hl % p.qpg;
      float m_all = NEG_BIG;
      for (uint32_t sl = 0; sl < wph; sl++) m_all = fmaxf(m_all, mm[(sl * hpc + g) * 8 + hq]);
      float o = 0.f, l = 0.f;
      for (uint32_t sl = 0; sl < wph; sl++) {
        const uint32_t wi = sl * hpc + g;
        const float e = ex2(mm[wi * 8 + hq] - m_all);
        o += mo[(wi * 8 + hq) * BP_HEAD_DIM + d] * e;
        l += ml[wi * 8 + hq] * e;
      }
      const uint32_t h = g0 * p.qpg + hl;  // query head within the context
      if (n_splits == 1) {
        p.out[static_cast<size_t>(h) * BP_HEAD_DIM + d] = __float2half_rn(o * (1.0f / l));
      } else {
        float* dst = p.partials + (static_cast<size_t>(split) * p.n_head + h) * BP_PART_STRIDE;
        dst[d] = o;
        if (d == 0) { dst[128] = m_all; dst[129] = l; }
      }
    }
  }
  // The producer drains its own copies before the CTA retires (all of them have
  // already completed unless a wait above gave up).
  if (warp == NW_ && lane == 0) {
    const uint32_t first = n_iter > ns ? n_iter - ns : 0;
    for (uint32_t it = first; it < n_iter; it++)
      if (!mbar_wait(smem_u32(&full_bar[it % ns]), (it / ns) & 1, 1u << 20)) atomicExch(p.err, 2u);
  }
}

}  // namespace

// Launch geometry. A stage holds 16 * (NW / hpc) tokens of `hpc` KV heads; a
// split is a whole number of stages, chosen so that the grid is at most one CTA
// per SM. nw (8 or 16 compute warps) and hpc (KV heads per CTA) are context
// options.
static uint32_t stage_tokens(const bp_attn_ctx* c) { return SUBTILE * (c->opt_nw / c->opt_hpc); }

uint32_t bp_decode_max_splits(const bp_attn_ctx* c) {
  const uint32_t sms = static_cast<uint32_t>(c->sm_count);
  return sms < COMBINE_MAX_SPLITS ? sms : COMBINE_MAX_SPLITS;
}

static uint32_t stages_per_split(const bp_attn_ctx* c, uint32_t cur_pos) {
  const uint32_t st = stage_tokens(c);
  const uint32_t n_st = (cur_pos + st - 1) / st;
  const uint32_t groups = c->cfg.n_kv_head / c->opt_hpc;
  uint32_t ctas = bp_decode_max_splits(c) / groups;
  if (ctas == 0) ctas = 1;
  return (n_st + ctas - 1) / ctas;
}

uint32_t bp_decode_splits(const bp_attn_ctx* c, uint32_t cur_pos) {
  if (bp_use_umma(c)) return bp_decode_umma_splits(c, cur_pos);
  if (c->variant == 1) {
    const uint32_t tps = 256, n = (cur_pos + tps - 1) / tps;
    return n > bp_decode_max_splits(c) ? bp_decode_max_splits(c) : n;
  }
  const uint32_t st = stage_tokens(c);
  const uint32_t n_st = (cur_pos + st - 1) / st;
  const uint32_t spp = stages_per_split(c, cur_pos);
  return (n_st + spp - 1) / spp;
}

cudaError_t bp_launch_scalar_attention(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q,
                                       __half* out, uint32_t cur_pos, uint32_t m, bool is_prefill,
                                       uint32_t* launches) {
  const float* k_d = reinterpret_cast<const float*>(c->kv[0] + bp_d_off(c, layer));
  const float* v_d = reinterpret_cast<const float*>(c->kv[1] + bp_d_off(c, layer));
  const uint32_t* k_qs = reinterpret_cast<const uint32_t*>(c->kv[0] + bp_qs_off(c, layer));
  const uint32_t* v_qs = reinterpret_cast<const uint32_t*>(c->kv[1] + bp_qs_off(c, layer));
  const float scale = 1.0f / sqrtf(static_cast<float>(BP_HEAD_DIM));
  uint32_t n_splits = 1, tps = cur_pos;
  if (!is_prefill) {
    n_splits = bp_decode_splits(c, cur_pos);
    tps = (cur_pos + n_splits - 1) / n_splits;
  } else {
    tps = m;
  }
  dim3 grid(n_splits, c->cfg.n_head, m);
  attn_scalar_kernel<<<grid, 128, 0, s>>>(q, k_d, k_qs, v_d, v_qs, c->partials, out, c->cfg.n_head,
                                          c->cfg.n_kv_head, cur_pos, tps, is_prefill ? 1u : 0u, scale);
  *launches += 1;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (n_splits > 1) {
    attn_combine_kernel<<<c->cfg.n_head, 128 * COMBINE_GROUPS, 0, s>>>(c->partials, out, c->cfg.n_head, n_splits);
    *launches += 1;
    e = cudaGetLastError();
  }
  return e;
}

uint32_t bp_decode_stage_tokens(const bp_attn_ctx* c) { return stage_tokens(c); }

template <int NW_>
static cudaError_t set_smem_attr() {
  const int max_smem = Geo<NW_>::max_stages() * Geo<NW_>::STAGE_BYTES + Geo<NW_>::MERGE_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<NW_, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(decode_mma_kernel<NW_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

// Opt the production kernels into their dynamic shared memory on the context's device.
cudaError_t bp_decode_init(bp_attn_ctx*) {
  cudaError_t e = set_smem_attr<8>();
  if (e != cudaSuccess) return e;
  return set_smem_attr<16>();
}

template <int NW_>
static cudaError_t launch_mma(bp_attn_ctx* c, cudaStream_t s, DecodeParams& p, uint32_t spp, uint32_t n_splits,
                              bool denorm) {
  using G = Geo<NW_>;
  p.n_stages = spp < G::max_stages() ? spp : G::max_stages();
  const size_t smem = static_cast<size_t>(p.n_stages) * G::STAGE_BYTES + G::MERGE_BYTES + 1024;
  dim3 grid(n_splits, c->cfg.n_kv_head / c->opt_hpc);
  auto kern = denorm ? decode_mma_kernel<NW_, true> : decode_mma_kernel<NW_, false>;
  kern<<<grid, (NW_ + 1) * 32, smem, s>>>(c->map_qs[0], c->map_d[0], c->map_qs[1], c->map_d[1], p);
  return cudaGetLastError();
}

// Meeting point of the ranks of a peer exchange, counter `slot`: every rank adds one to every
// rank's counter (system-scope release, after a system fence: the peer stores of the kernels
// before this one in the stream are complete by then), then waits (bounded, system-scope acquire
// loads) until its own counter has reached (meetings so far + 1) * ranks. Counters only grow, so a
// rank that runs ahead cannot confuse a slower one.
struct PeerFlags {
  uint32_t* f[BP_MAX_PEERS];
};
__global__ void __launch_bounds__(32)
peer_sync_kernel(PeerFlags flags, uint32_t n_ranks, uint32_t rank, uint32_t slot, uint32_t limit, uint32_t* epochs,
                 uint32_t* err) {
  bp::pdl_wait();
  if (threadIdx.x < n_ranks) {
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flags.f[threadIdx.x] + slot), "r"(1u) : "memory");
  }
  if (threadIdx.x == 0) {
    const uint32_t target = (epochs[slot] + 1u) * n_ranks;
    bool ok = false;
    for (uint32_t i = 0; i < limit && !ok; i++) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags.f[rank] + slot) : "memory");
      ok = static_cast<int32_t>(v - target) >= 0;
      if (!ok) __nanosleep(32);
    }
    if (!ok) atomicExch(err, 6u);
    epochs[slot] += 1u;
  }
}

cudaError_t bp_launch_peer_sync(bp_attn_ctx* c, cudaStream_t s, uint32_t slot) {
  PeerFlags f;
  for (uint32_t r = 0; r < BP_MAX_PEERS; r++) f.f[r] = r < c->n_px ? c->px_flag[r] : nullptr;
  return bp_launch(c->opt_pdl != 0, peer_sync_kernel, dim3(1), dim3(32), 0, s, f, c->n_px, c->cfg.shard, slot, c->opt_wait_limit,
                   c->px_epoch, c->err_dev);
}

// Fused layer step. With the tcgen05 kernel: one launch does the Q norm + RoPE, the new token's
// cache write and the split attention, a second one merges the splits. Otherwise: the separate kernels.
cudaError_t bp_launch_decode_fused(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q_raw, __half* q_roped,
                                   const __half* w_q, const __half* k_cur, const __half* v_cur, const __half* w_k,
                                   uint32_t pos, __half* out, uint32_t* launches) {
  if (c->variant == 0 && bp_use_umma(c)) {
    bp_fused_step fs;
    fs.q_roped = q_roped;
    fs.w_q = w_q;
    fs.w_k = w_k;
    fs.k_cur = k_cur;
    fs.v_cur = v_cur;
    uint32_t n_splits = 1;
    cudaError_t e = bp_launch_decode_umma(c, s, layer, q_raw, out, pos + 1, &n_splits, &fs);
    *launches += 1;
    if (e != cudaSuccess) return e;
    if (n_splits > 1) {
      *launches += 1;
      e = bp_launch(c->opt_pdl != 0, attn_combine_kernel, dim3(c->cfg.n_head), dim3(128 * COMBINE_GROUPS), 0, s,
                    static_cast<const float*>(c->partials), out, c->cfg.n_head, n_splits);
    }
    return e;
  }
  if (q_roped == nullptr) return cudaErrorInvalidValue;  // the separate kernels rotate q in a caller's buffer
  cudaError_t e = cudaMemcpyAsync(q_roped, q_raw, static_cast<size_t>(c->q_dim) * sizeof(__half), cudaMemcpyDeviceToDevice, s);
  if (e != cudaSuccess) return e;
  e = bp_launch_q_norm_rope(c, s, q_roped, w_q, pos, 1, launches);
  if (e != cudaSuccess) return e;
  e = bp_launch_kv_writeback(c, s, layer, k_cur, v_cur, w_k, pos, 1, launches);
  if (e != cudaSuccess) return e;
  return bp_launch_decode(c, s, layer, q_roped, out, pos + 1, launches);
}

cudaError_t bp_launch_decode(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q,
                             __half* out, uint32_t cur_pos, uint32_t* launches) {
  if (c->variant == 1) return bp_launch_scalar_attention(c, s, layer, q, out, cur_pos, 1, false, launches);
  if (bp_use_umma(c)) {
    uint32_t n_splits = 1;
    cudaError_t e = bp_launch_decode_umma(c, s, layer, q, out, cur_pos, &n_splits);
    *launches += 1;
    if (e != cudaSuccess) return e;
    // The kernel reports one split when it merged the splits itself (the default); the separate
    // merge kernel runs only with the option decode_in_kernel_merge = 0.
    if (n_splits > 1) {
      *launches += 1;
      e = bp_launch(c->opt_pdl != 0, attn_combine_kernel, dim3(c->cfg.n_head), dim3(128 * COMBINE_GROUPS), 0, s,
                    static_cast<const float*>(c->partials), out, c->cfg.n_head, n_splits);
    }
    return e;
  }
  if (!c->have_maps) return cudaErrorNotSupported;

  const uint32_t st = stage_tokens(c);
  const uint32_t spp = stages_per_split(c, cur_pos);
  const uint32_t n_splits = bp_decode_splits(c, cur_pos);
  DecodeParams p;
  p.q = q;
  p.out = out;
  p.partials = c->partials;
  p.err = c->err_dev;
  p.row_base = layer * c->cfg.max_seq;
  p.cur_pos = cur_pos;
  p.tps = spp * st;
  p.n_stages = 1;
  p.n_head = c->cfg.n_head;
  p.hpc = c->opt_hpc;
  p.qpg = c->qpg;
  p.d_swz = (16 * c->opt_hpc == 128) ? 1u : 0u;
  p.sm_scale_log2 = (1.0f / sqrtf(static_cast<float>(BP_HEAD_DIM))) * 1.4426950408889634f;
  cudaError_t e = c->opt_nw == 16 ? launch_mma<16>(c, s, p, spp, n_splits, c->variant != 2)
                                  : launch_mma<8>(c, s, p, spp, n_splits, c->variant != 2);
  *launches += 1;
  if (e != cudaSuccess) return e;
  if (n_splits > 1) {
    attn_combine_kernel<<<c->cfg.n_head, 128 * COMBINE_GROUPS, 0, s>>>(c->partials, out, c->cfg.n_head, n_splits);
    *launches += 1;
    e = cudaGetLastError();
  }
  return e;
}

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Some hosts cannot call cudaMalloc where they run this step: a real-time
// serving loop that has handed all device memory to its own arena, a plugin
// that is loaded into a process whose allocator is owned by someone else, or a
// caller that sits inside a region where allocation is forbidden. For them the
// split-KV scratch (one partial per split and query head) lives in a fixed
// array that is part of the library image: every GPU that loads the library
// holds these NOALLOC_SCRATCH_FLOATS * 4 bytes (about 1.1 MB) until the process
// exits. The price is a hard limit on the problem size (at most 64 query heads;
// the number of splits is capped at 32) and no re-entrancy: all calls share the
// one array, so two calls that overlap on the GPU (different streams, or
// different host threads) race on it. Nothing in the array has to be zero on
// entry: each call overwrites every partial it later reads, and what the
// previous call left behind is never read. The arithmetic runs on the plain
// CUDA-core kernels (attn_scalar_kernel + attn_combine_kernel), not on the
// tcgen05 kernel of bp_attn_decode, whose scratch protocol needs a context: the
// results agree within the attention tolerance, not bit for bit, and a call
// takes several times longer. The per-device address slot below is written
// without a lock; concurrent first calls from several host threads store the
// same value.
// ---------------------------------------------------------------------------
namespace {
constexpr uint32_t NOALLOC_MAX_HEADS = 64;
constexpr uint32_t NOALLOC_MAX_SPLITS = 32;
constexpr uint32_t NOALLOC_SCRATCH_FLOATS = NOALLOC_MAX_SPLITS * NOALLOC_MAX_HEADS * BP_PART_STRIDE;
constexpr int NOALLOC_MAX_DEVICES = 64;
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];
// Device address of the array above, per device. In host code the array's name
// is only a handle for the runtime; the address a kernel can use comes from
// cudaGetSymbolAddress with that device current.
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
}  // namespace

extern "C" int bp_attn_decode_static_scratch(void* stream, const void* q, const void* kv_k, const void* kv_v,
                                             void* out, uint32_t n_layer, uint32_t max_seq, uint32_t n_head,
                                             uint32_t n_kv_head, uint32_t layer, uint32_t cur_pos) {
  if (!q || !kv_k || !kv_v || !out) return BP_ERR_NULL;
  if (n_head == 0 || n_kv_head == 0 || n_head % n_kv_head != 0 || n_layer == 0 || max_seq == 0 || layer >= n_layer)
    return BP_ERR_CONFIG;
  if (n_head > NOALLOC_MAX_HEADS) return BP_ERR_CONFIG;  // beyond the fixed scratch: use bp_attn_decode
  if (cur_pos == 0) return BP_ERR_CONFIG;
  if (cur_pos > max_seq) return BP_ERR_CONTEXT_OVERFLOW;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return BP_ERR_CUDA;
  {
    // The scratch address belongs to the CURRENT device, so the cache (and with it the stream and
    // the other buffers) must live there too; a cache on another GPU is refused, not guessed at.
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, kv_k) != cudaSuccess) return BP_ERR_CUDA;
    if (attr.type == cudaMemoryTypeDevice && attr.device != dev) return BP_ERR_CONFIG;
  }
  if (!g_noalloc_ptr[dev]) {
    // First call on this device: resolve the array's device address (this does
    // not allocate). Make this first call outside any stream capture.
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch) != cudaSuccess || !p) return BP_ERR_CUDA;
    g_noalloc_ptr[dev] = p;
  }
  const uint32_t kv_dim = n_kv_head * BP_HEAD_DIM, nb = kv_dim / BP_QK8;
  const uint64_t d_total = static_cast<uint64_t>(n_layer) * max_seq * nb * 4u;
  const uint64_t d_off = static_cast<uint64_t>(layer) * max_seq * nb * 4u;
  const uint64_t qs_off = d_total + static_cast<uint64_t>(layer) * max_seq * kv_dim;
  const uint8_t* kb = static_cast<const uint8_t*>(kv_k);
  const uint8_t* vb = static_cast<const uint8_t*>(kv_v);
  uint32_t n_splits = (cur_pos + 255) / 256;
  if (n_splits > NOALLOC_MAX_SPLITS) n_splits = NOALLOC_MAX_SPLITS;
  const uint32_t tps = (cur_pos + n_splits - 1) / n_splits;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(n_splits, n_head, 1);
  attn_scalar_kernel<<<grid, 128, 0, st>>>(static_cast<const __half*>(q), reinterpret_cast<const float*>(kb + d_off),
                                           reinterpret_cast<const uint32_t*>(kb + qs_off),
                                           reinterpret_cast<const float*>(vb + d_off),
                                           reinterpret_cast<const uint32_t*>(vb + qs_off), g_noalloc_ptr[dev],
                                           static_cast<__half*>(out), n_head, n_kv_head, cur_pos, tps, 0u,
                                           1.0f / sqrtf(static_cast<float>(BP_HEAD_DIM)));
  if (cudaGetLastError() != cudaSuccess) return BP_ERR_CUDA;
  if (n_splits > 1) {
    attn_combine_kernel<<<n_head, 128 * COMBINE_GROUPS, 0, st>>>(g_noalloc_ptr[dev], static_cast<__half*>(out),
                                                                 n_head, n_splits);
    if (cudaGetLastError() != cudaSuccess) return BP_ERR_CUDA;
  }
  return BP_OK;
}
