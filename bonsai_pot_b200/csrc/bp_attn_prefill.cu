// Batched-prefill causal attention over the Q8_0 KV cache. Replaces
// attention.wgsl (dispatch_attention with is_prefill = 1, src/forward.rs:501-532).
//
// Flash attention on the 5th-generation tensor cores (tcgen05.mma kind::f16,
// accumulators in TMEM). One CTA owns one KV head and a tile of 128 query rows:
// the 128 / qpg consecutive tokens of the tile times the qpg query heads of the
// group, so every dequantised K/V tile is shared by all heads of the group.
// Per tile of 128 keys:
//   producer warp   TMA: int8 K and V tiles (128-byte swizzle) + their FP32 block scales
//   dequant warps   int8 -> f16 (value * block scale), written as UMMA operand tiles:
//                   K as the K-major B operand of S = Q K^T, V as the MN-major B operand of O += P V
//   issuer warp     8 UMMAs (M 128, N 128, K 16) for S into TMEM, 8 for O
//   softmax warps   thread = query row = TMEM lane: scale, causal mask, online max / sum,
//                   P as f16 into the K-major A operand tile; O is rescaled in TMEM
//                   (tcgen05.ld / st) only when a row maximum moved
// Inside each group of four head dims the operand tiles hold the order
// (d0, d2, d1, d3): that is what the cheapest int8 expansion yields, it is applied
// to Q as well (the contraction does not care) and undone when O is written.
// Every wait is bounded; a timeout sets the context's error word and the CTA
// winds down and frees its TMEM.
#include "bp_common.cuh"
#include "bp_ptx.cuh"

cudaError_t bp_launch_scalar_attention(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q,
                                       __half* out, uint32_t cur_pos, uint32_t m, bool is_prefill,
                                       uint32_t* launches);
bool bp_make_kv_maps(bp_attn_ctx* c, int kind, uint32_t rows_box, uint32_t d_inner, bool d_swizzle,
                     CUtensorMap* map_qs, CUtensorMap* map_d);

namespace {

using namespace bp;

constexpr unsigned FULL = 0xffffffffu;
constexpr float NEG_BIG = -1e30f;
constexpr uint32_t BM = 128, BN = 128;
constexpr uint32_t P_THREADS = 320;              // producer, issuer, 4 dequant warps, 4 softmax warps
constexpr uint32_t P_TMEM_COLS = 512;            // S: 2 x 128 columns, O: 128 columns
constexpr uint32_t P_WAIT_LIMIT = 1u << 22;
constexpr uint32_t OPER_B = 2 * 16384;           // one f16 operand tile: 2 chunks of [128 rows][128 B]
constexpr uint32_t I8_STAGE_B = 2 * 16384 + 2 * 2048;  // int8 K, V tiles + their scale rows
constexpr uint32_t OFF_Q = 0, OFF_KF = OPER_B, OFF_VF = 2 * OPER_B, OFF_P = 3 * OPER_B, OFF_I8 = 4 * OPER_B;
constexpr uint32_t P_SMEM = OFF_I8 + 2 * I8_STAGE_B + 1024;

struct PrefillParams {
  const __half* q;
  __half* out;
  uint32_t* err;
  uint32_t row_base, m, n_head, qpg, n_qtiles;
  float scale_log2;
};

// Physical byte offset of 16-byte unit `u16` (0..15) of row `r` in an operand tile.
__device__ __forceinline__ uint32_t oper_off(uint32_t r, uint32_t u16) {
  return (u16 >> 3) * 16384 + r * 128 + (((u16 & 7) ^ (r & 7)) << 4);
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Four int8 of one word -> four f16 scaled by `s2` (both halves the same scale), in the order
// (b0, b2), (b1, b3): the byte x + 128 under 0x64 is the f16 1024 + x + 128; minus 1152, times scale.
__device__ __forceinline__ void dequant4(uint32_t w, __half2 s2, uint32_t& even, uint32_t& odd) {
  const __half2 bias = __half2half2(__ushort_as_half(0x6480));  // 1152
  const uint32_t x = w ^ 0x80808080u;
  uint32_t e = (x & 0x00ff00ffu) | 0x64006400u;
  uint32_t o = ((x >> 8) & 0x00ff00ffu) | 0x64006400u;
  __half2 eh = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&e), bias), s2);
  __half2 oh = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&o), bias), s2);
  even = *reinterpret_cast<uint32_t*>(&eh);
  odd = *reinterpret_cast<uint32_t*>(&oh);
}

// One row (128 int8 + 4 block scales) of a TMA-swizzled int8 tile -> one row of an f16 operand tile.
// `live` = false writes zeros (keys beyond the sequence: their cache rows are undefined).
__device__ __forceinline__ void dequant_row(const uint8_t* src_tile, const uint8_t* scales, uint8_t* dst_tile, uint32_t t,
                                            bool live) {
  const float4 sc = *reinterpret_cast<const float4*>(scales + t * 16);
  const float scb[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
  for (uint32_t c = 0; c < 8; c++) {  // 16-byte chunks of the int8 row: dims 16c .. 16c+15
    uint4 w = *reinterpret_cast<const uint4*>(src_tile + t * 128 + ((c ^ (t & 7)) << 4));
    const __half2 s2 = __float2half2_rn(live ? scb[c >> 1] : 0.f);
    if (!live) w = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);  // value 0: no NaN from junk
    uint32_t a[8];
    dequant4(w.x, s2, a[0], a[1]);
    dequant4(w.y, s2, a[2], a[3]);
    dequant4(w.z, s2, a[4], a[5]);
    dequant4(w.w, s2, a[6], a[7]);
    *reinterpret_cast<uint4*>(dst_tile + oper_off(t, 2 * c)) = make_uint4(a[0], a[1], a[2], a[3]);
    *reinterpret_cast<uint4*>(dst_tile + oper_off(t, 2 * c + 1)) = make_uint4(a[4], a[5], a[6], a[7]);
  }
}

__global__ void __launch_bounds__(P_THREADS, 1)
prefill_umma_kernel(const __grid_constant__ CUtensorMap map_kq, const __grid_constant__ CUtensorMap map_kd,
                    const __grid_constant__ CUtensorMap map_vq, const __grid_constant__ CUtensorMap map_vd,
                    const PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[2], empty_bar[2], s_ready[2], s_free[2];
  __shared__ __align__(8) uint64_t kf_ready, kf_free, vf_ready, vf_free, p_ready, o_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile uint32_t abort_s;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t g = blockIdx.y;
  const uint32_t qtile = p.n_qtiles - 1 - blockIdx.x;  // long (late) tiles first
  const uint32_t tq_tokens = BM / p.qpg;               // tokens per query tile
  const uint32_t tq0 = qtile * tq_tokens;
  const uint32_t n_keys = min(tq0 + tq_tokens, p.m);   // keys [0, n_keys) can be attended by this tile
  const uint32_t n_tiles = (n_keys + BN - 1) / BN;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; i++) {
      mbar_init(smem_u32(&full_bar[i]), 1);
      mbar_init(smem_u32(&empty_bar[i]), 4);
      mbar_init(smem_u32(&s_ready[i]), 1);
      mbar_init(smem_u32(&s_free[i]), 4);
    }
    mbar_init(smem_u32(&kf_ready), 4);
    mbar_init(smem_u32(&kf_free), 1);
    mbar_init(smem_u32(&vf_ready), 4);
    mbar_init(smem_u32(&vf_free), 1);
    mbar_init(smem_u32(&p_ready), 4);
    mbar_init(smem_u32(&o_done), 1);
    abort_s = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_s), P_TMEM_COLS);
  // Q tile: row r = (token tq0 + r / qpg, head g * qpg + r % qpg), dims in (d0, d2, d1, d3) order.
  for (uint32_t i = threadIdx.x; i < BM * 16; i += P_THREADS) {
    const uint32_t r = i >> 4, u = i & 15;
    const uint32_t tok = tq0 + r / p.qpg, head = g * p.qpg + r % p.qpg;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tok < p.m) v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(tok) * p.n_head + head) * BP_HEAD_DIM + 8 * u);
    const uint4 w = make_uint4(prmt(v.x, v.y, 0x5410), prmt(v.x, v.y, 0x7632), prmt(v.z, v.w, 0x5410), prmt(v.z, v.w, 0x7632));
    *reinterpret_cast<uint4*>(smem_gen + OFF_Q + oper_off(r, u)) = w;
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (abort_s) return;
    if (!mbar_wait(smem_u32(bar), parity, P_WAIT_LIMIT)) {
      abort_s = 1;
      atomicExch(p.err, 5u);
    }
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      prefetch_tensormap(&map_kq);
      prefetch_tensormap(&map_vq);
      prefetch_tensormap(&map_kd);
      prefetch_tensormap(&map_vd);
      for (uint32_t i = 0; i < n_tiles; i++) {
        const uint32_t s = i & 1, use = i >> 1;
        if (use > 0) wait(&empty_bar[s], (use - 1) & 1);
        if (abort_s) break;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t stage = smem_base + OFF_I8 + s * I8_STAGE_B;
        const int row = static_cast<int>(p.row_base + i * BN);
        mbar_arrive_expect_tx(bar, I8_STAGE_B);
        tma_load_3d(stage, &map_kq, bar, 0, static_cast<int>(g), row);
        tma_load_2d(stage + 32768, &map_kd, bar, static_cast<int>(g * 16), row);
        tma_load_3d(stage + 16384, &map_vq, bar, 0, static_cast<int>(g), row);
        tma_load_2d(stage + 32768 + 2048, &map_vd, bar, static_cast<int>(g * 16), row);
      }
    }
  } else if (warp == 1) {
    // ---------------- UMMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = umma_idesc(1, 0, 0, 0, 0, BM, BN);  // f32 = f16 (K-major) x f16 (K-major)
      constexpr uint32_t IDESC_PV = umma_idesc(1, 0, 0, 0, 1, BM, BN);  // f32 += f16 (K-major) x f16 (MN-major)
      const uint64_t dk = umma_desc_sw128(0, 16, 1024);       // K-major operands
      const uint64_t dmn = umma_desc_sw128(0, 16384, 1024);   // V: next 64 dims 16 KB away, 8 key rows 1 KB apart
      const uint64_t qa = dk + ((smem_base + OFF_Q) >> 4), kb = dk + ((smem_base + OFF_KF) >> 4);
      const uint64_t pa = dk + ((smem_base + OFF_P) >> 4), vb = dmn + ((smem_base + OFF_VF) >> 4);
      auto issue_qk = [&](uint32_t i) {
        wait(&kf_ready, i & 1);
        if (i >= 2) wait(&s_free[i & 1], ((i >> 1) - 1) & 1);
        tc_fence_after();
#pragma unroll
        for (uint32_t ks = 0; ks < 8; ks++) {  // 16 dims per UMMA: chunk ks / 4, 32 bytes per step inside it
          const uint32_t o16 = (ks >> 2) * (16384 >> 4) + (ks & 3) * 2;
          umma_f16(tmem + (i & 1) * BN, qa + o16, kb + o16, IDESC_QK, ks);
        }
        umma_commit(smem_u32(&s_ready[i & 1]));
        umma_commit(smem_u32(&kf_free));
      };
      if (n_tiles > 0) issue_qk(0);
      for (uint32_t i = 0; i < n_tiles; i++) {
        if (i + 1 < n_tiles) issue_qk(i + 1);
        wait(&p_ready, i & 1);
        wait(&vf_ready, i & 1);
        tc_fence_after();
#pragma unroll
        for (uint32_t ks = 0; ks < 8; ks++) {  // 16 keys per UMMA
          const uint32_t a16 = (ks >> 2) * (16384 >> 4) + (ks & 3) * 2;
          umma_f16(tmem + 2 * BN, pa + a16, vb + ks * (16 * 128 >> 4), IDESC_PV, (i | ks) ? 1u : 0u);
        }
        umma_commit(smem_u32(&vf_free));
        umma_commit(smem_u32(&o_done));
      }
    }
  } else if (warp < 6) {
    // ---------------- dequant: thread = key row of the tile ----------------
    const uint32_t t = (warp - 2) * 32 + lane;
    for (uint32_t i = 0; i < n_tiles; i++) {
      const uint32_t s = i & 1;
      const uint8_t* stage = smem_gen + OFF_I8 + s * I8_STAGE_B;
      const bool live = i * BN + t < n_keys;
      wait(&full_bar[s], (i >> 1) & 1);
      if (i > 0) wait(&kf_free, (i - 1) & 1);
      dequant_row(stage, stage + 32768, smem_gen + OFF_KF, t, live);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&kf_ready));
      if (i > 0) wait(&vf_free, (i - 1) & 1);
      dequant_row(stage + 16384, stage + 32768 + 2048, smem_gen + OFF_VF, t, live);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&vf_ready));
        mbar_arrive(smem_u32(&empty_bar[s]));
      }
    }
  } else {
    // ---------------- softmax: thread = query row = TMEM lane ----------------
    const uint32_t quad = warp & 3, r = quad * 32 + lane;
    const uint32_t lane_addr = (quad * 32) << 16;
    const uint32_t tok = tq0 + r / p.qpg, head = g * p.qpg + r % p.qpg;
    float m_run = NEG_BIG, l_run = 0.f;
    for (uint32_t i = 0; i < n_tiles; i++) {
      const uint32_t b = i & 1;
      wait(&s_ready[b], (i >> 1) & 1);
      tc_fence_after();
      float sc[128];
#pragma unroll
      for (uint32_t c = 0; c < 4; c++) {
        uint32_t raw[32];
        tmem_ld32(tmem + lane_addr + b * BN + 32 * c, raw);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j++) sc[32 * c + j] = __uint_as_float(raw[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_free[b]));
      // causal mask: key i*BN + c is visible to this row iff key <= tok (only the last tile can cut)
      if ((i + 1) * BN > tq0 + 1) {
        const uint32_t k0 = i * BN;
#pragma unroll
        for (int c = 0; c < 128; c++) if (k0 + c > tok) sc[c] = NEG_BIG;
      }
      float mx = sc[0];
#pragma unroll
      for (int c = 1; c < 128; c++) mx = fmaxf(mx, sc[c]);
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      const float corr = ex2(m_run - m_new);
      const bool moved = m_new > m_run;
      m_run = m_new;
      float sum = 0.f;
      uint32_t ph[64];
#pragma unroll
      for (int c = 0; c < 64; c++) {
        const float p0 = ex2(fmaf(sc[2 * c], p.scale_log2, -m_new));
        const float p1 = ex2(fmaf(sc[2 * c + 1], p.scale_log2, -m_new));
        sum += p0 + p1;
        __half2 h = __floats2half2_rn(p0, p1);
        ph[c] = *reinterpret_cast<uint32_t*>(&h);
      }
      l_run = l_run * corr + sum;
      // P and O are single-buffered: the previous tile's O += P V must have completed
      if (i > 0) wait(&o_done, (i - 1) & 1);
      tc_fence_after();
      if (i > 0 && __any_sync(FULL, moved)) {
#pragma unroll
        for (uint32_t c = 0; c < 4; c++) {
          uint32_t o[32];
          tmem_ld32(tmem + lane_addr + 2 * BN + 32 * c, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
          tmem_st32(tmem + lane_addr + 2 * BN + 32 * c, o);
        }
        tmem_st_wait();
      }
#pragma unroll
      for (uint32_t u = 0; u < 16; u++)
        *reinterpret_cast<uint4*>(smem_gen + OFF_P + oper_off(r, u)) = make_uint4(ph[4 * u], ph[4 * u + 1], ph[4 * u + 2], ph[4 * u + 3]);
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_ready));
    }
    // ---- O / l -> f16, undoing the (d0, d2, d1, d3) order ----
    if (n_tiles > 0) wait(&o_done, (n_tiles - 1) & 1);
    tc_fence_after();
    const float inv_l = 1.0f / l_run;
    __half* dst = p.out + (static_cast<size_t>(tok) * p.n_head + head) * BP_HEAD_DIM;
#pragma unroll
    for (uint32_t c = 0; c < 4; c++) {
      uint32_t o[32];
      tmem_ld32(tmem + lane_addr + 2 * BN + 32 * c, o);
      tmem_ld_wait();
      if (tok < p.m) {
#pragma unroll
        for (int q4 = 0; q4 < 8; q4++) {  // columns (4q4 .. 4q4+3) hold dims (d0, d2, d1, d3)
          const float d0 = __uint_as_float(o[4 * q4]) * inv_l, d2 = __uint_as_float(o[4 * q4 + 1]) * inv_l;
          const float d1 = __uint_as_float(o[4 * q4 + 2]) * inv_l, d3 = __uint_as_float(o[4 * q4 + 3]) * inv_l;
          __half2 lo = __floats2half2_rn(d0, d1), hi = __floats2half2_rn(d2, d3);
          *reinterpret_cast<uint2*>(dst + 32 * c + 4 * q4) =
              make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, P_TMEM_COLS);
}

}  // namespace

uint32_t bp_prefill_stage_tokens() { return BN; }

cudaError_t bp_prefill_init(bp_attn_ctx* c) {
  c->have_pmaps = true;
  for (int kind = 0; kind < 2 && c->have_pmaps; kind++)
    c->have_pmaps = bp_make_kv_maps(c, kind, BN, 16, false, &c->pmap_qs[kind], &c->pmap_d[kind]);
  return cudaFuncSetAttribute(prefill_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(P_SMEM));
}

cudaError_t bp_launch_prefill(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q,
                              __half* out, uint32_t m, uint32_t* launches) {
  const bool pow2 = (c->qpg & (c->qpg - 1)) == 0;
  if (c->variant == 1 || !c->have_pmaps || !pow2) return bp_launch_scalar_attention(c, s, layer, q, out, m, m, true, launches);
  PrefillParams p;
  p.q = q;
  p.out = out;
  p.err = c->err_dev;
  p.row_base = layer * c->cfg.max_seq;
  p.m = m;
  p.n_head = c->cfg.n_head;
  p.qpg = c->qpg;
  const uint32_t tq_tokens = BM / c->qpg;
  p.n_qtiles = (m + tq_tokens - 1) / tq_tokens;
  p.scale_log2 = (1.0f / sqrtf(static_cast<float>(BP_HEAD_DIM))) * 1.4426950408889634f;
  dim3 grid(p.n_qtiles, c->cfg.n_kv_head);
  prefill_umma_kernel<<<grid, P_THREADS, P_SMEM, s>>>(c->pmap_qs[0], c->pmap_d[0], c->pmap_qs[1], c->pmap_d[1], p);
  *launches += 1;
  return cudaGetLastError();
}
