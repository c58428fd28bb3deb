// Split-KV decode attention on the 5th-generation tensor cores (tcgen05, int8
// UMMA, accumulators in TMEM). Same contract as decode_mma_kernel: one CTA per
// (token range, group of KV heads) writes a partial (o, m, l) per query head.
//
// Why: with warp-level MMA every cache byte passes through registers and costs
// ALU work to become an f16 operand. Here the int8 tiles that TMA drops into
// shared memory ARE the tensor-core operands:
//   S^T[token][head]  = K tile (A, K-major, 128 tokens x 32 dims of one Q8_0 block)
//                       x Q^T (B, 15-bit integer Q split into a high and a low byte row)
//   O^T[dim][head]    = V tile (A, MN-major: the 128 dims of a token row are contiguous)
//                       x P'^T (B, P' = p * V block scale as a 23-bit integer in three byte rows)
// so the only per-byte work left on the SM is none at all; per TOKEN the
// softmax warps do about 350 instructions per 128 tokens of one KV head.
// The integer products are exact; Q is quantised to 15 bits per block of 32 dims
// (finer than its f16 input) and P' to 23 bits of the stage's largest V scale.
//
// Roles (800 threads): warp 0 TMA producer, warps 1-2 QK issuers (warp 1 owns TMEM), warps 3-4 PV
// issuers, warps 5-20 four softmax groups (thread = token row = TMEM lane), warps 21-24 accumulate
// (thread = head dim = TMEM lane; they also quantise Q at the start and write the
// partials at the end). Every mbarrier wait is bounded; after a timeout the CTA
// stops waiting, drains and frees TMEM, and reports through the error word.
//
// Around that core the same launch can do the rest of a layer's decode step:
//   fused step   the Q preparation normalises and rotates the raw q first, and the CTAs of
//                the last split quantise the new token's K / V rows, store them to the cache
//                and patch them into their last stage (bp_attn_decode_layer);
//   merge        the CTAs of a head group merge its splits themselves, through tagged partials;
//   exchange     final outputs are also stored into every rank's gathered buffer (peer stores).
#include "bp_common.cuh"
#include "bp_ptx.cuh"
#include "bp_norm_quant.cuh"

namespace {

using namespace bp;

constexpr unsigned FULL = 0xffffffffu;
constexpr float NEG_BIG = -1e30f;
constexpr uint32_t UT = 128;                 // tokens per stage = UMMA M
constexpr uint32_t TILE_B = UT * 128;        // int8 tile of one head and stage: 16 KB
constexpr uint32_t U_MAX_STAGES = 8;             // upper bound of K stages and of V slots
constexpr uint32_t NGRP = 4;                      // softmax groups working on different jobs in parallel
constexpr uint32_t MERGE_BAR = 8;                 // named barrier: the merger's accumulate and softmax warps
constexpr uint32_t SHARE_BAR = 9;                 // named barrier: the four accumulate warps combining their shares
constexpr uint32_t FIN_BAR = 6;                   // named barrier: softmax warps arrive, accumulate warps wait
constexpr uint32_t NISS = 2;                     // UMMA issuer warps per kind (QK, PV)
constexpr uint32_t U_FIRST_SM_WARP = 1 + 2 * NISS;  // warp 0 producer, then the issuers
constexpr uint32_t U_THREADS = (U_FIRST_SM_WARP + 4 * NGRP + 4) * 32;
constexpr uint32_t TMEM_COLS = 512;          // per softmax group: D1 (64 columns) and D2 (64 columns)
constexpr uint32_t NO_SLOT = 0xffu;           // px_meet: no meeting in this launch
constexpr uint32_t U_SMEM_BUDGET = 226 * 1024;  // dynamic shared memory; the static part needs the rest of 227 KB

struct UmmaParams {
  const __half* q;
  __half* out;
  float* partials;
  uint32_t* err;
  uint32_t row_base, cur_pos, tps, nk, nv, n_head, qpg;  // nk K stages, nv V slots in shared memory
  float sm_scale_log2;
  // Fused layer step (fused = 1): q is the RAW query; the kernel normalises and rotates it itself
  // (optionally storing the result to q_roped), and the CTAs of the last split quantise the new
  // token's K / V rows (k_cur, v_cur), write them to the cache and patch them into their last stage.
  // Peer exchange (n_px > 0): every final output element is also stored into each rank's gathered
  // buffer (this rank's included) at px_off + head * 128 + dim: an all-gather by peer stores in the
  // epilogue instead of a collective after the kernel. The stores are complete when the grid is;
  // ranks meet afterwards with bp_peer_sync.
  uint32_t n_px, px_off;
  __half* const* px_out;  // in device memory: the parameter block stays small (a larger one costs about 1 % per launch)
  uint32_t merge;       // 1: the CTAs of a head group merge its splits themselves (merge_unit)
  uint2* ll;            // tagged partials [split][head][BP_LL_STRIDE]: (value bits, tag of the launch)
  uint32_t* epochs;     // per head group (grid y): the tag of the last merged launch
  uint32_t fused;
  float eps;
  __half* q_roped;
  const __half *w_q, *w_k, *k_cur, *v_cur, *rope_row;
  float *k_d, *v_d;        // the layer's scale sections
  uint32_t *k_qs, *v_qs;   // the layer's quant sections (as words)
  uint32_t n_kv_head;
  // Bounds of the waits: polls of an mbarrier (and of a meeting counter), polling rounds of the merge
  // (about 0.2 us each). When one runs out the CTA stores a code in *err, stops waiting and winds down.
  uint32_t wait_limit, poll_limit;
  // Rows from fresh_from on may have been written by a launch that is not certainly complete when
  // this kernel's prologue runs (dependent launches): stages that hold such rows are requested
  // only after the dependency wait. UINT32_MAX: every row older than the new token is settled.
  uint32_t fresh_from;
  uint32_t v_pre_all;   // 1: the first round of V tiles is requested during set-up, like the K stages
  // Meeting of the ranks without a kernel of its own (px_meet slot != none; set for layer L >= 1,
  // slot of layer L - 1): once the kernels before this one in the stream are complete (their peer
  // stores have landed by then), one thread of CTA (0, 0) adds one to every rank's counter of that
  // slot; before the grid ends, one thread waits, bounded, until every rank has done so: the
  // consumer's side of layer L - 1's gathered row. Nothing of it lies on this kernel's own path.
  // (Slot and rank are bytes of one word and the counters sit behind one pointer: the parameter
  // block stays small.)
  uint32_t px_meet;           // slot | this rank << 8; slot 0xff = none
  uint32_t* const* px_tab;    // in device memory: [r] rank r's meeting counters [64], [9] this rank's count of meetings per slot
  unsigned long long* dbg;  // optional cycle counters of CTA (0, 0); null in normal use
};

template <uint32_t HPC>
struct ULayout {
  // Two rings. A K stage holds what a job needs first and only briefly: the K tiles of the HPC heads
  // and BOTH scale rows of its 128 tokens; it is released as soon as the softmax group has read S and
  // the scales. A V slot holds one head's V tile, requested when that job's Q K^T is issued and held
  // until its P V has run. A stage that carried K and V together sat in shared memory for the load
  // latency plus the whole job, which is what bounded the stream.
  static constexpr uint32_t SCALE_B = UT * HPC * 16;                   // scale rows of one stage (K or V)
  static constexpr uint32_t KSTAGE_B = HPC * TILE_B + 2 * SCALE_B;     // 20,480 B for HPC = 1
  static constexpr uint32_t VSLOT_B = TILE_B;
  static constexpr uint32_t Q_B = HPC * 2048;                          // Q^T tiles: 16 rows x 128 B per head
  static constexpr uint32_t P_B = NGRP * 4 * 2048;                     // P'^T tiles: one per group x 4 blocks
  static constexpr uint32_t MISC_B = 4096;
  static constexpr uint32_t tail() { return Q_B + P_B + MISC_B; }
  static constexpr uint32_t ring(uint32_t nk, uint32_t nv) { return nk * KSTAGE_B + nv * VSLOT_B; }
  static constexpr uint32_t total(uint32_t nk, uint32_t nv) { return ring(nk, nv) + tail() + 1024; }
};

struct Misc {            // small shared state, lives in the MISC_B region
  float sq[8][4][4];     // Q block scales [head][query head][block] (pre-multiplied by the softmax scale)
  int xchg[NGRP][2][4][8];  // [softmax group][job parity][warp]: 4 score maxima, 4 V-scale maxima
  float info[NGRP][8];      // per group: corr[4], dequantisation factor of P' per block [4]
  float lsum[NGRP][4][4];   // final l per (softmax group, query head, warp)
  float mfin[NGRP][4];
  uint32_t tag;             // the launch's tag, for the softmax warps of a merging CTA
  float xm[4], xl[4], xo[4][32];  // mode-1 merge: the four accumulate warps' shares of a unit
};

__device__ __forceinline__ float s32_to_f32(uint32_t x) {  // exact for |x| < 2^22
  return __int_as_float(static_cast<int>(x) + 0x4B400000) - 12582912.0f;
}
__device__ __forceinline__ int f32_order(float f) {  // monotone map float -> int
  const int b = __float_as_int(f);
  return b >= 0 ? b : b ^ 0x7fffffff;
}
__device__ __forceinline__ float f32_unorder(int k) { return __int_as_float(k >= 0 ? k : k ^ 0x7fffffff); }

// Bounded mbarrier wait shared by every role (one copy of the code: the kernel's instruction
// footprint matters, cold instruction fetches cost more than the waits themselves).
__device__ __noinline__ void cta_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* err,
                                     uint32_t limit) {
  if (*abort_flag) return;
  if (!mbar_wait(smem_u32(bar), parity, limit)) {
    *abort_flag = 1;
    atomicExch(err, 3u);
  }
}

// One final output element: to this rank's output and, with a peer exchange, to every rank's gathered buffer.
__device__ __forceinline__ void put_out(const UmmaParams& p, uint32_t h, uint32_t d, float v) {
  const __half hv = __float2half_rn(v);
  p.out[static_cast<size_t>(h) * BP_HEAD_DIM + d] = hv;
  for (uint32_t r = 0; r < p.n_px; r++) p.px_out[r][p.px_off + static_cast<size_t>(h) * BP_HEAD_DIM + d] = hv;
}

// Merge of the splits (attention_merge.wgsl:70-130) inside the launch. CTAs publish their partial
// (o[128], m, l) per query head as (value, tag) pairs, the tag naming this launch (the head group's
// epoch + 1): one 8-byte store per value and no fence, because a reader that sees the tag sees the
// value stored with it. The output of a head group is cut into units of 32 elements (one query head
// x one quarter of the dims), and a unit is merged by one warp that has its own CTA's part at hand
// and polls the other splits' parts: lane k reads (m, l) of the k-th other split, the weights travel
// by shuffle, and the loads of a round are all in flight together. Who merges which unit (the mode is
// chosen per launch: up to 16 splits of up to 4 stages take mode 2):
//   mode 2 (up to 16 splits of up to 4 stages: launches bound by latency)  one CTA per head group, a full-length split, merges all units with its
//           softmax warps; its own partial stays in shared memory, so when it is the last to finish
//           the merge ends one L2 round trip later. One SM can only keep so many loads in flight:
//           with 16 units x 17 splits this took 2.5 us per polling round.
//   mode 1 (more splits)      unit u belongs to split u mod n_splits, whose accumulate warp of that
//           quarter holds the CTA's part in registers: one more hop (the slowest split's stores must
//           reach the others), but no SM is a bottleneck.
// One warp; `split` is the caller's, (a_own, m_own, l_own) its partial of head h at dim d.
template <uint32_t MERGE_W>  // partials of one element in flight per polling round
__device__ __forceinline__ void merge_unit(const UmmaParams& p, uint32_t lane, uint32_t n_splits, uint32_t split, uint32_t h,
                                           uint32_t d, float a_own, float m_own, float l_own, uint32_t tag,
                                           volatile uint32_t* abort_flag) {
  const uint32_t n_oth = n_splits - 1;  // the i-th other split is i for i < split, else i + 1
  const uint32_t sstride = p.n_head * BP_LL_STRIDE;  // 32-bit index arithmetic: the scratch has < 2^20 pairs
  const uint2* base = p.ll + h * BP_LL_STRIDE;
  float m_run = m_own, l_run = l_own, o_run = a_own;
  for (uint32_t c0 = 0; c0 < n_oth; c0 += 32) {
    const uint32_t nc = min(32u, n_oth - c0);
    float e_k = 0.f;
    for (uint32_t v0 = 0; v0 < nc; v0 += MERGE_W) {
      uint2 v[MERGE_W];
      uint2 mm, ls;
      for (uint32_t spin = 0;; spin++) {
        // Straight-line loads (indices clamped to the chunk's last split instead of branching around
        // a load): every load of the round is issued before the first is used. `first` is made opaque
        // so that the addresses are formed here, next to their loads: hoisted out of the polling loop
        // they would take two registers each and spill the loaded values, and a load whose result is
        // spilled is waited for at once.
        uint32_t first = c0;
        asm volatile("" : "+r"(first));
        const uint32_t i_ml = first + min(lane, nc - 1);
        const uint2* ml = base + (i_ml + (i_ml >= split ? 1u : 0u)) * sstride;
        mm = ld_tagged(ml + 128);
        ls = ld_tagged(ml + 129);
        const uint32_t k_max = nc - 1 - v0;
#pragma unroll
        for (uint32_t k = 0; k < MERGE_W; k++) {
          const uint32_t i = first + v0 + min(k, k_max);
          v[k] = ld_tagged(base + (i + (i >= split ? 1u : 0u)) * sstride + d);
        }
        bool ok = mm.y == tag && ls.y == tag;
#pragma unroll
        for (uint32_t k = 0; k < MERGE_W; k++) ok = ok && v[k].y == tag;
        if (__all_sync(FULL, ok)) break;
        const bool give_up = *abort_flag != 0 || spin >= p.poll_limit;
        if (__any_sync(FULL, give_up)) {  // warp-uniform exit: the shuffles below need every lane
          if (*abort_flag == 0) {
            *abort_flag = 1;
            atomicExch(p.err, 3u);
          }
          break;
        }
        __nanosleep(spin < 4 ? 64u : 256u);
      }
      if (v0 == 0) {
        const float m_k = lane < nc ? __uint_as_float(mm.x) : NEG_BIG;
        float m_c = m_k;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) m_c = fmaxf(m_c, __shfl_xor_sync(FULL, m_c, off));
        const float m_new = fmaxf(m_run, m_c);
        e_k = lane < nc ? ex2(m_k - m_new) : 0.f;
        float l_c = lane < nc ? __uint_as_float(ls.x) * e_k : 0.f;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) l_c += __shfl_xor_sync(FULL, l_c, off);
        const float scale = ex2(m_run - m_new);
        o_run *= scale;
        l_run = fmaf(l_run, scale, l_c);
        m_run = m_new;
      }
#pragma unroll
      for (uint32_t k = 0; k < MERGE_W; k++) {
        const float e = __shfl_sync(FULL, e_k, (v0 + k) & 31u);
        o_run = fmaf(__uint_as_float(v[k].x), v0 + k < nc ? e : 0.f, o_run);
      }
    }
  }
  put_out(p, h, d, o_run * (1.0f / l_run));
}

// A share of a unit's merge, for mode 1: the other splits first, first + stride, ... (`count` of
// them, numbered like merge_unit's: the i-th other split is i for i < split, else i + 1) are folded
// into the running (m, l, o) of this warp; no output. The four accumulate warps of a CTA take a
// quarter of the other splits each, so that a unit's merge is ONE polling round of at most MERGE_W
// partials per lane for up to 4 * MERGE_W + 1 splits (two rounds by one warp took 0.6 us longer at
// 18 splits, five rounds 2.5 us longer at 37), and combine their shares through shared memory.
template <uint32_t MERGE_W>
__device__ __forceinline__ void merge_part(const UmmaParams& p, uint32_t lane, uint32_t first, uint32_t stride, uint32_t count,
                                           uint32_t split, uint32_t h, uint32_t d, uint32_t tag, volatile uint32_t* abort_flag,
                                           float& m_run, float& l_run, float& o_run) {
  const uint32_t sstride = p.n_head * BP_LL_STRIDE;
  const uint2* base = p.ll + h * BP_LL_STRIDE;
  for (uint32_t c0 = 0; c0 < count; c0 += 32) {
    const uint32_t nc = min(32u, count - c0);
    float e_k = 0.f;
    for (uint32_t v0 = 0; v0 < nc; v0 += MERGE_W) {
      uint2 v[MERGE_W];
      uint2 mm, ls;
      for (uint32_t spin = 0;; spin++) {
        uint32_t c00 = c0;
        asm volatile("" : "+r"(c00));  // addresses are formed next to their loads (see merge_unit)
        const uint32_t i_ml = first + (c00 + min(lane, nc - 1)) * stride;
        const uint2* ml = base + (i_ml + (i_ml >= split ? 1u : 0u)) * sstride;
        mm = ld_tagged(ml + 128);
        ls = ld_tagged(ml + 129);
        const uint32_t k_max = nc - 1 - v0;
#pragma unroll
        for (uint32_t k = 0; k < MERGE_W; k++) {
          const uint32_t i = first + (c00 + v0 + min(k, k_max)) * stride;
          v[k] = ld_tagged(base + (i + (i >= split ? 1u : 0u)) * sstride + d);
        }
        bool ok = mm.y == tag && ls.y == tag;
#pragma unroll
        for (uint32_t k = 0; k < MERGE_W; k++) ok = ok && v[k].y == tag;
        if (__all_sync(FULL, ok)) break;
        const bool give_up = *abort_flag != 0 || spin >= p.poll_limit;
        if (__any_sync(FULL, give_up)) {
          if (*abort_flag == 0) {
            *abort_flag = 1;
            atomicExch(p.err, 3u);
          }
          break;
        }
        __nanosleep(spin < 4 ? 64u : 256u);
      }
      if (v0 == 0) {
        const float m_k = lane < nc ? __uint_as_float(mm.x) : NEG_BIG;
        float m_c = m_k;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) m_c = fmaxf(m_c, __shfl_xor_sync(FULL, m_c, off));
        const float m_new = fmaxf(m_run, m_c);
        e_k = lane < nc ? ex2(m_k - m_new) : 0.f;
        float l_c = lane < nc ? __uint_as_float(ls.x) * e_k : 0.f;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) l_c += __shfl_xor_sync(FULL, l_c, off);
        const float scale = ex2(m_run - m_new);
        o_run *= scale;
        l_run = fmaf(l_run, scale, l_c);
        m_run = m_new;
      }
#pragma unroll
      for (uint32_t k = 0; k < MERGE_W; k++) {
        const float e = __shfl_sync(FULL, e_k, (v0 + k) & 31u);
        o_run = fmaf(__uint_as_float(v[k].x), v0 + k < nc ? e : 0.f, o_run);
      }
    }
  }
}

// MODE: which merge code (see merge_unit) the instance carries. 1: mode 1 only, launched for long
// launches; 3: both, the mode chosen at run time, launched for short ones. These kernels move by a
// few percent with the sheer amount of code around their loops; measured on one GPU, per call at
// ctx 4096 / 32768: both codes in one kernel 8.09 / 20.45 us, one instance per mode 8.29 / 19.90 us.
// Hence this pairing.
template <uint32_t HPC, uint32_t MODE>
__global__ void __launch_bounds__(U_THREADS, 1)
decode_umma_kernel(const CUtensorMap* __restrict__ maps, const __grid_constant__ UmmaParams p) {
  // tensor maps in device memory (written by the host before any launch that reads them): K quants, K scales, V quants, V scales
  const CUtensorMap &map_kq = maps[0], &map_kd = maps[1], &map_vq = maps[2], &map_vd = maps[3];
  using L = ULayout<HPC>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[U_MAX_STAGES], k_empty[U_MAX_STAGES], v_full[U_MAX_STAGES], v_empty[U_MAX_STAGES];
  __shared__ __align__(8) uint64_t s_ready[4], s_free[4], p_ready[4], p_free[4], o_ready[4], o_free[4];
  __shared__ __align__(8) uint64_t q_bar, patched_bar, patched_v;
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile uint32_t abort_s;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned long long t_entry_ns = 0;
  if (p.dbg != nullptr && threadIdx.x == 0) {
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_entry_ns));
    atomicMin(&p.dbg[32], t_entry_ns);
  }
  // Programmatic dependent launch: the next kernel in the stream may be scheduled already (it
  // waits for this grid's completion itself). This grid waits (pdl_wait) before it touches what
  // the previous kernels produce (q, the newest cache row) and before its own global writes.
  if (threadIdx.x == 0) pdl_launch_dependents();
  const uint32_t ns = p.nk, nv = p.nv;  // ns: K stages
  const uint32_t g0 = blockIdx.y * HPC;
  const uint32_t split = blockIdx.x, n_splits = gridDim.x;
  const uint32_t tok_begin = split * p.tps;
  const uint32_t tok_end = min(tok_begin + p.tps, p.cur_pos);
  const uint32_t n_iter = (tok_end - tok_begin + UT - 1) / UT;
  const uint32_t n_jobs = n_iter * HPC;
  // V tiles requested during set-up: the first round (their slots are empty anyway, and the first
  // jobs' P V should not wait for a load that starts only when their Q K^T is issued)
  const uint32_t v_pre = p.v_pre_all ? (n_jobs < p.nv ? n_jobs : p.nv) : (n_jobs <= p.nv ? n_jobs : 0);

  const uint32_t ring_b = ns * L::KSTAGE_B + nv * L::VSLOT_B;  // K ring, then V ring: both multiples of 1024
  const uint32_t v_ring = smem_base + ns * L::KSTAGE_B;
  const uint32_t q_tiles = smem_base + ring_b;
  const uint32_t p_tiles = q_tiles + L::Q_B;
  Misc* misc = reinterpret_cast<Misc*>(smem_gen + ring_b + L::Q_B + L::P_B);

  // One K stage: K tiles of the HPC heads and both scale rows, 128 tokens from `it * UT`.
  auto issue_stage = [&](uint32_t it, uint32_t s) {
    const uint32_t bar = smem_u32(&full_bar[s]);
    const uint32_t stage = smem_base + s * L::KSTAGE_B;
    const int row = static_cast<int>(p.row_base + tok_begin + it * UT);
    // Older rows were written by launches that have long completed; rows from fresh_from on (the
    // newest token's, when a separate kernel wrote it just before this one) only by the time the
    // dependency wait returns. In the fused step this CTA writes the newest row itself and patches
    // it into the stage after the load.
    if (tok_begin + (it + 1) * UT > p.fresh_from) pdl_wait();
    mbar_arrive_expect_tx(bar, L::KSTAGE_B);
    tma_load_2d(stage + HPC * TILE_B, &map_kd, bar, static_cast<int>(g0 * 16), row);
    tma_load_2d(stage + HPC * TILE_B + L::SCALE_B, &map_vd, bar, static_cast<int>(g0 * 16), row);
    for (uint32_t g = 0; g < HPC; g++) tma_load_3d(stage + g * TILE_B, &map_kq, bar, 0, static_cast<int>(g0 + g), row);
  };
  // The V tile of job j (stage j / HPC, head j % HPC) into V slot j % nv.
  auto issue_v = [&](uint32_t j) {
    const uint32_t v = j % nv, bar = smem_u32(&v_full[v]);
    const int row = static_cast<int>(p.row_base + tok_begin + (j / HPC) * UT);
    mbar_arrive_expect_tx(bar, L::VSLOT_B);
    tma_load_3d(v_ring + v * L::VSLOT_B, &map_vq, bar, 0, static_cast<int>(g0 + j % HPC), row);
  };

  // ---- set-up: barriers, TMEM, zeroed operand tiles, quantised Q ----
  if (threadIdx.x == 0) {
    // Thread 0 initialises the first stage's barrier and requests that stage at once: its latency
    // (descriptor fetch + DRAM) is the longest item on the critical path of a CTA that starts late.
    // It requests the rest of the first round after the CTA-wide set-up barrier (measured: initialising
    // all of the ring's barriers and issuing the whole round first held every other warp at that
    // barrier for 0.9 us). The other barriers are initialised by the lanes of warps 2 and 3.
    abort_s = 0;
    mbar_init(smem_u32(&full_bar[0]), 1);
    fence_barrier_init();
    prefetch_tensormap(&map_kq);
    prefetch_tensormap(&map_kd);
    prefetch_tensormap(&map_vd);
    issue_stage(0, 0);
    prefetch_tensormap(&map_vq);
  } else if (warp == 3) {
    if (lane >= 1 && lane < ns) mbar_init(smem_u32(&full_bar[lane]), 1);
    if (lane >= 8 && lane - 8 < nv) mbar_init(smem_u32(&v_full[lane - 8]), 1);
    fence_barrier_init();
  } else if (warp == 2) {
    if (lane < 4) {
      mbar_init(smem_u32(&s_ready[lane]), 1);
      mbar_init(smem_u32(&p_free[lane]), 1);
    } else if (lane < 8) {
      mbar_init(smem_u32(&s_free[lane - 4]), 4);
      mbar_init(smem_u32(&o_ready[lane - 4]), 1);
    } else if (lane < 12) {
      mbar_init(smem_u32(&p_ready[lane - 8]), 4);
      mbar_init(smem_u32(&o_free[lane - 8]), 4);
    } else if (lane == 12) {
      mbar_init(smem_u32(&q_bar), 4);  // the four accumulate warps prepare Q
      mbar_init(smem_u32(&patched_bar), 1);
      mbar_init(smem_u32(&patched_v), 1);
    } else if (lane < 21) {
      if (lane - 13 < ns) mbar_init(smem_u32(&k_empty[lane - 13]), HPC * 4);  // the 4 warps of each job's softmax group
    } else if (lane < 29) {
      if (lane - 21 < nv) mbar_init(smem_u32(&v_empty[lane - 21]), 1);  // the tcgen05.commit behind the job's P V
    }
    fence_barrier_init();
  }
  {
    uint4* z = reinterpret_cast<uint4*>(smem_gen + ring_b);
    for (uint32_t i = threadIdx.x; i < (L::Q_B + L::P_B) / 16; i += U_THREADS) z[i] = make_uint4(0, 0, 0, 0);
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  // Q of head (g, hq), block b: 15-bit integers = 128 * hi + lo against the block's absmax; hi bytes
  // go to row hq, lo bytes to row 4 + hq of the head's Q^T tile (swizzled 128-byte rows). Done by the
  // accumulate warps while the producer already streams the first stages; the QK issuers wait on q_bar.
  uint32_t epoch = 0;  // accumulate warps: the head group's epoch, read once the previous launch is complete
  // In-kernel merge of the splits (merge_unit): 0 none, 1 spread over the CTAs, 2 by one CTA of the head
  // group: the last split when it is as long as the others (with the fused step it has the new row's
  // work on top, finishes last, and its partial never leaves the SM), else the first.
  // Evaluated where it is used, in the epilogues, so that nothing of it is held in registers through
  // the main loops.
  auto merge_plan = [&](uint32_t& mode, bool& is_merger) {
    mode = p.merge && n_splits > 1 ? (MODE == 1 ? 1u : (n_splits <= 16 && p.tps <= 4 * UT ? 2u : 1u)) : 0u;
    const uint32_t last_stages = (p.cur_pos - (n_splits - 1) * p.tps + UT - 1) / UT;
    const uint32_t merger_split = last_stages == p.tps / UT ? n_splits - 1 : 0;
    is_merger = mode == 2 && split == merger_split;
  };
  auto own_part = [&]() {  // the merger's own o: over the dead P' tiles
    return reinterpret_cast<float*>(smem_gen + ring_b + L::Q_B);
  };
  // (m, l) of query head hq of head g over this CTA's tokens: the softmax groups' values, merged
  auto head_ml = [&](uint32_t g, uint32_t hq, float& m, float& l) {
    m = NEG_BIG;
    for (uint32_t w = g; w < NGRP; w += HPC) m = fmaxf(m, misc->mfin[w][hq]);
    l = 0.f;
    for (uint32_t w = g; w < NGRP; w += HPC) {
      const float4 ls = *reinterpret_cast<const float4*>(misc->lsum[w][hq]);
      l += ((ls.x + ls.y) + (ls.z + ls.w)) * ex2(misc->mfin[w][hq] - m);
    }
  };
  auto prepare_q = [&](uint32_t aw) {  // aw = 0..3: the calling accumulate warp; warp aw takes heads aw, aw + 4, ...
    // The norm weight and this position's RoPE row are constants: bring them in while the previous
    // kernel still runs (the RoPE row of a new position is not in L2 yet).
    if (p.fused && aw == 0) {
      prefetch_l2(p.w_q + 4 * lane);
      prefetch_l2(p.rope_row + 4 * lane);
      prefetch_l2(p.w_k + 4 * lane);
    }
    pdl_wait();  // q is written by the kernel before this one
    if (p.merge && n_splits > 1) epoch = ld_relaxed_u32(p.epochs + blockIdx.y);  // used in the epilogue

    // lane l holds dims 4l .. 4l+3 of one head: a Q8_0 block is 8 lanes. One 8-byte load, three
    // shuffles for the block maximum, two 4-byte stores: short straight-line code, because this sits
    // on the critical path of every launch (the first Q K^T waits for it) and runs cold.
    for (uint32_t hl = aw; hl < HPC * p.qpg; hl += 4) {
      const uint32_t g = hl / p.qpg, hq = hl % p.qpg, b = lane >> 3;
      const size_t q_off = (static_cast<size_t>(g0 + g) * p.qpg + hq) * BP_HEAD_DIM;
      uint2 raw;
      if (p.fused) {
        // q_norm_rope of this head, rounded to f16 exactly as the stand-alone kernel stores it
        const Rot4 r = norm_rope(p.q + q_off, p.w_q, p.rope_row, p.eps, static_cast<int>(lane));
        const __half2 lo2 = __floats2half2_rn(r.v[0], r.v[1]), hi2 = __floats2half2_rn(r.v[2], r.v[3]);
        raw.x = *reinterpret_cast<const uint32_t*>(&lo2);
        raw.y = *reinterpret_cast<const uint32_t*>(&hi2);
        if (p.q_roped != nullptr && split == 0) *reinterpret_cast<uint2*>(p.q_roped + q_off + 4 * lane) = raw;
      } else {
        raw = *reinterpret_cast<const uint2*>(p.q + q_off + 4 * lane);
      }
      const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
      const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
      const float f[4] = {f01.x, f01.y, f23.x, f23.y};
      float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
      for (int off = 1; off <= 4; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(FULL, amax, off));
      const float sq = amax / 16383.0f, inv = amax > 0.f ? 16383.0f / amax : 0.f;
      uint32_t hi = 0, lo = 0;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int q = __float2int_rn(f[i] * inv);
        hi |= (static_cast<uint32_t>(q >> 7) & 0xffu) << (8 * i);
        lo |= (static_cast<uint32_t>(q) & 0x7fu) << (8 * i);
      }
      uint8_t* tile = smem_gen + ring_b + g * 2048;
      *reinterpret_cast<uint32_t*>(tile + swz128(hq * 128 + 4 * lane)) = hi;
      *reinterpret_cast<uint32_t*>(tile + swz128((4 + hq) * 128 + 4 * lane)) = lo;
      if ((lane & 7) == 0) misc->sq[g][hq][b] = sq * p.sm_scale_log2;
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&q_bar));
  };

  // Jobs: job j = (stage it, head g) with j = it * HPC + g. NGRP softmax groups
  // work in parallel; job j belongs to group w = j % NGRP, so a group always
  // sees the same head (w % HPC). Each group owns one D1, one D2 and one P'
  // buffer; its k-th job (k = j / NGRP) completes phase k of its barriers.
  // A wait that degrades to a no-op once any warp of the CTA has timed out.
  auto wait = [&](uint64_t* bar, uint32_t parity) { cta_wait(bar, parity, &abort_s, p.err, p.wait_limit); };
  auto put = [&](uint32_t h, uint32_t d, float v) { put_out(p, h, d, v); };
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      // the rest of the first round (stage 0 was requested during set-up)
      const uint32_t n_pre = n_iter < ns ? n_iter : ns;
      for (uint32_t it = 1; it < n_pre; it++) issue_stage(it, it);
      // a launch whose V tiles all fit at once requests them here too (it should not wait for them);
      // otherwise the Q K^T issuers request every V tile when its job starts
      for (uint32_t j = 0; j < v_pre; j++) issue_v(j);
    }
    __syncwarp();
    // Fused step, last split: the whole warp first quantises the new token's K / V rows of this
    // CTA's heads (the arithmetic of kv_writeback_kernel) and stores them to the cache.
    const bool new_row = p.fused && tok_end == p.cur_pos;
    uint32_t pk[HPC], pv[HPC];
    float dk[HPC], dv[HPC];
    if (new_row) {
      pdl_wait();  // k_cur / v_cur come from the kernel before this one
      const uint32_t pos = p.cur_pos - 1, kv_dim = p.n_kv_head * BP_HEAD_DIM;
#pragma unroll
      for (uint32_t g = 0; g < HPC; g++) {
        const size_t src = static_cast<size_t>(g0 + g) * BP_HEAD_DIM;
        const Rot4 kp = norm_rope(p.k_cur + src, p.w_k, p.rope_row, p.eps, static_cast<int>(lane));
        const uint2 vr = *reinterpret_cast<const uint2*>(p.v_cur + src + 4 * lane);
        const float2 v01 = __half22float2(*reinterpret_cast<const __half2*>(&vr.x));
        const float2 v23 = __half22float2(*reinterpret_cast<const __half2*>(&vr.y));
        const float vraw[4] = {v01.x, v01.y, v23.x, v23.y};
        pk[g] = quant4(kp.v, &dk[g]);
        pv[g] = quant4(vraw, &dv[g]);
        const size_t word = (static_cast<size_t>(pos) * kv_dim + src) / 4 + lane;
        p.k_qs[word] = pk[g];
        p.v_qs[word] = pv[g];
        if ((lane & 7) == 0) {
          const size_t blk = static_cast<size_t>(pos) * (kv_dim / BP_QK8) + (g0 + g) * 4 + (lane >> 3);
          p.k_d[blk] = dk[g];
          p.v_d[blk] = dv[g];
        }
      }
    }
    if (lane == 0) {
      uint32_t s = 0, use = 1;
      for (uint32_t it = ns; it < n_iter; it++) {
        wait(&k_empty[s], (use - 1) & 1);
        if (abort_s) break;
        issue_stage(it, s);
        if (++s == ns) { s = 0; use++; }
      }
    }
    __syncwarp();
    if (new_row) {
      // The last K stage and the last jobs' V slots were loaded with whatever the cache row held
      // before: once they have landed, the fresh row replaces it in shared memory (swizzled tile
      // rows, scale rows). K side first (the last Q K^T waits for it and only then requests its V
      // tile), V side when that tile is there (the last P V waits for it).
      const uint32_t it_last = n_iter - 1, s_last = it_last % ns;
      wait(&full_bar[s_last], (it_last / ns) & 1);
      const uint32_t r = p.cur_pos - 1 - (tok_begin + it_last * UT);
      uint8_t* stage = smem_gen + s_last * L::KSTAGE_B;
#pragma unroll
      for (uint32_t g = 0; g < HPC; g++) {
        *reinterpret_cast<uint32_t*>(stage + g * TILE_B + swz128(r * 128 + 4 * lane)) = pk[g];
        if ((lane & 7) == 0) {
          *reinterpret_cast<float*>(stage + HPC * TILE_B + (r * HPC + g) * 16 + 4 * (lane >> 3)) = dk[g];
          *reinterpret_cast<float*>(stage + HPC * TILE_B + L::SCALE_B + (r * HPC + g) * 16 + 4 * (lane >> 3)) = dv[g];
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&patched_bar));
#pragma unroll
      for (uint32_t g = 0; g < HPC; g++) {
        const uint32_t j = it_last * HPC + g, v = j % nv;
        wait(&v_full[v], (j / nv) & 1);
        *reinterpret_cast<uint32_t*>(smem_gen + ns * L::KSTAGE_B + v * L::VSLOT_B + swz128(r * 128 + 4 * lane)) = pv[g];
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&patched_v));
    }
    // Consumer side of the previous layer's meeting: one thread of the grid, idle by now, waits until
    // every rank has signalled that slot (all ranks' stores into this rank's gathered row have landed).
    const uint32_t px_slot = p.px_meet & 0xffu;
    if (px_slot != NO_SLOT && blockIdx.x == 0 && blockIdx.y == 0 && lane == 0) {
      pdl_wait();  // the meeting count was advanced by an earlier kernel
      uint32_t* epoch = p.px_tab[9] + px_slot;
      const uint32_t* flag = p.px_tab[(p.px_meet >> 8) & 0xffu] + px_slot;
      const uint32_t target = (*epoch + 1u) * p.n_px;
      bool ok = false;
      for (uint32_t i = 0; i < p.wait_limit && !ok; i++) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        ok = static_cast<int32_t>(v - target) >= 0;
        if (!ok) __nanosleep(64);
      }
      if (!ok) atomicExch(p.err, 6u);
      *epoch += 1u;
    }
  } else if (warp < 1 + NISS) {
    // ---------------- QK issuers: S^T[token][(block, byte row, head)] = K tile x Q^T ----------------
    // One UMMA per Q8_0 block (K = 32 dims). Issuer q takes the jobs j = q (mod NISS); issuing is
    // serial scalar work (about 100 instructions per job), hence more than one issuer.
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = umma_idesc(2, 1, 1, 0, 0, 128, 16);  // s32 = s8 (K-major) x s8
      const uint64_t dbase = umma_desc_sw128(0, 16, 1024);               // + (shared address >> 4)
      const uint32_t q = warp - 1;
      wait(&q_bar, 0);
      for (uint32_t j = q; j < n_jobs; j += NISS) {
        const uint32_t it = j / HPC, g = j % HPC, bi = j % NGRP, k = j / NGRP, s = it % ns, use = it / ns;
        wait(&full_bar[s], use & 1);
        if (p.fused && tok_end == p.cur_pos && it == n_iter - 1) wait(&patched_bar, 0);  // the new row is in place
        if (k > 0) wait(&s_free[bi], (k - 1) & 1);
        tc_fence_after();
        const uint64_t ka = dbase + ((smem_base + s * L::KSTAGE_B + g * TILE_B) >> 4);
        const uint64_t qb = dbase + ((q_tiles + g * 2048) >> 4);
#pragma unroll
        for (uint32_t b = 0; b < 4; b++) umma_i8(tmem + bi * 64 + 16 * b, ka + 2 * b, qb + 2 * b, IDESC_QK, 0u);
        umma_commit(smem_u32(&s_ready[bi]));
        // Now request the job's V tile (unless set-up did): it arrives while the softmax group works,
        // and its slot is occupied for one load latency instead of the load latency plus the whole job.
        if (j >= v_pre) {
          if (j >= nv) wait(&v_empty[j % nv], (j / nv - 1) & 1);
          if (!abort_s) issue_v(j);
        }
      }
    }
  } else if (warp < 1 + 2 * NISS) {
    // ---------------- PV issuers: O^T[dim][(block, byte row, head)] (+)= V tile x P'^T ----------------
    // The four blocks' P' tiles are 16 consecutive rows each of one 64-row K-major operand, so one
    // N = 64 UMMA per 32 tokens serves all of them and the V tile is read once; only the
    // (dims of block b) x (columns of block b) part of the result is used.
    if (lane == 0) {
      constexpr uint32_t IDESC_PV = umma_idesc(2, 1, 0, 1, 0, 128, 64);  // s32 += s8 (MN-major) x u8
      const uint64_t dbase = umma_desc_sw128(0, 16, 1024);
      const uint32_t q = warp - 1 - NISS;
      for (uint32_t j = q; j < n_jobs; j += NISS) {
        const uint32_t it = j / HPC, bi = j % NGRP, k = j / NGRP;
        const uint32_t v = j % nv;
        wait(&v_full[v], (j / nv) & 1);
        if (p.fused && tok_end == p.cur_pos && it == n_iter - 1) wait(&patched_v, 0);  // the new row is in place
        wait(&p_ready[bi], k & 1);
        if (k > 0) wait(&o_free[bi], (k - 1) & 1);
        tc_fence_after();
        const uint64_t va = dbase + ((v_ring + v * L::VSLOT_B) >> 4);
        const uint64_t pb = dbase + ((p_tiles + bi * 4 * 2048) >> 4);
#pragma unroll
        for (uint32_t kk = 0; kk < 4; kk++)
          umma_i8(tmem + NGRP * 64 + bi * 64, va + kk * (32 * 128 >> 4), pb + 2 * kk, IDESC_PV, kk);
        umma_commit(smem_u32(&o_ready[bi]));
        umma_commit(smem_u32(&p_free[bi]));
        umma_commit(smem_u32(&v_empty[v]));  // the V slot is free once this P V has run
      }
    }
  }
  else if (warp < U_FIRST_SM_WARP + 4 * NGRP) {
    // ---------------- softmax group w: thread = token row ----------------
    const uint32_t w = (warp - U_FIRST_SM_WARP) >> 2;  // four consecutive warps per group
    const uint32_t quad = warp & 3, t = quad * 32 + lane;
    const uint32_t lane_addr = (quad * 32) << 16;
    float m_run[4], l_part[4];
#pragma unroll
    for (int h = 0; h < 4; h++) { m_run[h] = NEG_BIG; l_part[h] = 0.f; }
    // Producer side of the previous layer's meeting, by a warp that has nothing to do until Q is ready:
    // once everything before this kernel in the stream is complete (the previous layer's peer stores
    // included), tell every rank.
    if ((p.px_meet & 0xffu) != NO_SLOT && blockIdx.x == 0 && blockIdx.y == 0 && warp == U_FIRST_SM_WARP && lane < p.n_px) {
      pdl_wait();
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.px_tab[lane] + (p.px_meet & 0xffu)), "r"(1u) : "memory");
    }
    wait(&q_bar, 0);  // the Q block scales in misc->sq are written by prepare_q

    for (uint32_t j = w; j < n_jobs; j += NGRP) {
      const uint32_t it = j / HPC, g = j % HPC, bi = w, k = j / NGRP;
      const uint8_t* stage = smem_gen + (it % ns) * L::KSTAGE_B;
      const bool valid = tok_begin + it * UT + t < tok_end;
      wait(&s_ready[bi], k & 1);
      tc_fence_after();
      uint32_t d[4][8];
#pragma unroll
      for (uint32_t b = 0; b < 4; b++) tmem_ld8(tmem + lane_addr + bi * 64 + 16 * b, d[b]);
      tmem_ld_wait();
      const float4 sk = *reinterpret_cast<const float4*>(stage + HPC * TILE_B + (t * HPC + g) * 16);
      float4 sv = *reinterpret_cast<const float4*>(stage + HPC * TILE_B + L::SCALE_B + (t * HPC + g) * 16);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&s_free[bi]));
        mbar_arrive(smem_u32(&k_empty[it % ns]));  // S and the scale rows are in registers: the K stage is done with
      }

      const float skb[4] = {sk.x, sk.y, sk.z, sk.w};
      float sc[4];
#pragma unroll
      for (int h = 0; h < 4; h++) {
        const float4 sq4 = *reinterpret_cast<const float4*>(&misc->sq[g][h][0]);
        const float sqb[4] = {sq4.x, sq4.y, sq4.z, sq4.w};
        float acc = 0.f;
#pragma unroll
        for (int b = 0; b < 4; b++) {
          const float dot = fmaf(s32_to_f32(d[b][h]), 128.0f, s32_to_f32(d[b][4 + h]));
          acc = fmaf(dot, skb[b] * sqb[b], acc);
        }
        sc[h] = valid ? acc : NEG_BIG;
      }
      if (!valid) sv = make_float4(0.f, 0.f, 0.f, 0.f);
      const float svb[4] = {sv.x, sv.y, sv.z, sv.w};

      // maxima over the 128 tokens of the stage: 4 score maxima, 4 V-scale maxima
      int red[8];
#pragma unroll
      for (int h = 0; h < 4; h++) red[h] = __reduce_max_sync(FULL, f32_order(sc[h]));
#pragma unroll
      for (int b = 0; b < 4; b++) red[4 + b] = static_cast<int>(__reduce_max_sync(FULL, __float_as_uint(svb[b])));
      if (lane == 0) {
        int4* dst = reinterpret_cast<int4*>(misc->xchg[w][k & 1][quad]);
        dst[0] = make_int4(red[0], red[1], red[2], red[3]);
        dst[1] = make_int4(red[4], red[5], red[6], red[7]);
      }
      named_bar_sync(1 + w, 128);
#pragma unroll
      for (int ww = 0; ww < 4; ww++) {
        const int4* src = reinterpret_cast<const int4*>(misc->xchg[w][k & 1][ww]);
        const int4 a = src[0], c = src[1];
        red[0] = max(red[0], a.x); red[1] = max(red[1], a.y); red[2] = max(red[2], a.z); red[3] = max(red[3], a.w);
        red[4] = max(red[4], c.x); red[5] = max(red[5], c.y); red[6] = max(red[6], c.z); red[7] = max(red[7], c.w);
      }
      float pj[4], corr[4];
#pragma unroll
      for (int h = 0; h < 4; h++) {
        const float m_new = fmaxf(m_run[h], f32_unorder(red[h]));
        corr[h] = ex2(m_run[h] - m_new);
        pj[h] = ex2(sc[h] - m_new);
        l_part[h] = l_part[h] * corr[h] + pj[h];
        m_run[h] = m_new;
      }
      float qscale[4], deq[4];
#pragma unroll
      for (int b = 0; b < 4; b++) {
        const float vmax = __int_as_float(red[4 + b]);
        qscale[b] = vmax > 0.f ? 8388607.0f / vmax : 0.f;
        deq[b] = vmax * (1.0f / 8388607.0f);
      }
      // the group's P' buffer and info slot are free once its previous job has been consumed
      if (k > 0) {
        wait(&p_free[bi], (k - 1) & 1);
        wait(&o_free[bi], (k - 1) & 1);
      }
      if (t == 0) {
        *reinterpret_cast<float4*>(&misc->info[bi][0]) = make_float4(corr[0], corr[1], corr[2], corr[3]);
        *reinterpret_cast<float4*>(&misc->info[bi][4]) = make_float4(deq[0], deq[1], deq[2], deq[3]);
      }
      // P'[h][b] = p[h] * sV[b] as a 23-bit integer: the low three bytes of (x * qscale + 2^23).
      // Byte rows of block b's tile: hi -> row h, mid -> row 4 + h, lo -> row 8 + h; this token's
      // column inside a swizzled row n is t ^ ((n & 7) << 4).
      uint8_t* pt = smem_gen + ring_b + L::Q_B + bi * 4 * 2048;
#pragma unroll
      for (int b = 0; b < 4; b++) {
        uint8_t* tile = pt + b * 2048;
#pragma unroll
        for (int h = 0; h < 4; h++) {
          const uint32_t bits = __float_as_uint(fmaf(pj[h] * svb[b], qscale[b], 8388608.0f));
          tile[h * 128 + (t ^ (h << 4))] = static_cast<uint8_t>(bits >> 16);
          tile[(4 + h) * 128 + (t ^ ((4 + h) << 4))] = static_cast<uint8_t>(bits >> 8);
          tile[(8 + h) * 128 + (t ^ (h << 4))] = static_cast<uint8_t>(bits);
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_ready[bi]));
    }
    // ---- l of every query head of this group: sum over the 128 token rows ----
#pragma unroll
    for (int h = 0; h < 4; h++) {
      float l = l_part[h];
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) l += __shfl_xor_sync(FULL, l, off);
      if (lane == 0) misc->lsum[w][h][quad] = l;
      if (t == 0) misc->mfin[w][h] = m_run[h];
    }
    __threadfence_block();
    named_bar_arrive(FIN_BAR, 128 * NGRP + 128);  // the accumulate warps merge the groups
  } else {
    // ---------------- accumulate: thread = head dim ----------------
    prepare_q(warp - (U_FIRST_SM_WARP + 4 * NGRP));
    const uint32_t quad = warp & 3, dim = quad * 32 + lane;
    const uint32_t lane_addr = (quad * 32) << 16;
    float o[NGRP][4];
#pragma unroll
    for (uint32_t w = 0; w < NGRP; w++)
#pragma unroll
      for (int h = 0; h < 4; h++) o[w][h] = 0.f;
    for (uint32_t j0 = 0; j0 < n_jobs; j0 += NGRP) {
#pragma unroll
      for (uint32_t w = 0; w < NGRP; w++) {
        const uint32_t j = j0 + w;
        if (j < n_jobs) {
          const uint32_t bi = w, k = j / NGRP;
          wait(&o_ready[bi], k & 1);
          tc_fence_after();
          uint32_t d[16];
          tmem_ld16(tmem + lane_addr + NGRP * 64 + bi * 64 + 16 * quad, d);  // this warp's dims are Q8_0 block `quad`
          tmem_ld_wait();
          const float4 corr = *reinterpret_cast<const float4*>(&misc->info[bi][0]);
          const float deq = misc->info[bi][4 + quad];
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&o_free[bi]));
          const float cr[4] = {corr.x, corr.y, corr.z, corr.w};
#pragma unroll
          for (int h = 0; h < 4; h++) {
            const float v = fmaf(s32_to_f32(d[h]), 65536.0f, fmaf(s32_to_f32(d[4 + h]), 256.0f, s32_to_f32(d[8 + h])));
            o[w][h] = fmaf(o[w][h], cr[h], v * deq);
          }
        }
      }
    }
    // ---- epilogue: partial (o, m, l) per query head, or the final output ----
    // Every group's O is in this thread's registers; the groups' maxima and sums arrive through
    // shared memory once the softmax warps are done. The groups w with w % HPC == g hold disjoint
    // token subsets of head g and are merged here.
    named_bar_sync(FIN_BAR, 128 * NGRP + 128);
    pdl_wait();  // the partials / output buffers may still be read by earlier kernels
    const uint32_t tag = epoch + 1 != 0 ? epoch + 1 : 1u;  // never 0: untouched scratch reads as tag 0
    uint32_t merge_mode;
    bool merger;
    merge_plan(merge_mode, merger);
    float acc_h[HPC * 4];  // this CTA's partial o per query head, at this thread's dim
#pragma unroll
    for (uint32_t g = 0; g < HPC; g++) {
#pragma unroll
      for (uint32_t hq = 0; hq < 4; hq++) {
        float m, l, acc = 0.f;
        head_ml(g, hq, m, l);
#pragma unroll
        for (uint32_t w = g; w < NGRP; w += HPC) acc += o[w][hq] * ex2(misc->mfin[w][hq] - m);
        acc_h[g * 4 + hq] = acc;
        const uint32_t h = (g0 + g) * p.qpg + hq;
        if (n_splits == 1) {
          put(h, dim, acc * (1.0f / l));
        } else if (MODE != 1 && merger) {  // stays in the CTA
          own_part()[(g * 4 + hq) * BP_HEAD_DIM + dim] = acc;
        } else if (merge_mode != 0) {  // tagged, for the CTAs that merge this head's units
          uint2* dst = p.ll + (split * p.n_head + h) * BP_LL_STRIDE;
          st_tagged(dst + dim, __float_as_uint(acc), tag);
          if (dim == 0) {
            st_tagged(dst + 128, __float_as_uint(m), tag);
            st_tagged(dst + 129, __float_as_uint(l), tag);
          }
        } else {  // plain, for attn_combine_kernel
          float* dst = p.partials + (static_cast<size_t>(split) * p.n_head + h) * BP_PART_STRIDE;
          dst[dim] = acc;
          if (dim == 0) { dst[128] = m; dst[129] = l; }
        }
      }
    }
    if (MODE != 1 && merger && dim == 0) misc->tag = tag;
    if (merge_mode == 1) {
      // This CTA's units: u = (query head hl, dim quarter qd) with u mod n_splits == split. All four
      // accumulate warps work on a unit: each folds a quarter of the other splits (warp `qd` starts from
      // the CTA's own part, which it holds in registers), then warp `qd` combines the four shares.
#pragma unroll 1
      for (uint32_t u = split; u < HPC * 16; u += n_splits) {
        const uint32_t hl = u >> 2, qd = u & 3;
        float m_r = NEG_BIG, l_r = 0.f, o_r = 0.f;
        if (quad == qd) {
          o_r = acc_h[0];
#pragma unroll
          for (uint32_t i = 1; i < HPC * 4; i++) o_r = hl == i ? acc_h[i] : o_r;
          head_ml(hl / 4, hl % 4, m_r, l_r);
        }
        const uint32_t n_oth = n_splits - 1;
        const uint32_t mine = quad < n_oth ? (n_oth - quad + 3) / 4 : 0;  // other splits quad, quad + 4, ...
        merge_part<10>(p, lane, quad, 4, mine, split, g0 * p.qpg + hl, qd * 32 + lane, tag, &abort_s, m_r, l_r, o_r);
        misc->xo[quad][lane] = o_r;
        if (lane == 0) {
          misc->xm[quad] = m_r;
          misc->xl[quad] = l_r;
        }
        __threadfence_block();
        named_bar_sync(SHARE_BAR, 128);
        if (quad == qd) {
          const float m_all = fmaxf(fmaxf(misc->xm[0], misc->xm[1]), fmaxf(misc->xm[2], misc->xm[3]));
          float o_all = 0.f, l_all = 0.f;
#pragma unroll
          for (uint32_t w = 0; w < 4; w++) {
            const float e = ex2(misc->xm[w] - m_all);
            o_all = fmaf(misc->xo[w][lane], e, o_all);
            l_all = fmaf(misc->xl[w], e, l_all);
          }
          put(g0 * p.qpg + hl, qd * 32 + lane, o_all * (1.0f / l_all));
          // The next launch's tag. Safe to advance once unit 0 is merged: its warps have seen every split's
          // tag, so every CTA of the group has read the epoch.
          if (u == 0 && lane == 0) *reinterpret_cast<volatile uint32_t*>(p.epochs + blockIdx.y) = tag;
        }
        if (u + n_splits < HPC * 16) named_bar_sync(SHARE_BAR, 128);  // the exchange area is reused
      }
    }
  }

  // Mode 2: the merger's softmax warps take the units (one call site, after the roles: their registers
  // are dead here and a round's loads all fit).
  uint32_t merge_mode_end;
  bool merger_end;
  merge_plan(merge_mode_end, merger_end);
  if constexpr (MODE != 1) if (merger_end && warp >= U_FIRST_SM_WARP) {
    __threadfence_block();
    named_bar_sync(MERGE_BAR, 128 * NGRP + 128);  // this CTA's own partial and the tag are in shared memory
    const uint32_t tag = misc->tag;
    pdl_wait();  // the output buffer may still be read by earlier kernels
#pragma unroll 1
    for (uint32_t u = warp - U_FIRST_SM_WARP; u < HPC * 16; u += 4 * NGRP + 4) {
      const uint32_t hl = u >> 2, d = (u & 3) * 32 + lane;
      float m, l;
      head_ml(hl / 4, hl % 4, m, l);
      merge_unit<15>(p, lane, n_splits, split, g0 * p.qpg + hl, d, own_part()[hl * BP_HEAD_DIM + d], m, l, tag, &abort_s);
      if (u == 0 && lane == 0) *reinterpret_cast<volatile uint32_t*>(p.epochs + blockIdx.y) = tag;  // as in mode 1
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
  if (p.dbg != nullptr && threadIdx.x == 0) {  // development aid: span of the launch in ns
    unsigned long long t_exit_ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_exit_ns));
    atomicMax(&p.dbg[33], t_exit_ns);
    atomicMax(&p.dbg[37], t_exit_ns - t_entry_ns);
  }
}

}  // namespace

uint32_t bp_decode_umma_stage_tokens() { return UT; }

template <uint32_t HPC>
static cudaError_t umma_attr() {
  cudaError_t e = cudaFuncSetAttribute(decode_umma_kernel<HPC, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(U_SMEM_BUDGET));
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(decode_umma_kernel<HPC, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(U_SMEM_BUDGET));
}

cudaError_t bp_decode_umma_init(bp_attn_ctx* c) {
  cudaError_t e = umma_attr<1>();
  if (e != cudaSuccess) return e;
  e = umma_attr<2>();
  if (e != cudaSuccess) return e;
  // The in-kernel merge makes the CTAs of a head group wait for one another, so a launch may never
  // have more CTAs than the device holds at once: ask the runtime instead of assuming one per SM.
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_umma_kernel<1, 1>, static_cast<int>(U_THREADS),
                                                    static_cast<size_t>(U_SMEM_BUDGET));
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  c->umma_resident = static_cast<uint32_t>(per_sm) * static_cast<uint32_t>(c->sm_count);
  return cudaSuccess;
}

// K stages and V slots that fit: equal numbers (a K stage is busy for a load latency plus the short
// wait for its softmax group, a V slot for a load latency plus the P V issue), at most U_MAX_STAGES.
template <uint32_t HPC>
static uint32_t umma_max_stages() {
  uint32_t n = (U_SMEM_BUDGET - ULayout<HPC>::tail() - 1024) / (ULayout<HPC>::KSTAGE_B + HPC * ULayout<HPC>::VSLOT_B);
  return n > U_MAX_STAGES ? U_MAX_STAGES : n;
}

// Geometry of the UMMA decode: stages of 128 tokens; the grid is
// (splits, n_kv_head / hpc) with splits * groups <= number of SMs.
static uint32_t umma_spp(const bp_attn_ctx* c, uint32_t cur_pos) {
  const uint32_t n_st = (cur_pos + UT - 1) / UT;
  const uint32_t groups = c->cfg.n_kv_head / c->opt_uhpc;
  const uint32_t budget = c->umma_resident < bp_decode_max_splits(c) ? c->umma_resident : bp_decode_max_splits(c);
  uint32_t ctas = budget / groups;
  if (ctas == 0) ctas = 1;
  // With few KV heads per device (a shard of a multi-GPU run) there are many more SMs than a head
  // can use well: a job costs about 1 us of streaming, merging one more split about 0.07 us at the
  // end of the launch, so beyond sqrt(15 * stages) splits the merge outgrows what it saves.
  const uint32_t cap = static_cast<uint32_t>(sqrtf(15.0f * static_cast<float>(n_st))) + 1;
  if (ctas > cap) ctas = cap < 8 ? 8 : cap;
  uint32_t spp = (n_st + ctas - 1) / ctas;
  // Short launches are merged by one CTA per head group, whose merge polls up to 15 other splits in
  // one round: 17 or 18 splits of up to 4 stages become at most 16 slightly longer ones.
  if (spp <= 4 && (n_st + spp - 1) / spp > 16 && (n_st + 15) / 16 <= 4) spp = (n_st + 15) / 16;
  // Two stages are one split: the second job runs on another softmax group of the same CTA, and nothing is
  // merged (6.0 us per layer against 7.1 at 200 keys). From three stages on the splits win (measured up to 4096).
  if (n_st == 2) spp = 2;
  return spp;
}

uint32_t bp_decode_umma_splits(const bp_attn_ctx* c, uint32_t cur_pos) {
  const uint32_t n_st = (cur_pos + UT - 1) / UT;
  const uint32_t spp = umma_spp(c, cur_pos);
  return (n_st + spp - 1) / spp;
}

template <uint32_t HPC>
static cudaError_t launch_umma(bp_attn_ctx* c, cudaStream_t s, UmmaParams& p, uint32_t spp, uint32_t n_splits) {
  uint32_t cap = umma_max_stages<HPC>();
  uint32_t v_cap = cap * HPC > U_MAX_STAGES ? U_MAX_STAGES : cap * HPC;
  if (c->opt_uring != 0) {  // tuning override: K stages * 16 + V slots, accepted when it fits
    const uint32_t k = c->opt_uring >> 4, v = c->opt_uring & 15;
    if (k >= 1 && v >= 1 && k <= U_MAX_STAGES && v <= U_MAX_STAGES && ULayout<HPC>::total(k, v) <= U_SMEM_BUDGET) {
      cap = k;
      v_cap = v;
    }
  }
  p.nk = spp < cap ? spp : cap;
  p.nv = spp * HPC < v_cap ? spp * HPC : v_cap;
  const size_t smem = ULayout<HPC>::total(p.nk, p.nv);
  dim3 grid(n_splits, c->cfg.n_kv_head / HPC);
  // Short launches (up to 16 splits of up to 4 stages) are merged by one CTA per head group, longer
  // ones by all CTAs of the group.
  if (n_splits <= 16 && spp <= 4)
    return bp_launch(c->opt_pdl != 0, decode_umma_kernel<HPC, 3>, grid, dim3(U_THREADS), smem, s, c->umaps_dev, p);
  return bp_launch(c->opt_pdl != 0, decode_umma_kernel<HPC, 1>, grid, dim3(U_THREADS), smem, s, c->umaps_dev, p);
}

cudaError_t bp_launch_decode_umma(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q, __half* out,
                                  uint32_t cur_pos, uint32_t* n_splits_out, const bp_fused_step* fs) {
  const uint32_t spp = umma_spp(c, cur_pos);
  const uint32_t n_splits = bp_decode_umma_splits(c, cur_pos);
  UmmaParams p;
  p.q = q;
  p.out = out;
  p.partials = c->partials;
  p.err = c->err_dev;
  p.row_base = layer * c->cfg.max_seq;
  p.cur_pos = cur_pos;
  p.tps = spp * UT;
  p.nk = p.nv = 1;
  p.n_head = c->cfg.n_head;
  p.qpg = c->qpg;
  p.sm_scale_log2 = (1.0f / sqrtf(static_cast<float>(BP_HEAD_DIM))) * 1.4426950408889634f;
  p.dbg = c->dbg_on ? c->dbg_dev : nullptr;
  p.n_px = c->n_px;
  p.px_off = layer * c->cfg.n_shards * c->q_dim + c->cfg.shard * c->q_dim;
  p.px_out = c->px_dev;
  // The in-kernel merge makes CTAs wait for one another: all of them must be resident at once,
  // which only a caller with the device to itself can promise (option exclusive_device). The
  // exchange lives in the in-kernel merge.
  p.merge = (c->opt_umerge && c->opt_exclusive) || c->n_px > 0;
  p.wait_limit = c->opt_wait_limit;
  p.poll_limit = c->opt_poll_limit;
  p.v_pre_all = c->opt_vpre;
  p.fresh_from = bp_fresh_from(c, layer);
  const uint32_t px_slot = c->n_px > 0 && c->opt_px_meet && layer > 0 ? (layer - 1) % 64 : NO_SLOT;
  p.px_meet = px_slot | c->cfg.shard << 8;
  p.px_tab = c->pxf_dev;
  p.ll = c->ll;
  p.epochs = c->epochs;
  p.fused = fs != nullptr ? 1u : 0u;
  p.eps = c->cfg.rms_eps;
  p.n_kv_head = c->cfg.n_kv_head;
  p.q_roped = nullptr;
  p.w_q = p.w_k = p.k_cur = p.v_cur = p.rope_row = nullptr;
  p.k_d = p.v_d = nullptr;
  p.k_qs = p.v_qs = nullptr;
  if (fs != nullptr) {
    p.q_roped = fs->q_roped;
    p.w_q = fs->w_q;
    p.w_k = fs->w_k;
    p.k_cur = fs->k_cur;
    p.v_cur = fs->v_cur;
    p.rope_row = c->rope + static_cast<size_t>(cur_pos - 1) * BP_HEAD_DIM;
    p.k_d = reinterpret_cast<float*>(c->kv[0] + bp_d_off(c, layer));
    p.v_d = reinterpret_cast<float*>(c->kv[1] + bp_d_off(c, layer));
    p.k_qs = reinterpret_cast<uint32_t*>(c->kv[0] + bp_qs_off(c, layer));
    p.v_qs = reinterpret_cast<uint32_t*>(c->kv[1] + bp_qs_off(c, layer));
  }
  *n_splits_out = p.merge ? 1 : n_splits;  // nothing left to merge for the caller
  if (fs != nullptr) bp_note_row_write(c, layer, cur_pos - 1);
  bp_note_sm_launch(c, n_splits * (c->cfg.n_kv_head / c->opt_uhpc));
  return c->opt_uhpc == 2 ? launch_umma<2>(c, s, p, spp, n_splits) : launch_umma<1>(c, s, p, spp, n_splits);
}
