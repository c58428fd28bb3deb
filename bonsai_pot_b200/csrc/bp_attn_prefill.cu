// Batched-prefill causal attention over the Q8_0 KV cache. Replaces
// attention.wgsl (dispatch_attention with is_prefill = 1, src/forward.rs:501-532).
//
// Two launches per layer:
//
// 1. prefill_expand_kernel: the m cache rows the batch just wrote are expanded
//    once, int8 * FP32 block scale -> f16, into a context-owned scratch
//    [K | V][rows][kv_dim]. Every key tile is used by m / 32 query tiles, so
//    expanding it once per layer instead of once per use takes the int8 work
//    out of the attention loop; the scratch (8 MB at 2048 tokens) stays in L2.
//
// 2. prefill_umma_kernel: flash attention on the 5th-generation tensor cores
//    (tcgen05.mma kind::f16, accumulators in TMEM). A work item is one KV head
//    and NQ query tiles of 128 rows each; a tile's rows are 128 / qpg
//    consecutive tokens times the qpg query heads of the group. Persistent
//    CTAs fetch items, longest first, from a global counter. Keys come in
//    tiles of 64. Three layouts (PLayout): one query tile per item and two CTAs
//    per SM (the default when there are more items than SMs: while one CTA is
//    between two items, 7 us of item fetch, Q load, pipeline fill and epilogue,
//    the other computes), one query tile and one CTA per SM (small batches), two
//    query tiles on one CTA per SM (every K / V tile loaded once for both).
//    Per key tile and per query tile X:
//      warps 0 .. NQ-1 request the K and V tiles (TMA, 128-byte swizzle, straight into UMMA operand
//                      layout) and issue O_X += P_X V (4 UMMAs M 128, N 128, K 16, P read from TMEM
//                      as the A operand); they poll their barriers and never block. With two query
//                      tiles warp 0 loads V and warp 1 loads K
//      Q K^T issuer X  S_X = Q_X K^T (8 UMMAs M 128, N 64, K 16) into one of the two 64-column
//                      buffers of X's S region in TMEM, up to two tiles ahead of P V
//                      (one thread issues a tcgen05.mma only every ~85 to 115 cycles, the tensor pipe
//                      takes one every 70 to 80 from several threads: hence an issuing thread per role
//                      and query tile)
//      softmax group X thread = query row = TMEM lane: scale, causal mask, online max / sum,
//                      P as f16 written over the tile's S buffer; O_X is rescaled in TMEM only
//                      when a row maximum grew by more than 2^8 (P stays below 2^8 meanwhile)
//    S is double-buffered so that a tile's softmax overlaps the MMAs of its neighbours.
//    TMEM per query tile: S (two buffers of 64 columns) and O, 128 columns each.
// Every wait is bounded; a timeout sets the context's error word and the CTA
// winds down and frees its TMEM.
#include "bp_common.cuh"
#include "bp_ptx.cuh"

cudaError_t bp_launch_scalar_attention(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q,
                                       __half* out, uint32_t cur_pos, uint32_t m, bool is_prefill,
                                       uint32_t* launches);
void* bp_tensor_map_encoder();

namespace {

using namespace bp;

constexpr unsigned FULL = 0xffffffffu;
constexpr float NEG_BIG = -1e30f;
constexpr uint32_t BM = 128, BN = 64;             // query rows per tile, keys per tile
constexpr uint32_t OPER_B = 2 * 16384;           // one f16 operand tile: 2 chunks of [128 rows][128 B]
constexpr uint32_t KV_TILE_B = 2 * 8192;          // one f16 K or V tile: 2 chunks of [64 keys][128 B]
constexpr uint32_t SW = 128;                      // TMEM columns of one query tile's S region (two 64-column buffers) and of O

template <uint32_t NQ, uint32_t CPS>  // query tiles per CTA (work item), CTAs per SM
struct PLayout {
  // NQ loader / P V issuer warps, NQ Q K^T issuer warps, NQ softmax groups of 4 warps.
  // One CTA per SM: four K and four V slots. Two CTAs per SM (one query tile and 256 TMEM columns each):
  // two slots each; while one CTA is between two work items (7 us of item fetch, Q load, pipeline fill
  // and epilogue per item) the other one computes.
  static_assert(CPS == 1 || (CPS == 2 && NQ == 1), "two CTAs per SM only with one query tile each");
  static constexpr uint32_t KV_SLOTS = CPS == 2 ? 2 : 4;
  static constexpr uint32_t TMEM_COLS = 256 * NQ;   // S_X at 128 X, O_X at 128 (NQ + X): 128 columns each
  static constexpr uint32_t TM_S = 0, TM_O = 128 * NQ;
  static constexpr uint32_t N_LOADERS = NQ;         // warps 0 .. NQ - 1 load tiles and issue P V, the next NQ warps issue Q K^T
  static constexpr uint32_t FIRST_SM_WARP = 2 * NQ;
  static constexpr uint32_t THREADS = 32 * FIRST_SM_WARP + NQ * 128;
  static constexpr uint32_t OFF_Q = 0, OFF_K = NQ * OPER_B, OFF_V = OFF_K + KV_SLOTS * KV_TILE_B;
  static constexpr uint32_t SMEM = OFF_V + KV_SLOTS * KV_TILE_B + 1024;
};

struct PrefillParams {
  const __half* q;
  __half* out;
  uint32_t* err;
  uint32_t* counter;        // work-item counter, zeroed by the expand kernel of the same layer
  uint32_t m, n_head, n_kv_head, qpg, n_groups;  // n_groups = ceil(m / (NQ * 128 / qpg))
  unsigned long long* dbg;  // development aid: cycle counters of CTA 0, null in normal use
  float scale_log2;
  uint32_t wait_limit;      // polls of an mbarrier before the CTA gives up and winds down
  // Peer exchange (n_px > 0): every output vector is also stored into each rank's gathered buffer
  // (this rank's included), row = token, at column px_col0 + head * 128 of rows px_row_stride wide:
  // the all-gather of the KV-head shards' outputs by peer stores in the epilogue.
  // The addresses sit in device memory, not here: a parameter block 64 bytes larger made the kernel
  // 2 % slower (58.8 against 57.4 us per layer at 2048 tokens), with or without the exchange.
  uint32_t n_px, px_col0, px_row_stride;
  __half* const* px_out;
};

// Physical byte offset of 16-byte unit `u16` (0..15) of row `r` in an operand tile.
__device__ __forceinline__ uint32_t oper_off(uint32_t r, uint32_t u16) {
  return (u16 >> 3) * 16384 + r * 128 + (((u16 & 7) ^ (r & 7)) << 4);
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// Packed FP32 pairs (sm_100): one instruction for two lanes of a 64-bit register pair.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1) {
  asm("{\n\t.reg .b64 ra, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\t"
      "add.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D (TMEM) (+)= A (TMEM: lane = row, one 32-bit column = two consecutive f16 of K) x B (smem descriptor).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Expansion of rows [0, rows_pad) of one layer: rows below m get int8 * scale (product in FP32,
// rounded once to f16, clamped to the finite range); rows m .. rows_pad - 1 get zeros, so that a
// masked key can never feed an Inf or NaN into P V. Thread = 8 consecutive dims of one row.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prefill_expand_kernel(const uint8_t* __restrict__ kv_k, const uint8_t* __restrict__ kv_v,
                                                             uint64_t d_off, uint64_t qs_off, __half* __restrict__ dst,
                                                             uint64_t dst_v_off, uint32_t kv_dim, uint32_t m, uint32_t rows_pad,
                                                             uint32_t* counter) {
  pdl_launch_dependents();
  pdl_wait();  // the cache rows were written by the kernel before this one; the scratch may still be read
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *counter = 0;
  const uint32_t per_row = kv_dim >> 3;
  const uint32_t idx = blockIdx.x * 256 + threadIdx.x;
  const uint32_t row = idx / per_row, u = idx % per_row;
  if (row >= rows_pad) return;
  const uint8_t* src = blockIdx.y ? kv_v : kv_k;
  __half* out = dst + (blockIdx.y ? dst_v_off : 0) + static_cast<size_t>(row) * kv_dim + 8 * u;
  uint4 w = make_uint4(0, 0, 0, 0);
  if (row < m) {
    const float scale = *reinterpret_cast<const float*>(src + d_off + (static_cast<size_t>(row) * (kv_dim >> 5) + (u >> 2)) * 4);
    const uint2 qv = *reinterpret_cast<const uint2*>(src + qs_off + static_cast<size_t>(row) * kv_dim + 8 * u);
    const uint32_t qw[2] = {qv.x, qv.y};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int a = static_cast<int8_t>(qw[j >> 1] >> (16 * (j & 1)));
      const int b = static_cast<int8_t>(qw[j >> 1] >> (16 * (j & 1) + 8));
      const float fa = fminf(fmaxf(static_cast<float>(a) * scale, -65504.f), 65504.f);
      const float fb = fminf(fmaxf(static_cast<float>(b) * scale, -65504.f), 65504.f);
      __half2 h = __floats2half2_rn(fa, fb);
      o[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    w = make_uint4(o[0], o[1], o[2], o[3]);
  }
  *reinterpret_cast<uint4*>(out) = w;
}

template <uint32_t NQ, uint32_t CPS, bool PX>  // PX: with the peer exchange in the epilogue (an instance of its own: the plain one pays nothing)
__global__ void __launch_bounds__(PLayout<NQ, CPS>::THREADS, CPS)
prefill_umma_kernel(const CUtensorMap* __restrict__ maps, const PrefillParams p) {
  // tensor maps in device memory, written once by the host when the context is created: K rows, V rows
  const CUtensorMap &map_k = maps[0], &map_v = maps[1];
  using L = PLayout<NQ, CPS>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t k_full[L::KV_SLOTS], v_full[L::KV_SLOTS];
  __shared__ __align__(8) uint64_t k_empty[NQ][L::KV_SLOTS], v_empty[NQ][L::KV_SLOTS];  // per query tile: it is done with the slot
  __shared__ __align__(8) uint64_t s_ready[NQ][2], p_ready[NQ][2], p_free[NQ][2], o_done[NQ];
  __shared__ uint32_t tmem_base_s, item_s;
  __shared__ volatile uint32_t abort_s;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tq_tokens = BM / p.qpg;               // tokens per query tile
  const uint32_t n_items = p.n_groups * p.n_kv_head;   // work items: (group of NQ query tiles, KV head)

  if (threadIdx.x == 0) {
    for (uint32_t i = 0; i < L::KV_SLOTS; i++) {
      mbar_init(smem_u32(&k_full[i]), 1);
      mbar_init(smem_u32(&v_full[i]), 1);
      for (uint32_t x = 0; x < NQ; x++) {
        mbar_init(smem_u32(&k_empty[x][i]), 1);
        mbar_init(smem_u32(&v_empty[x][i]), 1);
      }
    }
    for (uint32_t x = 0; x < NQ; x++) {
      mbar_init(smem_u32(&s_ready[x][0]), 1);
      mbar_init(smem_u32(&s_ready[x][1]), 1);
      mbar_init(smem_u32(&p_ready[x][0]), 4);
      mbar_init(smem_u32(&p_ready[x][1]), 4);
      mbar_init(smem_u32(&p_free[x][0]), 1);
      mbar_init(smem_u32(&p_free[x][1]), 1);
      mbar_init(smem_u32(&o_done[x]), 1);
    }
    abort_s = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_s), L::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  // Set-up above overlaps the previous kernel (programmatic dependent launch); everything below reads
  // what it wrote (the expanded rows, q, the item counter).
  if (threadIdx.x == 0) pdl_launch_dependents();
  pdl_wait();

  const bool dbg_on = p.dbg != nullptr && blockIdx.x == 0 && lane == 0;
  long long tw[4] = {0, 0, 0, 0};
  long long tph[4] = {0, 0, 0, 0};  // softmax phases: S load, maximum (+ rescale), exponentials, P store
  const long long t_begin = clock64();
  auto waitx = [&](uint64_t* bar, uint32_t parity, int slot) {
    if (abort_s) return;
    const long long t0 = dbg_on ? clock64() : 0;
    if (!mbar_wait(smem_u32(bar), parity, p.wait_limit)) {
      abort_s = 1;
      atomicExch(p.err, 5u);
    }
    if (dbg_on) tw[slot] += clock64() - t0;
  };

  // Barrier phases keep counting across work items: gkv = key tiles loaded so far by this CTA,
  // gx[X] = key tiles query tile X has gone through, od[X] for the once-per-item o_done;
  // nothing is re-initialised between items. A loader keeps, per (query tile, slot), whether
  // a release is outstanding and the phase it will complete (bit x * L::KV_SLOTS + slot).
  uint32_t gkv = 0, gx[NQ], od[NQ];
#pragma unroll
  for (uint32_t x = 0; x < NQ; x++) { gx[x] = 0; od[x] = 0; }
  uint32_t pend_k = 0, pend_v = 0, phase_k = 0, phase_v = 0;
  uint32_t vph = 0;  // softmax threads: next phase of "P V complete" per K/V slot, for their own query tile

  for (uint32_t round = 0;; round++) {
    // The first item of a CTA is its own index (the grid never has more CTAs than there are items); further
    // items come from the counter, fetched only when the CTA is free (fetching ahead would defeat
    // longest-first balancing).
    uint32_t item = blockIdx.x;
    if (round != 0) {
      if (threadIdx.x == 0) item_s = gridDim.x + atomicAdd(p.counter, 1u);
      __syncthreads();
      item = item_s;
    }
    if (item >= n_items) break;
    const uint32_t g = item % p.n_kv_head;
    const uint32_t group = p.n_groups - 1 - item / p.n_kv_head;  // long (late) groups first
    // query tile X: tokens [tq0[X], tq0[X] + tq_tokens); nx[X] key tiles (0 when it lies beyond the batch)
    uint32_t tq0[NQ], nx[NQ], n_tiles = 0;
#pragma unroll
    for (uint32_t x = 0; x < NQ; x++) {
      tq0[x] = (group * NQ + x) * tq_tokens;
      nx[x] = tq0[x] < p.m ? (min(tq0[x] + tq_tokens, p.m) + BN - 1) / BN : 0;
      n_tiles = max(n_tiles, nx[x]);
    }
    // Q tiles as K-major A operands: row r = (token tq0 + r / qpg, head g * qpg + r % qpg)
    {
      constexpr uint32_t Q_UNITS = NQ * BM * 16, Q_ITERS = (Q_UNITS + L::THREADS - 1) / L::THREADS;
      uint4 qv[Q_ITERS];
#pragma unroll
      for (uint32_t k = 0; k < Q_ITERS; k++) {  // every load of this thread is in flight before the first store
        const uint32_t i = threadIdx.x + k * L::THREADS;
        const uint32_t x = i / (BM * 16), r = (i >> 4) & (BM - 1), u = i & 15;
        const uint32_t tok = (group * NQ + x) * tq_tokens + r / p.qpg, head = g * p.qpg + r % p.qpg;
        qv[k] = make_uint4(0, 0, 0, 0);
        if (i < Q_UNITS && tok < p.m)
          qv[k] = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(tok) * p.n_head + head) * BP_HEAD_DIM + 8 * u);
      }
#pragma unroll
      for (uint32_t k = 0; k < Q_ITERS; k++) {
        const uint32_t i = threadIdx.x + k * L::THREADS;
        const uint32_t x = i / (BM * 16), r = (i >> 4) & (BM - 1), u = i & 15;
        if (i < Q_UNITS) *reinterpret_cast<uint4*>(smem_gen + L::OFF_Q + x * OPER_B + oper_off(r, u)) = qv[k];
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp < L::N_LOADERS) {
      // ---------------- loaders and P V issuers ----------------
      // Threads that never block. With two query tiles per CTA: warp 0 requests the V tiles and issues
      // O_0 += P_0 V, warp 1 requests the K tiles and issues O_1 += P_1 V. A single thread issuing the
      // P V of both query tiles was the bottleneck of this kernel: it needs about 1100 cycles per key tile
      // and query tile (polls, four MMAs at 115 cycles each, three commits), so a P tile waited some 1400
      // cycles for its turn and the softmax groups then waited as long for the next S. With one query
      // tile per CTA warp 0 does all of it.
      if (lane == 0) {
        constexpr uint32_t IDESC_PV = umma_idesc(1, 0, 0, 0, 1, BM, 128);  // f32 += f16 (TMEM) x f16 (MN-major), N = 128 dims
        const uint64_t dmn = umma_desc_sw128(0, 8192, 1024);    // V: next 64 dims 8 KB away, 8 key rows 1 KB apart
        const bool do_k = L::N_LOADERS == 1 || warp == 1, do_v = warp == 0;
        const uint32_t x = warp;                                // the query tile whose P V this thread issues
        const uint32_t n_pv = nx[x];
        uint32_t lk = do_k ? 0u : n_tiles, lv = do_v ? 0u : n_tiles, ip = 0, spins = 0;  // tiles requested, P V issued
        // the next tile of a stream, once every query tile that used the slot's last tile has released it
        auto try_load = [&](bool is_k, uint32_t& li, uint32_t& pend, uint32_t& phase) {
          const uint32_t s = (gkv + li) % L::KV_SLOTS;
          bool slot_free = true;
          uint32_t users = 0;
#pragma unroll
          for (uint32_t y = 0; y < NQ; y++) {
            const uint32_t bit = 1u << (y * L::KV_SLOTS + s);
            users |= li < nx[y] ? bit : 0u;
            if (pend & bit) {
              if (mbar_test(smem_u32(is_k ? &k_empty[y][s] : &v_empty[y][s]), (phase & bit) ? 1u : 0u)) {
                pend &= ~bit;
                phase ^= bit;
              } else {
                slot_free = false;
              }
            }
          }
          if (!slot_free) return false;
          pend |= users;
          uint64_t* full = is_k ? &k_full[s] : &v_full[s];
          mbar_arrive_expect_tx(smem_u32(full), KV_TILE_B);
          tma_load_3d(smem_base + (is_k ? L::OFF_K : L::OFF_V) + s * KV_TILE_B, is_k ? &map_k : &map_v, smem_u32(full), 0,
                      static_cast<int>(li * BN), static_cast<int>(2 * g));
          li++;
          return true;
        };
        while ((lk < n_tiles || lv < n_tiles || ip < n_pv) && !abort_s) {
          bool progressed = false;
          if (lk < n_tiles) progressed |= try_load(true, lk, pend_k, phase_k);
          if (lv < n_tiles) progressed |= try_load(false, lv, pend_v, phase_v);
          if (ip < n_pv) {
            const uint32_t i = ip, s = (gkv + i) % L::KV_SLOTS, c = gx[x] + i, b = c & 1;
            // one barrier per S buffer: the softmax group may run two tiles ahead of this test, and two
            // completions on one barrier would be indistinguishable from none
            if (mbar_test(smem_u32(&p_ready[x][b]), (c >> 1) & 1) &&
                mbar_test(smem_u32(&v_full[s]), ((gkv + i) / L::KV_SLOTS) & 1)) {
              tc_fence_after();
              const uint64_t vb = dmn + ((smem_base + L::OFF_V + s * KV_TILE_B) >> 4);
              const uint32_t s_col = tmem + L::TM_S + x * SW, o_col = tmem + L::TM_O + x * SW;
#pragma unroll
              for (uint32_t ks = 0; ks < 4; ks++)  // 16 keys per UMMA: 8 columns of P, 16 rows of V
                umma_f16_ts(o_col, s_col + 64 * b + 8 * ks, vb + ks * (16 * 128 >> 4), IDESC_PV, (i | ks) ? 1u : 0u);
              umma_commit(smem_u32(&p_free[x][b]));   // P V of tile i complete: the S buffer may take the next Q K^T,
              umma_commit(smem_u32(&v_empty[x][s]));  // the V slot is free and O_X is consistent
              if (++ip == n_pv) umma_commit(smem_u32(&o_done[x]));
              progressed = true;
            }
          }
          if (progressed) {
            spins = 0;
          } else if (++spins > p.wait_limit) {  // bounded like every other wait (a round is a few dozen cycles)
            abort_s = 1;
            atomicExch(p.err, 5u);
          }
        }
      }
    } else if (warp < L::FIRST_SM_WARP) {
      // ---------------- Q K^T issuer of query tile X ----------------
      // One issuing thread sustains about one tcgen05.mma per 115 cycles whatever its size; the tensor
      // pipe takes one 128 x 128 x 16 MMA per 70 to 80 cycles from several threads (measured). So the
      // issue work is spread: one thread per query tile for S = Q K^T (8 MMAs per key tile), one more
      // for all P V (4 per key tile and query tile).
      const uint32_t x = warp - L::N_LOADERS;
      const uint32_t n_mine = nx[x], c0 = gx[x];
      if (lane == 0 && n_mine > 0) {
        constexpr uint32_t IDESC_QK = umma_idesc(1, 0, 0, 0, 0, BM, BN);   // f32 = f16 (K-major) x f16 (K-major), N = 64 keys
        const uint64_t dk = umma_desc_sw128(0, 16, 1024);       // K-major operands
        const uint64_t qa = dk + ((smem_base + L::OFF_Q + x * OPER_B) >> 4);
        const uint32_t s_col = tmem + L::TM_S + x * SW;
        // S of tile i goes to buffer (c0 + i) & 1 of the query tile's S region; P of the tile is
        // written over it and read from there by P V. Q K^T runs up to two tiles ahead of P V: a
        // buffer is free again when the P V of its previous tile has completed (p_free).
        for (uint32_t i = 0; i < n_mine; i++) {
          const uint32_t s = (gkv + i) % L::KV_SLOTS, c = c0 + i, b = c & 1;
          waitx(&k_full[s], ((gkv + i) / L::KV_SLOTS) & 1, 0);
          if (c >= 2) waitx(&p_free[x][b], ((c >> 1) - 1) & 1, 2);
          tc_fence_after();
          const uint64_t kb = dk + ((smem_base + L::OFF_K + s * KV_TILE_B) >> 4);
#pragma unroll
          for (uint32_t ks = 0; ks < 8; ks++) {  // 16 dims per UMMA: chunk ks / 4, 32 bytes per step inside it
            const uint32_t qo = (ks >> 2) * (16384 >> 4) + (ks & 3) * 2, ko = (ks >> 2) * (8192 >> 4) + (ks & 3) * 2;
            umma_f16(s_col + 64 * b, qa + qo, kb + ko, IDESC_QK, ks);
          }
          umma_commit(smem_u32(&s_ready[x][b]));
        }
      }
    } else {
      // ---------------- softmax group X: thread = query row = TMEM lane ----------------
      const uint32_t x = (warp - L::FIRST_SM_WARP) >> 2, quad = warp & 3, r = quad * 32 + lane;
      const bool elected = ((warp - L::FIRST_SM_WARP) & 3) == 0 && lane == 0;  // releases the K slots for this query tile
      const uint32_t lane_addr = (quad * 32) << 16;
      const uint32_t s_addr = tmem + lane_addr + L::TM_S + x * SW, o_addr = tmem + lane_addr + L::TM_O + x * SW;
      const uint32_t tok = tq0[x] + r / p.qpg;
      const uint32_t n_mine = nx[x], c0 = gx[x];
      float m_run = NEG_BIG, l_run = 0.f;
      uint32_t prev_par = 0, prev_slot = 0;  // phase and slot of the previous tile's "P V complete" barrier
      for (uint32_t i = 0; i < n_mine; i++) {
        const uint32_t b = (c0 + i) & 1, slot = (gkv + i) % L::KV_SLOTS;
        waitx(&s_ready[x][b], ((c0 + i) >> 1) & 1, 0);
        tc_fence_after();
        const long long tp0 = dbg_on ? clock64() : 0;
        if (elected) mbar_arrive(smem_u32(&k_empty[x][slot]));  // Q K^T of tile i is complete
        uint32_t raw[64];
        tmem_ld32(s_addr + 64 * b, raw);
        tmem_ld32(s_addr + 64 * b + 32, raw + 32);
        tmem_ld_wait();
        const long long tp1 = dbg_on ? clock64() : 0;
        // causal mask: key i * BN + c is visible to this row iff key <= tok (only the last tile can cut)
        if ((i + 1) * BN > tq0[x] + 1) {
          const uint32_t k0 = i * BN;
#pragma unroll
          for (int c = 0; c < 64; c++)
            if (k0 + c > tok) raw[c] = __float_as_uint(NEG_BIG);
        }
        float mx[4] = {__uint_as_float(raw[0]), __uint_as_float(raw[1]), __uint_as_float(raw[2]), __uint_as_float(raw[3])};
#pragma unroll
        for (int c = 4; c < 60; c += 8) {
#pragma unroll
          for (int k = 0; k < 4; k++) mx[k] = max3(mx[k], __uint_as_float(raw[c + k]), __uint_as_float(raw[c + 4 + k]));
        }
#pragma unroll
        for (int k = 0; k < 4; k++) mx[k] = fmaxf(mx[k], __uint_as_float(raw[60 + k]));
        const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
        const bool grow = m_tile > m_run + 8.0f;        // lazy: keep the old maximum while P stays below 2^8
        const float m_new = grow ? m_tile : m_run;
        const float corr = grow ? ex2(m_run - m_new) : 1.0f;
        m_run = m_new;
        if (i > 0 && __any_sync(FULL, grow)) {
          // O_X may be rescaled only between two P V: the previous tile's must have completed (this
          // tile's is not issued before this thread hands over P)
          waitx(&v_empty[x][prev_slot], prev_par, 1);
          tc_fence_after();
#pragma unroll 1
          for (uint32_t c = 0; c < 8; c++) {
            uint32_t o[16];
            tmem_ld16(o_addr + 16 * c, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
            tmem_st16(o_addr + 16 * c, o);
          }
        }
        const long long tp2 = dbg_on ? clock64() : 0;
        // the completion of this tile's P V will be phase `vph bit slot` of its slot's barrier
        prev_par = (vph >> slot) & 1u;
        prev_slot = slot;
        vph ^= 1u << slot;
        // P over the first 32 columns of the buffer (every S value of this row is in registers by now)
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t ph[32];
        const float neg_m = -m_new;
#pragma unroll
        for (int c = 0; c < 32; c++) {
          float a0, a1;
          fma2(a0, a1, __uint_as_float(raw[2 * c]), __uint_as_float(raw[2 * c + 1]), p.scale_log2, neg_m);
          const float p0 = ex2(a0), p1 = ex2(a1);
          add2(sum[2 * (c & 1)], sum[2 * (c & 1) + 1], p0, p1);
          __half2 h = __floats2half2_rn(p0, p1);
          ph[c] = *reinterpret_cast<uint32_t*>(&h);
        }
        const long long tp3 = dbg_on ? clock64() : 0;
        tmem_st32(s_addr + 64 * b, ph);
        l_run = l_run * corr + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&p_ready[x][b]));
        if (dbg_on) {
          const long long tp4 = clock64();
          tph[0] += tp1 - tp0; tph[1] += tp2 - tp1; tph[2] += tp3 - tp2; tph[3] += tp4 - tp3;
        }
      }
      // ---- O / l -> f16 ----
      // A thread holds one output row (256 B of f16). Stored from here, 16 bytes at a time, a warp's store
      // instruction touches 32 different lines, and the load/store unit takes a cycle per line: 3800 cycles
      // per work item at 2048 tokens (48 us per layer when the rows went over NVLink). So the rows go to the
      // dead Q tile of this query tile first (16-byte chunks xor-swizzled by the row) and every warp then
      // writes the 32 rows its own lanes staged as whole 256-byte rows.
      if (n_mine > 0) {
        waitx(&o_done[x], od[x] & 1, 2);
        tc_fence_after();
        const float inv_l = 1.0f / l_run;
        uint8_t* stage = smem_gen + L::OFF_Q + x * OPER_B;
#pragma unroll
        for (uint32_t c = 0; c < 4; c++) {
          uint32_t o[32];
          tmem_ld32(o_addr + 32 * c, o);
          tmem_ld_wait();
#pragma unroll
          for (int q8 = 0; q8 < 4; q8++) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
              __half2 h = __floats2half2_rn(__uint_as_float(o[8 * q8 + 2 * k]) * inv_l, __uint_as_float(o[8 * q8 + 2 * k + 1]) * inv_l);
              w[k] = *reinterpret_cast<uint32_t*>(&h);
            }
            const uint4 w4 = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(stage + r * 256 + (((4 * c + q8) ^ (r & 15)) << 4)) = w4;
          }
        }
        __syncwarp();  // a warp reads back only the 32 rows its own lanes wrote
        if constexpr (!PX) {
          // two rows per store instruction: lanes 0-15 one row of 256 bytes, lanes 16-31 the next
#pragma unroll 4
          for (uint32_t rr = 0; rr < 32; rr += 2) {
            const uint32_t row = quad * 32 + rr + (lane >> 4), u = lane & 15;
            const uint32_t tok_r = tq0[x] + row / p.qpg, head_r = g * p.qpg + row % p.qpg;
            if (tok_r >= p.m) continue;
            const uint4 v = *reinterpret_cast<const uint4*>(stage + row * 256 + ((u ^ (row & 15)) << 4));
            *reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(tok_r) * p.n_head + head_r) * BP_HEAD_DIM + 8 * u) = v;
          }
        } else {
#pragma unroll 4
          for (uint32_t rr = 0; rr < 32; rr++) {
            const uint32_t row = quad * 32 + rr;
            const uint32_t tok_r = tq0[x] + row / p.qpg, head_r = g * p.qpg + row % p.qpg;
            if (tok_r >= p.m) continue;
            const uint2 v = *reinterpret_cast<const uint2*>(stage + row * 256 + (((lane >> 1) ^ (row & 15)) << 4) + (lane & 1) * 8);
            *reinterpret_cast<uint2*>(p.out + (static_cast<size_t>(tok_r) * p.n_head + head_r) * BP_HEAD_DIM + 4 * lane) = v;
            for (uint32_t pr = 0; pr < p.n_px; pr++)
              *reinterpret_cast<uint2*>(p.px_out[pr] + static_cast<size_t>(tok_r) * p.px_row_stride + p.px_col0 +
                                        head_r * BP_HEAD_DIM + 4 * lane) = v;
          }
        }
      }
    }
    gkv += n_tiles;
#pragma unroll
    for (uint32_t x = 0; x < NQ; x++) {
      gx[x] += nx[x];
      od[x] += nx[x] > 0 ? 1u : 0u;
    }
    tc_fence_before();
    __syncthreads();  // the item is finished by every role: Q, S and O can be reused
    tc_fence_after();
  }
  if (dbg_on && (warp == 0 || warp == L::N_LOADERS || warp == L::FIRST_SM_WARP || warp == L::FIRST_SM_WARP + 4)) {
    const uint32_t role = warp == 0 ? 0 : warp == L::N_LOADERS ? 1 : warp == L::FIRST_SM_WARP ? 2 : 3;
    p.dbg[role * 8] = static_cast<unsigned long long>(clock64() - t_begin);
    for (int k = 0; k < 4; k++) p.dbg[role * 8 + 1 + k] = static_cast<unsigned long long>(tw[k]);
    p.dbg[role * 8 + 7] = gkv;
    if (role == 2) for (int k = 0; k < 4; k++) p.dbg[40 + k] = static_cast<unsigned long long>(tph[k]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, L::TMEM_COLS);
}

}  // namespace

uint32_t bp_prefill_stage_tokens() { return BN; }

// Scratch of the expanded rows and the tensor maps over it: f16 (64 dims, rows, kv_dim / 64
// chunks) with a (64, 128, 2) box, so one load yields [2 chunks][128 rows][128 B] with the
// 128-byte swizzle: the K-major operand of Q K^T and, read MN-major, the B operand of P V.
cudaError_t bp_prefill_init(bp_attn_ctx* c) {
  typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  const uint32_t max_m = bp_attn_max_prefill(c);
  c->pf_rows = (max_m + BN - 1) / BN * BN;
  const size_t halves = static_cast<size_t>(c->pf_rows) * c->kv_dim;
  cudaError_t e = cudaMalloc(&c->pf_kv16, 2 * halves * sizeof(__half) + 256);
  if (e != cudaSuccess) return e;
  e = cudaMemset(c->pf_kv16, 0, 2 * halves * sizeof(__half) + 256);
  if (e != cudaSuccess) return e;
  c->pf_counter = reinterpret_cast<uint32_t*>(c->pf_kv16 + 2 * halves);
  encode_fn encode = reinterpret_cast<encode_fn>(bp_tensor_map_encoder());
  c->have_pmaps = encode != nullptr;
  for (int kind = 0; kind < 2 && c->have_pmaps; kind++) {
    cuuint64_t dims[3] = {64, c->pf_rows, c->kv_dim / 64};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(c->kv_dim) * 2, 128};
    cuuint32_t box[3] = {64, BN, 2};
    cuuint32_t es[3] = {1, 1, 1};
    c->have_pmaps = encode(&c->pmap16[kind], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, c->pf_kv16 + kind * halves, dims, strides, box,
                           es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  if (c->have_pmaps) {  // the kernel reads the maps from device memory (a smaller parameter block: these kernels feel its size)
    e = cudaMalloc(&c->pmaps_dev, 2 * sizeof(CUtensorMap));
    if (e != cudaSuccess) return e;
    e = cudaMemcpy(c->pmaps_dev, c->pmap16, 2 * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return e;
  }
  auto allow = [](auto kernel, uint32_t bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  };
  if ((e = allow(prefill_umma_kernel<1, 1, false>, PLayout<1, 1>::SMEM)) != cudaSuccess) return e;
  if ((e = allow(prefill_umma_kernel<1, 1, true>, PLayout<1, 1>::SMEM)) != cudaSuccess) return e;
  if ((e = allow(prefill_umma_kernel<1, 2, false>, PLayout<1, 2>::SMEM)) != cudaSuccess) return e;
  if ((e = allow(prefill_umma_kernel<1, 2, true>, PLayout<1, 2>::SMEM)) != cudaSuccess) return e;
  if ((e = allow(prefill_umma_kernel<2, 1, false>, PLayout<2, 1>::SMEM)) != cudaSuccess) return e;
  return allow(prefill_umma_kernel<2, 1, true>, PLayout<2, 1>::SMEM);
}

cudaError_t bp_launch_prefill(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q,
                              __half* out, uint32_t m, uint32_t* launches) {
  const bool pow2 = (c->qpg & (c->qpg - 1)) == 0 && c->qpg <= BM;
  if (c->variant == 1 || !c->have_pmaps || !pow2) {
    if (c->n_ppx != 0) return cudaErrorNotSupported;  // the exchange lives in the tensor-core kernel's epilogue
    return bp_launch_scalar_attention(c, s, layer, q, out, m, m, true, launches);
  }
  const uint32_t rows_pad = (m + BN - 1) / BN * BN;
  {
    const uint32_t threads = rows_pad * (c->kv_dim >> 3);
    dim3 grid((threads + 255) / 256, 2);
    cudaError_t e = bp_launch(c->opt_pdl != 0, prefill_expand_kernel, grid, dim3(256), 0, s, c->kv[0], c->kv[1], bp_d_off(c, layer),
                              bp_qs_off(c, layer), c->pf_kv16, static_cast<uint64_t>(c->pf_rows) * c->kv_dim, c->kv_dim, m,
                              rows_pad, c->pf_counter);
    *launches += 1;
    if (e != cudaSuccess) return e;
  }
  PrefillParams p;
  p.q = q;
  p.out = out;
  p.err = c->err_dev;
  p.counter = c->pf_counter;
  p.m = m;
  p.n_head = c->cfg.n_head;
  p.n_kv_head = c->cfg.n_kv_head;
  p.dbg = c->dbg_on ? c->dbg_dev : nullptr;
  p.qpg = c->qpg;
  p.scale_log2 = (1.0f / sqrtf(static_cast<float>(BP_HEAD_DIM))) * 1.4426950408889634f;
  p.wait_limit = c->opt_wait_limit;
  p.n_px = c->n_ppx;
  p.px_col0 = c->cfg.shard * c->q_dim;
  p.px_row_stride = c->cfg.n_shards * c->q_dim;
  p.px_out = c->ppx_dev;
  const uint32_t tq_tokens = BM / c->qpg;
  const uint32_t sms = static_cast<uint32_t>(c->sm_count);
  // Work items of ONE query tile, two CTAs per SM, whenever there are more items than SMs: measured
  // 49.0 against 50.9 us per layer at 2048 tokens and 25.3 against 28.3 at 1024 for items of two query
  // tiles on one CTA per SM (which load every K / V tile once for both). A batch with at most one item
  // per SM runs one CTA per SM with four slots. Option prefill_tiles_per_item: 0 = that choice, 1 = one
  // tile and one CTA per SM, 2 = two tiles (one CTA per SM), 3 = one tile and two CTAs per SM.
  auto launch = [&](auto kernel, uint32_t nq, uint32_t cps, uint32_t threads, uint32_t smem) {
    p.n_groups = (m + nq * tq_tokens - 1) / (nq * tq_tokens);
    const uint32_t n_items = p.n_groups * c->cfg.n_kv_head, slots = sms * cps, grid = n_items < slots ? n_items : slots;
    *launches += 1;
    bp_note_sm_launch(c, grid < sms ? grid : sms);
    return bp_launch(c->opt_pdl != 0, kernel, dim3(grid), dim3(threads), smem, s, c->pmaps_dev, p);
  };
  const bool px = p.n_px != 0;
  if (c->opt_pf_nq == 2)
    return px ? launch(prefill_umma_kernel<2, 1, true>, 2, 1, PLayout<2, 1>::THREADS, PLayout<2, 1>::SMEM)
              : launch(prefill_umma_kernel<2, 1, false>, 2, 1, PLayout<2, 1>::THREADS, PLayout<2, 1>::SMEM);
  const uint32_t items1 = (m + tq_tokens - 1) / tq_tokens * c->cfg.n_kv_head;
  if (c->opt_pf_nq == 3 || (c->opt_pf_nq == 0 && items1 > sms))
    return px ? launch(prefill_umma_kernel<1, 2, true>, 1, 2, PLayout<1, 2>::THREADS, PLayout<1, 2>::SMEM)
              : launch(prefill_umma_kernel<1, 2, false>, 1, 2, PLayout<1, 2>::THREADS, PLayout<1, 2>::SMEM);
  return px ? launch(prefill_umma_kernel<1, 1, true>, 1, 1, PLayout<1, 1>::THREADS, PLayout<1, 1>::SMEM)
            : launch(prefill_umma_kernel<1, 1, false>, 1, 1, PLayout<1, 1>::THREADS, PLayout<1, 1>::SMEM);
}
