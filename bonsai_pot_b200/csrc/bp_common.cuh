// Shared declarations of the attention library: the context object, launch
// entry points of each kernel file, and small device helpers.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <vector>

#include "../../include/bonsai_attn.h"

constexpr uint32_t BP_HEAD_DIM = 128;
constexpr uint32_t BP_QK8 = 32;          // Q8_0 block size
constexpr uint32_t BP_PART_STRIDE = 132; // floats per (split, head) partial: o[128], m, l, pad
constexpr uint32_t BP_LL_STRIDE = 132;   // (value, tag) pairs per (split, head) partial of the in-kernel merge: same order
constexpr uint32_t BP_MAX_PEERS = 8;     // ranks of a peer exchange

struct bp_attn_ctx {
  bp_attn_config cfg;
  uint32_t q_dim, kv_dim, nb, qpg;  // qpg = query heads per KV head
  uint64_t d_total, kv_bytes;
  uint8_t* kv[2];    // device: kv_k, kv_v (d-section then qs-section)
  __half* rope;      // device: [max_seq][64][2] (cos, sin)
  float* partials;   // device: split-KV scratch [max_splits][n_head][BP_PART_STRIDE]
  uint2* ll;         // device: tagged split partials of the in-kernel merge [max_splits][n_head][BP_LL_STRIDE] (value, tag)
  uint32_t* epochs;  // device: per head group, the tag of the last merged launch (64 words)
  uint32_t* err_host; // pinned, mapped: kernels store a non-zero code here when a bounded wait gives up
  uint32_t* err_dev;  // device alias of err_host
  uint32_t max_splits;
  unsigned long long* dbg_dev;  // 64 cycle counters written by a kernel when dbg_on
  bool dbg_on;
  // TMA descriptors over the cache, built once: quants as (128 B, kv heads,
  // rows), scales as (row bytes, rows); rows run over all layers.
  CUtensorMap map_qs[2];
  CUtensorMap map_d[2];
  bool have_maps;
  CUtensorMap umap_qs[2];  // tcgen05 decode: 128-token boxes
  CUtensorMap umap_d[2];
  CUtensorMap* umaps_dev;  // device copy of {umap_qs[0], umap_d[0], umap_qs[1], umap_d[1]}: the decode kernel takes the address
  bool have_umaps;
  // tcgen05 prefill: f16 expansion of the batch's cache rows [K | V][pf_rows][kv_dim], its
  // tensor maps (128-key boxes of one head) and the work-item counter behind it
  __half* pf_kv16;
  uint32_t pf_rows;
  uint32_t* pf_counter;
  CUtensorMap pmap16[2];
  CUtensorMap* pmaps_dev;  // device copy of pmap16[0..1]: the prefill kernel takes the address
  bool have_pmaps;
  // staging for the *_host entry points
  __half *stage_q, *stage_k, *stage_v, *stage_out, *stage_wq, *stage_wk;
  uint32_t stage_rows;
  cudaStream_t host_stream;
  uint8_t stage_w_host[2][BP_HEAD_DIM * 2];  // the norm weights last uploaded by a host-buffer call (they rarely change)
  bool stage_w_valid;
  int sm_count;
  uint32_t variant;
  uint32_t opt_nw;   // decode: compute warps per CTA (8 or 16)
  uint32_t opt_hpc;  // decode: KV heads per CTA (divides n_kv_head)
  uint32_t opt_uhpc; // tcgen05 decode: KV heads per CTA (1 or 2)
  // peer exchange of the decode outputs (bp_set_peer_exchange): each rank's gathered buffer
  // [n_layer][n_shards * q_dim] f16 and meeting counters [64], mapped into this process
  uint32_t n_px;
  __half* px_out[BP_MAX_PEERS];
  __half** px_dev;     // device copy of px_out, read by the decode kernel
  uint32_t* px_flag[BP_MAX_PEERS];
  uint32_t* px_epoch;  // device: meetings so far, per counter slot [64]
  uint32_t n_ppx;      // prefill exchange: every rank's gathered prefill buffer [rows][n_shards * q_dim]
  __half** ppx_dev;    // device: the n_ppx addresses
  uint32_t opt_uring;  // tcgen05 decode: 0 = default ring sizes, else K stages * 16 + V slots
  uint32_t opt_umerge; // tcgen05 decode: merge the splits in the decode kernel (1) or with a second kernel (0)
  uint32_t opt_pdl;  // launch the kernels of a layer with programmatic stream serialization (1) or plainly (0)
  uint32_t opt_token_graph;  // bp_decode_token_host: the layers' launches as one CUDA graph launch (1) or stream launches (0)
  struct bp_token_graph* tok_graph;  // the captured launches of bp_decode_token_host, or null
  uint32_t opt_pf_nq; // prefill: query tiles per work item (1 or 2), 0 = by batch size
  uint32_t opt_wait_limit;  // polls of an mbarrier / a meeting counter before a kernel gives up (BP_ERR_TIMEOUT)
  uint32_t opt_poll_limit;  // polling rounds of the in-kernel merge before it gives up
  uint32_t opt_exclusive;   // 1: the caller's kernels have the device to themselves (all CTAs of a launch are co-resident)
  uint32_t umma_resident;   // tcgen05 decode: CTAs the device holds at once (occupancy query), the bound of a launch whose CTAs wait for one another
  uint32_t opt_vpre;        // tcgen05 decode: request the first round of V tiles during set-up
  uint32_t opt_l2promo;     // L2 promotion of the cache tensor maps: 0 = 256 B, 1 = 128 B, 2 = 64 B, 3 = none
  uint32_t opt_px_meet;     // peer exchange: the decode kernel of layer L >= 1 holds the meeting of layer L - 1 itself
  uint32_t** pxf_dev;       // device table read by the decode kernel: px_flag[0..7], -, px_epoch
  // Dependent launches let a kernel's prologue run before earlier kernels have completed. A decode
  // kernel may request cache rows that early only when the launch that wrote them is certainly
  // complete: sm_seq counts the CTAs of kernels that hold a whole SM each; row_mark[layer] is its
  // value after the last launch that wrote rows of that layer, row_from[layer] the first row such
  // a recent launch wrote.
  uint64_t sm_seq;
  uint64_t* row_mark;
  uint32_t* row_from;
  uint32_t last_launches;
  int status;  // latched device-lost status, BP_OK otherwise
  bp_error_detail detail;
  char msg[256];
};

// Byte offset of layer `il`'s scales / quants inside a cache buffer
// (kv_layer_offsets, src/forward.rs:53-58).
__host__ __device__ inline uint64_t bp_d_off(const bp_attn_ctx* c, uint32_t il) {
  return (uint64_t)il * c->cfg.max_seq * c->nb * 4u;
}
__host__ __device__ inline uint64_t bp_qs_off(const bp_attn_ctx* c, uint32_t il) {
  return c->d_total + (uint64_t)il * c->cfg.max_seq * c->kv_dim;
}

// A launch as data: what a kernel node of a CUDA graph holds. A caller that keeps a captured step in a graph
// re-derives the launches whose arguments change from one execution to the next (the position of an attention
// call) through the ordinary launcher functions and patches the nodes with what they produced.
constexpr uint32_t BP_RECORD_MAX_ARGS = 12, BP_RECORD_ARG_BYTES = 1536;
struct bp_launch_record {
  void* func = nullptr;
  dim3 grid, block;
  size_t smem = 0;
  // the kernel arguments, one copy each, in order, in storage of the record's own (a token's 36 launches are
  // recorded before every token: no allocation on that path)
  uint32_t n_args = 0, used = 0;
  uint32_t arg_off[BP_RECORD_MAX_ARGS] = {};
  bool overflow = false;                   // an argument did not fit: the record cannot be replayed
  cudaGraphNode_t node = nullptr;          // mode 2: the node the launch became in the stream's capture
  alignas(64) uint8_t arg_bytes[BP_RECORD_ARG_BYTES];
  void* arg(uint32_t i) { return arg_bytes + arg_off[i]; }
};
// While a recorder is installed on the calling thread every bp_launch goes through it: mode 1 stores the launch
// and launches NOTHING, mode 2 launches and stores the launch with its graph node (the stream must be capturing).
struct bp_launch_recorder {
  int mode = 1;
  std::vector<bp_launch_record> records;
};
bp_launch_recorder*& bp_recorder();  // this thread's recorder, or null

template <typename T>
inline void bp_record_arg(bp_launch_record& r, const T& v) {
  const uint32_t off = (r.used + static_cast<uint32_t>(alignof(T)) - 1u) & ~(static_cast<uint32_t>(alignof(T)) - 1u);
  if (r.n_args >= BP_RECORD_MAX_ARGS || off + sizeof(T) > BP_RECORD_ARG_BYTES) {
    r.overflow = true;
    return;
  }
  memcpy(r.arg_bytes + off, &v, sizeof(T));
  r.arg_off[r.n_args++] = off;
  r.used = off + static_cast<uint32_t>(sizeof(T));
}

// Launches `kernel`; with `pdl` the launch carries programmatic stream serialization, so that the
// kernel's prologue overlaps the tail of its predecessor (the kernels call pdl_wait() themselves).
template <typename... KArgs, typename... Args>
inline cudaError_t bp_launch(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                             Args&&... args) {
  bp_launch_recorder* rec = bp_recorder();
  if (rec != nullptr) {
    rec->records.emplace_back();
    bp_launch_record& r = rec->records.back();
    r.func = reinterpret_cast<void*>(kernel);
    r.grid = grid;
    r.block = block;
    r.smem = smem;
    (bp_record_arg<KArgs>(r, static_cast<KArgs>(args)), ...);
    if (rec->mode == 1) return cudaSuccess;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e == cudaSuccess && rec != nullptr) {  // mode 2: the node this launch became (the only dependency of the stream's next node)
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    const cudaGraphNode_t* deps = nullptr;
    size_t n_deps = 0;
    e = cudaStreamGetCaptureInfo_v3(s, &st, nullptr, nullptr, &deps, nullptr, &n_deps);
    if (e == cudaSuccess && (st != cudaStreamCaptureStatusActive || n_deps != 1)) e = cudaErrorStreamCaptureUnsupported;
    if (e == cudaSuccess) rec->records.back().node = deps[0];
  }
  return e;
}

// Kernel launchers (one per kernel file). Each returns the cudaError_t of its
// launches and adds the number of kernels launched to *launches.
cudaError_t bp_launch_q_norm_rope(bp_attn_ctx* c, cudaStream_t s, __half* q, const __half* w,
                                  uint32_t pos_base, uint32_t m, uint32_t* launches);
// Same kernel over `rows` rows that all sit at the SAME position `pos` (one row per layer of one token).
cudaError_t bp_launch_q_norm_rope_rows(bp_attn_ctx* c, cudaStream_t s, __half* q, const __half* w,
                                       uint32_t pos, uint32_t rows, uint32_t* launches);
cudaError_t bp_launch_kv_writeback(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* k,
                                   const __half* v, const __half* w, uint32_t pos_base, uint32_t m,
                                   uint32_t* launches);
cudaError_t bp_launch_decode(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q,
                             __half* out, uint32_t cur_pos, uint32_t* launches);
cudaError_t bp_launch_prefill(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q,
                              __half* out, uint32_t m, uint32_t* launches);
// Meeting of the ranks of the peer exchange on counter `slot` (< 64): signal all, wait (bounded) for all.
cudaError_t bp_launch_peer_sync(bp_attn_ctx* c, cudaStream_t s, uint32_t slot);
// Book-keeping of the rule above. A launch that wrote rows [row0, ...) of `layer`; a launch of
// `ctas` CTAs that hold one SM each; the first row of `layer` a reader must not request before
// its dependency wait (UINT32_MAX: none).
void bp_note_row_write(bp_attn_ctx* c, uint32_t layer, uint32_t row0);
void bp_note_sm_launch(bp_attn_ctx* c, uint32_t ctas);
uint32_t bp_fresh_from(const bp_attn_ctx* c, uint32_t layer);
uint32_t bp_decode_splits(const bp_attn_ctx* c, uint32_t cur_pos);
uint32_t bp_decode_max_splits(const bp_attn_ctx* c);

// tcgen05 decode (bp_attn_decode_umma.cu)
cudaError_t bp_decode_umma_init(bp_attn_ctx* c);
uint32_t bp_decode_umma_stage_tokens();
uint32_t bp_decode_umma_splits(const bp_attn_ctx* c, uint32_t cur_pos);
// Extra inputs of the fused layer step: raw q goes in as `q`, the kernel normalises / rotates it and
// quantises the new token's K / V rows itself (q_roped may be null).
struct bp_fused_step {
  __half* q_roped;
  const __half *w_q, *w_k, *k_cur, *v_cur;
};
cudaError_t bp_launch_decode_umma(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q, __half* out,
                                  uint32_t cur_pos, uint32_t* n_splits_out, const bp_fused_step* fs = nullptr);
// q_norm_rope + kv_writeback at row `pos` + decode attention over pos + 1 keys as one step.
cudaError_t bp_launch_decode_fused(bp_attn_ctx* c, cudaStream_t s, uint32_t layer, const __half* q_raw, __half* q_roped,
                                   const __half* w_q, const __half* k_cur, const __half* v_cur, const __half* w_k,
                                   uint32_t pos, __half* out, uint32_t* launches);
inline bool bp_use_umma(const bp_attn_ctx* c) { return c->variant == 0 && c->qpg == 4 && c->have_umaps; }
