// Host side of the attention library: the context that owns the KV cache, the
// RoPE table and the split-KV scratch (the part of `Model` this path needs,
// src/model.rs:1148-1248), the guards of the five dispatch sites, the
// host-buffer entry points, cache import/export and the KvSnapshot blob.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>
#include <vector>

#include "bp_common.cuh"

cudaError_t bp_decode_init(bp_attn_ctx* c);
cudaError_t bp_prefill_init(bp_attn_ctx* c);
uint32_t bp_decode_stage_tokens(const bp_attn_ctx* c);
uint32_t bp_prefill_stage_tokens();

namespace {

constexpr char SNAP_MAGIC[8] = {'B', 'O', 'N', 'S', 'A', 'I', 'K', 'V'};
constexpr uint32_t SNAP_VERSION = 1;
constexpr uint64_t SNAP_HEADER = 32;

int fail(bp_attn_ctx* c, int status, const char* msg, uint32_t pos = 0, uint32_t n = 0,
         uint32_t max = 0, int cuda_error = 0) {
  if (c) {
    c->detail.status = status;
    c->detail.pos = pos;
    c->detail.n = n;
    c->detail.max = max;
    c->detail.cuda_error = cuda_error;
    snprintf(c->msg, sizeof c->msg, "%s", msg);
  }
  return status;
}

int fail_config(bp_attn_ctx* c, const char* what) {
  char buf[224];
  snprintf(buf, sizeof buf, "invalid config: %s", what);
  return fail(c, BP_ERR_CONFIG, buf);
}

int fail_overflow(bp_attn_ctx* c, uint32_t pos, uint32_t n, uint32_t max) {
  char buf[224];
  snprintf(buf, sizeof buf, "context overflow: pos %u + tokens %u > max_seq %u", pos, n, max);
  return fail(c, BP_ERR_CONTEXT_OVERFLOW, buf, pos, n, max);
}

// A failed CUDA call whose error is sticky means the context is gone for good:
// latch it, as the reference latches a lost wgpu device (src/model.rs:1081-1099).
int fail_cuda(bp_attn_ctx* c, cudaError_t e, const char* where) {
  char buf[224];
  snprintf(buf, sizeof buf, "CUDA error in %s: %s", where, cudaGetErrorString(e));
  if (c && (e == cudaErrorIllegalAddress || e == cudaErrorLaunchFailure ||
            e == cudaErrorIllegalInstruction || e == cudaErrorECCUncorrectable ||
            e == cudaErrorHardwareStackError || e == cudaErrorMisalignedAddress)) {
    c->status = BP_ERR_DEVICE_LOST;
    snprintf(buf, sizeof buf, "device lost (%s in %s)", cudaGetErrorString(e), where);
    return fail(c, BP_ERR_DEVICE_LOST, buf, 0, 0, 0, static_cast<int>(e));
  }
  return fail(c, BP_ERR_CUDA, buf, 0, 0, 0, static_cast<int>(e));
}

#define BP_CUDA(c, call)                                   \
  do {                                                     \
    cudaError_t e_ = (call);                               \
    if (e_ != cudaSuccess) return fail_cuda(c, e_, #call); \
  } while (0)

// Every compute entry point starts here (check_device, src/model.rs:1733-1741). A kernel whose
// bounded wait gave up has stored a code in the context's error word (mapped host memory): that
// latches BP_ERR_TIMEOUT, sticky like a lost device, because the merge tags and meeting counters on
// the device are undefined from then on.
int enter(bp_attn_ctx* c) {
  if (!c) return BP_ERR_NULL;
  if (c->status == BP_OK && c->err_host && *static_cast<volatile uint32_t*>(c->err_host) != 0) c->status = BP_ERR_TIMEOUT;
  if (c->status == BP_ERR_TIMEOUT)
    return fail(c, BP_ERR_TIMEOUT, "a bounded device-side wait gave up: context is unusable, snapshot it if needed and create a new one");
  if (c->status != BP_OK) return fail(c, c->status, "device lost: context is unusable, create a new one");
  return BP_OK;
}

// Entry of the calls that only copy the cache out (export, snapshot capture, introspection): they
// still work after a timeout, whose damage is confined to the scratch state of the kernels.
int enter_io(bp_attn_ctx* c) {
  const int s = enter(c);
  return s == BP_ERR_TIMEOUT ? BP_OK : s;
}

int bind_device(bp_attn_ctx* c) {
  BP_CUDA(c, cudaSetDevice(c->cfg.device));
  return BP_OK;
}

// f32 -> f16, round to nearest even (the cast of src/model.rs:1149).
uint16_t f32_to_f16(float f) {
  __half h = __float2half_rn(f);  // host path of cuda_fp16.h rounds to nearest even
  uint16_t u;
  memcpy(&u, &h, 2);
  return u;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

encode_tiled_fn get_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<encode_tiled_fn>(fn);
}

}  // namespace

void bp_note_sm_launch(bp_attn_ctx* c, uint32_t ctas) { c->sm_seq += ctas; }

// Launches that hold an SM each and lie between a write and a read bound how far the reader's
// prologue can run ahead of the writer: with more than two devices' worth of such CTAs in between,
// the writer's grid has retired before the reader's first CTA finds a free SM.
static bool recent_write(const bp_attn_ctx* c, uint32_t layer) {
  return c->opt_pdl != 0 && c->sm_seq - c->row_mark[layer] < 2ull * static_cast<uint64_t>(c->sm_count);
}

void bp_note_row_write(bp_attn_ctx* c, uint32_t layer, uint32_t row0) {
  if (recent_write(c, layer) && c->row_from[layer] < row0) row0 = c->row_from[layer];
  c->row_from[layer] = row0;
  c->row_mark[layer] = c->sm_seq;
}

uint32_t bp_fresh_from(const bp_attn_ctx* c, uint32_t layer) {
  return recent_write(c, layer) ? c->row_from[layer] : UINT32_MAX;
}

bp_launch_recorder*& bp_recorder() {
  static thread_local bp_launch_recorder* r = nullptr;
  return r;
}

void* bp_tensor_map_encoder() {
  static encode_tiled_fn encode = get_encode();
  return reinterpret_cast<void*>(encode);
}

// Tensor maps over one cache buffer. Quants: u8 (128 B, kv heads, rows) with a
// (128, 1, rows_box) box; scales: u8 (row bytes, rows) with an (inner, rows_box)
// box at byte offset `inner`-aligned. Rows run over all layers.
bool bp_make_kv_maps(bp_attn_ctx* c, int kind, uint32_t rows_box, uint32_t d_inner, bool d_swizzle,
                     CUtensorMap* map_qs, CUtensorMap* map_d) {
  static encode_tiled_fn encode = get_encode();
  if (!encode) return false;
  const CUtensorMapL2promotion promo = c->opt_l2promo == 1   ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                       : c->opt_l2promo == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                       : c->opt_l2promo == 3 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                                                             : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  const cuuint64_t rows = static_cast<cuuint64_t>(c->cfg.n_layer) * c->cfg.max_seq;
  {
    cuuint64_t dims[3] = {128, c->cfg.n_kv_head, rows};
    cuuint64_t strides[2] = {128, c->kv_dim};
    cuuint32_t box[3] = {128, 1, rows_box};
    cuuint32_t es[3] = {1, 1, 1};
    if (encode(map_qs, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, c->kv[kind] + c->d_total, dims, strides, box, es,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  {
    const uint32_t rb = c->nb * 4;
    cuuint64_t dims[2] = {rb, rows};
    cuuint64_t strides[1] = {rb};
    cuuint32_t box[2] = {d_inner, rows_box};
    cuuint32_t es[2] = {1, 1};
    if (encode(map_d, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, c->kv[kind], dims, strides, box, es,
               CU_TENSOR_MAP_INTERLEAVE_NONE, d_swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
               promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  return true;
}

// (Re)builds the decode tensor maps for the current nw / hpc options.
static size_t ll_bytes(const bp_attn_ctx* c) {
  return static_cast<size_t>(c->max_splits) * c->cfg.n_head * BP_LL_STRIDE * sizeof(uint2);
}

static bool rebuild_decode_maps(bp_attn_ctx* c) {
  c->have_maps = true;
  const uint32_t inner = 16 * c->opt_hpc;
  for (int kind = 0; kind < 2 && c->have_maps; kind++)
    c->have_maps = bp_make_kv_maps(c, kind, bp_decode_stage_tokens(c), inner, inner == 128, &c->map_qs[kind],
                                   &c->map_d[kind]);
  c->have_umaps = true;
  for (int kind = 0; kind < 2 && c->have_umaps; kind++)
    c->have_umaps = bp_make_kv_maps(c, kind, bp_decode_umma_stage_tokens(), 16 * c->opt_uhpc, false,
                                    &c->umap_qs[kind], &c->umap_d[kind]);
  if (c->have_umaps) {
    // The tcgen05 decode kernel reads its tensor maps from device memory: as kernel parameters they were 512
    // of its 900 parameter bytes, and these kernels get slower with the size of their parameter block.
    if (!c->umaps_dev && cudaMalloc(&c->umaps_dev, 4 * sizeof(CUtensorMap)) != cudaSuccess) c->have_umaps = false;
    const CUtensorMap host[4] = {c->umap_qs[0], c->umap_d[0], c->umap_qs[1], c->umap_d[1]};
    // synchronous, and after a device-wide synchronize: no launch that reads the old maps is in flight
    if (c->have_umaps && (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpy(c->umaps_dev, host, sizeof host, cudaMemcpyHostToDevice) != cudaSuccess))
      c->have_umaps = false;
  }
  return c->have_maps;
}

// Test aid: a CTA that asks for nearly all of an SM's shared memory, so that no tcgen05 decode or
// prefill CTA fits beside it, and leaves after a fixed time (bounded: at most 0.1 s).
constexpr int HOLD_SMEM = 200 * 1024;
__global__ void __launch_bounds__(32) hold_sm_kernel(unsigned long long ns) {
  extern __shared__ uint8_t hold_smem[];
  if (threadIdx.x == 0) {
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    hold_smem[0] = 1;
    do {
      __nanosleep(1000);
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    } while (t - t0 < ns && t - t0 < 100000000ull);
  }
}

extern "C" {

const char* bp_strerror(int status) {
  switch (status) {
    case BP_OK: return "ok";
    case BP_ERR_CONFIG: return "invalid config";
    case BP_ERR_CONTEXT_OVERFLOW: return "context overflow";
    case BP_ERR_PREFILL_TOO_LARGE: return "prefill batch exceeds max_prefill_tokens";
    case BP_ERR_DEVICE_LOST: return "device lost";
    case BP_ERR_CUDA: return "CUDA error";
    case BP_ERR_TIMEOUT: return "device-side wait timed out";
    case BP_ERR_NULL: return "null pointer argument";
    case BP_ERR_IO: return "io error";
    default: return "unknown status";
  }
}

int bp_attn_create(const bp_attn_config* cfg, bp_attn_ctx** out) {
  if (!cfg || !out) return BP_ERR_NULL;
  *out = nullptr;
  bp_attn_ctx* c = new (std::nothrow) bp_attn_ctx();
  if (!c) return BP_ERR_CUDA;
  memset(c, 0, sizeof *c);
  c->cfg = *cfg;
  *out = c;  // returned even on failure so the caller can read the message; destroy it either way

  // Validation, in the reference's words where it has them.
  if (cfg->head_dim != 128)
    return fail_config(c, "kv_writeback_fused.wgsl / q_norm_rope_fused.wgsl assume head_dim == 128");
  if (cfg->n_layer == 0 || cfg->n_head == 0 || cfg->n_kv_head == 0) return fail_config(c, "n_layer, n_head and n_kv_head must be > 0");
  if (cfg->n_head % cfg->n_kv_head != 0) return fail_config(c, "n_head must be a multiple of n_kv_head");
  if ((cfg->n_kv_head * cfg->head_dim) % 32 != 0) return fail_config(c, "kv_dim must be a multiple of 32 (Q8_0 block size)");
  if (cfg->max_seq == 0) return fail_config(c, "max_seq must be > 0");
  if (cfg->n_head / cfg->n_kv_head > 8) return fail_config(c, "at most 8 query heads per KV head are supported");
  if (cfg->n_kv_head != 1 && cfg->n_kv_head != 2 && cfg->n_kv_head != 4 && cfg->n_kv_head != 8)
    return fail_config(c, "a context holds 1, 2, 4 or 8 KV heads");
  if (cfg->n_shards == 0 || cfg->shard >= cfg->n_shards) return fail_config(c, "shard must be < n_shards and n_shards > 0");
  if (!(cfg->rms_eps >= 0.0f) || !(cfg->rope_freq_base > 0.0f)) return fail_config(c, "rms_eps must be >= 0 and rope_freq_base > 0");
  if (static_cast<uint64_t>(cfg->n_layer) * cfg->max_seq >= (1ull << 31)) return fail_config(c, "n_layer * max_seq must be < 2^31");

  c->q_dim = cfg->n_head * cfg->head_dim;
  c->kv_dim = cfg->n_kv_head * cfg->head_dim;
  c->nb = c->kv_dim / BP_QK8;
  c->qpg = cfg->n_head / cfg->n_kv_head;
  c->d_total = static_cast<uint64_t>(cfg->n_layer) * cfg->max_seq * c->nb * 4u;
  c->kv_bytes = c->d_total + static_cast<uint64_t>(cfg->n_layer) * cfg->max_seq * c->kv_dim;

  int n_dev = 0;
  cudaError_t e = cudaGetDeviceCount(&n_dev);
  if (e != cudaSuccess || n_dev == 0)
    return fail(c, BP_ERR_CUDA, "no CUDA device: this library has no CPU path", 0, 0, 0, static_cast<int>(e));
  if (cfg->device < 0 || cfg->device >= n_dev) return fail_config(c, "device ordinal out of range");
  BP_CUDA(c, cudaSetDevice(cfg->device));
  cudaDeviceProp prop;
  BP_CUDA(c, cudaGetDeviceProperties(&prop, cfg->device));
  if (prop.major != 10) return fail(c, BP_ERR_CUDA, "this library is built for sm_100a (B200) only");
  c->sm_count = prop.multiProcessorCount;

  BP_CUDA(c, cudaMalloc(&c->kv[0], c->kv_bytes));
  BP_CUDA(c, cudaMalloc(&c->kv[1], c->kv_bytes));

  // RoPE table: build_rope_table (src/model.rs:1756-1769) in f64, cast to f32
  // then to f16 (src/model.rs:1148-1149).
  {
    const size_t n = static_cast<size_t>(cfg->max_seq) * cfg->head_dim;
    std::vector<uint16_t> table(n);
    const uint32_t half = cfg->head_dim / 2;
    std::vector<double> theta(half);
    for (uint32_t j = 0; j < half; j++)
      theta[j] = pow(static_cast<double>(cfg->rope_freq_base), -2.0 * static_cast<double>(j) / static_cast<double>(cfg->head_dim));
    for (uint32_t p = 0; p < cfg->max_seq; p++) {
      for (uint32_t j = 0; j < half; j++) {
        const double angle = static_cast<double>(p) * theta[j];
        table[static_cast<size_t>(p) * cfg->head_dim + 2 * j] = f32_to_f16(static_cast<float>(cos(angle)));
        table[static_cast<size_t>(p) * cfg->head_dim + 2 * j + 1] = f32_to_f16(static_cast<float>(sin(angle)));
      }
    }
    BP_CUDA(c, cudaMalloc(&c->rope, n * 2));
    BP_CUDA(c, cudaMemcpy(c->rope, table.data(), n * 2, cudaMemcpyHostToDevice));
  }

  c->max_splits = bp_decode_max_splits(c);
  BP_CUDA(c, cudaMalloc(&c->partials, static_cast<size_t>(c->max_splits) * cfg->n_head * BP_PART_STRIDE * sizeof(float)));
  BP_CUDA(c, cudaMalloc(&c->ll, ll_bytes(c)));
  BP_CUDA(c, cudaMalloc(&c->epochs, 64 * sizeof(uint32_t)));
  BP_CUDA(c, cudaMemset(c->ll, 0, ll_bytes(c)));
  BP_CUDA(c, cudaMemset(c->epochs, 0, 64 * sizeof(uint32_t)));
  BP_CUDA(c, cudaMalloc(&c->dbg_dev, 64 * sizeof(unsigned long long)));
  BP_CUDA(c, cudaMemset(c->dbg_dev, 0, 64 * sizeof(unsigned long long)));
  BP_CUDA(c, cudaHostAlloc(&c->err_host, sizeof(uint32_t), cudaHostAllocMapped));
  *c->err_host = 0;
  BP_CUDA(c, cudaHostGetDevicePointer(&c->err_dev, c->err_host, 0));

  c->opt_nw = 8;
  c->opt_hpc = cfg->n_kv_head;
  c->opt_pdl = 1;
  c->opt_token_graph = 1;
  c->opt_umerge = 1;
  c->opt_uhpc = 1;  // one KV head per CTA measured faster than two at every context length tried
  c->opt_wait_limit = 1u << 22;
  c->opt_poll_limit = 1u << 18;
  c->opt_exclusive = 1;
  c->opt_vpre = 1;
  c->sm_seq = 1ull << 32;  // nothing written yet counts as written long ago
  c->row_mark = static_cast<uint64_t*>(calloc(cfg->n_layer, sizeof(uint64_t)));
  c->row_from = static_cast<uint32_t*>(calloc(cfg->n_layer, sizeof(uint32_t)));
  if (!c->row_mark || !c->row_from) return fail(c, BP_ERR_CUDA, "out of host memory");
  if (!rebuild_decode_maps(c)) return fail(c, BP_ERR_CUDA, "cuTensorMapEncodeTiled failed for the KV cache");
  BP_CUDA(c, bp_decode_init(c));
  BP_CUDA(c, bp_decode_umma_init(c));
  BP_CUDA(c, bp_prefill_init(c));
  BP_CUDA(c, cudaStreamCreateWithFlags(&c->host_stream, cudaStreamNonBlocking));
  return BP_OK;
}

// The decode launches of one token (one per layer, or two with the separate merge kernel) as a CUDA graph.
struct bp_token_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  std::vector<bp_launch_record> launches;  // as captured, with their nodes
  bp_launch_recorder patch;                // the recorder of the per-token pass (its storage is reused)
};
static void drop_token_graph(bp_attn_ctx* c) {
  if (!c->tok_graph) return;
  if (c->tok_graph->exec) cudaGraphExecDestroy(c->tok_graph->exec);
  if (c->tok_graph->graph) cudaGraphDestroy(c->tok_graph->graph);
  delete c->tok_graph;
  c->tok_graph = nullptr;
}

void bp_attn_destroy(bp_attn_ctx* c) {
  if (!c) return;
  if (c->kv[0] || c->rope) cudaSetDevice(c->cfg.device);
  cudaFree(c->kv[0]);
  cudaFree(c->kv[1]);
  cudaFree(c->rope);
  cudaFree(c->partials);
  cudaFree(c->ppx_dev);
  cudaFree(c->px_dev);
  cudaFree(c->umaps_dev);
  cudaFree(c->pmaps_dev);
  cudaFree(c->ll);
  cudaFree(c->epochs);
  cudaFree(c->px_epoch);
  cudaFree(c->pxf_dev);
  free(c->row_mark);
  free(c->row_from);
  cudaFree(c->pf_kv16);
  cudaFree(c->dbg_dev);
  if (c->err_host) cudaFreeHost(c->err_host);
  cudaFree(c->stage_q);
  cudaFree(c->stage_k);
  cudaFree(c->stage_v);
  cudaFree(c->stage_out);
  cudaFree(c->stage_wq);
  cudaFree(c->stage_wk);
  drop_token_graph(c);
  if (c->host_stream) cudaStreamDestroy(c->host_stream);
  delete c;
}

int bp_q_norm_rope(bp_attn_ctx* c, void* stream, void* q, const void* w_q_norm, uint32_t pos_base, uint32_t m) {
  if (int s = enter(c)) return s;
  if (!q || !w_q_norm) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (m == 0) return BP_OK;
  if (static_cast<uint64_t>(pos_base) + m > c->cfg.max_seq) return fail_overflow(c, pos_base, m, c->cfg.max_seq);
  c->last_launches = 0;
  BP_CUDA(c, bp_launch_q_norm_rope(c, static_cast<cudaStream_t>(stream), static_cast<__half*>(q),
                                   static_cast<const __half*>(w_q_norm), pos_base, m, &c->last_launches));
  return BP_OK;
}

int bp_kv_writeback(bp_attn_ctx* c, void* stream, uint32_t layer, const void* k_cur, const void* v_cur,
                    const void* w_k_norm, uint32_t pos_base, uint32_t m) {
  if (int s = enter(c)) return s;
  if (!k_cur || !v_cur || !w_k_norm) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (layer >= c->cfg.n_layer) return fail_config(c, "layer index out of range");
  if (static_cast<uint64_t>(pos_base) + m > c->cfg.max_seq) return fail_overflow(c, pos_base, m, c->cfg.max_seq);
  if (m == 0) return BP_OK;
  c->last_launches = 0;
  BP_CUDA(c, bp_launch_kv_writeback(c, static_cast<cudaStream_t>(stream), layer, static_cast<const __half*>(k_cur),
                                    static_cast<const __half*>(v_cur), static_cast<const __half*>(w_k_norm),
                                    pos_base, m, &c->last_launches));
  return BP_OK;
}

int bp_attn_decode(bp_attn_ctx* c, void* stream, uint32_t layer, const void* q, void* out, uint32_t cur_pos) {
  if (int s = enter(c)) return s;
  if (!q || !out) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (layer >= c->cfg.n_layer) return fail_config(c, "layer index out of range");
  if (cur_pos == 0) return fail_config(c, "decode attention needs at least one key (cur_pos >= 1)");
  if (cur_pos > c->cfg.max_seq) return fail_overflow(c, cur_pos - 1, 1, c->cfg.max_seq);
  if (c->n_px != 0 && !bp_use_umma(c))
    return fail_config(c, "the peer exchange is part of the tcgen05 decode kernel (variant 0)");
  c->last_launches = 0;
  BP_CUDA(c, bp_launch_decode(c, static_cast<cudaStream_t>(stream), layer, static_cast<const __half*>(q),
                              static_cast<__half*>(out), cur_pos, &c->last_launches));
  return BP_OK;
}

static int ensure_stage(bp_attn_ctx* c, uint32_t rows);

int bp_attn_decode_layer(bp_attn_ctx* c, void* stream, uint32_t layer, const void* q_raw, void* q_roped,
                         const void* w_q_norm, const void* k_cur, const void* v_cur, const void* w_k_norm,
                         uint32_t pos, void* out) {
  if (int s = enter(c)) return s;
  if (!q_raw || !w_q_norm || !k_cur || !v_cur || !w_k_norm || !out) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (layer >= c->cfg.n_layer) return fail_config(c, "layer index out of range");
  if (static_cast<uint64_t>(pos) + 1 > c->cfg.max_seq) return fail_overflow(c, pos, 1, c->cfg.max_seq);
  if (c->n_px != 0 && !bp_use_umma(c))
    return fail_config(c, "the peer exchange is part of the tcgen05 decode kernel (variant 0)");
  __half* qr = static_cast<__half*>(q_roped);
  if (qr == nullptr && !(c->variant == 0 && bp_use_umma(c))) {
    // the separate kernels rotate q in place: give them the context's staging row
    if (int s = bind_device(c)) return s;
    if (int s = ensure_stage(c, 1)) return s;
    qr = c->stage_q;
  }
  c->last_launches = 0;
  BP_CUDA(c, bp_launch_decode_fused(c, static_cast<cudaStream_t>(stream), layer, static_cast<const __half*>(q_raw), qr,
                                    static_cast<const __half*>(w_q_norm), static_cast<const __half*>(k_cur),
                                    static_cast<const __half*>(v_cur), static_cast<const __half*>(w_k_norm), pos,
                                    static_cast<__half*>(out), &c->last_launches));
  return BP_OK;
}

int bp_set_peer_exchange(bp_attn_ctx* c, uint32_t n_ranks, const uint64_t* out_ptrs, const uint64_t* flag_ptrs) {
  if (int s = enter(c)) return s;
  if (n_ranks == 0) {
    c->n_px = 0;
    return BP_OK;
  }
  if (!out_ptrs || !flag_ptrs) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (n_ranks != c->cfg.n_shards || n_ranks > BP_MAX_PEERS)
    return fail_config(c, "the peer exchange needs one buffer per shard (n_ranks == n_shards <= 8)");
  if (!bp_use_umma(c)) return fail_config(c, "the peer exchange is part of the tcgen05 decode kernel (4 query heads per KV head)");
  if (int s = bind_device(c)) return s;
  if (!c->px_epoch) {
    BP_CUDA(c, cudaMalloc(&c->px_epoch, 64 * sizeof(uint32_t)));
    BP_CUDA(c, cudaMemset(c->px_epoch, 0, 64 * sizeof(uint32_t)));
  }
  for (uint32_t r = 0; r < n_ranks; r++) {
    c->px_out[r] = reinterpret_cast<__half*>(static_cast<uintptr_t>(out_ptrs[r]));
    c->px_flag[r] = reinterpret_cast<uint32_t*>(static_cast<uintptr_t>(flag_ptrs[r]));
  }
  if (!c->px_dev) BP_CUDA(c, cudaMalloc(&c->px_dev, BP_MAX_PEERS * sizeof(__half*)));
  if (!c->pxf_dev) BP_CUDA(c, cudaMalloc(&c->pxf_dev, (BP_MAX_PEERS + 2) * sizeof(uint32_t*)));
  BP_CUDA(c, cudaDeviceSynchronize());  // no kernel may still read the old addresses
  BP_CUDA(c, cudaMemcpy(c->px_dev, c->px_out, n_ranks * sizeof(__half*), cudaMemcpyHostToDevice));
  {  // the decode kernel's table: every rank's counters, then this rank's two book-keeping arrays
    uint32_t* tab[BP_MAX_PEERS + 2] = {};
    for (uint32_t r = 0; r < n_ranks; r++) tab[r] = c->px_flag[r];
    tab[BP_MAX_PEERS + 1] = c->px_epoch;
    BP_CUDA(c, cudaMemcpy(c->pxf_dev, tab, sizeof tab, cudaMemcpyHostToDevice));
  }
  c->n_px = n_ranks;
  return BP_OK;
}

int bp_set_prefill_exchange(bp_attn_ctx* c, uint32_t n_ranks, const uint64_t* out_ptrs) {
  if (int s = enter(c)) return s;
  if (n_ranks == 0) {
    c->n_ppx = 0;
    return BP_OK;
  }
  if (!out_ptrs) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (n_ranks != c->cfg.n_shards || n_ranks > BP_MAX_PEERS)
    return fail_config(c, "the prefill exchange needs one buffer per shard (n_ranks == n_shards <= 8)");
  if (!c->have_pmaps || (c->qpg & (c->qpg - 1)) != 0 || c->qpg > 128)
    return fail_config(c, "the prefill exchange is part of the tensor-core prefill kernel");
  if (int s = bind_device(c)) return s;
  if (!c->ppx_dev) BP_CUDA(c, cudaMalloc(&c->ppx_dev, BP_MAX_PEERS * sizeof(__half*)));
  static_assert(sizeof(__half*) == sizeof(uint64_t), "device addresses are 64-bit");
  BP_CUDA(c, cudaDeviceSynchronize());  // no kernel may still read the old addresses
  BP_CUDA(c, cudaMemcpy(c->ppx_dev, out_ptrs, n_ranks * sizeof(uint64_t), cudaMemcpyHostToDevice));
  c->n_ppx = n_ranks;
  return BP_OK;
}

int bp_peer_sync(bp_attn_ctx* c, void* stream, uint32_t slot) {
  if (int s = enter(c)) return s;
  if (c->n_px == 0) return fail_config(c, "no peer exchange is set");
  if (slot >= 64) return fail_config(c, "peer sync slot must be below 64");
  BP_CUDA(c, bp_launch_peer_sync(c, static_cast<cudaStream_t>(stream), slot));
  return BP_OK;
}

uint32_t bp_attn_max_prefill(const bp_attn_ctx* c) {
  if (!c) return 0;
  return c->cfg.max_prefill ? (c->cfg.max_prefill < c->cfg.max_seq ? c->cfg.max_prefill : c->cfg.max_seq) : c->cfg.max_seq;
}

int bp_attn_prefill(bp_attn_ctx* c, void* stream, uint32_t layer, const void* q, void* out, uint32_t m) {
  if (int s = enter(c)) return s;
  if (!q || !out) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (layer >= c->cfg.n_layer) return fail_config(c, "layer index out of range");
  if (m == 0) return fail_config(c, "prefill needs at least one token");
  if (c->cfg.max_prefill && m > c->cfg.max_prefill) {
    char buf[224];
    snprintf(buf, sizeof buf, "prefill batch %u exceeds max_prefill_tokens %u", m, c->cfg.max_prefill);
    return fail(c, BP_ERR_PREFILL_TOO_LARGE, buf, 0, m, c->cfg.max_prefill);
  }
  if (m > c->cfg.max_seq) return fail_overflow(c, 0, m, c->cfg.max_seq);
  c->last_launches = 0;
  if (c->n_ppx != 0 && c->variant == 1)
    return fail_config(c, "the prefill exchange is part of the tensor-core prefill kernel (variant 0)");
  BP_CUDA(c, bp_launch_prefill(c, static_cast<cudaStream_t>(stream), layer, static_cast<const __half*>(q),
                               static_cast<__half*>(out), m, &c->last_launches));
  return BP_OK;
}

// ---------------------------------------------------------------------------
// Host-buffer entry points.
// ---------------------------------------------------------------------------
static int ensure_stage(bp_attn_ctx* c, uint32_t rows) {
  if (rows <= c->stage_rows) return BP_OK;
  cudaFree(c->stage_q); cudaFree(c->stage_k); cudaFree(c->stage_v); cudaFree(c->stage_out);
  c->stage_q = c->stage_k = c->stage_v = c->stage_out = nullptr;
  c->stage_rows = 0;
  BP_CUDA(c, cudaMalloc(&c->stage_q, static_cast<size_t>(rows) * c->q_dim * 2));
  BP_CUDA(c, cudaMalloc(&c->stage_out, static_cast<size_t>(rows) * c->q_dim * 2));
  BP_CUDA(c, cudaMalloc(&c->stage_k, static_cast<size_t>(rows) * c->kv_dim * 2));
  BP_CUDA(c, cudaMalloc(&c->stage_v, static_cast<size_t>(rows) * c->kv_dim * 2));
  if (!c->stage_wq) {
    BP_CUDA(c, cudaMalloc(&c->stage_wq, BP_HEAD_DIM * 2));
    BP_CUDA(c, cudaMalloc(&c->stage_wk, BP_HEAD_DIM * 2));
  }
  c->stage_rows = rows;
  return BP_OK;
}

// The two 256-byte norm weights of a host-buffer call are the same from call to call in a model: they go up
// only when their bytes differ from the last upload (two small copies less on the path of every token).
static int upload_norm_weights(bp_attn_ctx* c, cudaStream_t st, const void* wq, const void* wk) {
  if (c->stage_w_valid && memcmp(c->stage_w_host[0], wq, BP_HEAD_DIM * 2) == 0 && memcmp(c->stage_w_host[1], wk, BP_HEAD_DIM * 2) == 0)
    return BP_OK;
  c->stage_w_valid = false;
  memcpy(c->stage_w_host[0], wq, BP_HEAD_DIM * 2);
  memcpy(c->stage_w_host[1], wk, BP_HEAD_DIM * 2);
  // from the context's own copy: the caller's buffers may change as soon as the call returns
  BP_CUDA(c, cudaMemcpyAsync(c->stage_wq, c->stage_w_host[0], BP_HEAD_DIM * 2, cudaMemcpyHostToDevice, st));
  BP_CUDA(c, cudaMemcpyAsync(c->stage_wk, c->stage_w_host[1], BP_HEAD_DIM * 2, cudaMemcpyHostToDevice, st));
  c->stage_w_valid = true;
  return BP_OK;
}

static int layer_host(bp_attn_ctx* c, uint32_t layer, const void* q, const void* k, const void* v, const void* wq,
                      const void* wk, uint32_t pos_base, uint32_t m, bool prefill, void* out) {
  if (int s = enter(c)) return s;
  if (!q || !k || !v || !wq || !wk || !out) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (layer >= c->cfg.n_layer) return fail_config(c, "layer index out of range");
  if (m == 0) return fail_config(c, "at least one token is needed");
  if (prefill && c->cfg.max_prefill && m > c->cfg.max_prefill) {
    char buf[224];
    snprintf(buf, sizeof buf, "prefill batch %u exceeds max_prefill_tokens %u", m, c->cfg.max_prefill);
    return fail(c, BP_ERR_PREFILL_TOO_LARGE, buf, 0, m, c->cfg.max_prefill);
  }
  if (static_cast<uint64_t>(pos_base) + m > c->cfg.max_seq) return fail_overflow(c, pos_base, m, c->cfg.max_seq);
  if (int s = bind_device(c)) return s;
  if (int s = ensure_stage(c, m)) return s;
  cudaStream_t st = c->host_stream;
  const size_t qb = static_cast<size_t>(m) * c->q_dim * 2, kb = static_cast<size_t>(m) * c->kv_dim * 2;
  BP_CUDA(c, cudaMemcpyAsync(c->stage_q, q, qb, cudaMemcpyHostToDevice, st));
  BP_CUDA(c, cudaMemcpyAsync(c->stage_k, k, kb, cudaMemcpyHostToDevice, st));
  BP_CUDA(c, cudaMemcpyAsync(c->stage_v, v, kb, cudaMemcpyHostToDevice, st));
  if (int e = upload_norm_weights(c, st, wq, wk)) return e;
  uint32_t launches = 0;
  if (prefill) {
    BP_CUDA(c, bp_launch_q_norm_rope(c, st, c->stage_q, c->stage_wq, pos_base, m, &launches));
    BP_CUDA(c, bp_launch_kv_writeback(c, st, layer, c->stage_k, c->stage_v, c->stage_wk, pos_base, m, &launches));
    BP_CUDA(c, bp_launch_prefill(c, st, layer, c->stage_q, c->stage_out, m, &launches));
  } else if (c->variant == 0 && bp_use_umma(c)) {
    BP_CUDA(c, bp_launch_decode_fused(c, st, layer, c->stage_q, nullptr, c->stage_wq, c->stage_k, c->stage_v, c->stage_wk,
                                      pos_base, c->stage_out, &launches));
  } else {
    BP_CUDA(c, bp_launch_q_norm_rope(c, st, c->stage_q, c->stage_wq, pos_base, m, &launches));
    BP_CUDA(c, bp_launch_kv_writeback(c, st, layer, c->stage_k, c->stage_v, c->stage_wk, pos_base, m, &launches));
    BP_CUDA(c, bp_launch_decode(c, st, layer, c->stage_q, c->stage_out, pos_base + 1, &launches));
  }
  BP_CUDA(c, cudaMemcpyAsync(out, c->stage_out, qb, cudaMemcpyDeviceToHost, st));
  BP_CUDA(c, cudaStreamSynchronize(st));
  c->last_launches = launches;
  if (*c->err_host) return enter(c);  // latches BP_ERR_TIMEOUT
  return BP_OK;
}

int bp_decode_step_host(bp_attn_ctx* c, uint32_t layer, const void* q, const void* k, const void* v, const void* wq,
                        const void* wk, uint32_t pos, void* out) {
  return layer_host(c, layer, q, k, v, wq, wk, pos, 1, false, out);
}

static cudaError_t token_layer_call(bp_attn_ctx* c, cudaStream_t st, uint32_t il, uint32_t pos, uint32_t* launches) {
  return bp_launch_decode_fused(c, st, il, c->stage_q + static_cast<size_t>(il) * c->q_dim, nullptr, c->stage_wq,
                                c->stage_k + static_cast<size_t>(il) * c->kv_dim, c->stage_v + static_cast<size_t>(il) * c->kv_dim,
                                c->stage_wk, pos, c->stage_out + static_cast<size_t>(il) * c->q_dim, launches);
}

// The layers' launches of one token as ONE graph launch: kernels that follow one another in a graph start
// about a microsecond sooner than the same kernels launched into a stream. The graph is captured at the first
// token; for every later token the launcher functions run against a recorder that launches nothing, and the
// nodes take the launches they produced (the position is in every one of them). A launch of another shape
// (another kernel instance past a context-length threshold, another number of launches) captures anew.
static int token_graph_launch(bp_attn_ctx* c, cudaStream_t st, uint32_t pos, uint32_t* launches) {
  const uint32_t nl = c->cfg.n_layer;
  bool patched = false;
  if (c->tok_graph) {
    bp_launch_recorder& rec = c->tok_graph->patch;
    rec.mode = 1;
    rec.records.clear();
    bp_recorder() = &rec;
    cudaError_t e = cudaSuccess;
    for (uint32_t il = 0; il < nl && e == cudaSuccess; il++) e = token_layer_call(c, st, il, pos, launches);
    bp_recorder() = nullptr;
    BP_CUDA(c, e);
    const std::vector<bp_launch_record>& was = c->tok_graph->launches;
    patched = rec.records.size() == was.size();
    for (size_t i = 0; patched && i < was.size(); i++) {
      bp_launch_record& r = rec.records[i];
      if (r.func != was[i].func) {
        patched = false;
        break;
      }
      void* argv[BP_RECORD_MAX_ARGS];
      if (r.overflow) return fail(c, BP_ERR_CUDA, "a decode launch has more arguments than a launch record holds");
      for (uint32_t a = 0; a < r.n_args; a++) argv[a] = r.arg(a);
      cudaKernelNodeParams kp = {};
      kp.func = r.func;
      kp.gridDim = r.grid;
      kp.blockDim = r.block;
      kp.sharedMemBytes = static_cast<unsigned int>(r.smem);
      kp.kernelParams = argv;
      BP_CUDA(c, cudaGraphExecKernelNodeSetParams(c->tok_graph->exec, was[i].node, &kp));
    }
    if (!patched) *launches = 0;
  }
  if (!patched) {
    drop_token_graph(c);
    bp_token_graph* g = new bp_token_graph();
    c->tok_graph = g;
    bp_launch_recorder rec;
    rec.mode = 2;
    cudaError_t e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
      bp_recorder() = &rec;
      for (uint32_t il = 0; il < nl && e == cudaSuccess; il++) e = token_layer_call(c, st, il, pos, launches);
      bp_recorder() = nullptr;
      const cudaError_t e_end = cudaStreamEndCapture(st, &g->graph);  // always: the stream must leave capture mode
      if (e == cudaSuccess) e = e_end;
    }
    if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e != cudaSuccess) {
      drop_token_graph(c);
      BP_CUDA(c, e);
    }
    g->launches = std::move(rec.records);
  }
  BP_CUDA(c, cudaGraphLaunch(c->tok_graph->exec, st));
  return BP_OK;
}

int bp_decode_token_host(bp_attn_ctx* c, const void* q, const void* k, const void* v, const void* wq, const void* wk,
                         uint32_t pos, void* out) {
  if (int s = enter(c)) return s;
  if (!q || !k || !v || !wq || !wk || !out) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (static_cast<uint64_t>(pos) + 1 > c->cfg.max_seq) return fail_overflow(c, pos, 1, c->cfg.max_seq);
  if (int s = bind_device(c)) return s;
  const uint32_t nl = c->cfg.n_layer;
  if (int s = ensure_stage(c, nl)) return s;  // one staging row per layer
  cudaStream_t st = c->host_stream;
  const size_t qb = static_cast<size_t>(nl) * c->q_dim * 2, kb = static_cast<size_t>(nl) * c->kv_dim * 2;
  BP_CUDA(c, cudaMemcpyAsync(c->stage_q, q, qb, cudaMemcpyHostToDevice, st));
  BP_CUDA(c, cudaMemcpyAsync(c->stage_k, k, kb, cudaMemcpyHostToDevice, st));
  BP_CUDA(c, cudaMemcpyAsync(c->stage_v, v, kb, cudaMemcpyHostToDevice, st));
  if (int e = upload_norm_weights(c, st, wq, wk)) return e;
  uint32_t launches = 0;
  if (c->variant == 0 && bp_use_umma(c)) {
    // fused layer steps: the decode kernel normalises q and writes the new cache row itself
    if (c->opt_token_graph) {
      if (int s = token_graph_launch(c, st, pos, &launches)) return s;
    } else {
      for (uint32_t il = 0; il < nl; il++) BP_CUDA(c, token_layer_call(c, st, il, pos, &launches));
    }
  } else {
    // Q norm + RoPE of all layers' queries is one launch: every layer's row sits at the same position.
    BP_CUDA(c, bp_launch_q_norm_rope_rows(c, st, c->stage_q, c->stage_wq, pos, nl, &launches));
    for (uint32_t il = 0; il < nl; il++) {
      BP_CUDA(c, bp_launch_kv_writeback(c, st, il, c->stage_k + static_cast<size_t>(il) * c->kv_dim,
                                        c->stage_v + static_cast<size_t>(il) * c->kv_dim, c->stage_wk, pos, 1, &launches));
      BP_CUDA(c, bp_launch_decode(c, st, il, c->stage_q + static_cast<size_t>(il) * c->q_dim,
                                  c->stage_out + static_cast<size_t>(il) * c->q_dim, pos + 1, &launches));
    }
  }
  BP_CUDA(c, cudaMemcpyAsync(out, c->stage_out, qb, cudaMemcpyDeviceToHost, st));
  BP_CUDA(c, cudaStreamSynchronize(st));
  c->last_launches = launches;
  if (*c->err_host) return enter(c);  // latches BP_ERR_TIMEOUT
  return BP_OK;
}

int bp_prefill_layer_host(bp_attn_ctx* c, uint32_t layer, const void* q, const void* k, const void* v,
                          const void* wq, const void* wk, uint32_t m, void* out) {
  return layer_host(c, layer, q, k, v, wq, wk, 0, m, true, out);
}

// ---------------------------------------------------------------------------
// Cache sections and snapshots.
// ---------------------------------------------------------------------------
static int kv_copy(bp_attn_ctx* c, uint32_t kind, uint32_t layer, uint32_t sect, uint32_t pos, void* host, bool to_host) {
  if (int s = to_host ? enter_io(c) : enter(c)) return s;
  if (!host && pos) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (kind > 1 || sect > 1) return fail_config(c, "kind and sect must be 0 or 1");
  if (layer >= c->cfg.n_layer) return fail_config(c, "layer index out of range");
  if (pos > c->cfg.max_seq) return fail_overflow(c, 0, pos, c->cfg.max_seq);
  if (pos == 0) return BP_OK;
  if (int s = bind_device(c)) return s;
  uint8_t* dev = c->kv[kind] + (sect == 0 ? bp_d_off(c, layer) : bp_qs_off(c, layer));
  const size_t bytes = static_cast<size_t>(pos) * (sect == 0 ? c->nb * 4u : c->kv_dim);
  if (to_host) {
    BP_CUDA(c, cudaMemcpy(host, dev, bytes, cudaMemcpyDeviceToHost));
  } else {
    BP_CUDA(c, cudaMemcpy(dev, host, bytes, cudaMemcpyHostToDevice));
  }
  return BP_OK;
}

int bp_kv_export(bp_attn_ctx* c, uint32_t kind, uint32_t layer, uint32_t sect, uint32_t pos, void* host) {
  return kv_copy(c, kind, layer, sect, pos, host, true);
}
int bp_kv_import(bp_attn_ctx* c, uint32_t kind, uint32_t layer, uint32_t sect, uint32_t pos, const void* host) {
  return kv_copy(c, kind, layer, sect, pos, const_cast<void*>(host), false);
}

uint64_t bp_snapshot_payload_bytes(uint32_t n_layer, uint32_t kv_dim, uint32_t pos) {
  const uint64_t d_layer = static_cast<uint64_t>(pos) * (kv_dim / 32) * 4u;
  const uint64_t qs_layer = static_cast<uint64_t>(pos) * kv_dim;
  return 2u * static_cast<uint64_t>(n_layer) * (d_layer + qs_layer);
}

uint64_t bp_snapshot_payload_offset(uint32_t n_layer, uint32_t kv_dim, uint32_t pos, uint32_t kind, uint32_t il,
                                    uint32_t sect) {
  const uint64_t d_layer = static_cast<uint64_t>(pos) * (kv_dim / 32) * 4u;
  const uint64_t qs_layer = static_cast<uint64_t>(pos) * kv_dim;
  const uint64_t layer_bytes = d_layer + qs_layer;
  const uint64_t base = static_cast<uint64_t>(kind) * n_layer * layer_bytes + static_cast<uint64_t>(il) * layer_bytes;
  return sect == 0 ? base : base + d_layer;
}

uint64_t bp_snapshot_size(const bp_attn_ctx* c, uint32_t pos) {
  if (!c) return 0;
  return SNAP_HEADER + bp_snapshot_payload_bytes(c->cfg.n_layer, c->kv_dim * c->cfg.n_shards, pos);
}

// Strided copies between this shard's columns of the global rows and its dense
// device rows: `width` bytes at byte `col` of every `pitch`-byte global row.
static cudaError_t shard_copy(void* host_row0, size_t pitch, size_t col, uint8_t* dev, size_t width, uint32_t rows,
                              bool to_host) {
  if (to_host)
    return cudaMemcpy2D(static_cast<uint8_t*>(host_row0) + col, pitch, dev, width, width, rows, cudaMemcpyDeviceToHost);
  return cudaMemcpy2D(dev, width, static_cast<uint8_t*>(host_row0) + col, pitch, width, rows, cudaMemcpyHostToDevice);
}

int bp_snapshot_capture(bp_attn_ctx* c, uint32_t pos, void* blob, uint64_t blob_bytes) {
  if (int s = enter_io(c)) return s;
  if (!blob) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (pos > c->cfg.max_seq) return fail_overflow(c, 0, pos, c->cfg.max_seq);
  if (blob_bytes < bp_snapshot_size(c, pos)) return fail_config(c, "snapshot buffer is too small");
  if (int s = bind_device(c)) return s;
  const uint32_t kv_dim_g = c->kv_dim * c->cfg.n_shards;
  uint8_t* b = static_cast<uint8_t*>(blob);
  memcpy(b, SNAP_MAGIC, 8);
  const uint32_t hdr[6] = {SNAP_VERSION, c->cfg.n_layer, kv_dim_g, c->cfg.max_seq, pos, 0};
  memcpy(b + 8, hdr, 24);
  if (pos == 0) return BP_OK;
  uint8_t* payload = b + SNAP_HEADER;
  for (uint32_t kind = 0; kind < 2; kind++) {
    for (uint32_t il = 0; il < c->cfg.n_layer; il++) {
      uint8_t* d_dst = payload + bp_snapshot_payload_offset(c->cfg.n_layer, kv_dim_g, pos, kind, il, 0);
      uint8_t* q_dst = payload + bp_snapshot_payload_offset(c->cfg.n_layer, kv_dim_g, pos, kind, il, 1);
      BP_CUDA(c, shard_copy(d_dst, static_cast<size_t>(kv_dim_g / 32) * 4, static_cast<size_t>(c->cfg.shard) * c->nb * 4,
                            c->kv[kind] + bp_d_off(c, il), c->nb * 4, pos, true));
      BP_CUDA(c, shard_copy(q_dst, kv_dim_g, static_cast<size_t>(c->cfg.shard) * c->kv_dim,
                            c->kv[kind] + bp_qs_off(c, il), c->kv_dim, pos, true));
    }
  }
  return BP_OK;
}

int bp_snapshot_apply(bp_attn_ctx* c, const void* blob, uint64_t blob_bytes, uint32_t* pos_out) {
  if (int s = enter(c)) return s;
  if (!blob) return fail(c, BP_ERR_NULL, "null pointer argument");
  const uint8_t* b = static_cast<const uint8_t*>(blob);
  if (blob_bytes < SNAP_HEADER) return fail_config(c, "KvSnapshot blob too short: missing header");
  if (memcmp(b, SNAP_MAGIC, 8) != 0) return fail_config(c, "KvSnapshot blob has wrong magic");
  uint32_t hdr[6];
  memcpy(hdr, b + 8, 24);
  if (hdr[0] != SNAP_VERSION) return fail_config(c, "KvSnapshot blob has unsupported version");
  if (hdr[5] != 0) return fail_config(c, "KvSnapshot blob has non-zero reserved field");
  const uint32_t n_layer = hdr[1], kv_dim_g = hdr[2], pos = hdr[4];
  if (blob_bytes - SNAP_HEADER != bp_snapshot_payload_bytes(n_layer, kv_dim_g, pos))
    return fail_config(c, "KvSnapshot blob payload length does not match header");
  if (n_layer != c->cfg.n_layer || kv_dim_g != c->kv_dim * c->cfg.n_shards)
    return fail_config(c, "KvSnapshot does not match model: n_layer or kv_dim differs");
  if (pos > c->cfg.max_seq) return fail_overflow(c, 0, pos, c->cfg.max_seq);
  if (int s = bind_device(c)) return s;
  uint8_t* payload = const_cast<uint8_t*>(b) + SNAP_HEADER;
  for (uint32_t kind = 0; kind < 2 && pos; kind++) {
    for (uint32_t il = 0; il < n_layer; il++) {
      uint8_t* d_src = payload + bp_snapshot_payload_offset(n_layer, kv_dim_g, pos, kind, il, 0);
      uint8_t* q_src = payload + bp_snapshot_payload_offset(n_layer, kv_dim_g, pos, kind, il, 1);
      BP_CUDA(c, shard_copy(d_src, static_cast<size_t>(kv_dim_g / 32) * 4, static_cast<size_t>(c->cfg.shard) * c->nb * 4,
                            c->kv[kind] + bp_d_off(c, il), c->nb * 4, pos, false));
      BP_CUDA(c, shard_copy(q_src, kv_dim_g, static_cast<size_t>(c->cfg.shard) * c->kv_dim,
                            c->kv[kind] + bp_qs_off(c, il), c->kv_dim, pos, false));
    }
  }
  if (pos_out) *pos_out = pos;
  return BP_OK;
}

// ---------------------------------------------------------------------------
// Status and introspection.
// ---------------------------------------------------------------------------
int bp_ctx_status(const bp_attn_ctx* c) {
  if (!c) return BP_ERR_NULL;
  if (c->status != BP_OK) return c->status;
  // Meaningful once the stream that ran the kernels has been synchronised.
  if (c->err_host && *static_cast<volatile uint32_t*>(c->err_host)) return BP_ERR_TIMEOUT;
  return BP_OK;
}

void bp_ctx_inject_lost(bp_attn_ctx* c) {
  if (!c) return;
  c->status = BP_ERR_DEVICE_LOST;
  fail(c, BP_ERR_DEVICE_LOST, "device lost (injected by bp_ctx_inject_lost)");
}

void bp_last_error_detail(const bp_attn_ctx* c, bp_error_detail* out) {
  if (c && out) *out = c->detail;
}
const char* bp_last_error_message(const bp_attn_ctx* c) { return c ? c->msg : ""; }

void* bp_kv_device_ptr(bp_attn_ctx* c, uint32_t kind) { return (c && kind < 2) ? c->kv[kind] : nullptr; }
uint64_t bp_kv_buffer_bytes(const bp_attn_ctx* c) { return c ? c->kv_bytes : 0; }
const void* bp_rope_device_ptr(const bp_attn_ctx* c) { return c ? c->rope : nullptr; }

int bp_rope_table_copy(bp_attn_ctx* c, void* host_f16) {
  if (int s = enter_io(c)) return s;
  if (!host_f16) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (int s = bind_device(c)) return s;
  BP_CUDA(c, cudaMemcpy(host_f16, c->rope, static_cast<size_t>(c->cfg.max_seq) * BP_HEAD_DIM * 2, cudaMemcpyDeviceToHost));
  return BP_OK;
}

int bp_set_variant(bp_attn_ctx* c, uint32_t variant) {
  if (!c) return BP_ERR_NULL;
  if (variant > 3) return fail_config(c, "unknown kernel variant");
  c->variant = variant;
  return BP_OK;
}

int bp_set_option(bp_attn_ctx* c, const char* name, uint32_t value) {
  if (!c || !name) return BP_ERR_NULL;
  if (strcmp(name, "decode_warps") == 0) {
    if (value != 8 && value != 16) return fail_config(c, "decode_warps must be 8 or 16");
    c->opt_nw = value;
  } else if (strcmp(name, "decode_heads_per_cta") == 0) {
    if (value == 0 || c->cfg.n_kv_head % value != 0 || (value & (value - 1)) != 0)
      return fail_config(c, "decode_heads_per_cta must be a power of two that divides n_kv_head");
    c->opt_hpc = value;
  } else if (strcmp(name, "debug_counters") == 0) {
    c->dbg_on = value != 0;
    if (bind_device(c) != BP_OK) return BP_ERR_CUDA;
    unsigned long long init[64] = {};
    init[32] = ~0ull;  // slot 32 is a minimum
    BP_CUDA(c, cudaMemcpy(c->dbg_dev, init, sizeof init, cudaMemcpyHostToDevice));
    return BP_OK;
  } else if (strcmp(name, "decode_umma_heads_per_cta") == 0) {
    if ((value != 1 && value != 2) || c->cfg.n_kv_head % value != 0)
      return fail_config(c, "decode_umma_heads_per_cta must be 1 or 2 and divide n_kv_head");
    c->opt_uhpc = value;
    // the tags of the in-kernel merge advance per head group: a new grouping starts from a clean slate
    if (bind_device(c) != BP_OK) return BP_ERR_CUDA;
    BP_CUDA(c, cudaDeviceSynchronize());
    BP_CUDA(c, cudaMemset(c->ll, 0, ll_bytes(c)));
    BP_CUDA(c, cudaMemset(c->epochs, 0, 64 * sizeof(uint32_t)));
  } else if (strcmp(name, "decode_ring") == 0) {
    c->opt_uring = value;
    return BP_OK;
  } else if (strcmp(name, "decode_in_kernel_merge") == 0) {
    c->opt_umerge = value != 0;
    return BP_OK;
  } else if (strcmp(name, "dependent_launch") == 0) {
    c->opt_pdl = value != 0;
    return BP_OK;
  } else if (strcmp(name, "token_graph") == 0) {
    c->opt_token_graph = value != 0;
    if (!c->opt_token_graph) drop_token_graph(c);
    return BP_OK;
  } else if (strcmp(name, "wait_limit") == 0) {
    if (value == 0) return fail_config(c, "wait_limit must be > 0");
    c->opt_wait_limit = value;
    return BP_OK;
  } else if (strcmp(name, "merge_poll_limit") == 0) {
    if (value == 0) return fail_config(c, "merge_poll_limit must be > 0");
    c->opt_poll_limit = value;
    return BP_OK;
  } else if (strcmp(name, "exclusive_device") == 0) {
    if (value == 0 && c->n_px != 0)
      return fail_config(c, "the peer exchange lives in the in-kernel merge, which needs the device to itself");
    c->opt_exclusive = value != 0;
    return BP_OK;
  } else if (strcmp(name, "decode_v_preload") == 0) {
    c->opt_vpre = value != 0;
    return BP_OK;
  } else if (strcmp(name, "peer_meet_in_kernel") == 0) {
    c->opt_px_meet = value != 0;
    return BP_OK;
  } else if (strcmp(name, "tma_l2_promotion") == 0) {
    if (value > 3) return fail_config(c, "tma_l2_promotion must be 0 (256 B), 1 (128 B), 2 (64 B) or 3 (none)");
    c->opt_l2promo = value;
  } else if (strcmp(name, "prefill_tiles_per_item") == 0) {
    if (value > 3) return fail_config(c, "prefill_tiles_per_item must be 0 (by batch size), 1, 2 or 3");
    c->opt_pf_nq = value;
    return BP_OK;
  } else {
    return fail_config(c, "unknown option");
  }
  if (c->opt_hpc > c->opt_nw) c->opt_hpc = c->opt_nw;
  if (bind_device(c) != BP_OK) return BP_ERR_CUDA;
  if (!rebuild_decode_maps(c)) return fail(c, BP_ERR_CUDA, "cuTensorMapEncodeTiled failed for the KV cache");
  return BP_OK;
}

int bp_debug_counters(bp_attn_ctx* c, uint64_t* out64) {
  if (int s = enter_io(c)) return s;
  if (!out64) return fail(c, BP_ERR_NULL, "null pointer argument");
  if (int s = bind_device(c)) return s;
  BP_CUDA(c, cudaMemcpy(out64, c->dbg_dev, 64 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  return BP_OK;
}

int bp_debug_hold_sms(void* stream, uint32_t n_ctas, uint32_t microseconds) {
  if (n_ctas == 0 || n_ctas > 1024 || microseconds > 100000) return BP_ERR_CONFIG;
  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BP_ERR_CUDA;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(hold_sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, HOLD_SMEM) != cudaSuccess)
      return BP_ERR_CUDA;
    attr_set[dev] = true;
  }
  hold_sm_kernel<<<n_ctas, 32, HOLD_SMEM, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned long long>(microseconds) * 1000ull);
  return cudaGetLastError() == cudaSuccess ? BP_OK : BP_ERR_CUDA;
}

uint32_t bp_last_launch_count(const bp_attn_ctx* c) { return c ? c->last_launches : 0; }
uint32_t bp_decode_num_splits(const bp_attn_ctx* c, uint32_t cur_pos) {
  if (!c || cur_pos == 0) return 0;
  return bp_decode_splits(c, cur_pos);
}

}  // extern "C"
