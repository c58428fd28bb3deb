/*
 * bonsai_attn.h - C ABI of the B200 (sm_100a) attention hot path for bonsai-pot.
 *
 * The reference engine (Rust + WGSL on wgpu) has no plugin seam for this path:
 * its five attention dispatch sites are private functions of src/forward.rs
 * that record compute dispatches on buffers owned by `Model`. This header cuts
 * the seam at those five sites. Each entry point names the reference interface
 * it replaces (paths relative to the reference repository). A Rust `-sys`
 * crate, or any other FFI, binds exactly these symbols.
 *
 * Conventions (mirroring the reference):
 *   - One opaque context owns the KV cache (`kv_k`, `kv_v`), the RoPE table and
 *     the split-KV scratch, as `Model` does (src/model.rs:1184-1248). Callers
 *     own the activations and pass raw DEVICE pointers to IEEE binary16 data
 *     (pointer = the reference's `act` buffer + element offset).
 *   - A context is not thread-safe and serves one sequence at a time
 *     (src/session.rs:69-88). Every call is asynchronous on the CUDA stream it
 *     is given (`void*` = `cudaStream_t`, NULL = the default stream); nothing
 *     synchronises except the `*_host` calls, import/export and snapshots.
 *   - Guards run before any GPU work and return a status, never abort
 *     (src/session.rs:163-176, src/forward.rs:982-994). A lost device latches:
 *     every later call returns BP_ERR_DEVICE_LOST (src/model.rs:1733-1741).
 *   - KV cache bytes are the reference's: per buffer a d-section of FP32 block
 *     scales followed by a qs-section of int8 quants (src/forward.rs:40-58).
 *   - There is no CPU fallback: without a CUDA device every compute entry point
 *     returns BP_ERR_CUDA.
 */
#ifndef BONSAI_ATTN_H
#define BONSAI_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct bp_attn_ctx bp_attn_ctx;

/* Status codes; the comment names the `PotError` variant each one carries
 * (src/error.rs:7-40). */
enum {
  BP_OK = 0,
  BP_ERR_CONFIG = 1,            /* PotError::Config(&str) */
  BP_ERR_CONTEXT_OVERFLOW = 2,  /* PotError::ContextOverflow { pos, n, max } */
  BP_ERR_PREFILL_TOO_LARGE = 3, /* PotError::PrefillTooLarge { n, max } */
  BP_ERR_DEVICE_LOST = 4,       /* PotError::DeviceLost */
  BP_ERR_CUDA = 5,              /* a CUDA runtime/driver call failed (no reference counterpart) */
  BP_ERR_TIMEOUT = 6,           /* a bounded device-side wait gave up (a TMA / MMA barrier inside a kernel, or the
                                   meeting of the ranks): the kernel wound down instead of hanging; its results and
                                   the context's device-side counters are undefined. Sticky, like DeviceLost: take a
                                   snapshot if the cache is still wanted, destroy the context, create a new one. */
  BP_ERR_NULL = 7,              /* a required pointer argument was NULL */
  BP_ERR_IO = 8                 /* PotError::Io { path, source }: a model file could not be read (bonsai_model.h) */
};

/* The fields of the reference's `Config` + `LoadOptions` that this path reads
 * (src/model.rs:534-566, 658-837). Validation rules are the reference's:
 * head_dim == 128 (src/model.rs:1179-1183), kv_dim % 32 == 0
 * (src/model.rs:1174-1178), n_head % n_kv_head == 0 (src/model.rs:672-676),
 * max_seq > 0. */
typedef struct bp_attn_config {
  uint32_t n_layer;
  uint32_t n_head;    /* query heads held by THIS context (a shard holds n_head_global / n_shards) */
  uint32_t n_kv_head; /* KV heads held by THIS context */
  uint32_t head_dim;  /* must be 128 */
  uint32_t max_seq;
  float rms_eps;
  float rope_freq_base;
  uint32_t max_prefill; /* 0 = no cap; 512 reproduces the reference's M_MAX (src/model.rs:502) */
  uint32_t n_shards;    /* KV-head shards the model is split into: 1, 2, 4 or 8 */
  uint32_t shard;       /* index of this shard, < n_shards */
  int32_t device;       /* CUDA device ordinal */
} bp_attn_config;

/* Struct fields of the last error (ContextOverflow / PrefillTooLarge). */
typedef struct bp_error_detail {
  int32_t status;
  uint32_t pos, n, max;
  int32_t cuda_error;
} bp_error_detail;

/* Replaces the KV-cache / RoPE-table / attn_partials part of
 * `Model::load_with_options` (src/model.rs:1148-1165, 1174-1248, 1756-1769).
 * Cache contents are undefined after creation, as in the reference. */
int bp_attn_create(const bp_attn_config* cfg, bp_attn_ctx** out);
void bp_attn_destroy(bp_attn_ctx* ctx);

/* `dispatch_q_norm_rope_fused` (src/forward.rs:392-413, params
 * src/model.rs:255-262, kernel src/shaders/q_norm_rope_fused.wgsl).
 * q: device f16 [m][n_head*128], normalised and rotated in place. */
int bp_q_norm_rope(bp_attn_ctx* ctx, void* stream, void* q, const void* w_q_norm, uint32_t pos_base,
                   uint32_t m);

/* `dispatch_kv_writeback_fused` (src/forward.rs:359-388, params
 * src/model.rs:265-276, kernel src/shaders/kv_writeback_fused.wgsl).
 * k_cur, v_cur: device f16 [m][n_kv_head*128]; writes cache rows
 * [pos_base, pos_base + m) of `layer`. pos_base + m > max_seq gives
 * BP_ERR_CONTEXT_OVERFLOW. */
int bp_kv_writeback(bp_attn_ctx* ctx, void* stream, uint32_t layer, const void* k_cur,
                    const void* v_cur, const void* w_k_norm, uint32_t pos_base, uint32_t m);

/* The `attention_split` + `attention_merge` pair of `layer_post_kv_in_pass`
 * (src/forward.rs:822-856, params src/model.rs:213-234). q, out: device f16
 * [n_head*128]. cur_pos = pos + 1 keys are attended (the new token included);
 * 1 <= cur_pos <= max_seq. */
int bp_attn_decode(bp_attn_ctx* ctx, void* stream, uint32_t layer, const void* q, void* out,
                   uint32_t cur_pos);

/* One decode step of one layer as ONE call: what `encode_step_matvec` does
 * with three dispatches (src/forward.rs:612-631: q_norm_rope_fused,
 * kv_writeback_fused at row `pos`, attention_split + attention_merge over
 * pos + 1 keys). Same arithmetic and the same cache bytes as the three
 * separate calls; on the tcgen05 decode path the decode kernel does the Q
 * norm + RoPE and the new row's quantisation itself, which removes two kernel
 * boundaries per layer. q_raw: device f16 [n_head*128], NOT modified;
 * q_roped: device f16 [n_head*128] receiving the normalised, rotated q, or
 * NULL when the caller has no use for it; k_cur, v_cur: device f16
 * [n_kv_head*128]; out: device f16 [n_head*128]. Asynchronous on `stream`. */
int bp_attn_decode_layer(bp_attn_ctx* ctx, void* stream, uint32_t layer, const void* q_raw, void* q_roped,
                         const void* w_q_norm, const void* k_cur, const void* v_cur, const void* w_k_norm,
                         uint32_t pos, void* out);

/* Peer exchange of the decode outputs between KV-head shards (no counterpart
 * in the reference, which runs on one device). out_ptrs[r] / flag_ptrs[r] are
 * device addresses, valid IN THIS PROCESS, of rank r's gathered output buffer
 * (f16 [n_layer][n_shards * n_head * 128]) and of its meeting counters
 * (uint32 [64], zero at the start); r = 0 .. n_ranks-1 with n_ranks ==
 * n_shards, this rank's own buffers included (peer-mapped memory: CUDA IPC,
 * VMM or a symmetric-memory allocator). From then on the tcgen05 decode kernel
 * stores every output element of its heads into all ranks' gathered buffers
 * (row = layer, columns of this shard) as it produces them: the all-gather of
 * head outputs happens inside the kernel's epilogue, by peer stores over
 * NVLink. The stores are complete when the kernel is. n_ranks = 0 switches the
 * exchange off. */
int bp_set_peer_exchange(bp_attn_ctx* ctx, uint32_t n_ranks, const uint64_t* out_ptrs,
                         const uint64_t* flag_ptrs);
/* The same for batched prefill: out_ptrs[r] is the device address, valid in
 * this process, of rank r's gathered prefill output (f16 [rows][n_shards *
 * n_head * 128], rows >= the largest m passed to bp_attn_prefill). From then
 * on the tensor-core prefill kernel stores every output vector of its heads
 * into all ranks' gathered buffers as well (row = token, columns of this
 * shard). The ranks meet with bp_peer_sync (whose counters come from
 * bp_set_peer_exchange). n_ranks = 0 switches it off. */
int bp_set_prefill_exchange(bp_attn_ctx* ctx, uint32_t n_ranks, const uint64_t* out_ptrs);
/* Meeting point of the ranks, enqueued on `stream`: tells every rank that this
 * rank's kernels up to here have completed (their peer stores included) and
 * waits (bounded; a timeout latches BP_ERR_TIMEOUT) until every rank has said
 * so on counter `slot` (< 64; each slot counts its own meetings). Call it
 * where the gathered outputs are needed: after a layer's decode call with slot
 * = layer mod 64 when the next operation consumes that layer's gathered row,
 * or once per token when nothing in between does. */
int bp_peer_sync(bp_attn_ctx* ctx, void* stream, uint32_t slot);
/* Meeting without a kernel of its own: with the option "peer_meet_in_kernel" = 1
 * the tcgen05 decode kernel of every layer L >= 1 holds the meeting of layer
 * L - 1 on slot (L - 1) mod 64 itself. Once the kernels before it on the stream
 * are complete (layer L - 1's peer stores have landed by then) one of its
 * threads tells every rank, and before the grid ends one thread waits (bounded;
 * a timeout latches BP_ERR_TIMEOUT) until every rank has said so: the decode
 * kernel stands in for the consumer of layer L - 1's gathered row, and the
 * meeting costs no launch and lies off the kernel's own critical path. The
 * caller must then NOT call bp_peer_sync for those slots; the LAST layer's row
 * has no next layer and is met with bp_peer_sync(ctx, stream, (n_layer - 1) mod
 * 64) once per token. All ranks must make the same calls in the same order. */

/* `dispatch_attention(.., pos = 0, m_tokens = m, is_prefill = true)`
 * (src/forward.rs:501-532, params src/model.rs:195-210, kernel
 * src/shaders/attention.wgsl). q, out: device f16 [m][n_head*128]; token i
 * attends to cache rows [0, i]. m > max_prefill (when non-zero) gives
 * BP_ERR_PREFILL_TOO_LARGE, m > max_seq gives BP_ERR_CONTEXT_OVERFLOW. */
int bp_attn_prefill(bp_attn_ctx* ctx, void* stream, uint32_t layer, const void* q, void* out,
                    uint32_t m);

/* Largest m `bp_attn_prefill` accepts (the reference's
 * `Model::max_prefill_tokens`, src/model.rs:502). */
uint32_t bp_attn_max_prefill(const bp_attn_ctx* ctx);

/* One decode step of one layer with HOST buffers: copies q, k_cur, v_cur
 * (f16, pinned or pageable) to the device, runs q_norm_rope, kv_writeback at
 * row `pos`, decode attention over pos + 1 keys, copies the f16 [n_head*128]
 * result back and synchronises. This is the sequence of
 * `encode_step_matvec` for one layer (src/forward.rs:612-631) as seen from a
 * host that keeps its activations in host memory. */
int bp_decode_step_host(bp_attn_ctx* ctx, uint32_t layer, const void* q_host, const void* k_host,
                        const void* v_host, const void* w_q_norm_host, const void* w_k_norm_host,
                        uint32_t pos, void* out_host);

/* One decode token through ALL layers with HOST buffers: the attention part of
 * one `Session::step` (src/forward.rs:578-672), which the reference submits as
 * a single command buffer per token. q_host, out_host: f16 [n_layer][n_head*128];
 * k_host, v_host: f16 [n_layer][n_kv_head*128]. One host-to-device copy per
 * input, the kernels of every layer in order, one copy back, one synchronise. */
int bp_decode_token_host(bp_attn_ctx* ctx, const void* q_host, const void* k_host, const void* v_host,
                         const void* w_q_norm_host, const void* w_k_norm_host, uint32_t pos,
                         void* out_host);

/* One prefill pass of one layer with HOST buffers (the three dispatches of
 * `layer_step_matmul_in_pass`, src/forward.rs:1141-1172): q [m][n_head*128],
 * k, v [m][n_kv_head*128] in, out [m][n_head*128] back, synchronised. */
int bp_prefill_layer_host(bp_attn_ctx* ctx, uint32_t layer, const void* q_host, const void* k_host,
                          const void* v_host, const void* w_q_norm_host, const void* w_k_norm_host,
                          uint32_t m, void* out_host);

/* Cache section copies, the per-layer copies of `kv_snapshot::capture` /
 * `apply` (src/kv_snapshot.rs:204-372). kind: 0 = K, 1 = V; sect: 0 = d
 * (FP32 scales, pos * kv_dim/32 * 4 bytes), 1 = qs (int8, pos * kv_dim
 * bytes); rows [0, pos). `host` is host memory. Synchronous. */
int bp_kv_export(bp_attn_ctx* ctx, uint32_t kind, uint32_t layer, uint32_t sect, uint32_t pos,
                 void* host);
int bp_kv_import(bp_attn_ctx* ctx, uint32_t kind, uint32_t layer, uint32_t sect, uint32_t pos,
                 const void* host);

/* `KvSnapshot` blob ("BONSAIKV" v1): 32-byte header + payload
 * (src/kv_snapshot.rs:8-17, 30-32, 69-80, 150-169). */
uint64_t bp_snapshot_payload_bytes(uint32_t n_layer, uint32_t kv_dim, uint32_t pos);
uint64_t bp_snapshot_payload_offset(uint32_t n_layer, uint32_t kv_dim, uint32_t pos, uint32_t kind,
                                    uint32_t layer, uint32_t sect);
/* Size of the whole blob (header included) for `pos` tokens of this context. */
uint64_t bp_snapshot_size(const bp_attn_ctx* ctx, uint32_t pos);
/* `Session::snapshot` -> `KvSnapshot::to_bytes`: writes bp_snapshot_size bytes.
 * On a sharded context the blob is written in the GLOBAL row order: header
 * kv_dim = n_shards * local kv_dim, and only this shard's columns of each row
 * are touched, so n_shards calls on the same buffer assemble the full blob. */
int bp_snapshot_capture(bp_attn_ctx* ctx, uint32_t pos, void* blob, uint64_t blob_bytes);
/* `KvSnapshot::from_bytes` + `validate_against` + `kv_snapshot::apply`
 * (src/kv_snapshot.rs:104-140, 184-199, 312-372). Returns the restored `pos`
 * in *pos_out. Header errors give BP_ERR_CONFIG, pos > max_seq gives
 * BP_ERR_CONTEXT_OVERFLOW { pos: 0, n: pos, max }. */
int bp_snapshot_apply(bp_attn_ctx* ctx, const void* blob, uint64_t blob_bytes, uint32_t* pos_out);

/* `Model::is_device_lost` / `check_device` (src/model.rs:1719-1741): BP_OK or
 * the latched status. */
int bp_ctx_status(const bp_attn_ctx* ctx);
/* Host-side stand-in for `Model::__destroy_device_for_test`
 * (src/model.rs:1743-1751): latches BP_ERR_DEVICE_LOST without touching the
 * GPU, so every later call fails fast. */
void bp_ctx_inject_lost(bp_attn_ctx* ctx);
void bp_last_error_detail(const bp_attn_ctx* ctx, bp_error_detail* out);
/* Display text of the last error, in the wording of src/error.rs:7-40. */
const char* bp_last_error_message(const bp_attn_ctx* ctx);
const char* bp_strerror(int status);

/* Introspection for tests, benchmarks and an exchange layer built on top. */
void* bp_kv_device_ptr(bp_attn_ctx* ctx, uint32_t kind);       /* whole kv_k / kv_v buffer */
uint64_t bp_kv_buffer_bytes(const bp_attn_ctx* ctx);           /* size of each */
const void* bp_rope_device_ptr(const bp_attn_ctx* ctx);        /* f16 [max_seq][64][2] */
int bp_rope_table_copy(bp_attn_ctx* ctx, void* host_f16);      /* host copy of the same */
/* Selects the decode kernel family: 0 = production (tcgen05 int8 UMMA; falls
 * back to 3 when the context has other than 4 query heads per KV head), 1 = plain
 * CUDA-core cross-check kernels, 2 = warp-MMA kernel with the conservative int8
 * expansion, 3 = warp-MMA kernel. */
int bp_set_variant(bp_attn_ctx* ctx, uint32_t variant);
/* Tuning knobs of the decode kernel: "decode_warps" (8 or 16 compute warps per
 * CTA) and "decode_heads_per_cta" (KV heads streamed by one CTA; a power of two
 * dividing n_kv_head), "decode_umma_heads_per_cta" (1 or 2, tcgen05 decode) and
 * "prefill_tiles_per_item" (layout of the prefill kernel: 1 = work items of one
 * query tile, one CTA per SM; 2 = two query tiles, one CTA per SM; 3 = one query
 * tile, two CTAs per SM; 0 = chosen by batch size: 3 when there are more work
 * items than SMs, else 1). Launch structure: "dependent_launch" (1 = kernels are
 * launched with programmatic stream serialization, the default), "token_graph" (1 = the
 * layers' launches of bp_decode_token_host go to the device as one CUDA graph launch, its
 * nodes given the new position's launch arguments before every token, the default; 0 =
 * stream launches), "decode_in_kernel_merge"
 * (1 = the tcgen05 decode kernel merges its splits itself, the default; 0 = a
 * second kernel does), "decode_ring" (K stages * 16 + V slots of the tcgen05
 * decode kernel, 0 = as many as fit), "decode_v_preload" (1 = the first round of
 * V tiles is requested during set-up, the default), "tma_l2_promotion" (0 = 256 B,
 * the default, 1 = 128 B, 2 = 64 B, 3 = none). Results do not depend on any of
 * them beyond rounding. The in-kernel merge keeps per-context state on the device
 * (a tag per launch): compute calls on one context must not overlap on different
 * streams.
 * Co-residency: with the in-kernel merge the CTAs of a head group wait (bounded)
 * for one another's partials, which is only correct when every CTA of the launch
 * is resident at once. The grid is sized from the runtime's occupancy figure for
 * an otherwise idle device; a caller whose other work (another stream, another
 * process through MPS, a green context) may hold SMs while decode runs must set
 * "exclusive_device" = 0: the splits are then merged by a second kernel that
 * waits for nobody. Left at 1 on a shared device, a launch whose CTAs cannot all
 * start ends in BP_ERR_TIMEOUT after "merge_poll_limit" polling rounds (default
 * 2^18, about 0.2 us each). The peer exchange needs "exclusive_device" = 1.
 * Bounds of the device-side waits: "wait_limit" (polls of an mbarrier or of a
 * meeting counter before a kernel gives up, default 2^22) and "merge_poll_limit".
 * Peer exchange: "peer_meet_in_kernel" (see above, after bp_peer_sync). */
int bp_set_option(bp_attn_ctx* ctx, const char* name, uint32_t value);
/* Development aid: with the option "debug_counters" set to 1 the tcgen05 decode
 * kernel's first CTA records, per warp role (producer, UMMA issuer, softmax,
 * accumulate), its cycles in the main loop and in each kind of wait; this call
 * synchronises and copies the 64 counters (8 per role) to the host. */
int bp_debug_counters(bp_attn_ctx* ctx, uint64_t* out64);
/* Test aid: occupies `n_ctas` SMs (one CTA each, holding nearly all of the SM's
 * shared memory so that no tcgen05 CTA fits beside it) for `microseconds`
 * (at most 100000) on `stream`, then leaves. Used to test decode under
 * co-tenancy ("exclusive_device" = 0) without a second process. */
int bp_debug_hold_sms(void* stream, uint32_t n_ctas, uint32_t microseconds);
/* Number of kernels the last compute call launched. */
uint32_t bp_last_launch_count(const bp_attn_ctx* ctx);
/* Number of split-KV partitions `bp_attn_decode` uses at `cur_pos`. */
uint32_t bp_decode_num_splits(const bp_attn_ctx* ctx, uint32_t cur_pos);

/* No counterpart in the reference. Decode attention for callers that cannot
 * allocate device memory where they call it - a host whose allocator owns all
 * of the GPU, a plugin inside someone else's process, a no-allocation region of
 * a serving loop. It takes no context: the caller passes the query, the two
 * whole cache buffers in the reference layout (d-section then qs-section, see
 * bp_kv_device_ptr) and the output, and the split-KV scratch is a fixed array
 * inside the library image (about 1.1 MB on every GPU that loads the library,
 * held until exit). After the first call on a device the call allocates
 * nothing (the first one makes the CUDA runtime load the library's device code
 * and looks up the array's device address; make it before any stream capture).
 * It runs the plain CUDA-core kernels, not the tcgen05 kernel of
 * bp_attn_decode: its result agrees with bp_attn_decode's within the attention
 * tolerance (|x - ref| <= 2e-3 + 1e-2 |ref|), not bit for bit, and a call is
 * several times slower (DESIGN.md gives the measured times). Limits: n_head <=
 * 64 (BP_ERR_CONFIG beyond that; use bp_attn_decode), head_dim 128, at most 32
 * splits (longer contexts get longer splits). The CURRENT device must be the one
 * that holds the cache, the other buffers and the stream (a cache on another
 * device gives BP_ERR_CONFIG). All calls share the one array: calls that overlap
 * on the GPU race, so keep them on one stream. Nothing has to be cleared
 * between calls. Asynchronous on `stream`. */
int bp_attn_decode_static_scratch(void* stream, const void* q, const void* kv_k, const void* kv_v, void* out,
                                  uint32_t n_layer, uint32_t max_seq, uint32_t n_head, uint32_t n_kv_head,
                                  uint32_t layer, uint32_t cur_pos);

#ifdef __cplusplus
}
#endif
#endif /* BONSAI_ATTN_H */
