/*
 * bonsai_model.h - C ABI of the engine AROUND the attention path: model directory,
 * the non-attention operators of a layer, one-token and batched forward passes, the
 * sampler and the session loop. Same conventions as bonsai_attn.h (status codes,
 * opaque owners, device pointers to f16 activations, no torch types); the attention
 * inside every forward pass is the library's own (bonsai_attn.h).
 *
 * Each entry names the reference interface it stands for (paths inside the reference
 * repository). Results of the operators are the reference's bit for bit under the
 * evaluation rules stated at the top of oracle/engine.c (the CPU restatement these
 * kernels are tested against); attention outputs keep their own tolerance.
 */
#ifndef BONSAI_MODEL_H
#define BONSAI_MODEL_H

#include <stddef.h>
#include <stdint.h>

#include "bonsai_attn.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- operators (device pointers; asynchronous on `stream`) -------------------------
 * A Q1_0 tensor [n][k] is given by its two arrays as the model directory stores them
 * (manifest d_offset / qs_offset, src/model.rs:586-606): `d` = f16 block scales
 * [n][k/128], `qs` = sign bytes [n][k/128][16]. The one-token matvec kernels read the
 * signs in a layout of their own: `bits` = bp_op_q1_relayout(qs), same size as `qs`. */
int bp_op_q1_relayout(void* stream, const void* qs, void* bits_out, uint64_t n_blocks);
/* dispatch_matvec_q1_0 (src/forward.rs:212-248, matvec_q1_0.wgsl): y[n] (+)= W x */
int bp_op_matvec_q1_0(void* stream, const void* d, const void* bits, uint32_t k, uint32_t n, const void* x, void* y,
                      uint32_t accumulate);
/* dispatch_matvec_q1_0_fused_normed (src/forward.rs:287-334, matvec_q1_0_fused_normed.wgsl): up to three
 * tensors over rms_norm(x) * w_norm; every n[i] must be a multiple of 16. */
int bp_op_matvec_q1_0_fused_normed(void* stream, uint32_t k, const void* x, const void* w_norm, float eps, uint32_t n_ranges,
                                   const void* const* d, const void* const* bits, const uint32_t* n, void* const* out);
/* dispatch_matvec_q1_0_silu (src/forward.rs:250-285, matvec_q1_0_silu.wgsl): y (+)= W (silu(gate) * up) */
int bp_op_matvec_q1_0_silu(void* stream, const void* d, const void* bits, uint32_t k, uint32_t n, const void* gate, const void* up,
                           void* y, uint32_t accumulate);
/* Tuning aid of the three matvec kernels: rows a lane works on at once, 1, 2 or 4 (0 = chosen by the
 * tensor's height, the default); + 8 = only the general kernel instances (tensors of 4096 and 12288 inputs
 * otherwise run instances compiled for that width). Results do not depend on it. Process-wide. */
void bp_op_set_matvec_rows(uint32_t rows_per_lane);
/* dispatch_rms_norm (src/forward.rs:188-210, rms_norm.wgsl); in == out allowed */
int bp_op_rms_norm(void* stream, const void* in, void* out, const void* w, uint32_t group_size, uint32_t n_groups, float eps);
/* dispatch_silu_mul (src/forward.rs:474-499, silu_mul.wgsl) */
int bp_op_silu_mul(void* stream, const void* gate, const void* up, void* out, uint64_t n);
/* the embed dispatch of encode_step_matvec / prefill_matmul_topk (src/forward.rs:593-606, embed.wgsl);
 * tokens: device uint32 [m] */
int bp_op_embed(void* stream, const void* d, const void* qs, uint32_t k, const void* tokens, uint32_t m, void* x);
/* dispatch_quantize_act (src/forward.rs:415-441, quantize_q8_0.wgsl): d_out f32 [m][k/32], qs_out int8 [m][k] */
int bp_op_quantize_q8_0(void* stream, const void* x, uint32_t k, uint32_t m, void* d_out, void* qs_out);
/* dispatch_matmul_q1_0 (src/forward.rs:443-472, matmul_q1_0_q8_0.wgsl): y[m][n] (+)= A W^T */
int bp_op_matmul_q1_0_q8_0(void* stream, const void* d, const void* qs, uint32_t k, uint32_t n, uint32_t m, const void* a_d,
                           const void* a_qs, void* y, uint32_t accumulate);
/* Tuning aid of the matmul: 0 = chosen by the batch (CUDA cores up to 32 tokens, mma.sync above, the
 * default), 1 = CUDA cores (dp4a), 2 = mma.sync (int8; tiles of 128 tokens, of 64, or whole waves of the former and
 * the rest as the latter, whichever fills the device's waves best), 3 = tcgen05 (f16 operands), 4 / 5 = mma.sync with tiles of 64 / 128 tokens only. Results do not
 * depend on it. Process-wide. */
void bp_op_set_matmul_variant(uint32_t variant);
/* The tcgen05 matmul waits on barriers, with a bound. Synchronizes the device and returns BP_ERR_TIMEOUT
 * if such a wait of a bp_op_matmul_q1_0_q8_0 launch gave up since the last call (its output is then
 * unspecified), BP_ERR_CUDA if the device reports an error, else BP_OK. A model reports the same through
 * its own status. */
int bp_op_device_status(void);
/* dispatch_topk_reduce (src/forward.rs:336-357, topk_reduce.wgsl): the min(k, 32) largest logits, descending,
 * with their indices; out_val f32, out_idx uint32 (device) */
int bp_op_topk_reduce(void* stream, const void* logits, uint32_t n, uint32_t k, void* out_val, void* out_idx);

/* ---- model directory ------------------------------------------------------------- */
typedef struct bp_model bp_model;

/* The hyper-parameters of config.ini (`Config`, src/model.rs:534-556) plus the load options in force. */
typedef struct bp_model_config {
  uint32_t n_layer, n_embd, n_ff, n_head, n_kv_head, head_dim, n_vocab, eos_token_id, q_dim, kv_dim;
  float rope_freq_base, rms_eps;
  uint32_t tied_embeddings;
  uint32_t max_seq; /* LoadOptions::max_seq */
  uint32_t m_max;   /* Model::max_prefill_tokens = 512 (src/model.rs:502) */
} bp_model_config;

/* parse_config_ini + validate_cfg (src/model.rs:568-837) on the host only: BP_OK, BP_ERR_IO (config.ini
 * cannot be read) or BP_ERR_CONFIG with the reference's message in `msg`. */
int bp_model_check_dir(const char* dir, char* msg, size_t msg_len);
/* Model::load_with_options (src/model.rs:861-1620): reads config.ini and the five weight files, uploads
 * them, creates the attention context (max_seq positions). `*out` is set even on failure (message). */
int bp_model_load(const char* dir, uint32_t max_seq, int32_t device, bp_model** out);
void bp_model_free(bp_model* m);
int bp_model_get_config(const bp_model* m, bp_model_config* out);
const char* bp_model_last_error(const bp_model* m);
void bp_model_error_detail(const bp_model* m, bp_error_detail* out);
/* The attention context the model owns (cache export / import, options, status). */
bp_attn_ctx* bp_model_attn(bp_model* m);

/* step_matvec_topk (src/forward.rs:733-745; encode_step_matvec :578-672): one token at position `pos` through every layer, then
 * output_norm, LM head and top-k; logits / indices: host arrays of k <= 32 entries. Synchronous. */
int bp_model_step_topk(bp_model* m, uint32_t token, uint32_t pos, uint32_t k, float* logits, uint32_t* indices);
/* bp_model_step_topk runs as ONE CUDA graph launch by default (token copy, embed, every layer, output suffix,
 * result copies), captured at the first step; before each later step the attention nodes are given the
 * launch arguments of the new position, and the step is captured again when those launches change shape
 * (another kernel instance past a context-length threshold). Same kernels, same arguments, same results as
 * the stream launches; enable = 0 returns to those. The graph is used with the tcgen05 decode kernel
 * (4 query heads per KV head, kernel family 0) and while the attention tap is off. */
int bp_model_set_step_graph(bp_model* m, uint32_t enable);
/* Steps that ran as a graph launch since the model was loaded. */
uint64_t bp_model_graph_steps(const bp_model* m);
/* prefill_matmul_topk (src/forward.rs:975-1073; layer_step_matmul_in_pass :1075-1253): n <= m_max tokens at positions 0 .. n - 1, batched. */
int bp_model_prefill_topk(bp_model* m, const uint32_t* tokens, uint32_t n, uint32_t k, float* logits, uint32_t* indices);
/* prefill_matvec_loop_topk (src/forward.rs:914-968): the one-token path over every token, any pos_base. */
int bp_model_prefill_loop_topk(bp_model* m, const uint32_t* tokens, uint32_t n, uint32_t pos_base, uint32_t k, float* logits,
                               uint32_t* indices);
/* Test hook: row `row` of the residual stream `x` after the last forward pass (f16 [n_embd], host),
 * and the f16 logits of the last forward pass (host [n_vocab]). */
int bp_model_read_hidden(bp_model* m, uint32_t row, void* x_host);
int bp_model_read_logits(bp_model* m, void* logits_host);
/* Test hook: attention outputs of layer `layer` are copied to / taken from host memory around the
 * attention call of the next bp_model_step_topk (f16 [n_layer][q_dim]). mode 0 = off, 1 = record
 * into buf, 2 = replace by buf. Lets the non-attention operators be compared bit for bit with the
 * CPU restatement while the attention kernel keeps its own tolerance. */
int bp_model_attn_tap(bp_model* m, uint32_t mode, void* buf_host);

/* ---- sampler and session ----------------------------------------------------------- */
/* `Sampler` (src/session.rs:13-35): top_k 0 = None, top_p < 0 = None. */
typedef struct bp_sampler {
  float temperature;
  uint32_t top_k;
  float top_p;
  uint64_t seed;
} bp_sampler;
void bp_sampler_default(bp_sampler* s);                                     /* Sampler::default */
uint32_t bp_effective_k(const bp_sampler* s);                               /* effective_k, src/session.rs:346-352 */
float bp_uniform_f32(uint64_t seed);                                        /* uniform_f32, src/session.rs:419-428 */
/* sample_from_topk (src/session.rs:357-417): host function, no GPU. */
uint32_t bp_sample_from_topk(const float* logits, const uint32_t* indices, uint32_t n, const bp_sampler* s, uint32_t pos);

typedef struct bp_session bp_session;
enum { BP_STOP_EOS = 0, BP_STOP_MAX_TOKENS = 1 }; /* StopReason */
int bp_session_create(bp_model* m, bp_session** out);  /* Model::new_session */
void bp_session_free(bp_session* s);
uint32_t bp_session_pos(const bp_session* s);
void bp_session_reset(bp_session* s);
/* Session::prefill (src/session.rs:162-183): needs pos == 0 (BP_ERR_CONFIG otherwise). */
int bp_session_prefill(bp_session* s, const uint32_t* tokens, uint32_t n, const bp_sampler* sampler, uint32_t* chosen);
/* Session::prefill_one_at_a_time (src/session.rs:185-200) */
int bp_session_prefill_one_at_a_time(bp_session* s, const uint32_t* tokens, uint32_t n, const bp_sampler* sampler, uint32_t* chosen);
/* Session::step (src/session.rs:202-216) */
int bp_session_step(bp_session* s, uint32_t token, const bp_sampler* sampler, uint32_t* chosen);
/* Session::generate_streaming (src/session.rs:229-344). stop: called with every sampled token, non-zero
 * ends the run with BP_STOP_EOS (the token is not emitted); NULL = the model's eos_token_id. on_token:
 * called with every emitted token, may be NULL. out_tokens (may be NULL) receives up to max_new_tokens. */
typedef int (*bp_stop_fn)(uint32_t token, void* user);
typedef void (*bp_token_fn)(uint32_t token, void* user);
int bp_session_generate(bp_session* s, uint32_t first_token, uint32_t max_new_tokens, const bp_sampler* sampler, bp_stop_fn stop,
                        bp_token_fn on_token, void* user, uint32_t* out_tokens, uint32_t* n_out, int32_t* stop_reason);
/* Session::snapshot / restore (src/session.rs:124-140): the blob of bp_snapshot_capture at the session's pos. */
uint64_t bp_session_snapshot_size(const bp_session* s);
int bp_session_snapshot(bp_session* s, void* blob, uint64_t blob_bytes);
int bp_session_restore(bp_session* s, const void* blob, uint64_t blob_bytes);

#ifdef __cplusplus
}
#endif
#endif /* BONSAI_MODEL_H */
