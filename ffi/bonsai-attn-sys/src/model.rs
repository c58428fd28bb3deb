//! Raw bindings of `include/bonsai_model.h`: the rest of the engine around the attention path
//! (single operators on Q1_0 weights, model directory, forward passes, sampler, session).
//! A host that keeps the reference's own `Model` / `Session` needs none of this; it is here
//! for hosts that want the whole engine from the library.
//!
//! UNBUILT like the rest of the crate; kept in step with the header by `tests/test_ffi_crate.py`.
#![allow(non_camel_case_types)]
use crate::{bp_attn_ctx, bp_error_detail};
use std::os::raw::{c_char, c_int, c_void};

#[repr(C)]
pub struct bp_model {
    _private: [u8; 0],
}
#[repr(C)]
pub struct bp_session {
    _private: [u8; 0],
}

/// `Config` (src/model.rs:534-556) plus the load options in force.
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct bp_model_config {
    pub n_layer: u32,
    pub n_embd: u32,
    pub n_ff: u32,
    pub n_head: u32,
    pub n_kv_head: u32,
    pub head_dim: u32,
    pub n_vocab: u32,
    pub eos_token_id: u32,
    pub q_dim: u32,
    pub kv_dim: u32,
    pub rope_freq_base: f32,
    pub rms_eps: f32,
    pub tied_embeddings: u32,
    pub max_seq: u32,
    pub m_max: u32,
}

/// `Sampler` (src/session.rs:13-35): `top_k` 0 = None, `top_p` < 0 = None.
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct bp_sampler {
    pub temperature: f32,
    pub top_k: u32,
    pub top_p: f32,
    pub seed: u64,
}

pub const BP_STOP_EOS: i32 = 0;
pub const BP_STOP_MAX_TOKENS: i32 = 1;

pub type bp_stop_fn = Option<unsafe extern "C" fn(token: u32, user: *mut c_void) -> c_int>;
pub type bp_token_fn = Option<unsafe extern "C" fn(token: u32, user: *mut c_void)>;

#[link(name = "bonsai_attn")]
extern "C" {
    // ---- operators (one per dispatch_* function of src/forward.rs) ----
    pub fn bp_op_q1_relayout(stream: *mut c_void, qs: *const c_void, bits_out: *mut c_void, n_blocks: u64) -> c_int;
    pub fn bp_op_matvec_q1_0(stream: *mut c_void, d: *const c_void, bits: *const c_void, k: u32, n: u32, x: *const c_void, y: *mut c_void, accumulate: u32) -> c_int;
    pub fn bp_op_matvec_q1_0_fused_normed(stream: *mut c_void, k: u32, x: *const c_void, w_norm: *const c_void, eps: f32, n_ranges: u32, d: *const *const c_void, bits: *const *const c_void, n: *const u32, out: *const *mut c_void) -> c_int;
    pub fn bp_op_matvec_q1_0_silu(stream: *mut c_void, d: *const c_void, bits: *const c_void, k: u32, n: u32, gate: *const c_void, up: *const c_void, y: *mut c_void, accumulate: u32) -> c_int;
    pub fn bp_op_set_matvec_rows(rows_per_lane: u32);
    pub fn bp_op_rms_norm(stream: *mut c_void, input: *const c_void, out: *mut c_void, w: *const c_void, group_size: u32, n_groups: u32, eps: f32) -> c_int;
    pub fn bp_op_silu_mul(stream: *mut c_void, gate: *const c_void, up: *const c_void, out: *mut c_void, n: u64) -> c_int;
    pub fn bp_op_embed(stream: *mut c_void, d: *const c_void, qs: *const c_void, k: u32, tokens: *const c_void, m: u32, x: *mut c_void) -> c_int;
    pub fn bp_op_quantize_q8_0(stream: *mut c_void, x: *const c_void, k: u32, m: u32, d_out: *mut c_void, qs_out: *mut c_void) -> c_int;
    pub fn bp_op_matmul_q1_0_q8_0(stream: *mut c_void, d: *const c_void, qs: *const c_void, k: u32, n: u32, m: u32, a_d: *const c_void, a_qs: *const c_void, y: *mut c_void, accumulate: u32) -> c_int;
    pub fn bp_op_set_matmul_variant(variant: u32);
    pub fn bp_op_device_status() -> c_int;
    pub fn bp_op_topk_reduce(stream: *mut c_void, logits: *const c_void, n: u32, k: u32, out_val: *mut c_void, out_idx: *mut c_void) -> c_int;

    // ---- model directory and forward passes ----
    pub fn bp_model_check_dir(dir: *const c_char, msg: *mut c_char, msg_len: usize) -> c_int;
    pub fn bp_model_load(dir: *const c_char, max_seq: u32, device: i32, out: *mut *mut bp_model) -> c_int;
    pub fn bp_model_free(m: *mut bp_model);
    pub fn bp_model_get_config(m: *const bp_model, out: *mut bp_model_config) -> c_int;
    pub fn bp_model_last_error(m: *const bp_model) -> *const c_char;
    pub fn bp_model_error_detail(m: *const bp_model, out: *mut bp_error_detail);
    pub fn bp_model_attn(m: *mut bp_model) -> *mut bp_attn_ctx;
    pub fn bp_model_step_topk(m: *mut bp_model, token: u32, pos: u32, k: u32, logits: *mut f32, indices: *mut u32) -> c_int;
    pub fn bp_model_set_step_graph(m: *mut bp_model, enable: u32) -> c_int;
    pub fn bp_model_graph_steps(m: *const bp_model) -> u64;
    pub fn bp_model_prefill_topk(m: *mut bp_model, tokens: *const u32, n: u32, k: u32, logits: *mut f32, indices: *mut u32) -> c_int;
    pub fn bp_model_prefill_loop_topk(m: *mut bp_model, tokens: *const u32, n: u32, pos_base: u32, k: u32, logits: *mut f32, indices: *mut u32) -> c_int;
    pub fn bp_model_read_hidden(m: *mut bp_model, row: u32, x_host: *mut c_void) -> c_int;
    pub fn bp_model_read_logits(m: *mut bp_model, logits_host: *mut c_void) -> c_int;
    pub fn bp_model_attn_tap(m: *mut bp_model, mode: u32, buf_host: *mut c_void) -> c_int;

    // ---- sampler and session ----
    pub fn bp_sampler_default(s: *mut bp_sampler);
    pub fn bp_effective_k(s: *const bp_sampler) -> u32;
    pub fn bp_uniform_f32(seed: u64) -> f32;
    pub fn bp_sample_from_topk(logits: *const f32, indices: *const u32, n: u32, s: *const bp_sampler, pos: u32) -> u32;
    pub fn bp_session_create(m: *mut bp_model, out: *mut *mut bp_session) -> c_int;
    pub fn bp_session_free(s: *mut bp_session);
    pub fn bp_session_pos(s: *const bp_session) -> u32;
    pub fn bp_session_reset(s: *mut bp_session);
    pub fn bp_session_prefill(s: *mut bp_session, tokens: *const u32, n: u32, sampler: *const bp_sampler, chosen: *mut u32) -> c_int;
    pub fn bp_session_prefill_one_at_a_time(s: *mut bp_session, tokens: *const u32, n: u32, sampler: *const bp_sampler, chosen: *mut u32) -> c_int;
    pub fn bp_session_step(s: *mut bp_session, token: u32, sampler: *const bp_sampler, chosen: *mut u32) -> c_int;
    pub fn bp_session_generate(s: *mut bp_session, first_token: u32, max_new_tokens: u32, sampler: *const bp_sampler, stop: bp_stop_fn, on_token: bp_token_fn, user: *mut c_void, out_tokens: *mut u32, n_out: *mut u32, stop_reason: *mut i32) -> c_int;
    pub fn bp_session_snapshot_size(s: *const bp_session) -> u64;
    pub fn bp_session_snapshot(s: *mut bp_session, blob: *mut c_void, blob_bytes: u64) -> c_int;
    pub fn bp_session_restore(s: *mut bp_session, blob: *const c_void, blob_bytes: u64) -> c_int;
}
