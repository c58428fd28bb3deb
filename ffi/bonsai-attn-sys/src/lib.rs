//! Raw bindings of `include/bonsai_attn.h`, the C ABI of the B200 attention path
//! (`libbonsai_attn.so`), plus the mapping of its status codes to the reference's
//! `PotError` (src/error.rs:7-40).
//!
//! UNBUILT: no Rust toolchain exists where this repository is developed, so this crate has
//! never been compiled. It is kept in step with the header by a test that parses this file
//! (`tests/test_ffi_crate.py`: every exported function, its argument count, every status
//! constant and the two `repr(C)` structs).
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_int, c_void};

/// `include/bonsai_model.h`: operators, model directory, forward passes, sampler, session.
pub mod model;

/// Opaque context: owns `kv_k`, `kv_v`, the RoPE table and the split-KV scratch
/// (what `Model` owns for this path, src/model.rs:1148-1248).
#[repr(C)]
pub struct bp_attn_ctx {
    _private: [u8; 0],
}

/// `bp_attn_config`: the fields of `Config` + `LoadOptions` this path reads
/// (src/model.rs:534-566, 658-837).
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct bp_attn_config {
    pub n_layer: u32,
    pub n_head: u32,
    pub n_kv_head: u32,
    pub head_dim: u32,
    pub max_seq: u32,
    pub rms_eps: f32,
    pub rope_freq_base: f32,
    /// 512 = the reference's M_MAX (src/model.rs:502); 0 = no cap.
    pub max_prefill: u32,
    pub n_shards: u32,
    pub shard: u32,
    pub device: i32,
}

/// Struct fields of the last error (`ContextOverflow { pos, n, max }`, `PrefillTooLarge { n, max }`).
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct bp_error_detail {
    pub status: i32,
    pub pos: u32,
    pub n: u32,
    pub max: u32,
    pub cuda_error: i32,
}

pub const BP_OK: c_int = 0;
pub const BP_ERR_CONFIG: c_int = 1;
pub const BP_ERR_CONTEXT_OVERFLOW: c_int = 2;
pub const BP_ERR_PREFILL_TOO_LARGE: c_int = 3;
pub const BP_ERR_DEVICE_LOST: c_int = 4;
pub const BP_ERR_CUDA: c_int = 5;
pub const BP_ERR_TIMEOUT: c_int = 6;
pub const BP_ERR_NULL: c_int = 7;
pub const BP_ERR_IO: c_int = 8;

#[link(name = "bonsai_attn")]
extern "C" {
    pub fn bp_attn_create(cfg: *const bp_attn_config, out: *mut *mut bp_attn_ctx) -> c_int;
    pub fn bp_attn_destroy(ctx: *mut bp_attn_ctx);
    pub fn bp_q_norm_rope(
        ctx: *mut bp_attn_ctx, stream: *mut c_void, q: *mut c_void, w_q_norm: *const c_void, pos_base: u32,
        m: u32
    ) -> c_int;
    pub fn bp_kv_writeback(
        ctx: *mut bp_attn_ctx, stream: *mut c_void, layer: u32, k_cur: *const c_void, v_cur: *const c_void,
        w_k_norm: *const c_void, pos_base: u32, m: u32
    ) -> c_int;
    pub fn bp_attn_decode(
        ctx: *mut bp_attn_ctx, stream: *mut c_void, layer: u32, q: *const c_void, out: *mut c_void, cur_pos: u32
    ) -> c_int;
    pub fn bp_attn_decode_layer(
        ctx: *mut bp_attn_ctx, stream: *mut c_void, layer: u32, q_raw: *const c_void, q_roped: *mut c_void,
        w_q_norm: *const c_void, k_cur: *const c_void, v_cur: *const c_void, w_k_norm: *const c_void, pos: u32,
        out: *mut c_void
    ) -> c_int;
    pub fn bp_set_peer_exchange(
        ctx: *mut bp_attn_ctx, n_ranks: u32, out_ptrs: *const u64, flag_ptrs: *const u64
    ) -> c_int;
    pub fn bp_set_prefill_exchange(ctx: *mut bp_attn_ctx, n_ranks: u32, out_ptrs: *const u64) -> c_int;
    pub fn bp_peer_sync(ctx: *mut bp_attn_ctx, stream: *mut c_void, slot: u32) -> c_int;
    pub fn bp_attn_prefill(
        ctx: *mut bp_attn_ctx, stream: *mut c_void, layer: u32, q: *const c_void, out: *mut c_void, m: u32
    ) -> c_int;
    pub fn bp_attn_max_prefill(ctx: *const bp_attn_ctx) -> u32;
    pub fn bp_decode_step_host(
        ctx: *mut bp_attn_ctx, layer: u32, q_host: *const c_void, k_host: *const c_void, v_host: *const c_void,
        w_q_norm_host: *const c_void, w_k_norm_host: *const c_void, pos: u32, out_host: *mut c_void
    ) -> c_int;
    pub fn bp_decode_token_host(
        ctx: *mut bp_attn_ctx, q_host: *const c_void, k_host: *const c_void, v_host: *const c_void,
        w_q_norm_host: *const c_void, w_k_norm_host: *const c_void, pos: u32, out_host: *mut c_void
    ) -> c_int;
    pub fn bp_prefill_layer_host(
        ctx: *mut bp_attn_ctx, layer: u32, q_host: *const c_void, k_host: *const c_void, v_host: *const c_void,
        w_q_norm_host: *const c_void, w_k_norm_host: *const c_void, m: u32, out_host: *mut c_void
    ) -> c_int;
    pub fn bp_kv_export(
        ctx: *mut bp_attn_ctx, kind: u32, layer: u32, sect: u32, pos: u32, host: *mut c_void
    ) -> c_int;
    pub fn bp_kv_import(
        ctx: *mut bp_attn_ctx, kind: u32, layer: u32, sect: u32, pos: u32, host: *const c_void
    ) -> c_int;
    pub fn bp_snapshot_payload_bytes(n_layer: u32, kv_dim: u32, pos: u32) -> u64;
    pub fn bp_snapshot_payload_offset(n_layer: u32, kv_dim: u32, pos: u32, kind: u32, layer: u32, sect: u32) -> u64;
    pub fn bp_snapshot_size(ctx: *const bp_attn_ctx, pos: u32) -> u64;
    pub fn bp_snapshot_capture(ctx: *mut bp_attn_ctx, pos: u32, blob: *mut c_void, blob_bytes: u64) -> c_int;
    pub fn bp_snapshot_apply(ctx: *mut bp_attn_ctx, blob: *const c_void, blob_bytes: u64, pos_out: *mut u32) -> c_int;
    pub fn bp_ctx_status(ctx: *const bp_attn_ctx) -> c_int;
    pub fn bp_ctx_inject_lost(ctx: *mut bp_attn_ctx);
    pub fn bp_last_error_detail(ctx: *const bp_attn_ctx, out: *mut bp_error_detail);
    pub fn bp_last_error_message(ctx: *const bp_attn_ctx) -> *const c_char;
    pub fn bp_strerror(status: c_int) -> *const c_char;
    pub fn bp_kv_device_ptr(ctx: *mut bp_attn_ctx, kind: u32) -> *mut c_void;
    pub fn bp_kv_buffer_bytes(ctx: *const bp_attn_ctx) -> u64;
    pub fn bp_rope_device_ptr(ctx: *const bp_attn_ctx) -> *const c_void;
    pub fn bp_rope_table_copy(ctx: *mut bp_attn_ctx, host_f16: *mut c_void) -> c_int;
    pub fn bp_set_variant(ctx: *mut bp_attn_ctx, variant: u32) -> c_int;
    pub fn bp_set_option(ctx: *mut bp_attn_ctx, name: *const c_char, value: u32) -> c_int;
    pub fn bp_debug_counters(ctx: *mut bp_attn_ctx, out64: *mut u64) -> c_int;
    pub fn bp_debug_hold_sms(stream: *mut c_void, n_ctas: u32, microseconds: u32) -> c_int;
    pub fn bp_last_launch_count(ctx: *const bp_attn_ctx) -> u32;
    pub fn bp_decode_num_splits(ctx: *const bp_attn_ctx, cur_pos: u32) -> u32;
    pub fn bp_attn_decode_static_scratch(
        stream: *mut c_void, q: *const c_void, kv_k: *const c_void, kv_v: *const c_void, out: *mut c_void,
        n_layer: u32, max_seq: u32, n_head: u32, n_kv_head: u32, layer: u32, cur_pos: u32
    ) -> c_int;
}

/// The error type of the host crate, restated here so that this file stands alone; a real
/// integration uses `bonsai_pot::PotError` (src/error.rs:7-40) instead.
#[derive(Debug)]
pub enum AttnError {
    /// `PotError::Config(&str)`
    Config(String),
    /// `PotError::ContextOverflow { pos, n, max }`
    ContextOverflow { pos: u32, n: u32, max: u32 },
    /// `PotError::PrefillTooLarge { n, max }`
    PrefillTooLarge { n: u32, max: u32 },
    /// `PotError::DeviceLost`: the context is unusable for good. A device-side wait that ran
    /// out (`BP_ERR_TIMEOUT`) and a sticky CUDA error belong here too: both are latched by the
    /// library, every later compute call fails fast, and recovery is the reference's (snapshot
    /// if wanted, new context, restore; tests/gpu_integration.rs:268-336).
    DeviceLost { status: c_int, message: String },
}

/// Maps a status of this ABI to the error a `Session` / `Model` method returns.
///
/// # Safety
/// `ctx` must be a live context, or null when `st` came from a call that takes none.
pub unsafe fn check(ctx: *const bp_attn_ctx, st: c_int) -> Result<(), AttnError> {
    if st == BP_OK {
        return Ok(());
    }
    let mut d = bp_error_detail::default();
    let mut message = String::new();
    if !ctx.is_null() {
        bp_last_error_detail(ctx, &mut d);
        let p = bp_last_error_message(ctx);
        if !p.is_null() {
            message = std::ffi::CStr::from_ptr(p).to_string_lossy().into_owned();
        }
    }
    if message.is_empty() {
        message = std::ffi::CStr::from_ptr(bp_strerror(st)).to_string_lossy().into_owned();
    }
    Err(match st {
        BP_ERR_CONTEXT_OVERFLOW => AttnError::ContextOverflow { pos: d.pos, n: d.n, max: d.max },
        BP_ERR_PREFILL_TOO_LARGE => AttnError::PrefillTooLarge { n: d.n, max: d.max },
        BP_ERR_DEVICE_LOST | BP_ERR_TIMEOUT | BP_ERR_CUDA => AttnError::DeviceLost { status: st, message },
        BP_ERR_CONFIG | BP_ERR_NULL | BP_ERR_IO => AttnError::Config(message),
        _ => AttnError::Config(message),
    })
}

/// `Model::check_device` (src/model.rs:1733-1741).
///
/// # Safety
/// `ctx` must be a live context.
pub unsafe fn check_device(ctx: *const bp_attn_ctx) -> Result<(), AttnError> {
    check(ctx, bp_ctx_status(ctx))
}
