"""Host-side mirror of the reference's attention dispatch sites.

`AttnContext` plays the part of `Model` for this path (it owns the KV cache, the
RoPE table and the split-KV scratch, src/model.rs:1148-1248) and exposes the
five dispatches of src/forward.rs under the reference's names:

    dispatch_q_norm_rope_fused    src/forward.rs:392-413
    dispatch_kv_writeback_fused   src/forward.rs:359-388
    dispatch_attention            src/forward.rs:501-532  (batched prefill)
    dispatch_attention_decode     src/forward.rs:822-856  (attention_split + attention_merge)

Every method calls straight into the C ABI of include/bonsai_attn.h; there is no
Python or CPU implementation behind it. Arguments are device pointers
(`int`) or anything with a `data_ptr()` (a CUDA torch tensor).
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from .errors import raise_for_status

HEAD_DIM = 128


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):  # numpy array (host entry points only)
        return x.ctypes.data
    raise TypeError(f"cannot take a pointer from {type(x)!r}")


def _stream(stream):
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream  # torch.cuda.Stream


class AttnContext:
    """Owns the Q8_0 KV cache of one model (or of one KV-head shard of it)."""

    def __init__(self, n_layer=36, n_head=32, n_kv_head=8, max_seq=1024, rms_eps=1e-6, rope_freq_base=1e6,
                 head_dim=HEAD_DIM, max_prefill=0, n_shards=1, shard=0, device=0):
        self._lib = _lib.load()
        self._h = C.c_void_p()
        self.cfg = _lib.Config(n_layer, n_head, n_kv_head, head_dim, max_seq, rms_eps, rope_freq_base,
                               max_prefill, n_shards, shard, device)
        st = self._lib.bp_attn_create(C.byref(self.cfg), C.byref(self._h))
        if st != 0:
            msg = self._message()
            self.close()
            raise_for_status(st, msg)
        self.n_layer, self.n_head, self.n_kv_head, self.max_seq = n_layer, n_head, n_kv_head, max_seq
        self.q_dim, self.kv_dim = n_head * head_dim, n_kv_head * head_dim
        self.nb = self.kv_dim // 32

    # -- plumbing ----------------------------------------------------------
    def _message(self):
        return (self._lib.bp_last_error_message(self._h) or b"").decode() if self._h else ""

    def _check(self, st):
        if st == 0:
            return
        d = _lib.ErrorDetail()
        self._lib.bp_last_error_detail(self._h, C.byref(d))
        raise_for_status(st, self._message(), pos=d.pos, n=d.n, max=d.max, cuda_error=d.cuda_error)

    def close(self):
        if self._h:
            self._lib.bp_attn_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- the five dispatch sites ------------------------------------------
    def dispatch_q_norm_rope_fused(self, q, w_q_norm, pos_base, m_tokens, stream=None):
        """q: f16 [m][n_head*128], normalised + rotated in place."""
        self._check(self._lib.bp_q_norm_rope(self._h, _stream(stream), _ptr(q), _ptr(w_q_norm), pos_base, m_tokens))

    def dispatch_kv_writeback_fused(self, layer_il, k_cur, v_cur, w_k_norm, pos_base, m_tokens, stream=None):
        """k_cur, v_cur: f16 [m][n_kv_head*128] -> cache rows [pos_base, pos_base + m)."""
        self._check(self._lib.bp_kv_writeback(self._h, _stream(stream), layer_il, _ptr(k_cur), _ptr(v_cur),
                                              _ptr(w_k_norm), pos_base, m_tokens))

    def dispatch_attention_decode(self, layer_il, q, out, cur_pos, stream=None):
        """attention_split + attention_merge: q, out f16 [n_head*128]; keys [0, cur_pos)."""
        self._check(self._lib.bp_attn_decode(self._h, _stream(stream), layer_il, _ptr(q), _ptr(out), cur_pos))

    def decode_layer(self, layer_il, q_raw, w_q_norm, k_cur, v_cur, w_k_norm, pos, out, q_roped=None, stream=None):
        """One decode step of one layer as one call (q_norm_rope_fused + kv_writeback_fused at row
        `pos` + decode attention over pos + 1 keys). q_raw is not modified; q_roped (optional)
        receives the normalised, rotated q."""
        self._check(self._lib.bp_attn_decode_layer(self._h, _stream(stream), layer_il, _ptr(q_raw),
                                                   _ptr(q_roped) if q_roped is not None else None, _ptr(w_q_norm),
                                                   _ptr(k_cur), _ptr(v_cur), _ptr(w_k_norm), pos, _ptr(out)))

    def set_peer_exchange(self, out_ptrs, flag_ptrs):
        """Peer exchange of decode outputs: device addresses (valid in this process) of every rank's
        gathered buffer [n_layer][n_shards*n_head*128] f16 and meeting counters [64] uint32."""
        n = len(out_ptrs)
        arr_o = (C.c_uint64 * max(n, 1))(*[int(p) for p in out_ptrs])
        arr_f = (C.c_uint64 * max(n, 1))(*[int(p) for p in flag_ptrs])
        self._check(self._lib.bp_set_peer_exchange(self._h, n, arr_o, arr_f))

    def set_prefill_exchange(self, out_ptrs):
        """Peer exchange of prefill outputs: device addresses (valid in this process) of every rank's
        gathered buffer [rows][n_shards*n_head*128] f16; an empty list switches it off."""
        n = len(out_ptrs)
        arr_o = (C.c_uint64 * max(n, 1))(*[int(p) for p in out_ptrs])
        self._check(self._lib.bp_set_prefill_exchange(self._h, n, arr_o))

    def peer_sync(self, slot=0, stream=None):
        """Meeting of the ranks on the stream: this rank's kernels so far are complete (peer stores
        included), and so are every other rank's up to their matching call."""
        self._check(self._lib.bp_peer_sync(self._h, _stream(stream), slot))

    def dispatch_attention(self, layer_il, q, out, m_tokens, stream=None):
        """Batched prefill (pos = 0, is_prefill = true): q, out f16 [m][n_head*128]."""
        self._check(self._lib.bp_attn_prefill(self._h, _stream(stream), layer_il, _ptr(q), _ptr(out), m_tokens))

    def max_prefill_tokens(self):
        return self._lib.bp_attn_max_prefill(self._h)

    # -- host-buffer entry points -----------------------------------------
    def decode_step_host(self, layer_il, q, k_cur, v_cur, w_q_norm, w_k_norm, pos, out):
        self._check(self._lib.bp_decode_step_host(self._h, layer_il, _ptr(q), _ptr(k_cur), _ptr(v_cur),
                                                  _ptr(w_q_norm), _ptr(w_k_norm), pos, _ptr(out)))

    def decode_token_host(self, q, k_cur, v_cur, w_q_norm, w_k_norm, pos, out):
        """All layers of one decode token: q/out [n_layer][q_dim], k/v [n_layer][kv_dim], host memory."""
        self._check(self._lib.bp_decode_token_host(self._h, _ptr(q), _ptr(k_cur), _ptr(v_cur), _ptr(w_q_norm),
                                                   _ptr(w_k_norm), pos, _ptr(out)))

    def prefill_layer_host(self, layer_il, q, k_cur, v_cur, w_q_norm, w_k_norm, m_tokens, out):
        self._check(self._lib.bp_prefill_layer_host(self._h, layer_il, _ptr(q), _ptr(k_cur), _ptr(v_cur),
                                                    _ptr(w_q_norm), _ptr(w_k_norm), m_tokens, _ptr(out)))

    # -- cache sections ------------------------------------------------------
    def kv_export(self, kind, layer_il, sect, pos, host):
        self._check(self._lib.bp_kv_export(self._h, kind, layer_il, sect, pos, _ptr(host)))

    def kv_import(self, kind, layer_il, sect, pos, host):
        self._check(self._lib.bp_kv_import(self._h, kind, layer_il, sect, pos, _ptr(host)))

    def kv_device_ptr(self, kind):
        return self._lib.bp_kv_device_ptr(self._h, kind)

    def kv_buffer_bytes(self):
        return self._lib.bp_kv_buffer_bytes(self._h)

    def rope_table(self):
        """Host copy of the f16 RoPE table as a numpy array [max_seq][128]."""
        import numpy as np
        out = np.empty((self.max_seq, HEAD_DIM), dtype=np.float16)
        self._check(self._lib.bp_rope_table_copy(self._h, out.ctypes.data))
        return out

    # -- status ---------------------------------------------------------------
    def is_device_lost(self):
        return self._lib.bp_ctx_status(self._h) == 4

    def status(self):
        return self._lib.bp_ctx_status(self._h)

    def inject_device_lost(self):
        """Test hook: latch the lost-device state on the host (no GPU fault)."""
        self._lib.bp_ctx_inject_lost(self._h)

    def set_variant(self, variant):
        self._check(self._lib.bp_set_variant(self._h, variant))

    def set_option(self, name, value):
        """Decode tuning knobs: "decode_warps" (8/16), "decode_heads_per_cta"."""
        self._check(self._lib.bp_set_option(self._h, name.encode(), value))

    def debug_counters(self):
        """64 cycle counters of the last tcgen05 decode launch (option "debug_counters" must be 1)."""
        buf = (C.c_uint64 * 64)()
        self._check(self._lib.bp_debug_counters(self._h, buf))
        return list(buf)

    def last_launch_count(self):
        return self._lib.bp_last_launch_count(self._h)

    def decode_num_splits(self, cur_pos):
        return self._lib.bp_decode_num_splits(self._h, cur_pos)
