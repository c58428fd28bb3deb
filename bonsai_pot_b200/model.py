"""Host-side mirror of the reference's public API around the attention path: `Model`,
`Session`, `Sampler`, `GenerateOptions`, `StopReason` (src/model.rs, src/session.rs).
Every method calls into the C ABI of include/bonsai_model.h; the forward passes, the
sampler and the session loop live in the library, not here."""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np

from . import _lib
from .attention import AttnContext
from .errors import raise_for_status
from .kv_snapshot import KvSnapshot

TOPK_MAX = 32  # src/model.rs:279


@dataclass
class Sampler:
    """`Sampler` (src/session.rs:13-35)."""
    temperature: float = 1.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    seed: int = 0

    def _c(self):
        return _lib.SamplerStruct(self.temperature, self.top_k or 0, -1.0 if self.top_p is None else self.top_p, self.seed)


class StopReason(enum.Enum):
    Eos = 0
    MaxTokens = 1


@dataclass
class GenerateOptions:
    """`GenerateOptions` (src/session.rs:43-62); stop_pred None = the model's eos_token_id."""
    max_new_tokens: int = 32
    stop_pred: Optional[Callable[[int], bool]] = None
    sampler: Sampler = field(default_factory=Sampler)


def effective_k(sampler: Sampler) -> int:
    return int(_lib.load().bp_effective_k(C.byref(sampler._c())))


def uniform_f32(seed: int) -> float:
    return float(_lib.load().bp_uniform_f32(seed & 0xFFFFFFFFFFFFFFFF))


def sample_from_topk(logits, indices, sampler: Sampler, pos: int) -> int:
    """`sample_from_topk` (src/session.rs:357-417), evaluated by the library (host code)."""
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    ix = np.ascontiguousarray(indices, dtype=np.uint32)
    return int(_lib.load().bp_sample_from_topk(lg.ctypes.data_as(C.POINTER(C.c_float)), ix.ctypes.data_as(C.POINTER(C.c_uint32)),
                                               len(lg), C.byref(sampler._c()), pos))


def check_dir(path) -> None:
    """parse_config_ini + validate_cfg on the host; raises the matching error."""
    buf = C.create_string_buffer(512)
    st = _lib.load().bp_model_check_dir(str(path).encode(), buf, len(buf))
    raise_for_status(st, buf.value.decode())


class Model:
    """`Model::load_with_options` (src/model.rs:861-1620): weights, activations and the KV cache on one GPU."""

    def __init__(self, model_dir, max_seq=1024, device=0):
        self._lib = _lib.load()
        self._h = C.c_void_p()
        st = self._lib.bp_model_load(str(model_dir).encode(), max_seq, device, C.byref(self._h))
        if st != 0:
            msg = (self._lib.bp_model_last_error(self._h) or b"").decode() if self._h else ""
            self.close()
            raise_for_status(st, msg)
        self.cfg = _lib.ModelConfig()
        self._lib.bp_model_get_config(self._h, C.byref(self.cfg))

    def close(self):
        if self._h:
            self._lib.bp_model_free(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st):
        if st == 0:
            return
        d = _lib.ErrorDetail()
        self._lib.bp_model_error_detail(self._h, C.byref(d))
        raise_for_status(st, (self._lib.bp_model_last_error(self._h) or b"").decode(), pos=d.pos, n=d.n, max=d.max,
                         cuda_error=d.cuda_error)

    def max_seq_len(self):
        return self.cfg.max_seq

    def max_prefill_tokens(self):
        return self.cfg.m_max

    def new_session(self) -> "Session":
        return Session(self)

    def attention(self) -> AttnContext:
        """The attention context the model owns, as a non-owning `AttnContext` (cache export, options, status)."""
        ctx = AttnContext.__new__(AttnContext)
        ctx._lib = self._lib
        ctx._h = C.c_void_p(self._lib.bp_model_attn(self._h))
        ctx.close = lambda: None
        c = self.cfg
        ctx.n_layer, ctx.n_head, ctx.n_kv_head, ctx.max_seq = c.n_layer, c.n_head, c.n_kv_head, c.max_seq
        ctx.q_dim, ctx.kv_dim, ctx.nb = c.q_dim, c.kv_dim, c.kv_dim // 32
        return ctx

    def is_device_lost(self):
        return self._lib.bp_ctx_status(self._lib.bp_model_attn(self._h)) != 0

    def _topk_call(self, fn, *args, k):
        logits = (C.c_float * TOPK_MAX)()
        idx = (C.c_uint32 * TOPK_MAX)()
        self._check(fn(self._h, *args, k, logits, idx))
        k = max(1, min(k, TOPK_MAX))
        return np.array(logits[:k], dtype=np.float32), np.array(idx[:k], dtype=np.uint32)

    def step_topk(self, token, pos, k=TOPK_MAX):
        """`step_matvec_topk`: (logits[k], indices[k]) of one token at `pos`."""
        return self._topk_call(self._lib.bp_model_step_topk, token, pos, k=k)

    def set_step_graph(self, enable: bool) -> None:
        """One-token steps as one CUDA graph launch (the default) or as stream launches."""
        self._check(self._lib.bp_model_set_step_graph(self._h, 1 if enable else 0))

    def graph_steps(self) -> int:
        """Steps that ran as a graph launch since the model was loaded."""
        return int(self._lib.bp_model_graph_steps(self._h))

    def prefill_topk(self, tokens, k=TOPK_MAX):
        """`prefill_matmul_topk`: batched prefill of positions 0 .. n - 1."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        return self._topk_call(self._lib.bp_model_prefill_topk, t.ctypes.data_as(C.POINTER(C.c_uint32)), len(t), k=k)

    def prefill_loop_topk(self, tokens, pos_base=0, k=TOPK_MAX):
        """`prefill_matvec_loop_topk`: the one-token path over every token."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        return self._topk_call(self._lib.bp_model_prefill_loop_topk, t.ctypes.data_as(C.POINTER(C.c_uint32)), len(t), pos_base, k=k)

    def hidden(self, row=0):
        out = np.empty(self.cfg.n_embd, dtype=np.float16)
        self._check(self._lib.bp_model_read_hidden(self._h, row, out.ctypes.data))
        return out

    def logits(self):
        out = np.empty(self.cfg.n_vocab, dtype=np.float16)
        self._check(self._lib.bp_model_read_logits(self._h, out.ctypes.data))
        return out

    def attn_tap(self, mode, buf=None):
        """Test hook: 1 = record every layer's attention output of the next steps into `buf`
        (f16 [n_layer][q_dim]), 2 = replace it by `buf`, 0 = off."""
        self._tap_keepalive = buf
        self._check(self._lib.bp_model_attn_tap(self._h, mode, None if buf is None else buf.ctypes.data))


class Session:
    """`Session` (src/session.rs:89-344): position bookkeeping, guards, sampling and the generate loop."""

    def __init__(self, model: Model):
        self.model = model
        self._lib = model._lib
        self._h = C.c_void_p()
        model._check(self._lib.bp_session_create(model._h, C.byref(self._h)))

    def __del__(self):
        try:
            if self._h:
                self._lib.bp_session_free(self._h)
                self._h = C.c_void_p()
        except Exception:
            pass

    def pos(self):
        return int(self._lib.bp_session_pos(self._h))

    def reset(self):
        self._lib.bp_session_reset(self._h)

    def _tokens_call(self, fn, tokens, sampler):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        chosen = C.c_uint32(0)
        self.model._check(fn(self._h, t.ctypes.data_as(C.POINTER(C.c_uint32)), len(t), C.byref(sampler._c()), C.byref(chosen)))
        return int(chosen.value)

    def prefill(self, tokens, sampler: Sampler) -> int:
        return self._tokens_call(self._lib.bp_session_prefill, tokens, sampler)

    def prefill_one_at_a_time(self, tokens, sampler: Sampler) -> int:
        return self._tokens_call(self._lib.bp_session_prefill_one_at_a_time, tokens, sampler)

    def step(self, token, sampler: Sampler) -> int:
        chosen = C.c_uint32(0)
        self.model._check(self._lib.bp_session_step(self._h, token, C.byref(sampler._c()), C.byref(chosen)))
        return int(chosen.value)

    def generate_streaming(self, first_token, opts: GenerateOptions, on_token=None) -> StopReason:
        stop = _lib.STOP_FN(lambda tok, _u: 1 if opts.stop_pred(tok) else 0) if opts.stop_pred is not None else _lib.STOP_FN()
        emit = _lib.TOKEN_FN(lambda tok, _u: on_token(tok)) if on_token is not None else _lib.TOKEN_FN()
        n_out, reason = C.c_uint32(0), C.c_int32(0)
        self.model._check(self._lib.bp_session_generate(self._h, first_token, opts.max_new_tokens, C.byref(opts.sampler._c()), stop, emit,
                                                        None, None, C.byref(n_out), C.byref(reason)))
        return StopReason(reason.value)

    def generate(self, first_token, opts: GenerateOptions):
        out = []
        reason = self.generate_streaming(first_token, opts, out.append)
        return out, reason

    def snapshot(self) -> KvSnapshot:
        size = int(self._lib.bp_session_snapshot_size(self._h))
        buf = (C.c_uint8 * size)()
        self.model._check(self._lib.bp_session_snapshot(self._h, buf, size))
        return KvSnapshot.from_bytes(bytes(buf))

    def restore(self, snap: KvSnapshot):
        blob = snap.to_bytes()
        self.model._check(self._lib.bp_session_restore(self._h, blob, len(blob)))
