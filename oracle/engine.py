"""CPU engine: the reference's forward passes restated on the host (TEST INFRASTRUCTURE ONLY).

Reads a model directory (its own small config.ini reader, independent of the library's),
and runs the one-token path (`encode_step_matvec`, src/forward.rs:578-672) and the batched
prefill (`prefill_matmul_topk`, src/forward.rs:975-1253) with the operators of engine.c and the
attention functions of oracle.c, in the reference's dispatch order. PARITY UNPINNED for
numerics, as stated in engine.c. Only `tests/` and the CPU arm of `bench.py` may import this.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import oracle as O

_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(dtype=np.int8, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u32, _u64, _f32, _int = C.c_uint32, C.c_uint64, C.c_float, C.c_int
_SIG = {
    "orc_exp_det": (C.c_float, [C.c_float]),
    "orc_embed": (None, [_u8p, _u64, _u64, _u32, _u32p, _u32, _u16p]),
    "orc_rms_norm": (None, [_u16p, _u16p, _u16p, _u32, _u32, _f32]),
    "orc_matvec_q1_0": (None, [_u8p, _u64, _u64, _u32, _u32, _u16p, _u16p, _int]),
    "orc_matvec_q1_0_fused_normed": (None, [_u8p, _u32, _u16p, _u16p, _f32, _u32, C.POINTER(_u64), C.POINTER(_u64),
                                            C.POINTER(_u32), C.POINTER(C.c_void_p)]),
    "orc_matvec_q1_0_silu": (None, [_u8p, _u64, _u64, _u32, _u32, _u16p, _u16p, _u16p, _int]),
    "orc_silu_mul": (None, [_u16p, _u16p, _u16p, _u64]),
    "orc_quantize_q8_0": (None, [_u16p, _u32, _u32, _f32p, _i8p]),
    "orc_matmul_q1_0_q8_0": (None, [_u8p, _u64, _u64, _u32, _u32, _u32, _f32p, _i8p, _u16p, _int]),
    "orc_topk_reduce": (None, [_u16p, _u32, _u32, _f32p, _u32p]),
}
_bound = {}


def _lib(native=False):
    lib = O.lib(native)
    if id(lib) not in _bound:
        for name, (res, args) in _SIG.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _bound[id(lib)] = True
    return lib


def _h(a):  # f16 array -> contiguous u16 view
    a = np.ascontiguousarray(a)
    return a.view(np.uint16) if a.dtype == np.float16 else a


# ------------------------------------------------------------------ operators ----
def exp_det(x):
    return float(_lib().orc_exp_det(float(x)))


def embed(w, d_off, qs_off, k, tokens):
    t = np.ascontiguousarray(tokens, dtype=np.uint32)
    out = np.empty(len(t) * k, dtype=np.uint16)
    _lib().orc_embed(w, d_off, qs_off, k, t, len(t), out)
    return out.view(np.float16).reshape(len(t), k)


def rms_norm(x, w, group_size, n_groups, eps):
    out = np.empty(group_size * n_groups, dtype=np.uint16)
    _lib().orc_rms_norm(_h(x).reshape(-1), out, _h(w), group_size, n_groups, eps)
    return out.view(np.float16).reshape(n_groups, group_size)


def matvec(w, d_off, qs_off, k, n, x, y=None, native=False):
    """y (+)= W x; returns the new y (f16 [n]). y given = accumulate."""
    out = np.zeros(n, dtype=np.uint16) if y is None else _h(y).reshape(-1).copy()
    _lib(native).orc_matvec_q1_0(w, d_off, qs_off, k, n, _h(x).reshape(-1), out, 0 if y is None else 1)
    return out.view(np.float16)


def matvec_fused_normed(w, k, x, w_norm, eps, ranges, native=False):
    """ranges: [(d_off, qs_off, n)]; returns one f16 array per range."""
    nr = len(ranges)
    outs = [np.empty(n, dtype=np.uint16) for _, _, n in ranges]
    d = (_u64 * nr)(*[r[0] for r in ranges])
    q = (_u64 * nr)(*[r[1] for r in ranges])
    n = (_u32 * nr)(*[r[2] for r in ranges])
    o = (C.c_void_p * nr)(*[a.ctypes.data for a in outs])
    _lib(native).orc_matvec_q1_0_fused_normed(w, k, _h(x).reshape(-1), _h(w_norm), eps, nr, d, q, n, o)
    return [a.view(np.float16) for a in outs]


def matvec_silu(w, d_off, qs_off, k, n, gate, up, y=None, native=False):
    out = np.zeros(n, dtype=np.uint16) if y is None else _h(y).reshape(-1).copy()
    _lib(native).orc_matvec_q1_0_silu(w, d_off, qs_off, k, n, _h(gate).reshape(-1), _h(up).reshape(-1), out, 0 if y is None else 1)
    return out.view(np.float16)


def silu_mul(gate, up):
    g, u = _h(gate).reshape(-1), _h(up).reshape(-1)
    out = np.empty(g.size, dtype=np.uint16)
    _lib().orc_silu_mul(g, u, out, g.size)
    return out.view(np.float16).reshape(np.shape(gate))


def quantize_q8_0(x, k, m):
    d = np.empty(m * (k // 32), dtype=np.float32)
    qs = np.empty(m * k, dtype=np.int8)
    _lib().orc_quantize_q8_0(_h(x).reshape(-1), k, m, d, qs)
    return d, qs


def matmul(w, d_off, qs_off, k, n, m, a_d, a_qs, y=None):
    out = np.zeros(m * n, dtype=np.uint16) if y is None else _h(y).reshape(-1).copy()
    _lib().orc_matmul_q1_0_q8_0(w, d_off, qs_off, k, n, m, a_d, a_qs, out, 0 if y is None else 1)
    return out.view(np.float16).reshape(m, n)


def topk_reduce(logits, k):
    lg = _h(logits).reshape(-1)
    kk = min(k, 32)
    vals, idx = np.empty(kk, dtype=np.float32), np.empty(kk, dtype=np.uint32)
    _lib().orc_topk_reduce(lg, lg.size, k, vals, idx)
    return vals, idx


# --------------------------------------------------------------- model on the host ----
def read_config(path):
    """config.ini -> (globals dict of strings, manifest dict name -> dict); parse_config_ini, src/model.rs:568-656."""
    g, manifest, cur = {}, {}, None
    with open(os.path.join(path, "config.ini")) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            if line.startswith("[") and line.endswith("]"):
                cur = manifest.setdefault(line[1:-1], {})
            elif " = " in line:
                k, v = line.split(" = ", 1)
                (g if cur is None else cur)[k] = v
    return g, manifest


class HostModel:
    """The weights of a model directory in host memory and the two forward passes over them."""

    def __init__(self, path, max_seq):
        g, self.manifest = read_config(path)
        self.n_layer, self.n_embd, self.n_ff = int(g["n_layer"]), int(g["n_embd"]), int(g["n_ff"])
        self.n_head, self.n_kv_head, self.head_dim = int(g["n_head"]), int(g["n_kv_head"]), int(g["head_dim"])
        self.n_vocab, self.q_dim, self.kv_dim = int(g["n_vocab"]), int(g["q_dim"]), int(g["kv_dim"])
        self.rms_eps, self.rope_freq_base = float(np.float32(g["rms_eps"])), float(np.float32(g["rope_freq_base"]))
        self.tied = g["tied_embeddings"] == "true"
        self.files = {}
        for name in ("weights_attn.bin", "weights_ffn_gate_up.bin", "weights_ffn_down.bin", "weights_norms.bin",
                     "weights_embed_lmhead.bin"):
            self.files[name] = np.fromfile(os.path.join(path, name), dtype=np.uint8)
        self.max_seq = max_seq
        self.sh = O.Shape(n_layer=self.n_layer, n_head=self.n_head, n_kv_head=self.n_kv_head, max_seq=max_seq,
                          rms_eps=self.rms_eps, rope_freq_base=self.rope_freq_base)
        self.rope = O.rope_table_f16(self.sh)
        self.kv_k, self.kv_v = self.sh.new_cache(), self.sh.new_cache()
        self.attn_override = None   # test hook: f16 [n_layer][q_dim] used instead of the attention oracle (one-token path)
        self.attn_record = None

    def q1(self, name):
        e = self.manifest[name]
        shape = [int(s) for s in e["shape"].split(",")]
        return self.files[e["buffer"]], int(e["d_offset"]), int(e["qs_offset"]), shape[0], shape[1]

    def f16(self, name):
        e = self.manifest[name]
        n = int(e["shape"].split(",")[0])
        off = int(e["offset"])
        return self.files[e["buffer"]][off:off + 2 * n].view(np.float16)

    def _suffix(self, x_row, k):
        xn = rms_norm(x_row, self.f16("output_norm.weight"), self.n_embd, 1, self.rms_eps)[0]
        w, d, q, kk, n = self.q1("token_embd.weight" if self.tied else "output.weight")
        self.last_logits = matvec(w, d, q, kk, n, xn)
        return topk_reduce(self.last_logits, k)

    def step(self, token, pos, k=32, suffix=True):
        """encode_step_matvec (src/forward.rs:578-672): returns (logits[k], indices[k]); self.x is the residual stream."""
        w, d, q, kk, _ = self.q1("token_embd.weight")
        x = embed(w, d, q, kk, [token])[0]
        sh = self.sh
        for il in range(self.n_layer):
            p = f"blk.{il}."
            wa = self.files["weights_attn.bin"]
            rq, rk, rv = (self.q1(p + t) for t in ("attn_q.weight", "attn_k.weight", "attn_v.weight"))
            qv, kc, vc = matvec_fused_normed(wa, self.n_embd, x, self.f16(p + "attn_norm.weight"), self.rms_eps,
                                             [(r[1], r[2], r[4]) for r in (rq, rk, rv)])
            qn = O.q_norm_rope(sh, qv.reshape(1, -1), self.f16(p + "attn_q_norm.weight"), self.rope, pos, 1)
            O.kv_writeback(sh, kc.reshape(1, -1), vc.reshape(1, -1), self.f16(p + "attn_k_norm.weight"), self.rope,
                           self.kv_k, self.kv_v, il, pos, 1)
            if self.attn_override is not None:
                attn = np.ascontiguousarray(self.attn_override[il])
            else:
                attn = O.attn_decode(sh, qn, self.kv_k, self.kv_v, il, pos + 1)
            if self.attn_record is not None:
                self.attn_record[il] = attn
            w, d, q, kk, n = self.q1(p + "attn_output.weight")
            x = matvec(w, d, q, kk, n, attn, y=x)
            rg, ru = self.q1(p + "ffn_gate.weight"), self.q1(p + "ffn_up.weight")
            gate, up = matvec_fused_normed(rg[0], self.n_embd, x, self.f16(p + "ffn_norm.weight"), self.rms_eps,
                                           [(r[1], r[2], r[4]) for r in (rg, ru)])
            w, d, q, kk, n = self.q1(p + "ffn_down.weight")
            x = matvec_silu(w, d, q, kk, n, gate, up, y=x)
        self.x = x
        return self._suffix(x, k) if suffix else None

    def prefill(self, tokens, k=32):
        """prefill_matmul_topk (src/forward.rs:975-1253) at pos_base 0."""
        m, sh = len(tokens), self.sh
        w, d, q, kk, _ = self.q1("token_embd.weight")
        x = embed(w, d, q, kk, tokens)
        for il in range(self.n_layer):
            p = f"blk.{il}."
            xn = rms_norm(x, self.f16(p + "attn_norm.weight"), self.n_embd, m, self.rms_eps)
            a_d, a_qs = quantize_q8_0(xn, self.n_embd, m)
            qv, kc, vc = (matmul(*self.q1(p + t)[:3], self.n_embd, self.q1(p + t)[4], m, a_d, a_qs)
                          for t in ("attn_q.weight", "attn_k.weight", "attn_v.weight"))
            qn = O.q_norm_rope(sh, qv, self.f16(p + "attn_q_norm.weight"), self.rope, 0, m)
            O.kv_writeback(sh, kc, vc, self.f16(p + "attn_k_norm.weight"), self.rope, self.kv_k, self.kv_v, il, 0, m)
            attn = O.attn_prefill(sh, qn, self.kv_k, self.kv_v, il, m)
            a_d, a_qs = quantize_q8_0(attn, self.q_dim, m)
            w, d, q, kk, n = self.q1(p + "attn_output.weight")
            x = matmul(w, d, q, kk, n, m, a_d, a_qs, y=x)
            xn = rms_norm(x, self.f16(p + "ffn_norm.weight"), self.n_embd, m, self.rms_eps)
            a_d, a_qs = quantize_q8_0(xn, self.n_embd, m)
            gate, up = (matmul(*self.q1(p + t)[:3], self.n_embd, self.q1(p + t)[4], m, a_d, a_qs)
                        for t in ("ffn_gate.weight", "ffn_up.weight"))
            ffn_in = silu_mul(gate, up)
            a_d, a_qs = quantize_q8_0(ffn_in, self.n_ff, m)
            w, d, q, kk, n = self.q1(p + "ffn_down.weight")
            x = matmul(w, d, q, kk, n, m, a_d, a_qs, y=x)
        self.x = x
        return self._suffix(x[m - 1], k)
