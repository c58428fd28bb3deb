"""Python face of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Loads ``liboracle.so`` (built from ``oracle.c`` by the Makefile beside it) and
wraps each function for numpy arrays. Also holds a numpy "twin" of the
norm + RoPE + quantise math, written independently of the C code, so that the
two restatements check each other bit for bit.

PARITY UNPINNED: the reference (Rust + WGSL on wgpu/Vulkan) cannot be built or
run here and ships no golden vectors for this path. The reference's own unit
tests pin only the cache/snapshot layout and the RoPE-table sample values;
those pins are re-checked in ``tests/test_oracle_pins.py``.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
arm of ``bench.py`` may import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import struct
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
HEAD_DIM = 128
PARTIAL_STRIDE = 130
ATTN_CHUNK = 16

_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u32, _u64, _f32, _int = C.c_uint32, C.c_uint64, C.c_float, C.c_int


def build(native: bool = False) -> str:
    """Compile the oracle if its shared object is missing; return its path."""
    name = "liboracle_native.so" if native else "liboracle.so"
    path = os.path.join(HERE, name)
    srcs = [os.path.join(HERE, f) for f in ("oracle.c", "engine.c", "Makefile")]
    stale = not os.path.exists(path) or any(os.path.getmtime(f) > os.path.getmtime(path) for f in srcs)
    if native or stale:
        args = ["make", "-C", HERE] + (["-B", "native"] if native else ["-B"])
        subprocess.run(args, check=True, capture_output=True)
    return path


def _load(native: bool = False) -> C.CDLL:
    lib = C.CDLL(build(native))
    sig = {
        "orc_f16_to_f32": (C.c_float, [C.c_uint16]),
        "orc_f32_to_f16": (C.c_uint16, [C.c_float]),
        "orc_kv_d_total": (_u64, [_u32, _u32, _u32]),
        "orc_kv_total_bytes": (_u64, [_u32, _u32, _u32]),
        "orc_buf_d_offset": (_u64, [_u32, _u32, _u32]),
        "orc_buf_qs_offset": (_u64, [_u32, _u32, _u32, _u32]),
        "orc_payload_bytes": (_u64, [_u32, _u32, _u32]),
        "orc_payload_offset": (_u64, [_u32] * 6),
        "orc_build_rope_table_f32": (None, [_u32, _f32, _u32, _f32p]),
        "orc_build_rope_table_f16": (None, [_u32, _f32, _u32, _u16p]),
        "orc_kv_writeback": (None, [_u16p, _u16p, _u16p, _u16p, _u8p, _u8p] + [_u32] * 6 + [_f32, _int, _int]),
        "orc_quantize_rows": (None, [_u16p, _u8p] + [_u32] * 6),
        "orc_q_norm_rope": (None, [_u16p, _u16p, _u16p, _u32, _u32, _u32, _f32, _int, _int]),
        "orc_attn_split": (None, [_u16p, _u8p, _u8p, _f32p] + [_u32] * 6),
        "orc_attn_merge": (None, [_f32p, _u16p, _u32, _u32]),
        "orc_attn_decode": (None, [_u16p, _u8p, _u8p, _u16p] + [_u32] * 6),
        "orc_attn_prefill": (None, [_u16p, _u8p, _u8p, _u16p] + [_u32] * 6),
        "orc_attn_exact": (None, [_u16p, _u8p, _u8p, _f32p] + [_u32] * 7),
        "orc_num_threads": (_int, []),
        "orc_rsqrt_rn": (C.c_float, [C.c_float]),
        "orc_rsqrt_long_double": (C.c_float, [C.c_float]),
        "orc_rsqrt_sweep": (_u64, [_u32, _u64, _u32]),
        "orc_set_threads": (None, [_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


_LIB = None
_LIB_NATIVE = None


def lib(native: bool = False) -> C.CDLL:
    global _LIB, _LIB_NATIVE
    if native:
        if _LIB_NATIVE is None:
            _LIB_NATIVE = _load(True)
        return _LIB_NATIVE
    if _LIB is None:
        _LIB = _load(False)
    return _LIB


def _u16(a: np.ndarray) -> np.ndarray:
    """View an f16 (or u16) array as contiguous u16."""
    a = np.ascontiguousarray(a)
    return a.view(np.uint16) if a.dtype == np.float16 else a


class Shape:
    """Model shape for the path (the fields of the reference's `Config` that the
    five kernels read: src/model.rs:672-676, 1174-1183)."""

    def __init__(self, n_layer=36, n_head=32, n_kv_head=8, max_seq=1024, rms_eps=1e-6, rope_freq_base=1e6):
        self.n_layer, self.n_head, self.n_kv_head, self.max_seq = n_layer, n_head, n_kv_head, max_seq
        self.head_dim = HEAD_DIM
        self.q_dim = n_head * HEAD_DIM
        self.kv_dim = n_kv_head * HEAD_DIM
        self.nb = self.kv_dim // 32
        self.rms_eps, self.rope_freq_base = rms_eps, rope_freq_base

    @property
    def d_total(self):
        return self.n_layer * self.max_seq * self.nb * 4

    @property
    def kv_bytes(self):
        return self.d_total + self.n_layer * self.max_seq * self.kv_dim

    def new_cache(self, fill=0):
        return np.full(self.kv_bytes, fill, dtype=np.uint8)

    def d_section(self, kv, layer):
        """f32 view [max_seq][nb] of one layer's scales."""
        o = layer * self.max_seq * self.nb * 4
        return kv[o:o + self.max_seq * self.nb * 4].view(np.float32).reshape(self.max_seq, self.nb)

    def qs_section(self, kv, layer):
        """int8 view [max_seq][kv_dim] of one layer's quants."""
        o = self.d_total + layer * self.max_seq * self.kv_dim
        return kv[o:o + self.max_seq * self.kv_dim].view(np.int8).reshape(self.max_seq, self.kv_dim)


# ------------------------------------------------------------ C-backed calls --

def rope_table_f32(head_dim, base, max_seq):
    out = np.empty(max_seq * head_dim, dtype=np.float32)
    lib().orc_build_rope_table_f32(head_dim, base, max_seq, out)
    return out


def rope_table_f16(sh: Shape):
    out = np.empty(sh.max_seq * HEAD_DIM, dtype=np.uint16)
    lib().orc_build_rope_table_f16(HEAD_DIM, sh.rope_freq_base, sh.max_seq, out)
    return out.view(np.float16)


def kv_writeback(sh, k_cur, v_cur, w_k_norm, rope, kv_k, kv_v, layer, pos_base, m, tree=0, contract=0, native=False):
    lib(native).orc_kv_writeback(_u16(k_cur), _u16(v_cur), _u16(w_k_norm), _u16(rope), kv_k, kv_v, sh.n_layer,
                                 sh.max_seq, sh.n_kv_head, layer, pos_base, m, sh.rms_eps, tree, contract)


def quantize_rows(sh, x, kv, layer, pos_base, m):
    lib().orc_quantize_rows(_u16(x), kv, sh.n_layer, sh.max_seq, sh.kv_dim, layer, pos_base, m)


def q_norm_rope(sh, q, w_q_norm, rope, pos_base, m, tree=0, contract=0, native=False):
    """Returns the normed + rotated copy of q (f16 [m][q_dim])."""
    out = _u16(q).copy()
    lib(native).orc_q_norm_rope(out, _u16(w_q_norm), _u16(rope), sh.n_head, pos_base, m, sh.rms_eps, tree, contract)
    return out.view(np.float16)


def attn_split(sh, q, kv_k, kv_v, layer, cur_pos):
    n_chunks = -(-cur_pos // ATTN_CHUNK)
    partials = np.zeros(sh.n_head * n_chunks * PARTIAL_STRIDE, dtype=np.float32)
    lib().orc_attn_split(_u16(q), kv_k, kv_v, partials, sh.n_layer, sh.max_seq, sh.n_head, sh.n_kv_head, layer, cur_pos)
    return partials.reshape(sh.n_head, n_chunks, PARTIAL_STRIDE)


def attn_merge(sh, partials):
    n_chunks = partials.shape[1]
    out = np.empty(sh.q_dim, dtype=np.uint16)
    lib().orc_attn_merge(np.ascontiguousarray(partials).reshape(-1), out, sh.n_head, n_chunks)
    return out.view(np.float16)


def attn_decode(sh, q, kv_k, kv_v, layer, cur_pos, native=False):
    out = np.empty(sh.q_dim, dtype=np.uint16)
    lib(native).orc_attn_decode(_u16(q), kv_k, kv_v, out, sh.n_layer, sh.max_seq, sh.n_head, sh.n_kv_head, layer, cur_pos)
    return out.view(np.float16)


def attn_prefill(sh, q, kv_k, kv_v, layer, m, native=False):
    out = np.empty(m * sh.q_dim, dtype=np.uint16)
    lib(native).orc_attn_prefill(_u16(q), kv_k, kv_v, out, sh.n_layer, sh.max_seq, sh.n_head, sh.n_kv_head, layer, m)
    return out.view(np.float16).reshape(m, sh.q_dim)


def attn_exact(sh, q, kv_k, kv_v, layer, m, key_base):
    """Two-pass softmax in binary64 over the dequantised cache -> f32 [m][q_dim]."""
    out = np.empty(m * sh.q_dim, dtype=np.float32)
    lib().orc_attn_exact(_u16(q), kv_k, kv_v, out, sh.n_layer, sh.max_seq, sh.n_head, sh.n_kv_head, layer, m, key_base)
    return out.reshape(m, sh.q_dim)


def num_threads(native=False):
    return lib(native).orc_num_threads()


def set_threads(n, native=False):
    """Thread count of the OpenMP loops from now on (a launcher's OMP_NUM_THREADS=1 does not bind the baseline)."""
    lib(native).orc_set_threads(int(n))


# ------------------------------------------------------------- numpy twin ----
# Written from the shader text (kv_writeback_fused.wgsl:65-166,
# q_norm_rope_fused.wgsl:49-95), not from oracle.c. All arithmetic stays in
# np.float32 so that every operation rounds once, as the C code does.

def _np_sumsq(x):  # x: [..., 128] f32, canonical butterfly tree
    sq = x * x
    idx = np.arange(128)
    for off in (16, 8, 4, 2, 1):
        sq = sq + sq[..., idx ^ off]
    return (sq[..., 0] + sq[..., 32]) + (sq[..., 64] + sq[..., 96])


def _np_rsqrt(x):  # binary64 evaluation, one rounding to f32
    return (1.0 / np.sqrt(x.astype(np.float64))).astype(np.float32)


def np_norm_rope(x_f16, w_f16, rope_rows_f16, eps):
    """x: [rows][128] f16, rope_rows: [rows][128] f16 -> [rows][128] f32."""
    raw = x_f16.astype(np.float32)
    total = _np_sumsq(raw)
    inv_h = _np_rsqrt(total / np.float32(128.0) + np.float32(eps))
    xn = (raw * inv_h[:, None]) * w_f16.astype(np.float32)[None, :]
    c = rope_rows_f16[:, 0::2].astype(np.float32)
    s = rope_rows_f16[:, 1::2].astype(np.float32)
    lo, hi = xn[:, :64], xn[:, 64:]
    return np.concatenate([lo * c - hi * s, lo * s + hi * c], axis=1)


def np_quant_blocks(x_f32):
    """x: [rows][n] f32 with n % 32 == 0 -> (d [rows][n/32] f32, q [rows][n] int8)."""
    rows, n = x_f32.shape
    xb = x_f32.reshape(rows, n // 32, 32)
    amax = np.abs(xb).max(axis=2)
    d = amax / np.float32(127.0)
    with np.errstate(divide="ignore"):
        inv = np.where(d > 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    r = np.rint(xb * inv[:, :, None])
    q = np.clip(r, -127.0, 127.0).astype(np.int8)
    return d.astype(np.float32), q.reshape(rows, n)


def np_kv_writeback(sh, k_cur, v_cur, w_k_norm, rope, kv_k, kv_v, layer, pos_base, m):
    rope = rope.reshape(sh.max_seq, HEAD_DIM)
    k = k_cur.reshape(m, sh.n_kv_head, HEAD_DIM)
    k_post = np.empty((m, sh.n_kv_head, HEAD_DIM), dtype=np.float32)
    for g in range(sh.n_kv_head):
        k_post[:, g] = np_norm_rope(k[:, g], w_k_norm, rope[pos_base:pos_base + m], sh.rms_eps)
    dk, qk = np_quant_blocks(k_post.reshape(m, sh.kv_dim))
    dv, qv = np_quant_blocks(v_cur.reshape(m, sh.kv_dim).astype(np.float32))
    sh.d_section(kv_k, layer)[pos_base:pos_base + m] = dk
    sh.qs_section(kv_k, layer)[pos_base:pos_base + m] = qk
    sh.d_section(kv_v, layer)[pos_base:pos_base + m] = dv
    sh.qs_section(kv_v, layer)[pos_base:pos_base + m] = qv


def np_q_norm_rope(sh, q, w_q_norm, rope, pos_base, m):
    rope = rope.reshape(sh.max_seq, HEAD_DIM)
    qh = q.reshape(m, sh.n_head, HEAD_DIM)
    out = np.empty_like(qh)
    for h in range(sh.n_head):
        out[:, h] = np_norm_rope(qh[:, h], w_q_norm, rope[pos_base:pos_base + m], sh.rms_eps).astype(np.float16)
    return out.reshape(m, sh.q_dim)


def np_dequant(sh, kv, layer, n_rows):
    """f32 [n_rows][kv_dim] = scale * int8, as load_k/load_v compute it."""
    d = sh.d_section(kv, layer)[:n_rows]
    q = sh.qs_section(kv, layer)[:n_rows].astype(np.float32)
    return (q.reshape(n_rows, sh.nb, 32) * d[:, :, None]).reshape(n_rows, sh.kv_dim)


# ----------------------------------------------------- snapshot blob (host) --
# src/kv_snapshot.rs:30-32 (magic, version, header size), :69-80 (to_bytes),
# :104-140 (from_bytes), :150-169 (payload layout).

MAGIC = b"BONSAIKV"
VERSION = 1
HEADER_BYTES = 32


def payload_bytes(n_layer, kv_dim, pos):
    return int(lib().orc_payload_bytes(n_layer, kv_dim, pos))


def payload_offset(n_layer, kv_dim, pos, kind, il, sect):
    return int(lib().orc_payload_offset(n_layer, kv_dim, pos, kind, il, sect))


def snapshot_blob(sh: Shape, kv_k, kv_v, pos):
    """Byte-exact `KvSnapshot::to_bytes` of host cache buffers for rows [0, pos)."""
    out = bytearray(MAGIC + struct.pack("<6I", VERSION, sh.n_layer, sh.kv_dim, sh.max_seq, pos, 0))
    for kv in (kv_k, kv_v):
        for il in range(sh.n_layer):
            out += sh.d_section(kv, il)[:pos].tobytes()
            out += sh.qs_section(kv, il)[:pos].tobytes()
    return bytes(out)


def snapshot_parse(blob: bytes):
    """`KvSnapshot::from_bytes`: returns (n_layer, kv_dim, max_seq, pos, payload) or raises ValueError."""
    if len(blob) < HEADER_BYTES:
        raise ValueError("KvSnapshot blob too short: missing header")
    if blob[:8] != MAGIC:
        raise ValueError("KvSnapshot blob has wrong magic")
    version, n_layer, kv_dim, max_seq, pos, reserved = struct.unpack("<6I", blob[8:32])
    if version != VERSION:
        raise ValueError("KvSnapshot blob has unsupported version")
    if reserved != 0:
        raise ValueError("KvSnapshot blob has non-zero reserved field")
    if len(blob) - HEADER_BYTES != payload_bytes(n_layer, kv_dim, pos):
        raise ValueError("KvSnapshot blob payload length does not match header")
    return n_layer, kv_dim, max_seq, pos, blob[HEADER_BYTES:]
