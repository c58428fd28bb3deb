"""`KvSnapshot`: the host-resident "BONSAIKV" v1 blob of the cache rows
[0, pos) (reference: src/kv_snapshot.rs). The bytes are produced and consumed
by the C ABI (`bp_snapshot_capture` / `bp_snapshot_apply`); this class is the
reference's value type around them."""
from __future__ import annotations

import ctypes as C
import struct

from . import _lib
from .errors import ConfigError

MAGIC = b"BONSAIKV"
VERSION = 1
HEADER_BYTES = 32


def payload_bytes(n_layer, kv_dim, pos):
    """src/kv_snapshot.rs:150-154."""
    return int(_lib.load().bp_snapshot_payload_bytes(n_layer, kv_dim, pos))


def payload_offset(n_layer, kv_dim, pos, kind, il, sect):
    """src/kv_snapshot.rs:158-169; kind 0 = K, 1 = V; sect 0 = d, 1 = qs."""
    return int(_lib.load().bp_snapshot_payload_offset(n_layer, kv_dim, pos, kind, il, sect))


class KvSnapshot:
    def __init__(self, n_layer, kv_dim, max_seq, pos, payload: bytes):
        self._n_layer, self._kv_dim, self._max_seq, self._pos = n_layer, kv_dim, max_seq, pos
        self.payload = bytes(payload)

    pos = property(lambda self: self._pos)
    n_layer = property(lambda self: self._n_layer)
    kv_dim = property(lambda self: self._kv_dim)
    max_seq = property(lambda self: self._max_seq)

    def to_bytes(self) -> bytes:
        """src/kv_snapshot.rs:69-80."""
        return MAGIC + struct.pack("<6I", VERSION, self._n_layer, self._kv_dim, self._max_seq, self._pos, 0) + self.payload

    @classmethod
    def from_bytes(cls, blob: bytes) -> "KvSnapshot":
        """src/kv_snapshot.rs:104-140."""
        if len(blob) < HEADER_BYTES:
            raise ConfigError("invalid config: KvSnapshot blob too short: missing header")
        if blob[:8] != MAGIC:
            raise ConfigError("invalid config: KvSnapshot blob has wrong magic")
        version, n_layer, kv_dim, max_seq, pos, reserved = struct.unpack("<6I", blob[8:32])
        if version != VERSION:
            raise ConfigError("invalid config: KvSnapshot blob has unsupported version")
        if reserved != 0:
            raise ConfigError("invalid config: KvSnapshot blob has non-zero reserved field")
        if len(blob) - HEADER_BYTES != payload_bytes(n_layer, kv_dim, pos):
            raise ConfigError("invalid config: KvSnapshot blob payload length does not match header")
        return cls(n_layer, kv_dim, max_seq, pos, blob[HEADER_BYTES:])

    def clone(self) -> "KvSnapshot":
        return KvSnapshot(self._n_layer, self._kv_dim, self._max_seq, self._pos, bytes(self.payload))

    # -- device side ---------------------------------------------------------
    @classmethod
    def capture(cls, ctxs, pos) -> "KvSnapshot":
        """`Session::snapshot`: read rows [0, pos) of every layer. `ctxs` is one
        AttnContext, or the list of all KV-head shards (each fills its columns)."""
        ctxs = list(ctxs) if isinstance(ctxs, (list, tuple)) else [ctxs]
        lib = _lib.load()
        size = int(lib.bp_snapshot_size(ctxs[0]._h, pos))
        buf = (C.c_uint8 * size)()
        for ctx in ctxs:
            ctx._check(lib.bp_snapshot_capture(ctx._h, pos, buf, size))
        return cls.from_bytes(bytes(buf))

    def apply(self, ctxs) -> int:
        """`Session::restore`: validate against the context(s) and write the rows back. Returns pos."""
        ctxs = list(ctxs) if isinstance(ctxs, (list, tuple)) else [ctxs]
        lib = _lib.load()
        blob = self.to_bytes()
        pos = C.c_uint32(0)
        for ctx in ctxs:
            ctx._check(lib.bp_snapshot_apply(ctx._h, blob, len(blob), C.byref(pos)))
        return pos.value
