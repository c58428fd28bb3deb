"""CPU tests of the boundary: the shared library loads, exports every symbol the
header declares, validates configurations like the reference does, and the pure
host functions (snapshot layout, KvSnapshot parsing) behave like the reference's."""
import ctypes as C
import os
import re
import struct

import pytest

import bonsai_pot_b200 as bp
from bonsai_pot_b200 import _lib, kv_snapshot
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "bonsai_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bp_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(_lib.SIGNATURES) == names  # the ctypes table covers the header exactly


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(bp.CudaError):
        bp.AttnContext(max_seq=64)


@pytest.mark.parametrize("kwargs,needle", [
    (dict(head_dim=64), "head_dim == 128"),
    (dict(n_head=30, n_kv_head=8), "multiple of n_kv_head"),
    (dict(max_seq=0), "max_seq"),
    (dict(n_layer=0), "must be > 0"),
    (dict(n_head=32, n_kv_head=2), "at most 8 query heads"),
    (dict(n_shards=2, shard=2), "shard"),
])
def test_config_validation_runs_before_any_gpu_work(kwargs, needle):
    args = dict(n_layer=2, n_head=32, n_kv_head=8, max_seq=64)
    args.update(kwargs)
    with pytest.raises(bp.ConfigError) as e:
        bp.AttnContext(**args)
    assert needle in str(e.value) and str(e.value).startswith("invalid config: ")


def test_snapshot_layout_functions_match_reference_pins():
    assert kv_snapshot.payload_bytes(36, 1024, 512) == 42_467_328
    assert kv_snapshot.payload_bytes(36, 1024, 32768) == 2_717_908_992
    assert kv_snapshot.payload_bytes(36, 1024, 0) == 0
    for kind in range(2):
        for il in (0, 7, 35):
            for sect in range(2):
                assert kv_snapshot.payload_offset(36, 1024, 16, kind, il, sect) == O.payload_offset(36, 1024, 16, kind, il, sect)


def test_kvsnapshot_value_type():
    # src/kv_snapshot.rs:392-428, 470-514
    pos = 4
    payload = bytes(i & 0xFF for i in range(kv_snapshot.payload_bytes(36, 1024, pos)))
    snap = bp.KvSnapshot(36, 1024, 1024, pos, payload)
    blob = snap.to_bytes()
    assert blob[:8] == b"BONSAIKV" and len(blob) == 32 + len(payload)
    back = bp.KvSnapshot.from_bytes(blob)
    assert (back.n_layer, back.kv_dim, back.max_seq, back.pos) == (36, 1024, 1024, pos)
    assert back.payload == payload
    assert O.snapshot_parse(blob)[4] == payload  # the oracle reads the same bytes
    empty = bp.KvSnapshot(36, 1024, 1024, 0, b"")
    assert len(empty.to_bytes()) == 32 and bp.KvSnapshot.from_bytes(empty.to_bytes()).pos == 0
    for mutate in (lambda b: b"\xff" + b[1:], lambda b: b[:-1], lambda b: b[:8] + struct.pack("<I", 2) + b[12:],
                   lambda b: b[:28] + b"\x01" + b[29:], lambda b: b[:16]):
        with pytest.raises(bp.ConfigError):
            bp.KvSnapshot.from_bytes(mutate(blob))
    clone = snap.clone()
    clone.payload = b"\x00" + clone.payload[1:]
    assert snap.payload[0:1] != b"\x00" or snap.payload == payload


def test_strerror_and_null_handling():
    lib = _lib.load()
    assert lib.bp_strerror(0) == b"ok"
    assert b"overflow" in lib.bp_strerror(2)
    assert lib.bp_ctx_status(None) == 7
    assert lib.bp_attn_create(None, None) == 7
    assert lib.bp_q_norm_rope(None, None, None, None, 0, 1) == 7
    assert lib.bp_attn_max_prefill(None) == 0
    lib.bp_attn_destroy(None)  # no-op
