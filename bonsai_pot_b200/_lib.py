"""Builds and loads the C-ABI shared library (`libbonsai_attn.so`).

The library is compiled in-tree with nvcc for sm_100a only. Loading never falls
back to anything else: if the shared object is missing and cannot be built, the
import of the compute API fails.
"""
from __future__ import annotations

import ctypes as C
import glob
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libbonsai_attn.so")
HEADER = os.path.join(os.path.dirname(HERE), "include", "bonsai_attn.h")
MODEL_HEADER = os.path.join(os.path.dirname(HERE), "include", "bonsai_model.h")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + [HEADER, MODEL_HEADER]
    return any(os.path.getmtime(p) > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu under csrc/ into one shared object."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH] + sources()
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


class Config(C.Structure):
    """`bp_attn_config` of include/bonsai_attn.h."""
    _fields_ = [
        ("n_layer", C.c_uint32), ("n_head", C.c_uint32), ("n_kv_head", C.c_uint32), ("head_dim", C.c_uint32),
        ("max_seq", C.c_uint32), ("rms_eps", C.c_float), ("rope_freq_base", C.c_float),
        ("max_prefill", C.c_uint32), ("n_shards", C.c_uint32), ("shard", C.c_uint32), ("device", C.c_int32),
    ]


class ErrorDetail(C.Structure):
    _fields_ = [("status", C.c_int32), ("pos", C.c_uint32), ("n", C.c_uint32), ("max", C.c_uint32),
                ("cuda_error", C.c_int32)]


_vp, _u32, _u64, _int = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int

# name -> (restype, argtypes); must list every symbol the header declares.
SIGNATURES = {
    "bp_attn_create": (_int, [C.POINTER(Config), C.POINTER(_vp)]),
    "bp_attn_destroy": (None, [_vp]),
    "bp_q_norm_rope": (_int, [_vp, _vp, _vp, _vp, _u32, _u32]),
    "bp_kv_writeback": (_int, [_vp, _vp, _u32, _vp, _vp, _vp, _u32, _u32]),
    "bp_attn_decode": (_int, [_vp, _vp, _u32, _vp, _vp, _u32]),
    "bp_attn_prefill": (_int, [_vp, _vp, _u32, _vp, _vp, _u32]),
    "bp_attn_max_prefill": (_u32, [_vp]),
    "bp_decode_step_host": (_int, [_vp, _u32, _vp, _vp, _vp, _vp, _vp, _u32, _vp]),
    "bp_decode_token_host": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _vp]),
    "bp_prefill_layer_host": (_int, [_vp, _u32, _vp, _vp, _vp, _vp, _vp, _u32, _vp]),
    "bp_kv_export": (_int, [_vp, _u32, _u32, _u32, _u32, _vp]),
    "bp_kv_import": (_int, [_vp, _u32, _u32, _u32, _u32, _vp]),
    "bp_snapshot_payload_bytes": (_u64, [_u32, _u32, _u32]),
    "bp_snapshot_payload_offset": (_u64, [_u32] * 6),
    "bp_snapshot_size": (_u64, [_vp, _u32]),
    "bp_snapshot_capture": (_int, [_vp, _u32, _vp, _u64]),
    "bp_snapshot_apply": (_int, [_vp, _vp, _u64, C.POINTER(_u32)]),
    "bp_ctx_status": (_int, [_vp]),
    "bp_ctx_inject_lost": (None, [_vp]),
    "bp_last_error_detail": (None, [_vp, C.POINTER(ErrorDetail)]),
    "bp_last_error_message": (C.c_char_p, [_vp]),
    "bp_strerror": (C.c_char_p, [_int]),
    "bp_kv_device_ptr": (_vp, [_vp, _u32]),
    "bp_kv_buffer_bytes": (_u64, [_vp]),
    "bp_rope_device_ptr": (_vp, [_vp]),
    "bp_rope_table_copy": (_int, [_vp, _vp]),
    "bp_set_variant": (_int, [_vp, _u32]),
    "bp_set_option": (_int, [_vp, C.c_char_p, _u32]),
    "bp_debug_counters": (_int, [_vp, C.POINTER(C.c_uint64)]),
    "bp_debug_hold_sms": (_int, [_vp, _u32, _u32]),
    "bp_last_launch_count": (_u32, [_vp]),
    "bp_decode_num_splits": (_u32, [_vp, _u32]),
    "bp_attn_decode_layer": (_int, [_vp, _vp, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _vp]),
    "bp_set_peer_exchange": (_int, [_vp, _u32, _vp, _vp]),
    "bp_set_prefill_exchange": (_int, [_vp, _u32, _vp]),
    "bp_peer_sync": (_int, [_vp, _vp, _u32]),
    "bp_attn_decode_static_scratch": (_int, [_vp, _vp, _vp, _vp, _vp] + [_u32] * 6),
}



class ModelConfig(C.Structure):
    """`bp_model_config` of include/bonsai_model.h."""
    _fields_ = [(k, C.c_uint32) for k in ("n_layer", "n_embd", "n_ff", "n_head", "n_kv_head", "head_dim", "n_vocab",
                                           "eos_token_id", "q_dim", "kv_dim")] + \
               [("rope_freq_base", C.c_float), ("rms_eps", C.c_float), ("tied_embeddings", C.c_uint32),
                ("max_seq", C.c_uint32), ("m_max", C.c_uint32)]


class SamplerStruct(C.Structure):
    """`bp_sampler` of include/bonsai_model.h."""
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float), ("seed", C.c_uint64)]


STOP_FN = C.CFUNCTYPE(C.c_int, C.c_uint32, C.c_void_p)
TOKEN_FN = C.CFUNCTYPE(None, C.c_uint32, C.c_void_p)
_f32p, _u32p, _pp = C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.POINTER(C.c_void_p)
_smp = C.POINTER(SamplerStruct)

# name -> (restype, argtypes); must list every symbol include/bonsai_model.h declares.
MODEL_SIGNATURES = {
    "bp_op_q1_relayout": (_int, [_vp, _vp, _vp, _u64]),
    "bp_op_matvec_q1_0": (_int, [_vp, _vp, _vp, _u32, _u32, _vp, _vp, _u32]),
    "bp_op_matvec_q1_0_fused_normed": (_int, [_vp, _u32, _vp, _vp, C.c_float, _u32, _pp, _pp, _u32p, _pp]),
    "bp_op_matvec_q1_0_silu": (_int, [_vp, _vp, _vp, _u32, _u32, _vp, _vp, _vp, _u32]),
    "bp_op_set_matvec_rows": (None, [_u32]),
    "bp_op_rms_norm": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, C.c_float]),
    "bp_op_silu_mul": (_int, [_vp, _vp, _vp, _vp, _u64]),
    "bp_op_embed": (_int, [_vp, _vp, _vp, _u32, _vp, _u32, _vp]),
    "bp_op_quantize_q8_0": (_int, [_vp, _vp, _u32, _u32, _vp, _vp]),
    "bp_op_matmul_q1_0_q8_0": (_int, [_vp, _vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp, _u32]),
    "bp_op_set_matmul_variant": (None, [_u32]),
    "bp_op_device_status": (_int, []),
    "bp_op_topk_reduce": (_int, [_vp, _vp, _u32, _u32, _vp, _vp]),
    "bp_model_check_dir": (_int, [C.c_char_p, C.c_char_p, C.c_size_t]),
    "bp_model_load": (_int, [C.c_char_p, _u32, C.c_int32, _pp]),
    "bp_model_free": (None, [_vp]),
    "bp_model_get_config": (_int, [_vp, C.POINTER(ModelConfig)]),
    "bp_model_last_error": (C.c_char_p, [_vp]),
    "bp_model_error_detail": (None, [_vp, C.POINTER(ErrorDetail)]),
    "bp_model_attn": (_vp, [_vp]),
    "bp_model_step_topk": (_int, [_vp, _u32, _u32, _u32, _f32p, _u32p]),
    "bp_model_set_step_graph": (_int, [_vp, _u32]),
    "bp_model_graph_steps": (_u64, [_vp]),
    "bp_model_prefill_topk": (_int, [_vp, _u32p, _u32, _u32, _f32p, _u32p]),
    "bp_model_prefill_loop_topk": (_int, [_vp, _u32p, _u32, _u32, _u32, _f32p, _u32p]),
    "bp_model_read_hidden": (_int, [_vp, _u32, _vp]),
    "bp_model_read_logits": (_int, [_vp, _vp]),
    "bp_model_attn_tap": (_int, [_vp, _u32, _vp]),
    "bp_sampler_default": (None, [_smp]),
    "bp_effective_k": (_u32, [_smp]),
    "bp_uniform_f32": (C.c_float, [_u64]),
    "bp_sample_from_topk": (_u32, [_f32p, _u32p, _u32, _smp, _u32]),
    "bp_session_create": (_int, [_vp, _pp]),
    "bp_session_free": (None, [_vp]),
    "bp_session_pos": (_u32, [_vp]),
    "bp_session_reset": (None, [_vp]),
    "bp_session_prefill": (_int, [_vp, _u32p, _u32, _smp, _u32p]),
    "bp_session_prefill_one_at_a_time": (_int, [_vp, _u32p, _u32, _smp, _u32p]),
    "bp_session_step": (_int, [_vp, _u32, _smp, _u32p]),
    "bp_session_generate": (_int, [_vp, _u32, _u32, _smp, STOP_FN, TOKEN_FN, _vp, _u32p, _u32p, C.POINTER(C.c_int32)]),
    "bp_session_snapshot_size": (_u64, [_vp]),
    "bp_session_snapshot": (_int, [_vp, _vp, _u64]),
    "bp_session_restore": (_int, [_vp, _vp, _u64]),
}

_LIB = None


def load() -> C.CDLL:
    """Load the shared library, building it first when sources are newer."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = LIB_PATH
    if needs_build():
        try:
            path = build()
        except (RuntimeError, FileNotFoundError) as e:
            if not os.path.exists(LIB_PATH):
                raise ImportError(f"libbonsai_attn.so is missing and could not be built: {e}") from e
    lib = C.CDLL(path)
    for name, (res, args) in list(SIGNATURES.items()) + list(MODEL_SIGNATURES.items()):
        fn = getattr(lib, name)  # AttributeError here = the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib
