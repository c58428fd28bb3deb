"""Model directories in the reference's on-disk format, with SYNTHETIC weights.

The reference converts a GGUF file into a flat directory (scripts/extract.py:95-232):
`config.ini` (hyper-parameters, then one `[tensor]` section per tensor) and five weight
files. A Q1_0 tensor [n_in, n_out] is stored as an array of f16 block scales [n_out][n_in/128]
followed (4-byte padded) by an array of 16-byte sign blocks [n_out][n_in/128][16], bit e of a
block = weight e. No real checkpoint exists where this repository is built, so this module
WRITES directories of that format from a seed: sign bits Bernoulli(0.5), block scales
|N(0, 0.02)| as f16, norm weights 1.0 (the random-init model BASELINE.json describes).
Reading and validating a directory is the library's job (bp_model_load / bp_model_check_dir).
"""
from __future__ import annotations

import os

import numpy as np

BONSAI_8B = dict(n_layer=36, n_embd=4096, n_ff=12288, n_head=32, n_kv_head=8, head_dim=128, n_vocab=151936)
TINY = dict(n_layer=2, n_embd=512, n_ff=1536, n_head=8, n_kv_head=2, head_dim=128, n_vocab=2048)


def _pad4(n):
    return (n + 3) & ~3


def write_synthetic_model(path, shape=None, seed=0, scale_sigma=0.02, eos_token_id=None, rope_freq_base=1e6, rms_eps=1e-6,
                          tied_embeddings=True):
    """Writes config.ini and the five weight files under `path`; returns the config dict."""
    shape = dict(TINY if shape is None else shape)
    os.makedirs(path, exist_ok=True)
    cfg = dict(shape)
    cfg.update(rope_freq_base=float(rope_freq_base), rms_eps=float(rms_eps),
               eos_token_id=shape["n_vocab"] - 1 if eos_token_id is None else eos_token_id,
               padding_token_id=0, add_bos=False, context_length=40960, rope_orig_context=40960)
    cfg["n_kv_groups"] = cfg["n_head"] // cfg["n_kv_head"]
    cfg["q_dim"] = cfg["n_head"] * cfg["head_dim"]
    cfg["kv_dim"] = cfg["n_kv_head"] * cfg["head_dim"]
    cfg["tied_embeddings"] = bool(tied_embeddings)
    rng = np.random.default_rng([seed, 0xB0A5])
    manifest = {}

    def q1_0(f, name, n_in, n_out):
        nb = n_in // 128
        entry = dict(dtype="Q1_0", shape=[n_in, n_out], buffer=os.path.basename(f.name), offset=f.tell())
        entry["d_offset"] = f.tell()
        f.write(np.abs(rng.standard_normal((n_out, nb), dtype=np.float32) * scale_sigma).astype(np.float16).tobytes())
        f.write(b"\0" * (_pad4(f.tell()) - f.tell()))
        entry["qs_offset"] = f.tell()
        f.write(rng.integers(0, 256, size=(n_out, nb, 16), dtype=np.uint8).tobytes())
        f.write(b"\0" * (_pad4(f.tell()) - f.tell()))
        entry["nb"] = nb
        entry["length"] = f.tell() - entry["offset"]
        manifest[name] = entry

    def f16_ones(f, name, n):
        entry = dict(dtype="F16", shape=[n], buffer=os.path.basename(f.name), offset=f.tell())
        f.write(np.ones(n, dtype=np.float16).tobytes())
        f.write(b"\0" * (_pad4(f.tell()) - f.tell()))
        entry["length"] = f.tell() - entry["offset"]
        manifest[name] = entry

    e, ff, q, kv, v, hd, nl = (cfg[k] for k in ("n_embd", "n_ff", "q_dim", "kv_dim", "n_vocab", "head_dim", "n_layer"))
    with open(os.path.join(path, "weights_attn.bin"), "wb") as f:
        for il in range(nl):
            q1_0(f, f"blk.{il}.attn_q.weight", e, q)
            q1_0(f, f"blk.{il}.attn_k.weight", e, kv)
            q1_0(f, f"blk.{il}.attn_v.weight", e, kv)
            q1_0(f, f"blk.{il}.attn_output.weight", q, e)
    with open(os.path.join(path, "weights_ffn_gate_up.bin"), "wb") as f:
        for il in range(nl):
            q1_0(f, f"blk.{il}.ffn_gate.weight", e, ff)
            q1_0(f, f"blk.{il}.ffn_up.weight", e, ff)
    with open(os.path.join(path, "weights_ffn_down.bin"), "wb") as f:
        for il in range(nl):
            q1_0(f, f"blk.{il}.ffn_down.weight", ff, e)
    with open(os.path.join(path, "weights_norms.bin"), "wb") as f:
        for il in range(nl):
            f16_ones(f, f"blk.{il}.attn_norm.weight", e)
            f16_ones(f, f"blk.{il}.attn_q_norm.weight", hd)
            f16_ones(f, f"blk.{il}.attn_k_norm.weight", hd)
            f16_ones(f, f"blk.{il}.ffn_norm.weight", e)
        f16_ones(f, "output_norm.weight", e)
    with open(os.path.join(path, "weights_embed_lmhead.bin"), "wb") as f:
        q1_0(f, "token_embd.weight", e, v)
        if not tied_embeddings:
            q1_0(f, "output.weight", e, v)

    def fmt(x):
        if isinstance(x, bool):
            return "true" if x else "false"
        if isinstance(x, list):
            return ",".join(str(i) for i in x)
        return str(x)

    with open(os.path.join(path, "config.ini"), "w", newline="\n") as f:
        for k, x in cfg.items():
            f.write(f"{k} = {fmt(x)}\n")
        for name, entry in manifest.items():
            f.write(f"\n[{name}]\n")
            for k, x in entry.items():
                f.write(f"{k} = {fmt(x)}\n")
    return cfg
