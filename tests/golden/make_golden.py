"""Regenerates the golden fixtures of this folder from the CPU oracle.

    python tests/golden/make_golden.py

The reference engine (Rust + WGSL on wgpu) cannot run here, so these vectors
are NOT outputs of the reference: they freeze what the oracle
(oracle/oracle.c, checked against the constants and layouts the reference's
tests hold) computes on small seeded inputs. They serve two purposes: the CPU
suite notices if the oracle's arithmetic ever drifts, and the GPU suite can
compare the CUDA path with committed bytes. Inputs are not stored; they are
re-derived from bonsai_pot_b200.synth with the seeds recorded in each file.

Shapes are cut down to 8 query heads / 2 KV heads to keep the files small.
Files (all numpy .npz, 10 - 40 KB each):
  writeback_m5.npz     kv_writeback of 5 tokens at pos_base 3: K/V scales and int8 rows, q after norm + RoPE
  decode_past40.npz   config-0 style decode over 40 past tokens + the new one: cache rows, f16 output
  prefill_m21.npz      causal prefill of 21 tokens: f16 output
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from bonsai_pot_b200 import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402
from tests.helpers import build_decode_case  # noqa: E402


def norm_weight(seed):
    return (1 + 0.1 * np.random.default_rng(seed).standard_normal(128)).astype(np.float16)


def writeback_case():
    sh = O.Shape(n_layer=2, n_head=8, n_kv_head=2, max_seq=16)
    rope = O.rope_table_f16(sh)
    layer, pos_base, m = 1, 3, 5
    k = synth.tensor(11, 2, layer, synth.T_K_NEW, (m, sh.kv_dim))
    v = synth.tensor(11, 2, layer, synth.T_V_NEW, (m, sh.kv_dim))
    q = synth.tensor(11, 2, layer, synth.T_Q, (m, sh.q_dim))
    w_k, w_q = norm_weight(21), norm_weight(22)
    kv_k, kv_v = sh.new_cache(), sh.new_cache()
    O.kv_writeback(sh, k, v, w_k, rope, kv_k, kv_v, layer, pos_base, m)
    qn = O.q_norm_rope(sh, q, w_q, rope, pos_base, m)
    sl = slice(pos_base, pos_base + m)
    return dict(seed=11, cfg_id=2, layer=layer, pos_base=pos_base, m=m, w_k_seed=21, w_q_seed=22,
                k_d=sh.d_section(kv_k, layer)[sl].copy(), k_qs=sh.qs_section(kv_k, layer)[sl].copy(),
                v_d=sh.d_section(kv_v, layer)[sl].copy(), v_qs=sh.qs_section(kv_v, layer)[sl].copy(),
                q_out=qn.view(np.uint16).copy())


def decode_case():
    sh = O.Shape(n_layer=1, n_head=8, n_kv_head=2, max_seq=64)
    n_past = 40
    c = build_decode_case(sh, seed=5, cfg_id=0, layer=0, n_past=n_past)
    out = O.attn_decode(sh, c["qn"], c["kv_k"], c["kv_v"], 0, c["cur_pos"])
    rows = slice(0, n_past + 1)
    return dict(seed=5, cfg_id=0, n_past=n_past,
                k_d=sh.d_section(c["kv_k"], 0)[rows].copy(), k_qs=sh.qs_section(c["kv_k"], 0)[rows].copy(),
                v_d=sh.d_section(c["kv_v"], 0)[rows].copy(), v_qs=sh.qs_section(c["kv_v"], 0)[rows].copy(),
                qn=c["qn"].view(np.uint16).copy(), out=out.view(np.uint16).copy())


def prefill_case():
    sh = O.Shape(n_layer=1, n_head=8, n_kv_head=2, max_seq=64)
    rope = O.rope_table_f16(sh)
    m = 21
    q = O.q_norm_rope(sh, synth.tensor(9, 2, 0, synth.T_Q, (m, sh.q_dim)), synth.ones_weight(), rope, 0, m)
    k = synth.tensor(9, 2, 0, synth.T_K_NEW, (m, sh.kv_dim))
    v = synth.tensor(9, 2, 0, synth.T_V_NEW, (m, sh.kv_dim))
    kv_k, kv_v = sh.new_cache(), sh.new_cache()
    O.kv_writeback(sh, k, v, synth.ones_weight(), rope, kv_k, kv_v, 0, 0, m)
    out = O.attn_prefill(sh, q, kv_k, kv_v, 0, m)
    return dict(seed=9, cfg_id=2, m=m, out=out.view(np.uint16).copy())


CASES = {"writeback_m5": writeback_case, "decode_past40": decode_case, "prefill_m21": prefill_case}

if __name__ == "__main__":
    for name, fn in CASES.items():
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **fn())
        print(name, os.path.getsize(path), "bytes")
