"""Shared helpers for the tests: synthetic workloads and tolerance checks."""
import numpy as np

from bonsai_pot_b200 import synth
from oracle import oracle as O

ATOL, RTOL = 2e-3, 1e-2  # attention outputs: |x - ref| <= 2e-3 + 1e-2 * |ref| vs the binary64 softmax


def within_tolerance(x, ref):
    x = np.asarray(x, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    err = np.abs(x - ref)
    ok = bool(np.all(err <= ATOL + RTOL * np.abs(ref)))
    big = np.abs(ref) >= 1e-2
    max_rel = float((err[big] / np.abs(ref[big])).max()) if big.any() else 0.0
    return ok, float(err.max()), max_rel


def build_decode_case(sh, seed, cfg_id, layer, n_past, w_q=None, w_k=None):
    """Config-0 style workload on the CPU oracle: `n_past` rows of plainly
    quantised N(0,1) K/V, then the new token written at row n_past through
    kv_writeback, and q normalised + rotated at the same position.
    Returns dict with host cache buffers, raw inputs and oracle results."""
    w_q = synth.ones_weight() if w_q is None else w_q
    w_k = synth.ones_weight() if w_k is None else w_k
    rope = O.rope_table_f16(sh)
    kv_k, kv_v = sh.new_cache(), sh.new_cache()
    k_past = synth.tensor(seed, cfg_id, layer, synth.T_K_PAST, (n_past, sh.kv_dim))
    v_past = synth.tensor(seed, cfg_id, layer, synth.T_V_PAST, (n_past, sh.kv_dim))
    if n_past:
        O.quantize_rows(sh, k_past, kv_k, layer, 0, n_past)
        O.quantize_rows(sh, v_past, kv_v, layer, 0, n_past)
    q = synth.tensor(seed, cfg_id, layer, synth.T_Q, (1, sh.q_dim))
    k_new = synth.tensor(seed, cfg_id, layer, synth.T_K_NEW, (1, sh.kv_dim))
    v_new = synth.tensor(seed, cfg_id, layer, synth.T_V_NEW, (1, sh.kv_dim))
    O.kv_writeback(sh, k_new, v_new, w_k, rope, kv_k, kv_v, layer, n_past, 1)
    qn = O.q_norm_rope(sh, q, w_q, rope, n_past, 1)
    return dict(rope=rope, kv_k=kv_k, kv_v=kv_v, k_past=k_past, v_past=v_past, q=q, k_new=k_new, v_new=v_new,
                qn=qn, w_q=w_q, w_k=w_k, cur_pos=n_past + 1)
