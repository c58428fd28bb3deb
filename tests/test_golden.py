"""Golden fixtures (tests/golden/*.npz, frozen oracle outputs on seeded inputs):
the oracle must keep reproducing them bit for bit on the CPU, and the CUDA path
must match them (cache bytes, scales and rotated q bit-exact; attention
outputs within the stated tolerance). The fixtures are regenerated with
tests/golden/make_golden.py, whose case builders are reused here."""
import importlib.util
import os

import numpy as np
import pytest

from bonsai_pot_b200 import synth
from oracle import oracle as O
from tests.helpers import build_decode_case, within_tolerance

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLD, "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)


def load(name):
    with np.load(os.path.join(GOLD, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_oracle_reproduces_golden(name):
    gold, now = load(name), make_golden.CASES[name]()
    assert sorted(gold) == sorted(now)
    for key, val in now.items():
        val = np.asarray(val)
        if val.dtype == np.float32:
            assert np.array_equal(val.view(np.uint32), gold[key].view(np.uint32)), (name, key)
        else:
            assert np.array_equal(val, gold[key]), (name, key)


# ------------------------------------------------------------------ GPU ----

def _gpu():
    torch = pytest.importorskip("torch")
    import bonsai_pot_b200 as bp
    return torch, bp


def _dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.gpu
def test_cuda_writeback_matches_golden():
    torch, bp = _gpu()
    g = load("writeback_m5")
    layer, pos_base, m = int(g["layer"]), int(g["pos_base"]), int(g["m"])
    sh = O.Shape(n_layer=2, n_head=8, n_kv_head=2, max_seq=16)
    k = synth.tensor(int(g["seed"]), int(g["cfg_id"]), layer, synth.T_K_NEW, (m, sh.kv_dim))
    v = synth.tensor(int(g["seed"]), int(g["cfg_id"]), layer, synth.T_V_NEW, (m, sh.kv_dim))
    q = synth.tensor(int(g["seed"]), int(g["cfg_id"]), layer, synth.T_Q, (m, sh.q_dim))
    w_k, w_q = make_golden.norm_weight(int(g["w_k_seed"])), make_golden.norm_weight(int(g["w_q_seed"]))
    with bp.AttnContext(n_layer=2, n_head=8, n_kv_head=2, max_seq=16) as ctx:
        ctx.dispatch_kv_writeback_fused(layer, _dev(torch, k), _dev(torch, v), _dev(torch, w_k), pos_base, m)
        qd = _dev(torch, q)
        ctx.dispatch_q_norm_rope_fused(qd, _dev(torch, w_q), pos_base, m)
        torch.cuda.synchronize()
        got = {}
        for kind, tag in enumerate("kv"):
            d = np.empty((pos_base + m, sh.nb), dtype=np.float32)
            qs = np.empty((pos_base + m, sh.kv_dim), dtype=np.int8)
            ctx.kv_export(kind, layer, 0, pos_base + m, d)
            ctx.kv_export(kind, layer, 1, pos_base + m, qs)
            got[tag + "_d"], got[tag + "_qs"] = d[pos_base:], qs[pos_base:]
        q_out = qd.cpu().numpy().view(np.uint16)
    for key in ("k_d", "v_d"):
        assert np.array_equal(got[key].view(np.uint32), g[key].view(np.uint32)), key
    for key in ("k_qs", "v_qs"):
        assert np.array_equal(got[key], g[key]), key
    assert np.array_equal(q_out.reshape(-1), g["q_out"].reshape(-1))


@pytest.mark.gpu
@pytest.mark.parametrize("variant", [0, 1, 3])
def test_cuda_decode_matches_golden(variant):
    torch, bp = _gpu()
    g = load("decode_past40")
    n_past = int(g["n_past"])
    sh = O.Shape(n_layer=1, n_head=8, n_kv_head=2, max_seq=64)
    with bp.AttnContext(n_layer=1, n_head=8, n_kv_head=2, max_seq=64) as ctx:
        ctx.set_variant(variant)
        for kind, tag in enumerate("kv"):
            ctx.kv_import(kind, 0, 0, n_past + 1, np.ascontiguousarray(g[tag + "_d"]))
            ctx.kv_import(kind, 0, 1, n_past + 1, np.ascontiguousarray(g[tag + "_qs"]))
        out = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
        ctx.dispatch_attention_decode(0, _dev(torch, g["qn"].view(np.float16)), out, n_past + 1)
        torch.cuda.synchronize()
        got = out.cpu().numpy().astype(np.float32)
    ok, max_abs, max_rel = within_tolerance(got, g["out"].view(np.float16).astype(np.float32).reshape(-1))
    assert ok, (max_abs, max_rel)  # max-abs 2e-3 + max-rel 1e-2, as for every attention output


@pytest.mark.gpu
@pytest.mark.parametrize("variant", [0, 1])
def test_cuda_prefill_matches_golden(variant):
    torch, bp = _gpu()
    g = load("prefill_m21")
    m = int(g["m"])
    sh = O.Shape(n_layer=1, n_head=8, n_kv_head=2, max_seq=64)
    q = synth.tensor(int(g["seed"]), int(g["cfg_id"]), 0, synth.T_Q, (m, sh.q_dim))
    k = synth.tensor(int(g["seed"]), int(g["cfg_id"]), 0, synth.T_K_NEW, (m, sh.kv_dim))
    v = synth.tensor(int(g["seed"]), int(g["cfg_id"]), 0, synth.T_V_NEW, (m, sh.kv_dim))
    w = _dev(torch, synth.ones_weight())
    with bp.AttnContext(n_layer=1, n_head=8, n_kv_head=2, max_seq=64) as ctx:
        ctx.set_variant(variant)
        qd = _dev(torch, q)
        ctx.dispatch_q_norm_rope_fused(qd, w, 0, m)
        ctx.dispatch_kv_writeback_fused(0, _dev(torch, k), _dev(torch, v), w, 0, m)
        out = torch.zeros(m, sh.q_dim, dtype=torch.float16, device="cuda")
        ctx.dispatch_attention(0, qd, out, m)
        torch.cuda.synchronize()
        got = out.cpu().numpy().astype(np.float32)
    ok, max_abs, max_rel = within_tolerance(got, g["out"].view(np.float16).astype(np.float32).reshape(m, -1))
    assert ok, (max_abs, max_rel)
