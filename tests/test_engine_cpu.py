"""CPU tests of the engine around the attention path: the sampler against the reference's own unit tests
(src/session.rs:430-572, the only golden values the reference holds for this part), the model-directory
reader and validator against the reference's rules and messages (src/model.rs:568-837), the C-ABI table
of include/bonsai_model.h, and sanity of the CPU restatement of the operators (oracle/engine.c)."""
import os
import re

import numpy as np
import pytest

import bonsai_pot_b200 as bp
from bonsai_pot_b200 import _lib, model, model_dir
from oracle import engine as E

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ------------------------------------------------------------------ sampler ----
def greedy():
    return bp.Sampler(temperature=0.0)


def test_sampler_pins_of_the_reference_unit_tests():
    logits, indices = [3.0, 2.0, 1.0], [42, 7, 99]
    assert model.sample_from_topk(logits, indices, greedy(), 0) == 42                       # greedy_temperature_zero
    assert model.sample_from_topk(logits, indices, bp.Sampler(top_k=1, temperature=1.0), 0) == 42  # greedy_top_k_one
    for seed in range(20):                                                                   # top_p_zero_picks_argmax
        assert model.sample_from_topk(logits, indices, bp.Sampler(top_p=0.0, temperature=1.0, seed=seed), 0) == 42
    s = bp.Sampler(temperature=1e9, seed=42)                                                 # seed_determinism
    flat, idx = [1.0] * 8, list(range(8))
    r1, r2, r3 = (model.sample_from_topk(flat, idx, s, p) for p in (5, 5, 6))
    assert r1 == r2 and r1 != r3
    assert model.sample_from_topk([], [], bp.Sampler(), 0) == 0                              # empty_input_returns_zero
    assert model.sample_from_topk([float("inf"), 1.0, 0.0], indices, bp.Sampler(temperature=1.0), 0) == 42  # non_finite
    assert model.effective_k(bp.Sampler(top_k=None)) == 32                                   # effective_k_caps_to_topk_max
    assert model.effective_k(bp.Sampler(top_k=0)) == 32
    assert model.effective_k(bp.Sampler(top_k=100)) == 32
    assert model.effective_k(bp.Sampler(top_k=5)) == 5
    for seed in range(1000):                                                                 # uniform_f32_in_range
        assert 0.0 <= model.uniform_f32(seed) < 1.0
    d = bp.Sampler()                                                                         # sampler_default_values
    assert (d.temperature, d.top_k, d.top_p, d.seed) == (1.0, None, None, 0)
    o = bp.GenerateOptions()                                                                 # generate_options_default
    assert o.max_new_tokens == 32 and o.stop_pred is None and o.sampler.temperature == 1.0


def test_sampler_matches_an_independent_restatement():
    """sample_from_topk restated in numpy float32 (SplitMix64, softmax, nucleus cut, multinomial walk)."""
    def uniform(seed):
        m = (1 << 64) - 1
        z = (seed + 0x9E3779B97F4A7C15) & m
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        z ^= z >> 31
        return np.float32(z >> 40) / np.float32(1 << 24)

    def ref(logits, indices, s, pos):
        lg = np.asarray(logits, dtype=np.float32)
        kk = s.top_k if s.top_k and s.top_k < len(lg) else len(lg)
        inv_t = np.float32(1.0) / np.float32(s.temperature)
        probs = np.exp((lg[:kk].astype(np.float64) * inv_t - np.float64(lg[0] * inv_t)).astype(np.float32))
        total = np.float32(0)
        for p in probs:
            total = np.float32(total + p)
        probs = (probs / total).astype(np.float32)
        cutoff = np.float32(1.0 if s.top_p is None else min(max(s.top_p, 0.0), 1.0))
        cum, keep = np.float32(0), kk
        for i, p in enumerate(probs):
            cum = np.float32(cum + p)
            if cum >= cutoff:
                keep = i + 1
                break
        kept = np.float32(0)
        for p in probs[:keep]:
            kept = np.float32(kept + p)
        r = np.float32(uniform(s.seed + pos) * kept)
        acc = np.float32(0)
        for i in range(keep):
            acc = np.float32(acc + probs[i])
            if r < acc:
                return indices[i]
        return indices[keep - 1]

    rng = np.random.default_rng(3)
    agree = 0
    for trial in range(300):
        lg = np.sort(rng.standard_normal(32).astype(np.float32) * 3)[::-1]
        idx = rng.permutation(1000)[:32].tolist()
        s = bp.Sampler(temperature=float(rng.uniform(0.3, 2.0)), top_k=[None, 5, 20][trial % 3],
                       top_p=[None, 0.9, 0.5][(trial // 3) % 3], seed=int(rng.integers(0, 2 ** 40)))
        agree += model.sample_from_topk(lg, idx, s, trial) == ref(lg, idx, s, trial)
    assert agree >= 297  # libm's expf against numpy's may differ in the last bit on a rare draw


# -------------------------------------------------------- model directory ----
def edit_config(path, fn):
    p = os.path.join(path, "config.ini")
    text = fn(open(p).read())
    with open(p, "w") as f:
        f.write(text)


def test_model_dir_reader_and_validator(tmp_path):
    d = str(tmp_path / "m")
    model_dir.write_synthetic_model(d)
    model.check_dir(d)  # as written: valid
    with pytest.raises(bp.IoError) as e:   # model_load_bad_path_is_io_error (tests/gpu_integration.rs:43-47)
        model.check_dir(str(tmp_path / "does-not-exist"))
    assert "config.ini" in str(e.value)
    cases = [
        (lambda t: t.replace("add_bos = false", "add_bos = true"), "add_bos=true"),
        (lambda t: t.replace("n_kv_groups = 4", "n_kv_groups = 3"), "n_kv_groups != n_head / n_kv_head"),
        (lambda t: t.replace("q_dim = 1024", "q_dim = 1000"), "q_dim != n_head * head_dim"),
        (lambda t: t.replace("kv_dim = 256", "kv_dim = 128"), "kv_dim != n_kv_head * head_dim"),
        (lambda t: t.replace("rope_orig_context = 40960", "rope_orig_context = 0"), "rope_orig_context must be > 0"),
        (lambda t: t.replace("n_layer = 2", "n_layer = two"), "config.ini field has invalid value"),
        (lambda t: t.replace("n_vocab = 2048\n", ""), "config.ini missing required field"),
        (lambda t: t.replace("[blk.1.ffn_down.weight]", "[blk.1.ffn_sideways.weight]"), "expected tensor missing"),
        (lambda t: t.replace("dtype = F16", "dtype = F32", 1), "tensor has wrong dtype"),
        (lambda t: t.replace("shape = 512,1024", "shape = 512,1000", 1), "tensor has wrong shape"),
        (lambda t: t.replace("buffer = weights_ffn_down.bin", "buffer = weights_attn.bin", 1), "wrong buffer file"),
        (lambda t: t.replace("nb = 4", "nb = 5", 1), "nb != n_in/128"),
        (lambda t: t.replace("qs_offset = 8192", "qs_offset = 8196", 1), "qs_offset != pad4"),
        (lambda t: t.replace("length = 73728", "length = 73732", 1), "length mismatch"),
    ]
    original = open(os.path.join(d, "config.ini")).read()
    for fn, needle in cases:
        edit_config(d, lambda _t: fn(original))
        with pytest.raises(bp.ConfigError) as e:
            model.check_dir(d)
        assert needle in str(e.value) and str(e.value).startswith("invalid config: "), (needle, str(e.value))
    edit_config(d, lambda _t: original)
    model.check_dir(d)


def test_model_header_and_ctypes_table_agree():
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "bonsai_model.h")).read(), flags=re.S)
    declared = sorted(set(re.findall(r"\b(bp_[a-z0-9_]+)\s*\(", text)) - {"bp_stop_fn", "bp_token_fn"})
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(_lib.MODEL_SIGNATURES) == declared


# ------------------------------------------------ the CPU restatement itself ----
def test_exp_det_is_within_three_ulp():
    xs = np.concatenate([np.linspace(-87, 88, 20001), np.linspace(-1, 1, 2001)]).astype(np.float32)
    got = np.array([E.exp_det(x) for x in xs], dtype=np.float32)
    want = np.exp(xs.astype(np.float64))
    ulp = np.spacing(want.astype(np.float32)).astype(np.float64)
    assert np.max(np.abs(got.astype(np.float64) - want) / ulp) < 3.0


def test_fused_and_unfused_paths_of_the_restatement_agree_closely(tmp_path):
    """rms_norm + matvec (the prefill-style composition) and the fused matvec differ only by rounding order; the
    one-token path and the batched path must pick the same first token (tests/gpu_integration.rs:122-139)."""
    d = str(tmp_path / "m")
    model_dir.write_synthetic_model(d, seed=4)
    hm = E.HostModel(d, 64)
    rng = np.random.default_rng(0)
    x = rng.standard_normal(hm.n_embd).astype(np.float16)
    w, d_off, qs_off, k, n = hm.q1("blk.0.attn_q.weight")
    ones = hm.f16("blk.0.attn_norm.weight")
    fused = E.matvec_fused_normed(w, k, x, ones, hm.rms_eps, [(d_off, qs_off, n)])[0].astype(np.float32)
    plain = E.matvec(w, d_off, qs_off, k, n, E.rms_norm(x, ones, k, 1, hm.rms_eps)[0]).astype(np.float32)
    assert np.max(np.abs(fused - plain)) < 2e-2 * np.max(np.abs(plain))
    prompt = [1, 2, 3, 4, 5, 6, 7, 8]
    a = E.HostModel(d, 64)
    for i, t in enumerate(prompt):
        lg_a, ix_a = a.step(t, i, suffix=i == len(prompt) - 1) or (None, None)
    b = E.HostModel(d, 64)
    lg_b, ix_b = b.prefill(prompt)
    assert ix_a[0] == ix_b[0]
    assert np.max(np.abs(lg_a - lg_b)) < 0.05


def test_topk_restatement_is_a_correct_top_k_with_ties():
    rng = np.random.default_rng(5)
    logits = (rng.integers(-40, 40, size=5001) / 8).astype(np.float16)  # many ties
    vals, idx = E.topk_reduce(logits, 32)
    assert np.all(np.diff(vals) <= 0)
    assert np.array_equal(vals, logits[idx].astype(np.float32))
    assert len(set(idx.tolist())) == 32
    assert np.array_equal(np.sort(vals)[::-1], np.sort(logits.astype(np.float32))[::-1][:32])
