"""GPU tests of the engine around the attention path: every non-attention kernel through the C ABI of
include/bonsai_model.h against the CPU restatement (oracle/engine.c) BIT FOR BIT on the same seeded inputs;
the one-token forward pass with the GPU's attention outputs fed to the CPU pass (so that the comparison of
the residual stream and the logits is exact while attention keeps its own tolerance); and the session
behaviour the reference tests in tests/gpu_integration.rs."""
import ctypes as C

import numpy as np
import pytest

import bonsai_pot_b200 as bp
from bonsai_pot_b200 import _lib, model_dir
from oracle import engine as E

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits_equal(t, ref):
    got = t.cpu().numpy()
    return np.array_equal(got.view(np.uint16).reshape(-1), np.ascontiguousarray(ref).view(np.uint16).reshape(-1))


def random_q1(rng, k, n, sigma=0.02):
    """A Q1_0 tensor as (bytes, d_off, qs_off) in the model-directory layout, plus device copies and re-laid-out bits."""
    nb = k // 128
    d = np.abs(rng.standard_normal((n, nb)).astype(np.float32) * sigma).astype(np.float16)
    qs = rng.integers(0, 256, size=(n, nb, 16), dtype=np.uint8)
    blob = np.concatenate([d.view(np.uint8).reshape(-1), qs.reshape(-1)])
    d_dev, qs_dev = dev(d), dev(qs)
    bits = torch.empty_like(qs_dev)
    lib = _lib.load()
    assert lib.bp_op_q1_relayout(None, qs_dev.data_ptr(), bits.data_ptr(), n * nb) == 0
    return blob, 0, d.nbytes, d_dev, qs_dev, bits


@pytest.mark.parametrize("k,n,accumulate", [(4096, 4096, True), (512, 40, False), (12288, 4096, True), (4096, 151936, False),
                                            (9728, 100, True), (128, 1, False)])
def test_matvec_q1_0_bit_exact(k, n, accumulate):
    rng = np.random.default_rng(k + n)
    blob, d_off, qs_off, d_dev, _, bits = random_q1(rng, k, n)
    x = rng.standard_normal(k).astype(np.float16)
    y0 = rng.standard_normal(n).astype(np.float16)
    want = E.matvec(blob, d_off, qs_off, k, n, x, y=y0 if accumulate else None)
    xd = dev(x)  # named: a temporary's memory may be handed to the next allocation
    lib = _lib.load()
    try:
        for rows in (0, 1, 2, 4, 8, 9, 10):  # every kernel layout: by height, rows per lane; + 8 = the general instances only
            lib.bp_op_set_matvec_rows(rows)
            y = dev(y0.copy())
            assert lib.bp_op_matvec_q1_0(None, d_dev.data_ptr(), bits.data_ptr(), k, n, xd.data_ptr(), y.data_ptr(), int(accumulate)) == 0
            torch.cuda.synchronize()
            assert bits_equal(y, want), rows
    finally:
        lib.bp_op_set_matvec_rows(0)


@pytest.mark.parametrize("k,ns", [(4096, (4096, 1024, 1024)), (4096, (12288, 12288)), (512, (1024, 256, 256)), (2560, (32,))])
def test_matvec_fused_normed_bit_exact(k, ns):
    rng = np.random.default_rng(k + len(ns))
    parts = [random_q1(rng, k, n) for n in ns]
    blob = np.concatenate([p[0] for p in parts])
    offs, base = [], 0
    for p, n in zip(parts, ns):
        offs.append((base + p[1], base + p[2], n))
        base += p[0].size
    x = (rng.standard_normal(k) * 3).astype(np.float16)
    w_norm = (1 + 0.1 * rng.standard_normal(k)).astype(np.float16)
    want = E.matvec_fused_normed(blob, k, x, w_norm, 1e-6, offs)
    nr = len(ns)
    arr = lambda vals: (C.c_void_p * nr)(*vals)
    xd, wd = dev(x), dev(w_norm)
    lib = _lib.load()
    try:
        for rows in (0, 1, 2, 4, 8, 9, 10):
            lib.bp_op_set_matvec_rows(rows)
            outs = [torch.zeros(n, dtype=torch.float16, device="cuda") for n in ns]
            st = lib.bp_op_matvec_q1_0_fused_normed(None, k, xd.data_ptr(), wd.data_ptr(), 1e-6, nr,
                                                    arr([p[3].data_ptr() for p in parts]), arr([p[5].data_ptr() for p in parts]),
                                                    (C.c_uint32 * nr)(*ns), arr([o.data_ptr() for o in outs]))
            assert st == 0
            torch.cuda.synchronize()
            for o, w in zip(outs, want):
                assert bits_equal(o, w), rows
    finally:
        lib.bp_op_set_matvec_rows(0)


@pytest.mark.parametrize("k,n", [(12288, 4096), (1536, 512), (9728, 24)])
def test_matvec_silu_bit_exact(k, n):
    rng = np.random.default_rng(k)
    blob, d_off, qs_off, d_dev, _, bits = random_q1(rng, k, n)
    gate = (rng.standard_normal(k) * 4).astype(np.float16)
    gate[:4] = [30.0, -30.0, 0.0, -65504.0]
    up = rng.standard_normal(k).astype(np.float16)
    y0 = rng.standard_normal(n).astype(np.float16)
    want = E.matvec_silu(blob, d_off, qs_off, k, n, gate, up, y=y0)
    y, gd, ud = dev(y0.copy()), dev(gate), dev(up)
    assert _lib.load().bp_op_matvec_q1_0_silu(None, d_dev.data_ptr(), bits.data_ptr(), k, n, gd.data_ptr(), ud.data_ptr(),
                                              y.data_ptr(), 1) == 0
    torch.cuda.synchronize()
    assert bits_equal(y, want)


def test_rms_norm_silu_mul_embed_quantize_bit_exact():
    lib = _lib.load()
    rng = np.random.default_rng(1)
    for n, groups in ((4096, 7), (512, 1), (2560, 3)):
        x = (rng.standard_normal((groups, n)) * 2).astype(np.float16)
        w = (1 + 0.2 * rng.standard_normal(n)).astype(np.float16)
        out = torch.zeros(groups, n, dtype=torch.float16, device="cuda")
        xd, wd = dev(x), dev(w)
        assert lib.bp_op_rms_norm(None, xd.data_ptr(), out.data_ptr(), wd.data_ptr(), n, groups, 1e-6) == 0
        torch.cuda.synchronize()
        assert bits_equal(out, E.rms_norm(x, w, n, groups, 1e-6))
        inplace = dev(x.copy())  # in == out, as the output norm uses it
        assert lib.bp_op_rms_norm(None, inplace.data_ptr(), inplace.data_ptr(), wd.data_ptr(), n, groups, 1e-6) == 0
        torch.cuda.synchronize()
        assert bits_equal(inplace, E.rms_norm(x, w, n, groups, 1e-6))
    gate = (rng.standard_normal((5, 1536)) * 5).astype(np.float16)
    up = rng.standard_normal((5, 1536)).astype(np.float16)
    out = torch.zeros(5, 1536, dtype=torch.float16, device="cuda")
    gd, ud = dev(gate), dev(up)
    assert lib.bp_op_silu_mul(None, gd.data_ptr(), ud.data_ptr(), out.data_ptr(), gate.size) == 0
    torch.cuda.synchronize()
    assert bits_equal(out, E.silu_mul(gate, up))
    blob, d_off, qs_off, d_dev, qs_dev, _ = random_q1(rng, 512, 300)
    tokens = np.array([0, 299, 17, 17, 123], dtype=np.uint32)
    x = torch.zeros(5, 512, dtype=torch.float16, device="cuda")
    td = dev(tokens)
    assert lib.bp_op_embed(None, d_dev.data_ptr(), qs_dev.data_ptr(), 512, td.data_ptr(), 5, x.data_ptr()) == 0
    torch.cuda.synchronize()
    assert bits_equal(x, E.embed(blob, d_off, qs_off, 512, tokens))
    act = (rng.standard_normal((9, 1536)) * 3).astype(np.float16)
    act[0, :32] = 0  # an all-zero block: d = 0, quants 0
    d_out = torch.zeros(9 * 48, dtype=torch.float32, device="cuda")
    q_out = torch.zeros(9 * 1536, dtype=torch.int8, device="cuda")
    ad = dev(act)
    assert lib.bp_op_quantize_q8_0(None, ad.data_ptr(), 1536, 9, d_out.data_ptr(), q_out.data_ptr()) == 0
    torch.cuda.synchronize()
    want_d, want_q = E.quantize_q8_0(act, 1536, 9)
    assert np.array_equal(d_out.cpu().numpy().view(np.uint32), want_d.view(np.uint32))
    assert np.array_equal(q_out.cpu().numpy(), want_q)


@pytest.mark.parametrize("k,n,m,accumulate", [(512, 256, 1, False), (512, 200, 7, True), (1536, 512, 130, True), (4096, 1024, 64, False),
                                              (512, 200, 40, True), (1024, 300, 257, False), (256, 128, 33, False)])
def test_matmul_q1_0_q8_0_bit_exact(k, n, m, accumulate):
    lib = _lib.load()
    rng = np.random.default_rng(k + m)
    blob, d_off, qs_off, d_dev, qs_dev, _ = random_q1(rng, k, n)
    act = (rng.standard_normal((m, k)) * 2).astype(np.float16)
    a_d, a_qs = E.quantize_q8_0(act, k, m)
    y0 = rng.standard_normal((m, n)).astype(np.float16)
    want = E.matmul(blob, d_off, qs_off, k, n, m, a_d, a_qs, y=y0 if accumulate else None)
    add, aqd = dev(a_d), dev(a_qs)
    try:
        for variant in (0, 1, 2, 3, 4, 5):  # by batch size, CUDA cores, mma.sync, tcgen05, mma.sync with 64- / 128-token tiles: the same bits
            lib.bp_op_set_matmul_variant(variant)
            y = dev(y0.copy())
            assert lib.bp_op_matmul_q1_0_q8_0(None, d_dev.data_ptr(), qs_dev.data_ptr(), k, n, m, add.data_ptr(), aqd.data_ptr(),
                                              y.data_ptr(), int(accumulate)) == 0
            assert lib.bp_op_device_status() == 0
            assert bits_equal(y, want), variant
    finally:
        lib.bp_op_set_matmul_variant(0)


@pytest.mark.parametrize("k,n,m,accumulate", [(256, 24576, 512, True), (256, 6144, 512, False), (128, 6144, 300, True),
                                              (128, 19000, 450, False)])
def test_matmul_tile_choices_agree(k, n, m, accumulate):
    """The mma.sync matmul picks its tiles by how they fill the device: 128-token tiles, 64-token tiles, or whole
    waves of 128-token tiles followed by 64-token tiles for the rest in a second launch (these shapes reach that
    choice on a 148-SM device). The three must give the same bits; the 128-token form is checked against the CPU
    restatement in the test above."""
    lib = _lib.load()
    gen = torch.Generator(device="cuda").manual_seed(k + n + m)
    nb = k // 128
    d = (torch.rand(n, nb, device="cuda", generator=gen) * 0.02).half()
    qs = torch.randint(0, 256, (n, nb, 16), device="cuda", dtype=torch.uint8, generator=gen)
    a_d = torch.rand(m, k // 32, device="cuda", generator=gen) * 0.05
    a_qs = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8, generator=gen)
    y0 = torch.randn(m, n, device="cuda", generator=gen).half()
    got = {}
    try:
        for variant in (5, 4, 0):
            lib.bp_op_set_matmul_variant(variant)
            y = y0.clone()
            assert lib.bp_op_matmul_q1_0_q8_0(None, d.data_ptr(), qs.data_ptr(), k, n, m, a_d.data_ptr(), a_qs.data_ptr(), y.data_ptr(),
                                              int(accumulate)) == 0
            assert lib.bp_op_device_status() == 0
            got[variant] = y
    finally:
        lib.bp_op_set_matmul_variant(0)
    assert torch.equal(got[5].view(torch.int16), got[4].view(torch.int16))
    assert torch.equal(got[5].view(torch.int16), got[0].view(torch.int16))
    assert not torch.equal(got[5], y0)


@pytest.mark.parametrize("n,k,ties", [(151936, 32, False), (5001, 32, True), (2048, 5, True), (7, 32, False)])
def test_topk_reduce_identical_including_ties(n, k, ties):
    rng = np.random.default_rng(n)
    logits = ((rng.integers(-40, 40, size=n) / 8) if ties else rng.standard_normal(n) * 3).astype(np.float16)
    padded = np.concatenate([logits, np.zeros(2, dtype=np.float16)])
    vals = torch.zeros(32, dtype=torch.float32, device="cuda")
    idx = torch.zeros(32, dtype=torch.int32, device="cuda")
    pd = dev(padded)
    assert _lib.load().bp_op_topk_reduce(None, pd.data_ptr(), n, k, vals.data_ptr(), idx.data_ptr()) == 0
    torch.cuda.synchronize()
    want_v, want_i = E.topk_reduce(logits, k)
    kk = min(k, 32)
    assert np.array_equal(vals.cpu().numpy()[:kk].view(np.uint32), want_v.view(np.uint32))
    assert np.array_equal(idx.cpu().numpy()[:kk].astype(np.uint32), want_i)


# ----------------------------------------------------------------- forward passes ----
WIDE = dict(n_layer=2, n_embd=4096, n_ff=12288, n_head=32, n_kv_head=8, head_dim=128, n_vocab=151936)  # Bonsai-8B widths


@pytest.mark.parametrize("shape", [None, WIDE])
def test_one_token_pass_matches_the_cpu_pass_bit_for_bit(tmp_path, shape):
    """Several decode steps. The GPU pass records its attention outputs; the CPU pass uses them in place of its
    own attention (both write the same cache rows), so every other operator must reproduce the residual stream,
    the logits and the top-32 bit for bit."""
    d = str(tmp_path / "m")
    cfg = model_dir.write_synthetic_model(d, shape=shape, seed=11)
    hm = E.HostModel(d, 64)
    with bp.Model(d, max_seq=64) as gm:
        tap = np.zeros((cfg["n_layer"], cfg["q_dim"]), dtype=np.float16)
        gm.attn_tap(1, tap)
        token = 7
        for pos in range(4):
            lg, ix = gm.step_topk(token, pos)
            x_gpu, logits_gpu = gm.hidden(0), gm.logits()
            hm.attn_override = tap.copy()
            hm.attn_record = np.zeros_like(tap)
            want_lg, want_ix = hm.step(token, pos)
            assert np.array_equal(ix, want_ix) and np.array_equal(lg.view(np.uint32), want_lg.view(np.uint32)), pos
            # x was normalised in place by the output suffix on both sides
            assert np.array_equal(logits_gpu.view(np.uint16), hm.last_logits.view(np.uint16)), pos
            # normalised in place by the output suffix on both sides: the residual stream, exactly
            want_x = E.rms_norm(hm.x, hm.f16("output_norm.weight"), hm.n_embd, 1, hm.rms_eps)[0]
            assert np.array_equal(x_gpu.view(np.uint16), want_x.view(np.uint16)), pos
            token = int(ix[1])  # not the argmax (a random tied-embedding model echoes its input): vary the stream
        # cache rows written by both sides are identical (bit-exact K/V quantisation inside the fused decode step)
        ctx = gm.attention()
        for il in range(cfg["n_layer"]):
            for kind, kv in enumerate((hm.kv_k, hm.kv_v)):
                dd = np.empty((4, hm.sh.nb), dtype=np.float32)
                qq = np.empty((4, hm.sh.kv_dim), dtype=np.int8)
                ctx.kv_export(kind, il, 0, 4, dd)
                ctx.kv_export(kind, il, 1, 4, qq)
                assert np.array_equal(dd.view(np.uint32), hm.sh.d_section(kv, il)[:4].view(np.uint32))
                assert np.array_equal(qq, hm.sh.qs_section(kv, il)[:4])


@pytest.mark.parametrize("exclusive_device", [1, 0])
def test_graph_steps_are_identical_to_stream_steps(tmp_path, exclusive_device):
    """The one-token step as one CUDA graph launch (attention nodes patched per position, the step captured
    again when the attention launch changes shape) against the same step as stream launches: same kernels and
    arguments, so hidden state, logits and top-k must be identical bit for bit, over positions that cross
    several 128-token stages of the decode kernel and after a reset to position 0. With exclusive_device = 0 an
    attention call is two launches from three stages on (the splits are merged by a second kernel): the graph
    then holds two patched nodes per layer and is captured again where the count changes."""
    d = str(tmp_path / "m")
    model_dir.write_synthetic_model(d, seed=5)
    n = 300
    rng = np.random.default_rng(1)
    toks = rng.integers(0, 2048, n)
    outs = []
    for graph in (True, False):
        with bp.Model(d, max_seq=512) as gm:
            gm.set_step_graph(graph)
            gm.attention().set_option("exclusive_device", exclusive_device)
            rows = []
            for pos in list(range(n)) + [0, 1, 2]:
                lg, ix = gm.step_topk(int(toks[pos]), pos, k=32 if pos % 3 else 5)
                if pos % 16 == 0 or pos > n - 4:
                    rows.append((lg.copy(), ix.copy(), gm.hidden(0), gm.logits()))
                else:
                    rows.append((lg.copy(), ix.copy()))
            assert gm.graph_steps() == (n + 3 if graph else 0)
            assert not gm.attention().status()
            outs.append(rows)
    for a, b in zip(*outs):
        for u, v in zip(a, b):
            assert u.shape == v.shape and np.array_equal(u.view(np.uint8), v.view(np.uint8))


def test_free_running_passes_agree_on_the_top_candidates(tmp_path):
    """Without feeding attention across: GPU engine and CPU engine each with their own attention, one-token
    path and batched prefill. Attention differs within its tolerance, so logits are compared loosely and the
    chosen (greedy) tokens must be the same; the two GPU prefill paths must pick the same first token
    (tests/gpu_integration.rs:122-139)."""
    d = str(tmp_path / "m")
    model_dir.write_synthetic_model(d, seed=3)
    prompt = [1, 2, 3, 4, 5, 6, 7, 8]
    cpu = E.HostModel(d, 64)
    want_lg, want_ix = cpu.prefill(prompt)
    with bp.Model(d, max_seq=64) as gm:
        lg_mm, ix_mm = gm.prefill_topk(prompt)
        assert ix_mm[0] == want_ix[0] and np.max(np.abs(lg_mm - want_lg)) < 0.05
        x_mm = gm.hidden(len(prompt) - 1).astype(np.float32)
    with bp.Model(d, max_seq=64) as gm:
        lg_mv, ix_mv = gm.prefill_loop_topk(prompt)
        assert ix_mv[0] == ix_mm[0] and np.max(np.abs(lg_mv - lg_mm)) < 0.05
        cpu2 = E.HostModel(d, 64)
        for i, t in enumerate(prompt):
            out = cpu2.step(t, i, suffix=i == len(prompt) - 1)
        assert out[1][0] == ix_mv[0] and np.max(np.abs(out[0] - lg_mv)) < 0.05


def test_batched_prefill_is_identical_across_matmul_kernels(tmp_path):
    """A 40-token prefill takes the tensor-core matmul (one launch for Q, K and V, one for gate and up); the
    CUDA-core kernel and the tcgen05 kernel must give the same bits all the way to the logits."""
    d = str(tmp_path / "m")
    model_dir.write_synthetic_model(d, seed=5)
    prompt = [(7 * i + 3) % 200 for i in range(40)]
    lib = _lib.load()
    got = {}
    try:
        for variant in (1, 0, 3, 4, 5):
            lib.bp_op_set_matmul_variant(variant)
            with bp.Model(d, max_seq=64) as gm:
                lg, ix = gm.prefill_topk(prompt)
                got[variant] = (lg.copy(), ix.copy(), gm.hidden(len(prompt) - 1).copy(), gm.logits().copy())
    finally:
        lib.bp_op_set_matmul_variant(0)
    for variant in (0, 3):
        for a, b in zip(got[1], got[variant]):
            assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), variant


# ---------------------------------------------------------------------- session ----
def greedy():
    return bp.Sampler(temperature=0.0)


def greedy_opts(n):
    return bp.GenerateOptions(max_new_tokens=n, stop_pred=lambda _t: False, sampler=greedy())


def test_session_behaviour_of_the_reference_integration_tests(tmp_path):
    d = str(tmp_path / "m")
    model_dir.write_synthetic_model(d, seed=5)
    with pytest.raises(bp.IoError):                      # model_load_bad_path_is_io_error
        bp.Model(str(tmp_path / "does-not-exist"))
    prompt = [1, 2, 3, 4, 5, 6, 7, 8]
    with bp.Model(d, max_seq=1024) as m:
        s = m.new_session()
        s.prefill(prompt, greedy())
        assert s.pos() == 8
        with pytest.raises(bp.ConfigError):              # prefill_pos_nonzero_rejected
            s.prefill(prompt, greedy())
        s2 = m.new_session()
        with pytest.raises((bp.PrefillTooLarge, bp.ContextOverflow)):   # prefill_too_large_rejected
            s2.prefill([1] * 513, greedy())

        def run(sampler, n):
            sess = m.new_session()
            first = sess.prefill(prompt, sampler)
            toks, reason = sess.generate(first, bp.GenerateOptions(max_new_tokens=n, stop_pred=lambda _t: False, sampler=sampler))
            return first, toks, reason
        f1, t1, r1 = run(greedy(), 16)                   # greedy_is_byte_deterministic
        f2, t2, _ = run(greedy(), 16)
        assert (f1, t1) == (f2, t2) and len(t1) == 16 and r1 == bp.StopReason.MaxTokens
        a, b = m.new_session(), m.new_session()          # matvec_matmul_parity_first_token
        assert a.prefill(prompt, greedy()) == b.prefill_one_at_a_time(prompt, greedy())
        seeded = bp.Sampler(temperature=1.0, seed=42)    # seeded_sampler_reproducibility
        assert run(seeded, 8)[:2] == run(seeded, 8)[:2]
        assert run(seeded, 8)[:2] != run(bp.Sampler(temperature=1.0, seed=43), 8)[:2]
        fired = []                                       # generate_max_tokens_zero_returns_immediately
        s3 = m.new_session()
        assert s3.generate_streaming(0, greedy_opts(0), fired.append) == bp.StopReason.MaxTokens and not fired
        # stop predicate: the first sampled token stops the run and is not emitted
        s4 = m.new_session()
        first = s4.prefill(prompt, greedy())
        toks, reason = s4.generate(first, bp.GenerateOptions(max_new_tokens=5, stop_pred=lambda _t: True, sampler=greedy()))
        assert toks == [] and reason == bp.StopReason.Eos and s4.pos() == 9
        # snapshot_restore_round_trip_continues_identically
        s5 = m.new_session()
        first = s5.prefill(prompt, greedy())
        snap = s5.snapshot()
        cont1, _ = s5.generate(first, greedy_opts(6))
        s6 = m.new_session()
        s6.restore(bp.KvSnapshot.from_bytes(snap.to_bytes()))
        assert s6.pos() == 8
        cont2, _ = s6.generate(first, greedy_opts(6))
        assert cont1 == cont2
        # a context that runs out of positions reports it with the reference's fields
        with bp.Model(d, max_seq=10) as small:
            s7 = small.new_session()
            first = s7.prefill(prompt, greedy())
            with pytest.raises(bp.ContextOverflow) as e:
                s7.generate(first, greedy_opts(8))
            assert e.value.max == 10 and e.value.n == 1
