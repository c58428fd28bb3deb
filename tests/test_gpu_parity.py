"""GPU parity tests: every kernel is called through the C ABI and compared with
the CPU oracle on the same seeded inputs. Cache bytes and scales must be
bit-exact; attention outputs must satisfy |x - ref| <= 2e-3 + 1e-2 |ref| against
the binary64 softmax over the dequantised cache."""
import numpy as np
import pytest

import bonsai_pot_b200 as bp
from bonsai_pot_b200 import synth
from oracle import oracle as O
from tests.helpers import build_decode_case, within_tolerance

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def load_cache(ctx, sh, kv_k, kv_v, layer, rows):
    """Copy `rows` rows of one layer from host cache buffers into the context."""
    for kind, kv in enumerate((kv_k, kv_v)):
        ctx.kv_import(kind, layer, 0, rows, np.ascontiguousarray(sh.d_section(kv, layer)[:rows]))
        ctx.kv_import(kind, layer, 1, rows, np.ascontiguousarray(sh.qs_section(kv, layer)[:rows]))


def read_cache(ctx, sh, layer, rows):
    out = []
    for kind in range(2):
        d = np.empty((rows, sh.nb), dtype=np.float32)
        q = np.empty((rows, sh.kv_dim), dtype=np.int8)
        ctx.kv_export(kind, layer, 0, rows, d)
        ctx.kv_export(kind, layer, 1, rows, q)
        out.append((d, q))
    return out


def make_ctx(sh, **kw):
    return bp.AttnContext(n_layer=sh.n_layer, n_head=sh.n_head, n_kv_head=sh.n_kv_head, max_seq=sh.max_seq,
                          rms_eps=sh.rms_eps, rope_freq_base=sh.rope_freq_base, **kw)


# ---------------------------------------------------------------- K1 / K2 ----

def test_rope_table_bit_exact():
    sh = O.Shape(n_layer=1, max_seq=4096)
    with make_ctx(sh) as ctx:
        assert np.array_equal(ctx.rope_table().view(np.uint16).reshape(-1), O.rope_table_f16(sh).view(np.uint16))


@pytest.mark.parametrize("pos_base,m,layer", [(0, 1, 0), (512, 1, 2), (0, 7, 1), (3, 512, 2), (0, 2048, 0), (4095, 1, 2)])
def test_kv_writeback_bit_exact(pos_base, m, layer):
    sh = O.Shape(n_layer=3, max_seq=4096)
    rope = O.rope_table_f16(sh)
    k = synth.tensor(0, 2, layer, synth.T_K_NEW, (m, sh.kv_dim))
    v = synth.tensor(0, 2, layer, synth.T_V_NEW, (m, sh.kv_dim))
    w = (1 + 0.1 * np.random.default_rng(7).standard_normal(128)).astype(np.float16)
    ref_k, ref_v = sh.new_cache(), sh.new_cache()
    O.kv_writeback(sh, k, v, w, rope, ref_k, ref_v, layer, pos_base, m)
    with make_ctx(sh) as ctx:
        ctx.dispatch_kv_writeback_fused(layer, dev(k), dev(v), dev(w), pos_base, m)
        torch.cuda.synchronize()
        (kd, kq), (vd, vq) = read_cache(ctx, sh, layer, pos_base + m)
    sl = slice(pos_base, pos_base + m)
    assert np.array_equal(kq[sl], sh.qs_section(ref_k, layer)[sl])
    assert np.array_equal(kd[sl].view(np.uint32), sh.d_section(ref_k, layer)[sl].view(np.uint32))
    assert np.array_equal(vq[sl], sh.qs_section(ref_v, layer)[sl])
    assert np.array_equal(vd[sl].view(np.uint32), sh.d_section(ref_v, layer)[sl].view(np.uint32))


@pytest.mark.parametrize("pos_base,m", [(0, 1), (513, 1), (0, 512), (100, 2048)])
def test_q_norm_rope_bit_exact(pos_base, m):
    sh = O.Shape(n_layer=1, max_seq=4096)
    rope = O.rope_table_f16(sh)
    q = synth.tensor(1, 2, 0, synth.T_Q, (m, sh.q_dim))
    w = (1 + 0.1 * np.random.default_rng(8).standard_normal(128)).astype(np.float16)
    ref = O.q_norm_rope(sh, q, w, rope, pos_base, m)
    with make_ctx(sh) as ctx:
        qd = dev(q)
        ctx.dispatch_q_norm_rope_fused(qd, dev(w), pos_base, m)
        got = host(qd)
    assert np.array_equal(got.view(np.uint16).reshape(-1), ref.view(np.uint16).reshape(-1))


def test_writeback_edge_values():
    """All-zero blocks (d = 0), exact ties and the f16 maximum."""
    sh = O.Shape(n_layer=1, n_head=4, n_kv_head=1, max_seq=8)
    rope = O.rope_table_f16(sh)
    k = np.zeros((2, 128), dtype=np.float16)
    v = np.zeros((2, 128), dtype=np.float16)
    v[0, 32:64] = np.linspace(-2, 2, 32)
    v[0, 64:69] = [127.0, 0.5, 1.5, 2.5, -0.5]
    v[1, 0] = 65504.0
    v[1, 1] = -65504.0
    k[1, :] = 3.0
    w = synth.ones_weight()
    ref_k, ref_v = sh.new_cache(), sh.new_cache()
    O.kv_writeback(sh, k, v, w, rope, ref_k, ref_v, 0, 0, 2)
    with make_ctx(sh) as ctx:
        ctx.dispatch_kv_writeback_fused(0, dev(k), dev(v), dev(w), 0, 2)
        torch.cuda.synchronize()
        (kd, kq), (vd, vq) = read_cache(ctx, sh, 0, 2)
    assert np.array_equal(kq, sh.qs_section(ref_k, 0)[:2]) and np.array_equal(vq, sh.qs_section(ref_v, 0)[:2])
    assert np.array_equal(kd.view(np.uint32), sh.d_section(ref_k, 0)[:2].view(np.uint32))
    assert np.array_equal(vd.view(np.uint32), sh.d_section(ref_v, 0)[:2].view(np.uint32))
    assert vd[0, 0] == 0 and list(vq[0, 64:69]) == [127, 0, 2, 2, 0]


# ------------------------------------------------------------------ decode ----

def run_decode(ctx, sh, case, layer, variant=0):
    ctx.set_variant(variant)
    out = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
    ctx.dispatch_attention_decode(layer, dev(case["qn"]), out, case["cur_pos"])
    torch.cuda.synchronize()
    assert ctx.status() == 0
    return host(out)


@pytest.mark.parametrize("variant", [0, 1, 2, 3])
def test_decode_every_small_position(variant):
    """cur_pos 1..72 and the tile edges around 128/256/512: every tail length of
    the 16-token sub-tile and of the split is exercised."""
    sh = O.Shape(n_layer=2, max_seq=1024)
    positions = list(range(1, 73)) + [127, 128, 129, 255, 256, 257, 511, 512, 513]
    case = build_decode_case(sh, seed=0, cfg_id=0, layer=1, n_past=max(positions) - 1)
    with make_ctx(sh) as ctx:
        load_cache(ctx, sh, case["kv_k"], case["kv_v"], 1, max(positions))
        for cur_pos in positions:
            c = dict(case, cur_pos=cur_pos)
            got = run_decode(ctx, sh, c, 1, variant)
            exact = O.attn_exact(sh, case["qn"], case["kv_k"], case["kv_v"], 1, 1, cur_pos - 1)[0]
            ok, max_abs, max_rel = within_tolerance(got, exact)
            assert ok, (variant, cur_pos, max_abs, max_rel)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_decode_config0_end_to_end(seed):
    """BASELINE config 0: 512 past tokens, the new token goes through
    q_norm_rope + kv_writeback on the GPU, then decode over 513 keys."""
    sh = O.Shape(n_layer=1, max_seq=1024)
    case = build_decode_case(sh, seed=seed, cfg_id=0, layer=0, n_past=512)
    with make_ctx(sh) as ctx:
        load_cache(ctx, sh, case["kv_k"], case["kv_v"], 0, 512)  # past rows only
        qd = dev(case["q"])
        ctx.dispatch_q_norm_rope_fused(qd, dev(case["w_q"]), 512, 1)
        ctx.dispatch_kv_writeback_fused(0, dev(case["k_new"]), dev(case["v_new"]), dev(case["w_k"]), 512, 1)
        out = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
        ctx.dispatch_attention_decode(0, qd, out, 513)
        torch.cuda.synchronize()
        assert np.array_equal(host(qd).view(np.uint16).reshape(-1), case["qn"].view(np.uint16).reshape(-1))
        (kd, kq), (vd, vq) = read_cache(ctx, sh, 0, 513)
        assert np.array_equal(kq, sh.qs_section(case["kv_k"], 0)[:513])
        assert np.array_equal(kd.view(np.uint32), sh.d_section(case["kv_k"], 0)[:513].view(np.uint32))
        assert np.array_equal(vq, sh.qs_section(case["kv_v"], 0)[:513])
        assert np.array_equal(vd.view(np.uint32), sh.d_section(case["kv_v"], 0)[:513].view(np.uint32))
        got = host(out)
    exact = O.attn_exact(sh, case["qn"], case["kv_k"], case["kv_v"], 0, 1, 512)[0]
    ref_order = O.attn_decode(sh, case["qn"], case["kv_k"], case["kv_v"], 0, 513).astype(np.float32)
    ok, max_abs, max_rel = within_tolerance(got, exact)
    assert ok, (max_abs, max_rel)
    assert within_tolerance(got, ref_order)[0]


@pytest.mark.parametrize("variant", [0, 3])
@pytest.mark.parametrize("n_past", [0, 1, 126, 127, 128, 129, 511, 700, 4095])
def test_decode_layer_fused_equals_the_three_dispatches(n_past, variant):
    """bp_attn_decode_layer = q_norm_rope_fused + kv_writeback_fused + decode attention in one call
    (src/forward.rs:612-631): the cache rows and the rotated q are bit-exact against the oracle, the raw q
    is left alone, and the output equals the separate calls' output bit for bit."""
    sh = O.Shape(n_layer=2, max_seq=4096)
    layer = 1
    rng = np.random.default_rng(31)
    w_q = (1 + 0.1 * rng.standard_normal(128)).astype(np.float16)
    w_k = (1 + 0.1 * rng.standard_normal(128)).astype(np.float16)
    case = build_decode_case(sh, seed=3, cfg_id=0, layer=layer, n_past=n_past, w_q=w_q, w_k=w_k)
    with make_ctx(sh) as ctx:
        ctx.set_variant(variant)
        if n_past:
            load_cache(ctx, sh, case["kv_k"], case["kv_v"], layer, n_past)  # past rows only
        q_raw = dev(case["q"])
        q_roped = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
        out = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
        ctx.decode_layer(layer, q_raw, dev(w_q), dev(case["k_new"]), dev(case["v_new"]), dev(w_k), n_past, out,
                         q_roped=q_roped)
        torch.cuda.synchronize()
        assert np.array_equal(host(q_raw).view(np.uint16).reshape(-1), case["q"].view(np.uint16).reshape(-1))
        assert np.array_equal(host(q_roped).view(np.uint16).reshape(-1), case["qn"].view(np.uint16).reshape(-1))
        (kd, kq), (vd, vq) = read_cache(ctx, sh, layer, n_past + 1)
        assert np.array_equal(kq, sh.qs_section(case["kv_k"], layer)[:n_past + 1])
        assert np.array_equal(kd.view(np.uint32), sh.d_section(case["kv_k"], layer)[:n_past + 1].view(np.uint32))
        assert np.array_equal(vq, sh.qs_section(case["kv_v"], layer)[:n_past + 1])
        assert np.array_equal(vd.view(np.uint32), sh.d_section(case["kv_v"], layer)[:n_past + 1].view(np.uint32))
        fused = host(out).copy()
        # the same step through the three dispatches, and once more fused without a q_roped buffer
        out2 = torch.zeros_like(out)
        ctx.dispatch_attention_decode(layer, q_roped, out2, n_past + 1)
        out3 = torch.zeros_like(out)
        ctx.decode_layer(layer, q_raw, dev(w_q), dev(case["k_new"]), dev(case["v_new"]), dev(w_k), n_past, out3)
        torch.cuda.synchronize()
        assert np.array_equal(fused.view(np.uint16), host(out2).view(np.uint16))
        assert np.array_equal(fused.view(np.uint16), host(out3).view(np.uint16))
    exact = O.attn_exact(sh, case["qn"], case["kv_k"], case["kv_v"], layer, 1, n_past)[0]
    ok, max_abs, max_rel = within_tolerance(fused, exact)
    assert ok, (max_abs, max_rel)


def test_peer_exchange_epilogue_on_one_rank():
    """The decode kernel's peer-store epilogue with a single rank acting as its own peer: the gathered
    buffer receives every layer's outputs, and the meeting kernel counts one arrival per call on its slot."""
    sh = O.Shape(n_layer=3, max_seq=2048)
    case = build_decode_case(sh, seed=4, cfg_id=0, layer=0, n_past=1500)
    with make_ctx(sh) as ctx:
        gathered = torch.zeros(sh.n_layer, sh.q_dim, dtype=torch.float16, device="cuda")
        flags = torch.zeros(64, dtype=torch.int32, device="cuda")
        ctx.set_peer_exchange([gathered.data_ptr()], [flags.data_ptr()])
        outs = []
        for token in range(2):
            for layer in range(sh.n_layer):
                load_cache(ctx, sh, case["kv_k"], case["kv_v"], 0, 1500) if layer == 0 and token == 0 else None
                out = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
                n_keys = 1501 if layer == 0 else 1
                if layer > 0:  # other layers: a single key written by the fused step itself
                    ctx.decode_layer(layer, dev(case["q"]), dev(case["w_q"]), dev(case["k_new"]), dev(case["v_new"]),
                                     dev(case["w_k"]), 0, out)
                else:
                    ctx.decode_layer(0, dev(case["q"]), dev(case["w_q"]), dev(case["k_new"]), dev(case["v_new"]),
                                     dev(case["w_k"]), 1500, out)
                outs.append(out)
            ctx.peer_sync(slot=5)
            torch.cuda.synchronize()
            assert ctx.status() == 0
            for layer in range(sh.n_layer):
                assert torch.equal(gathered[layer], outs[token * sh.n_layer + layer])
            assert flags[5].item() == token + 1 and flags[:5].abs().sum().item() == 0
        ctx.set_peer_exchange([], [])
    ref = O.attn_decode(sh, case["qn"], case["kv_k"], case["kv_v"], 0, 1501).astype(np.float32)
    assert within_tolerance(host(outs[0]), ref)[0]


@pytest.mark.parametrize("ctx_len,layer", [(4096, 1), (32768, 1)])
def test_decode_long_context(ctx_len, layer):
    """BASELINE configs 1 and 3 at full context length (two layers allocated,
    the second one used so that the layer offset is exercised)."""
    sh = O.Shape(n_layer=2, max_seq=ctx_len)
    case = build_decode_case(sh, seed=0, cfg_id=3, layer=layer, n_past=ctx_len - 1)
    exact = O.attn_exact(sh, case["qn"], case["kv_k"], case["kv_v"], layer, 1, ctx_len - 1)[0]
    with make_ctx(sh) as ctx:
        load_cache(ctx, sh, case["kv_k"], case["kv_v"], layer, ctx_len)
        for variant in (0, 1, 3):
            got = run_decode(ctx, sh, case, layer, variant)
            ok, max_abs, max_rel = within_tolerance(got, exact)
            assert ok, (variant, max_abs, max_rel)
        a = run_decode(ctx, sh, case, layer, 0)
        b = run_decode(ctx, sh, case, layer, 0)
        assert np.array_equal(a.view(np.uint16), b.view(np.uint16))  # run-to-run determinism


@pytest.mark.parametrize("n_kv_head", [1, 2, 4])
def test_decode_on_a_kv_head_shard(n_kv_head):
    """A context that holds n_kv_head of the 8 KV heads (and 4x as many query
    heads) must reproduce the matching slice of the full result."""
    full = O.Shape(n_layer=1, max_seq=2048)
    n_past = 1500
    case = build_decode_case(full, seed=4, cfg_id=3, layer=0, n_past=n_past)
    exact = O.attn_exact(full, case["qn"], case["kv_k"], case["kv_v"], 0, 1, n_past)[0]
    n_shards = 8 // n_kv_head
    shard = n_shards - 1
    sh = O.Shape(n_layer=1, n_head=4 * n_kv_head, n_kv_head=n_kv_head, max_seq=2048)
    cols = slice(shard * sh.kv_dim, (shard + 1) * sh.kv_dim)
    bcols = slice(shard * sh.nb, (shard + 1) * sh.nb)
    qcols = slice(shard * sh.q_dim, (shard + 1) * sh.q_dim)
    with make_ctx(sh, n_shards=n_shards, shard=shard) as ctx:
        for kind, kv in enumerate((case["kv_k"], case["kv_v"])):
            ctx.kv_import(kind, 0, 0, n_past + 1, np.ascontiguousarray(full.d_section(kv, 0)[:n_past + 1, bcols]))
            ctx.kv_import(kind, 0, 1, n_past + 1, np.ascontiguousarray(full.qs_section(kv, 0)[:n_past + 1, cols]))
        for variant in (0, 1, 3):
            ctx.set_variant(variant)
            out = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
            ctx.dispatch_attention_decode(0, dev(case["qn"][:, qcols]), out, n_past + 1)
            torch.cuda.synchronize()
            ok, max_abs, max_rel = within_tolerance(host(out), exact[qcols])
            assert ok, (variant, max_abs, max_rel)


# ----------------------------------------------------------------- prefill ----

def prefill_case(sh, seed, layer, m):
    rope = O.rope_table_f16(sh)
    q = synth.tensor(seed, 2, layer, synth.T_Q, (m, sh.q_dim))
    k = synth.tensor(seed, 2, layer, synth.T_K_NEW, (m, sh.kv_dim))
    v = synth.tensor(seed, 2, layer, synth.T_V_NEW, (m, sh.kv_dim))
    w = synth.ones_weight()
    kv_k, kv_v = sh.new_cache(), sh.new_cache()
    O.kv_writeback(sh, k, v, w, rope, kv_k, kv_v, layer, 0, m)
    qn = O.q_norm_rope(sh, q, w, rope, 0, m)
    return dict(q=q, k=k, v=v, w=w, kv_k=kv_k, kv_v=kv_v, qn=qn)


@pytest.mark.parametrize("m", [1, 5, 33, 64, 100, 512])
@pytest.mark.parametrize("variant", [0, 1])
def test_prefill_pass_matches_oracle(m, variant):
    """BASELINE config 2 for one layer: q_norm_rope, kv_writeback and the causal
    attention in one pass, as layer_step_matmul_in_pass issues them."""
    sh = O.Shape(n_layer=2, max_seq=2048)
    c = prefill_case(sh, seed=0, layer=1, m=m)
    exact = O.attn_exact(sh, c["qn"], c["kv_k"], c["kv_v"], 1, m, 0)
    with make_ctx(sh) as ctx:
        ctx.set_variant(variant)
        qd = dev(c["q"])
        out = torch.zeros(m, sh.q_dim, dtype=torch.float16, device="cuda")
        ctx.dispatch_q_norm_rope_fused(qd, dev(c["w"]), 0, m)
        ctx.dispatch_kv_writeback_fused(1, dev(c["k"]), dev(c["v"]), dev(c["w"]), 0, m)
        ctx.dispatch_attention(1, qd, out, m)
        torch.cuda.synchronize()
        got = host(out)
        (kd, kq), _ = read_cache(ctx, sh, 1, m)
        assert np.array_equal(kq, sh.qs_section(c["kv_k"], 1)[:m])
    ok, max_abs, max_rel = within_tolerance(got, exact)
    assert ok, (m, variant, max_abs, max_rel)
    if m <= 100:
        ref_order = O.attn_prefill(sh, c["qn"], c["kv_k"], c["kv_v"], 1, m).astype(np.float32)
        assert within_tolerance(got, ref_order)[0]


def test_prefill_2048_beyond_the_reference_cap():
    """pp = 2048 is larger than the reference's M_MAX = 512; the oracle defines it."""
    sh = O.Shape(n_layer=1, max_seq=2048)
    m = 2048
    c = prefill_case(sh, seed=1, layer=0, m=m)
    exact = O.attn_exact(sh, c["qn"], c["kv_k"], c["kv_v"], 0, m, 0)
    with make_ctx(sh) as ctx:
        load_cache(ctx, sh, c["kv_k"], c["kv_v"], 0, m)
        out = torch.zeros(m, sh.q_dim, dtype=torch.float16, device="cuda")
        ctx.dispatch_attention(0, dev(c["qn"]), out, m)
        torch.cuda.synchronize()
        got = host(out)
    ok, max_abs, max_rel = within_tolerance(got, exact)
    assert ok, (max_abs, max_rel)


def test_prefill_and_decode_paths_agree_on_the_gpu():
    """The invariant of tests/gpu_integration.rs:122-139."""
    sh = O.Shape(n_layer=1, max_seq=256)
    m = 200
    c = prefill_case(sh, seed=3, layer=0, m=m)
    with make_ctx(sh) as ctx:
        load_cache(ctx, sh, c["kv_k"], c["kv_v"], 0, m)
        qd = dev(c["qn"])
        out = torch.zeros(m, sh.q_dim, dtype=torch.float16, device="cuda")
        ctx.dispatch_attention(0, qd, out, m)
        pre = host(out)
        for tok in (0, 15, 16, 17, 63, 64, 199):
            o1 = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
            ctx.dispatch_attention_decode(0, qd[tok], o1, tok + 1)
            torch.cuda.synchronize()
            ok, max_abs, _ = within_tolerance(host(o1), pre[tok].astype(np.float32))
            assert ok and max_abs <= 2e-3, (tok, max_abs)


# ------------------------------------------------ guards, latch, snapshots ----

def test_guards_fire_before_gpu_work():
    sh = O.Shape(n_layer=2, max_seq=64)
    with make_ctx(sh, max_prefill=16) as ctx:
        buf = torch.zeros(64 * sh.q_dim, dtype=torch.float16, device="cuda")
        w = dev(synth.ones_weight())
        with pytest.raises(bp.ContextOverflow) as e:
            ctx.dispatch_kv_writeback_fused(0, buf, buf, w, 60, 5)
        assert (e.value.pos, e.value.n, e.value.max) == (60, 5, 64)
        assert str(e.value) == "context overflow: pos 60 + tokens 5 > max_seq 64"
        with pytest.raises(bp.PrefillTooLarge) as e:  # tests/gpu_integration.rs:87-100
            ctx.dispatch_attention(0, buf, buf, 17)
        assert (e.value.n, e.value.max) == (17, 16)
        assert str(e.value) == "prefill batch 17 exceeds max_prefill_tokens 16"
        assert ctx.max_prefill_tokens() == 16
        with pytest.raises(bp.ContextOverflow):
            ctx.dispatch_attention_decode(0, buf, buf, 65)
        with pytest.raises(bp.ConfigError):
            ctx.dispatch_attention_decode(2, buf, buf, 1)
        with pytest.raises(bp.ConfigError):
            ctx.dispatch_attention_decode(0, buf, buf, 0)
        assert ctx.status() == 0  # none of these latched anything


def test_device_lost_latch_and_recovery_by_snapshot():
    """tests/gpu_integration.rs:268-336, with the loss injected on the host: every
    later call fails fast; recovery is a new context plus Session::restore."""
    sh = O.Shape(n_layer=2, max_seq=128)
    case = build_decode_case(sh, seed=5, cfg_id=0, layer=1, n_past=90)
    ctx = make_ctx(sh)
    load_cache(ctx, sh, case["kv_k"], case["kv_v"], 1, 91)
    load_cache(ctx, sh, case["kv_k"], case["kv_v"], 0, 91)
    before = run_decode(ctx, sh, case, 1)
    snap = bp.KvSnapshot.capture(ctx, 91)
    ctx.inject_device_lost()
    assert ctx.is_device_lost()
    out = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
    for call in (lambda: ctx.dispatch_attention_decode(1, dev(case["qn"]), out, 91),
                 lambda: ctx.dispatch_q_norm_rope_fused(out, out, 0, 1),
                 lambda: ctx.kv_export(0, 0, 0, 1, np.zeros(32, np.float32)),
                 lambda: bp.KvSnapshot.capture(ctx, 1)):
        with pytest.raises(bp.DeviceLost):
            call()
    ctx.close()
    fresh = make_ctx(O.Shape(n_layer=2, max_seq=256))  # a different max_seq is allowed
    assert not fresh.is_device_lost()
    assert bp.KvSnapshot.from_bytes(snap.to_bytes()).apply(fresh) == 91
    out2 = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
    fresh.dispatch_attention_decode(1, dev(case["qn"]), out2, 91)
    torch.cuda.synchronize()
    assert np.array_equal(host(out2).view(np.uint16), before.view(np.uint16))
    fresh.close()


def test_snapshot_blob_is_byte_identical_to_the_reference_layout():
    sh = O.Shape(n_layer=3, max_seq=64)
    rope = O.rope_table_f16(sh)
    kv_k, kv_v = sh.new_cache(), sh.new_cache()
    w = synth.ones_weight()
    pos = 40
    with make_ctx(sh) as ctx:
        for il in range(3):
            k = synth.tensor(6, 2, il, synth.T_K_NEW, (pos, sh.kv_dim))
            v = synth.tensor(6, 2, il, synth.T_V_NEW, (pos, sh.kv_dim))
            O.kv_writeback(sh, k, v, w, rope, kv_k, kv_v, il, 0, pos)
            ctx.dispatch_kv_writeback_fused(il, dev(k), dev(v), dev(w), 0, pos)
        torch.cuda.synchronize()
        snap = bp.KvSnapshot.capture(ctx, pos)
        assert snap.to_bytes() == O.snapshot_blob(sh, kv_k, kv_v, pos)
        assert bp.KvSnapshot.capture(ctx, 0).to_bytes() == O.snapshot_blob(sh, kv_k, kv_v, 0)
        too_long = bp.KvSnapshot(3, 1024, 64, 65, bytes(O.payload_bytes(3, 1024, 65)))
        with pytest.raises(bp.ContextOverflow) as e:
            too_long.apply(ctx)
        assert (e.value.pos, e.value.n, e.value.max) == (0, 65, 64)
        with pytest.raises(bp.ConfigError):
            bp.KvSnapshot(4, 1024, 64, 1, bytes(O.payload_bytes(4, 1024, 1))).apply(ctx)


def test_sharded_snapshot_assembles_the_global_blob():
    full = O.Shape(n_layer=2, max_seq=32)
    rope = O.rope_table_f16(full)
    pos = 20
    kv_k, kv_v = full.new_cache(), full.new_cache()
    k = synth.tensor(7, 2, 0, synth.T_K_NEW, (pos, full.kv_dim))
    v = synth.tensor(7, 2, 0, synth.T_V_NEW, (pos, full.kv_dim))
    w = synth.ones_weight()
    for il in range(2):
        O.kv_writeback(full, k, v, w, rope, kv_k, kv_v, il, 0, pos)
    part = O.Shape(n_layer=2, n_head=16, n_kv_head=4, max_seq=32)
    shards = [make_ctx(part, n_shards=2, shard=s) for s in range(2)]
    for s, ctx in enumerate(shards):
        cols = slice(s * part.kv_dim, (s + 1) * part.kv_dim)
        for il in range(2):
            ctx.dispatch_kv_writeback_fused(il, dev(k[:, cols]), dev(v[:, cols]), dev(w), 0, pos)
    torch.cuda.synchronize()
    snap = bp.KvSnapshot.capture(shards, pos)
    assert snap.kv_dim == 1024 and snap.to_bytes() == O.snapshot_blob(full, kv_k, kv_v, pos)
    fresh = [make_ctx(part, n_shards=2, shard=s) for s in range(2)]
    assert snap.apply(fresh) == pos
    assert bp.KvSnapshot.capture(fresh, pos).to_bytes() == snap.to_bytes()
    for c in shards + fresh:
        c.close()


def test_host_entry_points_equal_the_device_path():
    sh = O.Shape(n_layer=2, max_seq=1024)
    case = build_decode_case(sh, seed=8, cfg_id=0, layer=1, n_past=700)
    with make_ctx(sh) as ctx:
        load_cache(ctx, sh, case["kv_k"], case["kv_v"], 1, 700)
        out_h = np.zeros(sh.q_dim, dtype=np.float16)
        ctx.decode_step_host(1, case["q"], case["k_new"], case["v_new"], case["w_q"], case["w_k"], 700, out_h)
        assert ctx.last_launch_count() >= 1  # one fused layer step (the splits are merged inside the launch)
        got_dev = run_decode(ctx, sh, case, 1)
        assert np.array_equal(out_h.view(np.uint16), got_dev.view(np.uint16))
        m = 48
        c = prefill_case(sh, seed=9, layer=0, m=m)
        out_p = np.zeros((m, sh.q_dim), dtype=np.float16)
        ctx.prefill_layer_host(0, c["q"], c["k"], c["v"], c["w"], c["w"], m, out_p)
        exact = O.attn_exact(sh, c["qn"], c["kv_k"], c["kv_v"], 0, m, 0)
        assert within_tolerance(out_p, exact)[0]


def test_token_host_entry_point_equals_per_layer_calls():
    sh = O.Shape(n_layer=3, max_seq=512)
    rng_cases = [build_decode_case(sh, seed=10, cfg_id=1, layer=il, n_past=300) for il in range(3)]
    q = np.concatenate([c["q"] for c in rng_cases]); k = np.concatenate([c["k_new"] for c in rng_cases])
    v = np.concatenate([c["v_new"] for c in rng_cases])
    w = synth.ones_weight()
    with make_ctx(sh) as ctx:
        for il, c in enumerate(rng_cases):
            load_cache(ctx, sh, c["kv_k"], c["kv_v"], il, 300)
        out = np.zeros((3, sh.q_dim), dtype=np.float16)
        ctx.decode_token_host(q, k, v, w, w, 300, out)
        for il, c in enumerate(rng_cases):
            exact = O.attn_exact(sh, c["qn"], c["kv_k"], c["kv_v"], il, 1, 300)[0]
            assert within_tolerance(out[il], exact)[0]
            (kd, kq), _ = read_cache(ctx, sh, il, 301)
            assert np.array_equal(kq[300], sh.qs_section(c["kv_k"], il)[300])
        with pytest.raises(bp.ContextOverflow):
            ctx.decode_token_host(q, k, v, w, w, 512, out)


def test_token_host_graph_launch_is_identical_to_stream_launches():
    """bp_decode_token_host sends the layers' launches as one CUDA graph launch whose nodes are patched for
    every token's position (captured again when the launch changes shape): tokens at positions that cross
    several 128-token stages and the 16-split threshold of the decode kernel, then back to a short context,
    against the same calls as stream launches on a second context. Outputs and cache rows bit for bit."""
    sh = O.Shape(n_layer=3, max_seq=4096)
    rng = np.random.default_rng(21)
    w = synth.ones_weight()
    positions = list(range(0, 6)) + list(range(126, 131)) + list(range(2040, 2052)) + [3000, 3001, 4095, 7, 8]
    seq = [(rng.standard_normal(3 * sh.q_dim).astype(np.float16), rng.standard_normal(3 * sh.kv_dim).astype(np.float16),
            rng.standard_normal(3 * sh.kv_dim).astype(np.float16)) for _ in positions]
    results = []
    for graph in (1, 0):
        with make_ctx(sh) as ctx:
            ctx.set_option("token_graph", graph)
            fill = np.random.default_rng(22)  # the same cache rows under both runs
            for il in range(3):
                for kind in range(2):
                    ctx.kv_import(kind, il, 0, 4096, (fill.random((4096, sh.nb), dtype=np.float32) * 0.05 + 0.001))
                    ctx.kv_import(kind, il, 1, 4096, fill.integers(-127, 128, (4096, sh.kv_dim), dtype=np.int8))
            outs = []
            for (q, k, v), pos in zip(seq, positions):
                out = np.zeros((3, sh.q_dim), dtype=np.float16)
                ctx.decode_token_host(q, k, v, w, w, pos, out)
                outs.append(out.copy())
            assert not ctx.status()
            rows = [read_cache(ctx, sh, il, 4096) for il in range(3)]
            results.append((outs, rows))
    for a, b in zip(results[0][0], results[1][0]):
        assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
    for ra, rb in zip(results[0][1], results[1][1]):
        for (da, qa), (db, qb) in zip(ra, rb):
            assert np.array_equal(da.view(np.uint32), db.view(np.uint32)) and np.array_equal(qa, qb)


@pytest.mark.parametrize("warps,hpc", [(16, 8), (8, 4), (8, 2), (16, 1), (8, 1)])
def test_decode_tuning_options_do_not_change_results(warps, hpc):
    sh = O.Shape(n_layer=2, max_seq=4096)
    case = build_decode_case(sh, seed=11, cfg_id=1, layer=1, n_past=3000)
    with make_ctx(sh) as ctx:
        load_cache(ctx, sh, case["kv_k"], case["kv_v"], 1, 3001)
        ctx.set_option("decode_warps", warps)
        ctx.set_option("decode_heads_per_cta", hpc)
        ctx.set_option("decode_umma_heads_per_cta", 1 if hpc == 1 else 2)
        for cur_pos in (1, 17, 100, 777, 3001):
            for variant in (0, 3):
                got = run_decode(ctx, sh, dict(case, cur_pos=cur_pos), 1, variant)
                exact = O.attn_exact(sh, case["qn"], case["kv_k"], case["kv_v"], 1, 1, cur_pos - 1)[0]
                ok, max_abs, max_rel = within_tolerance(got, exact)
                assert ok, (warps, hpc, variant, cur_pos, max_abs, max_rel)
            got = run_decode(ctx, sh, dict(case, cur_pos=cur_pos), 1)
            exact = O.attn_exact(sh, case["qn"], case["kv_k"], case["kv_v"], 1, 1, cur_pos - 1)[0]
            ok, max_abs, max_rel = within_tolerance(got, exact)
            assert ok, (warps, hpc, cur_pos, max_abs, max_rel)
        with pytest.raises(bp.ConfigError):
            ctx.set_option("decode_warps", 12)


@pytest.mark.parametrize("merge,pdl", [(0, 1), (1, 0), (0, 0)])
def test_decode_launch_structure_options_do_not_change_results(merge, pdl):
    """Separate merge kernel vs in-kernel merge, plain vs programmatic dependent launches: results stay
    within tolerance of the exact softmax and within 1e-3 of the default structure (the partials are
    the same; the two merges sum the splits in different groupings)."""
    sh = O.Shape(n_layer=1, max_seq=4096)
    case = build_decode_case(sh, seed=12, cfg_id=1, layer=0, n_past=4000)
    with make_ctx(sh) as ctx:
        load_cache(ctx, sh, case["kv_k"], case["kv_v"], 0, 4001)
        base = run_decode(ctx, sh, case, 0)
        ctx.set_option("decode_in_kernel_merge", merge)
        ctx.set_option("dependent_launch", pdl)
        got = run_decode(ctx, sh, case, 0)
        exact = O.attn_exact(sh, case["qn"], case["kv_k"], case["kv_v"], 0, 1, 4000)[0]
        ok, max_abs, max_rel = within_tolerance(got, exact)
        assert ok, (merge, pdl, max_abs, max_rel)
        assert np.abs(got.astype(np.float32) - base.astype(np.float32)).max() <= 1e-3


@pytest.mark.parametrize("tiles_per_item", [1, 2, 3])
@pytest.mark.parametrize("m", [65, 129, 512, 700, 2048])
def test_prefill_tile_modes_against_the_scalar_kernel(m, tiles_per_item):
    """Both work-item shapes of the tensor-core prefill kernel (one or two query tiles per item), on sizes
    that give every SM an item and some SMs several, against the plain CUDA-core kernel on the same cache.
    Repeated launches: a hand-over between the kernel's roles that only fails under some timing shows here."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(100 + m)
    with bp.AttnContext(n_layer=1, max_seq=2048) as ctx:
        w = torch.ones(128, dtype=torch.float16, device="cuda")
        q = torch.randn(m, 4096, generator=gen, device="cuda").half()
        k = torch.randn(m, 1024, generator=gen, device="cuda").half()
        v = torch.randn(m, 1024, generator=gen, device="cuda").half()
        ctx.dispatch_q_norm_rope_fused(q, w, 0, m)
        ctx.dispatch_kv_writeback_fused(0, k, v, w, 0, m)
        ref = torch.zeros(m, 4096, dtype=torch.float16, device="cuda")
        ctx.set_variant(1)
        ctx.dispatch_attention(0, q, ref, m)
        torch.cuda.synchronize()
        ctx.set_variant(0)
        ctx.set_option("prefill_tiles_per_item", tiles_per_item)
        for _ in range(3):
            out = torch.full((m, 4096), float("nan"), dtype=torch.float16, device="cuda")
            ctx.dispatch_attention(0, q, out, m)
            torch.cuda.synchronize()
            assert ctx.status() == 0
            ok, max_abs, max_rel = within_tolerance(host(out), host(ref).astype(np.float32))
            assert ok, (m, tiles_per_item, max_abs, max_rel)


@pytest.mark.parametrize("n_head,n_kv_head", [(2, 1), (6, 2), (8, 2)])
def test_norm_rope_quant_bit_exact_for_other_head_counts(n_head, n_kv_head):
    """The batched kernels take 4, 2 or 1 heads per warp depending on what divides the head count: every
    grouping must give the oracle's bits."""
    m = 2048
    sh = O.Shape(n_layer=1, n_head=n_head, n_kv_head=n_kv_head, max_seq=m)
    rope = O.rope_table_f16(sh)
    rng = np.random.default_rng(17)
    w = (1 + 0.1 * rng.standard_normal(128)).astype(np.float16)
    q = synth.tensor(5, 2, 0, synth.T_Q, (m, sh.q_dim))
    k = synth.tensor(5, 2, 0, synth.T_K_NEW, (m, sh.kv_dim))
    v = synth.tensor(5, 2, 0, synth.T_V_NEW, (m, sh.kv_dim))
    ref_k, ref_v = sh.new_cache(), sh.new_cache()
    O.kv_writeback(sh, k, v, w, rope, ref_k, ref_v, 0, 0, m)
    ref_q = O.q_norm_rope(sh, q, w, rope, 0, m)
    with make_ctx(sh) as ctx:
        qd = dev(q)
        ctx.dispatch_q_norm_rope_fused(qd, dev(w), 0, m)
        ctx.dispatch_kv_writeback_fused(0, dev(k), dev(v), dev(w), 0, m)
        torch.cuda.synchronize()
        (kd, kq), (vd, vq) = read_cache(ctx, sh, 0, m)
        assert np.array_equal(host(qd).view(np.uint16).reshape(-1), ref_q.view(np.uint16).reshape(-1))
    assert np.array_equal(kq, sh.qs_section(ref_k, 0)[:m]) and np.array_equal(vq, sh.qs_section(ref_v, 0)[:m])
    assert np.array_equal(kd.view(np.uint32), sh.d_section(ref_k, 0)[:m].view(np.uint32))
    assert np.array_equal(vd.view(np.uint32), sh.d_section(ref_v, 0)[:m].view(np.uint32))


@pytest.mark.parametrize("n_head,n_kv_head", [(4, 1), (8, 2), (16, 4)])
def test_prefill_on_a_kv_head_shard(n_head, n_kv_head):
    """A context that holds the heads of one of N shards (n_head / N, n_kv_head / N): the tensor-core
    prefill kernel against the plain CUDA-core kernel on the same cache, 700 tokens."""
    m = 700
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7 * n_head)
    with bp.AttnContext(n_layer=1, n_head=n_head, n_kv_head=n_kv_head, max_seq=1024, n_shards=8 // n_kv_head,
                        shard=0) as ctx:
        w = torch.ones(128, dtype=torch.float16, device="cuda")
        q = torch.randn(m, n_head * 128, generator=gen, device="cuda").half()
        k = torch.randn(m, n_kv_head * 128, generator=gen, device="cuda").half()
        v = torch.randn(m, n_kv_head * 128, generator=gen, device="cuda").half()
        ctx.dispatch_q_norm_rope_fused(q, w, 0, m)
        ctx.dispatch_kv_writeback_fused(0, k, v, w, 0, m)
        ref = torch.zeros(m, n_head * 128, dtype=torch.float16, device="cuda")
        ctx.set_variant(1)
        ctx.dispatch_attention(0, q, ref, m)
        torch.cuda.synchronize()
        ctx.set_variant(0)
        for tiles in (0, 1, 2, 3):
            ctx.set_option("prefill_tiles_per_item", tiles)
            out = torch.full((m, n_head * 128), float("nan"), dtype=torch.float16, device="cuda")
            ctx.dispatch_attention(0, q, out, m)
            torch.cuda.synchronize()
            assert ctx.status() == 0
            ok, max_abs, max_rel = within_tolerance(host(out), host(ref).astype(np.float32))
            assert ok, (n_head, n_kv_head, tiles, max_abs, max_rel)


@pytest.mark.parametrize("n_kv_head,ctx_len", [(1, 32768), (2, 20000), (8, 4096), (8, 4100), (8, 16384)])
def test_decode_merge_of_many_splits(n_kv_head, ctx_len):
    """The in-kernel merge of the splits (one merging CTA for short launches, all CTAs of a head group for
    long ones, more than 32 splits on a one-head shard) against the separate combine kernel and the
    warp-MMA family on the same cache, twice in a row (the second launch must see fresh tags)."""
    n_head = 4 * n_kv_head
    gen = torch.Generator(device="cuda")
    gen.manual_seed(ctx_len + n_kv_head)
    with bp.AttnContext(n_layer=1, n_head=n_head, n_kv_head=n_kv_head, max_seq=ctx_len, n_shards=8 // n_kv_head,
                        shard=0) as ctx:
        w = torch.ones(128, dtype=torch.float16, device="cuda")
        for r0 in range(0, ctx_len, 4096):
            rows = min(4096, ctx_len - r0)
            k = torch.randn(rows, n_kv_head * 128, generator=gen, device="cuda").half()
            v = torch.randn(rows, n_kv_head * 128, generator=gen, device="cuda").half()
            ctx.dispatch_kv_writeback_fused(0, k, v, w, r0, rows)
        q = torch.randn(n_head * 128, generator=gen, device="cuda").half()
        ctx.dispatch_q_norm_rope_fused(q, w, ctx_len - 1, 1)
        outs = {}
        for name, variant, merge in (("mma", 3, 1), ("combine", 0, 0), ("in_kernel", 0, 1), ("in_kernel_again", 0, 1)):
            ctx.set_variant(variant)
            ctx.set_option("decode_in_kernel_merge", merge)
            out = torch.full((n_head * 128,), float("nan"), dtype=torch.float16, device="cuda")
            ctx.dispatch_attention_decode(0, q, out, ctx_len)
            torch.cuda.synchronize()
            assert ctx.status() == 0
            outs[name] = host(out).astype(np.float32)
        assert np.array_equal(outs["in_kernel"], outs["in_kernel_again"])
        for name in ("combine", "in_kernel"):
            ok, max_abs, max_rel = within_tolerance(outs[name], outs["mma"])
            assert ok, (name, max_abs, max_rel)


def test_prefill_peer_exchange_of_two_shards_on_one_device():
    """Two KV-head shards (as two contexts on this device) run batched prefill with the peer exchange
    on: each 'rank' owns a gathered buffer [m][2 * q_dim], both kernels store their heads' outputs into
    both buffers, and both buffers must end up as the two local outputs side by side."""
    m, n_head, n_kv_head = 300, 16, 4
    q_dim = n_head * 128
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11)
    gathered = [torch.full((m, 2 * q_dim), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
    w = torch.ones(128, dtype=torch.float16, device="cuda")
    local = []
    ctxs = [bp.AttnContext(n_layer=1, n_head=n_head, n_kv_head=n_kv_head, max_seq=512, n_shards=2, shard=s)
            for s in range(2)]
    try:
        for s, ctx in enumerate(ctxs):
            q = torch.randn(m, q_dim, generator=gen, device="cuda").half()
            k = torch.randn(m, n_kv_head * 128, generator=gen, device="cuda").half()
            v = torch.randn(m, n_kv_head * 128, generator=gen, device="cuda").half()
            ctx.dispatch_q_norm_rope_fused(q, w, 0, m)
            ctx.dispatch_kv_writeback_fused(0, k, v, w, 0, m)
            ref = torch.zeros(m, q_dim, dtype=torch.float16, device="cuda")
            ctx.dispatch_attention(0, q, ref, m)  # exchange off: the plain result
            ctx.set_prefill_exchange([g.data_ptr() for g in gathered])
            out = torch.zeros(m, q_dim, dtype=torch.float16, device="cuda")
            ctx.dispatch_attention(0, q, out, m)
            torch.cuda.synchronize()
            assert ctx.status() == 0
            assert torch.equal(out, ref)
            local.append(out)
            ctx.set_variant(1)  # the CUDA-core kernel has no exchange: a configuration error, not a silent skip
            with pytest.raises(bp.errors.ConfigError):
                ctx.dispatch_attention(0, q, out, m)
            ctx.set_variant(0)
            ctx.set_prefill_exchange([])
        want = torch.cat(local, dim=1)
        for g in gathered:
            assert torch.equal(g, want)
    finally:
        for ctx in ctxs:
            ctx.close()
