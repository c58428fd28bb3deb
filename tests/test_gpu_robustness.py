"""GPU tests of the failure-detection and launch-ordering behaviour of the C ABI.

No test here faults, traps or hangs a GPU: the only failure they provoke is a
bounded device-side wait that runs out (a counter nobody increments), after
which the kernel returns and the host reads a status. Mirrors the device-lost
tests of the reference (tests/gpu_integration.rs:268-336) for the one failure
the CUDA path adds, a timed-out wait."""
import numpy as np
import pytest

import bonsai_pot_b200 as bp
from bonsai_pot_b200 import _lib
from oracle import oracle as O
from tests.helpers import build_decode_case, within_tolerance

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def make_ctx(sh, **kw):
    return bp.AttnContext(n_layer=sh.n_layer, n_head=sh.n_head, n_kv_head=sh.n_kv_head, max_seq=sh.max_seq,
                          rms_eps=sh.rms_eps, rope_freq_base=sh.rope_freq_base, **kw)


def load_cache(ctx, sh, kv_k, kv_v, layer, rows, cols=None, bcols=None):
    for kind, kv in enumerate((kv_k, kv_v)):
        d = sh.d_section(kv, layer)[:rows]
        q = sh.qs_section(kv, layer)[:rows]
        if cols is not None:
            d, q = d[:, bcols], q[:, cols]
        ctx.kv_import(kind, layer, 0, rows, np.ascontiguousarray(d))
        ctx.kv_import(kind, layer, 1, rows, np.ascontiguousarray(q))


def test_meeting_that_never_completes_times_out_and_latches():
    """A two-rank exchange in which the second rank never signals: the bounded wait of bp_peer_sync
    runs out, the kernel returns, the context reports BP_ERR_TIMEOUT from then on, every compute call
    fails fast, the cache can still be captured, and a fresh context restored from that snapshot
    continues with identical results."""
    full = O.Shape(n_layer=2, max_seq=256)
    n_past = 200
    case = build_decode_case(full, seed=9, cfg_id=0, layer=1, n_past=n_past)
    sh = O.Shape(n_layer=2, n_head=16, n_kv_head=4, max_seq=256)  # shard 0 of 2
    cols, bcols, qcols = slice(0, sh.kv_dim), slice(0, sh.nb), slice(0, sh.q_dim)
    ctx = make_ctx(sh, n_shards=2, shard=0)
    try:
        for layer in range(2):
            load_cache(ctx, full, case["kv_k"], case["kv_v"], layer, n_past + 1, cols, bcols)
        q = dev(case["qn"][:, qcols])
        before = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
        ctx.dispatch_attention_decode(1, q, before, n_past + 1)
        torch.cuda.synchronize()
        snap_before = bp.KvSnapshot.capture(ctx, n_past + 1).to_bytes()
        # both ranks' buffers live on this device; rank 1 does not exist, so its signal never comes
        gathered = [torch.zeros(sh.n_layer, 2 * sh.q_dim, dtype=torch.float16, device="cuda") for _ in range(2)]
        flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
        ctx.set_peer_exchange([g.data_ptr() for g in gathered], [f.data_ptr() for f in flags])
        ctx.set_option("wait_limit", 20000)  # about a millisecond of polling
        out = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
        ctx.dispatch_attention_decode(1, q, out, n_past + 1)
        ctx.peer_sync(slot=3)
        torch.cuda.synchronize()  # returns: the wait is bounded
        assert torch.equal(out, before)  # the decode itself was fine
        assert flags[0][3].item() == 1 and flags[1][3].item() == 1  # this rank signalled both
        assert ctx.status() == bp.errors.BP_ERR_TIMEOUT
        for call in (lambda: ctx.dispatch_attention_decode(1, q, out, n_past + 1),
                     lambda: ctx.dispatch_q_norm_rope_fused(out, out, 0, 1),
                     lambda: ctx.peer_sync(slot=3),
                     lambda: ctx.dispatch_attention(0, q, out, 1)):
            with pytest.raises(bp.DeviceTimeout):
                call()
        # the cache is intact and can be taken along
        snap = bp.KvSnapshot.capture(ctx, n_past + 1)
        assert snap.to_bytes() == snap_before
    finally:
        ctx.close()
    fresh = make_ctx(sh, n_shards=2, shard=0)
    try:
        assert fresh.status() == 0
        assert bp.KvSnapshot.from_bytes(snap_before).apply(fresh) == n_past + 1
        again = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
        fresh.dispatch_attention_decode(1, q, again, n_past + 1)
        torch.cuda.synchronize()
        assert fresh.status() == 0
        assert torch.equal(again, before)
    finally:
        fresh.close()


def test_in_kernel_meeting_that_never_completes_times_out():
    """The same with the meeting inside the decode kernel (option peer_meet_in_kernel): layer 1's kernel
    signals layer 0's slot to both ranks and waits for both; the absent second rank never signals."""
    sh = O.Shape(n_layer=2, n_head=16, n_kv_head=4, max_seq=512)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    with make_ctx(sh, n_shards=2, shard=0) as ctx:
        w = torch.ones(128, dtype=torch.float16, device="cuda")
        for layer in range(2):
            k = torch.randn(400, sh.kv_dim, generator=gen, device="cuda").half()
            v = torch.randn(400, sh.kv_dim, generator=gen, device="cuda").half()
            ctx.dispatch_kv_writeback_fused(layer, k, v, w, 0, 400)
        q = torch.randn(sh.q_dim, generator=gen, device="cuda").half()
        gathered = [torch.zeros(sh.n_layer, 2 * sh.q_dim, dtype=torch.float16, device="cuda") for _ in range(2)]
        flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
        ctx.set_peer_exchange([g.data_ptr() for g in gathered], [f.data_ptr() for f in flags])
        ctx.set_option("peer_meet_in_kernel", 1)
        ctx.set_option("wait_limit", 20000)
        out = torch.zeros(2, sh.q_dim, dtype=torch.float16, device="cuda")
        ctx.dispatch_attention_decode(0, q, out[0], 400)
        torch.cuda.synchronize()
        assert ctx.status() == 0 and flags[0][0].item() == 0  # layer 0 holds no meeting
        ctx.dispatch_attention_decode(1, q, out[1], 400)
        torch.cuda.synchronize()
        assert flags[0][0].item() == 1 and flags[1][0].item() == 1 and flags[0][1].item() == 0
        assert torch.equal(gathered[0][:, :sh.q_dim], out)  # the outputs themselves arrived
        assert ctx.status() == bp.errors.BP_ERR_TIMEOUT
        with pytest.raises(bp.DeviceTimeout):
            ctx.dispatch_attention_decode(0, q, out[0], 400)


def test_meeting_held_by_the_decode_kernel_itself():
    """One rank acting as its own peer (kernels that wait for one another cannot run as separate
    launches on one GPU, so a second rank's kernels are left to the multi-GPU benchmark): every decode
    launch of layer L >= 1 signals layer L - 1's slot and waits for it, bp_peer_sync meets the last
    layer, token after token; outputs land in the gathered buffer and every slot counts one meeting
    per token."""
    n_layer, ctx_len = 3, 3000
    sh = O.Shape(n_layer=n_layer, max_seq=ctx_len)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(23)
    w = torch.ones(128, dtype=torch.float16, device="cuda")
    with make_ctx(sh) as ctx:
        for layer in range(n_layer):
            k = torch.randn(ctx_len, sh.kv_dim, generator=gen, device="cuda").half()
            v = torch.randn(ctx_len, sh.kv_dim, generator=gen, device="cuda").half()
            ctx.dispatch_kv_writeback_fused(layer, k, v, w, 0, ctx_len)
        q = torch.randn(n_layer, sh.q_dim, generator=gen, device="cuda").half()
        plain = torch.zeros(n_layer, sh.q_dim, dtype=torch.float16, device="cuda")
        for layer in range(n_layer):
            ctx.dispatch_attention_decode(layer, q[layer], plain[layer], ctx_len)
        gathered = torch.zeros(n_layer, sh.q_dim, dtype=torch.float16, device="cuda")
        flags = torch.zeros(64, dtype=torch.int32, device="cuda")
        ctx.set_peer_exchange([gathered.data_ptr()], [flags.data_ptr()])
        ctx.set_option("peer_meet_in_kernel", 1)
        for token in range(3):
            gathered.zero_()
            out = torch.zeros(n_layer, sh.q_dim, dtype=torch.float16, device="cuda")
            for layer in range(n_layer):
                ctx.dispatch_attention_decode(layer, q[layer], out[layer], ctx_len)
            ctx.peer_sync(slot=n_layer - 1)
            torch.cuda.synchronize()
            assert ctx.status() == 0
            assert torch.equal(out, plain) and torch.equal(gathered, plain)
            assert flags[:n_layer].tolist() == [token + 1] * n_layer


def test_decode_is_correct_while_other_work_holds_sms():
    """With "exclusive_device" = 0 the decode call must not depend on all of its CTAs being resident:
    a filler kernel on another stream holds 40 SMs for 20 ms while a 32K-context
    decode (one CTA per SM on an idle device) runs, and the result is still the oracle's, status 0."""
    ctx_len, layer = 32768, 0
    sh = O.Shape(n_layer=1, max_seq=ctx_len)
    case = build_decode_case(sh, seed=0, cfg_id=3, layer=layer, n_past=ctx_len - 1)
    exact = O.attn_exact(sh, case["qn"], case["kv_k"], case["kv_v"], layer, 1, ctx_len - 1)[0]
    with make_ctx(sh) as ctx:
        load_cache(ctx, sh, case["kv_k"], case["kv_v"], layer, ctx_len)
        ctx.set_option("exclusive_device", 0)
        q = dev(case["qn"])
        out = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
        filler, work = torch.cuda.Stream(), torch.cuda.Stream()
        torch.cuda.synchronize()
        # 40 SMs are taken for 20 ms: the decode grid (one CTA per SM of an idle device) cannot be resident at once
        assert _lib.load().bp_debug_hold_sms(filler.cuda_stream, 40, 20000) == 0
        with torch.cuda.stream(work):
            for _ in range(3):
                ctx.dispatch_attention_decode(layer, q, out, ctx_len, stream=work)
        work.synchronize()
        assert ctx.last_launch_count() == 2  # split pass + separate merge kernel
        assert ctx.status() == 0
        torch.cuda.synchronize()
        ok, max_abs, max_rel = within_tolerance(host(out), exact)
        assert ok, (max_abs, max_rel)
        # and the peer exchange, which lives in the in-kernel merge, refuses this mode
        ctx.set_option("exclusive_device", 1)
        g = torch.zeros(1, sh.q_dim, dtype=torch.float16, device="cuda")
        f = torch.zeros(64, dtype=torch.int32, device="cuda")
        ctx.set_peer_exchange([g.data_ptr()], [f.data_ptr()])
        with pytest.raises(bp.ConfigError):
            ctx.set_option("exclusive_device", 0)


def test_peer_exchange_refuses_kernel_families_without_it():
    """With a peer exchange set, the decode entry points must not silently skip the peer stores when
    another kernel family is selected: a configuration error, as batched prefill gives."""
    sh = O.Shape(n_layer=1, max_seq=256)
    with make_ctx(sh) as ctx:
        g = torch.zeros(1, sh.q_dim, dtype=torch.float16, device="cuda")
        f = torch.zeros(64, dtype=torch.int32, device="cuda")
        buf = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
        kvb = torch.zeros(sh.kv_dim, dtype=torch.float16, device="cuda")
        w = torch.ones(128, dtype=torch.float16, device="cuda")
        ctx.set_peer_exchange([g.data_ptr()], [f.data_ptr()])
        for variant in (1, 2, 3):
            ctx.set_variant(variant)
            with pytest.raises(bp.ConfigError):
                ctx.dispatch_attention_decode(0, buf, buf, 1)
            with pytest.raises(bp.ConfigError):
                ctx.decode_layer(0, buf, w, kvb, kvb, w, 0, buf)
        ctx.set_variant(0)
        ctx.decode_layer(0, buf, w, kvb, kvb, w, 0, buf)
        torch.cuda.synchronize()
        assert ctx.status() == 0


@pytest.mark.parametrize("n_layer", [1, 2])
def test_fused_tokens_in_one_graph_on_a_shallow_stack(n_layer):
    """Dependent launches let a decode kernel request cache rows before its predecessors have
    finished. On a one- or two-layer context the launch that wrote the newest rows is that close:
    several fused tokens captured in ONE CUDA graph must give exactly what plain launches give
    (outputs and cache bytes), i.e. no kernel may read a row before it is written."""
    sh = O.Shape(n_layer=n_layer, max_seq=2048)
    n_tok, pos0 = 24, 300
    gen = torch.Generator(device="cuda")
    gen.manual_seed(77)
    w = torch.ones(128, dtype=torch.float16, device="cuda")
    k0 = torch.randn(n_layer, pos0, sh.kv_dim, generator=gen, device="cuda").half()
    v0 = torch.randn(n_layer, pos0, sh.kv_dim, generator=gen, device="cuda").half()
    q = torch.randn(n_tok, n_layer, sh.q_dim, generator=gen, device="cuda").half()
    # keys that dominate the softmax, so that a missed newest row changes the output visibly
    k = (torch.randn(n_tok, n_layer, sh.kv_dim, generator=gen, device="cuda") * 4).half()
    v = torch.randn(n_tok, n_layer, sh.kv_dim, generator=gen, device="cuda").half()
    results = {}
    for mode in ("plain", "graph"):
        with make_ctx(sh) as ctx:
            ctx.set_option("dependent_launch", 1 if mode == "graph" else 0)
            for layer in range(n_layer):
                ctx.dispatch_kv_writeback_fused(layer, k0[layer], v0[layer], w, 0, pos0)
            out = torch.zeros(n_tok, n_layer, sh.q_dim, dtype=torch.float16, device="cuda")
            stream = torch.cuda.Stream()

            def tokens():
                for t in range(n_tok):
                    for layer in range(n_layer):
                        ctx.decode_layer(layer, q[t, layer], w, k[t, layer], v[t, layer], w, pos0 + t, out[t, layer],
                                         stream=stream)

            torch.cuda.synchronize()
            with torch.cuda.stream(stream):
                if mode == "graph":
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        tokens()
                    for _ in range(3):  # replays overwrite the same rows with the same bytes
                        g.replay()
                else:
                    tokens()
            torch.cuda.synchronize()
            assert ctx.status() == 0
            rows = pos0 + n_tok
            cache = []
            for layer in range(n_layer):
                for kind in range(2):
                    d = np.empty((rows, sh.nb), dtype=np.float32)
                    qs_ = np.empty((rows, sh.kv_dim), dtype=np.int8)
                    ctx.kv_export(kind, layer, 0, rows, d)
                    ctx.kv_export(kind, layer, 1, rows, qs_)
                    cache.append((d.copy(), qs_.copy()))
            results[mode] = (host(out).copy(), cache)
    assert np.array_equal(results["plain"][0].view(np.uint16), results["graph"][0].view(np.uint16))
    for (d0, q0), (d1, q1) in zip(results["plain"][1], results["graph"][1]):
        assert np.array_equal(d0.view(np.uint32), d1.view(np.uint32)) and np.array_equal(q0, q1)
