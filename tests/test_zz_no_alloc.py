"""The allocation-free decode entry point, bp_attn_decode_static_scratch.

It exists for hosts that may not allocate device memory at the point where they
run decode attention (their own arena owns the GPU, or they run inside a region
where allocation is forbidden), so its split-KV scratch is a fixed array in the
library image. The test calls it through the C ABI twice in a row, with
different key counts so that the second call finds the first call's leftovers in
the shared scratch, and checks each result against the context-based
bp_attn_decode on the same cache, within the tolerance the other attention tests
use. A second test walks the split-count edges (a single split, which writes
the output directly; the step to two splits; the cap of 32 splits beyond 8192
keys) and a model with 8 query heads per KV head and 64 query heads, the
largest the fixed scratch holds. Both check the size limits. This file sorts
last on purpose."""
import numpy as np
import pytest

import bonsai_pot_b200 as bp
from bonsai_pot_b200 import _lib
from oracle import oracle as O
from tests.helpers import build_decode_case, within_tolerance

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def test_static_scratch_decode_matches_context_decode_twice_in_a_row():
    lib = _lib.load()
    sh = O.Shape(n_layer=2, max_seq=4096)
    layer = 1
    case = build_decode_case(sh, seed=21, cfg_id=1, layer=layer, n_past=4000)
    with bp.AttnContext(n_layer=2, max_seq=4096) as ctx:
        for kind, kv in enumerate((case["kv_k"], case["kv_v"])):
            ctx.kv_import(kind, layer, 0, 4001, np.ascontiguousarray(sh.d_section(kv, layer)[:4001]))
            ctx.kv_import(kind, layer, 1, 4001, np.ascontiguousarray(sh.qs_section(kv, layer)[:4001]))
        q = torch.from_numpy(np.ascontiguousarray(case["qn"])).cuda()
        stream = torch.cuda.current_stream().cuda_stream
        for cur_pos in (4001, 300):  # many splits first, then few: stale partials stay in the scratch
            ref = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
            got = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
            ctx.dispatch_attention_decode(layer, q, ref, cur_pos)
            st = lib.bp_attn_decode_static_scratch(stream, q.data_ptr(), ctx.kv_device_ptr(0), ctx.kv_device_ptr(1),
                                                   got.data_ptr(), sh.n_layer, sh.max_seq, sh.n_head, sh.n_kv_head,
                                                   layer, cur_pos)
            assert st == 0
            torch.cuda.synchronize()
            ok, max_abs, max_rel = within_tolerance(got.cpu().numpy(), ref.cpu().numpy().astype(np.float32))
            assert ok, (cur_pos, max_abs, max_rel)
            exact = O.attn_exact(sh, case["qn"], case["kv_k"], case["kv_v"], layer, 1, cur_pos - 1)[0]
            assert within_tolerance(got.cpu().numpy(), exact)[0]
        # sizes beyond the fixed scratch are refused, not truncated
        assert lib.bp_attn_decode_static_scratch(stream, q.data_ptr(), ctx.kv_device_ptr(0), ctx.kv_device_ptr(1),
                                                 got.data_ptr(), 2, 4096, 128, 8, 0, 10) == 1
        assert lib.bp_attn_decode_static_scratch(stream, q.data_ptr(), ctx.kv_device_ptr(0), ctx.kv_device_ptr(1),
                                                 got.data_ptr(), 2, 4096, 32, 8, 0, 4097) == 2
        assert lib.bp_attn_decode_static_scratch(stream, None, None, None, None, 2, 4096, 32, 8, 0, 1) == 7


def test_static_scratch_split_edges_and_other_head_ratio():
    """cur_pos 1, 256 (one split: no scratch at all), 257 (two), 8193 and 12000 (the 32-split cap:
    splits grow instead) on 64 query heads over 8 KV heads, against bp_attn_decode and the exact softmax."""
    lib = _lib.load()
    sh = O.Shape(n_layer=1, n_head=64, n_kv_head=8, max_seq=12288)
    case = build_decode_case(sh, seed=3, cfg_id=1, layer=0, n_past=11999)
    with bp.AttnContext(n_layer=1, n_head=64, n_kv_head=8, max_seq=12288) as ctx:
        for kind, kv in enumerate((case["kv_k"], case["kv_v"])):
            ctx.kv_import(kind, 0, 0, 12000, np.ascontiguousarray(sh.d_section(kv, 0)[:12000]))
            ctx.kv_import(kind, 0, 1, 12000, np.ascontiguousarray(sh.qs_section(kv, 0)[:12000]))
        q = torch.from_numpy(np.ascontiguousarray(case["qn"])).cuda()
        stream = torch.cuda.current_stream().cuda_stream
        for cur_pos in (12000, 1, 8193, 256, 257):
            ref = torch.zeros(sh.q_dim, dtype=torch.float16, device="cuda")
            got = torch.full((sh.q_dim,), float("nan"), dtype=torch.float16, device="cuda")
            ctx.dispatch_attention_decode(0, q, ref, cur_pos)
            st = lib.bp_attn_decode_static_scratch(stream, q.data_ptr(), ctx.kv_device_ptr(0), ctx.kv_device_ptr(1),
                                                   got.data_ptr(), 1, 12288, 64, 8, 0, cur_pos)
            assert st == 0
            torch.cuda.synchronize()
            ok, max_abs, max_rel = within_tolerance(got.cpu().numpy(), ref.cpu().numpy().astype(np.float32))
            assert ok, (cur_pos, max_abs, max_rel)
            exact = O.attn_exact(sh, case["qn"], case["kv_k"], case["kv_v"], 0, 1, cur_pos - 1)[0]
            assert within_tolerance(got.cpu().numpy(), exact)[0], cur_pos
        # one head more than the scratch holds
        assert lib.bp_attn_decode_static_scratch(stream, q.data_ptr(), ctx.kv_device_ptr(0), ctx.kv_device_ptr(1),
                                                 got.data_ptr(), 1, 12288, 72, 8, 0, 10) == 1
