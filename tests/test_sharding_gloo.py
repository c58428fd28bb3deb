"""world_size-2 (and 4) gloo tests of the KV-head sharding logic on CPU: every
rank computes its heads with the CPU oracle standing in for the kernels, the
head outputs are all-gathered, and the result must equal the unsharded oracle;
the per-rank snapshot columns must assemble the reference's global blob."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bonsai_pot_b200.sharding import HeadShard, all_gather_heads
from oracle import oracle as O
from tests.helpers import build_decode_case


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_past, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = O.Shape(n_layer=1, max_seq=256)
        case = build_decode_case(full, seed=3, cfg_id=3, layer=0, n_past=n_past)
        shard = HeadShard(rank, world, full.n_head, full.n_kv_head)
        part = O.Shape(n_layer=1, n_head=shard.n_head_local, n_kv_head=shard.n_kv_local, max_seq=256)
        # this rank's slice of the cache and of q, in the narrower row layout of a shard context
        kv = []
        for src in (case["kv_k"], case["kv_v"]):
            dst = part.new_cache()
            part.d_section(dst, 0)[:] = full.d_section(src, 0)[:, shard.scale_cols]
            part.qs_section(dst, 0)[:] = full.qs_section(src, 0)[:, shard.kv_cols]
            kv.append(dst)
        q_local = np.ascontiguousarray(case["qn"][:, shard.q_cols])
        out_local = O.attn_decode(part, q_local, kv[0], kv[1], 0, n_past + 1)
        gathered = all_gather_heads(torch.from_numpy(out_local.copy()), shard)
        ref = O.attn_decode(full, case["qn"], case["kv_k"], case["kv_v"], 0, n_past + 1)
        assert np.array_equal(gathered.numpy().view(np.uint16), ref.view(np.uint16)), "gathered heads differ"
        # a 2-row "prefill" result gathers row by row
        two = torch.from_numpy(np.stack([out_local, out_local]))
        g2 = all_gather_heads(two, shard)
        assert g2.shape == (2, full.q_dim) and np.array_equal(g2[1].numpy().view(np.uint16), ref.view(np.uint16))
        # snapshot columns: every rank fills its columns of the global payload
        pos = n_past + 1
        blob = np.zeros(O.payload_bytes(1, full.kv_dim, pos), dtype=np.uint8)
        for kind in range(2):
            d_off = O.payload_offset(1, full.kv_dim, pos, kind, 0, 0)
            q_off = O.payload_offset(1, full.kv_dim, pos, kind, 0, 1)
            d_view = blob[d_off:d_off + pos * full.nb * 4].view(np.float32).reshape(pos, full.nb)
            q_view = blob[q_off:q_off + pos * full.kv_dim].view(np.int8).reshape(pos, full.kv_dim)
            d_view[:, shard.scale_cols] = part.d_section(kv[kind], 0)[:pos]
            q_view[:, shard.kv_cols] = part.qs_section(kv[kind], 0)[:pos]
        t = torch.from_numpy(blob)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)  # disjoint columns: the sum assembles the blob
        assert bytes(t.numpy()) == O.snapshot_blob(full, case["kv_k"], case["kv_v"], pos)[32:]
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_head_sharding_all_gather_equals_unsharded(world, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 100, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_head_shard_geometry():
    s = HeadShard(3, 4, 32, 8)
    assert (s.n_head_local, s.n_kv_local) == (8, 2)
    assert s.q_cols == slice(3072, 4096) and s.kv_cols == slice(768, 1024) and s.scale_cols == slice(24, 32)
    assert s.context_kwargs() == dict(n_head=8, n_kv_head=2, n_shards=4, shard=3)
    assert HeadShard(0, 1, 32, 8).q_cols == slice(0, 4096)
    with pytest.raises(ValueError):
        HeadShard(0, 3, 32, 8)
    with pytest.raises(ValueError):
        HeadShard(2, 2, 32, 8)
