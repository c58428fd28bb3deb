"""KV-head sharding of the attention path over the ranks of one node.

All five kernels are independent per KV-head group (a KV head and the query
heads that share it), so rank r of N owns KV heads [r*n_kv/N, (r+1)*n_kv/N) and
the matching query heads, holds only its slice of the cache, and the one
exchange step is an all-gather of the f16 head outputs (NCCL over NVLink on
GPUs, gloo in the CPU tests). The reference has no multi-GPU path; this is the
partition `bp_attn_config.n_shards / shard` describes.
"""
from __future__ import annotations

from dataclasses import dataclass

HEAD_DIM = 128


@dataclass(frozen=True)
class HeadShard:
    """Column ranges of one rank inside the global [.., n_head*128] / [.., n_kv_head*128] rows."""
    rank: int
    world: int
    n_head: int       # global query heads
    n_kv_head: int    # global KV heads

    def __post_init__(self):
        if self.world < 1 or not (0 <= self.rank < self.world):
            raise ValueError("rank must be in [0, world)")
        if self.n_kv_head % self.world != 0:
            raise ValueError("the KV heads must divide evenly over the ranks")
        if self.n_head % self.n_kv_head != 0:
            raise ValueError("n_head must be a multiple of n_kv_head")

    @property
    def n_kv_local(self):
        return self.n_kv_head // self.world

    @property
    def n_head_local(self):
        return self.n_head // self.world

    @property
    def q_cols(self):
        w = self.n_head_local * HEAD_DIM
        return slice(self.rank * w, (self.rank + 1) * w)

    @property
    def kv_cols(self):
        w = self.n_kv_local * HEAD_DIM
        return slice(self.rank * w, (self.rank + 1) * w)

    @property
    def scale_cols(self):
        w = self.n_kv_local * HEAD_DIM // 32
        return slice(self.rank * w, (self.rank + 1) * w)

    def context_kwargs(self):
        """Keyword arguments for AttnContext of this rank's shard."""
        return dict(n_head=self.n_head_local, n_kv_head=self.n_kv_local, n_shards=self.world, shard=self.rank)


def all_gather_heads(out_local, shard: HeadShard, out_full=None, group=None):
    """All-gather the per-rank head outputs [..., n_head_local*128] into [..., n_head*128].

    Rows are gathered rank-major per row, i.e. the result has the reference's
    head order. With world == 1 the input is returned."""
    import torch
    import torch.distributed as dist
    if shard.world == 1:
        return out_local
    lead = out_local.shape[:-1]
    w = out_local.shape[-1]
    flat = out_local.reshape(-1, w).contiguous()
    gathered = torch.empty((shard.world * flat.shape[0], w), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(gathered, flat, group=group)  # rank-major concatenation along dim 0
    full = gathered.view(shard.world, flat.shape[0], w).permute(1, 0, 2).reshape(*lead, shard.world * w)
    if out_full is not None:
        out_full.copy_(full)
        return out_full
    return full.contiguous()
