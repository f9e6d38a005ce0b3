"""Fixed-size sharding of one call over ranks by (batch row, KV head) unit.

Batch rows and KV heads are independent in this operator (a query head only reads its own KV head),
so a ``[B, Hq, N, D]`` call splits into ``B * Hkv`` units with no data-path communication: the batch is
split first, then, when there are more ranks than batch rows, the KV heads of a batch row.  What remains
for the caller is the sum of the coefficient gradients over the ranks that share a query head (one small
all-reduce, as for any data-parallel parameter gradient); ranks that hold different KV heads own
different rows of ``factor`` and need no exchange for them.  The reference is single-GPU
(oal_attention/hd_block_gemm_adapters.py:347-415 takes the whole batch); this is the split the
batch x KV-head partition of the work implies.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class UnitShard:
    """The part of a ``[B, Hq, N, D]`` / ``[B, Hkv, N, D]`` problem one rank owns."""

    batch: slice
    kv_heads: slice
    q_heads: slice
    units: int            # (batch row, KV head) units of this rank

    def take(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *more_q: torch.Tensor):
        """Contiguous shards of q, k, v (and of any further tensors laid out like q, e.g. the upstream gradient)."""
        cut_q = lambda t: t[self.batch, self.q_heads].contiguous()
        cut_kv = lambda t: t[self.batch, self.kv_heads].contiguous()
        return (cut_q(q), cut_kv(k), cut_kv(v), *(cut_q(t) for t in more_q))

    def factor_rows(self, factor: torch.Tensor) -> torch.Tensor:
        """Rows of a per-head ``factor [Hq, P]`` (a shared ``[P]`` factor is returned as it is)."""
        return factor if factor.ndim == 1 else factor[self.q_heads].contiguous()

    def group_rows(self, dim_groups: torch.Tensor) -> torch.Tensor:
        return dim_groups if dim_groups.ndim == 1 else dim_groups[self.q_heads].contiguous()


def unit_shard(batch: int, q_heads: int, kv_heads: int, rank: int, world: int) -> UnitShard:
    """Shard ``rank`` of ``world``.  ``world`` must divide ``batch``, or be a multiple of it with
    ``world / batch`` dividing ``kv_heads``."""
    if not 0 <= rank < world:
        raise ValueError("rank must lie in [0, world)")
    if q_heads % kv_heads:
        raise ValueError("query heads must be divisible by key/value heads")
    rep = q_heads // kv_heads
    if batch % world == 0:
        per = batch // world
        return UnitShard(slice(rank * per, (rank + 1) * per), slice(0, kv_heads), slice(0, q_heads), per * kv_heads)
    if world % batch == 0 and kv_heads % (world // batch) == 0:
        parts = world // batch
        per = kv_heads // parts
        b, part = divmod(rank, parts)
        return UnitShard(slice(b, b + 1), slice(part * per, (part + 1) * per),
                         slice(part * per * rep, (part + 1) * per * rep), per)
    raise ValueError(f"{batch} batch rows x {kv_heads} KV heads do not split evenly over {world} ranks")
