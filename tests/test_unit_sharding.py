"""Fixed-size (batch row, KV head) sharding: index logic on the CPU, and a world-size-2 gloo run in which
the ranks' shards reassemble the whole call (the oracle stands in for the kernels: the helper only cuts)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oal_b200.unit_sharding import unit_shard


@pytest.mark.parametrize("batch,hq,hkv,world", [(4, 14, 2, 1), (4, 14, 2, 2), (4, 14, 2, 4), (4, 14, 2, 8), (2, 8, 4, 8),
                                                (6, 4, 2, 3)])
def test_shards_cover_every_unit_exactly_once(batch, hq, hkv, world):
    rep = hq // hkv
    seen = torch.zeros(batch, hkv, dtype=torch.int32)
    for rank in range(world):
        s = unit_shard(batch, hq, hkv, rank, world)
        seen[s.batch, s.kv_heads] += 1
        assert s.q_heads.start == s.kv_heads.start * rep and s.q_heads.stop == s.kv_heads.stop * rep
        assert s.units == (s.batch.stop - s.batch.start) * (s.kv_heads.stop - s.kv_heads.start)
    assert torch.all(seen == 1)


def test_uneven_splits_are_refused():
    with pytest.raises(ValueError):
        unit_shard(4, 14, 2, 0, 3)
    with pytest.raises(ValueError):
        unit_shard(4, 14, 2, 0, 16)
    with pytest.raises(ValueError):
        unit_shard(4, 14, 2, 8, 8)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    from oal_b200 import synthetic
    from oracle import oal_oracle as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    case = synthetic.qwen_head_case(3, batch=1, n=48, hq=4, hkv=2, g=4, bf16=False)
    shard = unit_shard(1, 4, 2, rank, world)
    q, k, v, dout = shard.take(case.q, case.k, case.v, case.grad_out)
    factor = shard.factor_rows(case.factor)
    a, b, c = orc.expand_factor(factor, q.shape[1], case.kernel_eps)
    r = orc.dense_backward(q.double(), k.double(), v.double(), shard.group_rows(case.dim_groups), a, b, c,
                           scale=case.scale, grad_out=dout.double())
    gathered = [None] * world
    dist.all_gather_object(gathered, {key: r[key] for key in ("out", "dq", "dk", "dv", "dA")})
    if rank == 0:
        torch.save(gathered, os.path.join(out_dir, "shards.pt"))
    dist.destroy_process_group()


def test_two_gloo_ranks_reassemble_the_whole_call(tmp_path):
    from oal_b200 import synthetic
    from oracle import oal_oracle as orc

    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    parts = torch.load(tmp_path / "shards.pt")
    case = synthetic.qwen_head_case(3, batch=1, n=48, hq=4, hkv=2, g=4, bf16=False)
    a, b, c = orc.expand_factor(case.factor, 4, case.kernel_eps)
    whole = orc.dense_backward(case.q.double(), case.k.double(), case.v.double(), case.dim_groups, a, b, c,
                               scale=case.scale, grad_out=case.grad_out.double())
    for key in ("out", "dq", "dk", "dv"):
        assert torch.allclose(torch.cat([p[key] for p in parts], dim=1), whole[key], rtol=1e-12, atol=1e-12), key
    assert torch.allclose(torch.cat([p["dA"] for p in parts]), whole["dA"], rtol=1e-12, atol=1e-12)


def test_single_unit_shards_pass_the_plan_layout_check():
    """One (batch row, KV head) unit per rank: the shard has two dimensions of size 1, whose strides are
    whatever the slice left them (`.contiguous()` returns such a tensor unchanged); the plan must take it."""
    from oal_b200.hd_block_gemm import build_hd_block_gemm_plan

    q = torch.randn(4, 14, 256, 64)
    k = torch.randn(4, 2, 256, 64)
    v = torch.randn(4, 2, 256, 64)
    shard = unit_shard(4, 14, 2, rank=5, world=8)
    qs, ks, vs = shard.take(q, k, v)
    assert ks.shape == (1, 1, 256, 64) and ks.is_contiguous()
    plan = build_hd_block_gemm_plan(qs, ks, vs, requested_gradient_mask=(False,) * 6)
    assert plan.geometry[:3] == (1, 7, 1)
    bad = q.transpose(2, 3).contiguous().transpose(2, 3)[:1, :7]
    with pytest.raises(ValueError, match="row-major"):
        build_hd_block_gemm_plan(bad, ks, vs, requested_gradient_mask=(False,) * 6)
