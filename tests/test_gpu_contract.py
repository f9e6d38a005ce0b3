"""Semantics the reference's operator tests pin (tests/operators/test_grouped_quadratic.py:188-335,
:399-414 there), replayed on the CUDA operator in fp32 mode against the fp64 dense oracle."""

import pytest
import torch

import oal_b200
from oracle import oal_oracle as orc

pytestmark = pytest.mark.gpu
ERR = orc.normalized_max_error


def _case(batch=2, query_heads=4, key_heads=2, sequence=37, dimension=8, value_dimension=5):
    g = torch.Generator().manual_seed(20260802)
    return (torch.randn(batch, query_heads, sequence, dimension, generator=g),
            torch.randn(batch, key_heads, sequence, dimension, generator=g),
            torch.randn(batch, key_heads, sequence, value_dimension, generator=g))


def _factor():
    return torch.tensor((1.1, 0.5, 0.9, 0.4, 0.8, 0.7))


def _groups(query_heads=4, dimension=8):
    m = torch.ones((query_heads, dimension), dtype=torch.int32)
    m[:, : dimension // 2] = 0
    return m


def _oracle(q, k, v, groups, factor, kernel_eps=1e-6):
    a, b, c = orc.expand_factor(factor.double(), q.shape[1], kernel_eps)
    return orc.dense_forward(q.double(), k.double(), v.double(), groups, a, b, c, scale=q.shape[-1] ** -0.5)


@pytest.mark.parametrize("group_shape", ["shared", "per_head"])
@pytest.mark.parametrize("factor_shape", ["shared", "per_head"])
def test_group_and_factor_broadcast_combinations(group_shape, factor_shape):
    q, k, v = _case()
    groups = _groups()
    factor = _factor()
    pg = groups[0] if group_shape == "shared" else groups
    pf = factor if factor_shape == "shared" else factor.expand(q.shape[1], -1).clone()
    out = oal_b200.oal_attention(q.cuda(), k.cuda(), v.cuda(), pg.cuda(), pf.cuda())
    want, _, _ = _oracle(q, k, v, pg, pf)
    assert ERR(out, want) < 1e-5


def test_broadcast_factor_gradient_reduces_across_query_heads():
    q, k, v = (t.cuda() for t in _case(batch=1))
    groups = _groups().cuda()
    shared = _factor().cuda().requires_grad_()
    oal_b200.oal_attention(q, k, v, groups, shared).square().sum().backward()
    per_head = _factor().expand(q.shape[1], -1).clone().cuda().requires_grad_()
    oal_b200.oal_attention(q, k, v, groups, per_head).square().sum().backward()
    assert ERR(shared.grad, per_head.grad.sum(0)) < 1e-5


def test_inactive_padded_factor_entries_do_not_change_output_or_gradient():
    q, k, v = (t.cuda() for t in _case(query_heads=2, key_heads=1, dimension=4))
    groups = torch.tensor(((0, 0, 1, 1), (0, 0, 0, 0)), dtype=torch.int32).cuda()
    factor = _factor().expand(2, -1).clone().cuda().requires_grad_()
    out = oal_b200.oal_attention(q, k, v, groups, factor)
    out[:, 1].square().sum().backward()
    assert torch.count_nonzero(factor.grad[0]) == 0
    assert torch.count_nonzero(factor.grad[1, 3:]) == 0
    changed = factor.detach().clone()
    changed[1, 3:] += 100.0
    out2 = oal_b200.oal_attention(q, k, v, groups, changed)
    assert ERR(out2[:, 1], out[:, 1].detach()) < 1e-6


def test_output_dtype_only_changes_normalized_output():
    q, k, v = (t.cuda() for t in _case(query_heads=1, key_heads=1))
    groups = _groups(1).cuda()[0]
    o32, n32, d32 = oal_b200.oal_attention(q, k, v, groups, _factor().cuda(), return_unnormalized=True)
    o16, n16, d16 = oal_b200.oal_attention(q, k, v, groups, _factor().cuda(), return_unnormalized=True,
                                           output_dtype=torch.float16)
    assert o16.dtype == torch.float16 and n16.dtype == torch.float32 and d16.dtype == torch.float32
    assert torch.equal(n16, n32) and torch.equal(d16, d32)
    assert ERR(o16, o32) < 2e-3


def test_fp16_inputs_fp32_mode():
    q, k, v = _case(dimension=64, value_dimension=64, sequence=150)
    groups = _groups(4, 64)
    out = oal_b200.oal_attention(q.half().cuda(), k.half().cuda(), v.half().cuda(), groups.cuda(), _factor().cuda())
    want, _, _ = _oracle(q.half().float(), k.half().float(), v.half().float(), groups, _factor())
    assert out.dtype == torch.float16 and ERR(out, want) < 2e-3


def test_workspace_too_small_is_a_value_error():
    import ctypes

    from oal_b200 import _lib
    from oal_b200.hd_block_gemm import make_problem

    problem = make_problem((1, 2, 1, 256, 64, 64), groups=2, io_dtype=torch.bfloat16, out_dtype=torch.bfloat16,
                           precision="bf16_tensorcore", chunk=128, scale=0.125, floor=1e-38)
    dummy = torch.zeros(64, device="cuda")
    p = _lib.ptr(dummy)
    rc = _lib.load().oal_forward(ctypes.byref(problem), p, p, p, p, p, p, p, p, p, p, p, p, None, p, 16, p, None)
    with pytest.raises(ValueError, match="workspace too small"):
        _lib.check(rc)
