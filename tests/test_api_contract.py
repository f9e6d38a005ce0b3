"""Call-surface contract of the public entry points, replaying the reference's own operator tests
where they do not need the arithmetic (tests/operators/test_grouped_quadratic.py:338-396 there):
same exception types for the same invalid inputs, validated before any device work."""

import math

import pytest
import torch

import oal_b200
from oal_b200.hd_block_gemm import PLAN_OPTION_FIELDS, build_hd_block_gemm_plan


def _case(batch=2, query_heads=4, key_heads=2, sequence=3, dimension=4, value_dimension=3, dtype=torch.float32):
    g = torch.Generator().manual_seed(20260802)
    return (torch.randn(batch, query_heads, sequence, dimension, generator=g, dtype=dtype),
            torch.randn(batch, key_heads, sequence, dimension, generator=g, dtype=dtype),
            torch.randn(batch, key_heads, sequence, value_dimension, generator=g, dtype=dtype))


def _factor(dtype=torch.float32):
    return torch.tensor((1.1, 0.5, 0.9, 0.4, 0.8, 0.7), dtype=dtype)


def _groups(query_heads=4, dimension=4):
    m = torch.ones((query_heads, dimension), dtype=torch.int32)
    m[:, :2] = 0
    return m


@pytest.mark.parametrize("bad_groups", [
    torch.tensor((0.0, 0.0, 1.0, 1.0)),
    torch.tensor((-1, 0, 1, 1), dtype=torch.int64),
    torch.tensor((0, 2, 2, 2), dtype=torch.int64),
    torch.tensor((1, 1, 2, 2), dtype=torch.int64),
    torch.tensor((0, 0, 2, 2), dtype=torch.int64),
    torch.tensor((0, 0, 2**32, 2**32), dtype=torch.int64),
])
def test_invalid_dim_groups_are_rejected(bad_groups):
    q, k, v = _case(query_heads=1, key_heads=1)
    with pytest.raises((TypeError, ValueError), match="dim_groups|group"):
        oal_b200.oal_attention(q, k, v, bad_groups, _factor())


def test_invalid_shapes_and_factor_lengths_are_rejected():
    q, k, v = _case()
    groups = _groups()
    with pytest.raises(ValueError, match="query-head"):
        oal_b200.oal_attention(q, k, v, groups[:2], _factor())
    with pytest.raises(ValueError, match="triangular|factor"):
        oal_b200.oal_attention(q, k, v, groups, torch.ones(5))
    with pytest.raises(ValueError, match="factor"):
        oal_b200.oal_attention(q, k, v, groups, torch.ones(2, 6))
    with pytest.raises(TypeError, match="floating"):
        oal_b200.oal_attention(q, k, v, groups, torch.ones(6, dtype=torch.int64))
    with pytest.raises(ValueError, match="divisible"):
        oal_b200.oal_attention(q[:, :3], k, v, groups[:3], _factor())
    with pytest.raises(ValueError, match="same dtype"):
        oal_b200.oal_attention(q.half(), k, v, groups, _factor())


@pytest.mark.parametrize("kernel_eps", [0.0, -1.0, math.inf, 1e-50, True, "1e-6"])
def test_invalid_kernel_epsilon_is_rejected(kernel_eps):
    q, k, v = _case(query_heads=1, key_heads=1)
    with pytest.raises((TypeError, ValueError), match="kernel_eps"):
        oal_b200.oal_attention(q, k, v, torch.tensor((0, 0, 1, 1), dtype=torch.int32), _factor(),
                               kernel_eps=kernel_eps)


def test_invalid_execution_causal_and_cpu_dispatch_are_rejected():
    q, k, v = _case(query_heads=1, key_heads=1)
    groups = torch.tensor((0, 0, 1, 1), dtype=torch.int32)
    with pytest.raises(ValueError, match="execution"):
        oal_b200.oal_attention(q, k, v, groups, _factor(), execution="torch")
    with pytest.raises(ValueError, match="causal"):
        oal_b200.oal_attention(q, k, v, groups, _factor(), causal=False)
    with pytest.raises(TypeError, match="causal"):
        oal_b200.oal_attention(q, k, v, groups, _factor(), causal=1)
    with pytest.raises(TypeError, match="output_dtype"):
        oal_b200.oal_attention(q, k, v, groups, _factor(), output_dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA"):
        oal_b200.oal_attention(q, k, v, groups, _factor(), execution="triton")
    with pytest.raises(RuntimeError, match="reference"):
        oal_b200.oal_attention(q, k, v, groups, _factor(), execution="reference")
    with pytest.raises(TypeError, match="FP32 working precision|float64"):
        oal_b200.grouped_causal_attention(q.double(), k.double(), v.double(), groups, _factor())


def test_plan_exposes_the_option_fields_callers_read_back():
    q, k, v = _case(sequence=300, dimension=64, value_dimension=64)
    plan = build_hd_block_gemm_plan(q, k, v, token_block=64, feature_wave_blocks=4, precision="fp32_ieee",
                                    requested_gradient_mask=(True,) * 6, backward_schedule="shared_wave",
                                    key_feature_impl="triton_materialized", save_local_score=True,
                                    key_retention="forward", groups=2)
    for name in PLAN_OPTION_FIELDS:
        assert hasattr(plan, name), name
    assert plan.token_block == 64 and plan.feature_wave_blocks == 4 and plan.number_blocks == 5
    assert plan.backward_schedule == "shared_wave" and plan.key_retention == "forward"
    assert len(plan.plan_id) == 64
    again = build_hd_block_gemm_plan(q, k, v, token_block=64, feature_wave_blocks=4, precision="fp32_ieee",
                                     requested_gradient_mask=(True,) * 6, backward_schedule="shared_wave",
                                     key_feature_impl="triton_materialized", save_local_score=True,
                                     key_retention="forward", groups=2)
    assert again.plan_id == plan.plan_id


@pytest.mark.parametrize("kwargs,exc", [
    (dict(token_block=0), ValueError),
    (dict(feature_wave_blocks=99), ValueError),
    (dict(precision="fp8"), ValueError),
    (dict(precision=7), TypeError),
    (dict(backward_schedule="wave"), ValueError),
    (dict(query_feature_token_tile=3), ValueError),
    (dict(key_retention="all"), ValueError),
    (dict(feature_padding="f2160"), ValueError),          # needs D = 64
    (dict(query_consumer_stages=("fold",)), ValueError),
    (dict(query_producer_fold_strategy="split"), ValueError),
    (dict(save_local_score="yes"), TypeError),
    (dict(requested_gradient_mask=(True,) * 5), ValueError),
    (dict(requested_gradient_mask=[True] * 6), TypeError),
    (dict(memory_budget_bytes=1), ValueError),
    (dict(precision="bf16_tensorcore"), ValueError),      # CPU fp32 tensors
    (dict(output_dtype=torch.int8), TypeError),
])
def test_plan_rejects_invalid_options(kwargs, exc):
    q, k, v = _case()
    base = dict(requested_gradient_mask=(True,) * 6)
    base.update(kwargs)
    with pytest.raises(exc):
        build_hd_block_gemm_plan(q, k, v, **base)


def test_plan_rejects_bad_geometry():
    q, k, v = _case()
    with pytest.raises(ValueError, match="contiguous"):
        build_hd_block_gemm_plan(q.transpose(1, 2), k, v, requested_gradient_mask=(False,) * 6)
    big = torch.zeros(1, 1, 2, 65)
    with pytest.raises(ValueError, match="head_dimension"):
        build_hd_block_gemm_plan(big, big, big, requested_gradient_mask=(False,) * 6)
    with pytest.raises(TypeError):
        build_hd_block_gemm_plan(q.double(), k.double(), v.double(), requested_gradient_mask=(False,) * 6)


# ---- helper-level cases of the reference's operator tests (tests/operators/test_grouped_quadratic.py:464-512
# there): group tables stay a logical broadcast, packed factor -> PSD coefficients, pair counts ----------------

def test_shared_dim_groups_stay_one_row():
    from oal_b200.grouped_quadratic import _canonicalize_dim_groups

    canonical = _canonicalize_dim_groups(torch.tensor((0, 0, 1, 1), dtype=torch.int64), query_heads=4,
                                         head_dimension=4, gmax=2, q_device=torch.device("cpu"))
    assert canonical.ndim == 1 and canonical.shape == (4,) and canonical.dtype == torch.int32


def test_packed_factor_expansion_matches_psd_coefficients():
    from oal_b200.grouped_quadratic import _expand_factor_coefficients

    constant, linear, quadratic = _expand_factor_coefficients(_factor(torch.float64), query_heads=1, gmax=2,
                                                              kernel_eps=0.07, working_dtype=torch.float64)
    lower = torch.tensor(((1.1, 0.0, 0.0), (0.5, 0.9, 0.0), (0.4, 0.8, 0.7)), dtype=torch.float64)
    matrix = lower @ lower.T
    torch.testing.assert_close(constant, matrix[0, 0].view(1) + 0.07)
    torch.testing.assert_close(linear, 2 * matrix[0, 1:].view(1, 2))
    torch.testing.assert_close(quadratic, matrix[1:, 1:].view(1, 2, 2))
    assert quadratic.is_contiguous()
    # and the per-head form with a gradient: d(sum C)/dL through the explicit products
    factor = torch.rand(3, 6, dtype=torch.float64).requires_grad_()
    _, _, c = _expand_factor_coefficients(factor, query_heads=3, gmax=2, kernel_eps=1e-6, working_dtype=torch.float64)
    c.sum().backward()
    assert factor.grad.shape == (3, 6) and torch.isfinite(factor.grad).all()


def test_packed_pair_count_is_triangular():
    from oal_b200.grouped_quadratic import _infer_gmax

    for gmax in (1, 2, 8, 16):
        assert _infer_gmax((gmax + 1) * (gmax + 2) // 2) == gmax
    with pytest.raises(ValueError):
        _infer_gmax(7)
