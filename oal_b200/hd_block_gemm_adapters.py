"""OAL grouped coefficients for the causal HD attention API.

Same three entry points, keyword names and return triple as the reference
(oal_attention/hd_block_gemm_adapters.py:120-415):
``prepare_grouped_hd_block_gemm`` freezes geometry, groups and the plan once,
``run_prepared_grouped_hd_block_gemm`` expands the live ``factor`` into (A, B, C)
with differentiable torch ops and enters the autograd Function,
``grouped_causal_attention`` does both.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .grouped_quadratic import (
    _canonicalize_dim_groups,
    _expand_factor_coefficients,
    _resolve_scale,
    _resolve_working_dtype,
    _validate_factor,
    _validate_kernel_eps,
    _validate_qkv,
)
from .hd_block_gemm import HDParallelBlockPlan, build_hd_block_gemm_plan
from .hd_block_gemm_autograd import (
    GroupTables,
    build_group_tables,
    hd_parallel_block_gemm,
    hd_parallel_block_gemm_autograd,
)

# oal_attention/hd_block_gemm_adapters.py:24
_POSITIVE_FP32_FLOOR = float(torch.finfo(torch.float32).tiny * torch.finfo(torch.float32).eps)


def _requested_gradient_mask(q, k, v, *, coefficient_source_requires_grad: bool):
    live = torch.is_grad_enabled()
    coefficient_grad = live and coefficient_source_requires_grad
    return (live and q.requires_grad, live and k.requires_grad, live and v.requires_grad,
            coefficient_grad, coefficient_grad, coefficient_grad)


@dataclass(frozen=True)
class _PreparedGroupedHdBlockGemm:
    """Immutable structural state for repeated invocations (no factor-derived values)."""

    plan: HDParallelBlockPlan
    groups: torch.Tensor
    tables: GroupTables
    gmax: int
    scale: float
    kernel_eps: float
    normalization_floor: float
    out_token_major: bool = False      # `out` is [B, N, Hq, 64] (an addition: see prepare_grouped_hd_block_gemm)


def prepare_grouped_hd_block_gemm(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dim_groups: torch.Tensor,
    factor: torch.Tensor,
    *,
    scale: float | None = None,
    kernel_eps: float = 1e-6,
    token_block: int = 128,
    feature_wave_blocks: int | None = None,
    memory_budget_bytes: int | None = None,
    model_residency_bytes: int = 0,
    precision: str = "fp32_ieee",
    key_feature_impl: str = "generic_materialized",
    key_fold_impl: str = "generic_materialized",
    query_feature_impl: str = "generic_materialized",
    query_feature_token_tile: int = 1,
    query_fold_impl: str = "generic_materialized",
    query_fold_token_tile: int = 1,
    query_fold_input: str = "staged_fp32",
    query_gradient_flow: str = "materialized",
    query_producer_fold_strategy: str | None = None,
    query_consumer_stages: tuple[str, ...] | None = None,
    query_consumer_fusion: str | None = None,
    backward_schedule: str = "split",
    gradient_staging: str = "per_wave",
    forward_normalize_impl: str = "torch",
    backward_normalize_impl: str = "torch",
    kv_cross_impl: str = "split",
    save_local_score: bool = False,
    key_retention: str = "none",
    feature_padding: str = "none",
    output_dtype: torch.dtype | None = None,
    output_layout: str = "heads_first",
) -> _PreparedGroupedHdBlockGemm:
    """Freeze geometry/groups once for an explicitly repeated workload.

    ``output_layout`` (an addition to the reference's signature): ``"heads_first"`` returns ``out`` as
    ``[B, Hq, N, Dv]`` like the reference; ``"tokens_first"`` returns it as ``[B, N, Hq, Dv]``, which the
    kernels write directly, so the caller's restore step (transpose + contiguous copy,
    qwen_lora_experiment/attention/common.py:575-596) disappears; the upstream gradient of ``out`` is then
    expected in that layout too.  Tensor-core precision, Dv = 64 and at most 8 groups per head only."""
    if output_layout not in ("heads_first", "tokens_first"):
        raise ValueError("output_layout must be 'heads_first' or 'tokens_first'")
    q, k, v = _validate_qkv(q, k, v)
    factor, gmax = _validate_factor(factor, query_heads=q.shape[1], q_device=q.device)
    working_dtype = _resolve_working_dtype(q.dtype, factor.dtype)
    if working_dtype != torch.float32:
        raise TypeError("grouped HD Block-GEMM requires FP32 working precision")
    resolved_eps = _validate_kernel_eps(kernel_eps, working_dtype=working_dtype)
    canonical_groups = _canonicalize_dim_groups(dim_groups, query_heads=q.shape[1],
                                                head_dimension=q.shape[-1], gmax=gmax, q_device=q.device)
    gradient_mask = _requested_gradient_mask(q, k, v, coefficient_source_requires_grad=factor.requires_grad)
    plan = build_hd_block_gemm_plan(
        q, k, v,
        token_block=token_block, feature_wave_blocks=feature_wave_blocks,
        memory_budget_bytes=memory_budget_bytes, model_residency_bytes=model_residency_bytes,
        requested_gradient_mask=gradient_mask, precision=precision,
        key_feature_impl=key_feature_impl, key_fold_impl=key_fold_impl,
        query_feature_impl=query_feature_impl, query_feature_token_tile=query_feature_token_tile,
        query_fold_impl=query_fold_impl, query_fold_token_tile=query_fold_token_tile,
        query_fold_input=query_fold_input, query_gradient_flow=query_gradient_flow,
        query_producer_fold_strategy=query_producer_fold_strategy,
        query_consumer_stages=query_consumer_stages, query_consumer_fusion=query_consumer_fusion,
        backward_schedule=backward_schedule, gradient_staging=gradient_staging,
        forward_normalize_impl=forward_normalize_impl, backward_normalize_impl=backward_normalize_impl,
        kv_cross_impl=kv_cross_impl, save_local_score=save_local_score, key_retention=key_retention,
        feature_padding=feature_padding, output_dtype=output_dtype, groups=gmax,
    )
    groups = (canonical_groups.unsqueeze(0).expand(q.shape[1], -1)
              if canonical_groups.ndim == 1 else canonical_groups).detach().clone()
    return _PreparedGroupedHdBlockGemm(
        plan=plan, groups=groups, tables=build_group_tables(groups, gmax), gmax=gmax,
        scale=_resolve_scale(scale, q.shape[-1]), kernel_eps=resolved_eps,
        normalization_floor=_POSITIVE_FP32_FLOOR, out_token_major=output_layout == "tokens_first")


def run_prepared_grouped_hd_block_gemm(prepared, q, k, v, factor):
    """Run one live invocation against an explicit immutable preparation."""
    if not isinstance(prepared, _PreparedGroupedHdBlockGemm):
        raise TypeError("prepared must be an explicit grouped HD Block-GEMM preparation")
    q, k, v = _validate_qkv(q, k, v)
    factor, gmax = _validate_factor(factor, query_heads=q.shape[1], q_device=q.device)
    if gmax != prepared.gmax:
        raise ValueError("factor group geometry does not match the preparation")
    if _resolve_working_dtype(q.dtype, factor.dtype) != torch.float32:
        raise TypeError("grouped HD Block-GEMM requires FP32 working precision")
    plan = prepared.plan
    if tuple(q.shape) + tuple(k.shape[1:2]) + tuple(v.shape[-1:]) != (
            plan.batch_size, plan.query_heads, plan.sequence_length, plan.head_dimension,
            plan.key_value_heads, plan.value_dimension):
        raise ValueError("live tensor geometry does not match the preparation")
    if str(q.dtype).removeprefix("torch.") != plan.input_dtype or str(q.device) != plan.device:
        raise ValueError("live tensor dtype/device does not match the preparation")
    gradient_mask = _requested_gradient_mask(q, k, v, coefficient_source_requires_grad=factor.requires_grad)
    if gradient_mask != plan.requested_gradient_mask:
        raise ValueError("live gradient mode does not match the preparation")
    a, b, c = _expand_factor_coefficients(factor, query_heads=plan.query_heads, gmax=prepared.gmax,
                                          kernel_eps=prepared.kernel_eps, working_dtype=torch.float32)
    return run_grouped_coefficients(q, k, v, a.contiguous(), b.contiguous(), c.contiguous(),
                                    tables=prepared.tables, plan=plan, scale=prepared.scale,
                                    normalization_floor=prepared.normalization_floor,
                                    out_token_major=prepared.out_token_major)


def run_grouped_coefficients(q, k, v, a, b, c, *, tables, plan, scale, normalization_floor, out_token_major=False):
    """Enter the kernels with explicit per-head coefficients A [Hq], B [Hq,G], C [Hq,G,G]."""
    run = hd_parallel_block_gemm_autograd if any(plan.requested_gradient_mask) else hd_parallel_block_gemm
    return run(q, k, v, a, b, c, tables=tables, scale=scale, eps=normalization_floor, plan=plan,
               out_token_major=out_token_major)


def grouped_causal_attention(q, k, v, dim_groups, factor, **kwargs):
    """Prepare and run one grouped causal invocation with a live factor.

    Keyword arguments are those of ``prepare_grouped_hd_block_gemm``.
    """
    prepared = prepare_grouped_hd_block_gemm(q, k, v, dim_groups, factor, **kwargs)
    return run_prepared_grouped_hd_block_gemm(prepared, q, k, v, factor)


def grouped_coefficient_attention(q, k, v, dim_groups, constant, linear, quadratic, *, scale=None,
                                  precision="fp32_ieee", output_dtype=None,
                                  normalization_floor=_POSITIVE_FP32_FLOOR):
    """Same operator with the expanded coefficients given directly
    (``constant [Hq]``, ``linear [Hq,G]``, ``quadratic [Hq,G,G]`` symmetric), the
    form the reference oracle takes (oal_attention/grouped_reference.py:181-193)."""
    q, k, v = _validate_qkv(q, k, v)
    hq, g = linear.shape
    if constant.shape != (hq,) or quadratic.shape != (hq, g, g) or hq != q.shape[1]:
        raise ValueError("coefficients must have shapes [Hq], [Hq,G], [Hq,G,G]")
    groups = _canonicalize_dim_groups(dim_groups, query_heads=hq, head_dimension=q.shape[-1], gmax=g,
                                      q_device=q.device)
    groups = groups.unsqueeze(0).expand(hq, -1) if groups.ndim == 1 else groups
    live = torch.is_grad_enabled()
    coef = live and (constant.requires_grad or linear.requires_grad or quadratic.requires_grad)
    mask = (live and q.requires_grad, live and k.requires_grad, live and v.requires_grad, coef, coef, coef)
    plan = build_hd_block_gemm_plan(q, k, v, precision=precision, requested_gradient_mask=mask,
                                    output_dtype=output_dtype, groups=g)
    if coef:   # the Function differentiates all three together
        constant, linear, quadratic = (t if t.requires_grad else t.detach().requires_grad_()
                                       for t in (constant, linear, quadratic))
    return run_grouped_coefficients(q, k, v, constant, linear, quadratic,
                                    tables=build_group_tables(groups, g), plan=plan,
                                    scale=_resolve_scale(scale, q.shape[-1]),
                                    normalization_floor=normalization_floor)


_grouped_hd_block_gemm_forward = grouped_causal_attention
_prepare_grouped_hd_block_gemm = prepare_grouped_hd_block_gemm
_run_prepared_grouped_hd_block_gemm = run_prepared_grouped_hd_block_gemm

__all__ = (
    "grouped_causal_attention",
    "prepare_grouped_hd_block_gemm",
    "run_prepared_grouped_hd_block_gemm",
    "grouped_coefficient_attention",
)
