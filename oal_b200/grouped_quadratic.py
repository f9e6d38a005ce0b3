"""Public grouped quadratic attention API on the B200 kernels.

Keeps the call surface and the validation behaviour (exception types and
conditions) of the reference's ``oal_attention``
(oal_attention/grouped_quadratic.py:277-397; helpers :31-243).  Execution always
goes to the CUDA library of this package: ``execution="auto"`` and
``execution="triton"`` (the name of the reference's accelerated branch) both
select it; ``execution="reference"`` -- the pure-torch statement -- is not part
of this package and raises.
"""

from __future__ import annotations

import math
from typing import Literal

import torch

_SUPPORTED_FLOATING_DTYPES = frozenset({torch.float16, torch.bfloat16, torch.float32, torch.float64})
_SUPPORTED_FACTOR_DTYPES = frozenset({torch.float32, torch.float64})


def _resolve_working_dtype(q_dtype: torch.dtype, factor_dtype: torch.dtype) -> torch.dtype:
    promoted = torch.promote_types(q_dtype, factor_dtype)
    return torch.float64 if promoted == torch.float64 else torch.float32


def _validate_kernel_eps(kernel_eps: object, *, working_dtype: torch.dtype) -> float:
    if isinstance(kernel_eps, bool) or not isinstance(kernel_eps, (int, float)):
        raise TypeError("kernel_eps must be a positive finite Python scalar")
    try:
        resolved = float(kernel_eps)
    except OverflowError:
        raise ValueError("kernel_eps must be finite") from None
    if not math.isfinite(resolved) or resolved <= 0.0:
        raise ValueError("kernel_eps must be finite and positive")
    limits = torch.finfo(working_dtype)
    if resolved < limits.tiny * limits.eps or resolved > limits.max:
        raise ValueError("kernel_eps must remain finite and positive in the computation dtype")
    return resolved


def _validate_output_dtype(output_dtype: object) -> None:
    if output_dtype is not None and (
        not isinstance(output_dtype, torch.dtype) or output_dtype not in _SUPPORTED_FLOATING_DTYPES
    ):
        raise TypeError("output_dtype must be a supported floating torch.dtype")


def _infer_gmax(parameter_count: int) -> int:
    discriminant = 1 + 8 * parameter_count
    root = math.isqrt(discriminant)
    if root * root != discriminant or (root - 1) % 2 != 0:
        raise ValueError("factor last dimension must be a valid packed lower-triangular size")
    gmax = (root - 1) // 2 - 1
    if gmax < 1:
        raise ValueError("factor must reserve at least one dimension group")
    return gmax


def _validate_qkv(q: object, k: object, v: object):
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v)):
        raise TypeError("q, k, and v must be torch.Tensor objects")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k, and v must be rank-4 head-first tensors")
    if any(t.dtype not in _SUPPORTED_FLOATING_DTYPES for t in (q, k, v)):
        raise TypeError("q, k, and v must have floating-point dtypes")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError("q, k, and v must have the same dtype")
    if q.device != k.device or q.device != v.device:
        raise ValueError("q, k, and v must be on the same device")
    if q.shape[-1] != k.shape[-1]:
        raise ValueError("q and k must have the same feature dimension")
    if q.shape[0] != k.shape[0] or q.shape[0] != v.shape[0]:
        raise ValueError("q, k, and v must have the same batch size")
    if q.shape[2] != k.shape[2] or q.shape[2] != v.shape[2]:
        raise ValueError("q, k, and v must have the same sequence length")
    if k.shape[1] != v.shape[1]:
        raise ValueError("k and v must have the same KV head count")
    if q.shape[1] <= 0 or k.shape[1] <= 0:
        raise ValueError("q and k must have positive head counts")
    if any(dim <= 0 for dim in q.shape + v.shape[-1:]):
        raise ValueError("q, k, and v dimensions must be positive")
    if q.shape[1] % k.shape[1] != 0:
        raise ValueError("query head count must be divisible by KV head count")
    return q, k, v


def _validate_factor(factor: object, *, query_heads: int, q_device: torch.device):
    if not isinstance(factor, torch.Tensor):
        raise TypeError("factor must be a torch.Tensor")
    if factor.ndim not in (1, 2):
        raise ValueError("factor must have shape [P] or [Hq, P]")
    if factor.dtype not in _SUPPORTED_FACTOR_DTYPES:
        raise TypeError("factor must be a floating Tensor with dtype FP32 or FP64")
    if factor.device != q_device:
        raise ValueError("factor must be on the same device as q")
    if factor.shape[-1] <= 0:
        raise ValueError("factor must contain packed lower-triangular parameters")
    gmax = _infer_gmax(factor.shape[-1])
    if factor.ndim == 2 and factor.shape[0] != query_heads:
        raise ValueError("per-query-head factor first dimension must equal Hq")
    return factor, gmax


def _canonicalize_dim_groups(dim_groups: object, *, query_heads: int, head_dimension: int, gmax: int,
                             q_device: torch.device) -> torch.Tensor:
    """int32 ``[D]`` or ``[Hq, D]``; ids of every head must form the prefix 0..G_h-1, G_h <= gmax."""
    if not isinstance(dim_groups, torch.Tensor):
        raise TypeError("dim_groups must be a torch.Tensor")
    if dim_groups.dtype not in {torch.int32, torch.int64}:
        raise TypeError("dim_groups must use torch.int32 or torch.int64")
    if dim_groups.device != q_device:
        raise ValueError("dim_groups must be on the same device as q")
    if dim_groups.ndim == 1:
        if dim_groups.shape[0] != head_dimension:
            raise ValueError("dim_groups last dimension must equal D")
        per_head = dim_groups.unsqueeze(0)
    elif dim_groups.ndim == 2:
        if dim_groups.shape[0] != query_heads:
            raise ValueError("dim_groups first dimension must equal query-head count Hq")
        if dim_groups.shape[1] != head_dimension:
            raise ValueError("dim_groups last dimension must equal D")
        per_head = dim_groups
    else:
        raise ValueError("dim_groups must have shape [D] or [Hq, D]")
    # one device-to-host copy instead of the reference's per-head torch.unique loop
    table = per_head.detach().to("cpu", torch.int64)
    if not bool(((table >= 0) & (table < gmax)).all()):
        raise ValueError("dim_groups IDs must satisfy 0 <= id < Gmax")
    for row in table:
        used = torch.unique(row, sorted=True)
        if used.numel() == 0 or not torch.equal(used, torch.arange(used.numel())):
            raise ValueError("dim_groups IDs for every query head must form a continuous prefix")
    return dim_groups.to(dtype=torch.int32).contiguous()


class _ExpandFactorOnDevice(torch.autograd.Function):
    """fp32 CUDA factors: one kernel for the expansion and one for its gradient (``oal_expand_factor`` /
    ``oal_expand_factor_grad``) instead of about forty tensor operations and autograd nodes per step."""

    @staticmethod
    def forward(ctx, factor, query_heads: int, gmax: int, kernel_eps: float):
        import ctypes

        from . import _lib

        rows = factor.contiguous()
        rows = rows.unsqueeze(0) if rows.ndim == 1 else rows
        a = torch.empty(query_heads, dtype=torch.float32, device=factor.device)
        b = torch.empty(query_heads, gmax, dtype=torch.float32, device=factor.device)
        c = torch.empty(query_heads, gmax, gmax, dtype=torch.float32, device=factor.device)
        stream = ctypes.c_void_p(torch.cuda.current_stream(factor.device).cuda_stream)
        with _lib.device_guard(factor):
            _lib.check(_lib.load().oal_expand_factor(_lib.ptr(rows), rows.shape[0], query_heads, gmax, float(kernel_eps),
                                                     _lib.ptr(a), _lib.ptr(b), _lib.ptr(c), stream))
        ctx.save_for_backward(rows)
        ctx.geometry = (query_heads, gmax, factor.shape)
        return a, b, c

    @staticmethod
    def backward(ctx, grad_a, grad_b, grad_c):
        import ctypes

        from . import _lib

        (rows,) = ctx.saved_tensors
        query_heads, gmax, shape = ctx.geometry
        zeros = lambda *dims: torch.zeros(dims, dtype=torch.float32, device=rows.device)
        ga = zeros(query_heads) if grad_a is None else grad_a.float().contiguous()
        gb = zeros(query_heads, gmax) if grad_b is None else grad_b.float().contiguous()
        gc = zeros(query_heads, gmax, gmax) if grad_c is None else grad_c.float().contiguous()
        out = torch.empty_like(rows)
        stream = ctypes.c_void_p(torch.cuda.current_stream(rows.device).cuda_stream)
        with _lib.device_guard(rows):
            _lib.check(_lib.load().oal_expand_factor_grad(_lib.ptr(rows), rows.shape[0], query_heads, gmax, _lib.ptr(ga),
                                                          _lib.ptr(gb), _lib.ptr(gc), _lib.ptr(out), stream))
        return out.reshape(shape), None, None, None


def _expand_factor_coefficients(factor: torch.Tensor, *, query_heads: int, gmax: int, kernel_eps: float,
                                working_dtype: torch.dtype):
    """Packed lower triangle L -> A = M00 + eps, B = 2 M[0,1:], C = M[1:,1:], M = L L^T (differentiable)."""
    if factor.is_cuda and factor.dtype == torch.float32 and working_dtype == torch.float32:
        return _ExpandFactorOnDevice.apply(factor, query_heads, gmax, kernel_eps)
    factor_by_head = factor.unsqueeze(0) if factor.ndim == 1 else factor
    factor_by_head = factor_by_head.to(dtype=working_dtype)
    if factor_by_head.shape[0] == 1:
        factor_by_head = factor_by_head.expand(query_heads, -1)
    side = gmax + 1
    rows, columns = torch.tril_indices(side, side, device=factor.device)
    lower = torch.zeros((query_heads, side * side), dtype=working_dtype, device=factor.device)
    lower = lower.scatter(1, (rows * side + columns).unsqueeze(0).expand(query_heads, -1), factor_by_head)
    lower = lower.reshape(query_heads, side, side)
    # explicit products + sum: plain fp32 arithmetic whatever the ambient matmul precision
    matrix = (lower.unsqueeze(2) * lower.unsqueeze(1)).sum(dim=-1)
    constant = matrix[:, 0, 0] + kernel_eps
    linear = 2.0 * matrix[:, 0, 1:]
    quadratic = matrix[:, 1:, 1:].contiguous()
    return constant, linear, quadratic


def _validate_public_options(*, causal: object, execution: object, output_dtype: object,
                             return_unnormalized: object):
    if not isinstance(causal, bool):
        raise TypeError("causal must be a bool")
    if not causal:
        raise ValueError("grouped quadratic attention is causal-only; causal=False is no longer supported")
    if not isinstance(execution, str) or execution not in {"reference", "triton", "auto"}:
        raise ValueError("execution must be one of: reference, triton, auto")
    _validate_output_dtype(output_dtype)
    if not isinstance(return_unnormalized, bool):
        raise TypeError("return_unnormalized must be a bool")
    return causal, execution


def _resolve_scale(scale, head_dimension: int) -> float:
    if scale is None:
        return head_dimension ** -0.5
    if isinstance(scale, bool) or not isinstance(scale, (int, float)):
        raise TypeError("scale must be a finite Python scalar")
    try:
        resolved = float(scale)
    except OverflowError:
        raise ValueError("scale must be finite") from None
    if not math.isfinite(resolved):
        raise ValueError("scale must be finite")
    return resolved


def oal_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dim_groups: torch.Tensor,
    factor: torch.Tensor,
    *,
    scale: float | None = None,
    kernel_eps: float = 1e-6,
    causal: bool = True,
    execution: Literal["reference", "triton", "auto"] = "auto",
    output_dtype: torch.dtype | None = None,
    return_unnormalized: bool = False,
    precision: str | None = None,
):
    """Evaluate OAL's caller-grouped full PSD quadratic attention kernel on the GPU.

    ``precision`` (an addition to the reference signature) picks the arithmetic:
    ``"bf16_tensorcore"`` (default for bf16 inputs) or ``"fp32_ieee"`` (default
    otherwise).
    """
    from .hd_block_gemm_adapters import grouped_causal_attention

    q, k, v = _validate_qkv(q, k, v)
    causal, execution = _validate_public_options(causal=causal, execution=execution,
                                                 output_dtype=output_dtype,
                                                 return_unnormalized=return_unnormalized)
    factor, gmax = _validate_factor(factor, query_heads=q.shape[1], q_device=q.device)
    working_dtype = _resolve_working_dtype(q.dtype, factor.dtype)
    _validate_kernel_eps(kernel_eps, working_dtype=working_dtype)
    _canonicalize_dim_groups(dim_groups, query_heads=q.shape[1], head_dimension=q.shape[-1], gmax=gmax,
                             q_device=q.device)
    _resolve_scale(scale, q.shape[-1])
    if execution == "reference":
        raise RuntimeError("execution='reference' (the pure-torch statement) is not part of oal_b200")
    if q.device.type != "cuda":
        raise RuntimeError("oal_b200 grouped quadratic attention requires CUDA input")
    if working_dtype != torch.float32:
        raise TypeError("oal_b200 computes in FP32 working precision: float64 q/k/v or factor are not supported")
    if q.shape[-1] > 64:
        raise ValueError("oal_b200 grouped quadratic attention supports D<=64")
    if precision is None:
        precision = "bf16_tensorcore" if q.dtype == torch.bfloat16 else "fp32_ieee"
    output, numerator, denominator = grouped_causal_attention(
        q, k, v, dim_groups, factor, scale=scale, kernel_eps=kernel_eps, precision=precision,
        output_dtype=output_dtype)
    if return_unnormalized:
        return output, numerator, denominator
    return output


__all__ = ["oal_attention"]
