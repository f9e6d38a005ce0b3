"""Plan object of the HD entry points.

Mirrors the caller-visible part of the reference planner
(oal_attention/hd_block_gemm.py:223-537 ``build_hd_block_gemm_plan`` and
oal_attention/hd_block_gemm_plan.py:84-711 ``HDParallelBlockPlan``): geometry and
selector validation with the same exception types, a frozen plan exposing the
option fields callers read back (qwen_lora_experiment/attention/hd_runtime.py:95-116)
and a sha256 ``plan_id``.  The reference's 64-entry buffer table is replaced by
one workspace-size query into the CUDA library (``workspace_bytes``).

The implementation selectors (``*_impl``, ``backward_schedule``, ...) choose
between internals of the reference that do not exist here; they are validated
against the reference's legal values and recorded, nothing more.
"""

from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from math import ceil
from typing import Sequence

import torch

from . import _lib

_MAX_HEAD_DIMENSION = 64
_SUPPORTED_PRECISIONS = ("fp32_ieee", "bf16_tensorcore")
_DTYPE_NAMES = {torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float32: "float32",
                torch.float64: "float64"}
_FULL_AUX_RESULT_CONTRACT = "full_aux"

# oal_attention/hd_block_gemm_contracts.py:58-71
_IMPLS = ("generic_materialized", "triton_materialized")
_SELECTOR_VALUES = {
    "key_feature_impl": _IMPLS,
    "key_fold_impl": _IMPLS,
    "query_feature_impl": _IMPLS,
    "query_fold_impl": _IMPLS,
    "query_gradient_flow": ("materialized",),
    "backward_schedule": ("split", "shared_wave"),
    "gradient_staging": ("per_wave", "full_bf16"),
    "forward_normalize_impl": ("torch", "triton"),
    "backward_normalize_impl": ("torch", "triton"),
    "kv_cross_impl": ("split", "batched_dense"),
    "query_fold_input": ("staged_fp32", "raw"),
    "key_retention": ("none", "forward", "backward"),
    "feature_padding": ("none", "f2160"),
}
_TOKEN_TILES = (1, 2, 4)

PLAN_OPTION_FIELDS = (
    "token_block", "feature_wave_blocks", "memory_budget_bytes", "precision", "key_feature_impl",
    "key_fold_impl", "query_feature_impl", "query_feature_token_tile", "query_fold_impl",
    "query_fold_token_tile", "query_fold_input", "query_gradient_flow", "backward_schedule",
    "gradient_staging", "forward_normalize_impl", "backward_normalize_impl", "kv_cross_impl",
    "save_local_score", "key_retention", "feature_padding",
)


def _require_plain_int(value: object, *, name: str, minimum: int) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < minimum:
        comparison = "positive" if minimum == 1 else f">= {minimum}"
        raise ValueError(f"{name} must be a {comparison} integer")
    return value


def _contiguous_strides(shape) -> tuple[int, ...]:
    stride, rev = 1, []
    for dim in reversed(shape):
        rev.append(stride)
        stride *= dim
    return tuple(reversed(rev))


@dataclass(frozen=True)
class HDParallelBlockPlan:
    """Immutable description of one planned invocation."""

    token_block: int
    feature_wave_blocks: int
    memory_budget_bytes: int | None
    model_residency_bytes: int
    precision: str
    requested_precision: str
    key_feature_impl: str
    key_fold_impl: str
    query_feature_impl: str
    query_feature_token_tile: int
    query_fold_impl: str
    query_fold_token_tile: int
    query_fold_input: str
    query_gradient_flow: str
    backward_schedule: str
    gradient_staging: str
    forward_normalize_impl: str
    backward_normalize_impl: str
    kv_cross_impl: str
    save_local_score: bool
    key_retention: str
    feature_padding: str
    requested_gradient_mask: tuple[bool, bool, bool, bool, bool, bool]
    geometry: tuple[int, int, int, int, int, int]
    input_dtype: str
    output_dtype: str
    device_type: str
    device: str
    number_blocks: int
    chunk_tokens: int                 # tokens per chunk of the state scan actually used by the kernels
    forward_workspace_bytes: int
    backward_workspace_bytes: int
    saved_state_bytes: int
    plan_id: str = field(default="")

    @property
    def batch_size(self) -> int:
        return self.geometry[0]

    @property
    def query_heads(self) -> int:
        return self.geometry[1]

    @property
    def key_value_heads(self) -> int:
        return self.geometry[2]

    @property
    def sequence_length(self) -> int:
        return self.geometry[3]

    @property
    def head_dimension(self) -> int:
        return self.geometry[4]

    @property
    def value_dimension(self) -> int:
        return self.geometry[5]

    @property
    def gqa_ratio(self) -> int:
        return self.geometry[1] // self.geometry[2]

    @property
    def invocation_peak_bytes(self) -> int:
        return max(self.forward_workspace_bytes, self.backward_workspace_bytes) + self.saved_state_bytes

    @property
    def projected_live_bytes(self) -> int:
        return self.invocation_peak_bytes + self.model_residency_bytes


def _validate_geometry(q, k, v):
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v)):
        raise TypeError("Q, K, and V must be tensors")
    if any(t.ndim != 4 for t in (q, k, v)):
        raise ValueError("Q, K, and V must be rank-4 tensors")
    if any(d <= 0 for t in (q, k, v) for d in t.shape):
        raise ValueError("Q, K, and V geometry sizes must be positive")
    if any(t.layout != torch.strided for t in (q, k, v)):
        raise ValueError("Q, K, and V must use torch.strided layout")
    for t in (q, k, v):
        # the stride of a dimension of size 1 addresses nothing (a slice of one KV head keeps its parent's): only
        # the dimensions that are walked must have the row-major strides
        want = _contiguous_strides(tuple(t.shape))
        if any(n > 1 and have != need for n, have, need in zip(t.shape, t.stride(), want)):
            raise ValueError("Q, K, and V must use exact row-major contiguous layout")
    b, hq, n, d = q.shape
    kb, hkv, kn, kd = k.shape
    vb, vh, vn, dv = v.shape
    if b != kb or b != vb:
        raise ValueError("Q, K, and V must have the same batch size")
    if n != kn or n != vn:
        raise ValueError("Q, K, and V must have the same sequence length")
    if hkv != vh:
        raise ValueError("K and V must have the same key/value head count")
    if hq % hkv:
        raise ValueError("query heads must be divisible by key/value heads")
    if d != kd:
        raise ValueError("Q and K must have the same head dimension")
    if d > _MAX_HEAD_DIMENSION:
        raise ValueError(f"head_dimension must be no greater than {_MAX_HEAD_DIMENSION}")
    if dv > _MAX_HEAD_DIMENSION:
        raise ValueError(f"value_dimension must be no greater than {_MAX_HEAD_DIMENSION}")
    if q.device != k.device or q.device != v.device:
        raise ValueError("Q, K, and V must be on the same device")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError("Q, K, and V must have the same dtype")
    if q.dtype not in _DTYPE_NAMES:
        raise TypeError("Q, K, and V must be float16, bfloat16, float32, or float64")
    return b, hq, hkv, n, d, dv


def make_problem(geometry, *, groups: int, io_dtype: torch.dtype, out_dtype: torch.dtype, precision: str,
                 chunk: int, scale: float, floor: float, grad_mask: int = 0,
                 flags: int = 0) -> _lib.OalProblem:
    """Fill the C struct for a (padded) problem."""
    b, hq, hkv, n, _, _ = geometry
    return _lib.OalProblem(batch=b, q_heads=hq, kv_heads=hkv, seq_len=n, head_dim=_lib.HEAD_DIM,
                           value_dim=_lib.HEAD_DIM, groups=groups, chunk=chunk,
                           io_dtype=_lib.DTYPE_CODES[io_dtype], out_dtype=_lib.DTYPE_CODES[out_dtype],
                           precision=_lib.PRECISION_CODES[precision], grad_mask=grad_mask,
                           scale=scale, floor=floor, flags=flags)


def kernel_chunk_tokens(precision: str) -> int:
    """Tokens per chunk the kernels use: the tensor-core path scans 128-token chunks
    (one 128-row MMA tile per query head); the fp32 path sums token pairs exactly
    and has no chunks."""
    return 128 if precision == "bf16_tensorcore" else 0


def build_hd_block_gemm_plan(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    token_block: int = 128,
    feature_wave_blocks: int | None = None,
    precision: str = "fp32_ieee",
    result_contract: str = _FULL_AUX_RESULT_CONTRACT,
    key_feature_impl: str = "generic_materialized",
    key_fold_impl: str = "generic_materialized",
    query_feature_impl: str = "generic_materialized",
    query_feature_token_tile: int = 1,
    query_fold_impl: str = "generic_materialized",
    query_fold_token_tile: int = 1,
    query_fold_input: str = "staged_fp32",
    query_gradient_flow: str = "materialized",
    query_producer_fold_strategy: str | None = None,
    query_producer_partition_count: int | None = None,
    query_consumer_stages: Sequence[str] | None = None,
    query_consumer_fusion: str | None = None,
    backward_schedule: str = "split",
    gradient_staging: str = "per_wave",
    forward_normalize_impl: str = "torch",
    backward_normalize_impl: str = "torch",
    kv_cross_impl: str = "split",
    save_local_score: bool = False,
    key_retention: str = "none",
    output_dtype: torch.dtype | None = None,
    requested_gradient_mask: tuple[bool, bool, bool, bool, bool, bool],
    memory_budget_bytes: int | None = None,
    model_residency_bytes: int = 0,
    strict_backend: bool = True,
    feature_padding: str = "none",
    groups: int = 1,
) -> HDParallelBlockPlan:
    """Validate one invocation and size its workspaces (no device allocation)."""
    if not isinstance(result_contract, str):
        raise TypeError("result_contract must be a string")
    if result_contract != _FULL_AUX_RESULT_CONTRACT:
        raise NotImplementedError("only the full (out, numerator, denominator) result contract exists")
    geometry = _validate_geometry(q, k, v)
    b, hq, hkv, n, d, dv = geometry
    token_block = _require_plain_int(token_block, name="token_block", minimum=1)
    number_blocks = ceil(n / token_block)
    if feature_wave_blocks is None:
        feature_wave_blocks = number_blocks
    feature_wave_blocks = _require_plain_int(feature_wave_blocks, name="feature_wave_blocks", minimum=1)
    if feature_wave_blocks > number_blocks:
        raise ValueError("feature_wave_blocks cannot exceed the number of blocks")
    if not isinstance(precision, str):
        raise TypeError("precision must be a string")
    if precision not in _SUPPORTED_PRECISIONS:
        raise ValueError("unsupported HD Block-GEMM precision")
    if type(strict_backend) is not bool:
        raise TypeError("strict_backend must be a bool")
    if not isinstance(requested_gradient_mask, tuple):
        raise TypeError("requested_gradient_mask must be a tuple")
    if len(requested_gradient_mask) != 6:
        raise ValueError("requested_gradient_mask must contain exactly six bools")
    if any(type(x) is not bool for x in requested_gradient_mask):
        raise TypeError("requested_gradient_mask entries must be bool values")
    if memory_budget_bytes is not None:
        memory_budget_bytes = _require_plain_int(memory_budget_bytes, name="memory_budget_bytes", minimum=1)
    model_residency_bytes = _require_plain_int(model_residency_bytes, name="model_residency_bytes", minimum=0)
    if q.dtype == torch.float64:
        raise TypeError("HD Block-GEMM requires FP32 working precision (float64 inputs are not supported)")
    if precision == "bf16_tensorcore":
        if q.device.type != "cuda":
            raise ValueError("bf16_tensorcore requires CUDA")
        if q.dtype != torch.bfloat16:
            raise ValueError("bf16_tensorcore requires bfloat16 Q/K/V")
    selectors = dict(key_feature_impl=key_feature_impl, key_fold_impl=key_fold_impl,
                     query_feature_impl=query_feature_impl, query_fold_impl=query_fold_impl,
                     query_gradient_flow=query_gradient_flow, backward_schedule=backward_schedule,
                     gradient_staging=gradient_staging, forward_normalize_impl=forward_normalize_impl,
                     backward_normalize_impl=backward_normalize_impl, kv_cross_impl=kv_cross_impl,
                     query_fold_input=query_fold_input, key_retention=key_retention,
                     feature_padding=feature_padding)
    for name, value in selectors.items():
        if not isinstance(value, str):
            raise TypeError(f"{name} must be a string")
        if value not in _SELECTOR_VALUES[name]:
            raise ValueError(f"unsupported {name}")
    if feature_padding == "f2160" and d != 64:
        raise ValueError("feature_padding='f2160' requires D=64")
    for name, value in (("query_feature_token_tile", query_feature_token_tile),
                        ("query_fold_token_tile", query_fold_token_tile)):
        if not isinstance(value, int) or isinstance(value, bool) or value not in _TOKEN_TILES:
            raise ValueError(f"{name} must be one of 1, 2, 4")
    # retired exploration selectors of the reference: only their neutral values are legal
    if query_producer_fold_strategy not in (None, "none"):
        raise ValueError("query_producer_fold_strategy: OP-3 exploration is retired")
    if query_producer_partition_count is not None:
        raise ValueError("query_producer_partition_count: OP-3 exploration is retired")
    if query_consumer_stages is not None:
        if not isinstance(query_consumer_stages, Sequence) or isinstance(query_consumer_stages, (str, bytes)):
            raise TypeError("query_consumer_stages must be a sequence")
        if tuple(query_consumer_stages):
            raise ValueError("query_consumer_stages: OP-4 exploration is retired")
    if query_consumer_fusion not in (None, "none"):
        raise ValueError("query_consumer_fusion: exploration is retired")
    if type(save_local_score) is not bool:
        raise TypeError("save_local_score must be a bool")
    if output_dtype is None:
        out_dtype = q.dtype
    else:
        if not isinstance(output_dtype, torch.dtype):
            raise TypeError("output_dtype must be a torch.dtype")
        if output_dtype not in _DTYPE_NAMES:
            raise TypeError("output_dtype must be float16, bfloat16, float32, or float64")
        out_dtype = output_dtype
    groups = _require_plain_int(groups, name="groups", minimum=1)
    if groups > _lib.MAX_GROUPS:
        raise ValueError(f"at most {_lib.MAX_GROUPS} dimension groups per head are supported")

    chunk = kernel_chunk_tokens(precision)
    kernel_out = out_dtype if out_dtype != torch.float64 else torch.float32
    problem = make_problem(geometry, groups=groups, io_dtype=q.dtype, out_dtype=kernel_out,
                           precision=precision, chunk=chunk, scale=1.0, floor=1e-38)
    sizes = [_lib.workspace_bytes(problem, phase) for phase in (0, 1, 2)]
    if memory_budget_bytes is not None:
        peak = max(sizes[0], sizes[1]) + sizes[2] + model_residency_bytes
        if peak > memory_budget_bytes:
            raise ValueError("memory budget is below the exact invocation peak plus model residency")
    payload = dict(geometry=list(geometry), token_block=token_block, feature_wave_blocks=feature_wave_blocks,
                   precision=precision, mask=list(requested_gradient_mask), in_dtype=_DTYPE_NAMES[q.dtype],
                   out_dtype=_DTYPE_NAMES[out_dtype], device=str(q.device), selectors=selectors,
                   tiles=[query_feature_token_tile, query_fold_token_tile], save=save_local_score,
                   groups=groups, sizes=sizes)
    plan_id = hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":")).encode()).hexdigest()
    return HDParallelBlockPlan(
        token_block=token_block, feature_wave_blocks=feature_wave_blocks,
        memory_budget_bytes=memory_budget_bytes, model_residency_bytes=model_residency_bytes,
        precision=precision, requested_precision=precision,
        key_feature_impl=key_feature_impl, key_fold_impl=key_fold_impl,
        query_feature_impl=query_feature_impl, query_feature_token_tile=query_feature_token_tile,
        query_fold_impl=query_fold_impl, query_fold_token_tile=query_fold_token_tile,
        query_fold_input=query_fold_input, query_gradient_flow=query_gradient_flow,
        backward_schedule=backward_schedule, gradient_staging=gradient_staging,
        forward_normalize_impl=forward_normalize_impl, backward_normalize_impl=backward_normalize_impl,
        kv_cross_impl=kv_cross_impl, save_local_score=save_local_score, key_retention=key_retention,
        feature_padding=feature_padding, requested_gradient_mask=requested_gradient_mask,
        geometry=geometry, input_dtype=_DTYPE_NAMES[q.dtype], output_dtype=_DTYPE_NAMES[out_dtype],
        device_type=q.device.type, device=str(q.device), number_blocks=number_blocks,
        chunk_tokens=chunk, forward_workspace_bytes=sizes[0], backward_workspace_bytes=sizes[1],
        saved_state_bytes=sizes[2], plan_id=plan_id)
