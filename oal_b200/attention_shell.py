"""The caller of the operator inside a transformer layer: projections, RoPE, the prepared call, o_proj.

Mirror of the reference's attention shell and runtime bridge
(qwen_lora_experiment/attention/common.py:510-596: q/k/v projection, reshape to head-first
``[B, H, N, 64]``, rotary embedding on q and k only, contiguous tensors into the operator, restore to
``[B, N, Hq*64]``, one o_proj; qwen_lora_experiment/attention/hd_runtime.py:37-86: per-layer cache of
prepared calls keyed by the shapes / dtypes / gradient flags of the arguments, two entries per layer).
The projections are ordinary ``nn.Linear`` matrix products (library GEMMs); everything between them is
the CUDA operator of this package.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn

from .hd_block_gemm_adapters import prepare_grouped_hd_block_gemm, run_prepared_grouped_hd_block_gemm


@dataclass(frozen=True)
class ModelGeometry:
    """(layers, hidden, query heads, kv heads, head dim), as qwen_lora_experiment/backbones/spec.py:29-33."""

    num_layers: int = 24
    hidden_size: int = 896
    num_query_heads: int = 14
    num_kv_heads: int = 2
    head_dim: int = 64


QWEN_GEOMETRY = ModelGeometry()


class AttentionContractError(RuntimeError):
    """A tensor handed to the shell does not have the layout the layer promises."""


def rope_tables(sequence_length: int, head_dim: int, *, theta: float = 1.0e6, device=None,
                dtype=torch.float32) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin of shape ``[N, head_dim]`` in the rotate-half convention (frequencies repeated twice)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.arange(sequence_length, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rotary_pos_emb(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """Rotate q and k (``[B, H, N, D]``) by position; cos / sin are ``[N, D]``."""

    def rot(x):
        half = x.shape[-1] // 2
        return torch.cat((-x[..., half:], x[..., :half]), dim=-1)

    return q * cos + rot(q) * sin, k * cos + rot(k) * sin


class _RopePackFunction(torch.autograd.Function):
    """Rotary embedding of q and k fused with the move to the head-first layout (one CUDA pass per
    tensor in each direction); v is moved only.  bf16 CUDA tensors, head dimension 64."""

    @staticmethod
    def forward(ctx, q_flat, k_flat, v_flat, cos, sin, q_heads: int, kv_heads: int):
        from . import _lib
        from .hd_block_gemm_autograd import _stream_ptr

        b, n, _ = q_flat.shape
        q_flat, k_flat, v_flat = q_flat.contiguous(), k_flat.contiguous(), v_flat.contiguous()
        cos, sin = cos.float().contiguous(), sin.float().contiguous()
        q = torch.empty(b, q_heads, n, 64, dtype=q_flat.dtype, device=q_flat.device)
        k = torch.empty(b, kv_heads, n, 64, dtype=q_flat.dtype, device=q_flat.device)
        v = torch.empty(b, kv_heads, n, 64, dtype=q_flat.dtype, device=q_flat.device)
        with _lib.device_guard(q_flat):
            rc = _lib.load().oal_rope_pack(_lib.ptr(q_flat), _lib.ptr(k_flat), _lib.ptr(v_flat), _lib.ptr(cos),
                                           _lib.ptr(sin), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), b, n, q_heads,
                                           kv_heads, _stream_ptr(q_flat.device))
        _lib.check(rc)
        ctx.save_for_backward(cos, sin)
        ctx.geometry = (b, n, q_heads, kv_heads)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        from . import _lib
        from .hd_block_gemm_autograd import _stream_ptr

        cos, sin = ctx.saved_tensors
        b, n, hq, hkv = ctx.geometry
        mk = lambda g, h: None if g is None else torch.empty(b, n, h * 64, dtype=g.dtype, device=g.device)
        dq, dk, dv = (None if g is None else g.contiguous() for g in (dq, dk, dv))
        dq_flat, dk_flat, dv_flat = mk(dq, hq), mk(dk, hkv), mk(dv, hkv)
        dev = next(g for g in (dq, dk, dv) if g is not None).device
        with torch.cuda.device(dev):
            rc = _lib.load().oal_rope_unpack_grad(_lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(cos),
                                                  _lib.ptr(sin), _lib.ptr(dq_flat), _lib.ptr(dk_flat),
                                                  _lib.ptr(dv_flat), b, n, hq, hkv, _stream_ptr(dev))
        _lib.check(rc)
        return dq_flat, dk_flat, dv_flat, None, None, None, None


def _fused_prologue_applies(hidden_states: torch.Tensor, geometry: ModelGeometry) -> bool:
    return hidden_states.is_cuda and hidden_states.dtype == torch.bfloat16 and geometry.head_dim == 64


def project_qkv_and_apply_rope(*, q_proj: nn.Module, k_proj: nn.Module, v_proj: nn.Module,
                               hidden_states: torch.Tensor, position_embeddings, geometry: ModelGeometry = QWEN_GEOMETRY,
                               fused: bool | None = None):
    """Project q/k/v, reshape to native heads, rotate q and k only; returns contiguous head-first tensors.

    ``fused`` (default: whenever the tensors are bf16 on CUDA) does the rotation and the layout move in the
    library's single-pass kernels instead of torch's element-wise sequence.
    """
    if hidden_states.dim() != 3 or hidden_states.shape[-1] != geometry.hidden_size:
        raise AttentionContractError(f"hidden_states must be [B, N, {geometry.hidden_size}], got {tuple(hidden_states.shape)}")
    b, n, _ = hidden_states.shape
    cos, sin = position_embeddings
    if cos.shape != (n, geometry.head_dim) or sin.shape != cos.shape:
        raise AttentionContractError(f"position embeddings must be [{n}, {geometry.head_dim}]")
    if fused is None:
        fused = _fused_prologue_applies(hidden_states, geometry)
    if fused:
        return _RopePackFunction.apply(q_proj(hidden_states), k_proj(hidden_states), v_proj(hidden_states), cos, sin,
                                       geometry.num_query_heads, geometry.num_kv_heads)
    q = q_proj(hidden_states).reshape(b, n, geometry.num_query_heads, geometry.head_dim).transpose(1, 2)
    k = k_proj(hidden_states).reshape(b, n, geometry.num_kv_heads, geometry.head_dim).transpose(1, 2)
    v = v_proj(hidden_states).reshape(b, n, geometry.num_kv_heads, geometry.head_dim).transpose(1, 2)
    q, k = apply_rotary_pos_emb(q, k, cos.to(q.dtype), sin.to(q.dtype))
    return q.contiguous(), k.contiguous(), v.contiguous()


def project_token_major_output(*, token_output: torch.Tensor, o_proj: nn.Module, geometry: ModelGeometry = QWEN_GEOMETRY):
    """Operator output already in ``[B, N, Hq, D]`` (``output_layout="tokens_first"``): a view and one o_proj."""
    b, n, h, d = token_output.shape
    if h != geometry.num_query_heads or d != geometry.head_dim:
        raise AttentionContractError(f"token_output must be [B, N, {geometry.num_query_heads}, {geometry.head_dim}]")
    return o_proj(token_output.reshape(b, n, geometry.hidden_size))


def restore_and_project_output(*, head_output: torch.Tensor, o_proj: nn.Module, geometry: ModelGeometry = QWEN_GEOMETRY):
    """``[B, Hq, N, D]`` back to ``[B, N, hidden]`` and one o_proj."""
    b, h, n, d = head_output.shape
    if h != geometry.num_query_heads or d != geometry.head_dim:
        raise AttentionContractError(f"head_output must be [B, {geometry.num_query_heads}, N, {geometry.head_dim}]")
    return o_proj(head_output.transpose(1, 2).contiguous().reshape(b, n, geometry.hidden_size))


class PreparedCallCache:
    """Per-layer cache of prepared operator calls (qwen_lora_experiment/attention/hd_runtime.py:37-86)."""

    def __init__(self, *, precision: str = "bf16_tensorcore", kernel_eps: float = 1e-6,
                 output_layout: str = "heads_first"):
        self.precision = precision
        self.kernel_eps = kernel_eps
        self.output_layout = output_layout
        self._entries: dict[object, list] = {}

    def grouped(self, q, k, v, dim_groups, factor, *, cache_key):
        signature = (tuple(q.shape), tuple(k.shape), tuple(v.shape), str(q.dtype), str(q.device),
                     torch.is_grad_enabled(), q.requires_grad, k.requires_grad, v.requires_grad,
                     tuple(factor.shape), str(factor.dtype), factor.requires_grad, tuple(dim_groups.shape))
        entries = self._entries.setdefault(cache_key, [])
        prepared = next((p for s, p in entries if s == signature), None)
        if prepared is None:
            prepared = prepare_grouped_hd_block_gemm(q, k, v, dim_groups, factor, kernel_eps=self.kernel_eps,
                                                     precision=self.precision, output_layout=self.output_layout)
            entries.append((signature, prepared))
            if len(entries) > 2:
                del entries[0]
        return run_prepared_grouped_hd_block_gemm(prepared, q, k, v, factor)


class LoRALinear(nn.Module):
    """Frozen base weight plus a trainable rank-``r`` update scaled by ``alpha / r``."""

    def __init__(self, in_features: int, out_features: int, *, rank: int, alpha: float, bias: bool, dtype, device=None):
        super().__init__()
        self.base = nn.Linear(in_features, out_features, bias=bias, dtype=dtype, device=device)
        for p in self.base.parameters():
            p.requires_grad_(False)
        self.lora_a = nn.Parameter(torch.empty(rank, in_features, dtype=dtype, device=device))
        self.lora_b = nn.Parameter(torch.zeros(out_features, rank, dtype=dtype, device=device))
        nn.init.kaiming_uniform_(self.lora_a, a=math.sqrt(5))
        self.scaling = alpha / rank

    def forward(self, x):
        return self.base(x) + (x @ self.lora_a.t()) @ self.lora_b.t() * self.scaling


class OalAttentionLayer(nn.Module):
    """Attention block of one layer with the grouped-quadratic operator in place of softmax attention.

    ``dim_groups`` int32 ``[Hq, 64]`` is fixed; ``factor`` fp32 ``[Hq, P]`` (packed lower-triangular
    factor of the PSD coefficient matrix) is trained together with the LoRA matrices.
    """

    def __init__(self, layer_id: int, dim_groups: torch.Tensor, factor: torch.Tensor, *, cache: PreparedCallCache,
                 geometry: ModelGeometry = QWEN_GEOMETRY, lora_rank: int = 16, lora_alpha: float = 32.0,
                 dtype=torch.bfloat16, device=None):
        super().__init__()
        g = geometry
        kv = g.num_kv_heads * g.head_dim
        mk = lambda i, o, bias: LoRALinear(i, o, rank=lora_rank, alpha=lora_alpha, bias=bias, dtype=dtype, device=device)
        self.q_proj, self.k_proj, self.v_proj = mk(g.hidden_size, g.hidden_size, True), mk(g.hidden_size, kv, True), mk(g.hidden_size, kv, True)
        self.o_proj = mk(g.hidden_size, g.hidden_size, False)
        self.register_buffer("dim_groups", dim_groups.to(torch.int32), persistent=True)
        self.factor = nn.Parameter(factor.to(torch.float32))
        self.layer_id, self.geometry, self.cache = layer_id, g, cache

    def forward(self, hidden_states, position_embeddings):
        q, k, v = project_qkv_and_apply_rope(q_proj=self.q_proj, k_proj=self.k_proj, v_proj=self.v_proj,
                                             hidden_states=hidden_states, position_embeddings=position_embeddings,
                                             geometry=self.geometry)
        out, _, _ = self.cache.grouped(q, k, v, self.dim_groups, self.factor, cache_key=self.layer_id)
        if self.cache.output_layout == "tokens_first":       # the kernels wrote [B, N, Hq, D]: no restore copy
            return project_token_major_output(token_output=out, o_proj=self.o_proj, geometry=self.geometry)
        return restore_and_project_output(head_output=out, o_proj=self.o_proj, geometry=self.geometry)
