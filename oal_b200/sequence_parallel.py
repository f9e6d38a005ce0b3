"""Sequence-parallel causal attention: every rank owns a contiguous token range.

The reference is single-GPU; long sequences only ever meet its chunk scan
(oal_attention/hd_block_gemm_runtime.py:313-320).  Here the same scan is cut across
ranks: a rank first computes the sum of its own chunk-state increments, the ranks
exchange those sums with ONE all-gather (NCCL over NVLink on GPUs, gloo in the CPU
tests of the host logic), each rank adds up the contributions of the ranks before
it and scans its range starting from that state.  The backward mirrors it with the
state gradient and the ranks after it.  The exchanged tensor always lands in local
memory before a kernel reads it; no kernel touches a peer's memory.

Coefficient gradients (dA, dB, dC and hence d factor) are sums over tokens, so each
rank holds a partial sum; ``reduce_coefficient_grads=True`` all-reduces them inside
the backward so every rank sees the full gradient.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from . import _lib
from .grouped_quadratic import _expand_factor_coefficients
from .hd_block_gemm import make_problem
from .hd_block_gemm_adapters import _PreparedGroupedHdBlockGemm, prepare_grouped_hd_block_gemm
from .hd_block_gemm_autograd import (
    _grad_bits,
    _pad_last,
    _stream_ptr,
    backward_impl,
    backward_operands,
    defer_status,
    forward_impl,
)


def exclusive_prefix_over_ranks(local: torch.Tensor, group=None, *, reverse: bool = False) -> torch.Tensor:
    """Sum of ``local`` over the ranks before this one (after this one when ``reverse``).

    One all-gather, then a local sum in rank order, so the result does not depend on the
    collective's reduction order and is identical on every run.
    """
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return torch.zeros_like(local)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    gathered = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    if local.is_cuda:
        dist.all_gather_into_tensor(gathered, local.contiguous(), group=group)   # one NCCL call, no copy-out
    else:
        dist.all_gather(list(gathered.unbind(0)), local.contiguous(), group=group)
    part = gathered[rank + 1:] if reverse else gathered[:rank]
    if part.shape[0] == 0:
        return torch.zeros_like(local)
    total = part[0].clone()
    for r in range(1, part.shape[0]):       # fixed order: rank r, then r + 1, ...
        total += part[r]
    return total


def local_state_total(k: torch.Tensor, v: torch.Tensor, plan, groups: int = 1, workspace=None) -> torch.Tensor:
    """fp32 ``[B*Hkv, 2432, 80]``: this rank's contribution to the running state.  With ``workspace``
    (``plan.forward_workspace_bytes`` bytes) the chunk-state increments stay there for the forward."""
    lib = _lib.load()
    B, Hq, Hkv, N, D, Dv = plan.geometry
    kp, vp = _pad_last(k), _pad_last(v)
    problem = make_problem(plan.geometry, groups=groups, io_dtype=k.dtype, out_dtype=k.dtype,
                           precision=plan.precision, chunk=plan.chunk_tokens, scale=1.0, floor=1e-38)
    total = torch.empty(B * Hkv, _lib.STATE_ROWS, _lib.E_PAD, dtype=torch.float32, device=k.device)
    ws = workspace if workspace is not None else torch.empty(max(_lib.workspace_bytes(problem, 0), 16),
                                                             dtype=torch.uint8, device=k.device)
    status = torch.zeros(1, dtype=torch.int32, device=k.device)
    with _lib.device_guard(kp):
        rc = lib.oal_forward_local_state(ctypes.byref(problem), _lib.ptr(kp), _lib.ptr(vp), _lib.ptr(total),
                                         _lib.ptr(ws), ws.numel(), _lib.ptr(status), _stream_ptr(k.device))
    _lib.check(rc)
    defer_status(status, "forward state stage")      # a bounded wait that gave up in state_update
    return total


def local_dstate_total(saved_inputs, num, den, saved_state, tables, scale, floor, plan, mask, grad_out,
                       grad_num, grad_den, workspace):
    """Stage A of the backward into ``workspace``; returns this rank's state-gradient sum."""
    lib = _lib.load()
    qp, kp, vp, a32, b32, c32 = saved_inputs
    B, Hq, Hkv, N, D, Dv = plan.geometry
    # the same padded operands and kernel-side output dtype as the backward proper: the stage it leaves in
    # the workspace is reused there
    kernel_out, num_p, den_c, go, gn, gd = backward_operands(plan, num, den, grad_out, grad_num, grad_den)
    problem = make_problem(plan.geometry, groups=tables.group_count, io_dtype=qp.dtype, out_dtype=kernel_out,
                           precision=plan.precision, chunk=plan.chunk_tokens, scale=float(scale),
                           floor=float(floor), grad_mask=_grad_bits(mask))
    total = torch.empty(B * Hkv, _lib.STATE_ROWS, _lib.E_PAD, dtype=torch.float32, device=qp.device)
    status = torch.zeros(1, dtype=torch.int32, device=qp.device)
    with _lib.device_guard(qp):
        rc = lib.oal_backward_local_state(
            ctypes.byref(problem), _lib.ptr(qp), _lib.ptr(tables.dim_perm), _lib.ptr(tables.group_start),
            _lib.ptr(a32), _lib.ptr(b32), _lib.ptr(c32), _lib.ptr(num_p), _lib.ptr(den_c),
            _lib.ptr(saved_state), _lib.ptr(go), _lib.ptr(gn), _lib.ptr(gd), _lib.ptr(total), _lib.ptr(workspace),
            workspace.numel(), _lib.ptr(status), _stream_ptr(qp.device))
    _lib.check(rc)
    defer_status(status, "backward state stage")     # a bounded wait that gave up in dstate_heads
    return total


class _SequenceParallelFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, q, k, v, a, b, c, prepared: _PreparedGroupedHdBlockGemm, group, reduce_coef: bool):
        plan = prepared.plan
        mask = tuple(bool(x) for x in ctx.needs_input_grad[:6])
        ctx.set_materialize_grads(False)
        ws = torch.empty(max(plan.forward_workspace_bytes, 16), dtype=torch.uint8, device=q.device)
        state_in = exclusive_prefix_over_ranks(local_state_total(k, v, plan, prepared.gmax, workspace=ws), group)
        out, num, den, saved_state, padded = forward_impl(q, k, v, a, b, c, prepared.tables, prepared.scale,
                                                          prepared.normalization_floor, plan, state_in=state_in,
                                                          check="defer" if any(mask) else True, workspace=ws,
                                                          reuse_state_stage=True)
        ctx.forward_status = forward_impl.last_pending
        ctx.prepared, ctx.group, ctx.mask, ctx.reduce_coef = prepared, group, mask, reduce_coef
        ctx.input_dtypes = tuple(t.dtype for t in (q, k, v, a, b, c))
        if any(mask):
            ctx.save_for_backward(*padded, num, den, saved_state)
        return out, num, den

    @staticmethod
    def backward(ctx: Any, grad_output, grad_numerator, grad_denominator):
        if torch.is_grad_enabled():
            raise RuntimeError("HD Block-GEMM does not support double backward")
        saved = ctx.saved_tensors
        padded, num, den, state = saved[:6], saved[6], saved[7], saved[8]
        prepared, plan, mask = ctx.prepared, ctx.prepared.plan, ctx.mask
        if grad_output is None and grad_numerator is None and grad_denominator is None:
            return (None,) * 9
        if ctx.forward_status is not None:
            if not torch.cuda.is_current_stream_capturing():
                ctx.forward_status.check(block=False)    # this call's own forward, if it has finished
        ws = torch.empty(max(plan.backward_workspace_bytes, 16), dtype=torch.uint8, device=num.device)
        local = local_dstate_total(padded, num, den, state, prepared.tables, prepared.scale,
                                   prepared.normalization_floor, plan, mask, grad_output, grad_numerator,
                                   grad_denominator, ws)
        dstate_in = exclusive_prefix_over_ranks(local, ctx.group, reverse=True)
        grads = list(backward_impl(padded, num, den, state, prepared.tables, prepared.scale,
                                   prepared.normalization_floor, plan, mask, grad_output, grad_numerator,
                                   grad_denominator, dstate_in=dstate_in, workspace=ws, reuse_state_stage=True,
                                   forward_status=ctx.forward_status))
        if ctx.reduce_coef and dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            for g in grads[3:]:
                if g is not None:
                    dist.all_reduce(g, group=ctx.group)
        result = [None if (not want or g is None) else g.to(dt)
                  for want, g, dt in zip(mask, grads, ctx.input_dtypes)]
        return (*result, None, None, None)


def sequence_parallel_attention(q, k, v, dim_groups, factor, *, group=None, scale=None, kernel_eps=1e-6,
                                reduce_coefficient_grads: bool = True, prepared=None):
    """Causal grouped-quadratic attention over a sequence split across the ranks of ``group``.

    ``q, k, v`` hold this rank's contiguous token range (ranges are ordered by rank);
    returns this range's ``(out, numerator, denominator)``.  bf16 tensors on CUDA only.
    """
    if prepared is None:
        prepared = prepare_grouped_hd_block_gemm(q, k, v, dim_groups, factor, scale=scale, kernel_eps=kernel_eps,
                                                 precision="bf16_tensorcore")
    plan = prepared.plan
    a, b, c = _expand_factor_coefficients(factor, query_heads=plan.query_heads, gmax=prepared.gmax,
                                          kernel_eps=prepared.kernel_eps, working_dtype=torch.float32)
    return _SequenceParallelFunction.apply(q, k, v, a.contiguous(), b.contiguous(), c.contiguous(), prepared,
                                           group, reduce_coefficient_grads)
