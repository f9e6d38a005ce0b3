"""autograd boundary of the operator.

Counterpart of the reference's ``_HDParallelBlockGemmFunction``
(oal_attention/hd_block_gemm_autograd.py:85-204): three differentiable outputs
``(out, numerator, denominator)``, first-order backward only, gradients returned
in the input dtypes, the plan's gradient mask must equal ``needs_input_grad``.
The tensor inputs are the group-aware coefficients ``A [Hq]``, ``B [Hq,G]``,
``C [Hq,G,G]`` (what the sibling Function of the reference takes,
oal_attention/triton/grouped_quadratic_backward.py:136-151): with the groups
known, the kernels can form the intra-chunk weights from G small dot products.
The expansion factor -> (A, B, C) stays ordinary differentiable torch code in
the adapters, as in the reference (hd_block_gemm_adapters.py:278-301).
"""

from __future__ import annotations

import ctypes
import itertools
import threading
from dataclasses import dataclass
from typing import Any

import torch
import torch.nn.functional as F

from . import _lib
from .hd_block_gemm import HDParallelBlockPlan, make_problem

_DENOMINATOR_ERROR = "HD Block-GEMM denominator must be finite and strictly positive"


@dataclass(frozen=True)
class GroupTables:
    """Device-resident description of the dimension groups of every query head."""

    dim_perm: torch.Tensor      # int32 [Hq, 64]: dims sorted by group id (padded dims first, group 0)
    group_start: torch.Tensor   # int32 [Hq, 17]: group g owns dim_perm[h, start[g]:start[g+1]]
    group_count: int            # G = extent of B / C


def build_group_tables(groups: torch.Tensor, group_count: int) -> GroupTables:
    """``groups`` int [Hq, D] (D <= 64) -> sorted permutation + offsets on the same device."""
    hq, d = groups.shape
    g64 = groups.to(torch.int64)
    if d < _lib.HEAD_DIM:
        g64 = F.pad(g64, (0, _lib.HEAD_DIM - d), value=0)
    perm = torch.argsort(g64, dim=1, stable=True).to(torch.int32)
    counts = torch.zeros(hq, _lib.MAX_GROUPS, dtype=torch.int64, device=groups.device)
    counts.scatter_add_(1, g64, torch.ones_like(g64))
    start = torch.zeros(hq, _lib.MAX_GROUPS + 1, dtype=torch.int64, device=groups.device)
    start[:, 1:] = counts.cumsum(1)
    return GroupTables(perm.contiguous(), start.to(torch.int32).contiguous(), int(group_count))


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    """The device's current stream as a raw handle (the accessor without the Stream object when torch has it:
    this runs four times per training step on the host's critical path)."""
    if _RAW_STREAM is not None and device.index is not None:
        return ctypes.c_void_p(_RAW_STREAM(device.index))
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _grad_bits(mask) -> int:
    bits = 0
    if mask[0]:
        bits |= _lib.GRAD_Q
    if mask[1]:
        bits |= _lib.GRAD_K
    if mask[2]:
        bits |= _lib.GRAD_V
    if any(mask[3:]):
        bits |= _lib.GRAD_COEF
    return bits


def _pad_last(t: torch.Tensor) -> torch.Tensor:
    d = t.shape[-1]
    return t if d == _lib.HEAD_DIM else F.pad(t, (0, _lib.HEAD_DIM - d)).contiguous()


def _raise_for_bits(bits: int, where: str = "") -> None:
    if bits & _lib.STATUS_WAIT_TIMEOUT:
        raise RuntimeError(f"oal_b200 kernel gave up on a bounded wait (device status word {bits:#x}){where}")
    if bits & _lib.STATUS_BAD_LAYOUT:
        raise ValueError(f"a head's group layout does not fit the kernels{where}")
    if bits & (_lib.STATUS_NONFINITE | _lib.STATUS_DENOMINATOR):
        raise RuntimeError(f"{_DENOMINATOR_ERROR} (device status {bits}){where}")


def raise_on_status(status: torch.Tensor) -> None:
    """One host synchronisation at the point where the reference synchronises
    (oal_attention/hd_block_gemm_runtime.py:392-408)."""
    _raise_for_bits(int(status.item()))


# Deferred status words.  The reference synchronises after every forward because "a device-side
# assertion can poison a CUDA context ... until a safe asynchronous status mechanism is available"
# (hd_block_gemm_runtime.py:395-398).  The status word is that mechanism: when autograd will run a
# backward anyway, the forward only queues an asynchronous copy of its status word to pinned host
# memory (``oal_status_defer``: a ring of pinned words and a copy stream inside the library) and keeps the
# ticket.  The backward of the same call looks at exactly that ticket before it launches anything --
# without waiting: the host normally runs ahead of the GPU, and a wait here would serialise host and
# device in every step (measured: it costs the whole forward time per step and stalls input pipelines).
# A ticket that is not finished yet stays on a per-device list that every later entry into the library
# drains without blocking; ``check_pending_status(block=True)`` drains it completely and is the call to
# make before an optimizer step consumes the gradients.  Every error names the call it belongs to.
_PENDING: dict = {}
_PENDING_LOCK = threading.Lock()
_CALL_IDS = itertools.count(1)
_PENDING_LIMIT = 256          # a ticket stays valid for 1023 later ones on its device: drain well before that


@dataclass
class PendingStatus:
    ticket: int
    call_id: int
    what: str
    done: bool = False
    device_word: torch.Tensor | None = None     # kept alive until the copy has run

    def check(self, block: bool) -> bool:
        """Raise if the word reports a problem; returns False when it is not yet known (non-blocking)."""
        if self.done:
            return True
        value = ctypes.c_int32(0)
        rc = _lib.load().oal_status_poll(self.ticket, 1 if block else 0, ctypes.byref(value))
        if rc == 0:
            return False
        self.done = True
        self.device_word = None
        _lib.check(rc)
        _raise_for_bits(int(value.value), f" [{self.what}, call {self.call_id}]")
        return True


# Status words of calls that were recorded into a CUDA graph: nothing may be polled or copied to the host
# while a stream is capturing, and a replay runs no Python, so these words stay on the device (they live
# in the graph's memory pool and are rewritten by every replay) until check_captured_status() reads them.
_CAPTURED: dict = {}


def check_captured_status(device=None) -> None:
    """One host synchronisation: raise if any call recorded into a CUDA graph on ``device`` (default: every
    device) reported a problem in the replays so far.  Call it where a training loop synchronises anyway."""
    with _PENDING_LOCK:
        keys = list(_CAPTURED) if device is None else [torch.device(device).index if not isinstance(device, int) else device]
        words = [(w, what) for key in keys for w, what in _CAPTURED.get(key, [])]
    if not words:
        return
    values = torch.stack([w.reshape(()) for w, _ in words]).cpu().tolist()
    for bits, (_, what) in zip(values, words):
        _raise_for_bits(int(bits), f" [{what}, recorded in a CUDA graph]")


def forget_captured_status(device=None) -> None:
    """Drop the recorded words (when the graphs that own them are destroyed)."""
    with _PENDING_LOCK:
        if device is None:
            _CAPTURED.clear()
        else:
            _CAPTURED.pop(torch.device(device).index if not isinstance(device, int) else device, None)


def defer_status(status: torch.Tensor, what: str = "forward", *, guarded: bool = False) -> "PendingStatus | None":
    """Queue the copy of a call's status word to pinned host memory; returns the entry that owns the ticket.

    The copy runs on a stream of the library's own, never on the caller's: the device runs all
    device-to-host copies of a process through one copy queue, so a 4-byte copy on the compute stream
    waits behind whatever large result copy the application has in flight on another stream, and the
    kernels after it wait too (measured: 0.6 ms per step beside a 64 MB result copy).  ``guarded``: the
    caller already holds the device guard of ``status``."""
    device = status.device
    if torch.cuda.is_current_stream_capturing():
        with _PENDING_LOCK:
            _CAPTURED.setdefault(device.index, []).append((status, what))
        return None
    ticket = ctypes.c_int64(0)
    lib = _lib.load()
    if guarded:
        rc = lib.oal_status_defer(_lib.ptr(status), _stream_ptr(device), ctypes.byref(ticket))
    else:
        with _lib.device_guard(status):
            rc = lib.oal_status_defer(_lib.ptr(status), _stream_ptr(device), ctypes.byref(ticket))
    _lib.check(rc)
    entry = PendingStatus(int(ticket.value), next(_CALL_IDS), what, device_word=status)
    with _PENDING_LOCK:
        queue = _PENDING.setdefault(device.index, [])
        queue.append(entry)
        overfull = len(queue) > _PENDING_LIMIT
    if overfull:
        check_pending_status(block=True, device=device)
    return entry


def check_pending_status(block: bool = False, device=None) -> None:
    """Raise for any finished call whose device status word reported a problem.

    ``device``: a torch device / index, or None for every device.  With ``block`` the queues are
    drained completely (call it before an optimizer step when a forward ran without its backward)."""
    if torch.cuda.is_current_stream_capturing():
        return                  # no event may be queried while a stream is capturing
    with _PENDING_LOCK:
        keys = list(_PENDING) if device is None else [torch.device(device).index if not isinstance(device, int) else device]
    for key in keys:
        while True:
            with _PENDING_LOCK:
                queue = _PENDING.get(key) or []
                entry = queue[0] if queue else None
            if entry is None:
                break
            try:
                finished = entry.check(block)
            except Exception:
                with _PENDING_LOCK:
                    if queue and queue[0] is entry:
                        queue.pop(0)
                raise
            if not finished:
                break
            with _PENDING_LOCK:
                if queue and queue[0] is entry:
                    queue.pop(0)


def forward_impl(q, k, v, a, b, c, tables: GroupTables, scale: float, floor: float,
                 plan: HDParallelBlockPlan, *, state_in=None, check=True, workspace=None, reuse_state_stage=False,
                 out_token_major=False):
    """Launch the forward kernels.  Returns (out, num, den[B,Hq,N,1], saved_state, padded q,k,v).

    ``check``: True = synchronise and raise on the status word now; "defer" = queue it (the queued
    entry is left in ``forward_impl.last_pending`` for the caller that owns the backward).
    ``workspace`` / ``reuse_state_stage``: sequence parallelism passes the workspace in which
    ``oal_forward_local_state`` has just left the chunk-state increments of this very call.
    ``out_token_major``: ``out`` comes back as ``[B, N, Hq, 64]`` (what the output projection reads)."""
    if q.device.type != "cuda":
        raise RuntimeError("oal_b200 runs on CUDA tensors only (there is no CPU path)")
    check_pending_status(device=q.device)
    lib = _lib.load()
    B, Hq, Hkv, N, D, Dv = plan.geometry
    qp, kp, vp = _pad_last(q), _pad_last(k), _pad_last(v)
    out_dtype = getattr(torch, plan.output_dtype)
    kernel_out = out_dtype if out_dtype != torch.float64 else torch.float32
    dev = q.device
    problem = make_problem(plan.geometry, groups=tables.group_count, io_dtype=q.dtype, out_dtype=kernel_out,
                           precision=plan.precision, chunk=plan.chunk_tokens, scale=float(scale),
                           floor=float(floor), grad_mask=_lib.GRAD_REUSE_STATE_STAGE if reuse_state_stage else 0,
                           flags=_lib.FLAG_OUT_TOKEN_MAJOR if out_token_major else 0)
    if out_token_major and Dv != _lib.HEAD_DIM:
        raise ValueError("the token-major output layout needs value_dimension == 64")
    out = torch.empty((B, N, Hq, _lib.HEAD_DIM) if out_token_major else (B, Hq, N, _lib.HEAD_DIM),
                      dtype=kernel_out, device=dev)
    num = torch.empty(B, Hq, N, _lib.HEAD_DIM, dtype=torch.float32, device=dev)
    den = torch.empty(B, Hq, N, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ws = workspace if workspace is not None else torch.empty(max(plan.forward_workspace_bytes, 16),
                                                             dtype=torch.uint8, device=dev)
    saved = (torch.empty(plan.saved_state_bytes, dtype=torch.uint8, device=dev)
             if plan.saved_state_bytes else None)
    a32, b32, c32 = (t.detach().to(torch.float32).contiguous() for t in (a, b, c))
    with _lib.device_guard(qp):
        rc = lib.oal_forward(ctypes.byref(problem), _lib.ptr(qp), _lib.ptr(kp), _lib.ptr(vp),
                             _lib.ptr(tables.dim_perm), _lib.ptr(tables.group_start), _lib.ptr(a32),
                             _lib.ptr(b32), _lib.ptr(c32), _lib.ptr(out), _lib.ptr(num), _lib.ptr(den),
                             _lib.ptr(saved), _lib.ptr(state_in), _lib.ptr(ws), ws.numel(), _lib.ptr(status),
                             _stream_ptr(dev))
        _lib.check(rc)
        forward_impl.last_pending = defer_status(status, "forward", guarded=True) if check == "defer" else None
    if check and check != "defer":
        if torch.cuda.is_current_stream_capturing():
            defer_status(status, "forward")          # recorded: read by check_captured_status()
        else:
            raise_on_status(status)
    if Dv != _lib.HEAD_DIM:
        out, num = out[..., :Dv].contiguous(), num[..., :Dv].contiguous()
    if out_dtype != kernel_out:
        out = out.to(out_dtype)
    return out, num, den.view(B, Hq, N, 1), saved, (qp, kp, vp, a32, b32, c32)


def backward_operands(plan: HDParallelBlockPlan, num, den, grad_out, grad_num, grad_den):
    """Kernel-side dtype of out and the padded, contiguous (num, den, grad_out, grad_num, grad_den)
    the backward entry points read: every [.., Dv] tensor is zero-padded to 64 columns."""
    out_dtype = getattr(torch, plan.output_dtype)
    kernel_out = out_dtype if out_dtype != torch.float64 else torch.float32

    def prep(gt, dtype, width):
        if gt is None:
            return None
        gt = gt.to(dtype)
        if gt.shape[-1] != width and width == _lib.HEAD_DIM:
            gt = F.pad(gt, (0, width - gt.shape[-1]))
        return gt.contiguous()

    return (kernel_out, prep(num, torch.float32, _lib.HEAD_DIM), den.contiguous(),
            prep(grad_out, kernel_out, _lib.HEAD_DIM), prep(grad_num, torch.float32, _lib.HEAD_DIM),
            prep(grad_den, torch.float32, 1))


def backward_impl(saved_inputs, num, den, saved_state, tables: GroupTables, scale, floor,
                  plan: HDParallelBlockPlan, mask, grad_out, grad_num, grad_den, *, dstate_in=None,
                  workspace=None, reuse_state_stage=False, forward_status: "PendingStatus | None" = None,
                  out_token_major=False):
    """Launch the backward kernels; returns (dq, dk, dv, dA, dB, dC) with None where not requested.

    ``workspace`` / ``reuse_state_stage``: sequence parallelism passes the workspace that
    ``oal_backward_local_state`` has just filled so that stage is not computed twice."""
    lib = _lib.load()
    qp, kp, vp, a32, b32, c32 = saved_inputs
    B, Hq, Hkv, N, D, Dv = plan.geometry
    dev = qp.device
    if forward_status is not None and not torch.cuda.is_current_stream_capturing():
        forward_status.check(block=False)      # this call's own forward, if it has finished: raise before launching
    check_pending_status(device=dev)
    kernel_out, num_p, den_c, go, gn, gd = backward_operands(plan, num, den, grad_out, grad_num, grad_den)
    bits = _grad_bits(mask)
    problem = make_problem(plan.geometry, groups=tables.group_count, io_dtype=qp.dtype, out_dtype=kernel_out,
                           precision=plan.precision, chunk=plan.chunk_tokens, scale=float(scale),
                           floor=float(floor),
                           grad_mask=bits | (_lib.GRAD_REUSE_STATE_STAGE if reuse_state_stage else 0),
                           flags=_lib.FLAG_OUT_TOKEN_MAJOR if out_token_major else 0)
    G = tables.group_count
    dq = torch.empty_like(qp) if bits & _lib.GRAD_Q else None
    dk = torch.empty_like(kp) if bits & _lib.GRAD_K else None
    dv = torch.empty_like(vp) if bits & _lib.GRAD_V else None
    dA = torch.empty(Hq, dtype=torch.float32, device=dev) if bits & _lib.GRAD_COEF else None
    dB = torch.empty(Hq, G, dtype=torch.float32, device=dev) if bits & _lib.GRAD_COEF else None
    dC = torch.empty(Hq, G, G, dtype=torch.float32, device=dev) if bits & _lib.GRAD_COEF else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ws = workspace if workspace is not None else torch.empty(max(plan.backward_workspace_bytes, 16),
                                                             dtype=torch.uint8, device=dev)
    with _lib.device_guard(qp):
        rc = lib.oal_backward(ctypes.byref(problem), _lib.ptr(qp), _lib.ptr(kp), _lib.ptr(vp),
                              _lib.ptr(tables.dim_perm), _lib.ptr(tables.group_start), _lib.ptr(a32),
                              _lib.ptr(b32), _lib.ptr(c32), _lib.ptr(num_p), _lib.ptr(den_c),
                              _lib.ptr(saved_state), _lib.ptr(go), _lib.ptr(gn), _lib.ptr(gd), _lib.ptr(dq),
                              _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(dA), _lib.ptr(dB), _lib.ptr(dC),
                              _lib.ptr(dstate_in), _lib.ptr(ws), ws.numel(), _lib.ptr(status), _stream_ptr(dev))
        _lib.check(rc)
        if plan.precision == "bf16_tensorcore":
            defer_status(status, "backward", guarded=True)    # only a bounded wait that gave up can set it here
    if D != _lib.HEAD_DIM:
        dq = None if dq is None else dq[..., :D].contiguous()
        dk = None if dk is None else dk[..., :D].contiguous()
    if Dv != _lib.HEAD_DIM:
        dv = None if dv is None else dv[..., :Dv].contiguous()
    return dq, dk, dv, dA, dB, dC


class _HDParallelBlockGemmFunction(torch.autograd.Function):
    """Planned forward + analytic first-order backward on the CUDA kernels."""

    @staticmethod
    def forward(ctx: Any, q, k, v, a, b, c, tables: GroupTables, scale: float, eps: float,
                plan: HDParallelBlockPlan, out_token_major: bool = False):
        mask = tuple(bool(x) for x in ctx.needs_input_grad[:6])
        if plan.requested_gradient_mask != mask:
            raise ValueError("plan gradient mask must exactly match the six tensor inputs")
        ctx.set_materialize_grads(False)
        out, num, den, saved_state, padded = forward_impl(q, k, v, a, b, c, tables, scale, eps, plan,
                                                          check="defer" if any(mask) else True,
                                                          out_token_major=out_token_major)
        ctx.forward_status = forward_impl.last_pending
        ctx.out_token_major = out_token_major
        ctx.tables, ctx.scale, ctx.eps, ctx.plan, ctx.mask = tables, float(scale), float(eps), plan, mask
        ctx.input_dtypes = tuple(t.dtype for t in (q, k, v, a, b, c))
        ctx.has_state = saved_state is not None
        if any(mask):
            tensors = list(padded) + [num, den]
            if saved_state is not None:
                tensors.append(saved_state)
            ctx.save_for_backward(*tensors)
        return out, num, den

    @staticmethod
    def backward(ctx: Any, grad_output, grad_numerator, grad_denominator):
        if torch.is_grad_enabled():
            raise RuntimeError("HD Block-GEMM does not support double backward")
        saved = ctx.saved_tensors
        padded, num, den = saved[:6], saved[6], saved[7]
        state = saved[8] if ctx.has_state else None
        mask = ctx.mask
        if grad_output is None and grad_numerator is None and grad_denominator is None:
            return (None,) * 11
        dq, dk, dv, dA, dB, dC = backward_impl(padded, num, den, state, ctx.tables, ctx.scale, ctx.eps,
                                               ctx.plan, mask, grad_output, grad_numerator,
                                               grad_denominator, forward_status=ctx.forward_status,
                                               out_token_major=ctx.out_token_major)
        grads = [dq, dk, dv, dA, dB, dC]
        result = []
        for requested, g, dtype in zip(mask, grads, ctx.input_dtypes):
            if not requested:
                result.append(None)
            elif g is None:
                raise RuntimeError("requested HD Block-GEMM gradient was not produced")
            else:
                result.append(g.to(dtype))
        return (*result, None, None, None, None, None)


def hd_parallel_block_gemm(q, k, v, a, b, c, *, tables, scale, eps, plan, out_token_major=False):
    """Forward only (no autograd graph), same return triple."""
    out, num, den, _, _ = forward_impl(q, k, v, a, b, c, tables, scale, eps, plan, out_token_major=out_token_major)
    return out, num, den


def hd_parallel_block_gemm_autograd(q, k, v, a, b, c, *, tables, scale, eps, plan, out_token_major=False):
    return _HDParallelBlockGemmFunction.apply(q, k, v, a, b, c, tables, scale, eps, plan, out_token_major)
