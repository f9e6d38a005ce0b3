"""One forward + backward of a prepared call recorded into a CUDA graph.

The reference queues every stage from Python on each step.  At small problem sizes (one or two
(batch row, KV head) units per GPU, as in the fixed-size split over many GPUs or short sequences) the
host needs longer to queue the roughly thirty launches of a step than the GPU needs to run them.  A
CUDA graph replays the recorded launches -- including the library's forks onto its internal streams --
with one call.  Everything the recorded calls allocate lives in the graph's memory pool, so inputs are
copied into fixed tensors before a replay and results are read from fixed tensors after it.

Status words of recorded calls cannot be polled from a replay (no Python runs): they stay on the
device and ``check_status()`` reads them with one synchronisation."""

from __future__ import annotations

import torch

from .hd_block_gemm_adapters import run_prepared_grouped_hd_block_gemm
from .hd_block_gemm_autograd import check_captured_status


class CapturedStep:
    """``CapturedStep(prepared, q, k, v, factor, grad_out)`` records ``out = op(q, k, v, factor);
    out.backward(grad_out)``; ``replay(...)`` runs it again on new values of the same shapes.

    Attributes after construction (fixed tensors, rewritten by every replay): ``out``, ``numerator``,
    ``denominator``, ``grad_q``, ``grad_k``, ``grad_v``, ``grad_factor``."""

    def __init__(self, prepared, q, k, v, factor, grad_out, *, warmup: int = 3):
        if not q.is_cuda:
            raise RuntimeError("oal_b200 runs on CUDA tensors only (there is no CPU path)")
        device = q.device
        self.prepared = prepared
        self.q, self.k, self.v = (t.detach().clone().requires_grad_() for t in (q, k, v))
        self.factor = factor.detach().clone().requires_grad_()
        self.grad_out_in = grad_out.detach().clone()
        current = torch.cuda.current_stream(device)
        side = torch.cuda.Stream(device)
        side.wait_stream(current)
        with torch.cuda.stream(side):           # streams, events and kernel attributes are created here, not in the graph
            for _ in range(max(warmup, 1)):
                self._run()
        current.wait_stream(side)
        for leaf in (self.q, self.k, self.v, self.factor):
            leaf.grad = None
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out, self.numerator, self.denominator = self._run()
        self.grad_q, self.grad_k, self.grad_v, self.grad_factor = self.q.grad, self.k.grad, self.v.grad, self.factor.grad

    def _run(self):
        for leaf in (self.q, self.k, self.v, self.factor):
            leaf.grad = None
        out, num, den = run_prepared_grouped_hd_block_gemm(self.prepared, self.q, self.k, self.v, self.factor)
        out.backward(self.grad_out_in)
        return out, num, den

    def replay(self, q=None, k=None, v=None, factor=None, grad_out=None):
        """Copy the given tensors into the recorded inputs (None = keep the previous values) and replay.
        Returns ``(out, grad_q, grad_k, grad_v, grad_factor)``: the fixed tensors, valid until the next replay."""
        with torch.no_grad():
            for dst, src in ((self.q, q), (self.k, k), (self.v, v), (self.factor, factor), (self.grad_out_in, grad_out)):
                if src is not None:
                    dst.copy_(src)
        self.graph.replay()
        return self.out, self.grad_q, self.grad_k, self.grad_v, self.grad_factor

    def check_status(self) -> None:
        """Raise if a recorded call reported a non-finite / non-positive denominator or a wait that gave up."""
        check_captured_status(self.q.device)
