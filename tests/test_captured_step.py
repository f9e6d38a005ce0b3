"""A forward + backward recorded into a CUDA graph gives the bits of the eager calls."""

import pytest
import torch

import oal_b200
from oal_b200 import synthetic
from oal_b200.captured_step import CapturedStep

pytestmark = pytest.mark.gpu


def _eager(prepared, q, k, v, factor, dout):
    q, k, v = (t.detach().clone().requires_grad_() for t in (q, k, v))
    factor = factor.detach().clone().requires_grad_()
    out, _, _ = oal_b200.run_prepared_grouped_hd_block_gemm(prepared, q, k, v, factor)
    out.backward(dout)
    return out.detach(), q.grad, k.grad, v.grad, factor.grad


def test_replay_matches_eager_calls_on_old_and_new_inputs():
    dev = torch.device("cuda")
    cases = [synthetic.qwen_head_case(s, batch=1, n=700, hq=14, hkv=2, g=8, bf16=True) for s in (51, 52)]
    first = cases[0]
    tensors = [[getattr(c, a).to(dev, torch.bfloat16) for a in ("q", "k", "v", "grad_out")] for c in cases]
    factors = [c.factor.to(dev) for c in cases]
    q, k, v, dout = tensors[0]
    prepared = oal_b200.prepare_grouped_hd_block_gemm(
        q.clone().requires_grad_(), k.clone().requires_grad_(), v.clone().requires_grad_(), first.dim_groups.to(dev),
        factors[0].clone().requires_grad_(), scale=first.scale, kernel_eps=first.kernel_eps, precision="bf16_tensorcore")
    step = CapturedStep(prepared, q, k, v, factors[0], dout)
    for (q, k, v, dout), factor in zip(tensors, factors):        # same dim_groups: the second case only changes values
        want = _eager(prepared, q, k, v, factor, dout)
        got = step.replay(q, k, v, factor, dout)
        torch.cuda.synchronize()
        for name, x, y in zip(("out", "dq", "dk", "dv", "dfactor"), got, want):
            assert torch.equal(x, y), name
    step.check_status()
    oal_b200.hd_block_gemm_autograd.forget_captured_status()
