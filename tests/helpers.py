"""Helpers shared by the GPU parity tests: run an OalCase through the operator and
through the CPU oracle, and compare with the reference's normalized max error."""

from __future__ import annotations

import torch

from oal_b200 import synthetic
from oracle import oal_oracle as orc

ERR = orc.normalized_max_error


def coefficients(case, dtype=torch.float64):
    if case.factor is not None:
        return orc.expand_factor(case.factor, case.q.shape[1], case.kernel_eps, dtype)
    return case.A.to(dtype), case.B.to(dtype), case.C.to(dtype)


def oracle_dense(case):
    """fp64 dense statement + closed-form gradients on the CPU."""
    a, b, c = coefficients(case)
    d = lambda x: None if x is None else x.double()
    r = orc.dense_backward(case.q.double(), case.k.double(), case.v.double(), case.dim_groups, a, b, c,
                           scale=case.scale, grad_out=d(case.grad_out), grad_num=d(case.grad_num),
                           grad_den=d(case.grad_den))
    if case.factor is not None:
        factor = case.factor.double().clone().requires_grad_()
        fa, fb, fc = orc.expand_factor(factor, case.q.shape[1], case.kernel_eps)
        ((fa * r["dA"]).sum() + (fb * r["dB"]).sum() + (fc * r["dC"]).sum()).backward()
        r["dfactor"] = factor.grad
    return r


def run_operator(case, *, precision, io_dtype=torch.float32, device="cuda", need=("q", "k", "v", "coef"),
                 output_dtype=None):
    """Forward + backward through the public entry points; returns a dict of CPU tensors."""
    import oal_b200

    q, k, v = (t.to(device=device, dtype=io_dtype) for t in (case.q, case.k, case.v))
    q.requires_grad_("q" in need)
    k.requires_grad_("k" in need)
    v.requires_grad_("v" in need)
    groups = case.dim_groups.to(device)
    res = {}
    if case.factor is not None:
        factor = case.factor.to(device=device, dtype=torch.float32).requires_grad_("coef" in need)
        out, num, den = oal_b200.grouped_causal_attention(q, k, v, groups, factor, scale=case.scale,
                                                          kernel_eps=case.kernel_eps, precision=precision,
                                                          output_dtype=output_dtype)
        leaves = dict(dfactor=factor)
    else:
        a, b, c = (t.to(device=device, dtype=torch.float32).requires_grad_("coef" in need)
                   for t in (case.A, case.B, case.C))
        out, num, den = oal_b200.grouped_coefficient_attention(q, k, v, groups, a, b, c, scale=case.scale,
                                                               precision=precision,
                                                               output_dtype=output_dtype)
        leaves = dict(dA=a, dB=b, dC=c)
    res.update(out=out, num=num, den=den)
    if need and case.grad_out is not None:
        grads_out = [case.grad_out.to(device=device, dtype=out.dtype)]
        outs = [out]
        if case.grad_num is not None:
            outs.append(num)
            grads_out.append(case.grad_num.to(device))
        if case.grad_den is not None:
            outs.append(den)
            grads_out.append(case.grad_den.to(device))
        torch.autograd.backward(outs, grads_out)
        for name, leaf in dict(dq=q, dk=k, dv=v, **leaves).items():
            if leaf.grad is not None:
                res[name] = leaf.grad
    return {k_: v_.detach().float().cpu() for k_, v_ in res.items()}


def assert_close(res, ref, tol, keys=None, label=""):
    worst = {}
    for key in keys or [k for k in res if k in ref]:
        worst[key] = ERR(res[key], ref[key])
    bad = {k: v for k, v in worst.items() if not v <= tol}
    assert not bad, f"{label} normalized max error above {tol}: {bad} (all: {worst})"
    return worst
