"""Seeded synthetic inputs for the OAL attention path.

The reference publishes no dataset for this path: its benchmark configurations
are shape + distribution descriptions (Qwen2.5-0.5B head geometry, a seeded
partition of the head dimension into groups, a few outlier channels, uniform
coefficients).  The generators below realise those descriptions with
``torch.Generator`` on the CPU so that every run, here or on another machine,
sees bit-identical inputs.  All tensors are returned on the CPU in fp32;
callers cast / move them.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class OalCase:
    """One problem instance: tensors plus the scalar options of the call."""

    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    dim_groups: torch.Tensor            # int32 [D] or [Hq, D]
    scale: float
    kernel_eps: float = 1e-6
    # exactly one of (factor) or (A, B, C) is set
    factor: torch.Tensor | None = None  # [P] or [Hq, P]
    A: torch.Tensor | None = None       # [Hq]
    B: torch.Tensor | None = None       # [Hq, G]
    C: torch.Tensor | None = None       # [Hq, G, G]
    grad_out: torch.Tensor | None = None
    grad_num: torch.Tensor | None = None
    grad_den: torch.Tensor | None = None
    meta: dict = field(default_factory=dict)


def partition_groups(d: int, sizes, gen: torch.Generator) -> tuple[torch.Tensor, torch.Tensor]:
    """Seeded permutation of the ``d`` dims cut into consecutive groups of ``sizes``.

    Returns (dim_groups int32 [d], permutation): group ``g`` holds the dims
    ``perm[offset_g : offset_g + sizes[g]]``.
    """
    assert sum(sizes) == d
    perm = torch.randperm(d, generator=gen)
    groups = torch.empty(d, dtype=torch.int32)
    off = 0
    for g, s in enumerate(sizes):
        groups[perm[off:off + s]] = g
        off += s
    return groups, perm


def _bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def config1_case(seed: int = 0, n: int = 256) -> OalCase:
    """B=1, Hq=Hkv=2, N=256, D=Dv=64, G=4 groups of 16, two outlier channels x10,
    directly specified coefficients ~U(0.1,1) with a symmetrised quadratic block.

    Such a quadratic block is not positive semi-definite, so the caller must
    check that every denominator is positive (tests advance the seed if not).
    """
    gen = torch.Generator().manual_seed(1000 + seed)
    hq, d = 2, 64
    groups, perm = partition_groups(d, [16, 16, 16, 16], gen)
    q = torch.randn(1, hq, n, d, generator=gen)
    k = torch.randn(1, hq, n, d, generator=gen)
    v = torch.randn(1, hq, n, d, generator=gen)
    out_ch = perm[:2]
    q[..., out_ch] *= 10.0
    k[..., out_ch] *= 10.0
    dout = torch.randn(1, hq, n, d, generator=gen)
    a = torch.rand(hq, generator=gen) * 0.9 + 0.1
    b = torch.rand(hq, 4, generator=gen) * 0.9 + 0.1
    u = torch.rand(hq, 4, 4, generator=gen) * 0.9 + 0.1
    c = 0.5 * (u + u.transpose(-1, -2))
    return OalCase(q, k, v, groups, scale=0.125, A=a, B=b, C=c, grad_out=dout,
                   meta=dict(name="config1", seed=seed))


QWEN_GROUP_SIZES = {
    1: [64],
    4: [16, 16, 16, 16],
    8: [2, 2, 4, 4, 8, 12, 16, 16],
    16: [4] * 16,
}


def qwen_head_case(seed: int = 0, *, batch: int = 4, n: int = 4096, hq: int = 14, hkv: int = 2,
                   g: int = 8, outlier_scale: float = 20.0, bf16: bool = True,
                   with_grad: bool = True) -> OalCase:
    """Qwen2.5-0.5B attention-layer shape (14 query / 2 KV heads, d=64).

    Groups: seeded partition with the sizes of ``QWEN_GROUP_SIZES[g]``; the four
    outlier channels are the first four dims of the permutation, i.e. they sit
    in the smallest groups, and are scaled by ``outlier_scale`` in q and k.
    Coefficients come from a seeded lower-triangular factor with U(0.1,1)
    entries (positive-definite kernel), one row per query head.  With ``bf16``
    the values of q, k, v and the upstream gradient are rounded to bf16 so that
    the oracle and the operator see the same numbers.
    """
    gen = torch.Generator().manual_seed(2000 + seed)
    d = 64
    sizes = QWEN_GROUP_SIZES[g]
    groups, perm = partition_groups(d, sizes, gen)
    q = torch.randn(batch, hq, n, d, generator=gen)
    k = torch.randn(batch, hkv, n, d, generator=gen)
    v = torch.randn(batch, hkv, n, d, generator=gen)
    out_ch = perm[:4]
    q[..., out_ch] *= outlier_scale
    k[..., out_ch] *= outlier_scale
    p = (g + 1) * (g + 2) // 2
    factor = torch.rand(hq, p, generator=gen) * 0.9 + 0.1
    dout = torch.randn(batch, hq, n, d, generator=gen) if with_grad else None
    if bf16:
        q, k, v = _bf16_round(q), _bf16_round(k), _bf16_round(v)
        if dout is not None:
            dout = _bf16_round(dout)
    return OalCase(q, k, v, groups, scale=d ** -0.5, kernel_eps=1e-6, factor=factor, grad_out=dout,
                   meta=dict(name=f"qwen_head_b{batch}_n{n}_g{g}", seed=seed))


def mixed_case(seed: int = 0, *, batch: int = 2, hq: int = 4, hkv: int = 2, n: int = 150, d: int = 64,
               dv: int = 64, gmax: int = 4, aux_grads: bool = True) -> OalCase:
    """Ragged N, GQA, per-head groups with different active group counts, and
    upstream gradients on all three outputs.  Heads use 1..gmax active groups;
    inactive factor entries are zero-padded the way the reference's parameter
    bank does it (active packing first, then zeros)."""
    gen = torch.Generator().manual_seed(3000 + seed)
    q = torch.randn(batch, hq, n, d, generator=gen)
    k = torch.randn(batch, hkv, n, d, generator=gen)
    v = torch.randn(batch, hkv, n, dv, generator=gen)
    groups = torch.zeros(hq, d, dtype=torch.int32)
    p = (gmax + 1) * (gmax + 2) // 2
    factor = torch.zeros(hq, p)
    for h in range(hq):
        active = 1 + (h % gmax)
        ids = torch.arange(d) % active
        groups[h] = ids[torch.randperm(d, generator=gen)].to(torch.int32)
        pa = (active + 1) * (active + 2) // 2
        factor[h, :pa] = torch.rand(pa, generator=gen) * 0.9 + 0.1
    case = OalCase(q, k, v, groups, scale=d ** -0.5, kernel_eps=1e-3, factor=factor,
                   grad_out=torch.randn(batch, hq, n, dv, generator=gen),
                   meta=dict(name=f"mixed_n{n}_d{d}", seed=seed))
    if aux_grads:
        case.grad_num = 0.1 * torch.randn(batch, hq, n, dv, generator=gen)
        case.grad_den = 0.1 * torch.randn(batch, hq, n, 1, generator=gen)
    return case


def tensor_digest(*tensors: torch.Tensor) -> str:
    """sha256 over the raw bytes of the tensors, to detect generator drift."""
    import hashlib

    h = hashlib.sha256()
    for t in tensors:
        h.update(t.detach().contiguous().cpu().numpy().tobytes())
    return h.hexdigest()
