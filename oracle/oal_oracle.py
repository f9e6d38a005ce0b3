"""CPU oracle for OAL's causal grouped-quadratic attention (TEST INFRASTRUCTURE ONLY).

This module is the checker, never the product: only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it.  The shipped
operator lives in ``oal_b200`` and runs hand-written CUDA; nothing in that
package imports this file and it has no CPU fallback.

Everything here is a restatement, in plain torch on the CPU, of the arithmetic
of the reference project (wuqianyue09/OAL).  Three independent statements of
the same function are kept so they can be checked against one another:

* ``dense_forward``      -- O(N^2) token-pair statement of the kernel
  ``w(i,j) = A + sum_g B_g s_g + sum_gg' C_gg' s_g s_g'`` with
  ``s_g = sum_{d in g} (scale q_i[d]) k_j[d]``.  It follows the independent
  dense statement the reference's own tests use
  (tests/operators/test_grouped_quadratic.py:31-84).
* ``state_forward``      -- the reference oracle's algorithm
  (oal_attention/grouped_reference.py:18-58 state build by cumulative sums,
  :61-99 coefficient selection, :102-178 numerator / denominator, :181-211
  normalisation and positivity check).
* ``chunked_forward_backward`` -- the chunked linear-attention form with an
  explicit analytic backward, following the reference's production path
  (oal_attention/hd_block_gemm_runtime.py:617-805 forward,
  oal_attention/hd_block_gemm_backward.py:191-308 normalisation VJP, :764-908
  dCarry and reverse scan, :1455-1992 per-block VJPs,
  oal_attention/hd_block_gemm_feature_backward.py:59-131,157-422 folds).
  This one has linear memory and is what the CPU baseline times.

Parity pinning: the functions are checked (tests/test_oracle.py) against the
two known-answer fixtures shipped by the reference
(tests/operators/fixtures/grouped_quadratic/*.json, re-emitted under
tests/golden/) and against golden vectors produced by importing the reference
package itself (tests/golden/make_golden.py).
"""

from __future__ import annotations

import math

import torch

# hd_block_gemm_adapters.py:24 -- the production path clamps the denominator at
# the smallest positive fp32 subnormal when normalising.
POSITIVE_FP32_FLOOR = float(torch.finfo(torch.float32).tiny * torch.finfo(torch.float32).eps)


# ---------------------------------------------------------------------------
# coefficients
# ---------------------------------------------------------------------------

def infer_gmax(parameter_count: int) -> int:
    """grouped_quadratic.py:59-73: P = (Gmax+1)(Gmax+2)/2."""
    disc = 1 + 8 * parameter_count
    root = math.isqrt(disc)
    if root * root != disc or (root - 1) % 2:
        raise ValueError("factor last dimension must be a valid packed lower-triangular size")
    gmax = (root - 1) // 2 - 1
    if gmax < 1:
        raise ValueError("factor must reserve at least one dimension group")
    return gmax


def expand_factor(factor: torch.Tensor, query_heads: int, kernel_eps: float,
                  dtype: torch.dtype = torch.float64):
    """Packed lower triangle L -> (A, B, C) with M = L L^T (grouped_quadratic.py:184-218).

    A = M00 + kernel_eps, B_g = 2 M_{0,g+1}, C_gg' = M_{g+1,g'+1}.
    """
    f = factor.to(dtype)
    if f.ndim == 1:
        f = f.unsqueeze(0)
    if f.shape[0] == 1:
        f = f.expand(query_heads, -1)
    gmax = infer_gmax(f.shape[-1])
    side = gmax + 1
    rows, cols = torch.tril_indices(side, side)
    lower = torch.zeros(query_heads, side, side, dtype=dtype)
    lower[:, rows, cols] = f
    m = lower @ lower.transpose(-1, -2)
    return m[:, 0, 0] + kernel_eps, 2.0 * m[:, 0, 1:], m[:, 1:, 1:].contiguous()


def _groups_per_head(dim_groups: torch.Tensor, query_heads: int) -> torch.Tensor:
    g = dim_groups.to(torch.int64)
    if g.ndim == 1:
        g = g.unsqueeze(0).expand(query_heads, -1)
    return g


# ---------------------------------------------------------------------------
# (1) dense O(N^2) statement
# ---------------------------------------------------------------------------

def dense_weights(q, k, dim_groups, A, B, C, *, scale: float):
    """Causal-masked kernel matrix w[b,h,i,j] and the per-group scores s[b,h,i,j,g]."""
    batch, hq, n, d = q.shape
    hkv = k.shape[1]
    groups = _groups_per_head(dim_groups, hq)
    gcount = B.shape[-1]
    onehot = torch.nn.functional.one_hot(groups, gcount).to(q.dtype)      # [Hq, D, G]
    kv_of = torch.arange(hq) // (hq // hkv)
    kq = k[:, kv_of]
    s = torch.einsum("bhid,bhjd,hdg->bhijg", q * scale, kq, onehot)
    w = (A[None, :, None, None]
         + torch.einsum("bhijg,hg->bhij", s, B)
         + torch.einsum("bhijg,hgf,bhijf->bhij", s, C, s))
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    return w * mask, s, mask


def dense_forward(q, k, v, dim_groups, A, B, C, *, scale: float):
    """(out, num, den) by explicit token pairs; differentiable torch code."""
    hq, hkv = q.shape[1], k.shape[1]
    w, _, _ = dense_weights(q, k, dim_groups, A, B, C, scale=scale)
    kv_of = torch.arange(hq) // (hq // hkv)
    num = w @ v[:, kv_of]
    den = w.sum(-1, keepdim=True)
    return num / den, num, den


def dense_backward(q, k, v, dim_groups, A, B, C, *, scale: float,
                   grad_out=None, grad_num=None, grad_den=None):
    """Closed-form first-order gradients of ``dense_forward`` (no autograd).

    dC is the symmetric closed form sum dW s_g s_g'.  The reference oracle's
    raw autograd gradient w.r.t. its ``quadratic_coefficients`` argument reads
    only C[g(r), g(c)] for r >= c (grouped_reference.py:86-98), so compare
    ``dC + dC^T`` (or the gradient w.r.t. ``factor``) against it.
    """
    batch, hq, n, d = q.shape
    hkv, dv = k.shape[1], v.shape[-1]
    rep = hq // hkv
    w, s, mask = dense_weights(q, k, dim_groups, A, B, C, scale=scale)
    kv_of = torch.arange(hq) // rep
    kq, vq = k[:, kv_of], v[:, kv_of]
    u = torch.cat([vq, torch.ones(batch, hq, n, 1, dtype=q.dtype)], -1)
    y = w @ u
    num, den = y[..., :dv], y[..., dv:]
    g = torch.zeros(batch, hq, n, dv + 1, dtype=q.dtype)
    if grad_out is not None:
        g[..., :dv] += grad_out / den
        g[..., dv:] += -(grad_out * num).sum(-1, keepdim=True) / den ** 2
    if grad_num is not None:
        g[..., :dv] += grad_num
    if grad_den is not None:
        g[..., dv:] += grad_den
    dW = (g @ u.transpose(-1, -2)) * mask
    dA = dW.sum((0, 2, 3))
    dB = torch.einsum("bhij,bhijg->hg", dW, s)
    dC = torch.einsum("bhij,bhijg,bhijf->hgf", dW, s, s)
    ds = dW[..., None] * (B[None, :, None, None, :] + 2 * torch.einsum("hgf,bhijf->bhijg", C, s))
    groups = _groups_per_head(dim_groups, hq)
    onehot = torch.nn.functional.one_hot(groups, B.shape[-1]).to(q.dtype)
    dsd = torch.einsum("bhijg,hdg->bhijd", ds, onehot)
    dq = scale * torch.einsum("bhijd,bhjd->bhid", dsd, kq)
    dk = torch.einsum("bhijd,bhid->bhjd", dsd, q * scale).view(batch, hkv, rep, n, d).sum(2)
    du = torch.einsum("bhij,bhie->bhje", w, g)
    dvv = du[..., :dv].reshape(batch, hkv, rep, n, dv).sum(2)
    return dict(out=num / den, num=num, den=den, dq=dq, dk=dk, dv=dvv, dA=dA, dB=dB, dC=dC)


# ---------------------------------------------------------------------------
# (2) the reference oracle's own algorithm: cumulative H0/H1/H2 states
# ---------------------------------------------------------------------------

def state_forward(q, k, v, dim_groups, A, B, C, *, scale: float):
    """(out, num, den) via causal cumulative-sum states (grouped_reference.py).

    Memory is O(B*H*N*D^2*Dv); use on small shapes only.
    """
    batch, hq, n, d = q.shape
    hkv, dv = k.shape[1], v.shape[-1]
    rows, cols = torch.tril_indices(d, d)
    u = torch.cat([v, torch.ones(batch, hkv, n, 1, dtype=v.dtype)], -1)
    h0 = u.cumsum(2)                                                   # :48-52
    h1 = (k.unsqueeze(-1) * u.unsqueeze(-2)).cumsum(2)
    h2 = ((k[..., rows] * k[..., cols]).unsqueeze(-1) * u.unsqueeze(-2)).cumsum(2)
    kv_of = torch.arange(hq) // (hq // hkv)
    h0, h1, h2 = h0[:, kv_of], h1[:, kv_of], h2[:, kv_of]
    groups = _groups_per_head(dim_groups, hq)
    lin = B.gather(1, groups)                                          # :83
    heads = torch.arange(hq)[:, None]
    quad = C[heads, groups[:, rows], groups[:, cols]]                  # :87-91
    mult = torch.where(rows == cols, 1.0, 2.0).to(q.dtype)             # :92-96
    qs = q * scale
    qp = qs[..., rows] * qs[..., cols]
    y = (A[None, :, None, None] * h0
         + (qs.unsqueeze(-1) * h1 * lin[None, :, None, :, None]).sum(-2)
         + (qp.unsqueeze(-1) * h2 * (quad * mult)[None, :, None, :, None]).sum(-2))
    num, den = y[..., :dv], y[..., dv:]
    if not (torch.isfinite(den) & (den > 0)).all():                    # :206-209
        raise RuntimeError("Grouped Quadratic denominator must be finite and strictly positive")
    return num / den, num, den


# ---------------------------------------------------------------------------
# (3) chunked linear-attention form, analytic backward (the timed CPU baseline)
# ---------------------------------------------------------------------------

def _pair_tables(d: int, dtype):
    rows, cols = torch.tril_indices(d, d)
    mult = torch.where(rows == cols, 1.0, 2.0).to(dtype)
    return rows, cols, mult


def key_features(k):
    """phi_k = [1, k_d, k_r k_c (r>=c)] (hd_block_gemm_feature_forward.py:225-253)."""
    rows, cols, _ = _pair_tables(k.shape[-1], k.dtype)
    return torch.cat([torch.ones_like(k[..., :1]), k, k[..., rows] * k[..., cols]], -1)


def query_features(qs, a, b_dim, c_pair_m):
    """phi_q = [A, B_{g(d)} q_d, m C_{g(r)g(c)} q_r q_c] (…feature_forward.py:373-385)."""
    rows, cols, _ = _pair_tables(qs.shape[-1], qs.dtype)
    shape = qs.shape[:-1] + (1,)
    return torch.cat([a[None, :, None, None].expand(shape),
                      qs * b_dim[None, :, None, :],
                      qs[..., rows] * qs[..., cols] * c_pair_m[None, :, None, :]], -1)


def chunked_forward_backward(q, k, v, dim_groups, A, B, C, *, scale: float, token_block: int = 64,
                             grad_out=None, grad_num=None, grad_den=None,
                             floor: float = POSITIVE_FP32_FLOOR):
    """Chunked forward and analytic backward in the working dtype of ``q``.

    Forward: block totals phi_k^T U, exclusive prefix over blocks, then
    Y = phi_q carry + tril(phi_q phi_k^T) U per block.  Backward: normalisation
    VJP, dCarry = phi_q^T G, reverse exclusive scan, per-block VJPs and the
    feature-map folds.  Returns a dict like ``dense_backward`` (gradients only
    when an upstream gradient is given).
    """
    batch, hq, n, d = q.shape
    hkv, dv = k.shape[1], v.shape[-1]
    rep = hq // hkv
    t = token_block
    nb = (n + t - 1) // t
    dt = q.dtype
    rows, cols, mult = _pair_tables(d, dt)
    groups = _groups_per_head(dim_groups, hq)
    heads = torch.arange(hq)[:, None]
    b_dim = B.gather(1, groups)
    c_pair = C[heads, groups[:, rows], groups[:, cols]]
    c_pair_m = c_pair * mult
    qs = q * scale
    u = torch.cat([v, torch.ones(batch, hkv, n, 1, dtype=dt)], -1)
    e = dv + 1
    f = 1 + d + rows.numel()

    def blk(c):
        return slice(c * t, min(n, (c + 1) * t))

    # forward ---------------------------------------------------------------
    carry = torch.zeros(batch, hkv, nb, f, e, dtype=dt)
    run = torch.zeros(batch, hkv, f, e, dtype=dt)
    for c in range(nb):
        carry[:, :, c] = run
        run = run + key_features(k[:, :, blk(c)]).transpose(-1, -2) @ u[:, :, blk(c)]
    y = torch.empty(batch, hq, n, e, dtype=dt)
    kv_of = torch.arange(hq) // rep
    for c in range(nb):
        sl = blk(c)
        pq = query_features(qs[:, :, sl], A, b_dim, c_pair_m)
        pk = key_features(k[:, :, sl])[:, kv_of]
        score = (pq @ pk.transpose(-1, -2)).tril()
        y[:, :, sl] = pq @ carry[:, kv_of, c] + score @ u[:, kv_of][:, :, sl]
    num, den = y[..., :dv], y[..., dv:]
    out = num / den.clamp_min(floor)
    result = dict(out=out, num=num, den=den)
    if grad_out is None and grad_num is None and grad_den is None:
        return result

    # backward ----------------------------------------------------------------
    den_w = den.clamp_min(floor)
    g = torch.zeros(batch, hq, n, e, dtype=dt)
    if grad_out is not None:
        g[..., :dv] = grad_out / den_w
        g[..., dv:] = -(grad_out * num).sum(-1, keepdim=True) / den_w / den_w * (den >= floor)
    if grad_num is not None:
        g[..., :dv] += grad_num
    if grad_den is not None:
        g[..., dv:] += grad_den
    dcarry = torch.zeros(batch, hkv, nb, f, e, dtype=dt)
    for c in range(nb):
        sl = blk(c)
        pq = query_features(qs[:, :, sl], A, b_dim, c_pair_m)
        dcarry[:, :, c] = (pq.transpose(-1, -2) @ g[:, :, sl]).view(batch, hkv, rep, f, e).sum(2)
    dtail = torch.zeros_like(dcarry)
    run = torch.zeros(batch, hkv, f, e, dtype=dt)
    for c in range(nb - 1, -1, -1):
        dtail[:, :, c] = run
        run = run + dcarry[:, :, c]

    dq = torch.empty_like(q)
    dk = torch.zeros_like(k)
    dvv = torch.zeros_like(v)
    dA = torch.zeros(hq, dtype=dt)
    db_dim = torch.zeros(hq, d, dtype=dt)
    dc_pair = torch.zeros(hq, rows.numel(), dtype=dt)
    for c in range(nb):
        sl = blk(c)
        qb, kb = qs[:, :, sl], k[:, :, sl]
        pq = query_features(qb, A, b_dim, c_pair_m)
        pk_kv = key_features(kb)
        pk = pk_kv[:, kv_of]
        ub = u[:, kv_of][:, :, sl]
        gb = g[:, :, sl]
        ds = (gb @ ub.transpose(-1, -2)).tril()
        score = (pq @ pk.transpose(-1, -2)).tril()
        dpq = gb @ carry[:, kv_of, c].transpose(-1, -2) + ds @ pk
        dpk = (ds.transpose(-1, -2) @ pq).view(batch, hkv, rep, -1, f).sum(2) \
            + u[:, :, sl] @ dtail[:, :, c].transpose(-1, -2)
        du = (score.transpose(-1, -2) @ gb).view(batch, hkv, rep, -1, e).sum(2) \
            + pk_kv @ dtail[:, :, c]
        dvv[:, :, sl] = du[..., :dv]
        # folds (chain rule through the feature maps)
        dA += dpq[..., 0].sum((0, 2))
        dlin, dpair = dpq[..., 1:1 + d], dpq[..., 1 + d:]
        db_dim += (dlin * qb).sum((0, 2))
        dc_pair += (dpair * qb[..., rows] * qb[..., cols] * mult).sum((0, 2))
        dqs = dlin * b_dim[None, :, None, :]
        wgt = dpair * c_pair_m[None, :, None, :]
        dqs = dqs.index_add(-1, rows, wgt * qb[..., cols]).index_add(-1, cols, wgt * qb[..., rows])
        dq[:, :, sl] = dqs * scale
        dkb = dpk[..., 1:1 + d].clone()
        pp = dpk[..., 1 + d:]
        dkb = dkb.index_add(-1, rows, pp * kb[..., cols]).index_add(-1, cols, pp * kb[..., rows])
        dk[:, :, sl] = dkb
    # per-dimension / per-pair coefficient gradients back to groups
    gcount = B.shape[-1]
    dB = torch.zeros(hq, gcount, dtype=dt).scatter_add(1, groups, db_dim)
    flat = groups[:, rows] * gcount + groups[:, cols]
    dC_lower = torch.zeros(hq, gcount * gcount, dtype=dt).scatter_add(1, flat, dc_pair).view(hq, gcount, gcount)
    dC = 0.5 * (dC_lower + dC_lower.transpose(-1, -2))
    result.update(dq=dq, dk=dk, dv=dvv, dA=dA, dB=dB, dC=dC)
    return result


def normalized_max_error(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max|x - ref| / max|ref| (the reference's own metric,
    oal_attention/build/probe_hd_bf16_bmm.py:1269-1282, without its clamp)."""
    x = x.detach().double().cpu()
    ref = ref.detach().double().cpu()
    scale = ref.abs().max().item()
    diff = (x - ref).abs().max().item()
    return diff / scale if scale > 0 else diff
