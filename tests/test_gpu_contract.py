"""Semantics the reference's operator tests pin (tests/operators/test_grouped_quadratic.py:188-335,
:399-414 there), replayed on the CUDA operator in fp32 mode against the fp64 dense oracle."""

import pytest
import torch

import oal_b200
from oracle import oal_oracle as orc

pytestmark = pytest.mark.gpu
ERR = orc.normalized_max_error


def _case(batch=2, query_heads=4, key_heads=2, sequence=37, dimension=8, value_dimension=5):
    g = torch.Generator().manual_seed(20260802)
    return (torch.randn(batch, query_heads, sequence, dimension, generator=g),
            torch.randn(batch, key_heads, sequence, dimension, generator=g),
            torch.randn(batch, key_heads, sequence, value_dimension, generator=g))


def _factor():
    return torch.tensor((1.1, 0.5, 0.9, 0.4, 0.8, 0.7))


def _groups(query_heads=4, dimension=8):
    m = torch.ones((query_heads, dimension), dtype=torch.int32)
    m[:, : dimension // 2] = 0
    return m


def _oracle(q, k, v, groups, factor, kernel_eps=1e-6):
    a, b, c = orc.expand_factor(factor.double(), q.shape[1], kernel_eps)
    return orc.dense_forward(q.double(), k.double(), v.double(), groups, a, b, c, scale=q.shape[-1] ** -0.5)


@pytest.mark.parametrize("group_shape", ["shared", "per_head"])
@pytest.mark.parametrize("factor_shape", ["shared", "per_head"])
def test_group_and_factor_broadcast_combinations(group_shape, factor_shape):
    q, k, v = _case()
    groups = _groups()
    factor = _factor()
    pg = groups[0] if group_shape == "shared" else groups
    pf = factor if factor_shape == "shared" else factor.expand(q.shape[1], -1).clone()
    out = oal_b200.oal_attention(q.cuda(), k.cuda(), v.cuda(), pg.cuda(), pf.cuda())
    want, _, _ = _oracle(q, k, v, pg, pf)
    assert ERR(out, want) < 1e-5


def test_broadcast_factor_gradient_reduces_across_query_heads():
    q, k, v = (t.cuda() for t in _case(batch=1))
    groups = _groups().cuda()
    shared = _factor().cuda().requires_grad_()
    oal_b200.oal_attention(q, k, v, groups, shared).square().sum().backward()
    per_head = _factor().expand(q.shape[1], -1).clone().cuda().requires_grad_()
    oal_b200.oal_attention(q, k, v, groups, per_head).square().sum().backward()
    assert ERR(shared.grad, per_head.grad.sum(0)) < 1e-5


def test_inactive_padded_factor_entries_do_not_change_output_or_gradient():
    q, k, v = (t.cuda() for t in _case(query_heads=2, key_heads=1, dimension=4))
    groups = torch.tensor(((0, 0, 1, 1), (0, 0, 0, 0)), dtype=torch.int32).cuda()
    factor = _factor().expand(2, -1).clone().cuda().requires_grad_()
    out = oal_b200.oal_attention(q, k, v, groups, factor)
    out[:, 1].square().sum().backward()
    assert torch.count_nonzero(factor.grad[0]) == 0
    assert torch.count_nonzero(factor.grad[1, 3:]) == 0
    changed = factor.detach().clone()
    changed[1, 3:] += 100.0
    out2 = oal_b200.oal_attention(q, k, v, groups, changed)
    assert ERR(out2[:, 1], out[:, 1].detach()) < 1e-6


def test_output_dtype_only_changes_normalized_output():
    q, k, v = (t.cuda() for t in _case(query_heads=1, key_heads=1))
    groups = _groups(1).cuda()[0]
    o32, n32, d32 = oal_b200.oal_attention(q, k, v, groups, _factor().cuda(), return_unnormalized=True)
    o16, n16, d16 = oal_b200.oal_attention(q, k, v, groups, _factor().cuda(), return_unnormalized=True,
                                           output_dtype=torch.float16)
    assert o16.dtype == torch.float16 and n16.dtype == torch.float32 and d16.dtype == torch.float32
    assert torch.equal(n16, n32) and torch.equal(d16, d32)
    assert ERR(o16, o32) < 2e-3


def test_fp16_inputs_fp32_mode():
    q, k, v = _case(dimension=64, value_dimension=64, sequence=150)
    groups = _groups(4, 64)
    out = oal_b200.oal_attention(q.half().cuda(), k.half().cuda(), v.half().cuda(), groups.cuda(), _factor().cuda())
    want, _, _ = _oracle(q.half().float(), k.half().float(), v.half().float(), groups, _factor())
    assert out.dtype == torch.float16 and ERR(out, want) < 2e-3


def test_workspace_too_small_is_a_value_error():
    import ctypes

    from oal_b200 import _lib
    from oal_b200.hd_block_gemm import make_problem

    problem = make_problem((1, 2, 1, 256, 64, 64), groups=2, io_dtype=torch.bfloat16, out_dtype=torch.bfloat16,
                           precision="bf16_tensorcore", chunk=128, scale=0.125, floor=1e-38)
    dummy = torch.zeros(64, device="cuda")
    p = _lib.ptr(dummy)
    rc = _lib.load().oal_forward(ctypes.byref(problem), p, p, p, p, p, p, p, p, p, p, p, p, None, p, 16, p, None)
    with pytest.raises(ValueError, match="workspace too small"):
        _lib.check(rc)


# ---- the rest of the public-entry semantics the reference pins (test_grouped_quadratic.py:135-183,
# :223-262, :417-427, :464-473 there), replayed through oal_b200.oal_attention on the GPU ----------------

def _dense(q, k, v, groups, factor, scale, kernel_eps=1e-6):
    a, b, c = orc.expand_factor(factor.double(), q.shape[1], kernel_eps)
    return orc.dense_forward(q.double(), k.double(), v.double(), groups, a, b, c, scale=scale)


def test_public_entry_matches_dense_oracle_with_unnormalized_outputs():
    q, k, v = _case(dimension=4)
    groups, factor = _groups(dimension=4), _factor()
    out, num, den = oal_b200.oal_attention(q.cuda(), k.cuda(), v.cuda(), groups.cuda(), factor.cuda(), scale=0.37,
                                           kernel_eps=0.07, causal=True, return_unnormalized=True)
    want, want_num, want_den = _dense(q, k, v, groups, factor, 0.37, 0.07)
    assert ERR(out, want) < 1e-5 and ERR(num, want_num) < 1e-5 and ERR(den, want_den) < 1e-5
    assert num.dtype == torch.float32 and den.dtype == torch.float32
    assert torch.isfinite(den).all() and (den > 0).all()


def test_fixed_initialization_is_independent_of_legal_group_partition():
    q, k, v = (t.cuda() for t in _case(query_heads=1, key_heads=1, dimension=4))
    factor = torch.tensor((1.0, 0.5, 0.5, 0.5, 0.5, 0.0)).cuda()
    out_a = oal_b200.oal_attention(q, k, v, torch.tensor((0, 0, 1, 1)).cuda(), factor)
    out_b = oal_b200.oal_attention(q, k, v, torch.tensor((0, 1, 0, 1)).cuda(), factor)
    assert ERR(out_a, out_b) < 1e-5


def test_cross_group_coefficient_changes_result():
    q, k, v = (t.cuda() for t in _case(query_heads=1, key_heads=1, dimension=4))
    groups = torch.tensor((0, 0, 1, 1), dtype=torch.int32).cuda()
    factor = _factor().cuda()
    no_cross = factor.clone()
    no_cross[3] = 0.0
    assert not torch.allclose(oal_b200.oal_attention(q, k, v, groups, factor),
                              oal_b200.oal_attention(q, k, v, groups, no_cross))


@pytest.mark.parametrize("precision,io_dtype,tol", [("fp32_ieee", torch.float32, 1e-4),
                                                     ("bf16_tensorcore", torch.bfloat16, 2e-2)])
def test_factor_and_qkv_gradients_match_dense_oracle_through_the_public_entry(precision, io_dtype, tol):
    q0, k0, v0 = (t.to(io_dtype).float() for t in _case(sequence=150))
    groups, factor0 = _groups(), _factor().expand(q0.shape[1], -1).clone()
    q, k, v = (t.to(device="cuda", dtype=io_dtype).requires_grad_() for t in (q0, k0, v0))
    factor = factor0.cuda().requires_grad_()
    out = oal_b200.oal_attention(q, k, v, groups.cuda(), factor, precision=precision, output_dtype=torch.float32)
    g = torch.Generator().manual_seed(7)
    dout = torch.randn(out.shape, generator=g)
    out.backward(dout.cuda())
    qd, kd, vd = (t.double().requires_grad_() for t in (q0, k0, v0))
    fd = factor0.double().requires_grad_()
    a, b, c = orc.expand_factor(fd, q0.shape[1], 1e-6)
    want, _, _ = orc.dense_forward(qd, kd, vd, groups, a, b, c, scale=q0.shape[-1] ** -0.5)
    want.backward(dout.double())
    assert ERR(out, want.detach()) < tol
    for got, ref in ((q.grad, qd.grad), (k.grad, kd.grad), (v.grad, vd.grad), (factor.grad, fd.grad)):
        assert ERR(got, ref) < tol


def test_default_scale_is_d_inverse_sqrt():
    q, k, v = (t.cuda() for t in _case(dimension=4))
    groups, factor = _groups(dimension=4).cuda(), _factor().cuda()
    assert ERR(oal_b200.oal_attention(q, k, v, groups, factor),
               oal_b200.oal_attention(q, k, v, groups, factor, scale=0.5)) < 1e-6
    with pytest.raises(ValueError):     # D > 64 is a reference-execution feature only
        wide = torch.randn(1, 1, 8, 72, device="cuda")
        oal_b200.oal_attention(wide, wide, wide, torch.zeros(72, dtype=torch.int32, device="cuda"),
                               torch.tensor((1.0, 0.5, 0.5), device="cuda"))


def test_shared_dim_groups_remain_a_logical_broadcast():
    q, k, v = (t.cuda() for t in _case())
    groups, factor = _groups(), _factor().cuda()
    shared = oal_b200.oal_attention(q, k, v, groups[0].cuda(), factor)
    expanded = oal_b200.oal_attention(q, k, v, groups.cuda(), factor)
    assert torch.equal(shared, expanded)


def test_bounded_wait_that_runs_out_reports_a_status_and_leaves_the_context_usable():
    """A wait with a short limit on a barrier nothing arrives on: the kernel gives up, stores the timeout
    flag with the wait site's id and returns; the host turns the word into the RuntimeError of the
    production path, and an ordinary call right afterwards works."""
    import ctypes

    from oal_b200 import _lib
    from oal_b200.hd_block_gemm_autograd import _raise_for_bits

    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.oal_selftest_wait_timeout(200_000, _lib.ptr(status), stream) == 0
    torch.cuda.synchronize()
    word = int(status.item())
    assert word == _lib.STATUS_WAIT_TIMEOUT | (0x7E << 8)
    with pytest.raises(RuntimeError, match="gave up on a bounded wait"):
        _raise_for_bits(word)
    assert lib.oal_selftest_wait_timeout(0, _lib.ptr(status), stream) == -1          # limits are validated
    assert lib.oal_selftest_wait_timeout(10_000_000, _lib.ptr(status), stream) == -1
    q, k, v = (t.cuda() for t in _case(batch=1))
    out = oal_b200.oal_attention(q, k, v, _groups().cuda(), _factor().cuda())
    want, _, _ = _oracle(*_case(batch=1), _groups(), _factor())
    assert ERR(out, want) < 1e-5


def test_every_library_call_runs_under_the_tensors_device(monkeypatch):
    """The kernels launch on the current device; the wrapper makes the tensors' device current around
    each call (the reference is plain torch code and follows its tensors)."""
    from oal_b200 import _lib

    entered = []
    real = _lib.device_guard

    def counting(t):
        entered.append(t.device)
        return real(t)

    monkeypatch.setattr(_lib, "device_guard", counting)
    q, k, v = (t.cuda().requires_grad_() for t in _case(batch=1))
    out = oal_b200.oal_attention(q, k, v, _groups().cuda(), _factor().cuda())
    out.sum().backward()
    assert len(entered) >= 2 and all(d == q.device for d in entered)


def test_operator_on_second_gpu_while_first_is_current():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    q0, k0, v0 = _case(batch=1)
    with torch.cuda.device(0):
        q, k, v = (t.to("cuda:1").requires_grad_() for t in (q0, k0, v0))
        out = oal_b200.oal_attention(q, k, v, _groups().to("cuda:1"), _factor().to("cuda:1"))
        out.sum().backward()
        torch.cuda.synchronize("cuda:1")
    want, _, _ = _oracle(q0, k0, v0, _groups(), _factor())
    assert out.device == torch.device("cuda:1") and ERR(out, want) < 1e-5
    assert torch.isfinite(q.grad).all()


def test_gradcheck_case_of_the_reference_on_the_gpu_entry():
    """The reference runs torch.autograd.gradcheck on its fp64 statement for B=1, H=1, N=2, D=2, Dv=1,
    groups (0, 1), kernel_eps 0.1 (tests/operators/test_grouped_quadratic.py:267-297 there).  The CUDA
    operator computes in fp32, so the same case is checked twice here: analytic gradients against the fp64
    dense statement, and against central differences of the operator's own forward along random directions."""
    q0, k0, v0 = _case(batch=1, query_heads=1, key_heads=1, sequence=2, dimension=2, value_dimension=1)
    f0 = torch.tensor((1.0, 0.4, 0.8, 0.2, 0.3, 0.7))
    groups = torch.tensor((0, 1), dtype=torch.int32)
    gen = torch.Generator().manual_seed(11)
    dout = torch.randn(1, 1, 2, 1, generator=gen)

    def run(q, k, v, f):
        return oal_b200.oal_attention(q, k, v, groups.cuda(), f, kernel_eps=0.1, precision="fp32_ieee")

    leaves = [t.clone().cuda().requires_grad_() for t in (q0, k0, v0, f0)]
    run(*leaves).backward(dout.cuda())
    ref = [t.double().requires_grad_() for t in (q0, k0, v0, f0)]
    a, b, c = orc.expand_factor(ref[3], 1, 0.1)
    want, _, _ = orc.dense_forward(ref[0], ref[1], ref[2], groups, a, b, c, scale=2 ** -0.5)
    want.backward(dout.double())
    for got, r in zip(leaves, ref):
        assert ERR(got.grad, r.grad) < 1e-4
    # central differences of the fp32 forward: step 1e-2 keeps rounding (1e-7 / 1e-2) below the tolerance
    for trial in range(4):
        dirs = [torch.randn(t.shape, generator=gen) for t in (q0, k0, v0, f0)]
        step = 1e-2
        plus = run(*[(t + step * d).cuda() for t, d in zip((q0, k0, v0, f0), dirs)])
        minus = run(*[(t - step * d).cuda() for t, d in zip((q0, k0, v0, f0), dirs)])
        numeric = float(((plus - minus).cpu() * dout).sum() / (2 * step))
        analytic = float(sum((leaf.grad.cpu() * d).sum() for leaf, d in zip(leaves, dirs)))
        assert abs(numeric - analytic) <= 2e-3 * max(1.0, abs(analytic)), (trial, numeric, analytic)


def test_group_ids_may_be_int64_on_the_gpu_entry():
    """The reference widens group ids to int64 for torch indexing
    (tests/operators/test_grouped_quadratic.py:439-461 there); here both widths give the same bits."""
    q, k, v = (t.cuda() for t in _case(query_heads=1, key_heads=1, dimension=4))
    factor = _factor().cuda()
    narrow = oal_b200.oal_attention(q, k, v, torch.tensor((0, 0, 1, 1), dtype=torch.int32).cuda(), factor)
    wide = oal_b200.oal_attention(q, k, v, torch.tensor((0, 0, 1, 1), dtype=torch.int64).cuda(), factor)
    assert torch.equal(narrow, wide)


@pytest.mark.parametrize("gmax", [1, 2, 8, 16])
@pytest.mark.parametrize("shared", [True, False])
def test_factor_expansion_kernel_matches_the_tensor_statement(gmax, shared):
    """Packed factor -> (A, B, C) and its gradient on the device (one kernel each) against the tensor-op
    statement of the same map that CPU tensors take (oal_attention/grouped_quadratic.py:184-219 there)."""
    from oal_b200.grouped_quadratic import _expand_factor_coefficients

    heads, pairs = 5, (gmax + 1) * (gmax + 2) // 2
    g = torch.Generator().manual_seed(gmax)
    f0 = torch.randn(pairs if shared else (heads, pairs), generator=g)
    weights = [torch.randn(heads, generator=g), torch.randn(heads, gmax, generator=g),
               torch.randn(heads, gmax, gmax, generator=g)]
    results = []
    for device in ("cpu", "cuda"):
        f = f0.double().requires_grad_() if device == "cpu" else f0.cuda().requires_grad_()
        dtype = torch.float64 if device == "cpu" else torch.float32
        a, b, c = _expand_factor_coefficients(f, query_heads=heads, gmax=gmax, kernel_eps=0.07, working_dtype=dtype)
        sum((t * w.to(t)).sum() for t, w in zip((a, b, c), weights)).backward()
        results.append([t.detach().cpu().double() for t in (a, b, c, f.grad)])
    for got, want in zip(results[1], results[0]):
        assert got.shape == want.shape and ERR(got, want) < 1e-6
    assert results[1][2].is_contiguous()


def test_status_ring_wraps_and_reports_the_right_call():
    """More deferred status words than the library's ring holds, drained as they finish; a nonzero word in
    the middle is raised with its own call id."""
    from oal_b200 import hd_block_gemm_autograd as hd

    hd.check_pending_status(block=True)
    clean = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(1500):
        hd.defer_status(clean, "probe")
    hd.check_pending_status(block=True)
    bad = torch.full((1,), 2, dtype=torch.int32, device="cuda")           # OAL_STATUS_DENOMINATOR
    hd.defer_status(clean, "probe")
    entry = hd.defer_status(bad, "marked")
    hd.defer_status(clean, "probe")
    with pytest.raises(RuntimeError, match=rf"marked, call {entry.call_id}\]"):
        hd.check_pending_status(block=True)
    hd.check_pending_status(block=True)                                     # the queue is usable afterwards
