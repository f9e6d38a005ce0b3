"""The allocation-free forward entry point, called through the C ABI.

Some hosts of the library cannot allocate device memory when they call it (a server whose memory
pool is frozen after start-up, a plugin invoked from a callback that must not allocate).  For them
``oal_forward_static_scratch`` keeps its scratch in an array inside the library.  This test calls
it twice in a row on different inputs and compares each result with the regular ``oal_forward``
(which takes a caller workspace) on the same inputs.  It lives in a file that sorts last so that a
run stopping at the first failure has already executed every other test.
"""

import ctypes

import pytest
import torch

from oal_b200 import _lib, synthetic
from oal_b200.hd_block_gemm import make_problem
from oal_b200.hd_block_gemm_autograd import build_group_tables
from oracle import oal_oracle as orc

pytestmark = pytest.mark.gpu


def _call(entry, case, use_static):
    lib = _lib.load()
    dev = torch.device("cuda")
    q, k, v = (t.to(dev, torch.bfloat16).contiguous() for t in (case.q, case.k, case.v))
    b, hq, n, _ = q.shape
    hkv = k.shape[1]
    a, bb, c = (t.float().to(dev).contiguous() for t in orc.expand_factor(case.factor, hq, case.kernel_eps))
    g = bb.shape[1]
    groups = case.dim_groups.to(dev)
    groups = groups.unsqueeze(0).expand(hq, -1) if groups.ndim == 1 else groups
    tables = build_group_tables(groups, g)
    problem = make_problem((b, hq, hkv, n, 64, 64), groups=g, io_dtype=torch.bfloat16, out_dtype=torch.bfloat16,
                           precision="bf16_tensorcore", chunk=128, scale=case.scale, floor=orc.POSITIVE_FP32_FLOOR)
    out = torch.empty(b, hq, n, 64, dtype=torch.bfloat16, device=dev)
    num = torch.empty(b, hq, n, 64, dtype=torch.float32, device=dev)
    den = torch.empty(b, hq, n, dtype=torch.float32, device=dev)
    saved = torch.empty(_lib.workspace_bytes(problem, 2), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    common = [ctypes.byref(problem), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(tables.dim_perm),
              _lib.ptr(tables.group_start), _lib.ptr(a), _lib.ptr(bb), _lib.ptr(c), _lib.ptr(out), _lib.ptr(num),
              _lib.ptr(den), _lib.ptr(saved)]
    if use_static:
        rc = lib.oal_forward_static_scratch(*common, _lib.ptr(status), stream)
    else:
        ws = torch.empty(_lib.workspace_bytes(problem, 0), dtype=torch.uint8, device=dev)
        rc = lib.oal_forward(*common, None, _lib.ptr(ws), ws.numel(), _lib.ptr(status), stream)
    _lib.check(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out.float().cpu(), num.cpu(), den.cpu(), saved.cpu()


def test_static_scratch_forward_matches_workspace_forward_twice():
    cases = [synthetic.qwen_head_case(31, batch=1, n=700, hq=14, hkv=2, g=8, bf16=True),   # 2 units x 6 chunks
             synthetic.qwen_head_case(32, batch=2, n=300, hq=4, hkv=2, g=4, bf16=True)]    # 4 units x 3 chunks
    for case in cases:
        want = _call("workspace", case, use_static=False)
        got = _call("static", case, use_static=True)
        for name, x, y in zip(("out", "num", "den", "saved_state"), got, want):
            if name == "saved_state":
                assert torch.equal(x, y), name
            else:
                assert orc.normalized_max_error(x, y) <= 1e-6, name


def _static_call_on_device_tensors(case):
    """Everything the call needs is created first; returns a closure that only makes the library call."""
    lib = _lib.load()
    dev = torch.device("cuda")
    q, k, v = (t.to(dev, torch.bfloat16).contiguous() for t in (case.q, case.k, case.v))
    b, hq, n, _ = q.shape
    hkv = k.shape[1]
    a, bb, c = (t.float().to(dev).contiguous() for t in orc.expand_factor(case.factor, hq, case.kernel_eps))
    groups = case.dim_groups.to(dev)
    groups = groups.unsqueeze(0).expand(hq, -1) if groups.ndim == 1 else groups
    tables = build_group_tables(groups, bb.shape[1])
    problem = make_problem((b, hq, hkv, n, 64, 64), groups=bb.shape[1], io_dtype=torch.bfloat16,
                           out_dtype=torch.bfloat16, precision="bf16_tensorcore", chunk=128, scale=case.scale,
                           floor=orc.POSITIVE_FP32_FLOOR)
    out = torch.empty(b, hq, n, 64, dtype=torch.bfloat16, device=dev)
    num = torch.empty(b, hq, n, 64, dtype=torch.float32, device=dev)
    den = torch.empty(b, hq, n, dtype=torch.float32, device=dev)
    saved = torch.empty(_lib.workspace_bytes(problem, 2), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    keep = (q, k, v, a, bb, c, tables, problem, out, num, den, saved, status)

    def call():
        return lib.oal_forward_static_scratch(
            ctypes.byref(problem), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(tables.dim_perm),
            _lib.ptr(tables.group_start), _lib.ptr(a), _lib.ptr(bb), _lib.ptr(c), _lib.ptr(out), _lib.ptr(num),
            _lib.ptr(den), _lib.ptr(saved), _lib.ptr(status), stream)

    return call, keep


def test_static_scratch_call_leaves_free_device_memory_unchanged():
    """The property in the entry point's name: once the first call on the device has resolved the array's
    address, a call neither takes nor returns device memory -- with the library's per-kernel event timing
    switched on as well (this entry point never times its launches, because creating events allocates)."""
    case = synthetic.qwen_head_case(33, batch=1, n=500, hq=6, hkv=2, g=8, bf16=True)
    call, keep = _static_call_on_device_tensors(case)
    _lib.check(call())                       # first call: address resolution, module load
    torch.cuda.synchronize()
    for profiling in (False, True):
        _lib.profile_enable(profiling)
        try:
            free_before, _ = torch.cuda.mem_get_info()
            _lib.check(call())
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
        finally:
            _lib.profile_enable(False)
        assert free_after == free_before, (profiling, free_before, free_after)
    assert int(keep[-1].item()) == 0


@pytest.mark.parametrize("batch,hkv,n,hq,accepted", [
    (2, 2, 512, 4, True),        # 4 units x 4 chunks = 16: the limit itself
    (1, 1, 2048, 2, True),       # 1 unit x 16 chunks
    (1, 1, 2049, 2, False),      # 17 chunks
    (17, 1, 100, 1, False),      # 17 units
    (1, 1, 128, 64, True),       # 64 query heads
    (1, 1, 128, 65, False),      # 65 query heads
])
def test_static_scratch_limits_are_exact(batch, hkv, n, hq, accepted):
    """Limits are checked before anything is launched: rejected problems may pass dummy tensors."""
    lib = _lib.load()
    if accepted:
        g = torch.Generator().manual_seed(n + hq)
        case = synthetic.OalCase(
            q=torch.randn(batch, hq, n, 64, generator=g), k=torch.randn(batch, hkv, n, 64, generator=g),
            v=torch.randn(batch, hkv, n, 64, generator=g), dim_groups=(torch.arange(64) % 2).to(torch.int32),
            scale=0.125, factor=torch.rand(hq, 6, generator=g) * 0.9 + 0.1)
        want = _call("workspace", case, use_static=False)
        got = _call("static", case, use_static=True)
        assert torch.equal(got[3], want[3])
        assert orc.normalized_max_error(got[0], want[0]) <= 1e-6
        return
    problem = make_problem((batch, hq, hkv, n, 64, 64), groups=2, io_dtype=torch.bfloat16, out_dtype=torch.bfloat16,
                           precision="bf16_tensorcore", chunk=128, scale=0.125, floor=1e-38)
    dummy = torch.zeros(16, device="cuda")
    p = _lib.ptr(dummy)
    assert lib.oal_forward_static_scratch(ctypes.byref(problem), p, p, p, p, p, p, p, p, p, p, p, p, p, None) == -3


def test_static_scratch_forward_rejects_oversized_problems():
    lib = _lib.load()
    problem = make_problem((4, 14, 2, 4096, 64, 64), groups=8, io_dtype=torch.bfloat16, out_dtype=torch.bfloat16,
                           precision="bf16_tensorcore", chunk=128, scale=0.125, floor=1e-38)
    dummy = torch.zeros(16, device="cuda")
    p = _lib.ptr(dummy)
    rc = lib.oal_forward_static_scratch(ctypes.byref(problem), p, p, p, p, p, p, p, p, p, p, p, p, p, None)
    assert rc == -3
    with pytest.raises(ValueError, match="static scratch limit"):
        _lib.check(rc)
