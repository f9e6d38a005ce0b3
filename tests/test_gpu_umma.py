"""Tensor-core building blocks: tcgen05.mma with each operand arrangement the attention
kernels use, against a float64 matmul of the same bf16 operands."""

import ctypes

import pytest
import torch

from oal_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("n,k", [(16, 16), (80, 64), (256, 128), (64, 32)])
def test_umma_gemm(mode, n, k):
    lib = _lib.load()
    gen = torch.Generator().manual_seed(100 * mode + n + k)
    if mode == 1:
        a = torch.randn(k, 128, generator=gen).bfloat16().cuda()
        b = torch.randn(k, n, generator=gen).bfloat16().cuda()
        want = a.double().t() @ b.double()
    else:
        a = torch.randn(128, k, generator=gen).bfloat16().cuda()
        b = torch.randn(n, k, generator=gen).bfloat16().cuda()
        want = a.double() @ b.double().t()
    d = torch.full((128, n), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.oal_selftest_umma(mode, n, k, _lib.ptr(a), _lib.ptr(b), _lib.ptr(d), _lib.ptr(status),
                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "bounded wait expired"
    err = (d.double() - want).abs().max().item() / want.abs().max().item()
    assert err < 1e-5, f"mode {mode} n={n} k={k}: normalized max error {err}"
