"""Sequence parallelism: host logic with gloo ranks on the CPU, kernel path by emulating the
ranks one after another on a single GPU, and the real NCCL path when two GPUs are present."""

import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oal_b200 import synthetic
from oal_b200.sequence_parallel import exclusive_prefix_over_ranks

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _prefix_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    local = torch.full((3, 5), float(rank + 1)) + torch.arange(5.0)
    fwd = exclusive_prefix_over_ranks(local, None)
    rev = exclusive_prefix_over_ranks(local, None, reverse=True)
    torch.save((fwd, rev), os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_exclusive_prefix_over_gloo_ranks(tmp_path, world):
    mp.spawn(_prefix_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    locals_ = [torch.full((3, 5), float(r + 1)) + torch.arange(5.0) for r in range(world)]
    for r in range(world):
        fwd, rev = torch.load(tmp_path / f"r{r}.pt")
        assert torch.equal(fwd, sum(locals_[:r], torch.zeros(3, 5)))
        assert torch.equal(rev, sum(locals_[r + 1:], torch.zeros(3, 5)))


def test_exclusive_prefix_without_process_group_is_zero():
    assert torch.count_nonzero(exclusive_prefix_over_ranks(torch.ones(4))) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("splits,dv,g", [((256, 256), 64, 8), ((128, 300, 212), 64, 8), ((256, 200), 32, 8),
                                         ((128, 256), 64, 16)])
def test_rank_emulation_matches_single_call(splits, dv, g):
    """Run the ranks' kernels one after another on one GPU, passing states by hand: the
    concatenated result must equal one call over the whole sequence (both use the same chunk
    arithmetic only when the split points are chunk-aligned, so compare within tolerance)."""
    import oal_b200
    from oal_b200.hd_block_gemm_adapters import prepare_grouped_hd_block_gemm
    from oal_b200.grouped_quadratic import _expand_factor_coefficients
    from oal_b200.hd_block_gemm_autograd import backward_impl, forward_impl
    from oal_b200.sequence_parallel import local_dstate_total, local_state_total
    from tests.helpers import ERR

    n = sum(splits)
    case = synthetic.qwen_head_case(9, batch=1, n=n, hq=4, hkv=2, g=g, bf16=True,
                                    outlier_scale=20.0 if g == 8 else 4.0)
    case.v, case.grad_out = case.v[..., :dv].contiguous(), case.grad_out[..., :dv].contiguous()
    dev = "cuda"
    q, k, v, dout = (t.to(dev, torch.bfloat16) for t in (case.q, case.k, case.v, case.grad_out))
    groups, factor = case.dim_groups.to(dev), case.factor.to(dev).requires_grad_()
    qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
    out, num, den = oal_b200.grouped_causal_attention(qf, kf, vf, groups, factor, scale=case.scale,
                                                      precision="bf16_tensorcore")
    out.backward(dout)
    full = dict(out=out, num=num, den=den, dq=qf.grad, dk=kf.grad, dv=vf.grad)

    bounds = [0]
    for s in splits:
        bounds.append(bounds[-1] + s)
    mask = (True,) * 6
    ranks = []
    for r in range(len(splits)):
        sl = slice(bounds[r], bounds[r + 1])
        qr, kr, vr = (t[:, :, sl].contiguous().requires_grad_() for t in (q, k, v))
        prep = prepare_grouped_hd_block_gemm(qr, kr, vr, groups, factor, scale=case.scale,
                                             precision="bf16_tensorcore")
        ranks.append(dict(q=qr, k=kr, v=vr, prep=prep, sl=sl, total=local_state_total(kr, vr, prep.plan, prep.gmax)))
    a, b, c = (t.detach().contiguous() for t in _expand_factor_coefficients(
        factor, query_heads=4, gmax=g, kernel_eps=case.kernel_eps, working_dtype=torch.float32))
    for r, st in enumerate(ranks):
        state_in = sum((x["total"] for x in ranks[:r]), torch.zeros_like(st["total"]))
        p = st["prep"]
        st["fwd"] = forward_impl(st["q"], st["k"], st["v"], a, b, c, p.tables, p.scale, p.normalization_floor,
                                 p.plan, state_in=state_in)
    for st in ranks:
        p = st["prep"]
        o, nm, dn, saved, padded = st["fwd"]
        st["ws"] = torch.empty(p.plan.backward_workspace_bytes, dtype=torch.uint8, device=dev)
        st["dtotal"] = local_dstate_total(padded, nm, dn, saved, p.tables, p.scale, p.normalization_floor,
                                          p.plan, mask, dout[:, :, st["sl"]].contiguous(), None, None, st["ws"])
    parts = dict(out=[], num=[], den=[], dq=[], dk=[], dv=[])
    for r, st in enumerate(ranks):
        p = st["prep"]
        o, nm, dn, saved, padded = st["fwd"]
        dstate_in = sum((x["dtotal"] for x in ranks[r + 1:]), torch.zeros_like(st["dtotal"]))
        # every rank has its own workspace here, still holding its stage-A results
        dq, dk, dv, dA, dB, dC = backward_impl(padded, nm, dn, saved, p.tables, p.scale, p.normalization_floor,
                                               p.plan, mask, dout[:, :, st["sl"]].contiguous(), None, None,
                                               dstate_in=dstate_in, workspace=st["ws"], reuse_state_stage=True)
        for key, val in dict(out=o, num=nm, den=dn, dq=dq, dk=dk, dv=dv).items():
            parts[key].append(val)
    for key, vals in parts.items():
        got = torch.cat(vals, dim=2)
        assert ERR(got, full[key]) < 1e-2, key      # bf16 outputs: one ulp near the maximum is 4e-3


def _nccl_script():
    return ROOT / "tests" / "sp_nccl_worker.py"


@pytest.mark.gpu
def test_nccl_sequence_parallel_at_configured_length():
    """N = 32768 over every GPU of the box (2, 4 or 8 ranks): against the single-GPU call and against the
    stored rows of the reference's chunked path."""
    gpus = torch.cuda.device_count()
    if gpus < 2:
        pytest.skip("needs two GPUs")
    world = 8 if gpus >= 8 else (4 if gpus >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(_nccl_script()), "32768"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "SP_OK" in res.stdout


@pytest.mark.gpu
def test_eight_rank_emulation_at_configured_length_against_reference_golden():
    """The sequence-parallel configuration itself (N = 32768 cut into 8 ranges of 4096 tokens) with the ranks'
    kernels run one after another on one GPU and the states passed by hand: against one call over the whole
    sequence (errors normalised by the whole result) and against the stored rows of the reference's chunked
    fp32 path (tests/golden/long_rows.npz).  The NCCL test runs the same ranges on real ranks when the box has
    more than one GPU."""
    import numpy as np

    import oal_b200
    from oal_b200.grouped_quadratic import _expand_factor_coefficients
    from oal_b200.hd_block_gemm_adapters import prepare_grouped_hd_block_gemm
    from oal_b200.hd_block_gemm_autograd import backward_impl, forward_impl
    from oal_b200.sequence_parallel import local_dstate_total, local_state_total

    world, n, dev = 8, 32768, "cuda"
    case = synthetic.qwen_head_case(7, batch=1, n=n, hq=14, hkv=2, g=8, bf16=True)
    q, k, v, dout = (t.to(dev, torch.bfloat16) for t in (case.q, case.k, case.v, case.grad_out))
    groups, factor = case.dim_groups.to(dev), case.factor.to(dev).requires_grad_()
    qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
    out, num, den = oal_b200.grouped_causal_attention(qf, kf, vf, groups, factor, scale=case.scale,
                                                      precision="bf16_tensorcore")
    out.backward(dout)
    full = dict(out=out, num=num, den=den, dq=qf.grad, dk=kf.grad, dv=vf.grad)
    a, b, c = (t.detach().contiguous() for t in _expand_factor_coefficients(
        case.factor.to(dev), query_heads=14, gmax=8, kernel_eps=case.kernel_eps, working_dtype=torch.float32))
    mask, ranks = (True,) * 6, []
    for r in range(world):
        sl = slice(r * n // world, (r + 1) * n // world)
        qr, kr, vr = (t[:, :, sl].contiguous().requires_grad_() for t in (q, k, v))
        prep = prepare_grouped_hd_block_gemm(qr, kr, vr, groups, factor, scale=case.scale, precision="bf16_tensorcore")
        ranks.append(dict(q=qr, k=kr, v=vr, prep=prep, sl=sl, total=local_state_total(kr, vr, prep.plan, prep.gmax)))
    for r, st in enumerate(ranks):
        p = st["prep"]
        state_in = sum((x["total"] for x in ranks[:r]), torch.zeros_like(st["total"]))
        st["fwd"] = forward_impl(st["q"], st["k"], st["v"], a, b, c, p.tables, p.scale, p.normalization_floor, p.plan,
                                 state_in=state_in)
    for st in ranks:
        p = st["prep"]
        _, nm, dn, saved, padded = st["fwd"]
        st["ws"] = torch.empty(p.plan.backward_workspace_bytes, dtype=torch.uint8, device=dev)
        st["dtotal"] = local_dstate_total(padded, nm, dn, saved, p.tables, p.scale, p.normalization_floor, p.plan, mask,
                                          dout[:, :, st["sl"]].contiguous(), None, None, st["ws"])
    parts = dict(out=[], num=[], den=[], dq=[], dk=[], dv=[])
    for r, st in enumerate(ranks):
        p = st["prep"]
        o, nm, dn, saved, padded = st["fwd"]
        dstate_in = sum((x["dtotal"] for x in ranks[r + 1:]), torch.zeros_like(st["dtotal"]))
        dq, dk, dv, _, _, _ = backward_impl(padded, nm, dn, saved, p.tables, p.scale, p.normalization_floor, p.plan, mask,
                                            dout[:, :, st["sl"]].contiguous(), None, None, dstate_in=dstate_in,
                                            workspace=st["ws"], reuse_state_stage=True)
        for key, val in dict(out=o, num=nm, den=dn, dq=dq, dk=dk, dv=dv).items():
            parts[key].append(val)
    got = {key: torch.cat(vals, dim=2).detach().float() for key, vals in parts.items()}
    for key, val in got.items():
        whole = full[key].detach().float()
        assert ((val - whole).abs().max() / whole.abs().max()).item() < 5e-3, key
    with np.load(ROOT / "tests" / "golden" / "long_rows.npz") as z:
        stride = int(z["row_stride"])
        for key, val in got.items():
            gold = torch.from_numpy(z["hd_" + key].astype("float64"))
            rows = val[:, :, ::stride].double().cpu()
            assert ((rows - gold).abs().max() / gold.abs().max()).item() < 2e-2, key
