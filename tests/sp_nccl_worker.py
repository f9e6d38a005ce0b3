"""torchrun worker of the NCCL sequence-parallel test: every rank scans its half of the sequence,
rank results are compared with one single-GPU call over the whole sequence."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import oal_b200  # noqa: E402
from oal_b200 import synthetic  # noqa: E402
from oal_b200.sequence_parallel import sequence_parallel_attention  # noqa: E402
from oracle.oal_oracle import normalized_max_error as ERR  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    n = 1024 * world
    case = synthetic.qwen_head_case(12, batch=1, n=n, hq=14, hkv=2, g=8, bf16=True)
    q, k, v, dout = (t.to(dev, torch.bfloat16) for t in (case.q, case.k, case.v, case.grad_out))
    groups = case.dim_groups.to(dev)
    sl = slice(rank * n // world, (rank + 1) * n // world)
    factor = case.factor.to(dev).requires_grad_()
    qr, kr, vr = (t[:, :, sl].contiguous().requires_grad_() for t in (q, k, v))
    out, num, den = sequence_parallel_attention(qr, kr, vr, groups, factor, scale=case.scale)
    out.backward(dout[:, :, sl].contiguous())
    # single-GPU truth of the same operator over the whole sequence
    f2 = case.factor.to(dev).requires_grad_()
    qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
    o2, n2, d2 = oal_b200.grouped_causal_attention(qf, kf, vf, groups, f2, scale=case.scale,
                                                   precision="bf16_tensorcore")
    o2.backward(dout)
    errs = dict(out=ERR(out, o2[:, :, sl]), num=ERR(num, n2[:, :, sl]), den=ERR(den, d2[:, :, sl]),
                dq=ERR(qr.grad, qf.grad[:, :, sl]), dk=ERR(kr.grad, kf.grad[:, :, sl]),
                dv=ERR(vr.grad, vf.grad[:, :, sl]), dfactor=ERR(factor.grad, f2.grad))
    bad = {k_: e for k_, e in errs.items() if not e < 5e-3}
    flag = torch.tensor([len(bad)], device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print("errors rank0:", errs)
        print("SP_OK" if flag.item() == 0 else f"SP_FAIL {bad}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
