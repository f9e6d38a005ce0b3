"""torchrun worker of the NCCL sequence-parallel test: every rank scans its share of the sequence;
rank results are compared with one single-GPU call over the whole sequence and, at the
sequence-parallel configuration's own length (N = 32768, the default), with the stored rows of the
reference's chunked fp32 path (tests/golden/long_rows.npz).

    torchrun --nproc-per-node R tests/sp_nccl_worker.py [total sequence length]
"""

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
    n = int(sys.argv[1]) if len(sys.argv) > 1 else 32768
    assert n % world == 0
    case = synthetic.qwen_head_case(7, batch=1, n=n, hq=14, hkv=2, g=8, bf16=True)
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
    # normalised by the size of the WHOLE single-GPU result, as every other comparison of the suite is: a
    # rank's own range can hold much smaller values than the sequence's maximum (with 8 ranks some do)
    def err(part, whole):
        whole = whole.detach().float()
        return ((part.detach().float() - whole[:, :, sl]).abs().max() / whole.abs().max().clamp_min(1e-30)).item()

    errs = dict(out=err(out, o2), num=err(num, n2), den=err(den, d2), dq=err(qr.grad, qf.grad), dk=err(kr.grad, kf.grad),
                dv=err(vr.grad, vf.grad), dfactor=ERR(factor.grad, f2.grad))
    bad = {k_: e for k_, e in errs.items() if not e < 5e-3}
    if n == 32768:
        # the reference's own rows (every 1024th token): this rank checks the ones that fall into its range
        import numpy as np

        with np.load(Path(__file__).resolve().parent / "golden" / "long_rows.npz") as z:
            gold = {key[3:]: torch.from_numpy(z[key].astype("float64")) for key in z.files if key.startswith("hd_")}
            stride = int(z["row_stride"])
        rows = slice(-(-sl.start // stride), -(-sl.stop // stride))
        mine = dict(out=out, num=num, den=den, dq=qr.grad, dk=kr.grad, dv=vr.grad)
        for key, t in mine.items():
            full_scale = gold[key].abs().max().item()
            got = t.detach().float().cpu()[:, :, (-sl.start % stride)::stride].double()
            diff = (got - gold[key][:, :, rows]).abs().max().item() / full_scale
            errs["ref_" + key] = diff
            if not diff < 2e-2:
                bad["ref_" + key] = diff
    if bad:
        print(f"rank {rank} out of tolerance: {bad}", flush=True)
    flag = torch.tensor([len(bad)], device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print("errors rank0:", errs)
        print("SP_OK" if flag.item() == 0 else f"SP_FAIL {bad}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
