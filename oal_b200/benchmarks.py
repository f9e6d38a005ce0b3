"""Secondary measurements of the operator (the headline number lives in bench.py at the repo root).

    python -m oal_b200.benchmarks sweep [--seq 1024,4096,16384,65536] [--groups 1,4,8,16]
        forward+backward time per token over sequence length and group count (B=1, 14 query /
        2 KV heads, d=64, bf16): time per token must stay flat in N, and the G axis shows what the
        per-group padding of the intra-chunk GEMMs costs.
    torchrun --nproc-per-node P -m oal_b200.benchmarks sp [--seq 32768]
        sequence-parallel forward+backward: the sequence is cut into P contiguous ranges, one
        all-gather of the range-final states per direction (NCCL).

    [torchrun --nproc-per-node P] -m oal_b200.benchmarks step [--layers 24] [--batch 8] [--seq 4096]
        model-level training step: Qwen2.5-0.5B-shaped decoder stack (random weights, LoRA rank 16 on
        q/k/v/o, trainable kernel factors, synthetic token ids) with the operator in every layer;
        forward, backward, gradient all-reduce of the trainable parameters across ranks (batch
        parallel), AdamW step.  Reports the share of the step spent in the operator's kernels.

Each measurement prints one JSON line (rank 0).  Inputs are the seeded synthetic tensors of
``oal_b200.synthetic``.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from . import _lib, synthetic
from .hd_block_gemm_adapters import prepare_grouped_hd_block_gemm, run_prepared_grouped_hd_block_gemm
from .hd_block_gemm_autograd import check_pending_status


def _time_steps(step, steps: int, warmup: int) -> float:
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    check_pending_status(block=True)
    return e0.elapsed_time(e1) / steps


def sweep(ns, gs, steps: int, warmup: int) -> None:
    dev = torch.device("cuda", 0)
    for g in gs:
        for n in ns:
            case = synthetic.qwen_head_case(7, batch=1, n=n, hq=14, hkv=2, g=g, bf16=True)
            q, k, v, dout = (t.to(dev, torch.bfloat16) for t in (case.q, case.k, case.v, case.grad_out))
            groups, factor = case.dim_groups.to(dev), case.factor.to(dev).requires_grad_()
            q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
            prepared = prepare_grouped_hd_block_gemm(q, k, v, groups, factor, scale=case.scale,
                                                     precision="bf16_tensorcore")

            def step():
                q.grad = k.grad = v.grad = factor.grad = None
                out, _, _ = run_prepared_grouped_hd_block_gemm(prepared, q, k, v, factor)
                out.backward(dout)

            ms = _time_steps(step, steps, warmup)
            # the same step as a CUDA graph replay: short sequences are bound by the host's queueing otherwise
            from .captured_step import CapturedStep

            captured = CapturedStep(prepared, q, k, v, factor.detach(), dout)
            graph_ms = _time_steps(captured.replay, steps, warmup)
            captured.check_status()
            print(json.dumps(dict(benchmark="sweep", n=n, groups=g, ms_per_step=ms, ns_per_token=ms * 1e6 / n,
                                  tokens_per_s=n / (ms * 1e-3), cuda_graph_ms_per_step=graph_ms,
                                  intra_chunk="tcgen05" if g <= 8 else "token-pair kernels")), flush=True)
            del q, k, v, dout, prepared, captured
            torch.cuda.empty_cache()


def sequence_parallel(n: int, steps: int, warmup: int, cuda_graph: bool = False) -> None:
    import torch.distributed as dist

    from .sequence_parallel import sequence_parallel_attention

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    case = synthetic.qwen_head_case(3, batch=1, n=n, hq=14, hkv=2, g=8, bf16=True)
    sl = slice(rank * n // world, (rank + 1) * n // world)
    q, k, v, dout = (t[:, :, sl].to(dev, torch.bfloat16).contiguous() for t in (case.q, case.k, case.v, case.grad_out))
    groups, factor = case.dim_groups.to(dev), case.factor.to(dev).requires_grad_()
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    prepared = prepare_grouped_hd_block_gemm(q, k, v, groups, factor, scale=case.scale, precision="bf16_tensorcore")

    def step():
        q.grad = k.grad = v.grad = factor.grad = None
        out, _, _ = sequence_parallel_attention(q, k, v, groups, factor, scale=case.scale, prepared=prepared)
        out.backward(dout)

    if world > 1:
        dist.barrier()
    from .sequence_parallel import exclusive_prefix_over_ranks

    state = torch.zeros(2, _lib.STATE_ROWS, _lib.E_PAD, device=dev)          # what one rank contributes per direction

    def exchange():                                                          # the two collectives of a step, alone
        exclusive_prefix_over_ranks(state, None)
        exclusive_prefix_over_ranks(state, None, reverse=True)

    eager_ms, exchange_only_ms = _time_steps(step, steps, warmup), _time_steps(exchange, steps, warmup)
    graph_ms, graph_error = -1.0, None
    if cuda_graph:
        # the rank's whole step, both all-gathers included, recorded once and replayed: recording queues nothing,
        # so a rank whose capture fails cannot leave the others waiting; the ranks vote before anyone replays
        graph = torch.cuda.CUDAGraph()
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(3):
                    step()
            torch.cuda.current_stream(dev).wait_stream(side)
            q.grad = k.grad = v.grad = factor.grad = None
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                step()
            recorded = 1.0
        except Exception as exc:
            recorded, graph_error = 0.0, repr(exc)[:300]
        vote = torch.tensor([recorded], device=dev)
        if world > 1:
            dist.all_reduce(vote, op=dist.ReduceOp.MIN)
        if vote.item() > 0:
            graph_ms = _time_steps(graph.replay, steps, warmup)
            from .hd_block_gemm_autograd import check_captured_status

            check_captured_status(dev)
    ms = torch.tensor([eager_ms, exchange_only_ms, graph_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        step_ms, exchange_ms, graph_ms = ms.tolist()
        extra = {}
        if cuda_graph:
            extra = (dict(cuda_graph_ms_per_step=graph_ms, cuda_graph_tokens_per_s=n / (graph_ms * 1e-3)) if graph_ms > 0
                     else dict(cuda_graph_error=graph_error or "capture failed on another rank"))
        print(json.dumps(dict(benchmark="sequence_parallel", n=n, ranks=world, ms_per_step=step_ms,
                              tokens_per_s=n / (step_ms * 1e-3), **extra,
                              exchange_ms_per_step=exchange_ms, exchange_share=exchange_ms / step_ms,
                              exchange_bytes_per_rank_per_direction=2 * _lib.STATE_ROWS * _lib.E_PAD * 4,
                              collective="one all-gather of the range-final fp32 states per direction (NCCL), "
                                         "summed locally in rank order")), flush=True)
    if cuda_graph:
        # a recorded graph holds the communicator's kernels: release it before the process group is torn down
        # (with the graph alive, the teardown waited until the launcher's timeout)
        graph.reset()
        del graph
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def training_step(layers: int, batch: int, n: int, steps: int, warmup: int) -> None:
    import torch.distributed as dist

    from .qwen_block import QwenOalStack

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234)                                   # same weights on every rank
    model = QwenOalStack(num_layers=layers, device=dev)
    params = model.trainable_parameters()
    opt = torch.optim.AdamW(params, lr=1e-4, weight_decay=0.0, fused=True)
    gen = torch.Generator(device=dev).manual_seed(99 + rank)  # each rank its own batch
    ids = torch.randint(0, model.embed.num_embeddings, (batch, n), generator=gen, device=dev)
    losses = []

    def step():
        opt.zero_grad(set_to_none=True)
        loss = model(ids)
        loss.backward()
        if world > 1:
            flat = torch.cat([p.grad.reshape(-1).float() for p in params])
            dist.all_reduce(flat)
            flat /= world
            off = 0
            for p in params:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad))
                off += p.numel()
        opt.step()
        losses.append(loss.detach())

    if world > 1:
        dist.barrier()
    ms = torch.tensor([_time_steps(step, steps, warmup)], device=dev, dtype=torch.float64)
    # the operator's share: its kernels timed by the library's own event pairs over one more step
    _lib.profile_enable(True)
    step()
    torch.cuda.synchronize()
    report = _lib.profile_report()
    _lib.profile_enable(False)
    op_ms = sum(v[1] for v in report.values()) if report else float("nan")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps(dict(benchmark="training_step", layers=layers, batch_per_rank=batch, n=n, ranks=world,
                              ms_per_step=ms.item(), tokens_per_s=world * batch * n / (ms.item() * 1e-3),
                              operator_ms_per_step=op_ms, operator_share=op_ms / ms.item(),
                              trainable_parameters=sum(p.numel() for p in params),
                              first_loss=float(losses[0]), last_loss=float(losses[-1]),
                              peak_memory_gb=torch.cuda.max_memory_allocated(dev) / 2**30)), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("mode", choices=["sweep", "sp", "step"])
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", default=None, help="sequence length(s), comma separated")
    ap.add_argument("--groups", default="1,4,8,16")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--cuda-graph", action="store_true", help="sp: also time the step as a CUDA graph replay")
    a = ap.parse_args()
    if a.mode == "sweep":
        ns = [int(x) for x in (a.seq or "1024,4096,16384,65536").split(",")]
        sweep(ns, [int(x) for x in a.groups.split(",")], a.steps, a.warmup)
    elif a.mode == "sp":
        sequence_parallel(int(a.seq or 32768), a.steps, a.warmup, a.cuda_graph)
    else:
        training_step(a.layers, a.batch, int(a.seq or 4096), a.steps, a.warmup)


if __name__ == "__main__":
    main()
