"""Benchmark of the OAL causal grouped-quadratic attention path (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward + backward of the operator over one batch of seeded synthetic input.
Workload: the Qwen2.5-0.5B attention-layer shape of the headline configuration
(B=4, 14 query / 2 KV heads, d=64, N=4096, G=8 groups {2,2,4,4,8,12,16,16}, four x20 outlier
channels, bf16 tensors, fp32 state).  With N GPUs every rank runs the same workload on its own
batch (batch x KV-head units are independent: no collective on the data path, weak scaling).

The one JSON line printed by rank 0 carries
  value      tokens/s with the inputs already resident in HBM (CUDA events, max over ranks)
  e2e        tokens/s through the public operator call with HOST tensors: pinned host -> device
             copies of q, k, v and the upstream gradient and device -> host copies of out, dq,
             dk, dv inside the timed region
  roofline   the dominant kernel against the measured bf16 tensor peak (MEASURED_PEAKS.json)
  cpu_baseline  the CPU oracle's chunked implementation of the same path on this box's cores
               (single-rank runs only: under torchrun the other ranks would sit in a barrier meanwhile)
  strong     the fixed-size split: the one B=4 call of the headline configuration sharded by
             (batch row, KV head) unit over the ranks (oal_b200.unit_sharding), same timing rules;
             timed twice, with every launch queued from Python (`eager`) and as a CUDA graph replay
             (`cuda_graph`, oal_b200.captured_step); the block's own tokens_per_s is the faster one (`mode`)
--impl reference times that CPU implementation alone (the reference is Python/torch CPU code for
this path; the oracle restates it): every step is one forward + backward over a bounded sample of
the workload (one batch row, cut shorter if this host is slow), timed for exactly --steps steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = dict(batch=4, hq=14, hkv=2, n=4096, g=8)
D = 64
METRIC = "oal_attention_fwd_bwd_tokens_per_s"


KERNEL_CHUNK = 128      # tokens per chunk of the state scan the kernels run (the reference's default plan uses 64)


def flop_per_token(hq: int, hkv: int, t: int = 64) -> float:
    """Algorithmic FLOPs per token position (multiply-add = 2, causal half only, no padding):
    (Hq+Hkv) 6 F E for the state GEMMs + Hq 3 (D+E)(T+1) for the intra-chunk ones."""
    f, e = 1 + D + D * (D + 1) // 2, D + 1
    return (hq + hkv) * 6 * f * e + hq * 3 * (D + e) * (t + 1)


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(tflops=float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 1420.0))),
                    tflops_burst=float(d.get("bf16_tflops", d.get("bf16_tflops_sustained", 1590.0))),
                    hbm=float(d.get("hbm_gbs", 6454.6)), source="measured")
    return dict(tflops=1400.0, tflops_burst=1590.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """SM clocks and throttle reasons (read-only) while the GPU is under load.

    A separate ``nvidia-smi`` process does the sampling, so that the Python thread that launches the
    kernels cannot starve it; samples are kept when their timestamp lies inside the window the caller
    marks (warm-up and timed steps).  Without nvidia-smi an NVML thread in this process is used.
    """

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.max_mhz, self.bits = index, [], None, 0
        self.stop, self.thread, self.error, self.proc = threading.Event(), None, None, None
        self.t_begin = self.t_end = None

    def _uuid(self):
        uuid = str(torch.cuda.get_device_properties(self.index).uuid)
        return uuid if uuid.startswith("GPU-") else "GPU-" + uuid

    def _run(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            try:
                handle = pynvml.nvmlDeviceGetHandleByUUID(self._uuid())
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            while not self.stop.is_set():
                now = time.time()
                mhz = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                try:
                    bits = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                except Exception:
                    bits = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                self.samples.append((now, mhz, bits))
                time.sleep(0.005)
        except Exception as exc:      # NVML missing: report no samples rather than fail the run
            self.error = repr(exc)

    def __enter__(self):
        import shutil
        import subprocess

        if self.index < 0:             # ranks other than 0 do not sample (rank 0 prints the line)
            return self
        smi = shutil.which("nvidia-smi")
        if smi:
            try:
                self.proc = subprocess.Popen([smi, f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                              "-i", self._uuid(), "-lms", "20"], stdout=subprocess.PIPE,
                                             stderr=subprocess.DEVNULL, text=True)
            except Exception as exc:
                self.error, self.proc = repr(exc), None
        if self.proc is None:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        time.sleep(0.3)               # let the sampler come up before the load starts
        return self

    def begin(self):
        self.t_begin = time.time()

    def end(self):
        self.t_end = time.time()

    def __exit__(self, *exc):
        if self.index < 0:
            self.window = []
            return
        if self.t_end is None:
            self.end()
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=5)
        if self.proc is not None:
            import datetime

            self.proc.terminate()
            try:
                text, _ = self.proc.communicate(timeout=5)
            except Exception:
                self.proc.kill()
                text = ""
            for line in text.splitlines():
                f = [x.strip() for x in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    mhz, self.max_mhz = float(f[1]), float(f[2])
                except ValueError:
                    continue
                bits = sum(bit for bit, col in ((0x8, 3), (0x40, 4), (0x20, 5), (0x4, 6)) if f[col] == "Active")
                self.samples.append((ts, mhz, bits))
        lo, hi = self.t_begin or 0.0, self.t_end
        kept = [(m, b) for t, m, b in self.samples if lo <= t <= hi]
        self.window = kept
        for _, b in kept:
            self.bits |= b

    def summary(self) -> dict:
        reasons = sorted(name for bit, name in self.REASONS.items() if self.bits & bit)
        mhz = [m for m, _ in self.window]
        out = dict(sm_mhz=statistics.median(mhz) if mhz else None, sm_max_mhz=self.max_mhz,
                   reasons=reasons, samples=len(mhz), sampler="nvidia-smi" if self.proc is not None else "nvml")
        if self.error:
            out["error"] = self.error
        return out


# --------------------------------------------------------------------------------------
# CPU arm: the oracle's chunked implementation (restating the reference's production path)
# --------------------------------------------------------------------------------------
def host_thread_setup() -> dict:
    """Use every core this process may run on, whatever a launcher put into the environment (torchrun
    exports OMP_NUM_THREADS=1); returns what was found, for the JSON line."""
    try:
        allowed = len(os.sched_getaffinity(0))
    except AttributeError:
        allowed = os.cpu_count() or 1
    info = dict(cpu_count=os.cpu_count(), affinity=allowed, omp_env=os.environ.get("OMP_NUM_THREADS"))
    torch.set_num_threads(max(1, allowed))
    info["threads"] = torch.get_num_threads()
    return info


def cpu_reference_run(steps: int, warmup: int, budget_s: float = 150.0) -> dict:
    """`steps` timed forward + backward passes of the oracle's chunked implementation after `warmup` untimed
    ones.  A step covers one batch row of the workload; if a probe shows that the whole run would not fit
    `budget_s`, the row is cut to a shorter prefix (the algorithm is linear in N, tokens/s stays comparable)."""
    from oal_b200 import synthetic
    from oracle import oal_oracle as orc

    host = host_thread_setup()
    full = dict(batch=1, hq=WORKLOAD["hq"], hkv=WORKLOAD["hkv"], n=WORKLOAD["n"], g=WORKLOAD["g"])
    case = synthetic.qwen_head_case(0, bf16=True, **full)
    a, b, c = orc.expand_factor(case.factor, full["hq"], case.kernel_eps, torch.float32)

    def one(n):
        t0 = time.perf_counter()
        orc.chunked_forward_backward(case.q[:, :, :n], case.k[:, :, :n], case.v[:, :, :n], case.dim_groups, a, b, c,
                                     scale=case.scale, token_block=64, grad_out=case.grad_out[:, :, :n])
        return time.perf_counter() - t0

    one(256)                                           # first-call costs (thread pool, allocator)
    per_token = one(512) / 512
    n = full["n"]
    while n > 512 and per_token * n * (steps + warmup) > budget_s:
        n //= 2
    for _ in range(warmup):
        one(n)
    times = [one(n) for _ in range(steps)]
    mean = sum(times) / len(times)
    return dict(tokens_per_s=n / mean, mean_s=mean, best_s=min(times), cores=host["affinity"], threads=host["threads"],
                host=host, steps=steps, warmup=warmup,
                sample=f"one batch row of the workload (B=1, Hq=14, Hkv=2, N={n} of 4096, G=8), fp32, chunk 64, "
                       f"mean of {steps} steps after {warmup} warm-up")


def cpu_config1_run() -> dict:
    """BASELINE config 1 exactly as specified, on the CPU: cumulative-state statement + autograd, fp32,
    B=1, Hq=Hkv=2, N=256, d=64, G=4 (the reference oracle's algorithm)."""
    from oal_b200 import synthetic
    from oracle import oal_oracle as orc

    case = synthetic.config1_case(0)
    best = None
    for it in range(3):
        q, k, v = (t.clone().requires_grad_() for t in (case.q, case.k, case.v))
        a, b, c = (t.clone().requires_grad_() for t in (case.A, case.B, case.C))
        t0 = time.perf_counter()
        out, _, _ = orc.state_forward(q, k, v, case.dim_groups, a, b, c, scale=case.scale)
        out.backward(case.grad_out)
        dt = time.perf_counter() - t0
        if it > 0:
            best = dt if best is None else min(best, dt)
    return dict(value=256 / best, unit="tokens/s", seconds=best, cores=torch.get_num_threads(),
                sample="config 1 (B=1, H=2, N=256, G=4), cumulative-state statement + autograd, fp32, best of 2 after 1 warm-up")


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = cpu_reference_run(max(1, args.steps), max(0, args.warmup))
    line = dict(metric=METRIC, value=r["tokens_per_s"], unit="tokens/s", n_gpus=args.gpus, steps=r["steps"],
                warmup=r["warmup"], ms_per_step=r["mean_s"] * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=dict(workload="qwen2.5-0.5b attention layer shape, causal fwd+bwd, one batch row per step "
                                     "(B=1, Hq=14, Hkv=2, N=4096, d=64, G=8)", chunk_tokens=64,
                            l2="inputs and state larger than L2", host=r["host"]),
                cpu_baseline=dict(value=r["tokens_per_s"], unit="tokens/s", cores=r["threads"], kind="port",
                                  sample=r["sample"]),
                e2e=dict(value=r["tokens_per_s"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
def run_gpu_arm(args) -> None:
    import torch.distributed as dist

    import oal_b200
    from oal_b200 import _lib, synthetic

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    w = dict(WORKLOAD, batch=args.batch)
    precision = args.precision
    sets = []
    for s in range(2):        # two input sets, alternated between steps
        case = synthetic.qwen_head_case(100 * rank + s, bf16=True, **w)
        host = dict(q=case.q.bfloat16().pin_memory(), k=case.k.bfloat16().pin_memory(),
                    v=case.v.bfloat16().pin_memory(), dout=case.grad_out.bfloat16().pin_memory())
        sets.append(dict(case=case, host=host, dev={k_: v_.to(dev) for k_, v_ in host.items()}))
    case0 = sets[0]["case"]
    groups = case0.dim_groups.to(dev)
    factor = case0.factor.to(dev).requires_grad_()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    q0 = sets[0]["dev"]["q"].clone().requires_grad_()
    k0 = sets[0]["dev"]["k"].clone().requires_grad_()
    v0 = sets[0]["dev"]["v"].clone().requires_grad_()
    prepared = oal_b200.prepare_grouped_hd_block_gemm(q0, k0, v0, groups, factor, scale=case0.scale,
                                                      kernel_eps=case0.kernel_eps, precision=precision,
                                                      token_block=64, feature_wave_blocks=4)

    def step(t):
        q = t["q"].detach().requires_grad_()
        k = t["k"].detach().requires_grad_()
        v = t["v"].detach().requires_grad_()
        factor.grad = None
        out, _, _ = oal_b200.run_prepared_grouped_hd_block_gemm(prepared, q, k, v, factor)
        out.backward(t["dout"])
        return out, q.grad, k.grad, v.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up, then the timed region: K steps, CUDA events on the launching stream, L2 flushed between
    # steps; the clock sampler keeps the samples taken while the GPU is under load (warm-up + timed steps)
    events = []
    with ClockSampler(local if rank == 0 else -1) as clocks:
        clocks.begin()
        for i in range(max(args.warmup, 3)):
            step(sets[i % 2]["dev"])
        barrier()
        launches0 = _lib.launch_count()
        for i in range(args.steps):
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step(sets[i % 2]["dev"])
            e1.record()
            events.append((e0, e1))
        barrier()
        clocks.end()
    launches = _lib.launch_count() - launches0
    total_ms = sum(a.elapsed_time(b) for a, b in events)
    clock_summary = clocks.summary()

    # ---- end to end through the public call with host tensors: every step copies its q, k, v and upstream
    # gradient from ONE pinned host buffer with one asynchronous copy and its out, dq, dk, dv back to ONE pinned
    # buffer with one copy (the four results are first packed on the device).  Copies run on their own streams so
    # that step i+1's upload and step i-1's download overlap step i's kernels, as any input pipeline would; the
    # timed region is wall clock from the first upload to the last download.
    names = ("q", "k", "v", "dout")
    sizes = [sets[0]["host"][n_].numel() for n_ in names]
    shapes = [tuple(sets[0]["host"][n_].shape) for n_ in names]
    offs = [0]
    for z in sizes:
        offs.append(offs[-1] + z)
    host_in = []
    for s_ in sets:                                     # pinned after set_device, one buffer per input set
        buf = torch.empty(offs[-1], dtype=torch.bfloat16).pin_memory()
        for n_, o, z in zip(names, offs, sizes):
            buf[o:o + z].copy_(s_["host"][n_].reshape(-1))
        host_in.append(buf)
    out_sizes = [sizes[0], sizes[0], sizes[1], sizes[2]]            # out, dq like q; dk like k; dv like v
    out_offs = [0]
    for z in out_sizes:
        out_offs.append(out_offs[-1] + z)
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    compute = torch.cuda.current_stream(dev)
    dev_in = [torch.empty(offs[-1], dtype=torch.bfloat16, device=dev) for _ in range(2)]
    dev_out = [torch.empty(out_offs[-1], dtype=torch.bfloat16, device=dev) for _ in range(2)]
    host_out = [torch.empty(out_offs[-1], dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    compute_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]

    def views(buf):
        return {n_: buf[o:o + z].view(sh) for n_, o, z, sh in zip(names, offs, sizes, shapes)}

    held = [None, None]

    def e2e_loop(n_steps):
        for i in range(n_steps):
            slot = i % 2
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(compute_done[slot])          # the step that last read this slot is finished
                dev_in[slot].copy_(host_in[i % 2], non_blocking=True)
                in_ready[slot].record(copy_in)
            compute.wait_event(in_ready[slot])
            compute.wait_event(out_done[slot])                  # the download that last read dev_out[slot]
            flush.fill_(i & 0xFF)
            results = step(views(dev_in[slot]))
            compute_done[slot].record(compute)
            with torch.cuda.stream(copy_out):                   # packing and download beside the next step's kernels
                copy_out.wait_event(compute_done[slot])
                for r_, o, z in zip(results, out_offs, out_sizes):
                    dev_out[slot][o:o + z].copy_(r_.reshape(-1))
                host_out[slot].copy_(dev_out[slot], non_blocking=True)
                out_done[slot].record(copy_out)
            # the step's result tensors stay allocated until their packing copies have run: the slot's previous
            # results are dropped only here, after this step waited for out_done[slot] on the compute stream
            held[slot] = results
        enqueued = time.perf_counter()
        torch.cuda.synchronize()
        return enqueued

    e2e_loop(2)
    barrier()
    t0 = time.perf_counter()
    e2e_enqueued = e2e_loop(args.steps)
    e2e_ms = (time.perf_counter() - t0) * 1e3
    e2e_host_ms = (e2e_enqueued - t0) * 1e3 / args.steps          # host time to queue one step
    barrier()
    h2d = host_in[0].numel() * host_in[0].element_size()
    d2h = host_out[0].numel() * host_out[0].element_size()

    # plain pinned-memory copy bandwidth of this rank's GPU: the floor of any end-to-end number
    def copy_gbs(dst, src, reps=5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            dst.copy_(src, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        return src.numel() * src.element_size() * reps / (e0.elapsed_time(e1) * 1e-3) / 1e9

    # rank 0 alone first (the other ranks wait), then every rank at once with both directions in flight together,
    # which is what the end-to-end loop does: on a multi-GPU host the second figure is the one that bounds it
    if rank == 0:
        solo = dict(h2d=copy_gbs(dev_in[0], host_in[0]), d2h=copy_gbs(host_out[0], dev_out[0]))
    barrier()

    def both_directions(reps=5):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        torch.cuda.synchronize()
        with torch.cuda.stream(copy_in):
            ev[0].record()
            for _ in range(reps):
                dev_in[0].copy_(host_in[0], non_blocking=True)
            ev[1].record()
        with torch.cuda.stream(copy_out):
            ev[2].record()
            for _ in range(reps):
                host_out[0].copy_(dev_out[0], non_blocking=True)
            ev[3].record()
        torch.cuda.synchronize()
        return h2d * reps / (ev[0].elapsed_time(ev[1]) * 1e-3) / 1e9, d2h * reps / (ev[2].elapsed_time(ev[3]) * 1e-3) / 1e9

    both_directions(1)
    barrier()
    conc = torch.tensor(both_directions(), dtype=torch.float64, device=dev)
    conc_min = conc.clone()
    if world > 1:
        dist.all_reduce(conc, op=dist.ReduceOp.SUM)
        dist.all_reduce(conc_min, op=dist.ReduceOp.MIN)
    copy_bw = None
    if rank == 0:
        copy_bw = dict(h2d=solo["h2d"], d2h=solo["d2h"], bytes=h2d,
                       note="rank 0 alone, 64 MiB pinned buffer, 5 back-to-back copies, one direction at a time",
                       all_ranks_both_directions=dict(h2d_sum=conc[0].item(), d2h_sum=conc[1].item(),
                                                      h2d_min_rank=conc_min[0].item(), d2h_min_rank=conc_min[1].item(),
                                                      note="every rank copying both ways at once, as the end-to-end "
                                                           "loop does: GB/s summed over ranks and of the slowest rank"))
    barrier()

    # ---- fixed-size split: the ONE headline call (B=4, 8 (batch row, KV head) units) sharded over the ranks
    from oal_b200.unit_sharding import unit_shard

    strong = None
    strong_graph, graph_error = None, None
    try:
        shard = unit_shard(WORKLOAD["batch"], WORKLOAD["hq"], WORKLOAD["hkv"], rank, world)
    except ValueError:
        shard = None
    strong_error = None
    ready = 0.0
    if shard is not None and args.batch == WORKLOAD["batch"]:
        # set-up and warm-up under a guard: a failure here must not take the headline numbers above with it,
        # and the ranks agree on whether to go on before anyone enters the timed loop
        try:
            case_s = synthetic.qwen_head_case(0, bf16=True, **WORKLOAD)      # the same inputs on every rank, cut locally
            qs, ks, vs, ds_ = (t.to(dev, torch.bfloat16).contiguous()
                               for t in shard.take(case_s.q, case_s.k, case_s.v, case_s.grad_out))
            factor_s = shard.factor_rows(case_s.factor).to(dev).requires_grad_()
            prep_s = oal_b200.prepare_grouped_hd_block_gemm(qs.clone().requires_grad_(), ks.clone().requires_grad_(),
                                                            vs.clone().requires_grad_(), groups, factor_s,
                                                            scale=case_s.scale, kernel_eps=case_s.kernel_eps,
                                                            precision=precision, token_block=64, feature_wave_blocks=4)

            def step_s():
                q_, k_, v_ = (t.detach().requires_grad_() for t in (qs, ks, vs))
                factor_s.grad = None
                out_, _, _ = oal_b200.run_prepared_grouped_hd_block_gemm(prep_s, q_, k_, v_, factor_s)
                out_.backward(ds_)

            for _ in range(max(args.warmup, 3)):
                step_s()
            torch.cuda.synchronize()
            ready = 1.0
        except Exception as exc:
            strong_error = repr(exc)[:300]
    vote = torch.tensor([ready], device=dev)
    if world > 1:
        dist.all_reduce(vote, op=dist.ReduceOp.MIN)
    if vote.item() > 0:
        barrier()
        ev = []
        for i in range(args.steps):
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step_s()
            e1.record()
            ev.append((e0, e1))
        barrier()
        strong = sum(a_.elapsed_time(b_) for a_, b_ in ev)
        # the same step recorded into a CUDA graph: at one or two units per rank the host needs about as long to
        # queue a step as the GPU to run it
        from oal_b200.captured_step import CapturedStep

        captured, graph_error = None, None
        try:
            captured = CapturedStep(prep_s, qs, ks, vs, factor_s.detach(), ds_)
            for _ in range(3):
                captured.replay()
            torch.cuda.synchronize()
        except Exception as exc:      # reported in the line; the eager numbers above stand on their own
            captured, graph_error = None, repr(exc)[:300]
        ok = torch.tensor([1.0 if captured is not None else 0.0], device=dev)
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() > 0:
            barrier()
            ev = []
            for i in range(args.steps):
                flush.fill_(i & 0xFF)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                captured.replay()
                e1.record()
                ev.append((e0, e1))
            barrier()
            strong_graph = sum(a_.elapsed_time(b_) for a_, b_ in ev)
            captured.check_status()

    # ---- per-kernel breakdown (separate pass with the library's event pairs switched on)
    _lib.profile_enable(True)
    prof_steps = min(args.steps, 5)
    for i in range(prof_steps):
        flush.fill_(i & 0xFF)
        step(sets[i % 2]["dev"])
    torch.cuda.synchronize()
    report = _lib.profile_report()
    _lib.profile_enable(False)

    times = torch.tensor([total_ms, e2e_ms, strong if strong is not None else -1.0,
                          strong_graph if strong_graph is not None else -1.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, strong_ms, strong_graph_ms = times.tolist()
    tokens_per_step = w["batch"] * w["n"] * world
    value = tokens_per_step * args.steps / (total_ms * 1e-3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms * 1e-3)

    if rank == 0:
        peaks = measured_peaks()
        fpt = flop_per_token(w["hq"], w["hkv"], 64)
        f, e = 1 + D + D * (D + 1) // 2, D + 1
        tok = w["batch"] * w["n"]
        # algorithmic FLOPs of each kernel per launch (unpadded F = 2145, E = 65; causal half, chunk 64
        # in the intra-chunk terms, exactly the terms of flop_per_token)
        intra = w["hq"] * (D + e) * 65 * tok
        kernel_flops = {
            "state_update": w["hkv"] * 2 * f * e * tok,
            "cross_read_q": w["hq"] * 2 * f * e * tok,
            "dstate_heads": w["hq"] * 2 * f * e * tok,
            "feature_grad_q": w["hq"] * 2 * f * e * tok,
            "feature_grad_k": w["hkv"] * 2 * f * e * tok,
            "cross_read_k": w["hkv"] * 2 * f * e * tok,
            "intra_forward": intra,            # s and W [v|1]
            "intra_backward_q": intra,         # dW and dq
            "intra_backward_kv": intra,        # dk and dv
        }
        # MMA FLOPs the intra-chunk kernels really execute per launch: stacked tile of 16 (G + 1) columns per
        # 16-key tile, 8 tiles per 128-token chunk under the causal mask as full 128-row tiles, the constant K
        # step (64 + 16), value + remainder chains on the backward side, dW over the 80-long value axis twice
        nr, ctas = 16 * (w["g"] + 1), w["batch"] * w["hq"] * (w["n"] // KERNEL_CHUNK)
        u_hi, u_lo = 2 * 128 * nr * 80, 2 * 128 * nr * 64
        executed_flops = {
            "intra_forward": ctas * 8 * (u_hi + 2 * 128 * 80 * 16),
            "intra_backward_q": ctas * (2 * 2 * 128 * 128 * 80 + 8 * (u_hi + u_lo + 2 * 128 * 64 * nr)),
            "intra_backward_kv": ctas * (2 * 2 * 128 * 128 * 80 + 8 * (u_hi + u_lo + 2 * 128 * 64 * nr + 2 * 128 * 80 * 16)),
        }
        kernels = {name: dict(launches=cnt, ms_per_launch=ms / max(cnt, 1), share=None)
                   for name, (cnt, ms) in report.items()}
        tot = sum(ms for _, ms in report.values()) or 1.0
        for name, (cnt, ms) in report.items():
            kernels[name]["share"] = round(ms / tot, 4)
            if name in kernel_flops:
                kernels[name]["tflops"] = round(kernel_flops[name] / (ms / max(cnt, 1) * 1e-3) / 1e12, 2)
            if name in executed_flops and precision == "bf16_tensorcore":
                kernels[name]["executed_mma_tflops"] = round(executed_flops[name] / (ms / max(cnt, 1) * 1e-3) / 1e12, 1)
        tc = {n_: k_ for n_, k_ in kernels.items() if n_ in kernel_flops}
        # DRAM bytes (read + write) per launch of each kernel in an ncu capture of ONE batch row, read from the
        # table that is kept next to the profile summaries; traffic grows in proportion to the batch
        ncu_dram_mb_per_row = {}
        table = ROOT / "profiles" / "ncu_dram_traffic_one_batch_row.txt"
        if table.exists():
            for ln in table.read_text().splitlines():
                f_ = ln.split()
                if len(f_) == 2 and not ln.startswith("#"):
                    ncu_dram_mb_per_row[f_[0]] = float(f_[1])
        roofline = None
        if tc:
            # the dominant kernel by device time
            top = max(tc, key=lambda n_: tc[n_]["ms_per_launch"] * tc[n_]["launches"])
            achieved = kernel_flops[top] / (tc[top]["ms_per_launch"] * 1e-3) / 1e12
            best = max(tc, key=lambda n_: tc[n_]["tflops"])
            roofline = dict(bound="tensor", kernel=top, achieved=round(achieved, 2), peak=peaks["tflops"],
                            unit="TFLOP/s", frac=round(achieved / peaks["tflops"], 4),
                            traffic=(round(ncu_dram_mb_per_row[top] * 1e6 * w["batch"]) if top in ncu_dram_mb_per_row
                                     else None),
                            traffic_note="bytes per launch: DRAM read + write of the kernel in an ncu capture of one "
                                         "batch row (table under profiles/), times the batch; null without the table",
                            peak_source=peaks["source"] + " (sustained bf16)",
                            note="algorithmic MMA FLOPs of the kernel (unpadded, causal half, chunk 64 as in "
                                 "flop_per_token) / its mean launch time",
                            executed_mma_tflops=tc[top].get("executed_mma_tflops"),
                            executed_note="MMA FLOPs the kernel really issues (stacked tile, remainder chain, full tiles "
                                          "under the causal mask); the achieved figure counts the reference's GEMMs for "
                                          "the same term",
                            frac_of_burst_peak=round(achieved / peaks["tflops_burst"], 4), burst_peak=peaks["tflops_burst"],
                            best_kernel=best, best_kernel_frac=round(tc[best]["tflops"] / peaks["tflops"], 4),
                            whole_step_frac=round(value / world * fpt / 1e12 / peaks["tflops"], 4),
                            whole_step_frac_of_burst_peak=round(value / world * fpt / 1e12 / peaks["tflops_burst"], 4))
        # the CPU leg runs on single-rank runs only: under torchrun the other ranks would hold their GPUs in a
        # barrier for as long as it takes, and the launcher's thread settings are not the host's own
        cpu = cpu_reference_run(2, 1, budget_s=40.0) if world == 1 and not args.no_cpu_baseline else None
        line = dict(metric=METRIC, value=value, unit="tokens/s", n_gpus=world, steps=args.steps,
                    warmup=max(args.warmup, 3), ms_per_step=total_ms / args.steps, higher_is_better=True,
                    scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
                    config=dict(workload=f"qwen2.5-0.5b attention layer shape, causal fwd+bwd (B={w['batch']} per GPU, "
                                         "Hq=14, Hkv=2, N=4096, d=64, G=8, bf16 io, fp32 state)",
                                precision=precision, parallelism=f"batch x kv-head units, {world} rank(s), no collective",
                                chunk_tokens=KERNEL_CHUNK, flop_model_chunk_tokens=64,
                                l2="256 MiB buffer written between timed steps", flop_per_token=fpt),
                    e2e=dict(value=e2e_value, unit="tokens/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                             copies_per_step=dict(h2d=1, d2h=1), copy_gbs=copy_bw, host_enqueue_ms_per_step=e2e_host_ms,
                             copy_bound_tokens_per_s=tok / max(h2d / (copy_bw["all_ranks_both_directions"]["h2d_min_rank"] * 1e9),
                                                               d2h / (copy_bw["all_ranks_both_directions"]["d2h_min_rank"] * 1e9)) * world,
                             note="uploads, kernels and downloads of neighbouring steps overlap; the slowest of the "
                                  "three bounds a step"),
                    gpu_launches=int(launches), clocks=clock_summary, roofline=roofline, kernels=kernels)
        if strong_ms > 0:
            units = WORKLOAD["batch"] * WORKLOAD["hkv"]
            tokens = WORKLOAD["batch"] * WORKLOAD["n"] * args.steps
            eager = dict(tokens_per_s=tokens / (strong_ms * 1e-3), ms_per_step=strong_ms / args.steps,
                         note="every launch queued from Python each step")
            line["strong"] = dict(eager, mode="eager", units_per_rank=units / world,
                                  workload="the one B=4 call sharded by (batch row, KV head) unit; coefficient "
                                           "gradients stay per-rank partial sums", eager=eager)
            if strong_graph_ms > 0:
                graph = dict(tokens_per_s=tokens / (strong_graph_ms * 1e-3), ms_per_step=strong_graph_ms / args.steps,
                             note="the same step recorded once with oal_b200.captured_step.CapturedStep and replayed")
                line["strong"]["cuda_graph"] = graph
                if strong_graph_ms < strong_ms:       # the headline of the block is the faster of the two ways to run it
                    line["strong"].update(tokens_per_s=graph["tokens_per_s"], ms_per_step=graph["ms_per_step"],
                                          mode="cuda_graph", note=graph["note"])
            elif graph_error:
                line["strong"]["cuda_graph"] = dict(error=graph_error)
        elif strong_error:
            line["strong"] = dict(error=strong_error)
        if cpu:
            line["cpu_baseline"] = dict(value=cpu["tokens_per_s"], unit="tokens/s", cores=cpu["threads"],
                                        kind="port", sample=cpu["sample"], host=cpu["host"])
            line["cpu_baseline_config1"] = cpu_config1_run()
        elif world > 1:
            line["cpu_baseline_note"] = "timed on single-rank runs only (see --gpus 1)"
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="bf16_tensorcore", choices=["bf16_tensorcore", "fp32_ieee"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=WORKLOAD["batch"],
                    help="batch rows per GPU (default: the headline workload's 4; smaller only for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
