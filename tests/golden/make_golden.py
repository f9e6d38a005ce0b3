"""Generate the golden vectors under tests/golden/ by running the REFERENCE itself.

Run once in a container that has the reference checkout (it is imported from
the directory given with ``--reference``); the produced files are committed and
the test-suite never needs the reference again.

    python tests/golden/make_golden.py --reference <checkout of wuqianyue09/OAL> [--only name,name]

Outputs
  kat_two_groups.json, kat_different_active_group_counts.json
      the two known-answer fixtures shipped (but never loaded) by the reference,
      tests/operators/fixtures/grouped_quadratic/*.json, re-emitted with the
      group lists converted to a per-dimension id table.  The generator checks
      that the reference reproduces its own recorded numbers before writing.
  config1.npz, mixed.npz, qwen_small.npz
      outputs and gradients of ``grouped_quadratic_reference`` /
      ``oal_attention(execution="reference")`` + autograd in fp64 on the seeded
      inputs of ``oal_b200.synthetic`` (only a digest of the inputs is stored:
      the tests regenerate them from the seed and compare the digest).
  qwen_n4096_rows.npz
      a long-sequence check: one KV head with its 7 query heads at N=4096,
      outputs / gradients of the reference's own chunked production path
      (``hd_attention.grouped_causal_attention(precision="fp32_ieee")``, CPU)
      and of the fp64 dense statement, stored for every 64th token only.
  config2_rows.npz
      the benchmarked configuration itself (B=4, 14 query / 2 KV heads, N=4096,
      G=8, the inputs of ``bench.py`` rank 0): every 64th token of batch rows 0
      and 3, all 14 heads, from the reference's chunked fp32 path and from the
      fp64 dense statement; dfactor over the whole batch.
  sweep_rows.npz
      one cell per group count G in {1, 4, 8, 16} of the sequence-length x
      group-count sweep at N=4096 (B=1, 14 / 2 heads): every 128th token, both
      references.
  long_rows.npz
      the sequence-parallel configuration (B=1, 14 / 2 heads, N=32768, chunk 64):
      every 1024th token of the reference's chunked fp32 path (the quadratic dense
      statement is not evaluated at this length).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from oal_b200 import synthetic  # noqa: E402


def _np(t):
    return t.detach().to(torch.float32).numpy()


def _reference_grads(ref, case, dtype=torch.float64):
    """Run the reference oracle + autograd for an OalCase; return dict of tensors."""
    from oal_attention import oal_attention
    from oal_attention.grouped_reference import grouped_quadratic_reference

    q, k, v = (t.to(dtype).clone().requires_grad_() for t in (case.q, case.k, case.v))
    res = {}
    if case.factor is not None:
        factor = case.factor.to(dtype).clone().requires_grad_()
        out, num, den = oal_attention(q, k, v, case.dim_groups, factor, scale=case.scale,
                                      kernel_eps=case.kernel_eps, execution="reference",
                                      return_unnormalized=True)
        leaves = dict(dq=q, dk=k, dv=v, dfactor=factor)
    else:
        a, b, c = (t.to(dtype).clone().requires_grad_() for t in (case.A, case.B, case.C))
        out, num, den = grouped_quadratic_reference(q, k, v, case.dim_groups, a, b, c, scale=case.scale,
                                                    kernel_eps=case.kernel_eps, causal=True)
        leaves = dict(dq=q, dk=k, dv=v, dA=a, dB=b, dC_raw=c)
    loss = (out * case.grad_out.to(dtype)).sum()
    if case.grad_num is not None:
        loss = loss + (num * case.grad_num.to(dtype)).sum()
    if case.grad_den is not None:
        loss = loss + (den * case.grad_den.to(dtype)).sum()
    loss.backward()
    res.update(out=out, num=num, den=den)
    for name, leaf in leaves.items():
        res[name] = leaf.grad
    if "dC_raw" in res:
        res["dC_sym"] = res["dC_raw"] + res["dC_raw"].transpose(-1, -2)
    return res


def _save(name, case, res, extra=None):
    arrays = {k: _np(v) for k, v in res.items()}
    arrays["input_digest"] = np.frombuffer(
        synthetic.tensor_digest(case.q, case.k, case.v, case.dim_groups).encode(), dtype=np.uint8)
    if extra:
        arrays.update(extra)
    np.savez_compressed(HERE / f"{name}.npz", **arrays)
    print(f"wrote {name}.npz:", {k: v.shape for k, v in arrays.items()})


def emit_kats(ref_root: Path):
    from oal_attention import oal_attention

    src = ref_root / "tests" / "operators" / "fixtures" / "grouped_quadratic"
    for stem in ("two_groups", "different_active_group_counts"):
        rec = json.loads((src / f"{stem}.json").read_text())
        d = rec["head_dimension"]
        table = []
        for head_groups in rec["groups"]:
            ids = [0] * d
            for gid, dims in enumerate(head_groups):
                for dim in dims:
                    ids[dim] = gid
            table.append(ids)
        q = torch.tensor(rec["q"], dtype=torch.float64)
        k = torch.tensor(rec["k"], dtype=torch.float64)
        v = torch.tensor(rec["v"], dtype=torch.float64)
        factor = torch.tensor(rec["packed_lower_triangular"], dtype=torch.float64)
        out, num, den = oal_attention(q, k, v, torch.tensor(table, dtype=torch.int32), factor,
                                      scale=rec["scale"], kernel_eps=rec["kernel_eps"],
                                      execution="reference", return_unnormalized=True)
        for got, key in ((out, "output"), (num, "numerator"), (den, "denominator")):
            want = torch.tensor(rec[key], dtype=torch.float64)
            assert torch.allclose(got, want, rtol=1e-12, atol=1e-13), (stem, key)
        emitted = dict(source=f"tests/operators/fixtures/grouped_quadratic/{stem}.json",
                       scale=rec["scale"], kernel_eps=rec["kernel_eps"], dim_groups=table,
                       factor=rec["packed_lower_triangular"], q=rec["q"], k=rec["k"], v=rec["v"],
                       numerator=rec["numerator"], denominator=rec["denominator"], output=rec["output"])
        (HERE / f"kat_{stem}.json").write_text(json.dumps(emitted))
        print("wrote", f"kat_{stem}.json")


def emit_config1():
    seed = 0
    while True:
        case = synthetic.config1_case(seed)
        try:
            res = _reference_grads(None, case)
        except RuntimeError:
            seed += 1
            continue
        if res["den"].min() > 0:
            break
        seed += 1
    _save("config1", case, res, dict(seed=np.array(seed)))


def emit_mixed():
    case = synthetic.mixed_case(0)
    _save("mixed", case, _reference_grads(None, case))


def emit_qwen_small():
    case = synthetic.qwen_head_case(0, batch=1, n=320, hq=7, hkv=1, g=8, bf16=True)
    _save("qwen_small", case, _reference_grads(None, case))


def emit_qwen_rows():
    """N=4096, one KV head: reference chunked fp32 path + fp64 dense statement, every 64th row."""
    from oal_attention.hd_attention import grouped_causal_attention
    from oracle import oal_oracle as orc

    case = synthetic.qwen_head_case(1, batch=1, n=4096, hq=7, hkv=1, g=8, bf16=True)
    stride = 64
    # (i) the reference's own production path on the CPU, fp32
    q, k, v = (t.clone().requires_grad_() for t in (case.q, case.k, case.v))
    factor = case.factor.clone().requires_grad_()
    out, num, den = grouped_causal_attention(q, k, v, case.dim_groups, factor, scale=case.scale,
                                             kernel_eps=case.kernel_eps, token_block=64,
                                             feature_wave_blocks=4, precision="fp32_ieee",
                                             backward_schedule="shared_wave")
    out.backward(case.grad_out)
    hd = dict(out=out, num=num, den=den, dq=q.grad, dk=k.grad, dv=v.grad, dfactor=factor.grad)
    # (ii) fp64 dense statement, one query head at a time
    a, b, c = orc.expand_factor(case.factor, 7, case.kernel_eps)
    acc = {}
    for h in range(7):
        r = orc.dense_backward(case.q[:, h:h + 1].double(), case.k.double(), case.v.double(),
                               case.dim_groups, a[h:h + 1], b[h:h + 1], c[h:h + 1], scale=case.scale,
                               grad_out=case.grad_out[:, h:h + 1].double())
        for name in ("out", "num", "den", "dq"):
            acc.setdefault(name, []).append(r[name])
        for name in ("dk", "dv"):
            acc[name] = acc.get(name, 0) + r[name]
        for name in ("dA", "dB", "dC"):
            acc.setdefault(name, []).append(r[name])
    dense = {n_: (torch.cat(v_, 1) if n_ in ("out", "num", "den", "dq") else
                  (torch.cat(v_, 0) if isinstance(v_, list) else v_)) for n_, v_ in acc.items()}
    arrays = {}
    for tag, res in (("hd", hd), ("dense", dense)):
        for name, t in res.items():
            if t.ndim == 4:
                t = t[:, :, ::stride]
            arrays[f"{tag}_{name}"] = t
    _save("qwen_n4096_rows", case, arrays, dict(row_stride=np.array(stride)))


def _hd_reference(case, token_block=64):
    """The reference's own chunked production path on the CPU in fp32 (forward + autograd backward)."""
    from oal_attention.hd_attention import grouped_causal_attention

    q, k, v = (t.clone().requires_grad_() for t in (case.q, case.k, case.v))
    factor = case.factor.clone().requires_grad_()
    out, num, den = grouped_causal_attention(q, k, v, case.dim_groups, factor, scale=case.scale,
                                             kernel_eps=case.kernel_eps, token_block=token_block,
                                             feature_wave_blocks=4, precision="fp32_ieee",
                                             backward_schedule="shared_wave")
    out.backward(case.grad_out)
    return dict(out=out.detach(), num=num.detach(), den=den.detach(), dq=q.grad, dk=k.grad, dv=v.grad,
                dfactor=factor.grad)


def _dense_by_head(case, batch_rows=None):
    """fp64 dense statement one (batch row, query head) at a time: O(N^2) memory per call only."""
    from oracle import oal_oracle as orc

    B, hq, n, _ = case.q.shape
    hkv = case.k.shape[1]
    rep = hq // hkv
    a, b, c = orc.expand_factor(case.factor, hq, case.kernel_eps)
    res = {name: torch.zeros_like(t, dtype=torch.float64)
           for name, t in dict(out=case.q, num=case.q, dq=case.q, dk=case.k, dv=case.v).items()}
    res["den"] = torch.zeros(B, hq, n, 1, dtype=torch.float64)
    res["dA"], res["dB"], res["dC"] = torch.zeros_like(a), torch.zeros_like(b), torch.zeros_like(c)
    for bi in (range(B) if batch_rows is None else batch_rows):
        for h in range(hq):
            kv = h // rep
            r = orc.dense_backward(case.q[bi:bi + 1, h:h + 1].double(), case.k[bi:bi + 1, kv:kv + 1].double(),
                                   case.v[bi:bi + 1, kv:kv + 1].double(), case.dim_groups, a[h:h + 1],
                                   b[h:h + 1], c[h:h + 1], scale=case.scale,
                                   grad_out=case.grad_out[bi:bi + 1, h:h + 1].double())
            for name in ("out", "num", "den", "dq"):
                res[name][bi, h] = r[name][0, 0]
            res["dk"][bi, kv] += r["dk"][0, 0]
            res["dv"][bi, kv] += r["dv"][0, 0]
            res["dA"][h] += r["dA"][0]
            res["dB"][h] += r["dB"][0]
            res["dC"][h] += r["dC"][0]
            print(f"  dense row {bi} head {h} done", flush=True)
    factor = case.factor.double().clone().requires_grad_()
    fa, fb, fc = orc.expand_factor(factor, hq, case.kernel_eps)
    ((fa * res["dA"]).sum() + (fb * res["dB"]).sum() + (fc * res["dC"]).sum()).backward()
    res["dfactor"] = factor.grad
    return res


def _rows(res, stride, batch_rows=None):
    out = {}
    for name, t in res.items():
        if t.ndim == 4:
            t = t[:, :, ::stride]
            if batch_rows is not None:
                t = t[list(batch_rows)]
        out[name] = t
    return out


def emit_config2_rows():
    """The benchmarked configuration: the inputs bench.py gives rank 0 (seed 0), both references."""
    case = synthetic.qwen_head_case(0, batch=4, n=4096, hq=14, hkv=2, g=8, bf16=True)
    stride, keep = 64, (0, 3)
    arrays = {}
    for name, t in _rows(_hd_reference(case), stride, keep).items():
        arrays[f"hd_{name}"] = t
    print("config2: reference chunked path done", flush=True)
    for name, t in _rows(_dense_by_head(case), stride, keep).items():
        arrays[f"dense_{name}"] = t
    _save("config2_rows", case, arrays, dict(row_stride=np.array(stride), batch_rows=np.array(keep)))


def emit_sweep_rows():
    """One cell per group count of the N x G sweep at N = 4096 (B=1, 14 / 2 heads)."""
    stride = 128
    arrays, digests = {}, []
    for g in (1, 4, 8, 16):
        case = synthetic.qwen_head_case(40 + g, batch=1, n=4096, hq=14, hkv=2, g=g, bf16=True)
        for name, t in _rows(_hd_reference(case), stride).items():
            arrays[f"g{g}_hd_{name}"] = _np(t)
        print(f"sweep G={g}: reference chunked path done", flush=True)
        for name, t in _rows(_dense_by_head(case), stride).items():
            arrays[f"g{g}_dense_{name}"] = _np(t)
        digests.append(synthetic.tensor_digest(case.q, case.k, case.v, case.dim_groups))
    arrays["input_digests"] = np.frombuffer("".join(digests).encode(), dtype=np.uint8)
    arrays["row_stride"] = np.array(stride)
    np.savez_compressed(HERE / "sweep_rows.npz", **arrays)
    print("wrote sweep_rows.npz:", {k: v.shape for k, v in arrays.items()})


def emit_long_rows():
    """Sequence-parallel configuration (N = 32768): every 1024th token of the reference's chunked path."""
    case = synthetic.qwen_head_case(7, batch=1, n=32768, hq=14, hkv=2, g=8, bf16=True)
    stride = 1024
    arrays = {f"hd_{name}": t for name, t in _rows(_hd_reference(case), stride).items()}
    _save("long_rows", case, arrays, dict(row_stride=np.array(stride)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_num_threads(8)
    todo = dict(kats=lambda: emit_kats(Path(args.reference)), config1=emit_config1, mixed=emit_mixed,
                qwen_small=emit_qwen_small, qwen_rows=emit_qwen_rows, config2_rows=emit_config2_rows,
                sweep_rows=emit_sweep_rows, long_rows=emit_long_rows)
    for name, fn in todo.items():
        if args.only and name not in args.only.split(","):
            continue
        fn()


if __name__ == "__main__":
    main()
