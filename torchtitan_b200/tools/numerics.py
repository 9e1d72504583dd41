"""Numerics debugging: record per-module activation (and gradient) statistics of one step and
compare two recordings to find the first module where two runs diverge.

    with ActivationTracer(model, grads=True) as tr:
        loss = step(model)
    tr.save("run_a.json")
    print(compare_traces("run_a.json", "run_b.json"))

Each record holds shape, dtype, mean, std, absmax, the count of non-finite values and a content
hash of the tensor's bytes, keyed by the module's fully-qualified name in execution order.
Parity: agent_tooling/numerics_debugging/activation_tracer.py and compare_numerics.py (which trace
at operator granularity and render HTML; this tool traces at module granularity and prints text).
"""

from __future__ import annotations

import hashlib
import json

import torch
import torch.nn as nn

__all__ = ["ActivationTracer", "compare_traces", "tensor_record"]


def tensor_record(t: torch.Tensor) -> dict:
    f = t.detach().float()
    fin = torch.isfinite(f)
    ok = f[fin] if not bool(fin.all()) else f
    raw = t.detach().contiguous().cpu()
    digest = hashlib.sha1(raw.view(torch.uint8).numpy().tobytes() if raw.numel() else b"").hexdigest()[:16]
    return {"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", ""),
            "mean": float(ok.mean()) if ok.numel() else 0.0, "std": float(ok.std()) if ok.numel() > 1 else 0.0,
            "absmax": float(ok.abs().max()) if ok.numel() else 0.0, "nonfinite": int((~fin).sum()), "hash": digest}


class ActivationTracer:
    def __init__(self, model: nn.Module, *, grads: bool = False, leaf_only: bool = False):
        self.model, self.grads, self.leaf_only = model, grads, leaf_only
        self.records: list[dict] = []
        self._handles = []

    def __enter__(self):
        for name, mod in self.model.named_modules():
            if self.leaf_only and any(True for _ in mod.children()):
                continue
            self._handles.append(mod.register_forward_hook(self._fwd(name or "<root>")))
            if self.grads:
                self._handles.append(mod.register_full_backward_hook(self._bwd(name or "<root>")))
        return self

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        self._handles.clear()

    def _fwd(self, name):
        def hook(_mod, _inp, out):
            for i, t in enumerate(out if isinstance(out, (tuple, list)) else (out,)):
                if isinstance(t, torch.Tensor):
                    self.records.append({"name": name, "kind": "out", "index": i, **tensor_record(t)})
        return hook

    def _bwd(self, name):
        def hook(_mod, grad_in, _grad_out):
            for i, t in enumerate(grad_in):
                if isinstance(t, torch.Tensor):
                    self.records.append({"name": name, "kind": "grad_in", "index": i, **tensor_record(t)})
        return hook

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.records, f)


def compare_traces(a, b, *, rtol: float = 1e-3, atol: float = 1e-6) -> str:
    """Text report: records present in only one trace, and the first record whose statistics differ."""
    def load(x):
        if isinstance(x, str):
            with open(x) as f:
                return json.load(f)
        return x.records if isinstance(x, ActivationTracer) else x

    ra, rb = load(a), load(b)
    lines = [f"{len(ra)} vs {len(rb)} records"]
    first = None
    identical = 0
    for i, (x, y) in enumerate(zip(ra, rb)):
        if (x["name"], x["kind"], x["index"]) != (y["name"], y["kind"], y["index"]):
            lines.append(f"execution order differs at record {i}: {x['name']}/{x['kind']} vs {y['name']}/{y['kind']}")
            break
        if x["hash"] == y["hash"]:
            identical += 1
            continue
        bad = [k for k in ("mean", "std", "absmax") if abs(x[k] - y[k]) > atol + rtol * max(abs(x[k]), abs(y[k]))]
        if x["nonfinite"] != y["nonfinite"]:
            bad.append("nonfinite")
        if bad and first is None:
            first = (i, x, y, bad)
    lines.append(f"{identical} records are bit-identical")
    if first is None:
        lines.append("no statistic differs beyond the tolerance")
    else:
        i, x, y, bad = first
        lines.append(f"first divergence at record {i}: {x['name']} ({x['kind']}[{x['index']}], shape {x['shape']}): "
                     + ", ".join(f"{k} {x[k]:.6g} vs {y[k]:.6g}" for k in bad))
    return "\n".join(lines)


def main(argv=None) -> None:
    import argparse

    ap = argparse.ArgumentParser(description="compare two activation traces")
    ap.add_argument("a")
    ap.add_argument("b")
    ap.add_argument("--rtol", type=float, default=1e-3)
    args = ap.parse_args(argv)
    print(compare_traces(args.a, args.b, rtol=args.rtol))


if __name__ == "__main__":
    main()
