"""Numerics debugging: record per-module activation (and gradient) statistics of one step and
compare two recordings to find the first module where two runs diverge.

    with ActivationTracer(model, grads=True) as tr:
        loss = step(model)
    tr.save("run_a.json")
    print(compare_traces("run_a.json", "run_b.json"))

Each record holds shape, dtype, mean, std, absmax, the count of non-finite values and a content
hash of the tensor's bytes, keyed by the module's fully-qualified name in execution order.
``OperatorTracer`` records at operator granularity instead (every ATen / ``tb200`` operator call through a
``TorchDispatchMode``, tagged with the module that was executing), and ``html_report`` renders a comparison as a
self-contained HTML table with the diverging rows highlighted.  Parity:
agent_tooling/numerics_debugging/activation_tracer.py and compare_numerics.py.
"""

from __future__ import annotations

import hashlib
import json

import torch
import torch.nn as nn

__all__ = ["ActivationTracer", "OperatorTracer", "compare_traces", "html_report", "tensor_record"]


def tensor_record(t: torch.Tensor) -> dict:
    f = t.detach().float()
    fin = torch.isfinite(f)
    ok = f[fin] if not bool(fin.all()) else f
    raw = t.detach().contiguous().cpu().reshape(-1)     # (0-d tensors cannot be viewed as bytes)
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


class OperatorTracer:
    """Records the tensor outputs of every operator executed inside the ``with`` block (forward and backward),
    keyed by operator name and by the innermost module whose forward was running.  Much finer than
    ``ActivationTracer`` (and much slower: every output is hashed on the host): meant for one small step."""

    def __init__(self, model: nn.Module | None = None, *, skip: tuple[str, ...] = ("aten.detach", "aten.view", "aten.t.",
                                                                                    "aten.transpose", "aten.slice",
                                                                                    "aten.alias", "aten.empty")):
        self.model, self.skip = model, skip
        self.records: list[dict] = []
        self._stack: list[str] = []
        self._handles = []
        self._mode = None

    def __enter__(self):
        from torch.utils._python_dispatch import TorchDispatchMode

        tracer = self

        class _Mode(TorchDispatchMode):
            def __torch_dispatch__(self, func, types, args=(), kwargs=None):
                out = func(*args, **(kwargs or {}))
                name = str(func)
                if not any(name.startswith(s) for s in tracer.skip):
                    outs = out if isinstance(out, (tuple, list)) else (out,)
                    for i, t in enumerate(outs):
                        if isinstance(t, torch.Tensor) and t.numel() and t.is_floating_point():
                            tracer.records.append({"name": f"{tracer._stack[-1] if tracer._stack else '<top>'}::{name}",
                                                   "kind": "op", "index": i, **tensor_record(t)})
                return out

        if self.model is not None:
            for mname, mod in self.model.named_modules():
                self._handles.append(mod.register_forward_pre_hook(self._push(mname or "<root>")))
                self._handles.append(mod.register_forward_hook(self._pop))
        self._mode = _Mode()
        self._mode.__enter__()
        return self

    def _push(self, name):
        def hook(_mod, _args):
            self._stack.append(name)
        return hook

    def _pop(self, _mod, _args, _out):
        if self._stack:
            self._stack.pop()
        return None

    def __exit__(self, *exc):
        self._mode.__exit__(*exc)
        for h in self._handles:
            h.remove()
        self._handles.clear()

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.records, f)


def _load_trace(x):
    if isinstance(x, str):
        with open(x) as f:
            return json.load(f)
    return x.records if hasattr(x, "records") else x


def html_report(a, b, path: str, *, rtol: float = 1e-3, atol: float = 1e-6, title: str = "numerics comparison") -> int:
    """Write a self-contained HTML table of two traces side by side; rows whose statistics differ beyond the
    tolerance are highlighted, bit-identical rows greyed.  Returns the number of diverging rows."""
    import html

    ra, rb = _load_trace(a), _load_trace(b)
    rows, bad_rows = [], 0
    for i in range(max(len(ra), len(rb))):
        x = ra[i] if i < len(ra) else None
        y = rb[i] if i < len(rb) else None
        if x is None or y is None or (x["name"], x["kind"], x["index"]) != (y["name"], y["kind"], y["index"]):
            rows.append(("order", i, x, y))
            bad_rows += 1
            continue
        if x["hash"] == y["hash"]:
            rows.append(("same", i, x, y))
            continue
        bad = any(abs(x[k] - y[k]) > atol + rtol * max(abs(x[k]), abs(y[k])) for k in ("mean", "std", "absmax"))
        bad = bad or x["nonfinite"] != y["nonfinite"]
        bad_rows += int(bad)
        rows.append(("diff" if bad else "close", i, x, y))
    css = ("body{font-family:monospace;font-size:12px} table{border-collapse:collapse} td,th{border:1px solid #ccc;padding:2px 6px}"
           " tr.same{color:#999} tr.diff{background:#fdd} tr.order{background:#fc8} tr.close{background:#ffd}")
    out = [f"<html><head><meta charset='utf-8'><title>{html.escape(title)}</title><style>{css}</style></head><body>",
           f"<h3>{html.escape(title)}</h3><p>{len(ra)} vs {len(rb)} records, {bad_rows} diverging</p><table>",
           "<tr><th>#</th><th>name</th><th>kind</th><th>shape</th><th>mean a</th><th>mean b</th><th>std a</th><th>std b</th>"
           "<th>absmax a</th><th>absmax b</th><th>nonfinite a / b</th></tr>"]

    def cell(r, k):
        return "" if r is None else (f"{r[k]:.6g}" if isinstance(r[k], float) else html.escape(str(r[k])))

    for cls, i, x, y in rows:
        r = x or y
        out.append(f"<tr class='{cls}'><td>{i}</td><td>{html.escape(r['name'])}</td><td>{r['kind']}[{r['index']}]</td>"
                   f"<td>{cell(r, 'shape')}</td><td>{cell(x, 'mean')}</td><td>{cell(y, 'mean')}</td><td>{cell(x, 'std')}</td>"
                   f"<td>{cell(y, 'std')}</td><td>{cell(x, 'absmax')}</td><td>{cell(y, 'absmax')}</td>"
                   f"<td>{cell(x, 'nonfinite')} / {cell(y, 'nonfinite')}</td></tr>")
    out.append("</table></body></html>")
    with open(path, "w") as f:
        f.write("\n".join(out))
    return bad_rows


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
    ap.add_argument("--html", default=None, help="also write an HTML report to this path")
    args = ap.parse_args(argv)
    print(compare_traces(args.a, args.b, rtol=args.rtol))
    if args.html:
        n = html_report(args.a, args.b, args.html, rtol=args.rtol)
        print(f"{n} diverging rows; report written to {args.html}")


if __name__ == "__main__":
    main()
