"""Checkpoint conversion between the native DCP layout and Hugging Face safetensors.

    python -m torchtitan_b200.scripts.convert_hf from_hf --module llama3 --flavor 8B --hf-dir ./assets/hf/Llama-3.1-8B \
        --out ./outputs/checkpoint/step-0
    python -m torchtitan_b200.scripts.convert_hf to_hf --module llama3 --flavor 8B --checkpoint ./outputs/checkpoint/step-1000 \
        --out ./hf_export

Both directions run on one CPU process and hold one copy of the weights in host memory.  Names
and fused-weight splits go through the family's state-dict adapter, so the result is what the
trainer's ``checkpoint.initial_load_in_hf`` / ``last_save_in_hf`` paths produce.
Parity: scripts/checkpoint_conversion/convert_from_hf.py and convert_to_hf.py.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from torchtitan_b200.models import get_model_spec
from torchtitan_b200.models.common.module import iter_checkpoint_slices


def _native_template(spec):
    """``{checkpoint name: (param fqn, row range or None, shape)}`` from a meta-device build."""
    with torch.device("meta"):
        model = spec.model.build()
    fused = dict(iter_checkpoint_slices(model))
    out = {}
    for k, p in list(model.named_parameters()) + [(k, b) for k, b in model.named_buffers() if k.endswith("expert_bias_E")]:
        if k in fused:
            for name, a, b in fused[k]:
                out[name] = (k, (a, b), (b - a, *p.shape[1:]))
        else:
            out[k] = (k, None, tuple(p.shape))
    return out


def from_hf(args) -> None:
    import torch.distributed.checkpoint as dcp
    from safetensors import safe_open

    spec = get_model_spec(args.module, args.flavor)
    adapter = spec.state_dict_adapter(spec.model, args.hf_dir)
    hf = {}
    for fn in sorted(f for f in os.listdir(args.hf_dir) if f.endswith(".safetensors")):
        with safe_open(os.path.join(args.hf_dir, fn), framework="pt", device="cpu") as f:
            for k in f.keys():
                hf[k] = f.get_tensor(k)
    native = adapter.from_hf(hf)
    template = _native_template(spec)
    missing = sorted(set(template) - set(native))
    if missing:
        raise SystemExit(f"the Hugging Face checkpoint lacks {len(missing)} tensors, e.g. {missing[:3]}")
    state = {f"model.{k}": native[k].to(getattr(torch, args.dtype)).contiguous() for k in template}
    os.makedirs(args.out, exist_ok=True)
    dcp.save(state, checkpoint_id=args.out, no_dist=True)
    print(f"wrote {len(state)} tensors to {args.out}")


@torch.no_grad()
def load_hf_into(model, spec, hf_dir: str) -> int:
    """Copy the ``*.safetensors`` weights of a Hugging Face folder into an already built native ``model`` (any device
    or dtype) through the family's state-dict adapter; returns the number of native tensors written."""
    from safetensors import safe_open

    adapter = spec.state_dict_adapter(spec.model, hf_dir)
    hf = {}
    files = sorted(f for f in os.listdir(hf_dir) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"{hf_dir}: no .safetensors files")
    for fn in files:
        with safe_open(os.path.join(hf_dir, fn), framework="pt", device="cpu") as f:
            for k in f.keys():
                hf[k] = f.get_tensor(k)
    native = adapter.from_hf(hf)
    fused = dict(iter_checkpoint_slices(model))
    n = 0
    for k, p in model.named_parameters():
        for name, a, b in fused.get(k, [(k, None, None)]):
            if name not in native:
                raise KeyError(f"{hf_dir}: the checkpoint lacks '{name}'")
            (p if a is None else p[a:b]).copy_(native[name].to(p.device, p.dtype))
            n += 1
    return n


def to_hf(args) -> None:
    import torch.distributed.checkpoint as dcp
    from safetensors.torch import save_file

    spec = get_model_spec(args.module, args.flavor)
    adapter = spec.state_dict_adapter(spec.model, None)
    template = _native_template(spec)
    state = {f"model.{k}": torch.empty(shape, dtype=getattr(torch, args.dtype)) for k, (_, _, shape) in template.items()}
    dcp.load(state, checkpoint_id=args.checkpoint, no_dist=True)
    hf = {k: v.contiguous() for k, v in adapter.to_hf({k[len("model."):]: v for k, v in state.items()}).items()}
    os.makedirs(args.out, exist_ok=True)
    save_file(hf, os.path.join(args.out, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(args.out, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": sum(v.numel() * v.element_size() for v in hf.values())},
                   "weight_map": {k: "model.safetensors" for k in hf}}, f, indent=2)
    print(f"wrote {len(hf)} tensors to {args.out}")


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("from_hf", "to_hf"):
        p = sub.add_parser(name)
        p.add_argument("--module", required=True)
        p.add_argument("--flavor", required=True)
        p.add_argument("--out", required=True)
        p.add_argument("--dtype", default="bfloat16")
        if name == "from_hf":
            p.add_argument("--hf-dir", required=True)
        else:
            p.add_argument("--checkpoint", required=True)
    args = ap.parse_args(argv)
    {"from_hf": from_hf, "to_hf": to_hf}[args.cmd](args)


if __name__ == "__main__":
    main()
