"""Fetch tokenizer / config / weight files of a Hugging Face repository into ``assets/hf/<name>``.

    python -m torchtitan_b200.scripts.download_hf_assets --repo_id meta-llama/Llama-3.1-8B \
        --assets tokenizer config [safetensors index] [--local_dir ./assets/hf] [--hf_token ...]

``--assets`` picks groups of files: ``tokenizer`` (tokenizer.json, tokenizer_config.json,
special_tokens_map.json, vocab / merges, tokenizer.model), ``config`` (config.json,
generation_config.json), ``index`` (model.safetensors.index.json), ``safetensors`` (the weight
shards).  ``--additional_patterns`` adds glob patterns.  Files that do not exist in the repository
are skipped with a note.  Needs network access and the ``huggingface_hub`` package.
Parity: scripts/download_hf_assets.py.
"""

from __future__ import annotations

import argparse
import fnmatch
import os

PATTERNS = {
    "tokenizer": ["tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "vocab.json", "vocab.txt",
                  "merges.txt", "tokenizer.model", "chat_template.jinja"],
    "config": ["config.json", "generation_config.json"],
    "index": ["model.safetensors.index.json"],
    "safetensors": ["*.safetensors"],
}


def select_files(all_files: list[str], assets: list[str], extra: list[str]) -> list[str]:
    pats = [p for a in assets for p in PATTERNS[a]] + list(extra)
    return sorted(f for f in all_files if any(fnmatch.fnmatch(os.path.basename(f), p) or fnmatch.fnmatch(f, p) for p in pats))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--repo_id", required=True)
    ap.add_argument("--assets", nargs="+", default=["tokenizer"], choices=sorted(PATTERNS))
    ap.add_argument("--additional_patterns", nargs="*", default=[])
    ap.add_argument("--local_dir", default="./assets/hf")
    ap.add_argument("--hf_token", default=os.environ.get("HF_TOKEN"))
    ap.add_argument("--revision", default=None)
    args = ap.parse_args(argv)
    try:
        from huggingface_hub import hf_hub_download, list_repo_files
    except ImportError as e:
        raise SystemExit("huggingface_hub is required: pip install huggingface_hub") from e
    files = list_repo_files(args.repo_id, token=args.hf_token, revision=args.revision)
    chosen = select_files(files, args.assets, args.additional_patterns)
    if not chosen:
        raise SystemExit(f"no file of {args.repo_id} matches the requested assets {args.assets}")
    dest = os.path.join(args.local_dir, args.repo_id.split("/")[-1])
    os.makedirs(dest, exist_ok=True)
    for f in chosen:
        print(f"downloading {f}")
        hf_hub_download(args.repo_id, f, local_dir=dest, token=args.hf_token, revision=args.revision)
    print(f"{len(chosen)} file(s) in {dest}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
