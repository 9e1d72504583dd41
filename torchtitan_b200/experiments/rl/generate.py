"""Run the generator of a registered RL job on its own::

    python -m torchtitan_b200.experiments.rl.generate --config rl_grpo_qwen3_0_6b_alphabet_sort \\
        --prompt "Sort these names: Charlie, Alice, Bob." --max-tokens 64 --temperature 0 [--num-samples 4] [--raw-prompt]

The job's model is built (weights from ``trainer.checkpoint.initial_load_path`` / ``trainer.hf_assets_path`` when the
config asks for an initial load, random otherwise), the prompt goes through the job's chat renderer unless
``--raw-prompt``, and ``--num-samples`` requests are decoded together by the continuous-batching engine.

Parity: torchtitan/experiments/rl/generate.py:48-256 (there: the vLLM engine with the trainer's model registered).
"""

from __future__ import annotations

import argparse
import asyncio
import dataclasses
import time

from torchtitan_b200.utils.logging import init_logger, logger

from . import config_registry
from .engine import GenerationEngine, place_model_
from .renderer import ChatRenderer

_DEFAULT_PROMPT = ("Sort these names alphabetically and put the final answer inside "
                   "<alphabetical_sorted>...</alphabetical_sorted>: Charlie, Alice, Bob.")


def _parse(argv):
    ap = argparse.ArgumentParser(description="generate with the model and sampling settings of an RL job")
    ap.add_argument("--config", default="rl_grpo_debug_alphabet_sort")
    ap.add_argument("--prompt", default=_DEFAULT_PROMPT)
    ap.add_argument("--raw-prompt", action="store_true", help="tokenise --prompt as it is instead of rendering a chat turn")
    ap.add_argument("--max-tokens", type=int, default=None)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--num-samples", type=int, default=1)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--device", default=None)
    return ap.parse_args(argv)


def generate(argv: list[str] | None = None) -> list[str]:
    import torch

    args = _parse(argv)
    factory = getattr(config_registry, args.config, None)
    if not callable(factory):
        raise ValueError(f"unknown RL config {args.config!r}")
    job = factory()
    job.validate()
    from torchtitan_b200.components.quantization import apply_converters
    from torchtitan_b200.models import get_model_spec

    t = job.trainer
    spec = t.model_spec or get_model_spec(t.model.name, t.model.flavor)
    apply_converters(spec.model, t.model.converters, t)
    device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    model = spec.model.build()
    model.init_states(seed=t.debug.seed or 0)
    model = place_model_(model, device, torch.bfloat16 if device.type == "cuda" else torch.float32)
    if t.checkpoint.initial_load_path or t.checkpoint.initial_load_in_hf:
        from torchtitan_b200.scripts.convert_hf import load_hf_into

        load_hf_into(model, spec, t.checkpoint.initial_load_path or t.hf_assets_path)
    import os

    if job.byte_tokenizer or not os.path.isdir(t.hf_assets_path):
        from torchtitan_b200.components.tokenizer import ByteTokenizer

        tok = ByteTokenizer()
    else:
        from torchtitan_b200.components.tokenizer import HuggingFaceTokenizer

        tok = HuggingFaceTokenizer(tokenizer_path=t.hf_assets_path)
    renderer = ChatRenderer(job.controller.renderer, tokenizer=tok)
    ids = (tok.encode(args.prompt, add_bos=True, add_eos=False) if args.raw_prompt
           else renderer.render_ids(messages=[{"role": "user", "content": args.prompt}]))
    over = {k: v for k, v in (("max_tokens", args.max_tokens), ("temperature", args.temperature), ("top_p", args.top_p))
            if v is not None}
    sampling = dataclasses.replace(job.controller.sampling, **over,
                                   stop_sequences=[*job.controller.sampling.stop_sequences, *renderer.stop_sequences])
    eng_cfg = dataclasses.replace(job.generator, max_num_seqs=max(args.num_samples, 1), threaded=False)

    async def run():
        eng = GenerationEngine(eng_cfg, model=model, eos_id=int(tok.eos_id) if tok.eos_id is not None else None)
        t0 = time.perf_counter()
        outs = await asyncio.gather(*(eng.generate(ids, request_id=f"sample={i}", sampling_config=dataclasses.replace(
            sampling, seed=None if args.seed is None else args.seed + i)) for i in range(args.num_samples)))
        dt = time.perf_counter() - t0
        await eng.close()
        n = sum(len(o.token_ids) for o in outs)
        logger.info(f"{n} tokens in {dt:.2f} s ({n / dt:.1f} tokens/s, {eng.steps} engine steps, prompt {len(ids)} tokens)")
        return outs

    texts = []
    for i, o in enumerate(asyncio.run(run())):
        texts.append(tok.decode(o.token_ids))
        logger.info(f"[{i}] ({o.finish_reason}, {len(o.token_ids)} tokens) {texts[-1]!r}")
    return texts


if __name__ == "__main__":
    init_logger()
    generate()
