"""``ForgeEngine``: the constructor half of the trainer for post-training stacks that drive their
own loop (parity: torchtitan/experiments/forge/engine.py:37-306)."""

from .engine import ForgeEngine

__all__ = ["ForgeEngine"]
