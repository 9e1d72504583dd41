"""Basic layers: Linear, Embedding, RMSNorm, RoPE, SwiGLU feed-forward.

Activations use the folded-token layout ``[T, dim]`` (no batch dimension); with
sequence parallelism each tensor-parallel rank holds ``T / tp`` rows between
blocks.  A layer becomes tensor-parallel through :meth:`shard_`, called while the
model is still on the meta device: it shrinks the parameter to the local slice and
records the slice so initialisation and checkpoints stay layout independent.

Parity: torchtitan/models/common/linear.py:26-70, embedding.py:25-79,
nn_modules.py:133-147, rope.py:84-346, feed_forward.py:18-75; tensor-parallel
placements as in torchtitan/models/common/decoder_sharding.py:24-376.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal

import torch
import torch.nn as nn

from torchtitan_b200.ops import functional as OF
from torchtitan_b200.ops import reference as ref
from torchtitan_b200.parallel import sharding as shd
from torchtitan_b200.parallel import tp_ops

from .module import InitSpec, Module, set_init

__all__ = ["Linear", "Embedding", "RMSNorm", "RoPE", "FeedForward", "TPContext", "ffn_hidden_dim"]


@dataclass
class TPContext:
    group: object
    size: int
    rank: int
    sequence_parallel: bool = True
    comm: str = "nccl"
    fused: object | None = None  # parallel.tp_fused.FusedTP when comm == "nvlink" on CUDA

    def fused_ok(self, x, *weights) -> bool:
        """The in-kernel collectives need sequence parallelism, bf16 CUDA rows and 256-row shards."""
        return (self.fused is not None and self.sequence_parallel and x.is_cuda and x.dtype == torch.bfloat16
                and x.dim() == 2 and all(type(w).__name__ == "Linear" and w.bias is None for w in weights))


def _block_slices(blocks: list[int], tp_size: int, tp_rank: int) -> list[tuple[int, int]]:
    """Row ranges of the tp-local part of a parameter made of stacked blocks
    (e.g. ``[q | k | v]``); every block is split evenly over the tp ranks."""
    out, base = [], 0
    for b in blocks:
        if b % tp_size:
            raise ValueError(f"block of {b} rows is not divisible by tp={tp_size}")
        step = b // tp_size
        out.append((base + tp_rank * step, base + (tp_rank + 1) * step))
        base += b
    return out


class Linear(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        in_features: int = 0
        out_features: int = 0
        bias: bool = False
        init_std: float = 0.02
        init_kind: str = "trunc_normal"
        init_cutoff: float | None = None
        """``None`` keeps the absolute cut-offs (-2, 2); a number means +-cutoff*std."""
        row_blocks: list[int] | None = None
        """Sizes of stacked output blocks for fused weights (``[q,k,v]`` or ``[w1,w3]``)."""

    def __init__(self, config: "Linear.Config", **_):
        super().__init__(config)
        c = config
        self.in_features, self.out_features = c.in_features, c.out_features
        self.weight = nn.Parameter(torch.empty(c.out_features, c.in_features))
        a, b = (-2.0, 2.0) if c.init_cutoff is None else (-c.init_cutoff * c.init_std, c.init_cutoff * c.init_std)
        set_init(self.weight, InitSpec(kind=c.init_kind, std=c.init_std, a=a, b=b))
        self.bias = None
        if c.bias:
            self.bias = nn.Parameter(torch.empty(c.out_features))
            set_init(self.bias, InitSpec(kind="zeros"))
        self.row_blocks = list(c.row_blocks) if c.row_blocks else [c.out_features]
        self.tp_mode: str | None = None

    def shard_(self, mode: Literal["colwise", "rowwise"], tp: TPContext) -> None:
        """Keep only this rank's slice (meta device): colwise = output rows, rowwise = input columns.  The slice
        dimension comes from the declared contract (``self.sharding``)."""
        self.tp_mode = mode
        full = (self.out_features, self.in_features)
        if mode == "colwise":
            self.sharding = shd.colwise_linear(tp.sequence_parallel, blocks=len(self.row_blocks) > 1,
                                               bias=self.bias is not None)
        else:
            if self.in_features % tp.size:
                raise ValueError("rowwise shard needs in_features divisible by tp")
            self.sharding = shd.rowwise_linear(tp.sequence_parallel)
        place = self.sharding.state_shardings["weight"].on("tp")
        blocks = self.row_blocks if place.dim == 0 else None
        self.weight = shd.shard_parameter(self.weight, place, tp.size, tp.rank, blocks=blocks, full_shape=full)
        if place.dim == 0:
            if self.bias is not None:
                self.bias = shd.shard_parameter(self.bias, self.sharding.state_shardings["bias"].on("tp"), tp.size, tp.rank,
                                                blocks=self.row_blocks, full_shape=(self.out_features,))
            self.row_blocks = [b - a for a, b in self.weight._tp_slices[1]]
            self.out_features = self.weight.shape[0]
        else:
            self.in_features = self.weight.shape[1]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return OF.linear(x, self.weight, self.bias)


class Embedding(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        num_embeddings: int = 0
        embedding_dim: int = 0
        init_std: float = 1.0

    def __init__(self, config: "Embedding.Config", **_):
        super().__init__(config)
        self.num_embeddings, self.embedding_dim = config.num_embeddings, config.embedding_dim
        self.weight = nn.Parameter(torch.empty(config.num_embeddings, config.embedding_dim))
        set_init(self.weight, InitSpec(kind="normal", std=config.init_std))
        self.tp: TPContext | None = None
        self.vocab_start = 0

    def shard_(self, tp: TPContext) -> None:
        """Vocabulary-parallel: rank r owns a contiguous range of rows."""
        if self.num_embeddings % tp.size:
            raise ValueError("vocab size must divide by tp for a vocab-parallel embedding")
        self.sharding = shd.vocab_parallel_embedding(tp.sequence_parallel)
        self.weight = shd.shard_parameter(self.weight, self.sharding.state_shardings["weight"].on("tp"), tp.size, tp.rank)
        self.tp = tp
        self.vocab_start = self.weight._tp_slices[1][0][0]

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        if self.tp is None:
            return OF.embedding(tokens, self.weight)
        n = self.weight.shape[0]
        local = tokens - self.vocab_start
        mine = (local >= 0) & (local < n)
        out = OF.embedding(local.clamp(0, n - 1), self.weight)
        out = out * mine.unsqueeze(-1).to(out.dtype)
        return shd.redistribute(out, self.sharding.out_src_shardings.on("tp"), self.sharding.out_dst_shardings.on("tp"),
                                self.tp)


class RMSNorm(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        eps: float = 1e-5
        elementwise_affine: bool = True

    def __init__(self, config: "RMSNorm.Config", **_):
        super().__init__(config)
        self.eps = config.eps
        self.dim = config.dim
        if config.elementwise_affine:
            self.weight = nn.Parameter(torch.empty(config.dim))
            set_init(self.weight, InitSpec(kind="ones"))
            self.weight._replicated_over_tp = True
            self.sharding = shd.sequence_parallel_norm()
        else:
            self.register_parameter("weight", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return OF.rms_norm(x, self.weight, self.eps)


class RoPE(Module):
    """Rotary embedding table + application.

    ``style="complex"`` rotates adjacent pairs (Llama), ``"cos_sin"`` uses the
    rotate-half convention (Qwen, DeepSeek).  The table ``[max_ctx, rot_dim]``
    holds ``cos | sin`` in fp32 and is indexed by the batch's ``positions``.
    """

    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        max_context_length: int = 2048
        theta: float = 10000.0
        style: Literal["complex", "cos_sin"] = "complex"
        scaling: Literal["none", "llama", "yarn"] = "none"
        scaling_factor: float = 8.0
        low_freq_factor: float = 1.0
        high_freq_factor: float = 4.0
        original_max_position_embeddings: int = 8192
        rope_factor: float = 1.0
        beta_fast: float = 32.0
        beta_slow: float = 1.0
        original_seq_len: int = 4096
        truncate: bool = True
        mrope_sections: tuple[int, ...] | None = None
        """Multimodal RoPE: how many of the ``dim / 2`` rotary frequencies follow the temporal,
        height and width position axis.  Positions are then ``[3, T]``."""
        mrope_interleaved: bool = False
        """Frequency f follows the height axis when ``f % 3 == 1`` and ``f < 3 * sections[1]``, the width axis when
        ``f % 3 == 2`` and ``f < 3 * sections[2]``, else the temporal axis (Qwen3-VL / Qwen3.5); otherwise the axes own
        contiguous runs of frequencies (Qwen2-VL)."""

    def __init__(self, config: "RoPE.Config", **_):
        super().__init__(config)
        self.interleaved = config.style == "complex"
        if config.mrope_sections is not None and sum(config.mrope_sections) * 2 != config.dim:
            raise ValueError(f"mrope_sections {config.mrope_sections} must sum to dim / 2 = {config.dim // 2}")
        self.register_buffer("cache", torch.empty(config.max_context_length, config.dim), persistent=False)

    def _table(self) -> torch.Tensor:
        c = self.config
        return ref.rope_table(
            c.dim, c.max_context_length, c.theta, c.scaling, scaling_factor=c.scaling_factor,
            low_freq_factor=c.low_freq_factor, high_freq_factor=c.high_freq_factor,
            original_max_pos=c.original_max_position_embeddings, rope_factor=c.rope_factor,
            beta_fast=c.beta_fast, beta_slow=c.beta_slow, original_seq_len=c.original_seq_len,
            truncate=c.truncate,
        )

    def init_buffers(self, device=None) -> None:
        dev = device if device is not None else self.cache.device
        if str(dev) == "meta":
            return
        self.cache = self._table().to(dev)

    def _table_for(self, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """``(table, positions)`` for the rotation op.  Multimodal ``[3, T]`` positions become a
        per-batch table whose row t takes every frequency from the row of its own axis' position
        (``cos | sin`` halves alike), indexed by ``arange(T)``."""
        if positions.dim() == 1:
            return self.cache, positions
        secs = self.config.mrope_sections
        if secs is None:
            raise ValueError("3-axis positions need RoPE.Config.mrope_sections")
        half = self.cache.shape[1] // 2
        if self.config.mrope_interleaved:
            f = torch.arange(half, device=positions.device)
            axis_of_freq = torch.zeros(half, dtype=torch.int64, device=positions.device)
            axis_of_freq[(f % 3 == 1) & (f < 3 * secs[1])] = 1
            axis_of_freq[(f % 3 == 2) & (f < 3 * secs[2])] = 2
        else:
            axis_of_freq = torch.repeat_interleave(torch.arange(len(secs), device=positions.device),
                                                   torch.tensor(secs, device=positions.device))      # [half]
        pos_tf = positions.long()[axis_of_freq].t()                                                   # [T, half]
        f = torch.arange(half, device=positions.device)
        table = torch.cat([self.cache[pos_tf, f], self.cache[pos_tf, f + half]], dim=1).contiguous()
        return table, torch.arange(positions.shape[1], device=positions.device, dtype=torch.int64)

    def forward(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        table, pos = self._table_for(positions)
        return OF.rope(x, table, pos, self.interleaved)

    def apply_packed_(self, qkv: torch.Tensor, positions: torch.Tensor, n_rot_heads: int, head_dim: int) -> torch.Tensor:
        table, pos = self._table_for(positions)
        return OF.rope_qk_(qkv, table, pos, self.interleaved, n_rot_heads, head_dim)


def ffn_hidden_dim(dim: int, multiple_of: int = 256, ffn_dim_multiplier: float | None = None) -> int:
    """SwiGLU hidden size rule (parity: torchtitan/models/common/feed_forward.py:18-31)."""
    hidden = int(2 * 4 * dim / 3)
    if ffn_dim_multiplier is not None:
        hidden = int(ffn_dim_multiplier * hidden)
    return multiple_of * ((hidden + multiple_of - 1) // multiple_of)


class FeedForward(Module):
    """SwiGLU MLP ``w2(silu(w1 x) * w3 x)`` with ``w1``/``w3`` fused into one GEMM.

    The fused weight ``w13`` stacks ``[w1; w3]`` and is exposed to checkpoints
    under the separate names.  When constructed with ``norm`` the pre-norm is
    folded into the first GEMM's autograd function (normalised activations are
    recomputed in backward instead of stored).
    """

    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        hidden_dim: int = 0
        w13: Linear.Config = field(default_factory=Linear.Config)
        w2: Linear.Config = field(default_factory=Linear.Config)

    def __init__(self, config: "FeedForward.Config", **_):
        super().__init__(config)
        c = config
        c.w13.in_features, c.w13.out_features = c.dim, 2 * c.hidden_dim
        c.w13.row_blocks = [c.hidden_dim, c.hidden_dim]
        c.w2.in_features, c.w2.out_features = c.hidden_dim, c.dim
        self.w13 = c.w13.build()
        self.w2 = c.w2.build()
        self.hidden_dim = c.hidden_dim
        self.tp: TPContext | None = None

    def shard_(self, tp: TPContext) -> None:
        self.w13.shard_("colwise", tp)
        self.w2.shard_("rowwise", tp)
        self.hidden_dim //= tp.size
        self.tp = tp

    def checkpoint_slices(self):
        f = self.hidden_dim
        return {"w13.weight": [("w1.weight", 0, f), ("w3.weight", f, 2 * f)]}

    def forward(self, x: torch.Tensor, norm: RMSNorm | None = None) -> torch.Tensor:
        """``x`` is ``[T(/tp), dim]``; returns the same layout."""
        tp = self.tp
        if tp is not None:
            if norm is not None:
                x = norm(x)
            if tp.fused_ok(x, self.w13, self.w2) and tp.fused.supported(x.shape[0] * tp.size, x.shape[1], self.hidden_dim):
                from torchtitan_b200.parallel import tp_fused

                gu = tp_fused.all_gather_linear(x, self.w13.weight, tp.fused)
                return tp_fused.linear_reduce_scatter(OF.swiglu(gu), self.w2.weight, tp.fused)
            if tp.sequence_parallel:
                x = tp_ops.all_gather_rows(x, tp)
            else:
                x = tp_ops.copy_to_tp(x, tp)
            gu = self.w13(x)
            y = OF.swiglu_linear(gu, self.w2.weight)
            return tp_ops.reduce_scatter_rows(y, tp) if tp.sequence_parallel else tp_ops.all_reduce(y, tp)
        # the fused norm + GEMM takes a plain RMSNorm; norm subclasses (offset gains ...) run as their own module
        if type(norm) is RMSNorm and type(self.w13) is Linear and norm.weight is not None:
            gu = OF.norm_linear(x, norm.weight, self.w13.weight, norm.eps)
        else:
            gu = self.w13(norm(x) if norm is not None else x)
        if type(self.w2) is Linear:
            return OF.swiglu_linear(gu, self.w2.weight)
        return self.w2(OF.swiglu(gu))
