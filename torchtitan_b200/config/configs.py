"""Job-level config sections shared by all trainers.

Field names and defaults follow torchtitan/config/configs.py:35-389 so a job
file written for the reference maps one-to-one onto these sections.  Fields that
only make sense for this framework (the fused NVLink paths, the B200 activation
policy) are added at the end of each section.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal

__all__ = [
    "TrainingConfig",
    "ParallelismConfig",
    "CompileConfig",
    "CommConfig",
    "DebugConfig",
    "ActivationCheckpointConfig",
    "ModelSelectConfig",
    "KernelConfig",
]


@dataclass(kw_only=True, slots=True)
class ModelSelectConfig:
    """Which registered model to train (TOML ``[model]`` section)."""

    name: str = "llama3"
    flavor: str = "debugmodel"
    converters: list[str] = field(default_factory=list)
    """Config-tree rewrites applied before build: ``mxfp8``, ``float8``, ``lora`` ..."""


@dataclass(kw_only=True, slots=True)
class TrainingConfig:
    num_tokens_per_microbatch_per_dp_rank: int = 16384
    """Tokens each data-parallel rank feeds through one forward/backward."""
    num_tokens_per_train_step: int = -1
    """Global tokens per optimizer step; -1 means one microbatch per dp rank."""
    max_context_length: int = 2048
    """Longest document (attention span); packing and the RoPE table use it."""
    max_norm: float = 1.0
    steps: int = 10000
    enable_cpu_offload: bool = False
    """Keep the sharded optimizer state (fp32 master weights, both moments: 12 bytes per parameter
    and rank) in pinned host memory; the optimizer step streams it through the GPU unit by unit."""
    disable_cuda_graphs: bool = True
    dtype: Literal["bfloat16", "float32"] = "float32"
    """Dtype of the master parameters."""
    mixed_precision_param: Literal["bfloat16", "float32"] = "bfloat16"
    """Dtype of the gathered compute parameters."""
    mixed_precision_reduce: Literal["float32"] = "float32"
    gc_freq: int = 50
    gc_debug: bool = False


@dataclass(kw_only=True, slots=True)
class ParallelismConfig:
    data_parallel_replicate_degree: int = 1
    data_parallel_shard_degree: int = -1
    fsdp_reshard_after_forward: Literal["default", "always", "never"] = "default"
    enable_fsdp_symm_mem: bool = False
    tensor_parallel_degree: int = 1
    enable_sequence_parallel: bool = True
    spmd_backend: Literal["partial_dtensor", "spmd_types", "native"] = "native"
    pipeline_parallel_degree: int = 1
    module_fqns_per_model_part: list[list[str]] | None = None
    pipeline_parallel_first_stage_less_layers: int = 1
    pipeline_parallel_last_stage_less_layers: int = 1
    pipeline_parallel_layers_per_stage: int | None = None
    pipeline_parallel_schedule: str = "1F1B"
    pipeline_parallel_schedule_csv: str | None = ""
    num_pp_microbatches: int = 1
    context_parallel_degree: int = 1
    context_parallel_load_balancer: str | None = "headtail"
    context_parallel_ptrr_mask_key: str | None = None
    expert_parallel_degree: int = 1
    # ---- framework-specific -------------------------------------------
    fsdp_comm: Literal["auto", "nccl", "nvlink"] = "auto"
    """``nvlink`` runs the gradient reduce-scatter and the parameter all-gather as in-kernel
    peer loads/stores over symmetric memory; ``nccl`` is the library baseline; ``auto`` uses
    NVLink when symmetric memory can be set up on every rank and NCCL otherwise."""
    tp_comm: Literal["nccl", "nvlink"] = "nccl"
    """``nvlink``: all-gather -> GEMM and GEMM -> reduce-scatter of the tensor-parallel linears run as one
    kernel each over symmetric memory (the eager form of the reference's async tensor parallelism)."""
    tp_symm_bytes: int = 2 << 30
    """Symmetric memory reserved per tensor-parallel group for gather / staging buffers."""
    cp_comm: Literal["allgather", "ring"] = "allgather"
    cp_transport: Literal["nccl", "nvlink"] = "nccl"
    """``nvlink``: the all-gather of K / V (and its reduce-scatter in backward) runs as peer loads over
    symmetric memory instead of NCCL."""
    cp_symm_bytes: int = 256 << 20
    ep_comm: Literal["nccl", "nvlink"] = "nccl"
    """``nvlink``: token dispatch / combine as in-kernel peer stores / loads over symmetric memory."""
    ep_capacity_factor: float = 0.0
    """Rows of the nvlink receive buffer = factor * tokens * top_k: static, no host read, CUDA-graph capturable.
    0 (default): worst-case buffers and one host read of the received row count per exchange (any imbalance fits)."""
    ep_overflow: Literal["error", "drop"] = "error"
    """Routed rows beyond the receive buffer of their rank: ``error`` stops training at the next status poll,
    ``drop`` leaves them out of the step (they contribute nothing to the layer output; a warning is logged)."""
    _tokens_per_rank: int = 0


@dataclass(kw_only=True, slots=True)
class CompileConfig:
    enable: bool = False
    enable_async_tensor_parallel: bool = False
    components: list[str] = field(default_factory=lambda: ["model", "loss"])
    backend: str = "inductor"
    passes: list[str] = field(default_factory=list)
    """Pass names of the reference's graph trainer (``cudagraph``, ``fsdp_reshard``, ``async_tp``, ``ep_overlap``,
    ``cpu_offload``, ``selective_remat``, ``full_remat``, ``precompile`` ...): each switches on the property of this
    framework that achieves it (``experiments/graph_trainer``)."""


@dataclass(kw_only=True, slots=True)
class CommConfig:
    init_timeout_seconds: int = 300
    train_timeout_seconds: int = 100
    trace_buf_size: int = 20000
    save_traces_folder: str = "comm_traces"
    save_traces_file_prefix: str = "rank_"
    mode: Literal["default", "fake_backend", "local_tensor", "torchcomms"] = "default"


@dataclass(kw_only=True, slots=True)
class DebugConfig:
    seed: int | None = None
    spmd_typechecking: bool = False
    deterministic: bool = False
    deterministic_warn_only: bool = False
    moe_force_load_balance: bool = False
    detect_anomaly: bool = False
    batch_invariant: bool = False
    print_config: bool = False
    save_config_file: str | None = None
    enable_structured_logging: bool = True


@dataclass(kw_only=True, slots=True)
class ActivationCheckpointConfig:
    """Activation recompute policy.

    ``selective`` keeps GEMM and attention outputs and recomputes the
    bandwidth-bound ops (norms, RoPE, SwiGLU) inside the fused autograd
    functions (``selective_ac_option = "op"``); ``"op_half_mm"`` recomputes
    whole blocks except attention and every second GEMM (the per-op save
    list of the reference), a number N recomputes every N-th block;
    ``full`` recomputes whole blocks; ``none`` keeps everything.
    Parity: torchtitan/distributed/activation_checkpoint.py:112-337.
    """

    mode: Literal["none", "selective", "full", "memory_budget"] = "selective"
    selective_ac_option: str = "op"
    preserve_rng_state: bool = True
    determinism_check: str = "default"
    debug: bool = False
    force_recompute_mm_shapes_by_fqns: list[str] = field(default_factory=lambda: ["moe.router.gate"])
    memory_budget: float = 0.5
    cpu_offload: bool = False
    """Move activations saved for backward to pinned host memory on a side stream."""
    cpu_offload_min_bytes: int = 1 << 20
    visualize_memory_budget_pareto: bool = False


@dataclass(kw_only=True, slots=True)
class KernelConfig:
    """Selects hand-written sm_100a kernels vs. the library baseline per op."""

    gemm: Literal["cublas", "tcgen05"] = "tcgen05"
    attention: Literal["sdpa", "native"] = "native"
    elementwise: Literal["native", "torch"] = "native"
