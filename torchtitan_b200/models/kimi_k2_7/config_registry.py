"""Registered Kimi / Moonlight training configs (parity: torchtitan/models/kimi_k2_7/config_registry.py)."""

from __future__ import annotations

from torchtitan_b200.components.optimizer import OptimizersContainer, ParamGroupConfig
from torchtitan_b200.models.deepseek_v3.config_registry import _full, deepseek_v3_debugmodel
from torchtitan_b200.trainer import Trainer

# Matrix parameters that train with Muon (Moonlight, arXiv 2502.16982, sec. 2.2): attention and MLP
# projections, routed and shared experts and the router gate; embeddings, norms, biases and the
# output head stay on AdamW.
MUON_PATTERN = (r"layers\.\d+\.(?:attention\.(?:wq|wq_a|wq_b|wkv_a|wkv_b|wo)\.weight|feed_forward\.w(?:13|1|2|3)\.weight|"
                r"moe\.routed_experts\.inner_experts\.w[123]_E[DF]{2}|moe\.router\.gate\.weight|"
                r"moe\.shared_experts\.w(?:13|1|2|3)\.weight)$")


def kimi_muon_optimizer(flavor: str, lr: float) -> OptimizersContainer.Config:
    """DistMuon for the matrices, AdamW for the rest (parity: kimi_k2_7/config_registry.py:286-462).

    Per-head Newton-Schulz: the query / key-value up-projections are orthogonalised one head's
    row block at a time, the fused gate/up projection one half at a time."""
    from torchtitan_b200.models.kimi_k2_7 import kimi_configs

    mc = kimi_configs[flavor]()
    att = mc.layers[0].attention
    ffn_rows = {}
    for blk in mc.layers:   # the fused w13 holds w1 over w3: two matrices of half the rows
        ff = getattr(blk, "feed_forward", None)
        if ff is not None and getattr(ff, "hidden_dim", 0):
            ffn_rows[r"feed_forward\.w13\.weight$"] = int(ff.hidden_dim)
        moe = getattr(blk, "moe", None)
        if moe is not None and getattr(moe, "shared_hidden_dim", 0):
            ffn_rows[r"shared_experts\.w13\.weight$"] = int(moe.shared_hidden_dim)
    block_rows = {
        r"attention\.(?:wq|wq_b)\.weight$": int(att.qk_nope_head_dim + att.qk_rope_head_dim),
        r"attention\.wkv_b\.weight$": int(att.qk_nope_head_dim + att.v_head_dim),
        **ffn_rows,
    }
    return OptimizersContainer.Config(
        lr=lr, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
        param_groups=[ParamGroupConfig(pattern=MUON_PATTERN, optimizer_name="DistMuon",
                                       optimizer_kwargs={"lr": lr, "weight_decay": 0.1,
                                                         "adjust_lr_fn": "match_rms_adamw", "block_rows": block_rows})],
    )


def kimi_debugmodel() -> Trainer.Config:
    cfg = deepseek_v3_debugmodel()
    cfg.model.name, cfg.model.flavor = "kimi_k2_7", "debugmodel"
    return cfg


def kimi_debugmodel_vl() -> Trainer.Config:
    cfg = kimi_debugmodel()
    cfg.model.flavor = "debugmodel_vl"
    cfg.dataloader.dataset = "synthetic_mm"
    return cfg


def kimi_debugmodel_muon() -> Trainer.Config:
    cfg = kimi_debugmodel()
    cfg.optimizer = kimi_muon_optimizer("debugmodel", cfg.optimizer.lr)
    return cfg


def kimi_moonlight() -> Trainer.Config:
    cfg = _full("moonlight", 2 * 8192, 8192, 4e-4, 10000, expert_parallel_degree=8)
    cfg.model.name = "kimi_k2_7"
    cfg.optimizer = kimi_muon_optimizer("moonlight", 4e-4)
    return cfg


def kimi_k2() -> Trainer.Config:
    cfg = _full("kimi_k2", 4 * 4096, 4096, 2e-4, 10000, expert_parallel_degree=8)
    cfg.model.name = "kimi_k2_7"
    cfg.optimizer = kimi_muon_optimizer("kimi_k2", 2e-4)
    return cfg


def kimi_vl_a3b() -> Trainer.Config:
    """Moonlight text decoder behind the vision tower, interleaved text / image data."""
    cfg = kimi_moonlight()
    cfg.model.flavor = "kimi_vl_a3b"
    cfg.dataloader.dataset = "mm_jsonl"
    return cfg
