"""Training metrics: throughput, TFLOPs, MFU, memory, loggers.

``tps = tokens / (dt * cp * tp * pp)`` is per-GPU throughput, ``tflops =
flops_per_token * tps / 1e12`` and ``mfu = 100 * flops_per_token * tps / peak``
(parity: torchtitan/components/metrics.py:455-541).  Metrics are logged every
``log_freq`` steps and on step 1.
"""

from __future__ import annotations

import os
import time
from collections import namedtuple
from dataclasses import dataclass
from datetime import datetime
from typing import Any

import torch

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import Color, NoColor, logger

__all__ = ["DeviceMemoryMonitor", "MetricsProcessor", "BaseLogger", "TensorBoardLogger", "WandBLogger", "LoggerContainer"]

DeviceMemStats = namedtuple(
    "DeviceMemStats",
    ["max_active_gib", "max_active_pct", "max_reserved_gib", "max_reserved_pct", "num_alloc_retries", "num_ooms"],
)


class DeviceMemoryMonitor:
    def __init__(self, device: torch.device):
        self.device = device
        self.is_cuda = device.type == "cuda"
        if self.is_cuda:
            self.device_name = torch.cuda.get_device_name(device)
            self.device_capacity = torch.cuda.get_device_properties(device).total_memory
            torch.cuda.reset_peak_memory_stats(device)
            torch.cuda.empty_cache()
        else:
            self.device_name, self.device_capacity = "cpu", 1
        self.device_capacity_gib = self.device_capacity / (1 << 30)

    def get_peak_stats(self) -> DeviceMemStats:
        if not self.is_cuda:
            return DeviceMemStats(0.0, 0.0, 0.0, 0.0, 0, 0)
        info = torch.cuda.memory_stats(self.device)
        act = info.get("active_bytes.all.peak", 0)
        res = info.get("reserved_bytes.all.peak", 0)
        gib = 1 << 30
        return DeviceMemStats(act / gib, 100 * act / self.device_capacity, res / gib, 100 * res / self.device_capacity,
                              info.get("num_alloc_retries", 0), info.get("num_ooms", 0))

    def reset_peak_stats(self) -> None:
        if self.is_cuda:
            torch.cuda.reset_peak_memory_stats(self.device)


class BaseLogger:
    def log(self, metrics: dict[str, Any], step: int) -> None:
        pass

    def close(self) -> None:
        pass


class TensorBoardLogger(BaseLogger):
    def __init__(self, log_dir: str, tag: str | None = None):
        from torch.utils.tensorboard import SummaryWriter

        self.tag = tag
        self.writer = SummaryWriter(log_dir, max_queue=1000)
        logger.info(f"TensorBoard logging enabled. Logs will be saved at {log_dir}")

    def log(self, metrics, step):
        for k, v in metrics.items():
            self.writer.add_scalar(k if self.tag is None else f"{self.tag}/{k}", v, step)

    def close(self):
        self.writer.close()


class WandBLogger(BaseLogger):
    def __init__(self, log_dir: str, config_dict: dict | None = None, tag: str | None = None):
        import wandb

        self.wandb, self.tag = wandb, tag
        os.makedirs(log_dir, exist_ok=True)
        wandb.init(entity=os.getenv("WANDB_TEAM"), project=os.getenv("WANDB_PROJECT", "torchtitan_b200"),
                   name=os.getenv("WANDB_RUN_NAME"), id=os.getenv("WANDB_RUN_ID"), notes=os.getenv("WANDB_RUN_NOTES"),
                   tags=os.getenv("WANDB_RUN_TAGS", "").split(",") if os.getenv("WANDB_RUN_TAGS") else None,
                   group=os.getenv("WANDB_RUN_GROUP"), job_type=os.getenv("WANDB_RUN_JOB_TYPE"),
                   resume_from=os.getenv("WANDB_RESUME_FROM"), fork_from=os.getenv("WANDB_FORK_FROM"),
                   dir=log_dir, config=config_dict)

    def log(self, metrics, step):
        self.wandb.log({(k if self.tag is None else f"{self.tag}/{k}"): v for k, v in metrics.items()}, step=step)

    def close(self):
        if self.wandb.run is not None:
            self.wandb.finish()


class LoggerContainer(BaseLogger):
    def __init__(self):
        self._loggers: list[BaseLogger] = []

    def add_logger(self, lg: BaseLogger) -> None:
        self._loggers.append(lg)

    @property
    def number_of_loggers(self) -> int:
        return len(self._loggers)

    def log(self, metrics, step):
        for lg in self._loggers:
            lg.log(metrics, step)

    def close(self):
        for lg in self._loggers:
            lg.close()


def metrics_rank(pdims) -> int:
    """Rank that owns the loss: rank 0, or the first rank of the last pipeline stage."""
    if pdims is not None and pdims.pp_enabled:
        return (pdims.world_size // pdims.pp) * (pdims.pp - 1)
    return 0


class MetricsProcessor(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        log_freq: int = 10
        enable_tensorboard: bool = False
        disable_color_printing: bool = False
        save_tb_folder: str = "tb"
        save_for_all_ranks: bool = False
        enable_wandb: bool = False

    def __init__(self, config: "MetricsProcessor.Config", *, pdims=None, device: torch.device | None = None,
                 dump_folder: str = "./outputs", job_config_dict: dict | None = None, tag: str | None = None, **_):
        self.config = config
        self.pdims = pdims
        self.device = device or torch.device("cpu")
        self.logger = LoggerContainer()
        rank = pdims.rank if pdims is not None else 0
        should = config.save_for_all_ranks or rank == metrics_rank(pdims)
        base = os.path.join(dump_folder, config.save_tb_folder, datetime.now().strftime("%Y%m%d-%H%M"))
        if config.save_for_all_ranks:
            base = os.path.join(base, f"rank_{rank}")
        if should and config.enable_tensorboard:
            self.logger.add_logger(TensorBoardLogger(base, tag))
        if should and config.enable_wandb:
            self.logger.add_logger(WandBLogger(base, job_config_dict, tag))
        self.device_memory_monitor = DeviceMemoryMonitor(self.device)
        self.color = NoColor() if config.disable_color_printing else Color()
        self.num_flops_per_token = -1.0
        self.gpu_peak_flops = -1.0
        self.quantized = False
        self.ntokens_since_last_log = 0
        self.data_loading_times: list[float] = []
        self.time_last_log = time.perf_counter()
        self.optimizers = None
        self.lr_schedulers = None
        self.model_parts = None

    def should_log(self, step: int) -> bool:
        return step == 1 or step % self.config.log_freq == 0

    def log(self, step: int, global_avg_loss: float, global_max_loss: float, grad_norm: float,
            extra_metrics: dict[str, Any] | None = None) -> dict[str, Any]:
        dt = time.perf_counter() - self.time_last_log
        nd = self.pdims.non_data_parallel_size if self.pdims is not None else 1
        tps = self.ntokens_since_last_log / (dt * nd)
        tflops = self.num_flops_per_token * tps / 1e12
        mfu = None if self.quantized or self.gpu_peak_flops <= 0 else 100 * self.num_flops_per_token * tps / self.gpu_peak_flops
        e2e = dt / self.config.log_freq
        dl = sum(self.data_loading_times) / max(1, len(self.data_loading_times))
        dl_pct = 100 * sum(self.data_loading_times) / max(dt, 1e-9)
        mem = self.device_memory_monitor.get_peak_stats()
        metrics = {
            "loss_metrics/global_avg_loss": global_avg_loss,
            "loss_metrics/global_max_loss": global_max_loss,
            "grad_norm": grad_norm,
            "throughput(tps)": tps,
            "tflops": tflops,
            "time_metrics/end_to_end(s)": e2e,
            "time_metrics/data_loading(s)": dl,
            "time_metrics/data_loading(%)": dl_pct,
            "memory/max_active(GiB)": mem.max_active_gib,
            "memory/max_active(%)": mem.max_active_pct,
            "memory/max_reserved(GiB)": mem.max_reserved_gib,
            "memory/max_reserved(%)": mem.max_reserved_pct,
            "memory/num_alloc_retries": mem.num_alloc_retries,
            "memory/num_ooms": mem.num_ooms,
        }
        if mfu is not None:
            metrics["mfu(%)"] = mfu
        if extra_metrics:
            metrics.update(extra_metrics)
        self.logger.log(metrics, step)
        c = self.color
        mfu_s = f"  {c.magenta}mfu: {mfu:.2f}%{c.reset}" if mfu is not None else ""
        logger.info(
            f"{c.red}step: {step:2}  {c.green}loss: {global_avg_loss:8.5f}  {c.orange}grad_norm: {grad_norm:7.4f}  "
            f"{c.turquoise}memory: {mem.max_reserved_gib:5.2f}GiB({mem.max_reserved_pct:.2f}%)  "
            f"{c.blue}tps: {round(tps):,}  {c.cyan}tflops: {tflops:,.2f}{mfu_s}{c.reset}"
        )
        self.ntokens_since_last_log = 0
        self.data_loading_times.clear()
        self.time_last_log = time.perf_counter()
        self.device_memory_monitor.reset_peak_stats()
        return metrics

    def log_validation(self, loss: float, step: int, extra_metrics: dict[str, Any] | None = None) -> None:
        dt = time.perf_counter() - self.time_last_log
        nd = self.pdims.non_data_parallel_size if self.pdims is not None else 1
        tps = self.ntokens_since_last_log / max(dt * nd, 1e-9)
        mem = self.device_memory_monitor.get_peak_stats()
        metrics = {"validation_metrics/loss": loss, "validation_metrics/throughput(tps)": tps,
                   "validation_metrics/memory/max_reserved(GiB)": mem.max_reserved_gib}
        if extra_metrics:
            metrics.update(extra_metrics)
        self.logger.log(metrics, step)
        c = self.color
        logger.info(f"{c.yellow}validate step: {step:2}  {c.green}loss: {loss:7.4f}  "
                    f"{c.turquoise}memory: {mem.max_reserved_gib:5.2f}GiB  {c.blue}tps: {round(tps):,}{c.reset}")
        self.ntokens_since_last_log = 0
        self.time_last_log = time.perf_counter()
        self.device_memory_monitor.reset_peak_stats()

    def close(self) -> None:
        self.logger.close()
