"""The trainer notices an expired bounded device wait: status words are polled every step."""

import pytest
import torch

from torchtitan_b200.config import ConfigManager
from torchtitan_b200.parallel.symm import StatusMonitor, status_monitor


def test_monitor_poll_reports_one_call_later_and_clears():
    mon = StatusMonitor()
    a, b = torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.int32)
    mon.register("path a", a)
    mon.register("path b", b)
    mon.poll()
    mon.poll()                      # nothing set: no error
    b[0] = 4
    mon.poll()                      # examines the copy taken before the bit was set, queues a new copy
    with pytest.raises(RuntimeError, match="path b"):
        mon.poll()
    assert int(b[0]) == 0           # the words are cleared when the error is raised
    mon.check()
    a[0] = 4
    with pytest.raises(RuntimeError, match="path a.*wait expired"):
        mon.check()
    a[0] = 8                        # the bits are decoded: an overflowing expert-parallel receive buffer
    with pytest.raises(RuntimeError, match="ep_capacity_factor"):
        mon.check()
    mon.tolerated = 8               # parallelism.ep_overflow = "drop": logged, cleared, not raised
    a[0] = 8
    mon.check()
    assert int(a[0]) == 0 and mon.tolerated_seen == 1
    a[0] = 12                       # an expired wait next to it still stops training
    with pytest.raises(RuntimeError, match="wait expired"):
        mon.check()


def test_trainer_raises_when_a_wait_timed_out(tmp_path):
    cfg = ConfigManager().parse_args([
        "--module", "llama3", "--config", "llama3_debugmodel", "--training.steps", "4",
        "--training.num_tokens_per_microbatch_per_dp_rank", "64", "--training.max_context_length", "64",
        "--training.mixed_precision_param", "float32", "--debug.seed", "0", "--dump_folder", str(tmp_path),
        "--debug.no-enable_structured_logging", "--metrics.log_freq", "100"])
    t = cfg.build()
    word = torch.zeros(1, dtype=torch.int32)
    status_monitor.register("fake NVLink path", word)
    it = t.batch_generator(t.dataloader)
    t.step = 2                      # not a logging step: only the asynchronous poll runs
    t.train_step(it)
    word[0] = 4                     # "a peer did not arrive"
    t.step += 1
    t.train_step(it)                # queues the copy that holds the bit
    t.step += 1
    with pytest.raises(RuntimeError, match="fake NVLink path"):
        t.train_step(it)
    t.close()
    status_monitor.clear()
