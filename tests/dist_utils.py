"""Spawn ``world`` CPU/gloo ranks running a function from a test module."""

import os
import socket
import sys
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errq, backend="gloo"):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch
    import torch.distributed as dist

    torch.set_num_threads(1)
    try:
        if backend == "nccl":
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            torch.cuda.set_device(rank)
            dist.init_process_group("cuda:nccl,cpu:gloo", rank=rank, world_size=world,
                                    device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_distributed(fn, world: int, *args, timeout: float = 240.0, backend: str = "gloo"):
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq, backend)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    failed = []
    for r, p in enumerate(procs):
        if p.is_alive():
            p.terminate()
            failed.append(f"rank {r} timed out")
        elif p.exitcode != 0:
            failed.append(f"rank {r} exit code {p.exitcode}")
    msgs = []
    while not errq.empty():
        msgs.append("rank %d:\n%s" % errq.get())
    assert not failed, "; ".join(failed) + "\n" + "\n".join(msgs)
