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


def _entry(rank, world, port, fn, args, errq, backend="gloo", env=None):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    # Multi-GPU tests keep every store on plain peer addresses: a rank that dies while its memory is
    # bound to an NVLink multicast object can fault the other ranks' GPUs.  The one test that
    # exercises multimem stores opts in through ``env``.  Bounded device waits give up after 10 s.
    os.environ.setdefault("TB200_MULTICAST", "0")
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    os.environ.setdefault("TB200_SYMM_TIMEOUT_S", "10")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if env:
        os.environ.update(env)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch
    import torch.distributed as dist

    torch.set_num_threads(1)
    try:
        if backend == "nccl":
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
        # leave in order: wait for the own GPU work, meet the peers at a last barrier (they reach it
        # through their own error path or at the end of ``fn``) and tear the process group down, so
        # that no rank exits while a peer still spins on its memory
        try:
            if backend == "nccl":
                torch.cuda.synchronize()
            if dist.is_initialized():
                dist.barrier()
                dist.destroy_process_group()
        except Exception:
            pass
        raise


def run_distributed(fn, world: int, *args, timeout: float = 240.0, backend: str = "gloo", env: dict | None = None):
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq, backend, env)) for r in range(world)]
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
