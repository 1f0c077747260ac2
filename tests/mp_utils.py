"""Helpers to run a function on several ranks as child processes (gloo on CPU, NCCL on GPUs)."""
import os
import socket
import traceback

import torch
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, backend, fn, args, errq):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    if backend != "nccl":
        # several ranks share the host's cores: without a cap every rank starts one thread per core
        torch.set_num_threads(max(1, (os.cpu_count() or 8) // max(world, 1)))
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
    except Exception:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # noqa: BLE001
                pass


def run_ranks(fn, world: int, backend: str = "gloo", args=(), timeout: float = 300.0):
    """Run ``fn(rank, world, *args)`` on ``world`` child processes; raises if any rank failed."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, backend, fn, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()  # exact child PIDs only
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    if hung:
        errs.append((-1, f"{len(hung)} rank(s) still running after {timeout}s"))
    bad = [p.exitcode for p in procs if p.exitcode not in (0, None)]
    if errs or bad:
        raise AssertionError("rank failures:\n" + "\n".join(f"[rank {r}] {t}" for r, t in errs) + f"\nexit codes {bad}")
