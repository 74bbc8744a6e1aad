"""Run a function on several CPU ranks (Gloo) as child processes; failures of any rank fail the test."""

import os
import socket
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world_size, port, fn, args, queue):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world_size), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world_size),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        import torch

        torch.set_num_threads(2)
        result = fn(rank, world_size, *args)
        queue.put((rank, "ok", result))
    except BaseException:  # noqa: BLE001 - report everything to the parent
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        try:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:
            pass


def run_distributed(fn, world_size: int, *args, timeout: float = 300):
    """Returns the list of per-rank results (rank order)."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world_size, port, fn, args, queue)) for r in range(world_size)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world_size):
            rank, status, payload = queue.get(timeout=timeout)
            if status == "error":
                raise RuntimeError(f"rank {rank} failed:\n{payload}")
            results[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world_size)]
