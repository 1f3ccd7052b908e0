"""Spawn helper for multi-process CPU (gloo) tests."""
import os
import socket
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn, args, ret):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["RANK"] = str(rank)
        os.environ["WORLD_SIZE"] = str(world)
        torch.set_num_threads(2)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        ret[rank] = ("ok", out)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # pragma: no cover - surfaced by the parent
        ret[rank] = ("err", traceback.format_exc())
        raise


def run_ranks(fn, world, *args, timeout=300):
    """Runs ``fn(rank, world, *args)`` on ``world`` gloo ranks; returns the list of return values."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    for p in procs:
        if p.is_alive():
            p.kill()
            raise TimeoutError("a rank did not finish")
    out = []
    for r in range(world):
        status, val = ret.get(r, ("err", "no result"))
        assert status == "ok", f"rank {r} failed:\n{val}"
        out.append(val)
    return out
