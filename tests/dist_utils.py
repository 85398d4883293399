"""Spawn N CPU ranks over gloo on 127.0.0.1 and run a function on each."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn, args, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.set_num_threads(2)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        ret[rank] = ("ok", out)
    except Exception:
        ret[rank] = ("err", traceback.format_exc())
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def run_ranks(world, fn, *args, timeout=300):
    """Returns the list of per-rank results; raises if any rank failed."""
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
            p.terminate()
            raise TimeoutError("rank did not finish")
    out = []
    for r in range(world):
        status, val = ret.get(r, ("err", "no result (process died)"))
        if status != "ok":
            raise RuntimeError(f"rank {r} failed:\n{val}")
        out.append(val)
    return out
