"""Spawns CPU ranks (gloo, 127.0.0.1) running a worker function; returns their results."""
import os
import socket
import tempfile
import traceback

import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn, args, outdir):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(2)
    try:
        res = fn(rank, world, *args)
        torch.save({"ok": True, "res": res}, os.path.join(outdir, f"r{rank}.pt"))
    except Exception:
        torch.save({"ok": False, "err": traceback.format_exc()}, os.path.join(outdir, f"r{rank}.pt"))
        raise
    finally:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()


def run_workers(world, fn, *args, timeout=240):
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        ctx = mp.get_context("spawn")
        procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, d)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        out = []
        for r, p in enumerate(procs):
            if p.is_alive():
                p.kill()
                raise TimeoutError(f"rank {r} did not finish in {timeout}s")
            f = os.path.join(d, f"r{r}.pt")
            if not os.path.exists(f):
                raise RuntimeError(f"rank {r} exited with code {p.exitcode} and no result")
            res = torch.load(f, weights_only=False)
            if not res["ok"]:
                raise RuntimeError(f"rank {r} failed:\n{res['err']}")
            out.append(res["res"])
        return out
