"""Spawn N CPU ranks (gloo, 127.0.0.1) that run a worker function and return picklable results."""
import os
import socket
import tempfile
import traceback

import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, outdir):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port), "CUDA_VISIBLE_DEVICES": ""})
    torch.set_num_threads(1)
    try:
        import torch.distributed as dist

        dist.init_process_group("gloo", rank=rank, world_size=world)
        res = fn(rank, world, *args)
        torch.save({"ok": True, "result": res}, os.path.join(outdir, f"r{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        torch.save({"ok": False, "error": traceback.format_exc()}, os.path.join(outdir, f"r{rank}.pt"))
        raise


def run_distributed(fn, world: int, *args, timeout: int = 240):
    with tempfile.TemporaryDirectory() as d:
        port = _free_port()
        ctx = mp.get_context("spawn")
        procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, d)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        alive = [p for p in procs if p.is_alive()]
        for p in alive:
            p.terminate()
        out = []
        for r in range(world):
            f = os.path.join(d, f"r{r}.pt")
            if not os.path.exists(f):
                raise RuntimeError(f"rank {r} produced no result (timeout or crash)")
            rec = torch.load(f, weights_only=False)
            if not rec["ok"]:
                raise RuntimeError(f"rank {r} failed:\n{rec['error']}")
            out.append(rec["result"])
        if alive:
            raise RuntimeError("some ranks did not exit in time")
        return out
