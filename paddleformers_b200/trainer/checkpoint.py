"""Training checkpoints: save, completeness detection, resume, optimizer-state resharding, async writes, rotation.

Directory layout of ``checkpoint-N`` (roles of the reference's formats in paddleformers/trainer/trainer.py:4730-4958,
paddleformers/trainer/utils/sharding_io.py:267-920 and paddleformers/trainer/unified_checkpoint/):

* ``model*.safetensors`` (+ index) and ``config.json`` — HF-compatible weights gathered over tp / ep
  (``PretrainedModel.save_pretrained``);
* ``optimizer/shard_<domain>_<rank>of<size>_m<tp>p<pp>e<ep>_r<writer>.pt`` — each sharding rank's fp32 master weights
  and Adam moments with the flat-buffer layout (``offsets``) needed to re-cut them for another sharding degree
  (``reshard_optimizer_state``). The ``m..p..e..`` tag is the writer's tensor / pipeline / expert coordinate: ranks
  that share a sharding coordinate but hold different model shards must never read each other's files;
* ``trainer_state.json``, ``scheduler.json``, ``rng_state_<rank>.pt`` (python / numpy / torch CPU / CUDA generators);
* ``saved_signal_<rank>`` written last by every rank and ``.checkpoint_done`` by rank 0 once all signals exist: a
  directory without them is an interrupted save and is skipped by ``get_last_checkpoint``.

``async_save`` moves tensors to host memory on the training thread and performs file IO on a background thread; the
next save (or the end of training) joins it first.
"""
from __future__ import annotations

import json
import os
import random
import re
import shutil
import threading
import time
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..utils.log import logger
from .trainer_utils import PREFIX_CHECKPOINT_DIR, _re_checkpoint, checkpoint_is_complete

_pending: List[threading.Thread] = []
_pending_lock = threading.Lock()


def model_parallel_tag(ps) -> str:
    """Tensor / pipeline / expert coordinate of a rank as it appears in optimizer shard file names."""
    try:
        ep = ps.rank_in("ep")
    except Exception:  # noqa: BLE001
        ep = 0
    return f"m{ps.coord.get('mp', 0):02d}p{ps.coord.get('pp', 0):02d}e{ep:02d}"


def _barrier():
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def wait_for_pending_saves():
    """Join the background writers. Threads are joined first and removed afterwards under a lock, so that a second
    caller (the mirror worker) never makes the list look empty while a writer still reads the pinned snapshot."""
    with _pending_lock:
        threads = list(_pending)
    for t in threads:
        t.join()
    with _pending_lock:
        for t in threads:
            if t in _pending:
                _pending.remove(t)


def _rng_state() -> Dict[str, object]:
    st = {"python": random.getstate(), "numpy": np.random.get_state(), "cpu": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
    return st


def _set_rng_state(st):
    random.setstate(st["python"])
    np.random.set_state(st["numpy"])
    torch.set_rng_state(st["cpu"])
    if "cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["cuda"])


def save_checkpoint(trainer, out_dir: str) -> None:
    args, ps = trainer.args, trainer.ps
    rank = args.process_index
    world = dist.get_world_size() if dist.is_initialized() else 1
    wait_for_pending_saves()
    os.makedirs(os.path.join(out_dir, "optimizer"), exist_ok=True)
    # markers of an interrupted save of the same step must not count towards this one
    for stale in (f"saved_signal_{rank}",) + ((".checkpoint_done",) if rank == 0 else ()):
        try:
            os.remove(os.path.join(out_dir, stale))
        except FileNotFoundError:
            pass
    _barrier()
    tag = model_parallel_tag(ps)
    rotate_limit = int(getattr(args, "save_total_limit", 0) or 0)
    zcc = getattr(trainer, "zcc", None)
    extra = None
    if zcc is not None:
        # zero-cost path: the shard is copied to pinned memory on a side stream; the working weights are rebuilt from the
        # fp32 master shards on resume, so the (collective, synchronous) HF export is skipped unless asked for
        if getattr(args, "zcc_save_model_weights", False):
            trainer.model.save_pretrained(out_dir)
        else:
            trainer.model.config.save_pretrained(out_dir)
        opt_state = zcc.snapshot()
        extra = zcc.extra_state()
    else:
        # 1. model weights (collective: tp gathers)
        trainer.model.save_pretrained(out_dir)
        if getattr(args, "save_checkpoint_format", "sharded") == "unified":
            save_unified_optimizer(trainer, out_dir)
        # 2. this rank's optimizer shards (moved to host now, written below or in the background)
        opt_state = trainer.optimizer.state_dict()
    files = {}
    for name, dom in opt_state["domains"].items():
        fname = f"shard_{name}_{dom['shard_rank']:03d}of{dom['shard_size']:03d}_{tag}_r{rank:05d}.pt"
        files[fname] = {"step": opt_state["step"], "lr": opt_state["lr"], "domain": name, "mp_tag": tag, **dom}
    rng = _rng_state()
    sched = trainer.lr_scheduler.state_dict()
    state_json = None
    if rank == 0:
        state_json = trainer.state

    def write():
        if zcc is not None:
            zcc.wait_host()                      # the copies into the pinned buffers have landed
            torch.save(extra, os.path.join(out_dir, f"extra_state_{rank}.pt"))
        for fname, payload in files.items():
            tmp = os.path.join(out_dir, "optimizer", fname + ".tmp")
            torch.save(payload, tmp)
            os.replace(tmp, os.path.join(out_dir, "optimizer", fname))
        torch.save(rng, os.path.join(out_dir, f"rng_state_{rank}.pt"))
        if rank == 0:
            state_json.save_to_json(os.path.join(out_dir, "trainer_state.json"))
            with open(os.path.join(out_dir, "scheduler.json"), "w") as f:
                json.dump(sched, f)
            with open(os.path.join(out_dir, "save_meta.json"), "w") as f:
                json.dump({"num_writers": world, "degrees": ps.degrees.__dict__, "time": time.time()}, f)
            with open(os.path.join(out_dir, "training_args.json"), "w") as f:
                f.write(args.to_json_string())
        with open(os.path.join(out_dir, f"saved_signal_{rank}"), "w") as f:
            f.write("done")
        if rank == 0:
            # completeness marker once every writer has signalled (polls the shared file system)
            deadline = time.time() + 600
            while time.time() < deadline:
                have = len([x for x in os.listdir(out_dir) if x.startswith("saved_signal_")])
                if have >= world:
                    with open(os.path.join(out_dir, ".checkpoint_done"), "w") as f:
                        f.write(str(world))
                    # older checkpoints go only now that this one is complete
                    if rotate_limit > 0:
                        rotate_checkpoints(os.path.dirname(os.path.abspath(out_dir)), rotate_limit)
                    break
                time.sleep(0.05)

    if args.async_save or zcc is not None:
        t = threading.Thread(target=write, daemon=False)
        t.start()
        with _pending_lock:
            _pending.append(t)
    else:
        write()
        _barrier()
    logger.info(f"saved checkpoint to {out_dir}")


UNIFIED_DIR = "unified_optimizer"


def save_unified_optimizer(trainer, out_dir: str) -> None:
    """Optimizer state under parameter names in safetensors, independent of the tensor / sharding / expert layout that
    wrote it: fp32 master weights and both Adam moments go through the same gathers and weight-map rules as the model
    weights (the reference's unified checkpoint, paddleformers/trainer/unified_checkpoint/unified_checkpoint.py:92)."""
    opt = trainer.optimizer
    for kind in ("master", "exp_avg", "exp_avg_sq"):
        state = opt.gather_full_state(kind)
        trainer.model.save_pretrained(os.path.join(out_dir, UNIFIED_DIR, kind), save_config=False,
                                      tensor_for=lambda obj, state=state: state.get(id(obj)))
    if trainer.args.process_index == 0:
        with open(os.path.join(out_dir, UNIFIED_DIR, "meta.json"), "w") as f:
            json.dump({"step": opt.step_count, "lr": opt.lr}, f)


def load_unified_optimizer(trainer, path: str) -> None:
    opt = trainer.optimizer
    views = opt.full_state_buffers()
    for kind in ("master", "exp_avg", "exp_avg_sq"):
        trainer.model.load_hf_checkpoint(os.path.join(path, UNIFIED_DIR, kind),
                                         target_for=lambda p, v=views[kind]: v.get(id(p)))
    with open(os.path.join(path, UNIFIED_DIR, "meta.json")) as f:
        meta = json.load(f)
    opt.commit_full_state(int(meta["step"]), float(meta["lr"]))


def load_checkpoint(trainer, path: str) -> None:
    from .trainer_callback import TrainerState

    if not checkpoint_is_complete(path):
        raise RuntimeError(f"checkpoint {path} is incomplete (interrupted save): refusing to resume from it")
    args, ps = trainer.args, trainer.ps
    rank = args.process_index
    has_weights = any(f.endswith(".safetensors") for f in os.listdir(path))
    if has_weights:
        trainer.model.load_hf_checkpoint(path)
    extra_file = os.path.join(path, f"extra_state_{rank}.pt")
    if os.path.exists(extra_file):
        from .zero_cost_checkpoint import load_extra_state

        load_extra_state(trainer.model, torch.load(extra_file, map_location="cpu", weights_only=False))
    opt = trainer.optimizer
    opt_dir = os.path.join(path, "optimizer")
    sd = {"domains": {}}
    unified = os.path.isdir(os.path.join(path, UNIFIED_DIR))
    saved_degrees = None
    meta_file = os.path.join(path, "save_meta.json")
    if os.path.exists(meta_file):
        with open(meta_file) as f:
            saved_degrees = json.load(f).get("degrees")
    layout_changed = saved_degrees is not None and any(
        int(saved_degrees.get(k, 1)) != int(getattr(ps.degrees, k)) for k in ("mp", "pp", "ep"))
    if unified and (layout_changed or getattr(args, "load_checkpoint_format", "sharded") == "unified"):
        load_unified_optimizer(trainer, path)          # tensor / pipeline / expert degrees differ: shards cannot be re-cut
        _finish_load(trainer, path, rank)
        return
    tag = model_parallel_tag(ps)
    solo_model = all(int(getattr(ps.degrees, k)) == 1 for k in ("mp", "pp", "ep"))
    for dom in opt.domains:
        want = f"shard_{dom.name}_{dom.shard_rank:03d}of{dom.shard_size:03d}_"
        names = sorted(f for f in os.listdir(opt_dir) if f.startswith(want) and f.endswith(".pt"))
        # this rank's own model shard; files without a tag come from checkpoints of a job without model parallelism
        cands = [f for f in names if f"_{tag}_" in f[len(want) - 1:]]
        if not cands and solo_model:
            cands = [f for f in names if _re_tag.search(f) is None]
        exact = [f for f in cands if f.endswith(f"_r{rank:05d}.pt")]
        if exact or cands:
            payload = torch.load(os.path.join(opt_dir, (exact or cands)[0]), map_location="cpu", weights_only=False)
        else:
            payload = reshard_optimizer_state(opt_dir, dom.name, dom.shard_rank, dom.shard_size, dom.numel,
                                              mp_tag=None if solo_model else tag)
        sd["domains"][dom.name] = payload
        sd["step"], sd["lr"] = payload["step"], payload["lr"]
    opt.load_state_dict(sd)
    _finish_load(trainer, path, rank)


def _finish_load(trainer, path: str, rank: int) -> None:
    from .trainer_callback import TrainerState

    st_file = os.path.join(path, "trainer_state.json")
    if os.path.exists(st_file):
        loaded = TrainerState.load_from_json(st_file)
        loaded.is_world_process_zero = trainer.state.is_world_process_zero
        trainer.state = loaded
    with open(os.path.join(path, "scheduler.json")) as f:
        trainer.lr_scheduler.load_state_dict(json.load(f))
    ema_file = os.path.join(path, f"ema_state_{rank}.pt")
    if os.path.exists(ema_file):
        from .ema import EMACallback

        for cb in trainer.callback_handler.callbacks:
            if isinstance(cb, EMACallback):
                cb.load_state_dict(torch.load(ema_file, map_location="cpu", weights_only=False))
    rng_file = os.path.join(path, f"rng_state_{rank}.pt")
    if os.path.exists(rng_file):
        _set_rng_state(torch.load(rng_file, weights_only=False))
    logger.info(f"resumed from {path} at step {trainer.state.global_step}")


_re_tag = re.compile(r"_m\d+p\d+e\d+_")


def reshard_optimizer_state(opt_dir: str, domain: str, new_rank: int, new_size: int, numel: int,
                            mp_tag: Optional[str] = None) -> Dict[str, object]:
    """Re-cut a domain saved with another sharding degree: concatenates the saved shards that overlap the new slice
    (the flat layout is independent of the sharding degree up to tail padding). ``mp_tag`` restricts the shards to
    those written by one tensor / pipeline / expert coordinate (``model_parallel_tag``); shards of different model
    shards have the same sizes and must not be mixed."""
    shards = {}
    for f in sorted(os.listdir(opt_dir)):
        if f.startswith(f"shard_{domain}_") and f.endswith(".pt"):
            if mp_tag is not None and f"_{mp_tag}_" not in f:
                continue
            p = torch.load(os.path.join(opt_dir, f), map_location="cpu", weights_only=False)
            if mp_tag is None and p["shard_rank"] in shards and p.get("mp_tag") != shards[p["shard_rank"]].get("mp_tag"):
                raise RuntimeError(f"optimizer domain {domain}: shards of several model-parallel coordinates found; "
                                   "pass mp_tag to choose one")
            shards[p["shard_rank"]] = p
    if not shards:
        raise FileNotFoundError(f"no optimizer shards for domain {domain} in {opt_dir}")
    old_size = next(iter(shards.values()))["shard_size"]
    if len(shards) != old_size:
        raise RuntimeError(f"optimizer domain {domain}: found {len(shards)} of {old_size} shards")
    any_p = shards[0]
    out = {"step": any_p["step"], "lr": any_p["lr"], "domain": domain, "offsets": any_p["offsets"], "numel": numel,
           "shard_rank": new_rank, "shard_size": new_size, "mp_tag": any_p.get("mp_tag")}
    n_new = numel // new_size
    lo, hi = new_rank * n_new, (new_rank + 1) * n_new
    for key in ("master", "exp_avg", "exp_avg_sq"):
        full = torch.cat([shards[r][key] for r in range(old_size)])
        if full.numel() < hi:
            full = torch.cat([full, full.new_zeros(hi - full.numel())])
        out[key] = full[lo:hi].clone()
    return out


def rotate_checkpoints(output_dir: str, limit: int) -> None:
    """Keep the newest ``limit`` COMPLETE checkpoints. Directories of saves that are still being written (or were
    interrupted) are neither counted nor deleted here, so the last complete checkpoint always survives."""
    cands = []
    for name in os.listdir(output_dir):
        m = _re_checkpoint.match(name)
        if m and checkpoint_is_complete(os.path.join(output_dir, name)):
            cands.append((int(m.group(1)), os.path.join(output_dir, name)))
    cands.sort()
    for _, path in cands[:-limit] if limit > 0 else []:
        shutil.rmtree(path, ignore_errors=True)
