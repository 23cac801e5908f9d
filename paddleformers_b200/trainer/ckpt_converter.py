"""Offline checkpoint tools: inspect a training checkpoint and re-cut its optimizer shards for another sharding degree
without starting a distributed job (the role of paddleformers/trainer/utils/ckpt_converter.py, which converts between the
reference's checkpoint layouts outside of training).

    python -m paddleformers_b200.trainer.ckpt_converter inspect  <checkpoint>
    python -m paddleformers_b200.trainer.ckpt_converter reshard  <checkpoint> <output> --sharding N

``reshard`` copies the weights, scheduler, trainer state and random-number states as they are and rewrites
``optimizer/shard_<domain>_<rank>of<N>_*.pt`` for N ranks. The flat layout of a domain does not depend on the sharding
degree (only its tail padding does), so this is a pure re-slicing; a run started on N sharding ranks then finds exactly
the files it looks for instead of re-cutting on every rank at start-up. Tensor / pipeline / expert degrees cannot be changed
this way: use the unified optimizer format for that (``save_checkpoint_format: unified``).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
from typing import Dict, List

import torch

from .checkpoint import reshard_optimizer_state
from .trainer_utils import checkpoint_is_complete

_ALIGN = 128


def list_domains(opt_dir: str) -> Dict[str, Dict[str, int]]:
    """domain -> {"shard_size", "numel", "files"} from the shard files of a checkpoint's ``optimizer`` folder."""
    out: Dict[str, Dict[str, int]] = {}
    for f in sorted(os.listdir(opt_dir)):
        if not (f.startswith("shard_") and f.endswith(".pt")):
            continue
        p = torch.load(os.path.join(opt_dir, f), map_location="cpu", weights_only=False)
        d = out.setdefault(p["domain"], {"shard_size": int(p["shard_size"]), "numel": int(p["numel"]), "files": 0,
                                         "step": int(p["step"]), "mp_tags": []})
        d["files"] += 1
        tag = p.get("mp_tag")
        if tag not in d["mp_tags"]:
            d["mp_tags"].append(tag)
    return out


def inspect(path: str) -> Dict[str, object]:
    info: Dict[str, object] = {"path": path, "complete": checkpoint_is_complete(path)}
    meta = os.path.join(path, "save_meta.json")
    if os.path.exists(meta):
        with open(meta) as f:
            info["save_meta"] = json.load(f)
    st = os.path.join(path, "trainer_state.json")
    if os.path.exists(st):
        with open(st) as f:
            info["global_step"] = json.load(f).get("global_step")
    info["weight_files"] = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    opt_dir = os.path.join(path, "optimizer")
    info["optimizer_domains"] = list_domains(opt_dir) if os.path.isdir(opt_dir) else {}
    info["unified_optimizer"] = os.path.isdir(os.path.join(path, "unified_optimizer"))
    return info


def reshard(path: str, out: str, sharding: int) -> List[str]:
    """Write a copy of checkpoint ``path`` at ``out`` whose optimizer shards are cut for ``sharding`` ranks. Returns the
    optimizer files written."""
    if not checkpoint_is_complete(path):
        raise RuntimeError(f"checkpoint {path} is incomplete (interrupted save)")
    if sharding < 1:
        raise ValueError("sharding must be >= 1")
    opt_dir = os.path.join(path, "optimizer")
    domains = list_domains(opt_dir)
    if not domains:
        raise FileNotFoundError(f"no optimizer shards under {opt_dir}")
    os.makedirs(os.path.join(out, "optimizer"), exist_ok=True)
    for f in os.listdir(path):                     # everything but the optimizer shards and the per-writer markers
        src = os.path.join(path, f)
        if f == "optimizer" or f.startswith("saved_signal_") or f == ".checkpoint_done" or f.startswith("rng_state_"):
            continue
        if os.path.isdir(src):
            shutil.copytree(src, os.path.join(out, f), dirs_exist_ok=True)
        else:
            shutil.copy2(src, os.path.join(out, f))
    written = []
    for name, d in domains.items():
        # the layout up to the last parameter is fixed; only the padding to a multiple of align * ranks changes
        any_file = next(f for f in sorted(os.listdir(opt_dir)) if f.startswith(f"shard_{name}_"))
        offsets = torch.load(os.path.join(opt_dir, any_file), map_location="cpu", weights_only=False)["offsets"]
        used = max((off + (cnt + _ALIGN - 1) // _ALIGN * _ALIGN) for off, cnt in offsets.values()) if offsets else d["numel"]
        unit = _ALIGN * sharding
        numel = (used + unit - 1) // unit * unit
        # one re-cut per tensor / pipeline / expert coordinate that wrote this domain: their shards have equal sizes
        # and different contents
        for ti, tag in enumerate(d["mp_tags"]):
            for r in range(sharding):
                payload = reshard_optimizer_state(opt_dir, name, r, sharding, numel, mp_tag=tag)
                mid = f"_{tag}" if tag else ""
                fname = f"shard_{name}_{r:03d}of{sharding:03d}{mid}_r{ti * sharding + r:05d}.pt"
                torch.save(payload, os.path.join(out, "optimizer", fname))
                written.append(fname)
    # random-number states belong to the old ranks: rank 0's is kept for every new rank so that a resume is deterministic
    rng0 = os.path.join(path, "rng_state_0.pt")
    for r in range(sharding):
        if os.path.exists(rng0):
            shutil.copy2(rng0, os.path.join(out, f"rng_state_{r}.pt"))
        with open(os.path.join(out, f"saved_signal_{r}"), "w") as f:
            f.write("done")
    meta_file = os.path.join(out, "save_meta.json")
    if os.path.exists(meta_file):
        with open(meta_file) as f:
            meta = json.load(f)
        meta["num_writers"] = sharding
        meta.setdefault("degrees", {})["sharding"] = sharding
        meta["resharded_from"] = os.path.abspath(path)
        with open(meta_file, "w") as f:
            json.dump(meta, f)
    with open(os.path.join(out, ".checkpoint_done"), "w") as f:
        f.write(str(sharding))
    return written


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ckpt_converter", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("inspect")
    a.add_argument("checkpoint")
    b = sub.add_parser("reshard")
    b.add_argument("checkpoint")
    b.add_argument("output")
    b.add_argument("--sharding", type=int, required=True)
    ns = ap.parse_args(argv)
    if ns.cmd == "inspect":
        print(json.dumps(inspect(ns.checkpoint), indent=2, default=str))
    else:
        files = reshard(ns.checkpoint, ns.output, ns.sharding)
        print(f"wrote {len(files)} optimizer shard files for {ns.sharding} ranks to {ns.output}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
