"""Trainer helpers: enums, LR schedules, speed metrics, seeding, checkpoint discovery.

Counterparts in the reference: paddleformers/trainer/trainer_utils.py (SchedulerType / get_scheduler :780,
speed_metrics :578-607, set_random_seed :354, get_last_checkpoint :458-513, IterableDatasetShard).
"""
from __future__ import annotations

import enum
import math
import os
import random
import re
import time
from typing import NamedTuple, Dict, Optional

import numpy as np
import torch

PREFIX_CHECKPOINT_DIR = "checkpoint"
_re_checkpoint = re.compile(r"^" + PREFIX_CHECKPOINT_DIR + r"\-(\d+)$")


class SchedulerType(str, enum.Enum):
    LINEAR = "linear"
    COSINE = "cosine"
    CONSTANT = "constant"
    CONSTANT_WITH_WARMUP = "constant_with_warmup"
    POLYNOMIAL = "polynomial"
    WSD = "warmup_stable_decay"


class OptimizerNames(str, enum.Enum):
    """Accepted values of ``TrainingArguments.optim`` (paddleformers/trainer/trainer_utils.py:528-537)."""

    ADAMW = "adamw"
    ADAMW_MINI = "adamw_mini"
    ADAMW_CUSTOM = "adamw_custom"
    MUON = "muon"


class ShardingOption(str, enum.Enum):
    SHARD_OP = "stage1"
    SHARD_GRAD_OP = "stage2"
    FULL_SHARD = "stage3"
    OFFLOAD = "offload"


class IntervalStrategy(str, enum.Enum):
    NO = "no"
    STEPS = "steps"
    EPOCH = "epoch"


def get_scheduler_lambda(name, num_warmup_steps: int, num_training_steps: int, min_lr_ratio: float = 0.0,
                         num_cycles: float = 0.5, power: float = 1.0, decay_steps: Optional[int] = None):
    """Multiplicative LR factor as a function of the optimizer step (step 0 = first update)."""
    name = SchedulerType(name)
    total = max(num_training_steps, 1)
    warm = max(num_warmup_steps, 0)

    def warmup(step):
        return float(step) / float(max(1, warm))

    if name == SchedulerType.CONSTANT:
        return lambda step: 1.0
    if name == SchedulerType.CONSTANT_WITH_WARMUP:
        return lambda step: warmup(step) if step < warm else 1.0
    if name == SchedulerType.LINEAR:
        return lambda step: warmup(step) if step < warm else max(
            min_lr_ratio, float(total - step) / float(max(1, total - warm)))
    if name == SchedulerType.COSINE:
        def f(step):
            if step < warm:
                return warmup(step)
            prog = float(step - warm) / float(max(1, total - warm))
            cos = 0.5 * (1.0 + math.cos(math.pi * num_cycles * 2.0 * min(prog, 1.0)))
            return min_lr_ratio + (1 - min_lr_ratio) * cos
        return f
    if name == SchedulerType.POLYNOMIAL:
        def f(step):
            if step < warm:
                return warmup(step)
            if step > total:
                return min_lr_ratio
            rem = 1 - (step - warm) / max(1, total - warm)
            return min_lr_ratio + (1 - min_lr_ratio) * rem ** power
        return f
    if name == SchedulerType.WSD:
        dsteps = decay_steps if decay_steps is not None else max(1, int(0.1 * total))
        stable_end = total - dsteps

        def f(step):
            if step < warm:
                return warmup(step)
            if step < stable_end:
                return 1.0
            prog = min(1.0, (step - stable_end) / max(1, dsteps))
            return min_lr_ratio + (1 - min_lr_ratio) * (1 - prog)
        return f
    raise ValueError(name)


class LRScheduler:
    def __init__(self, base_lr: float, fn):
        self.base_lr, self.fn, self.last_step = base_lr, fn, 0

    def get_lr(self) -> float:
        return self.base_lr * self.fn(self.last_step)

    def step(self):
        self.last_step += 1

    def state_dict(self):
        return {"last_step": self.last_step, "base_lr": self.base_lr}

    def load_state_dict(self, sd):
        self.last_step = int(sd["last_step"])
        self.base_lr = float(sd.get("base_lr", self.base_lr))


def speed_metrics(split: str, start_time: float, num_samples=None, num_steps=None, seq_length=None,
                  model_flops_per_token=None, world_size: int = 1) -> Dict[str, float]:
    """{split}_runtime, samples/s, steps/s, tokens/s/device and hardware TFLOPs/device, with the reference's
    definitions: tokens/s/device = samples/s * seq_length / world_size, TFLOPs = tokens/s/device * flops_per_token /
    2**40 (paddleformers/trainer/trainer_utils.py:591-602)."""
    runtime = time.time() - start_time
    out = {f"{split}_runtime": round(runtime, 4)}
    if runtime <= 0:
        return out
    if num_samples is not None:
        sps = num_samples / runtime
        out[f"{split}_samples_per_second"] = round(sps, 4)
        if seq_length is not None:
            tps = sps * seq_length / max(world_size, 1)
            out[f"{split}_tokens_per_second_per_device"] = round(tps, 4)
            if model_flops_per_token is not None:
                out[f"{split}_hardware_tflops_per_device"] = round(tps * model_flops_per_token / 2 ** 40, 4)
    if num_steps is not None:
        out[f"{split}_steps_per_second"] = round(num_steps / runtime, 4)
    return out


def tensor_md5(t: torch.Tensor) -> str:
    """Hex md5 of a tensor's bytes (bf16 is widened to fp32 first, which is exact). Used to compare runs bit for bit:
    loss values, batches, parameters after a resume."""
    import hashlib

    t = t.detach()
    if t.dtype == torch.bfloat16:
        t = t.float()
    return hashlib.md5(t.contiguous().cpu().numpy().tobytes()).hexdigest()


def state_digest(tensors) -> str:
    """One md5 over an ordered ``name -> tensor`` mapping (names included, so a renamed or reordered entry changes it)."""
    import hashlib

    h = hashlib.md5()
    for k, v in tensors.items():
        h.update(k.encode())
        h.update(tensor_md5(v).encode())
    return h.hexdigest()


def set_seed(seed: int):
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def set_random_seed(seed: int, parallel_state=None):
    """Global seed for data-order decisions, and a per-model-parallel-rank local seed for dropout / init of sharded
    tensors (paddleformers/trainer/trainer_utils.py:354): ranks that hold different shards must draw different
    numbers, ranks that hold replicas the same."""
    from ..parallel.topology import get_parallel_state

    ps = parallel_state or get_parallel_state()
    c = ps.coord
    local = seed + 1 + c["mp"] * 7 + c["pp"] * 1009 + ps.rank_in("ep") * 100003
    random.seed(seed + ps.dataset_rank)
    np.random.seed((seed + ps.dataset_rank) % (2 ** 32))
    torch.manual_seed(local)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(local)
    return local


class EvalPrediction(NamedTuple):
    """What ``compute_metrics`` receives: predictions and labels of the whole evaluation set, one row per example, padded
    with -100 to the longest row (paddleformers/trainer/trainer_utils.py ``EvalPrediction``)."""

    predictions: "np.ndarray"
    label_ids: Optional["np.ndarray"]


class PredictionOutput(NamedTuple):
    predictions: "np.ndarray"
    label_ids: Optional["np.ndarray"]
    metrics: Optional[Dict[str, float]]


class EvalSampler(torch.utils.data.Sampler):
    """Sequential indices of ONE data rank covering the whole set: global batch b holds examples
    [b * world * batch, (b + 1) * world * batch), rank r its r-th slice. The last global batch is filled up by wrapping
    around, so that every rank runs the same number of batches (collectives inside the model stay matched);
    ``padding_rows(b)`` tells which rows of this rank's batch b are such fill-ins and must not count."""

    def __init__(self, n: int, rank: int, world: int, batch: int):
        self.n, self.rank, self.world, self.batch = n, rank, world, batch
        self.num_batches = (n + world * batch - 1) // (world * batch) if n > 0 else 0

    def __len__(self):
        return self.num_batches * self.batch

    def _positions(self, b: int):
        base = (b * self.world + self.rank) * self.batch
        return range(base, base + self.batch)

    def padding_rows(self, b: int):
        return [i for i, p in enumerate(self._positions(b)) if p >= self.n]

    def __iter__(self):
        for b in range(self.num_batches):
            for p in self._positions(b):
                yield p % self.n


def get_last_checkpoint(folder: str, require_complete: bool = True) -> Optional[str]:
    """Newest ``checkpoint-N`` directory whose ``.checkpoint_done`` marker (or a per-rank ``saved_signal_*`` for every
    expected writer) exists; incomplete checkpoints of a crashed save are skipped
    (paddleformers/trainer/trainer_utils.py:458-513)."""
    if not os.path.isdir(folder):
        return None
    cands = []
    for name in os.listdir(folder):
        m = _re_checkpoint.match(name)
        if m and os.path.isdir(os.path.join(folder, name)):
            cands.append((int(m.group(1)), os.path.join(folder, name)))
    for _, path in sorted(cands, reverse=True):
        if not require_complete or checkpoint_is_complete(path):
            return path
    return None


def checkpoint_is_complete(path: str) -> bool:
    if os.path.exists(os.path.join(path, ".checkpoint_done")):
        return True
    meta = os.path.join(path, "save_meta.json")
    if os.path.exists(meta):
        import json

        with open(meta) as f:
            expect = json.load(f).get("num_writers", 1)
        have = len([f for f in os.listdir(path) if f.startswith("saved_signal_")])
        return have >= expect
    return False


class TrainerMemoryTracker:
    """Allocated / reserved / peak device memory in GB for the training log."""

    @staticmethod
    def snapshot() -> Dict[str, float]:
        if not torch.cuda.is_available():
            return {}
        gb = 1024 ** 3
        return {
            "max_memory_allocated": round(torch.cuda.max_memory_allocated() / gb, 3),
            "max_memory_reserved": round(torch.cuda.max_memory_reserved() / gb, 3),
            "memory_allocated": round(torch.cuda.memory_allocated() / gb, 3),
        }
