"""Sharding of iterable datasets over data ranks and broadcast of batches inside model-parallel groups.

``IterableDatasetShard`` plays the role of paddleformers/trainer/trainer_utils.py's class of the same name;
``DistDataLoader`` the role of paddleformers/data/dist_dataloader.py:42 (only the first rank of each tensor /
pipeline group reads data, the batch is broadcast to the others).
"""
from __future__ import annotations

from typing import Any, Dict, Iterator, Optional

import torch
import torch.distributed as dist
from torch.utils.data import IterableDataset


class IterableDatasetShard(IterableDataset):
    def __init__(self, dataset, batch_size: int, drop_last: bool, num_processes: int, process_index: int, seed: int = 0):
        self.dataset, self.batch_size, self.drop_last = dataset, batch_size, drop_last
        self.num_processes, self.process_index = num_processes, process_index
        self.epoch = 0

    def set_epoch(self, epoch):
        self.epoch = epoch
        if hasattr(self.dataset, "set_epoch"):
            self.dataset.set_epoch(epoch)

    def __iter__(self):
        real = self.batch_size * self.num_processes
        lo = self.process_index * self.batch_size
        buf, first = [], None
        for el in self.dataset:
            buf.append(el)
            if len(buf) == real:
                for i in range(lo, lo + self.batch_size):
                    yield buf[i]
                if first is None:
                    first = list(buf)
                buf = []
        if not self.drop_last and buf:
            if first is None:
                first = list(buf)
            while len(buf) < real:
                buf += first
            for i in range(lo, lo + self.batch_size):
                yield buf[i]


class DistDataLoader:
    """Wraps a loader so that only the source rank of ``group`` iterates it; every batch (a dict of tensors) is
    broadcast to the other ranks: first the structure (keys, shapes, dtypes) as an object, then the tensors."""

    def __init__(self, loader, group, src_rank_in_group: int = 0, device: Optional[torch.device] = None):
        self.loader, self.group, self.device = loader, group, device
        self.is_src = dist.get_rank(group) == src_rank_in_group if group is not None and dist.is_initialized() else True
        self.src_global = dist.get_global_rank(group, src_rank_in_group) if (group is not None and dist.is_initialized() and hasattr(group, "size") and group.size() > 1) else 0
        self.multi = group is not None and dist.is_initialized() and getattr(group, "size", lambda: 1)() > 1

    def __len__(self):
        return len(self.loader)

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        if not self.multi:
            yield from self.loader
            return
        it = iter(self.loader) if self.is_src else None
        while True:
            meta = [None]
            batch = None
            if self.is_src:
                try:
                    batch = next(it)
                    meta = [{k: (tuple(v.shape), v.dtype) for k, v in batch.items()}]
                except StopIteration:
                    meta = ["stop"]
            dist.broadcast_object_list(meta, src=self.src_global, group=self.group)
            if meta[0] == "stop":
                return
            out = {}
            for k, (shape, dtype) in meta[0].items():
                t = batch[k] if self.is_src else torch.empty(shape, dtype=dtype)
                if self.device is not None:
                    t = t.to(self.device)
                dist.broadcast(t, src=self.src_global, group=self.group)
                out[k] = t
            yield out
