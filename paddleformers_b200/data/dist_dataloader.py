"""Sharding of iterable datasets over data ranks and broadcast of batches inside model-parallel groups.

``IterableDatasetShard`` plays the role of paddleformers/trainer/trainer_utils.py's class of the same name;
``StreamDistDataLoader`` (one reader for the whole job, batches scattered to the data ranks) that of :257;
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


class StreamDistDataLoader:
    """Loader for a stream (an iterable dataset) that only ONE process reads: the first rank of ``stream_group`` pulls
    ``group size`` batches per step from the stream and scatters one to every data rank; each data rank then shares its
    batch with its tensor / pipeline / context-parallel peers through ``DistDataLoader``'s broadcast. Compared with
    ``IterableDatasetShard`` no rank reads and throws away the other ranks' samples, and a source that cannot be opened
    twice (a socket, a queue) works (paddleformers/data/dist_dataloader.py:257).

    ``dataset`` may be None on every rank but the reader. A background thread keeps ``reader_buffer_size`` global batches
    ready on the reader. An incomplete last global batch is dropped, so that all data ranks stop together."""

    def __init__(self, dataset, batch_size: int = 1, collate_fn=None, stream_group=None, model_parallel_group=None,
                 reader_buffer_size: int = 2, device: Optional[torch.device] = None):
        self.dataset, self.batch_size, self.collate_fn = dataset, int(batch_size), collate_fn or (lambda x: x)
        self.group, self.mp_group, self.device = stream_group, model_parallel_group, device
        self.buffer = max(int(reader_buffer_size), 1)
        on = dist.is_initialized()
        self.n = dist.get_world_size(stream_group) if on else 1
        self.rank = dist.get_rank(stream_group) if on else 0
        self.in_stream_group = self.rank >= 0
        self.src_global = dist.get_global_rank(stream_group, 0) if (on and stream_group is not None) else 0

    def _global_batches(self):
        """Reader side: lists of ``n`` collated batches."""
        items, batches = [], []
        for el in self.dataset:
            items.append(el)
            if len(items) == self.batch_size:
                batches.append(self.collate_fn(items))
                items = []
                if len(batches) == self.n:
                    yield batches
                    batches = []

    def _prefetched(self):
        import queue
        import threading

        q: "queue.Queue" = queue.Queue(maxsize=self.buffer)
        end = object()

        def work():
            try:
                for gb in self._global_batches():
                    q.put(gb)
                q.put(end)
            except BaseException as e:  # noqa: BLE001 - re-raised on the consumer side
                q.put(e)

        threading.Thread(target=work, daemon=True).start()
        while True:
            x = q.get()
            if x is end:
                return
            if isinstance(x, BaseException):
                raise x
            yield x

    def _scattered(self):
        if self.n == 1:
            for gb in self._prefetched():
                yield gb[0]
            return
        src = self._prefetched() if self.rank == 0 else None
        while True:
            recv = [None]
            send = None
            if self.rank == 0:
                gb = next(src, None)
                send = list(gb) if gb is not None else ["stop"] * self.n
            dist.scatter_object_list(recv, send, src=self.src_global, group=self.group)
            if isinstance(recv[0], str) and recv[0] == "stop":
                return
            yield recv[0]

    def __iter__(self):
        class _Once:                        # DistDataLoader wants an iterable; only the data rank of each group has one
            def __init__(s, gen):
                s.gen = gen

            def __iter__(s):
                return s.gen

        multi_mp = self.mp_group is not None and dist.is_initialized() and dist.get_world_size(self.mp_group) > 1
        if not multi_mp:
            for b in self._scattered():
                yield self._to_device(b)
            return
        is_data_rank = dist.get_rank(self.mp_group) == 0
        inner = DistDataLoader(_Once(self._scattered() if is_data_rank else iter(())), self.mp_group, 0, self.device)
        yield from inner

    def _to_device(self, b):
        if self.device is None or not isinstance(b, dict):
            return b
        return {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in b.items()}
