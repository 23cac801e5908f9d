"""Zero-cost checkpoints: snapshot the optimizer shard to pinned host memory on a side stream, persist it in the
background, never stall the training stream for either.

What the reference's ``ZeroCostCheckpointManager`` does with CUDA IPC and a worker process
(paddleformers/trainer/utils/zero_cost_checkpoint.py:918; the copies are its ``async_offload`` calls, :57-60). Here one
process per GPU already owns one contiguous fp32 master / moment shard per reduction domain, so a snapshot is three
large device-to-host copies per domain:

* ``snapshot()`` (called at a save step, after the optimizer update): a copy stream waits for the training stream,
  issues the copies into pre-allocated pinned buffers and records an event. The training stream is not blocked.
* ``before_update()`` (called before the next optimizer update): the training stream waits for that event, because the
  update overwrites what is being copied. A full forward + backward lies in between, so the wait is normally free.
* the writer thread waits for the event on the host, then writes the same ``optimizer/shard_*.pt`` files as a regular
  checkpoint. The working bf16 weights are not saved: resuming rebuilds them from the fp32 master shards
  (``ShardedAdamW.load_state_dict``), plus a small file of buffers and frozen parameters that no optimizer shard holds.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch


class ZeroCostCheckpointManager:
    def __init__(self, optimizer, model: torch.nn.Module):
        self.opt = optimizer
        self.model = model
        self.cuda = any(d.master.is_cuda for d in optimizer.domains)
        self.stream = torch.cuda.Stream() if self.cuda else None
        self.event: Optional[torch.cuda.Event] = None
        self.host: Dict[str, Dict[str, torch.Tensor]] = {}
        for dom in optimizer.domains:
            self.host[dom.name] = {k: torch.empty(getattr(dom, k).shape, dtype=getattr(dom, k).dtype, device="cpu",
                                                  pin_memory=self.cuda) for k in ("master", "exp_avg", "exp_avg_sq")}
        self.snapshots = 0

    def host_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for d in self.host.values() for t in d.values())

    def snapshot(self) -> Dict[str, object]:
        """Start copying the shard; returns the state dict whose tensors are valid once ``wait_host()`` returned."""
        opt = self.opt
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                for dom in opt.domains:
                    for k, h in self.host[dom.name].items():
                        h.copy_(getattr(dom, k), non_blocking=True)
                self.event = torch.cuda.Event()
                self.event.record(self.stream)
        else:
            for dom in opt.domains:
                for k, h in self.host[dom.name].items():
                    h.copy_(getattr(dom, k))
        self.snapshots += 1
        out = {"step": opt.step_count, "lr": opt.lr, "domains": {}}
        for dom in opt.domains:
            out["domains"][dom.name] = {**self.host[dom.name], "offsets": dict(dom.offsets), "numel": dom.numel,
                                        "shard_rank": dom.shard_rank, "shard_size": dom.shard_size}
        return out

    def extra_state(self) -> Dict[str, torch.Tensor]:
        """Buffers and parameters that are not in any optimizer shard (router bias buffers, frozen weights)."""
        owned = {id(p) for dom in self.opt.domains for _, p in dom.params}
        out = {f"buffer:{n}": b.detach().cpu() for n, b in self.model.named_buffers() if b is not None}
        out.update({f"param:{n}": p.detach().cpu() for n, p in self.model.named_parameters() if id(p) not in owned})
        return out

    def before_update(self):
        """Order the next optimizer update after the snapshot copies (device-side wait, no host stall)."""
        if self.cuda and self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)

    def wait_host(self):
        if self.cuda and self.event is not None:
            self.event.synchronize()


def load_extra_state(model: torch.nn.Module, extra: Dict[str, torch.Tensor]) -> None:
    buffers = dict(model.named_buffers())
    params = dict(model.named_parameters())
    with torch.no_grad():
        for key, t in extra.items():
            kind, name = key.split(":", 1)
            target = buffers.get(name) if kind == "buffer" else params.get(name)
            if target is not None:
                target.copy_(t)
