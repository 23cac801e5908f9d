"""Refined recompute: under per-layer activation recompute, named operations keep what they saved for the backward pass and
are not run again when the layer is recomputed (paddleformers/transformers/refined_recompute.py:166-258 ``no_recompute``,
:512-568 ``get_skip_recompute_ops``). Recomputing a decoder layer then costs the norms, rotary embedding and activations
only, not the attention kernel or the chosen GEMMs, for the price of holding those operations' inputs and outputs.

Mechanism (non-reentrant ``torch.utils.checkpoint``): the checkpoint discards every tensor that an operation saves for
backward and rebuilds them by running the function a second time. A kept operation

* in the original forward runs under an identity ``saved_tensors_hooks`` pair, which shadows the checkpoint's hook: its saved
  tensors stay alive in the graph, and its output is remembered;
* in the recomputation is skipped: the remembered output is handed to the operations that follow (they only need its value to
  rebuild their own saved tensors). Nothing is saved inside the skipped region in either pass, so the checkpoint's bookkeeping
  of saved tensors stays consistent.

Operation names are the reference's: ``attention_column_ln`` (qkv projection), ``flash_attn``, ``attention_row_ln`` (output
projection), ``mlp_column_ln`` (gate / up projection with its activation), ``mlp_row_ln`` (down projection).
"""
from __future__ import annotations

import math
import threading
from collections import deque
from typing import Callable, Dict, Iterable, Sequence, Set

import torch
import torch.utils.checkpoint

OP_NAMES = ("attention_column_ln", "flash_attn", "attention_row_ln", "mlp_column_ln", "mlp_row_ln")
STATS = {"kept": 0, "reused": 0}

_local = threading.local()


class _Frame:
    __slots__ = ("keep_ops", "calls", "outputs")

    def __init__(self, keep_ops: Set[str]):
        self.keep_ops, self.calls, self.outputs = keep_ops, 0, deque()


def _remember(out):
    if isinstance(out, torch.Tensor):
        d = out.detach()
        # operations that follow decide what to save from whether their inputs require gradients: keep that property
        return d.requires_grad_(True) if (out.requires_grad and d.is_floating_point()) else d
    if isinstance(out, (tuple, list)):
        return type(out)(_remember(o) for o in out)
    return out


def keep(name: str, fn: Callable, *args, **kwargs):
    """Run ``fn(*args, **kwargs)``; inside a refined-recompute frame that lists ``name`` the call is made once only."""
    fr = getattr(_local, "frame", None)
    if fr is None or name not in fr.keep_ops or not torch.is_grad_enabled():
        return fn(*args, **kwargs)
    if fr.calls == 1:                                     # original forward
        with torch.autograd.graph.saved_tensors_hooks(lambda t: t, lambda t: t):
            out = fn(*args, **kwargs)
        fr.outputs.append(_remember(out))
        STATS["kept"] += 1
        return out
    STATS["reused"] += 1
    return fr.outputs.popleft()                           # recomputation: same order of calls as the forward


def checkpoint_keeping(fn: Callable, keep_ops: Iterable[str], *args):
    """``torch.utils.checkpoint.checkpoint(fn, *args)`` whose operations named in ``keep_ops`` are not recomputed."""
    keep_ops = set(keep_ops)
    if not keep_ops:
        return torch.utils.checkpoint.checkpoint(fn, *args, use_reentrant=False)
    frame = _Frame(keep_ops)

    def framed(*a):
        frame.calls += 1
        prev = getattr(_local, "frame", None)
        _local.frame = frame
        try:
            return fn(*a)
        finally:
            _local.frame = prev

    return torch.utils.checkpoint.checkpoint(framed, *args, use_reentrant=False)


def kept_ops_of_layer(spec: Dict[str, int], layer_idx: int, num_layers: int, stage_layers: Sequence[int] = ()) -> Set[str]:
    """Operations that layer ``layer_idx`` keeps. ``spec[name] = n``: the operation is recomputed in ``n`` layers and kept in
    the other ``num_layers - n`` (n == 0: kept everywhere; n < 0: recomputed everywhere). Without pipeline stages the FIRST
    ``num_layers - n`` layers keep it; with ``stage_layers`` (the layers of this pipeline stage) every stage keeps it in its
    first ``ceil(share)`` layers, so that the memory is spread evenly over the stages."""
    out = set()
    for name, n in (spec or {}).items():
        if name not in OP_NAMES:
            raise ValueError(f"refined_recompute: unknown operation {name!r}; known: {', '.join(OP_NAMES)}")
        n = int(n)
        if n < 0:
            continue
        keep_layers = num_layers if n == 0 else max(num_layers - n, 0)
        if stage_layers and len(stage_layers) < num_layers:
            local = list(stage_layers)
            k = math.ceil(len(local) * keep_layers / max(num_layers, 1))
            if layer_idx in local[:k]:
                out.add(name)
        elif layer_idx < keep_layers:
            out.add(name)
    return out
