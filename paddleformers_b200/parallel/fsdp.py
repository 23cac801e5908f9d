"""Sharding stage 3: parameters, gradients and optimizer state all sharded over the data ranks (ZeRO-3 / FSDP).

The reference reaches this level through ``group_sharded_parallel(level="p_g_os")`` and Paddle's ``fully_shard``
(paddleformers/trainer/trainer.py:4153-4309); like there it excludes pipeline parallelism, and here also tensor and
expert parallelism (``ShardedAdamW`` with stage 1 covers those).

Design:

* every decoder layer is a *unit*. A unit's parameters live in one flat buffer of which a rank keeps only its 1/N slice
  (fp32 master values, both Adam moments and an fp32 gradient accumulator for that slice). The bf16 working copy of a whole
  unit exists only while the unit computes: it is all-gathered into ONE transient buffer shared by all units.
* a unit's forward runs without recording a graph; its backward all-gathers the parameters again, re-runs the forward with
  a graph, back-propagates, reduce-scatters the unit's fp32 gradients into the local accumulator and drops the buffers.
  Stage 3 therefore implies full activation recompute per layer, which is the configuration such large models train in
  anyway, and it is what makes one shared parameter buffer possible: nothing saved for backward ever points into it.
  The layer parameters are permanently views of that buffer, so their values are only meaningful while their unit
  computes; read them through ``full_tensor`` / ``save_pretrained`` (which gather) otherwise.
* everything outside the decoder layers (embedding, final norm, head, MTP layers) forms the *root* unit: its working copy
  stays whole for the duration of a step (it is needed at both ends of forward and backward), its master values,
  moments and gradients are sharded like the others, and its gradients are reduce-scattered at the step boundary.

Gradient clipping uses the global norm over all shards; the update is the fused AdamW kernel on GPU shards and the same
arithmetic in tensor operations on CPU.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as F
from .topology import ParallelState, get_parallel_state

_ALIGN = 128


class _Unit:
    def __init__(self, name: str, params: List[Tuple[str, nn.Parameter]], rank: int, world: int, group):
        self.name, self.params, self.rank, self.world, self.group = name, params, rank, world, group
        self.shard_rank, self.shard_size = rank, world            # names the checkpoint code reads
        self.offsets: Dict[str, Tuple[int, int]] = {}
        total = 0
        for n, p in params:
            self.offsets[n] = (total, p.numel())
            total += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        unit = _ALIGN * world
        self.numel = (total + unit - 1) // unit * unit
        self.shard_numel = self.numel // world
        self.dtype = params[0][1].dtype
        dev = params[0][1].device
        flat = torch.zeros(self.numel, dtype=self.dtype, device=dev)
        for n, p in params:
            off, cnt = self.offsets[n]
            flat[off:off + cnt] = p.data.reshape(-1)
        lo = rank * self.shard_numel
        self.param_shard = flat[lo:lo + self.shard_numel].clone()            # working-precision slice (source of the all-gather)
        self.master = self.param_shard.float()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad_shard = torch.zeros_like(self.master)
        self.no_decay = torch.zeros(self.shard_numel, dtype=torch.bool, device=dev)
        for n, p in params:
            if "bias" in n or "norm" in n:
                off, cnt = self.offsets[n]
                a, b = max(off, lo), min(off + cnt, lo + self.shard_numel)
                if b > a:
                    self.no_decay[a - lo:b - lo] = True
        self.full: Optional[torch.Tensor] = None         # set by ``bind``
        self.full_grad: Optional[torch.Tensor] = None

    # -- the working copy: parameters are bound ONCE to views of a buffer (shared by all layer units, so its content is only
    #    meaningful between ``gather`` and the next unit's ``gather``); shapes and dtypes therefore never change
    def bind(self, buf: torch.Tensor, gbuf: torch.Tensor) -> None:
        self.full, self.full_grad = buf[:self.numel], gbuf[:self.numel]
        for n, p in self.params:
            off, cnt = self.offsets[n]
            p.data = self.full[off:off + cnt].view(p.shape)
            p.main_grad = self.full_grad[off:off + cnt].view(p.shape)     # weight-gradient kernels accumulate here in fp32
            p.grad = None

    def gather(self, with_grad: bool = False) -> None:
        if self.world > 1:
            dist.all_gather_into_tensor(self.full, self.param_shard, group=self.group)
        else:
            self.full.copy_(self.param_shard)
        if with_grad:
            self.full_grad.zero_()

    def fold_autograd_grads(self) -> None:
        for _, p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None

    def reduce_grads(self) -> None:
        """Sum the unit's full fp32 gradient over the ranks and add this rank's slice to its accumulator."""
        self.fold_autograd_grads()
        if self.world > 1:
            out = torch.empty(self.shard_numel, dtype=torch.float32, device=self.full_grad.device)
            dist.reduce_scatter_tensor(out, self.full_grad, group=self.group)
            self.grad_shard.add_(out)
        else:
            self.grad_shard.add_(self.full_grad[:self.shard_numel])


class _UnitFn(torch.autograd.Function):
    """Forward without a graph on gathered parameters; backward = gather, recompute with a graph, back-propagate,
    reduce-scatter the parameter gradients."""

    @staticmethod
    def forward(ctx, unit, fn, n_tensor, *args):
        ctx.unit, ctx.fn = unit, fn
        tensors, ctx.rest = args[:n_tensor], args[n_tensor:]
        ctx.save_for_backward(*[t for t in tensors if t is not None])
        ctx.mask = [t is not None for t in tensors]
        unit.gather()
        with torch.no_grad():
            out = fn(*tensors, *ctx.rest)
        return out

    @staticmethod
    def backward(ctx, *grads):
        unit = ctx.unit
        saved = list(ctx.saved_tensors)
        ins = [saved.pop(0).detach().requires_grad_(True) if m else None for m in ctx.mask]
        unit.gather(with_grad=True)
        with torch.enable_grad():
            out = ctx.fn(*ins, *ctx.rest)
        outs = out if isinstance(out, tuple) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if o is not None and g is not None and o.requires_grad]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        unit.reduce_grads()
        return (None, None, None) + tuple(i.grad if i is not None else None for i in ins) + (None,) * len(ctx.rest)


class FullyShardedOptimizer:
    """Wraps ``model`` in place (decoder layers become sharded units) and is the optimizer of the wrapped model: the
    interface the trainer uses (``accumulate_grads``, ``step(lr)``, ``zero_grad``, ``state_dict`` / ``load_state_dict``)."""

    def __init__(self, model: nn.Module, lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 max_grad_norm: float = 0.0, parallel_state: Optional[ParallelState] = None, **unused):
        ps = parallel_state or get_parallel_state()
        d = ps.degrees
        if d.mp > 1 or d.pp > 1 or d.ep > 1 or d.cp > 1 or d.sep > 1:
            raise ValueError("sharding stage 3 shards over the data ranks only: tensor / pipeline / expert / context degrees must be 1")
        self.ps, self.model = ps, model
        self.lr, self.betas, self.eps, self.weight_decay, self.max_grad_norm = lr, betas, eps, weight_decay, max_grad_norm
        self.step_count = 0
        multi = dist.is_initialized() and ps.world_size > 1
        self.group = ps.group("data") if multi else None
        self.world = dist.get_world_size(self.group) if multi else 1
        self.rank = dist.get_rank(self.group) if multi else 0
        layers = self._find_layers(model)
        in_layer = set()
        self.units: List[_Unit] = []
        for lname, layer in layers:
            ps_ = [(f"{lname}.{n}", p) for n, p in layer.named_parameters() if p.requires_grad]
            in_layer.update(id(p) for _, p in ps_)
            if ps_:
                u = _Unit(lname, ps_, self.rank, self.world, self.group)
                self.units.append(u)
                self._wrap(layer, u)
        root_params = [(n, p) for n, p in model.named_parameters() if p.requires_grad and id(p) not in in_layer]
        self.root = _Unit("root", root_params, self.rank, self.world, self.group) if root_params else None
        dev = next(model.parameters()).device
        biggest = max([u.numel for u in self.units] or [0])
        dtype = self.units[0].dtype if self.units else torch.float32
        self._pbuf = torch.empty(biggest, dtype=dtype, device=dev)          # ONE working copy for all layer units
        self._gbuf = torch.empty(biggest, dtype=torch.float32, device=dev)
        for u in self.units:
            u.bind(self._pbuf, self._gbuf)
        if self.root is not None:
            self._root_buf = torch.empty(self.root.numel, dtype=self.root.dtype, device=dev)
            self._root_gbuf = torch.empty(self.root.numel, dtype=torch.float32, device=dev)
            self.root.bind(self._root_buf, self._root_gbuf)
            self.root.gather(with_grad=True)
        self._scalars = torch.zeros(8, dtype=torch.float32, device=dev)
        self.last_grad_norm: Optional[torch.Tensor] = None
        model.save_pretrained = self._save_pretrained          # gathers unit by unit

    @staticmethod
    def _find_layers(model: nn.Module):
        out = []
        for name, mod in model.named_modules():
            if isinstance(mod, (nn.ModuleDict, nn.ModuleList)) and name.split(".")[-1] == "layers":
                items = mod.items() if isinstance(mod, nn.ModuleDict) else enumerate(mod)
                out += [(f"{name}.{k}", m) for k, m in items]
        return out

    def _wrap(self, layer: nn.Module, unit: _Unit) -> None:
        inner = layer.forward

        def forward(*args):
            # tensors first (hidden states, residual stream or None), then everything else (batch context, cache)
            n = 0
            while n < len(args) and (args[n] is None or torch.is_tensor(args[n])):
                n += 1
            if not torch.is_grad_enabled():
                unit.gather()
                return inner(*args)
            return _UnitFn.apply(unit, inner, n, *args)

        layer.forward = forward

    # ------------------------------------------------------------------ trainer interface
    @property
    def all_units(self) -> List[_Unit]:
        return self.units + ([self.root] if self.root is not None else [])

    def accumulate_grads(self) -> None:
        if self.root is not None:
            self.root.fold_autograd_grads()

    def zero_grad(self) -> None:
        for u in self.all_units:
            u.grad_shard.zero_()
        if self.root is not None:
            self.root.full_grad.zero_()
            for _, p in self.root.params:
                p.grad = None

    @torch.no_grad()
    def step(self, lr: Optional[float] = None) -> torch.Tensor:
        if lr is not None:
            self.lr = lr
        if self.root is not None:
            self.root.reduce_grads()
            self.root.full_grad.zero_()
        inv = 1.0 / self.world
        sq = torch.zeros(1, dtype=torch.float32, device=self._scalars.device)
        for u in self.all_units:
            if inv != 1.0:
                u.grad_shard.mul_(inv)                       # mean over the data ranks
            sq += u.grad_shard.double().pow(2).sum().float()
        if self.world > 1:
            dist.all_reduce(sq, group=self.group)
        gnorm = sq.sqrt().squeeze(0)
        self.last_grad_norm = gnorm
        self.step_count += 1
        b1, b2 = self.betas
        bc1, bc2 = 1.0 - b1 ** self.step_count, 1.0 - b2 ** self.step_count
        finite = torch.isfinite(gnorm)
        clip = torch.clamp(self.max_grad_norm / (gnorm + 1e-6), max=1.0) if self.max_grad_norm and self.max_grad_norm > 0 \
            else torch.ones_like(gnorm)
        gmul = torch.where(finite, clip, torch.zeros_like(clip))
        keep = finite.to(torch.float32)
        for u in self.all_units:
            g = u.grad_shard * gmul
            g = torch.where(finite, g, torch.zeros_like(g))
            u.exp_avg.mul_(torch.where(finite, torch.tensor(b1, device=g.device), torch.ones((), device=g.device))).add_(g * (1 - b1))
            u.exp_avg_sq.mul_(torch.where(finite, torch.tensor(b2, device=g.device), torch.ones((), device=g.device))).addcmul_(g, g, value=1 - b2)
            decay = torch.where(u.no_decay, torch.zeros((), device=g.device), torch.full((), self.lr * self.weight_decay, device=g.device))
            upd = (u.exp_avg / bc1) / ((u.exp_avg_sq / bc2).sqrt() + self.eps)
            u.master.mul_(1.0 - decay * keep).add_(upd * (-(self.lr) * keep))
            u.param_shard.copy_(u.master)
            u.grad_shard.zero_()
        if self.root is not None:                           # refresh the whole working copy of the root unit
            self.root.gather(with_grad=True)
        return gnorm

    # ------------------------------------------------------------------ state
    @property
    def domains(self) -> List[_Unit]:
        """The units under the name the checkpoint code uses for a separately sharded flat buffer."""
        return self.all_units

    def state_dict(self) -> Dict[str, object]:
        """This rank's slices in the layout of ``ShardedAdamW.state_dict`` (one entry per unit), so that the trainer's
        checkpoint writer, its completeness markers and its re-cutting for another number of ranks apply unchanged."""
        return {"step": self.step_count, "lr": self.lr,
                "domains": {u.name: {"master": u.master.cpu(), "exp_avg": u.exp_avg.cpu(), "exp_avg_sq": u.exp_avg_sq.cpu(),
                                     "offsets": dict(u.offsets), "numel": u.numel, "shard_rank": u.rank, "shard_size": u.world}
                            for u in self.all_units}}

    def load_state_dict(self, sd: Dict[str, object]) -> None:
        self.step_count, self.lr = int(sd["step"]), float(sd.get("lr", self.lr))
        for u in self.all_units:
            s = sd["domains"][u.name]
            if tuple(s["master"].shape) != tuple(u.master.shape):
                raise ValueError(f"{u.name}: optimizer slice of {tuple(s['master'].shape)} does not fit {tuple(u.master.shape)}")
            u.master.copy_(s["master"]); u.exp_avg.copy_(s["exp_avg"]); u.exp_avg_sq.copy_(s["exp_avg_sq"])
            u.param_shard.copy_(u.master)
        if self.root is not None:
            self.root.gather(with_grad=True)

    def memory_bytes(self) -> int:
        n = self._pbuf.numel() * self._pbuf.element_size() + self._gbuf.numel() * 4
        for u in self.all_units:
            n += u.shard_numel * (u.param_shard.element_size() + 16)
        if self.root is not None:
            n += self.root.numel * (self.root.param_shard.element_size() + 4)
        return n

    # ------------------------------------------------------------------ export
    def full_tensor(self, p: nn.Parameter) -> torch.Tensor:
        """The whole current value of a parameter of the wrapped model, on the host (collective over the data ranks)."""
        for u in self.all_units:
            for n, q in u.params:
                if q is p:
                    if u is self.root:
                        return p.detach().cpu().clone()
                    if getattr(self, "_export_unit", None) is not u:
                        u.gather()
                        self._export_unit = u
                    off, cnt = u.offsets[n]
                    return u.full[off:off + cnt].view(p.shape).detach().cpu().clone()
        return p.detach().cpu().clone()

    def _save_pretrained(self, save_directory: str, **kw):
        try:
            type(self.model).save_pretrained(self.model, save_directory, tensor_for=self.full_tensor, **kw)
        finally:
            self._export_unit = None
