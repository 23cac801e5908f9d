"""Flat-buffer mixed-precision optimizer with optimizer-state sharding (ZeRO stage 1 / 2).

Design (the reference's sharding stage-1 "V2" / split_param semantics, paddleformers/trainer/training_args.py:
2288-2400 and Fleet's DygraphShardingOptimizerV2, plus its fp32 ``main_grad`` accumulation):

* Parameters of one reduction domain live in ONE flat working buffer (bf16 for bf16 models); every ``nn.Parameter``
  is a view into it, and every parameter gets a ``main_grad`` view into a flat fp32 gradient buffer. Weight-gradient
  kernels accumulate straight into ``main_grad``; gradients produced by ordinary autograd ops are folded in by
  ``accumulate_grads()`` after each micro-batch.
* Each rank of the sharding group owns a contiguous 1/N slice of every flat buffer: fp32 master weights and both
  Adam moments exist only for that slice. A step = reduce-scatter of the flat gradient (sum over the sharding group,
  plus all-reduce over the pure data-parallel group), global-norm clipping, the fused AdamW kernel on the slice
  (which also writes the bf16 working copy), and an all-gather of the working buffer.
* Expert parameters form their own domain, reduced over the ``moe_sharding`` group only, with gradient scale
  tp*cp/ep relative to dense parameters (paddleformers/trainer/training_args.py:2808-2815); the gradient norm is
  combined across domains and model-parallel groups like the reference's MoE-aware clip
  (paddleformers/utils/moe_hybrid_parallel_optimizer.py:60-160).
* On GPUs the flat buffers of a sharded domain live in symmetric (peer-mapped) memory and the step uses two fused
  kernels instead of three library collectives (``csrc/shard_comm.cu``): ``shard_reduce`` reads this rank's gradient
  slice out of every peer's buffer, sums in rank order, scales and accumulates the squared norm in one pass;
  ``adamw_push`` updates the slice and stores the bf16 weights into every rank's parameter buffer, which is the
  all-gather. ``PFB_FUSED_SHARDING=0`` keeps the NCCL reduce-scatter / all-gather path (the A/B baseline, and the path of
  CPU ranks).
* Weight decay follows the reference's name rule: parameters whose name contains "bias" or "norm" are not decayed
  (paddleformers/trainer/trainer.py:3645-3656).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as F
from .topology import ParallelState, get_parallel_state

_ALIGN = 128  # elements; keeps every shard boundary 512-byte aligned for the vectorised kernels


def _group_size(g) -> int:
    return g.size() if g is not None else 1


@dataclass
class _Domain:
    """One flat (params, grads, optimizer shard) set."""

    name: str
    params: List[Tuple[str, torch.nn.Parameter]]
    weight_decay: float
    shard_group: object
    shard_size: int
    shard_rank: int
    extra_reduce_group: object = None      # pure data-parallel replicas of the sharding group
    grad_scale: float = 1.0
    flat_param: torch.Tensor = None
    flat_grad: torch.Tensor = None
    master: torch.Tensor = None
    exp_avg: torch.Tensor = None
    exp_avg_sq: torch.Tensor = None
    offsets: Dict[str, Tuple[int, int]] = field(default_factory=dict)
    numel: int = 0
    is_expert: bool = False
    is_muon: bool = False          # matrices updated by the orthogonalised-momentum rule (see ShardedMuon)
    symm: Optional[dict] = None    # peer-memory state of the fused reduce / update kernels (None: library collectives)

    @property
    def shard_numel(self) -> int:
        return self.numel // self.shard_size

    def shard_slice(self, t: torch.Tensor) -> torch.Tensor:
        n = self.shard_numel
        return t[self.shard_rank * n:(self.shard_rank + 1) * n]


def default_no_decay(name: str) -> bool:
    return "bias" in name or "norm" in name


class ShardedAdamW:
    """AdamW over flat buffers; works for world size 1 (no sharding) up to any sharding / moe_sharding degree.
    Subclasses that set ``custom_update`` replace the update rule of a shard by their own ``_update`` (the gradient
    reduction, clipping and parameter all-gather stay the same)."""

    custom_update = False

    def __init__(self, model: torch.nn.Module, lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, max_grad_norm: float = 0.0, parallel_state: Optional[ParallelState] = None,
                 no_decay_fn: Callable[[str], bool] = default_no_decay, grad_dtype=torch.float32,
                 release_grads: bool = False):
        self.ps = parallel_state or get_parallel_state()
        self.lr = lr
        self.betas = betas
        self.eps = eps
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.model = model
        self.domains: List[_Domain] = []
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.release_grads = release_grads
        ps = self.ps
        d = ps.degrees
        groups: Dict[Tuple[bool, bool, torch.dtype], List] = {}
        for name, p in model.named_parameters():
            if not p.requires_grad:
                continue
            key = (bool(getattr(p, "is_expert", False)), bool(no_decay_fn(name)), p.dtype, bool(self._is_muon_param(name, p)))
            groups.setdefault(key, []).append((name, p))
        # Expert gradients are summed over the moe_sharding group (all ranks that hold the same experts: mp x data / ep of
        # them, context- and segment-parallel ranks counted as data ranks because dense gradients are averaged over them
        # too) and divided by its size; relative to dense parameters, which are averaged over the data ranks, that needs a
        # factor. With sequence parallelism the tensor-parallel ranks of the group hold DIFFERENT tokens, so the sum is the
        # gradient of every token once: factor mp / ep. Without it they hold the SAME tokens and the sum counts every
        # token mp times: factor 1 / ep. (The reference's factor tp * cp / ep, paddleformers/trainer/training_args.py:
        # 2808-2815, is the same rule for a trainer that always runs MoE layers sequence parallel and does not average dense
        # gradients over the context-parallel ranks.)
        sp = bool(getattr(getattr(model, "config", None), "sequence_parallel", False)) and d.mp > 1
        expert_scale = float(d.mp if sp else 1) / float(d.ep) if d.ep > 1 else 1.0
        for (is_expert, no_decay, dtype, is_muon), plist in sorted(groups.items(),
                                                                   key=lambda kv: (kv[0][0], kv[0][1], str(kv[0][2]), kv[0][3])):
            if is_expert and d.ep > 1:
                sg, ssz, srk, extra = ps.group("moe_sharding"), ps.size("moe_sharding"), ps.rank_in("moe_sharding"), None
            else:
                sg, ssz, srk = ps.group("sharding"), d.sharding, ps.coord["sharding"]
                extra = ps.group("dp_sep_cp") if d.dp * d.sep * d.cp > 1 else None
            dom = _Domain(name=f"{'expert' if is_expert else 'dense'}_{'nodecay' if no_decay else 'decay'}_{str(dtype)[6:]}"
                               + ("_muon" if is_muon else ""),
                          params=plist, weight_decay=0.0 if no_decay else weight_decay, shard_group=sg if ssz > 1 else None,
                          shard_size=ssz, shard_rank=srk, extra_reduce_group=extra,
                          grad_scale=expert_scale if is_expert else 1.0, is_expert=is_expert, is_muon=is_muon)
            self._build_domain(dom, dtype)
            self.domains.append(dom)
        dev = self.domains[0].flat_param.device if self.domains else torch.device("cpu")
        self._scalars = torch.zeros(8, dtype=torch.float32, device=dev)
        self._norm_acc = torch.zeros(1, dtype=torch.float32, device=dev)

    def _is_muon_param(self, name: str, p) -> bool:
        return False

    # ------------------------------------------------------------------ construction
    def _build_domain(self, dom: _Domain, dtype):
        total = 0
        for name, p in dom.params:
            n = (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
            dom.offsets[name] = (total, p.numel())
            total += n
        unit = _ALIGN * dom.shard_size
        total = (total + unit - 1) // unit * unit
        dom.numel = total
        dev = dom.params[0][1].device
        if self._fused_sharding_ok(dom, dtype, dev):
            from .symmetric_memory import SymmetricBuffer

            pbuf = SymmetricBuffer(total * 2, dom.shard_group, dev)
            gbuf = SymmetricBuffer(total * 4, dom.shard_group, dev)
            fbuf = SymmetricBuffer(2 * 8 * 4, dom.shard_group, dev)
            dom.flat_param = pbuf.tensor((total,), dtype)
            dom.flat_grad = gbuf.tensor((total,), torch.float32)
            dom.flat_param.zero_()
            dom.flat_grad.zero_()
            dom.symm = {"bufs": (pbuf, gbuf, fbuf), "param_ptrs": torch.tensor(pbuf.peer_ptrs, dtype=torch.int64),
                        "grad_ptrs": torch.tensor(gbuf.peer_ptrs, dtype=torch.int64),
                        "flag_ptrs": torch.tensor(fbuf.peer_ptrs, dtype=torch.int64),
                        "epoch": torch.zeros(1, dtype=torch.int32, device=dev)}
        else:
            dom.flat_param = torch.zeros(total, dtype=dtype, device=dev)
            dom.flat_grad = torch.zeros(total, dtype=torch.float32, device=dev)
        for name, p in dom.params:
            off, n = dom.offsets[name]
            view = dom.flat_param[off:off + n].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = dom.flat_grad[off:off + n].view(p.shape)
        dom.master = dom.shard_slice(dom.flat_param).float().clone()
        dom.exp_avg = torch.zeros_like(dom.master)
        dom.exp_avg_sq = torch.zeros_like(dom.master)

    def _fused_sharding_ok(self, dom: _Domain, dtype, dev) -> bool:
        if dom.shard_group is None or dev.type != "cuda" or dtype != torch.bfloat16 or dom.shard_size > 8:
            return False
        if os.environ.get("PFB_FUSED_SHARDING", "1") == "0" or dom.is_muon or self.custom_update:
            return False
        try:
            return F._build.load_extension() and hasattr(torch.ops.pfb200, "shard_reduce")
        except Exception:  # noqa: BLE001
            return False

    # ------------------------------------------------------------------ gradient handling
    def accumulate_grads(self):
        """Fold ``.grad`` of parameters whose gradient came from ordinary autograd ops into ``main_grad``."""
        for dom in self.domains:
            for _, p in dom.params:
                if p.grad is not None:
                    p.main_grad.add_(p.grad.to(torch.float32))
                    p.grad = None

    def zero_grad(self):
        for dom in self.domains:
            dom.flat_grad.zero_()
            for _, p in dom.params:
                p.grad = None

    def sync_sequence_parallel_grads(self):
        """All-reduce gradients of tp-replicated parameters that saw token-sharded activations
        (paddleformers/trainer/trainer_callback.py:936-963): packed into one buffer, one all-reduce, unpacked."""
        if self.ps.degrees.mp <= 1:
            return
        g = self.ps.group("mp")
        grads = [p.main_grad for dom in self.domains for _, p in dom.params if getattr(p, "sequence_parallel", False)]
        if not grads:
            return
        if len(grads) == 1:
            dist.all_reduce(grads[0], group=g)
            return
        flat = torch.cat([t.reshape(-1) for t in grads])
        dist.all_reduce(flat, group=g)
        torch._foreach_copy_([t.reshape(-1) for t in grads], list(flat.split([t.numel() for t in grads])))

    def _replicated_slices(self, shards):
        """Views of the local gradient shards that belong to parameters replicated over the tp group (the static list of
        slice bounds is computed once)."""
        if getattr(self, "_rep_bounds", None) is None:
            ps = self.ps
            bounds = []
            for di, dom in enumerate(self.domains):
                if dom.is_expert and ps.degrees.ep > 1:
                    continue
                n = dom.shard_numel
                lo = dom.shard_rank * n
                for name, p in dom.params:
                    if getattr(p, "shard_spec", None) is None or getattr(p, "shard_spec")[0] != "tp":
                        off, cnt = dom.offsets[name]
                        a, b = max(off, lo), min(off + cnt, lo + n)
                        if b > a:
                            bounds.append((di, a - lo, b - lo))
            self._rep_bounds = bounds
        return [shards[di][a:b] for di, a, b in self._rep_bounds]

    def _pp_shared_slices(self, shards):
        """Views of the local gradient shards of parameters that exist on two pipeline stages (a head tied to the input
        embedding, the embedding copy of multi-token-prediction layers), on every stage but the first: both copies hold the
        summed gradient, and the norm must count it once."""
        if getattr(self, "_pp_shared_bounds", None) is None:
            bounds = []
            if self.ps.degrees.pp > 1 and self.ps.coord["pp"] != 0:
                for di, dom in enumerate(self.domains):
                    n = dom.shard_numel
                    lo = dom.shard_rank * n
                    for name, p in dom.params:
                        if getattr(p, "pp_shared", None):
                            off, cnt = dom.offsets[name]
                            a, b = max(off, lo), min(off + cnt, lo + n)
                            if b > a:
                                bounds.append((di, a - lo, b - lo))
            self._pp_shared_bounds = bounds
        return [shards[di][a:b] for di, a, b in self._pp_shared_bounds]

    def reduce_gradients(self):
        """Sum gradients over the data replicas: reduce-scatter inside the sharding group, all-reduce over dp.
        Returns the local fp32 gradient shard of every domain (views of the flat gradient buffers)."""
        shards = []
        for dom in self.domains:
            n = dom.shard_numel
            world = dom.shard_size * (_group_size(dom.extra_reduce_group))
            scale = dom.grad_scale / world
            local = dom.shard_slice(dom.flat_grad)
            if dom.symm is not None:
                # one pass: peer loads of this rank's slice from every rank's buffer, fixed-order sum, scale, squared norm
                sy = dom.symm
                sy["epoch"].add_(1)
                ops = torch.ops.pfb200
                ops.shard_signal(sy["grad_ptrs"], sy["param_ptrs"], sy["flag_ptrs"], dom.shard_rank, 0, sy["epoch"])
                sy["norm"] = torch.zeros(1, dtype=torch.float32, device=local.device)
                ops.shard_reduce(dom.flat_grad, sy["grad_ptrs"], sy["param_ptrs"], sy["flag_ptrs"], dom.shard_rank, dom.shard_rank * n, n,
                                 scale, sy["norm"], sy["epoch"])
                if dom.extra_reduce_group is not None:
                    dist.all_reduce(local, group=dom.extra_reduce_group)
                    sy["norm"] = None          # the slice changed after the kernel's norm: recomputed below
                shards.append(local)
                continue
            if dom.shard_group is not None:
                dist.reduce_scatter_tensor(local, dom.flat_grad, group=dom.shard_group)
            if dom.extra_reduce_group is not None:
                dist.all_reduce(local, group=dom.extra_reduce_group)
            if scale != 1.0:
                local.mul_(scale)
            shards.append(local)
        return shards

    def _global_grad_norm(self, shards) -> torch.Tensor:
        ps = self.ps
        acc_dense = torch.zeros(1, dtype=torch.float32, device=self._norm_acc.device)
        acc_expert = torch.zeros_like(acc_dense)
        for dom, g in zip(self.domains, shards):
            acc = acc_expert if dom.is_expert else acc_dense
            if dom.symm is not None and dom.symm.get("norm") is not None:
                acc += dom.symm["norm"]             # accumulated by the reduce kernel
            elif g.is_cuda:
                ops = torch.ops.pfb200
                scratch = F._get_scratch(g.device, int(ops.sq_norm_scratch_elems()))
                ops.sq_norm_accum(g, acc, scratch)
            else:
                acc += g.double().pow(2).sum().float()
        # tp-replicated parameters appear on every tp rank: their share is counted once by dividing, which is exact
        # because replicated gradients are identical after the sequence-parallel sync.
        if ps.degrees.mp > 1:
            views = self._replicated_slices(shards)
            if views:
                # one multi-tensor norm over all replicated slices instead of a launch per parameter
                rep = torch.stack(torch._foreach_norm(views)).double().pow(2).sum().float().reshape(1)
                acc_dense = acc_dense - rep * (1.0 - 1.0 / ps.degrees.mp)  # experts with ep == 1 are folded in here too
        dup = self._pp_shared_slices(shards)
        if dup:
            acc_dense = acc_dense - torch.stack(torch._foreach_norm(dup)).double().pow(2).sum().float().reshape(1)
        total = torch.cat([acc_dense, acc_expert])
        if dist.is_initialized() and ps.world_size > 1:
            # dense shards: sum over sharding x mp x pp (x sep x cp hold identical copies -> not summed);
            # expert shards: sum over moe_sharding x ep x pp. Both reduce to "sum over all ranks, divided by the
            # number of identical copies".
            d = ps.degrees
            dense_copies = d.dp * d.sep * d.cp
            expert_copies = 1 if d.ep > 1 else dense_copies
            if d.ep == 1:
                expert_copies = dense_copies
            total = total / torch.tensor([dense_copies, expert_copies], dtype=torch.float32, device=total.device)
            dist.all_reduce(total)
        return total.sum().sqrt()

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, lr: Optional[float] = None) -> torch.Tensor:
        """Reduces gradients, clips, updates the local shard, all-gathers parameters, zeroes gradients.
        Returns the global gradient norm (device tensor, no host sync)."""
        if lr is not None:
            self.lr = lr
        self.accumulate_grads()
        self.sync_sequence_parallel_grads()
        shards = self.reduce_gradients()
        gnorm = self._global_grad_norm(shards)
        self.last_grad_norm = gnorm
        self.step_count += 1
        b1, b2 = self.betas
        bc1, bc2 = 1.0 - b1 ** self.step_count, 1.0 - b2 ** self.step_count
        finite = torch.isfinite(gnorm)
        if self.max_grad_norm and self.max_grad_norm > 0:
            clip = torch.clamp(self.max_grad_norm / (gnorm + 1e-6), max=1.0)
        else:
            clip = torch.ones_like(gnorm)
        sc = self._scalars
        sc[0] = self.lr
        sc[1] = torch.where(finite, clip, torch.zeros_like(clip))
        sc[2] = bc1
        sc[3] = bc2
        sc[4] = (~finite).to(torch.float32)   # non-finite gradient: skip the update
        for dom, g in zip(self.domains, shards):
            pslice = dom.shard_slice(dom.flat_param)
            if dom.is_muon:
                self._muon_update(dom, g, pslice, sc)
            elif self.custom_update:
                self._update(dom, g, pslice, sc)
            elif dom.symm is not None:
                # update + all-gather in one kernel: the bf16 weights are stored into every rank's parameter buffer
                sy = dom.symm
                ops = torch.ops.pfb200
                n = dom.shard_numel
                ops.adamw_push(dom.master, dom.exp_avg, dom.exp_avg_sq, dom.flat_grad, sy["grad_ptrs"], sy["param_ptrs"], sy["flag_ptrs"],
                               dom.shard_rank, dom.shard_rank * n, sc, b1, b2, self.eps, dom.weight_decay)
                ops.shard_signal(sy["grad_ptrs"], sy["param_ptrs"], sy["flag_ptrs"], dom.shard_rank, 1, sy["epoch"])
                # every rank has pushed (and therefore finished reading this rank's gradients): the buffer may be cleared and
                # the next forward pass may read the parameters
                ops.shard_wait(sy["flag_ptrs"], dom.shard_rank, 1, sy["epoch"])
                dom.flat_grad.zero_()
                continue
            elif g.is_cuda:
                p16 = pslice if pslice.dtype == torch.bfloat16 else None
                torch.ops.pfb200.adamw_step(dom.master, dom.exp_avg, dom.exp_avg_sq, g, p16, sc, b1, b2, self.eps,
                                            dom.weight_decay)
                F.kernel_launch_count()
                if p16 is None:
                    pslice.copy_(dom.master)
            else:
                self._adamw_cpu(dom, g, pslice, sc)
            if dom.shard_group is not None:
                dist.all_gather_into_tensor(dom.flat_param, pslice.clone(), group=dom.shard_group)
            dom.flat_grad.zero_()
        return gnorm

    def _muon_update(self, dom, g, pslice, sc):
        raise NotImplementedError

    def _adamw_cpu(self, dom, g, pslice, sc):
        if float(sc[4]) != 0.0:
            return
        b1, b2 = self.betas
        lr, gmul, bc1, bc2 = float(sc[0]), float(sc[1]), float(sc[2]), float(sc[3])
        gr = g * gmul
        dom.exp_avg.mul_(b1).add_(gr, alpha=1 - b1)
        dom.exp_avg_sq.mul_(b2).addcmul_(gr, gr, value=1 - b2)
        dom.master.mul_(1 - lr * dom.weight_decay)
        dom.master.addcdiv_(dom.exp_avg / bc1, (dom.exp_avg_sq / bc2).sqrt().add_(self.eps), value=-lr)
        pslice.copy_(dom.master)

    # ------------------------------------------------------------------ state
    def state_dict(self) -> Dict[str, object]:
        """This rank's shard: master weights and moments per domain, plus the layout needed to reshard."""
        out = {"step": self.step_count, "lr": self.lr, "domains": {}}
        for dom in self.domains:
            out["domains"][dom.name] = {
                "master": dom.master.cpu(), "exp_avg": dom.exp_avg.cpu(), "exp_avg_sq": dom.exp_avg_sq.cpu(),
                "offsets": dict(dom.offsets), "numel": dom.numel, "shard_rank": dom.shard_rank, "shard_size": dom.shard_size,
            }
        return out

    def load_state_dict(self, sd: Dict[str, object]) -> None:
        self.step_count = int(sd["step"])
        self.lr = float(sd.get("lr", self.lr))
        for dom in self.domains:
            s = sd["domains"][dom.name]
            assert s["shard_size"] == dom.shard_size and s["numel"] == dom.numel, \
                "optimizer shard layout differs: use checkpoint.reshard_optimizer_state() first"
            dom.master.copy_(s["master"])
            dom.exp_avg.copy_(s["exp_avg"])
            dom.exp_avg_sq.copy_(s["exp_avg_sq"])
            dom.shard_slice(dom.flat_param).copy_(dom.master)
            if dom.shard_group is not None:
                dist.all_gather_into_tensor(dom.flat_param, dom.shard_slice(dom.flat_param).clone(), group=dom.shard_group)

    # ------------------------------------------------------------------ parallelism-independent state
    def gather_full_state(self, kind: str) -> Dict[int, torch.Tensor]:
        """``kind`` in {master, exp_avg, exp_avg_sq}: for every parameter, an fp32 tensor of the parameter's (local) shape
        holding that state, assembled from the sharding group's slices (collective over each domain's sharding group).
        Keys are ``id(param)``. Together with the tensor-parallel gathers of the model writer this yields optimizer state
        that does not depend on the parallel layout."""
        out: Dict[int, torch.Tensor] = {}
        for dom in self.domains:
            local = getattr(dom, kind)
            if dom.shard_group is not None:
                full = torch.empty(dom.numel, dtype=local.dtype, device=local.device)
                dist.all_gather_into_tensor(full, local.contiguous(), group=dom.shard_group)
            else:
                full = local
            for name, p in dom.params:
                off, n = dom.offsets[name]
                out[id(p)] = full[off:off + n].view(p.shape)
        return out

    def full_state_buffers(self) -> Dict[str, Dict[int, torch.Tensor]]:
        """Writable fp32 staging tensors (one per parameter and state kind) plus a commit step: see ``commit_full_state``."""
        self._staging = {}
        views: Dict[str, Dict[int, torch.Tensor]] = {}
        for kind in ("master", "exp_avg", "exp_avg_sq"):
            views[kind] = {}
            for dom in self.domains:
                full = torch.zeros(dom.numel, dtype=torch.float32, device=dom.master.device)
                self._staging[(kind, dom.name)] = full
                for name, p in dom.params:
                    off, n = dom.offsets[name]
                    views[kind][id(p)] = full[off:off + n].view(p.shape)
        return views

    def commit_full_state(self, step: int, lr: Optional[float] = None) -> None:
        """Cut this rank's slices out of the staging tensors filled through ``full_state_buffers`` and rebuild the working
        weights from the master slices."""
        sd = {"step": step, "lr": self.lr if lr is None else lr, "domains": {}}
        for dom in self.domains:
            sd["domains"][dom.name] = {k: dom.shard_slice(self._staging[(k, dom.name)]) for k in ("master", "exp_avg", "exp_avg_sq")}
            sd["domains"][dom.name].update(shard_size=dom.shard_size, numel=dom.numel)
        self.load_state_dict(sd)
        self._staging = {}

    def memory_bytes(self) -> int:
        tot = 0
        for dom in self.domains:
            tot += dom.flat_param.numel() * dom.flat_param.element_size() + dom.flat_grad.numel() * 4 + dom.master.numel() * 12
        return tot


def newton_schulz_orthogonalize(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Approximate U V^T of G = U S V^T with the quintic Newton-Schulz iteration (coefficients 3.4445, -4.7750, 2.0315) on
    the Frobenius-normalised matrix, in bf16 on GPUs: singular values end up in roughly [0.7, 1.2], which is all the
    Muon update needs."""
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.to(torch.bfloat16 if G.is_cuda else torch.float32)
    transposed = X.shape[-2] > X.shape[-1]
    if transposed:
        X = X.transpose(-2, -1)
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        A = X @ X.transpose(-2, -1)
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    if transposed:
        X = X.transpose(-2, -1)
    return X.to(torch.float32)


class ShardedMuon(ShardedAdamW):
    """Muon for the hidden weight matrices, AdamW for everything else (embeddings, head, norms, biases, routers), over
    the same flat buffers and with the same gradient reduction and clipping. A matrix's update is its Nesterov momentum,
    orthogonalised by Newton-Schulz and scaled by 0.2 * sqrt(max(rows, cols)) so that one learning rate and one weight
    decay serve both rules. Stacked expert weights [E, N, K] are treated as E matrices. The reference exposes the same
    choice through Paddle's optimizer (paddleformers/trainer/trainer.py:3897).

    The orthogonalisation needs whole matrices: Muon domains must not be split over a sharding group (each rank then
    repeats the same update on its replica), which the constructor enforces."""

    def __init__(self, *args, momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5, **kw):
        self.momentum, self.nesterov, self.ns_steps = momentum, nesterov, ns_steps
        super().__init__(*args, **kw)
        for dom in self.domains:
            if dom.is_muon and dom.shard_size > 1:
                raise ValueError("ShardedMuon: hidden matrices cannot be sharded over the optimizer-sharding group; use "
                                 "sharding degree 1 (data parallel replicas repeat the update) or AdamW")

    def _is_muon_param(self, name: str, p) -> bool:
        if p.dim() < 2 or "embed" in name or "lm_head" in name or name.endswith("gate.weight"):
            return False
        return True

    def _muon_update(self, dom, g, pslice, sc):
        lr, gmul, skip = sc[0], sc[1], sc[4]
        dom.exp_avg.mul_(self.momentum).add_(g * gmul)                    # momentum buffer lives where Adam's first moment does
        upd = torch.zeros_like(dom.master)
        for name, p in dom.params:
            off, n = dom.offsets[name]
            m = dom.exp_avg[off:off + n].view(p.shape)
            gr = (g[off:off + n].view(p.shape) * gmul)
            d = gr + self.momentum * m if self.nesterov else m
            mats = d.reshape(-1, d.shape[-2], d.shape[-1])
            o = newton_schulz_orthogonalize(mats, self.ns_steps)
            scale = 0.2 * math.sqrt(max(d.shape[-2], d.shape[-1]))
            upd[off:off + n] = (o * scale).reshape(-1)
        keep = 1.0 - skip                                                  # non-finite gradients: leave the weights alone
        dom.master.mul_(1.0 - lr * dom.weight_decay * keep).add_(upd * (-(lr * keep)))
        pslice.copy_(dom.master)
