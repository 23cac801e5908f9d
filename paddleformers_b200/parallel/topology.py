"""Hybrid-parallel topology and process groups on ``torch.distributed``.

A job of ``world_size`` ranks is laid out on a grid of named axes. The dense view uses the reference's axis orders
(paddleformers/trainer/training_args.py:2207-2235): ``sharding_first`` = [dp, sharding, pp, sep, cp, mp] or
``pp_first`` = [dp, pp, sharding, sep, cp, mp] (last axis varies fastest, so tensor-parallel ranks are neighbours on
NVLink). Expert parameters see the ranks of one pipeline stage through a second view [moe_sharding, ep] with
``moe_sharding = world / (pp * ep)`` (paddleformers/trainer/training_args.py:2885-2905): expert parallel ranks are
contiguous, and the tensor/sharding/data axes fold into ep x moe_sharding.

``ParallelState`` owns one process group per axis (plus the fused data-parallel group used for data sharding and
loss averaging). With world size 1 everything degenerates to single-rank groups and no backend is initialised.
"""
from __future__ import annotations

import itertools
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


class Topology:
    """Named N-d grid of ranks; the last axis varies fastest (mirror of paddleformers/trainer/trainer_utils.py:158-218)."""

    def __init__(self, names: Sequence[str], dims: Sequence[int]):
        assert len(names) == len(dims)
        self.names = list(names)
        self.dims = list(dims)
        self.world_size = 1
        for d in dims:
            self.world_size *= d

    def coord(self, rank: int) -> Dict[str, int]:
        out = {}
        for n, d in zip(reversed(self.names), reversed(self.dims)):
            out[n] = rank % d
            rank //= d
        return out

    def rank(self, **coord) -> int:
        r = 0
        for n, d in zip(self.names, self.dims):
            r = r * d + coord[n]
        return r

    def get_dim(self, name: str) -> int:
        return self.dims[self.names.index(name)]

    def comm_list(self, axis: str) -> List[List[int]]:
        """All groups along ``axis``: ranks that share every other coordinate."""
        others = [n for n in self.names if n != axis]
        ranges = [range(self.get_dim(n)) for n in others]
        out = []
        for combo in itertools.product(*ranges):
            base = dict(zip(others, combo))
            out.append([self.rank(**dict(base, **{axis: i})) for i in range(self.get_dim(axis))])
        return out

    def fused_comm_list(self, axes: Sequence[str]) -> List[List[int]]:
        """Groups spanning several axes at once (e.g. dp x sharding for data sharding)."""
        others = [n for n in self.names if n not in axes]
        out = []
        for combo in itertools.product(*[range(self.get_dim(n)) for n in others]):
            base = dict(zip(others, combo))
            grp = []
            for inner in itertools.product(*[range(self.get_dim(a)) for a in axes]):
                grp.append(self.rank(**dict(base, **dict(zip(axes, inner)))))
            out.append(sorted(grp))
        return out


@dataclass
class ParallelDegrees:
    dp: int = 1
    sharding: int = 1
    pp: int = 1
    sep: int = 1
    cp: int = 1
    mp: int = 1
    ep: int = 1
    order: str = "sharding_first"

    @property
    def world(self) -> int:
        return self.dp * self.sharding * self.pp * self.sep * self.cp * self.mp

    @property
    def moe_sharding(self) -> int:
        return max(1, self.world // (self.pp * self.ep))

    def axis_order(self) -> List[str]:
        if self.order == "pp_first":
            return ["dp", "pp", "sharding", "sep", "cp", "mp"]
        return ["dp", "sharding", "pp", "sep", "cp", "mp"]


class _SingleGroup:
    """Stand-in for a process group of one rank (no backend needed)."""

    def size(self):
        return 1

    def rank(self):
        return 0


class ParallelState:
    AXES = ("dp", "sharding", "pp", "sep", "cp", "mp")

    def __init__(self, degrees: Optional[ParallelDegrees] = None, rank: Optional[int] = None, backend: Optional[str] = None,
                 create_groups: bool = True, nccl_config=None):
        from .nccl_config import load_nccl_config

        self.nccl_config = load_nccl_config(nccl_config)
        self.degrees = degrees or ParallelDegrees()
        d = self.degrees
        self.world_size = d.world
        self.global_rank = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
        self.topo = Topology(d.axis_order(), [getattr(d, a) for a in d.axis_order()])
        self.coord = self.topo.coord(self.global_rank)
        assert d.world % (d.pp * d.ep) == 0, f"ep={d.ep} must divide world/pp={d.world // d.pp}"
        self.groups: Dict[str, object] = {}
        self.group_ranks: Dict[str, List[int]] = {}
        self._build(create_groups and dist.is_initialized() and self.world_size > 1, backend)

    # ------------------------------------------------------------------ construction
    def _expert_view(self) -> Dict[str, List[List[int]]]:
        """ep / moe_sharding groups inside every pipeline stage."""
        d = self.degrees
        ep_groups, ms_groups = [], []
        for stage in range(d.pp):
            # ranks of this stage, ordered so that tensor-parallel neighbours stay adjacent
            stage_ranks = sorted(r for r in range(self.world_size) if self.topo.coord(r)["pp"] == stage)
            n = len(stage_ranks)
            ms = n // d.ep
            for i in range(ms):
                ep_groups.append(stage_ranks[i * d.ep:(i + 1) * d.ep])
            for j in range(d.ep):
                ms_groups.append(stage_ranks[j::d.ep])
        return {"ep": ep_groups, "moe_sharding": ms_groups}

    def _build(self, make: bool, backend: Optional[str]):
        lists = {a: self.topo.comm_list(a) for a in self.AXES}
        lists["data"] = self.topo.fused_comm_list(["dp", "sharding"])        # ranks that read different data
        lists["dp_sharding_cp"] = self.topo.fused_comm_list(["dp", "sharding", "sep", "cp"])  # dense grad averaging
        lists["model"] = self.topo.fused_comm_list(["pp", "sep", "cp", "mp"])  # ranks that hold one model replica
        lists["dp_sep_cp"] = self.topo.fused_comm_list(["dp", "sep", "cp"])   # replicas of one sharding rank
        lists.update(self._expert_view())
        for name, groups in lists.items():
            mine = None
            for ranks in groups:
                g = None
                if make and len(ranks) > 1:
                    from .nccl_config import make_pg_options

                    eff = backend or ("nccl" if torch.cuda.is_available() else "gloo")
                    opts = make_pg_options(self.nccl_config, name, eff)
                    g = dist.new_group(ranks=ranks, backend=backend, pg_options=opts) if opts is not None else \
                        dist.new_group(ranks=ranks, backend=backend)
                if self.global_rank in ranks:
                    mine = ranks
                    self.groups[name] = g if g is not None else _SingleGroup()
            self.group_ranks[name] = mine or [self.global_rank]
            if name not in self.groups:
                self.groups[name] = _SingleGroup()

    # ------------------------------------------------------------------ accessors
    def group(self, name: str):
        return self.groups[name]

    def size(self, name: str) -> int:
        return len(self.group_ranks[name])

    def rank_in(self, name: str) -> int:
        return self.group_ranks[name].index(self.global_rank)

    # reference-style names
    def get_model_parallel_world_size(self): return self.degrees.mp
    def get_model_parallel_rank(self): return self.coord["mp"]
    def get_model_parallel_group(self): return self.groups["mp"]
    def get_pipe_parallel_world_size(self): return self.degrees.pp
    def get_stage_id(self): return self.coord["pp"]
    def get_pipe_parallel_group(self): return self.groups["pp"]
    def get_sharding_parallel_world_size(self): return self.degrees.sharding
    def get_sharding_parallel_rank(self): return self.coord["sharding"]
    def get_sharding_parallel_group(self): return self.groups["sharding"]
    def get_data_parallel_world_size(self): return self.degrees.dp
    def get_data_parallel_rank(self): return self.coord["dp"]
    def get_data_parallel_group(self): return self.groups["dp"]
    def get_expert_parallel_world_size(self): return self.degrees.ep
    def get_expert_parallel_rank(self): return self.rank_in("ep")
    def get_expert_parallel_group(self): return self.groups["ep"]
    def get_moe_sharding_parallel_world_size(self): return self.degrees.moe_sharding
    def get_moe_sharding_parallel_group(self): return self.groups["moe_sharding"]
    def get_context_parallel_world_size(self): return self.degrees.cp
    def get_context_parallel_rank(self): return self.coord["cp"]
    def get_context_parallel_group(self): return self.groups["cp"]
    def get_sep_parallel_world_size(self): return self.degrees.sep
    def get_sep_parallel_rank(self): return self.coord["sep"]
    def get_sep_parallel_group(self): return self.groups["sep"]

    @property
    def is_first_stage(self): return self.coord["pp"] == 0

    @property
    def is_last_stage(self): return self.coord["pp"] == self.degrees.pp - 1

    @property
    def dataset_world_size(self) -> int:
        """Number of distinct data shards (paddleformers/trainer/training_args.py:3038-3101)."""
        return self.degrees.dp * self.degrees.sharding

    @property
    def dataset_rank(self) -> int:
        return self.coord["dp"] * self.degrees.sharding + self.coord["sharding"]

    def weight_name_suffix(self) -> Optional[str]:
        """tpXX_ppYY[_shardZZ] suffix of per-rank checkpoint files."""
        d = self.degrees
        parts = []
        if d.mp > 1:
            parts.append(f"tp{self.coord['mp']:02d}")
        if d.pp > 1:
            parts.append(f"pp{self.coord['pp']:02d}")
        if d.ep > 1:
            parts.append(f"ep{self.rank_in('ep'):02d}")
        return "_".join(parts) if parts else None


_STATE: Optional[ParallelState] = None


def get_parallel_state() -> ParallelState:
    global _STATE
    if _STATE is None:
        _STATE = ParallelState(ParallelDegrees(), rank=0, create_groups=False)
    return _STATE


def set_parallel_state(state: Optional[ParallelState]) -> None:
    global _STATE
    _STATE = state


def init_distributed(backend: Optional[str] = None, timeout_s: Optional[int] = None) -> None:
    """Initialise ``torch.distributed`` from the launcher's environment (RANK / WORLD_SIZE / MASTER_*)."""
    if dist.is_initialized() or int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        return
    import datetime

    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    kw = {}
    t = timeout_s or int(os.environ.get("PFB_PG_TIMEOUT", "0"))
    if t:
        kw["timeout"] = datetime.timedelta(seconds=t)
    if backend == "nccl":
        kw["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(backend=backend, **kw)


def initialize_parallel(degrees: ParallelDegrees, backend: Optional[str] = None, nccl_config=None) -> ParallelState:
    init_distributed(backend)
    world = dist.get_world_size() if dist.is_initialized() else 1
    assert degrees.world == world, f"parallel degrees {degrees} need {degrees.world} ranks, job has {world}"
    state = ParallelState(degrees, backend=backend, nccl_config=nccl_config)
    set_parallel_state(state)
    return state
