"""Per-group NCCL communicator options.

A JSON file (``TrainingArguments.nccl_comm_group_config``) maps group names of the hybrid topology (``mp``, ``pp``,
``sharding``, ``dp``, ``ep``, ``moe_sharding``, ``cp``, ``sep``, or ``default``) to communicator settings, so that for
example the latency-critical tensor-parallel group gets a high-priority stream and few CTAs while the bandwidth-bound
sharding group may use many - what the reference's ``init_nccl_config`` does for Fleet's groups
(paddleformers/trainer/trainer_utils.py:1636-1722).

    {"mp": {"high_priority": true, "max_ctas": 16}, "sharding": {"min_ctas": 16, "max_ctas": 32},
     "default": {"cga_cluster_size": 2}}

Unknown keys are rejected. On CPU (gloo) ranks the options are parsed and ignored.
"""
from __future__ import annotations

import json
from typing import Dict, Optional

_INT_KEYS = ("max_ctas", "min_ctas", "cga_cluster_size", "nvls_ctas", "traffic_class")
_STR_KEYS = ("net_name",)
_BOOL_KEYS = ("high_priority", "blocking", "split_share", "collnet_enable")
_GROUPS = ("default", "dp", "sharding", "pp", "sep", "cp", "mp", "ep", "moe_sharding", "data", "model")


def load_nccl_config(src) -> Dict[str, Dict[str, object]]:
    """``src``: a path to a JSON file, a JSON string, a dict, or None."""
    if not src:
        return {}
    if isinstance(src, str):
        cfg = json.loads(src) if src.lstrip().startswith("{") else json.load(open(src))
    else:
        cfg = dict(src)
    for g, opts in cfg.items():
        if g not in _GROUPS:
            raise ValueError(f"nccl config: unknown group {g!r}; expected one of {_GROUPS}")
        for k, v in opts.items():
            if k not in _INT_KEYS + _STR_KEYS + _BOOL_KEYS:
                raise ValueError(f"nccl config: unknown option {k!r} for group {g!r}")
            if k in _INT_KEYS and not isinstance(v, int):
                raise ValueError(f"nccl config: {g}.{k} must be an integer")
    return cfg


def group_options(cfg: Dict[str, Dict[str, object]], group: str) -> Dict[str, object]:
    out = dict(cfg.get("default", {}))
    out.update(cfg.get(group, {}))
    return out


def make_pg_options(cfg: Dict[str, Dict[str, object]], group: str, backend: Optional[str]):
    """``ProcessGroupNCCL.Options`` for ``dist.new_group(..., pg_options=...)``, or None when nothing is configured for the
    group or the backend is not NCCL."""
    opts = group_options(cfg, group)
    if not opts or (backend or "nccl") != "nccl":
        return None
    import torch.distributed as dist

    if not hasattr(dist, "ProcessGroupNCCL"):
        return None
    o = dist.ProcessGroupNCCL.Options(is_high_priority_stream=bool(opts.get("high_priority", False)))
    for k in _INT_KEYS + _STR_KEYS:
        if k in opts:
            setattr(o.config, k, opts[k])
    for k in ("blocking", "split_share", "collnet_enable"):
        if k in opts:
            setattr(o.config, k, int(bool(opts[k])) if k != "split_share" else bool(opts[k]))
    return o
