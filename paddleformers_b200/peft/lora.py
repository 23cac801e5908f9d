"""LoRA adapters: plain, rank-stabilised (rsLoRA), LoRA+ learning-rate groups, tensor-parallel aware and for stacked
MoE experts; merge / unmerge and adapter-only checkpoints.

Counterparts: paddleformers/peft/lora/lora_config.py:26 (``LoRAConfig``), lora_model.py:233 (``LoRAModel``),
lora_layers.py:64 (``LoRALinear``), :464 / :331 (column- / row-parallel variants), :860 (``LoRAMoeExperts``).
The low-rank path runs through the same tcgen05 GEMM wrappers as the base layers.
"""
from __future__ import annotations

import contextlib
import json
import math
import os
import re
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import functional as F
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, mark_as_sequence_parallel_parameter

LORA_CONFIG_NAME = "lora_config.json"
LORA_WEIGHTS_NAME = "lora_model.safetensors"


@dataclass
class LoRAConfig:
    r: int = 8
    lora_alpha: float = 16.0
    lora_dropout: float = 0.0
    target_modules: List[str] = field(default_factory=lambda: [".*qkv_proj", ".*o_proj", ".*gate_up_proj", ".*down_proj"])
    rslora: bool = False
    lora_plus_scale: float = 1.0        # learning-rate multiplier of the B matrices (LoRA+)
    trainable_modules: Optional[List[str]] = None   # extra fully-trainable modules (regex)
    merge_weights: bool = False
    base_model_name_or_path: Optional[str] = None

    @property
    def scaling(self) -> float:
        return self.lora_alpha / math.sqrt(self.r) if self.rslora else self.lora_alpha / self.r

    def save_pretrained(self, d: str):
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, LORA_CONFIG_NAME), "w") as f:
            json.dump(asdict(self), f, indent=2)

    @classmethod
    def from_pretrained(cls, d: str) -> "LoRAConfig":
        with open(os.path.join(d, LORA_CONFIG_NAME)) as f:
            return cls(**json.load(f))


class LoRALinear(nn.Module):
    """y = base(x) + scaling * (dropout(x) A^T) B^T. For tensor-parallel bases, A or B is sharded so that the
    low-rank path needs no extra collective: column-parallel -> B split on its output rows; row-parallel -> A split
    on its input columns and the partial result joins the base layer's reduction."""

    def __init__(self, base: nn.Module, cfg: LoRAConfig):
        super().__init__()
        self.base = base
        self.cfg = cfg
        w = base.weight
        out_f, in_f = w.shape
        self.scaling = cfg.scaling
        self.lora_A = nn.Parameter(torch.empty(cfg.r, in_f, dtype=w.dtype, device=w.device))
        self.lora_B = nn.Parameter(torch.zeros(out_f, cfg.r, dtype=w.dtype, device=w.device))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.lora_B.lora_plus = True
        # The factor that stays whole on every tensor-parallel rank meets only this rank's slice of the other factor, so its
        # gradient is a partial sum: it is added up over the group before the optimizer step, like the norm weights under
        # sequence parallelism.
        if isinstance(base, ColumnParallelLinear):
            self.lora_B.shard_spec = ("tp", 0, base.sections)
            if base.tp > 1:
                mark_as_sequence_parallel_parameter(self.lora_A)
        elif isinstance(base, RowParallelLinear):
            self.lora_A.shard_spec = ("tp", 1, None)
            if base.tp > 1:
                mark_as_sequence_parallel_parameter(self.lora_B)
        self.dropout = nn.Dropout(cfg.lora_dropout) if cfg.lora_dropout > 0 else None
        self.merged = False
        self.disabled = False
        base.weight.requires_grad_(False)
        if getattr(base, "bias", None) is not None:
            base.bias.requires_grad_(False)

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return getattr(self.base, "bias", None)

    def delta(self) -> torch.Tensor:
        return (self.lora_B.float() @ self.lora_A.float()) * self.scaling

    def merge(self):
        if not self.merged:
            self.base.weight.data += self.delta().to(self.base.weight.dtype)
            self.merged = True

    def unmerge(self):
        if self.merged:
            self.base.weight.data -= self.delta().to(self.base.weight.dtype)
            self.merged = False

    def forward(self, x):
        epilogue = getattr(self.base, "epilogue", None)
        if self.merged or self.disabled:
            return self.base(x) if not isinstance(self.base, nn.Linear) else F.linear(x, self.base.weight, self.base.bias)
        xin = self.dropout(x) if self.dropout is not None else x
        if isinstance(self.base, RowParallelLinear):
            # add the low-rank partial before the base layer's reduce-scatter / all-reduce
            y = F.linear(x, self.base.weight) + F.linear(F.linear(xin, self.lora_A), self.lora_B) * self.scaling
            from ..parallel.tensor_parallel import ReduceFromTP, ReduceScatterOp

            if self.base.tp > 1:
                y = ReduceScatterOp.apply(y, self.base.group) if self.base.sequence_parallel else ReduceFromTP.apply(y, self.base.group)
            return y + self.base.bias if self.base.bias is not None else y
        if isinstance(self.base, ColumnParallelLinear):
            from ..parallel.tensor_parallel import AllGatherOp, CopyToTP

            if self.base.tp > 1:
                x = AllGatherOp.apply(x, self.base.group) if self.base.sequence_parallel else CopyToTP.apply(x, self.base.group)
                xin = self.dropout(x) if self.dropout is not None else x
            y = F.linear(x, self.base.weight, self.base.bias) + F.linear(F.linear(xin, self.lora_A), self.lora_B) * self.scaling
            return F.swiglu(y) if epilogue == "swiglu" else y
        return F.linear(x, self.base.weight, self.base.bias) + F.linear(F.linear(xin, self.lora_A), self.lora_B) * self.scaling


class LoRAMoeExperts(nn.Module):
    """Per-expert low-rank updates of the stacked expert weights; applied by materialising W + scaling * B A for the
    grouped GEMM (expert matrices are small, the rank update is cheap next to the token GEMMs)."""

    def __init__(self, experts: nn.Module, cfg: LoRAConfig):
        super().__init__()
        self.experts, self.cfg, self.scaling = experts, cfg, cfg.scaling
        E, N2, H = experts.gate_up_proj.shape
        I = experts.down_proj.shape[2]
        dt, dev = experts.gate_up_proj.dtype, experts.gate_up_proj.device
        self.gu_A = nn.Parameter(torch.empty(E, cfg.r, H, dtype=dt, device=dev))
        self.gu_B = nn.Parameter(torch.zeros(E, N2, cfg.r, dtype=dt, device=dev))
        self.dn_A = nn.Parameter(torch.empty(E, cfg.r, I, dtype=dt, device=dev))
        self.dn_B = nn.Parameter(torch.zeros(E, H, cfg.r, dtype=dt, device=dev))
        for a in (self.gu_A, self.dn_A):
            nn.init.kaiming_uniform_(a.view(-1, a.shape[-1]), a=math.sqrt(5))
        for p in (self.gu_A, self.gu_B, self.dn_A, self.dn_B):
            p.is_expert = True
            p.shard_spec = ("ep", 0, None)
            if getattr(experts.gate_up_proj, "sequence_parallel", False):     # token slices per tensor-parallel rank: partial sums
                mark_as_sequence_parallel_parameter(p)
        experts.gate_up_proj.requires_grad_(False)
        experts.down_proj.requires_grad_(False)
        self.num_local, self.expert_offset = experts.num_local, experts.expert_offset
        self.disabled = False

    def forward(self, rows, block_expert, counts=None):
        if self.disabled:
            return self.experts(rows, block_expert, counts)
        gu = self.experts.gate_up_proj + (torch.bmm(self.gu_B.float(), self.gu_A.float()) * self.scaling).to(rows.dtype)
        dn = self.experts.down_proj + (torch.bmm(self.dn_B.float(), self.dn_A.float()) * self.scaling).to(rows.dtype)
        from ..nn.moe import _GroupedMlpFn

        if rows.is_cuda and rows.dtype == torch.bfloat16:
            return _GroupedMlpFn.apply(rows, gu, dn, block_expert)
        out = torch.zeros_like(rows)
        for b, e in enumerate(block_expert.tolist()):
            if e < 0:
                continue
            seg = rows[b * 128:(b + 1) * 128]
            g, u = torch.nn.functional.linear(seg, gu[e]).chunk(2, -1)
            out[b * 128:(b + 1) * 128] = torch.nn.functional.linear(torch.nn.functional.silu(g) * u, dn[e])
        return out


class LoRAModel(nn.Module):
    """Wraps a model: replaces matching linear layers by ``LoRALinear`` (and expert stacks by ``LoRAMoeExperts`` when
    ``".*experts"`` is targeted), freezes everything else."""

    def __init__(self, model: nn.Module, cfg: LoRAConfig):
        super().__init__()
        self.model, self.lora_config = model, cfg
        for p in model.parameters():
            p.requires_grad_(False)
        pats = [re.compile(p) for p in cfg.target_modules]
        from ..nn.moe import GroupedExperts
        from ..quantization.weight_only import QuantizationLinear

        for name, mod in list(model.named_modules()):
            if not any(p.fullmatch(name) or p.search(name) for p in pats):
                continue
            parent_name, _, leaf = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            if isinstance(mod, (nn.Linear, ColumnParallelLinear, RowParallelLinear, QuantizationLinear)):
                # a QuantizationLinear base (int8 / int4 / nf4) gives QLoRA: frozen quantised weights, bf16 adapters
                setattr(parent, leaf, LoRALinear(mod, cfg))
            elif isinstance(mod, GroupedExperts):
                setattr(parent, leaf, LoRAMoeExperts(mod, cfg))
        for pat in cfg.trainable_modules or []:
            rx = re.compile(pat)
            for n, p in model.named_parameters():
                if rx.search(n):
                    p.requires_grad_(True)
        self.config = getattr(model, "config", None)

    def forward(self, *a, **k):
        return self.model(*a, **k)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.model, name)

    @property
    def loss_accumulation_steps(self):
        return getattr(self.model, "loss_accumulation_steps", 1)

    @loss_accumulation_steps.setter
    def loss_accumulation_steps(self, n):
        # the trainer sets this on the model it was given: the wrapped model is the one that divides its loss by it
        self.model.loss_accumulation_steps = n

    def lora_modules(self):
        return [m for m in self.model.modules() if isinstance(m, (LoRALinear, LoRAMoeExperts))]

    @contextlib.contextmanager
    def disable_adapters(self):
        mods = self.lora_modules()
        for m in mods:
            m.disabled = True
        try:
            yield
        finally:
            for m in mods:
                m.disabled = False

    def merge(self):
        for m in self.lora_modules():
            if isinstance(m, LoRALinear):
                m.merge()

    def unmerge(self):
        for m in self.lora_modules():
            if isinstance(m, LoRALinear):
                m.unmerge()

    def print_trainable_parameters(self) -> str:
        t = sum(p.numel() for p in self.parameters() if p.requires_grad)
        a = sum(p.numel() for p in self.parameters())
        return f"trainable params: {t:,} || all params: {a:,} || trainable%: {100 * t / max(a, 1):.4f}"

    def lora_state_dict(self) -> Dict[str, torch.Tensor]:
        return {k: v.detach().cpu() for k, v in self.model.state_dict().items() if "lora_" in k or ".gu_" in k or ".dn_" in k}

    def save_pretrained(self, d: str):
        from safetensors.torch import save_file

        os.makedirs(d, exist_ok=True)
        sd = self.lora_state_dict()
        cfg = self.lora_config
        init = getattr(self, "loraga_init_dict", None)
        if init:
            # LoRA-GA shifted the frozen weights by -scaling * B0 A0 at initialisation. Saved adapters must apply to the
            # ORIGINAL base weights, so the saved pair is the rank-2r factorisation of B A - B0 A0:
            # [B | B0] @ [A ; -A0], with alpha doubled so that the scaling alpha / r stays what it was.
            import copy

            for name, t0 in init.items():
                # names recorded on the wrapper carry its own attribute prefix
                key = next((k for k in sd if name == k or name.endswith("." + k) or k.endswith("." + name)), None)
                if key is None:
                    continue
                t0 = t0.detach().cpu().to(sd[key].dtype)
                sd[key] = torch.cat([sd[key], -t0], dim=0) if name.endswith("lora_A") else torch.cat([sd[key], t0], dim=1)
            cfg = copy.copy(cfg)
            cfg.lora_alpha = cfg.lora_alpha * (math.sqrt(2.0) if cfg.rslora else 2.0)
            cfg.r = cfg.r * 2
        cfg.save_pretrained(d)
        save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(d, LORA_WEIGHTS_NAME))

    @classmethod
    def from_pretrained(cls, model: nn.Module, d: str) -> "LoRAModel":
        from safetensors.torch import load_file

        cfg = LoRAConfig.from_pretrained(d)
        wrapped = cls(model, cfg)
        sd = load_file(os.path.join(d, LORA_WEIGHTS_NAME))
        missing, unexpected = wrapped.model.load_state_dict(sd, strict=False)
        if unexpected:
            raise KeyError(f"unexpected LoRA tensors: {unexpected[:5]}")
        return wrapped

    def merged_model(self) -> nn.Module:
        """Returns the base model with adapters folded into the weights and the wrappers removed (export path)."""
        self.merge()
        for name, mod in list(self.model.named_modules()):
            if isinstance(mod, LoRALinear):
                parent_name, _, leaf = name.rpartition(".")
                parent = self.model.get_submodule(parent_name) if parent_name else self.model
                setattr(parent, leaf, mod.base)
        return self.model


def lora_plus_param_groups(model: nn.Module, lr: float, cfg: LoRAConfig):
    """LoRA+: B matrices train with ``lr * lora_plus_scale``."""
    a = [p for p in model.parameters() if p.requires_grad and not getattr(p, "lora_plus", False)]
    b = [p for p in model.parameters() if p.requires_grad and getattr(p, "lora_plus", False)]
    return [{"params": a, "lr": lr}, {"params": b, "lr": lr * cfg.lora_plus_scale}]
