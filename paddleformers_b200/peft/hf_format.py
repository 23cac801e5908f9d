"""Hugging Face PEFT adapter files <-> this framework's LoRA layers (single process / tensor-parallel degree 1).

PEFT stores one (A, B) pair per original projection (``...self_attn.q_proj.lora_A.weight``), this framework keeps the
projections fused (``qkv_proj``, ``gate_up_proj``) with one pair per fused layer:

* export: a fused pair (A [r, in], B [sum(sections), r]) is exactly a set of per-projection pairs that share A and take
  their rows of B, so ``adapter_model.safetensors`` + ``adapter_config.json`` written here load in PEFT unchanged;
* import: per-projection pairs with different A matrices become one fused pair of rank ``sum(r_i)``: A stacked, B block
  diagonal. The fused LoRA layers must therefore be created with that rank (``import_peft_adapter`` does it).

Only plain ``LoRALinear`` modules are covered; expert adapters have no PEFT counterpart.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Tuple

import torch

from .lora import LoRAConfig, LoRALinear, LoRAModel

ADAPTER_WEIGHTS = "adapter_model.safetensors"
ADAPTER_CONFIG = "adapter_config.json"
_PREFIX = "base_model.model."


def _splits(name: str, mod: LoRALinear, config) -> List[Tuple[str, int]]:
    """Original projection names and row counts of a (possibly fused) layer."""
    leaf = name.rsplit(".", 1)[-1]
    out = mod.lora_B.shape[0]
    parent = name.rsplit(".", 1)[0]
    if leaf == "qkv_proj" and not getattr(config, "hf_fused_qkv", False):
        q = config.num_attention_heads * config.head_dim
        kv = config.num_key_value_heads * config.head_dim
        return [(parent + ".q_proj", q), (parent + ".k_proj", kv), (parent + ".v_proj", kv)]
    if leaf == "gate_up_proj" and not getattr(config, "hf_fused_gate_up", False):
        return [(parent + ".gate_proj", out // 2), (parent + ".up_proj", out // 2)]
    return [(name, out)]


def export_peft_adapter(model: LoRAModel, out_dir: str) -> str:
    from safetensors.torch import save_file

    cfg, base_cfg = model.lora_config, model.config
    tensors: Dict[str, torch.Tensor] = {}
    targets = set()
    for name, mod in model.model.named_modules():
        if not isinstance(mod, LoRALinear):
            continue
        row = 0
        for proj, n in _splits(name, mod, base_cfg):
            tensors[f"{_PREFIX}{proj}.lora_A.weight"] = mod.lora_A.detach().cpu().clone()        # one copy per projection on disk
            tensors[f"{_PREFIX}{proj}.lora_B.weight"] = mod.lora_B.detach()[row:row + n].cpu().clone()
            targets.add(proj.rsplit(".", 1)[-1])
            row += n
    os.makedirs(out_dir, exist_ok=True)
    save_file(tensors, os.path.join(out_dir, ADAPTER_WEIGHTS), metadata={"format": "pt"})
    with open(os.path.join(out_dir, ADAPTER_CONFIG), "w") as f:
        json.dump({"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": cfg.r, "lora_alpha": cfg.lora_alpha,
                   "lora_dropout": cfg.lora_dropout, "use_rslora": cfg.rslora, "bias": "none", "fan_in_fan_out": False,
                   "target_modules": sorted(targets), "base_model_name_or_path": cfg.base_model_name_or_path,
                   "inference_mode": True}, f, indent=2)
    return out_dir


def import_peft_adapter(base_model: torch.nn.Module, adapter_dir: str) -> LoRAModel:
    """Wrap ``base_model`` with LoRA layers holding the adapters of a PEFT directory."""
    from safetensors.torch import load_file

    with open(os.path.join(adapter_dir, ADAPTER_CONFIG)) as f:
        ac = json.load(f)
    sd = load_file(os.path.join(adapter_dir, ADAPTER_WEIGHTS))
    sd = {k[len(_PREFIX):] if k.startswith(_PREFIX) else k: v for k, v in sd.items()}
    sd = {k.replace(".lora_A.default.", ".lora_A.").replace(".lora_B.default.", ".lora_B."): v for k, v in sd.items()}
    r, alpha, rs = int(ac["r"]), float(ac["lora_alpha"]), bool(ac.get("use_rslora", False))
    config = base_model.config
    # which fused layers receive adapters, and from how many original projections
    probe = LoRAModel(base_model, LoRAConfig(r=1, lora_alpha=1.0))      # wraps every default target; rebuilt below
    plans = {}
    for name, mod in probe.model.named_modules():
        if isinstance(mod, LoRALinear):
            parts = [(p, n) for p, n in _splits(name, mod, config) if f"{p}.lora_A.weight" in sd]
            if parts:
                plans[name] = (parts, _splits(name, mod, config))
    fused_rank = max(len(parts) for parts, _ in plans.values()) * r if plans else r
    # undo the probe wrapping, then wrap only the planned layers with the fused rank
    for name, mod in list(probe.model.named_modules()):
        if isinstance(mod, LoRALinear):
            parent_name, _, leaf = name.rpartition(".")
            parent = probe.model.get_submodule(parent_name) if parent_name else probe.model
            setattr(parent, leaf, mod.base)
    # scaling is alpha / r of the source adapters: keep it by scaling alpha with the rank inflation
    scale_alpha = alpha * (fused_rank / r) if not rs else alpha * (fused_rank / r) ** 0.5
    cfg = LoRAConfig(r=fused_rank, lora_alpha=scale_alpha, rslora=rs, lora_dropout=float(ac.get("lora_dropout", 0.0)),
                     target_modules=[name.replace(".", "[.]") + "$" for name in plans],
                     base_model_name_or_path=ac.get("base_model_name_or_path"))
    wrapped = LoRAModel(base_model, cfg)
    with torch.no_grad():
        for name, (parts, all_parts) in plans.items():
            mod = wrapped.model.get_submodule(name)
            mod.lora_A.zero_()
            mod.lora_B.zero_()
            row_of = {}
            row = 0
            for p, n in all_parts:
                row_of[p] = (row, n)
                row += n
            for i, (p, n) in enumerate(parts):
                a, b = sd[f"{p}.lora_A.weight"], sd[f"{p}.lora_B.weight"]
                mod.lora_A[i * r:(i + 1) * r].copy_(a)
                lo, cnt = row_of[p]
                mod.lora_B[lo:lo + cnt, i * r:(i + 1) * r].copy_(b)
    return wrapped
