"""Model merging over safetensors checkpoints: linear, SLERP and TIES, with DARE / magnitude-prune / trim
sparsification of task vectors, and LoRA -> base merging for export.

Counterparts: paddleformers/mergekit/merge_model.py (``MergeModel``), merge_method.py:19 (``MergeMethod``),
paddleformers/cli/export/export.py:83 (LoRA merge export). Tensors are processed one at a time so that host memory
stays bounded by the largest parameter.
"""
from __future__ import annotations

import json
import os
import shutil
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch


@dataclass
class MergeConfig:
    merge_method: str = "linear"            # linear | slerp | ties
    model_path_list: List[str] = field(default_factory=list)
    base_model_path: Optional[str] = None   # required for ties / task-vector sparsification
    weight_list: Optional[List[float]] = None
    sparsify_type: Optional[str] = None     # dare | magprune | trim
    reserve_p: float = 0.7                  # fraction of task-vector entries kept by the sparsifier
    slerp_t: float = 0.5
    output_path: str = "./merged"
    seed: int = 0
    rescale: bool = True
    max_shard_size_gb: float = 5.0          # output files are cut at this size; several files come with an index


def sparsify(delta: torch.Tensor, kind: Optional[str], keep: float, gen: torch.Generator, rescale: bool = True) -> torch.Tensor:
    if kind is None or keep >= 1.0:
        return delta
    if kind == "dare":
        mask = torch.rand(delta.shape, generator=gen) < keep
        out = delta * mask
        return out / keep if rescale else out
    if kind in ("trim", "magprune"):
        k = max(1, int(delta.numel() * keep))
        thresh = delta.abs().flatten().kthvalue(delta.numel() - k + 1)[0]
        mask = delta.abs() >= thresh
        if kind == "magprune" and rescale:
            return delta * mask * (delta.numel() / max(int(mask.sum()), 1)) ** 0.0 + 0 * delta
        return delta * mask
    raise ValueError(f"unknown sparsify type {kind!r}")


def merge_linear(tensors: Sequence[torch.Tensor], weights: Sequence[float]) -> torch.Tensor:
    tot = sum(weights)
    return sum(t.float() * (w / tot) for t, w in zip(tensors, weights))


def merge_slerp(a: torch.Tensor, b: torch.Tensor, t: float, eps: float = 1e-8) -> torch.Tensor:
    af, bf = a.float().flatten(), b.float().flatten()
    an, bn = af / (af.norm() + eps), bf / (bf.norm() + eps)
    dot = torch.clamp((an * bn).sum(), -1.0, 1.0)
    if abs(float(dot)) > 0.9995:
        return ((1 - t) * a.float() + t * b.float())
    theta = torch.acos(dot)
    s = torch.sin(theta)
    out = torch.sin((1 - t) * theta) / s * af + torch.sin(t * theta) / s * bf
    return out.view(a.shape)


def merge_ties(base: torch.Tensor, tensors: Sequence[torch.Tensor], weights: Sequence[float], keep: float,
               kind: Optional[str], gen: torch.Generator, rescale: bool) -> torch.Tensor:
    deltas = [sparsify(t.float() - base.float(), kind or "trim", keep, gen, rescale) * w for t, w in zip(tensors, weights)]
    stacked = torch.stack(deltas)
    sign = torch.sign(stacked.sum(0))
    agree = (torch.sign(stacked) == sign[None]) & (stacked != 0)
    num = (stacked * agree).sum(0)
    den = agree.sum(0).clamp(min=1)
    return base.float() + num / den


class MergeModel:
    def __init__(self, cfg: MergeConfig):
        self.cfg = cfg
        n = len(cfg.model_path_list)
        if n < 2 and cfg.merge_method != "ties":
            raise ValueError("merging needs at least two models")
        if cfg.merge_method == "slerp" and n != 2:
            raise ValueError("slerp merges exactly two models")
        if cfg.merge_method == "ties" and not cfg.base_model_path:
            raise ValueError("ties needs base_model_path")
        self.weights = cfg.weight_list or [1.0] * n

    def merge(self) -> str:
        from ..transformers.model_utils import _CheckpointReader
        from safetensors.torch import save_file

        cfg = self.cfg
        readers = [_CheckpointReader(p) for p in cfg.model_path_list]
        base = _CheckpointReader(cfg.base_model_path) if cfg.base_model_path else None
        gen = torch.Generator().manual_seed(cfg.seed)
        os.makedirs(cfg.output_path, exist_ok=True)
        out: Dict[str, torch.Tensor] = {}
        shards: List[Dict[str, str]] = []          # one {tensor name: file} map per written file
        limit = int(cfg.max_shard_size_gb * (1 << 30))
        held = 0

        def flush():
            nonlocal out, held
            if out:
                fname = f"model-{len(shards) + 1:05d}.safetensors"
                save_file(out, os.path.join(cfg.output_path, fname), metadata={"format": "pt"})
                shards.append({k: fname for k in out})
                out, held = {}, 0

        for name in sorted(readers[0].keys()):
            ts = [r.get(name) for r in readers]
            dtype = ts[0].dtype
            if not ts[0].is_floating_point():
                out[name] = ts[0]
                held += ts[0].numel() * ts[0].element_size()
                continue
            if cfg.merge_method == "linear":
                if cfg.sparsify_type and base is not None:
                    b = base.get(name).float()
                    deltas = [sparsify(t.float() - b, cfg.sparsify_type, cfg.reserve_p, gen, cfg.rescale) for t in ts]
                    m = b + merge_linear(deltas, self.weights)
                else:
                    m = merge_linear(ts, self.weights)
            elif cfg.merge_method == "slerp":
                m = merge_slerp(ts[0], ts[1], cfg.slerp_t)
            elif cfg.merge_method == "ties":
                m = merge_ties(base.get(name), ts, self.weights, cfg.reserve_p, cfg.sparsify_type, gen, cfg.rescale)
            else:
                raise ValueError(cfg.merge_method)
            out[name] = m.to(dtype).contiguous()
            held += out[name].numel() * out[name].element_size()
            if held >= limit:                      # only one output file's worth of merged tensors is alive at a time
                flush()
        flush()
        if len(shards) == 1:
            os.replace(os.path.join(cfg.output_path, "model-00001.safetensors"), os.path.join(cfg.output_path, "model.safetensors"))
        else:
            total = len(shards)
            weight_map = {}
            for i, m in enumerate(shards):
                final = f"model-{i + 1:05d}-of-{total:05d}.safetensors"
                os.replace(os.path.join(cfg.output_path, f"model-{i + 1:05d}.safetensors"), os.path.join(cfg.output_path, final))
                weight_map.update({k: final for k in m})
            import json

            with open(os.path.join(cfg.output_path, "model.safetensors.index.json"), "w") as f:
                json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=2, sort_keys=True)
        for fn in os.listdir(cfg.model_path_list[0]):
            if fn.endswith(".json") and "index" not in fn or fn.startswith("tokenizer") or fn.endswith(".model"):
                shutil.copy(os.path.join(cfg.model_path_list[0], fn), os.path.join(cfg.output_path, fn))
        return cfg.output_path


def merge_lora_and_export(base_model_dir: str, lora_dir: str, output_dir: str, dtype=None) -> str:
    """Fold LoRA adapters into the base weights and write an HF-compatible directory (weights, config, tokenizer)."""
    from ..peft.lora import LoRAModel
    from ..transformers.auto import AutoModelForCausalLM

    model = AutoModelForCausalLM.from_pretrained(base_model_dir, dtype=dtype)
    merged = LoRAModel.from_pretrained(model, lora_dir).merged_model()
    merged.save_pretrained(output_dir)
    for fn in os.listdir(base_model_dir):
        if fn.startswith("tokenizer") or fn in ("special_tokens_map.json", "generation_config.json", "vocab.json", "merges.txt") or fn.endswith(".model"):
            shutil.copy(os.path.join(base_model_dir, fn), os.path.join(output_dir, fn))
    return output_dir
