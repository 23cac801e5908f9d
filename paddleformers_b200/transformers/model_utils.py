"""``PretrainedModel``: construction from configs, Hugging Face safetensors loading and saving.

The public contract is the reference's (paddleformers/transformers/model_utils.py:1185 PretrainedModel,
:2702 from_pretrained, :3193 save_pretrained, :1366 from_config): checkpoints on disk are HF-compatible
``model.safetensors`` (or sharded ``model-0000x-of-0000y.safetensors`` with ``model.safetensors.index.json``) plus
``config.json``. Fused / stacked internal parameters are produced from HF tensors by the model's ``WeightMap`` and
each tensor- or expert-parallel rank only materialises its own shard; saving gathers shards back to full HF tensors
on the first rank of each parallel group with bounded host memory (one parameter at a time).
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, Iterable, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..parallel.topology import get_parallel_state
from ..utils.log import logger
from .configuration_utils import CONFIG_NAME, PretrainedConfig
from .conversion_utils import Rule, ShardSpec, WeightMap

SAFE_WEIGHTS_NAME = "model.safetensors"
SAFE_WEIGHTS_INDEX_NAME = "model.safetensors.index.json"


def _dtype_of(name):
    if isinstance(name, torch.dtype):
        return name
    return {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16,
            "bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[str(name).replace("torch.", "")]


def param_shard_spec(p: torch.Tensor) -> ShardSpec:
    spec = getattr(p, "shard_spec", None)
    if spec is None:
        return ShardSpec()
    kind, dim, sections = spec
    if kind == "tp":
        return ShardSpec(tp_dim=dim, sections=sections)
    if kind == "ep":
        return ShardSpec(ep_dim=dim)
    return ShardSpec()


class _CheckpointReader:
    """Lazy reader over one or several safetensors files of a HF directory."""

    def __init__(self, directory: str):
        from safetensors import safe_open

        self.dir = directory
        self._open = safe_open
        self._handles = {}
        index = os.path.join(directory, SAFE_WEIGHTS_INDEX_NAME)
        if os.path.exists(index):
            with open(index) as f:
                self.weight_map = json.load(f)["weight_map"]
        else:
            single = os.path.join(directory, SAFE_WEIGHTS_NAME)
            if not os.path.exists(single):
                cands = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
                if not cands:
                    raise FileNotFoundError(f"no safetensors weights in {directory}")
                self.weight_map = {}
                for c in cands:
                    with safe_open(os.path.join(directory, c), framework="pt") as h:
                        for k in h.keys():
                            self.weight_map[k] = c
            else:
                with safe_open(single, framework="pt") as h:
                    self.weight_map = {k: SAFE_WEIGHTS_NAME for k in h.keys()}

    def keys(self):
        return self.weight_map.keys()

    def has(self, name):
        return name in self.weight_map

    def get(self, name: str) -> torch.Tensor:
        file = self.weight_map[name]
        h = self._handles.get(file)
        if h is None:
            h = self._open(os.path.join(self.dir, file), framework="pt")
            self._handles[file] = h
        return h.get_tensor(name)


class PretrainedModel(nn.Module):
    config_class = PretrainedConfig
    base_model_prefix = "model"
    _keys_to_ignore_on_load_missing: List[str] = []

    def __init__(self, config: PretrainedConfig):
        super().__init__()
        self.config = config

    # ------------------------------------------------------------------ init
    def _init_weights(self, module: nn.Module) -> None:  # overridden
        pass

    def post_init(self):
        if getattr(self.config, "_skip_init", False):
            return
        self.apply(self._init_weights)

    def weight_map(self) -> WeightMap:
        return WeightMap([])

    @property
    def dtype(self):
        return next(self.parameters()).dtype

    @property
    def device(self):
        return next(self.parameters()).device

    def num_parameters(self, only_trainable: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not only_trainable)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_config(cls, config: PretrainedConfig, dtype=None, device=None, **kwargs):
        if dtype is not None:
            config.dtype = str(dtype).replace("torch.", "")
        return cls(config, dtype=_dtype_of(config.dtype), device=device)

    _from_config = from_config

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str, config: Optional[PretrainedConfig] = None, dtype=None,
                        device=None, convert_from_hf: bool = True, **config_overrides):
        from ..utils.download import resolve_dir

        directory = resolve_dir(pretrained_model_name_or_path)
        if config is None:
            config = cls.config_class.from_pretrained(directory, **config_overrides)
        if dtype is not None:
            config.dtype = str(dtype).replace("torch.", "")
        config._skip_init = True
        try:
            model = cls(config, dtype=_dtype_of(config.dtype), device=device)
        finally:
            config.__dict__.pop("_skip_init", None)
        model.load_hf_checkpoint(directory)
        return model

    # ------------------------------------------------------------------ loading
    def load_hf_checkpoint(self, directory: str, strict: bool = False, target_for=None) -> None:
        """``target_for(param) -> tensor | None`` redirects the copy: the loaded (and sharded) value of every parameter goes
        into the returned tensor instead of the parameter, parameters mapped to None are skipped. Used to read optimizer
        state stored under parameter names."""
        reader = _CheckpointReader(directory)
        wm = self.weight_map()
        ps = get_parallel_state()
        tp_rank, tp_size = ps.coord["mp"], ps.degrees.mp
        ep_rank, ep_size = (ps.rank_in("ep"), ps.degrees.ep)
        dequant = None
        qcfg = getattr(self.config, "quantization_config", None)
        if qcfg:
            from ..quantization.checkpoint_dequant import build_dequantizer

            dequant = build_dequantizer(qcfg, reader)
            qc = qcfg if isinstance(qcfg, dict) else getattr(qcfg, "__dict__", {})
            if qc.get("quant_method") == "mxfp4":
                from ..quantization.checkpoint_dequant import MXFP4Reader

                reader = MXFP4Reader(reader)          # "<name>" is served from "<name>_blocks" + "<name>_scales"
        missing, loaded = [], 0
        tied = bool(getattr(self.config, "tie_word_embeddings", False))

        def get(name):
            t = reader.get(name)
            if dequant is not None:
                t = dequant(name, t)
            return t

        local_targets = dict(self.named_parameters())
        local_targets.update({k: v for k, v in self.named_buffers() if k in self.state_dict()})
        targets = {self.global_param_name(k): v for k, v in local_targets.items()}
        if target_for is not None:
            targets = {k: v for k, v in targets.items() if target_for(v) is not None}
        with torch.no_grad():
            for name, p in targets.items():
                rule = wm.rule_for(name)
                spec = param_shard_spec(p)
                srcs = rule.source_names()
                if not all(reader.has(s) for s in srcs):
                    if name == "lm_head.weight" and reader.has("model.embed_tokens.weight"):
                        full = get("model.embed_tokens.weight")
                    elif reader.has(name):
                        # the checkpoint already stores this tensor in the fused internal layout (stacked experts
                        # [E, 2I, H] / [E, H, I] as written by recent Hugging Face releases)
                        full = get(name)
                    elif rule.op in ("stack", "stack_concat") and "{E}" in rule.sources[0] and \
                            reader.has(rule.sources[0].split("{E}")[0] + name.rsplit(".", 1)[-1]):
                        # the same, under the checkpoint's own prefix (a decoder nested inside a larger model)
                        full = get(rule.sources[0].split("{E}")[0] + name.rsplit(".", 1)[-1])
                    else:
                        missing.append(name)
                        continue
                else:
                    erange = None
                    if rule.op in ("stack", "stack_concat") and spec.ep_dim == 0 and ep_size > 1:
                        n = rule.num_experts // ep_size
                        erange = range(ep_rank * n, (ep_rank + 1) * n)
                        full = rule.forward(get, erange)
                        spec = ShardSpec(tp_dim=spec.tp_dim, sections=spec.sections)
                    else:
                        full = rule.forward(get)
                shard = spec.shard(full, tp_rank, tp_size, ep_rank, ep_size)
                if tuple(shard.shape) != tuple(p.shape):
                    raise ValueError(f"shape mismatch for {name}: checkpoint {tuple(shard.shape)} vs model {tuple(p.shape)}")
                dst = p if target_for is None else target_for(p)
                if dst is not None:
                    dst.copy_(shard.to(dst.dtype))
                loaded += 1
        missing = [m for m in missing if not any(re.search(pat, m) for pat in self._keys_to_ignore_on_load_missing)]
        if missing:
            msg = f"{len(missing)} parameters were not found in {directory} and keep their initial values: {missing[:8]}..."
            if strict:
                raise KeyError(msg)
            logger.warning(msg)
            for name in missing:
                mod_name = name.rsplit(".", 1)[0]
                try:
                    self._init_weights(self.get_submodule(mod_name))
                except Exception:  # noqa: BLE001 - names of pipeline stages are global, modules local
                    pass
        logger.info(f"loaded {loaded} tensors from {directory}")

    # ------------------------------------------------------------------ saving
    def hf_state_dict_items(self, tensor_for=None):
        """Yields (hf_name, full tensor on CPU) for every parameter this rank is responsible for writing.
        ``tensor_for(param_or_buffer) -> tensor | None`` substitutes the value that is written (same shape as the local
        parameter; None skips it): optimizer state saved under parameter names goes through the same gathers and rules.

        Tensor-parallel shards are all-gathered inside the tp group (rank 0 of the group writes); expert-parallel
        ranks each write their own experts (HF names carry the global expert id)."""
        ps = get_parallel_state()
        wm = self.weight_map()
        tp_size, tp_rank, tp_group = ps.degrees.mp, ps.coord["mp"], ps.group("mp")
        ep_size, ep_rank = ps.degrees.ep, ps.rank_in("ep")
        dense_writer = ps.dataset_rank == 0 and ps.coord["cp"] == 0 and ps.coord["sep"] == 0
        expert_writer = ps.rank_in("moe_sharding") == 0
        sd = self.state_dict()
        seen = set()
        for local_name, t in sd.items():
            name = self.global_param_name(local_name)
            if name in seen:   # a parameter shared by two pipeline stages is written once
                continue
            seen.add(name)
            if not self.owns_global_param(local_name):
                continue
            obj = self._param_or_buffer(local_name)
            spec = param_shard_spec(obj)
            is_expert = spec.ep_dim is not None
            if tensor_for is not None:
                t = tensor_for(obj)
                if t is None:
                    continue
            full = t.detach()
            if spec.tp_dim is not None and tp_size > 1:
                # every tensor-parallel rank takes part in the gather; one of them keeps the result
                shards = [torch.empty_like(full) for _ in range(tp_size)]
                dist.all_gather(shards, full.contiguous(), group=tp_group)
                full = spec.unshard(shards, tp_size)
            if is_expert:
                if not expert_writer or (tp_size > 1 and tp_rank != 0 and ep_size == 1):
                    continue
            elif not dense_writer or tp_rank != 0:
                continue
            rule = wm.rule_for(name)
            offset = ep_rank * full.shape[0] if (is_expert and ep_size > 1) else 0
            secs = spec.sections if (spec.sections is not None and rule.op == "concat") else None
            for hf_name, ten in rule.inverse(full.cpu(), secs, offset).items():
                yield hf_name, ten

    def global_param_name(self, local_name: str) -> str:
        """Name of a local parameter in the un-partitioned model (identity unless the model is a pipeline stage)."""
        return local_name

    def owns_global_param(self, local_name: str) -> bool:
        """False for copies of a parameter whose primary owner is another pipeline stage."""
        return True

    def _param_or_buffer(self, name: str):
        mod_name, _, leaf = name.rpartition(".")
        mod = self.get_submodule(mod_name) if mod_name else self
        return getattr(mod, leaf)

    def save_pretrained(self, save_directory: str, max_shard_size: int = 5 * 1024 ** 3, save_config: bool = True,
                        tensor_for=None) -> None:
        from safetensors.torch import save_file

        ps = get_parallel_state()
        os.makedirs(save_directory, exist_ok=True)
        writer_tag = ps.weight_name_suffix() if (ps.degrees.ep > 1 or ps.degrees.pp > 1) else None
        if writer_tag is None and ps.degrees.pp > 1:
            writer_tag = f"pp{ps.coord['pp']:02d}"
        shards: List[Dict[str, torch.Tensor]] = [{}]
        size = 0
        for hf_name, ten in self.hf_state_dict_items(tensor_for):
            nbytes = ten.numel() * ten.element_size()
            if size + nbytes > max_shard_size and shards[-1]:
                shards.append({})
                size = 0
            shards[-1][hf_name] = ten.contiguous()
            size += nbytes
        shards = [s for s in shards if s]
        weight_map = {}
        single = len(shards) == 1 and writer_tag is None
        for i, s in enumerate(shards):
            if single:
                fname = SAFE_WEIGHTS_NAME
            else:
                tag = f"-{writer_tag}" if writer_tag else ""
                fname = f"model{tag}-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            save_file(s, os.path.join(save_directory, fname), metadata={"format": "pt"})
            for k in s:
                weight_map[k] = fname
        # merge the weight maps of all writers into one index
        world = dist.get_world_size() if dist.is_initialized() else 1
        if world > 1:
            maps = [None] * world
            dist.all_gather_object(maps, weight_map)
            merged = {}
            for m in maps:
                merged.update(m or {})
            weight_map = merged
        is_main = (not dist.is_initialized()) or dist.get_rank() == 0
        if is_main:
            if not single:
                total = sum(os.path.getsize(os.path.join(save_directory, f)) for f in set(weight_map.values())
                            if os.path.exists(os.path.join(save_directory, f)))
                with open(os.path.join(save_directory, SAFE_WEIGHTS_INDEX_NAME), "w") as f:
                    json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2, sort_keys=True)
            if save_config:
                self.config.architectures = [type(self).__name__]
                self.config.save_pretrained(save_directory)
        if world > 1:
            dist.barrier()
