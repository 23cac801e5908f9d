"""Declarative mapping between Hugging Face checkpoint tensors and this framework's fused parameters.

The reference bridges its internal layout and HF names with "AOA" statements such as
``q,k,v -> qkv_proj.weight, fused_qkv`` (paddleformers/transformers/aoa_config_base.py:339-452,
paddleformers/transformers/llama/modeling.py:324-353). torch linears already use HF's ``[out, in]`` layout, so only
fusions remain here: concatenated projections (qkv, gate|up, MLA kv_a) and stacked experts. Every rule is
invertible, which gives ``save_pretrained`` for free, and every rule knows how to cut its target for a tensor /
expert parallel rank so that a rank only materialises its own shard.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch


@dataclass
class ShardSpec:
    """How a parameter is cut over the tensor-parallel (tp) and expert-parallel (ep) groups.

    ``tp_dim``: dimension split over tp (None = replicated). ``sections``: sizes of the fused sections along
    ``tp_dim`` in the *full* tensor; each section is split separately (fused qkv / gate|up). ``ep_dim``: dimension
    that indexes experts (split over ep)."""

    tp_dim: Optional[int] = None
    sections: Optional[List[int]] = None
    ep_dim: Optional[int] = None

    def shard(self, full: torch.Tensor, tp_rank: int, tp_size: int, ep_rank: int = 0, ep_size: int = 1) -> torch.Tensor:
        t = full
        if self.ep_dim is not None and ep_size > 1:
            n = t.shape[self.ep_dim] // ep_size
            t = t.narrow(self.ep_dim, ep_rank * n, n)
        if self.tp_dim is not None and tp_size > 1:
            secs = self.sections or [t.shape[self.tp_dim]]
            parts, off = [], 0
            for s in secs:
                assert s % tp_size == 0, f"section {s} not divisible by tp {tp_size}"
                n = s // tp_size
                parts.append(t.narrow(self.tp_dim, off + tp_rank * n, n))
                off += s
            t = torch.cat(parts, dim=self.tp_dim) if len(parts) > 1 else parts[0]
        return t.contiguous()

    def unshard(self, shards: Sequence[torch.Tensor], tp_size: int) -> torch.Tensor:
        """Inverse of ``shard`` over tp (``shards`` ordered by tp rank)."""
        if self.tp_dim is None or tp_size == 1:
            return shards[0]
        secs = self.sections or [shards[0].shape[self.tp_dim] * tp_size]
        out, off = [], 0
        for s in secs:
            n = s // tp_size
            out.extend(sh.narrow(self.tp_dim, off, n) for sh in shards)
            off += n
        return torch.cat(out, dim=self.tp_dim)


def _rope_rows(t: torch.Tensor, spec, inverse: bool) -> torch.Tensor:
    """``spec`` = head_dim (whole heads are rotary) or (head_size, rope_offset, rope_dim): inside every chunk of
    ``head_size`` rows only rows [rope_offset, rope_offset + rope_dim) carry the rotary embedding (MLA: each query head is
    [nope | rope]; the compressed kv projection is [latent | rope])."""
    fn = interleave_rope_rows if inverse else deinterleave_rope_rows
    if isinstance(spec, int):
        return fn(t, spec)
    head, off, rd = spec
    nh = t.shape[0] // head
    v = t.reshape(nh, head, *t.shape[1:]).clone()
    part = v[:, off:off + rd].reshape(nh * rd, *t.shape[1:])
    v[:, off:off + rd] = fn(part, rd).reshape(nh, rd, *t.shape[1:])
    return v.reshape(t.shape)


def deinterleave_rope_rows(t: torch.Tensor, head_dim: int) -> torch.Tensor:
    """Reorder the rows of a q / k projection (or bias) from the interleaved rotary layout, where the pair rotated
    together sits at rows (2i, 2i + 1) of each head, to the half-split layout (i, i + head_dim / 2) that the rotary
    kernels use. Attention scores are invariant under a common permutation of q and k features, so a checkpoint
    trained with interleaved rotation computes the same function after this permutation with half-split rotation."""
    nh = t.shape[0] // head_dim
    rest = t.shape[1:]
    return t.reshape(nh, head_dim // 2, 2, *rest).transpose(1, 2).reshape(t.shape)


def interleave_rope_rows(t: torch.Tensor, head_dim: int) -> torch.Tensor:
    """Inverse of ``deinterleave_rope_rows``."""
    nh = t.shape[0] // head_dim
    rest = t.shape[1:]
    return t.reshape(nh, 2, head_dim // 2, *rest).transpose(1, 2).reshape(t.shape)


def ungroup_qkv_rows(t: torch.Tensor, n_kv: int, q_per_kv: int, head_dim: int) -> torch.Tensor:
    """Rows stored per kv head as [q_0 .. q_{g-1}, k, v] (InternLM2's ``wqkv``) -> [all q heads | all k heads | all v heads]."""
    rest = t.shape[1:]
    v = t.reshape(n_kv, q_per_kv + 2, head_dim, *rest)
    q = v[:, :q_per_kv].reshape(n_kv * q_per_kv * head_dim, *rest)
    k = v[:, q_per_kv].reshape(n_kv * head_dim, *rest)
    val = v[:, q_per_kv + 1].reshape(n_kv * head_dim, *rest)
    return torch.cat([q, k, val], dim=0)


def group_qkv_rows(t: torch.Tensor, n_kv: int, q_per_kv: int, head_dim: int) -> torch.Tensor:
    """Inverse of ``ungroup_qkv_rows``."""
    rest = t.shape[1:]
    nq = n_kv * q_per_kv * head_dim
    q = t[:nq].reshape(n_kv, q_per_kv, head_dim, *rest)
    k = t[nq:nq + n_kv * head_dim].reshape(n_kv, 1, head_dim, *rest)
    v = t[nq + n_kv * head_dim:].reshape(n_kv, 1, head_dim, *rest)
    return torch.cat([q, k, v], dim=1).reshape(t.shape)


@dataclass
class Rule:
    """target <- op(sources). ``sources`` may contain ``{E}`` (expanded over experts for stack rules)."""

    target: str
    sources: List[str]
    op: str = "rename"  # rename | concat | stack | stack_concat
    dim: int = 0
    num_experts: int = 0
    expert_pairs: int = 1  # stack_concat: sources per expert (gate, up)
    sizes: Optional[List[int]] = None  # concat: size of each source along ``dim`` (default: equal parts)
    rope_deinterleave: Optional[Dict[int, object]] = None  # source index -> head_dim | (head_size, rope_offset, rope_dim):
    #                                                          rows stored in interleaved rotary order
    flatten: bool = False              # rename: the checkpoint stores the tensor with a leading unit dimension
    reshape: Optional[List[int]] = None        # rename: shape of the internal parameter (e.g. a Conv3d kernel used as a matrix)
    source_shape: Optional[List[int]] = None   # rename: shape of the tensor in the checkpoint, for the way back
    offset: float = 0.0                        # rename: internal = checkpoint + offset ((1 + w) norm weights)
    fn: Optional[Tuple[Callable, Callable]] = None      # rename: (checkpoint -> internal, internal -> checkpoint) for layouts
    #                                                     that no declarative field covers
    expert_base: int = 0                                # stack rules: checkpoint index of this group's first expert (two expert
    #                                                     groups of one layer numbered consecutively)
    qkv_groups: Optional[Tuple[int, int, int]] = None   # rename: (kv heads, q heads per kv head, head dim) of a checkpoint that
    #                                                     stores the fused projection grouped by kv head: [q.. q k v] per group

    def _load(self, i: int, t: torch.Tensor) -> torch.Tensor:
        if self.rope_deinterleave and i in self.rope_deinterleave:
            t = _rope_rows(t, self.rope_deinterleave[i], inverse=False)
        return t

    def _store(self, i: int, t: torch.Tensor) -> torch.Tensor:
        if self.rope_deinterleave and i in self.rope_deinterleave:
            t = _rope_rows(t, self.rope_deinterleave[i], inverse=True)
        return t

    def source_names(self) -> List[str]:
        if self.op in ("stack", "stack_concat"):
            return [s.format(E=self.expert_base + e) for e in range(self.num_experts) for s in self.sources]
        return list(self.sources)

    def forward(self, get: Callable[[str], torch.Tensor], expert_range: Optional[range] = None) -> torch.Tensor:
        if self.op == "rename":
            t = self._load(0, get(self.sources[0]))
            if self.qkv_groups is not None:
                t = ungroup_qkv_rows(t, *self.qkv_groups)
            if self.fn is not None:
                t = self.fn[0](t)
            if self.offset:
                t = t + self.offset
            if self.reshape is not None:
                return t.reshape(self.reshape)
            return t.reshape(-1) if self.flatten else t
        if self.op == "concat":
            return torch.cat([self._load(i, get(s)) for i, s in enumerate(self.sources)], dim=self.dim)
        er = expert_range if expert_range is not None else range(self.num_experts)
        if self.op == "stack":
            return torch.stack([get(self.sources[0].format(E=self.expert_base + e)) for e in er], dim=0)
        if self.op == "stack_concat":
            return torch.stack([torch.cat([get(s.format(E=self.expert_base + e)) for s in self.sources], dim=self.dim) for e in er], dim=0)
        raise ValueError(self.op)

    def inverse(self, tensor: torch.Tensor, section_sizes: Optional[List[int]] = None, expert_offset: int = 0) -> Dict[str, torch.Tensor]:
        if self.op == "rename":
            t = self._store(0, tensor)
            if self.qkv_groups is not None:
                t = group_qkv_rows(t, *self.qkv_groups)
            if self.fn is not None:
                t = self.fn[1](t)
            if self.offset:
                t = t - self.offset
            if self.source_shape is not None:
                return {self.sources[0]: t.reshape(self.source_shape)}
            return {self.sources[0]: t.reshape(1, -1) if self.flatten else t}
        if self.op == "concat":
            sizes = section_sizes or self.sizes or [tensor.shape[self.dim] // len(self.sources)] * len(self.sources)
            return {s: self._store(i, p).contiguous()
                    for i, (s, p) in enumerate(zip(self.sources, torch.split(tensor, sizes, dim=self.dim)))}
        out = {}
        for i in range(tensor.shape[0]):
            e = self.expert_base + expert_offset + i
            if self.op == "stack":
                out[self.sources[0].format(E=e)] = tensor[i].contiguous()
            else:
                sizes = section_sizes or [tensor.shape[1 + self.dim] // len(self.sources)] * len(self.sources)
                for s, p in zip(self.sources, torch.split(tensor[i], sizes, dim=self.dim)):
                    out[s.format(E=e)] = p.contiguous()
        return out


class WeightMap:
    """All rules of one model instance, indexed by internal parameter name."""

    def __init__(self, rules: Iterable[Rule], translation: Optional[Sequence[Sequence[str]]] = None):
        self.rules: Dict[str, Rule] = {r.target: r for r in rules}
        self.translation = [tuple(x) for x in (translation or [])]

    def translate(self, name: str) -> str:
        """Checkpoint-side spelling of a name for families that store the same tensors under other names."""
        for a, b in self.translation:
            name = name.replace(a, b)
        return name

    def rule_for(self, target: str) -> Rule:
        return self.rules.get(target) or Rule(target, [self.translate(target)])

    def hf_names(self) -> List[str]:
        out = []
        for r in self.rules.values():
            out.extend(r.source_names())
        return out


def expand_layers(template_rules: List[Rule], layer_ids: Iterable[int]) -> List[Rule]:
    out = []
    for i in layer_ids:
        for r in template_rules:
            out.append(Rule(r.target.replace("{L}", str(i)), [s.replace("{L}", str(i)) for s in r.sources], r.op, r.dim,
                            r.num_experts, r.expert_pairs, r.sizes, r.rope_deinterleave, r.flatten, r.reshape, r.source_shape, r.offset,
                            r.fn, r.expert_base, r.qkv_groups))
    return out
