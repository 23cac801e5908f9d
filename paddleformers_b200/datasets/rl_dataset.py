"""Data side of reinforcement learning from feedback: prompt datasets for rollouts and the batch container that RL
pipelines pass between their stages.

* ``RLHFDataset`` - prompts (and optional reference answers) from a jsonl file, rendered through the tokenizer's chat
  template on request, tokenised lazily, truncated or filtered at ``max_prompt_len``
  (paddleformers/datasets/rlhf_datasets/rl_dataset.py:83-174).
* ``rl_collate_fn`` - LEFT-pads prompts so that generation continues at the right edge of every row (:33-81).
* ``DataProto`` - a batch of tensors with equal leading dimension, per-sample non-tensor values (numpy object arrays) and
  batch-level ``meta_info``, with the operations an RL loop needs: select / pop / union, chunk / concat for data-parallel
  workers, repeat for several samples per prompt, reorder, mini-batch iteration, padding to a divisor
  (paddleformers/datasets/rlhf_datasets/protocol.py:211-600).
"""
from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterator, List, Optional, Sequence

import numpy as np
import torch


def left_padding(sequences: Sequence[torch.Tensor], padding_value: int = 0, max_length: Optional[int] = None) -> torch.Tensor:
    n = max_length or max(int(s.shape[0]) for s in sequences)
    out = torch.full((len(sequences), n), padding_value, dtype=sequences[0].dtype)
    for i, s in enumerate(sequences):
        s = s[-n:]
        out[i, n - s.shape[0]:] = s
    return out


def rl_collate_fn(items: List[dict], pad_token_id: int, requires_label: bool = False, max_prompt_len: Optional[int] = None) -> dict:
    ids = [torch.as_tensor(x["input_ids"], dtype=torch.long) for x in items]
    out = {"input_ids": left_padding(ids, pad_token_id, None if max_prompt_len is None else min(max_prompt_len, max(len(i) for i in ids)))}
    out["attention_mask"] = left_padding([torch.ones_like(i) for i in ids], 0, out["input_ids"].shape[1])
    # positions count real tokens only, so that a left-padded prompt sees the positions of the unpadded one
    out["position_ids"] = (out["attention_mask"].cumsum(-1) - 1).clamp(min=0)
    if requires_label:
        lab = [torch.as_tensor(x["label_ids"], dtype=torch.long) for x in items]
        n = max(len(x) for x in lab)
        out["label_ids"] = torch.stack([torch.cat([x, x.new_full((n - len(x),), pad_token_id)]) for x in lab])
    return out


class RLHFDataset(torch.utils.data.Dataset):
    def __init__(self, path: str, tokenizer, max_prompt_len: int = 1024, prompt_key: str = "src", requires_label: bool = False,
                 response_key: Optional[str] = None, apply_chat_template: bool = False, filter_overlong_prompts: bool = True,
                 chat_template_func: Optional[Callable] = None):
        self.tokenizer, self.max_prompt_len = tokenizer, int(max_prompt_len)
        self.prompt_key, self.response_key, self.requires_label = prompt_key, response_key, requires_label
        self.apply_chat_template, self.chat_template_func = apply_chat_template, chat_template_func
        with open(path, encoding="utf-8") as f:
            rows = [json.loads(line) for line in f if line.strip()]
        self._cache: Dict[int, dict] = {}
        self.rows = rows
        if filter_overlong_prompts:          # drop instead of truncating: a cut prompt asks a different question
            keep = [i for i in range(len(rows)) if len(self._prompt_ids(rows[i], truncate=False)) <= self.max_prompt_len]
            self.rows = [rows[i] for i in keep]

    def _render(self, prompt):
        if self.chat_template_func is not None:
            return self.chat_template_func(prompt)
        if self.apply_chat_template and getattr(self.tokenizer, "chat_template", None):
            msgs = prompt if isinstance(prompt, list) else [{"role": "user", "content": prompt}]
            return self.tokenizer.apply_chat_template(msgs, add_generation_prompt=True, tokenize=False)
        if isinstance(prompt, list):
            return "\n".join(m.get("content", "") for m in prompt)
        return prompt

    def _prompt_ids(self, row: dict, truncate: bool = True) -> List[int]:
        ids = self.tokenizer(self._render(row[self.prompt_key]), add_special_tokens=True)["input_ids"]
        return ids[-self.max_prompt_len:] if truncate else ids          # keep the end: the question sits there

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i: int) -> dict:
        if i not in self._cache:
            row = self.rows[i]
            item = {"input_ids": torch.tensor(self._prompt_ids(row), dtype=torch.long)}
            if self.requires_label:
                item["label_ids"] = torch.tensor(self.tokenizer(str(row[self.response_key]), add_special_tokens=False)["input_ids"],
                                                 dtype=torch.long)
            self._cache[i] = item
        return self._cache[i]


@dataclass
class DataProto:
    batch: Dict[str, torch.Tensor] = field(default_factory=dict)
    non_tensor_batch: Dict[str, np.ndarray] = field(default_factory=dict)
    meta_info: Dict[str, object] = field(default_factory=dict)

    def __post_init__(self):
        self.non_tensor_batch = {k: (v if isinstance(v, np.ndarray) else np.asarray(v, dtype=object))
                                 for k, v in self.non_tensor_batch.items()}
        self.check_consistency()

    # ------------------------------------------------------------------ basics
    def __len__(self) -> int:
        for v in self.batch.values():
            return int(v.shape[0])
        for v in self.non_tensor_batch.values():
            return int(v.shape[0])
        return 0

    def check_consistency(self) -> None:
        n = len(self)
        for k, v in list(self.batch.items()) + list(self.non_tensor_batch.items()):
            if int(v.shape[0]) != n:
                raise ValueError(f"{k}: leading dimension {v.shape[0]} differs from the batch size {n}")

    @classmethod
    def from_dict(cls, tensors: Dict[str, torch.Tensor], non_tensors: Optional[dict] = None, meta_info: Optional[dict] = None):
        return cls(dict(tensors), dict(non_tensors or {}), dict(meta_info or {}))

    @classmethod
    def from_single_dict(cls, data: dict, meta_info: Optional[dict] = None):
        t = {k: v for k, v in data.items() if torch.is_tensor(v)}
        return cls(t, {k: v for k, v in data.items() if k not in t}, dict(meta_info or {}))

    def __getitem__(self, idx):
        if isinstance(idx, (int, np.integer)):
            return {**{k: v[idx] for k, v in self.batch.items()}, **{k: v[idx] for k, v in self.non_tensor_batch.items()}}
        return DataProto({k: v[idx] for k, v in self.batch.items()}, {k: v[idx] for k, v in self.non_tensor_batch.items()},
                         self.meta_info)

    def to(self, device) -> "DataProto":
        self.batch = {k: v.to(device) for k, v in self.batch.items()}
        return self

    # ------------------------------------------------------------------ column operations
    def select(self, batch_keys=None, non_tensor_batch_keys=None, meta_info_keys=None, deepcopy: bool = False) -> "DataProto":
        b = {k: self.batch[k] for k in (batch_keys if batch_keys is not None else self.batch)}
        n = {k: self.non_tensor_batch[k] for k in (non_tensor_batch_keys if non_tensor_batch_keys is not None else self.non_tensor_batch)}
        m = {k: self.meta_info[k] for k in (meta_info_keys if meta_info_keys is not None else self.meta_info)}
        out = DataProto(b, n, m)
        return copy.deepcopy(out) if deepcopy else out

    def pop(self, batch_keys=None, non_tensor_batch_keys=None, meta_info_keys=None) -> "DataProto":
        b = {k: self.batch.pop(k) for k in (batch_keys or [])}
        n = {k: self.non_tensor_batch.pop(k) for k in (non_tensor_batch_keys or [])}
        m = {k: self.meta_info.pop(k) for k in (meta_info_keys or [])}
        return DataProto(b, n, m)

    def rename(self, old_keys, new_keys) -> "DataProto":
        old_keys = [old_keys] if isinstance(old_keys, str) else list(old_keys)
        new_keys = [new_keys] if isinstance(new_keys, str) else list(new_keys)
        if len(old_keys) != len(new_keys):
            raise ValueError("rename needs as many new names as old ones")
        for o, nn_ in zip(old_keys, new_keys):
            self.batch[nn_] = self.batch.pop(o)
        return self

    def union(self, other: "DataProto") -> "DataProto":
        """Add the other batch's columns; a column present in both must hold the same values."""
        if len(other) != len(self) and len(self) and len(other):
            raise ValueError("union needs equal batch sizes")
        for k, v in other.batch.items():
            if k in self.batch and not torch.equal(self.batch[k], v):
                raise ValueError(f"{k} differs between the two batches")
            self.batch[k] = v
        for k, v in other.non_tensor_batch.items():
            if k in self.non_tensor_batch and not np.array_equal(self.non_tensor_batch[k], v):
                raise ValueError(f"{k} differs between the two batches")
            self.non_tensor_batch[k] = v
        for k, v in other.meta_info.items():
            if k in self.meta_info and self.meta_info[k] != v:
                raise ValueError(f"meta_info[{k!r}] differs between the two batches")
            self.meta_info[k] = v
        return self

    # ------------------------------------------------------------------ row operations
    def chunk(self, chunks: int) -> List["DataProto"]:
        if len(self) % chunks:
            raise ValueError(f"batch size {len(self)} is not divisible by {chunks} (pad_to_divisor first)")
        n = len(self) // chunks
        return [self[i * n:(i + 1) * n] for i in range(chunks)]

    @staticmethod
    def concat(parts: List["DataProto"]) -> "DataProto":
        b = {k: torch.cat([p.batch[k] for p in parts], dim=0) for k in parts[0].batch}
        n = {k: np.concatenate([p.non_tensor_batch[k] for p in parts], axis=0) for k in parts[0].non_tensor_batch}
        return DataProto(b, n, parts[0].meta_info)

    def reorder(self, indices: torch.Tensor) -> "DataProto":
        idx = indices.cpu().numpy()
        self.batch = {k: v[indices.to(v.device)] for k, v in self.batch.items()}
        self.non_tensor_batch = {k: v[idx] for k, v in self.non_tensor_batch.items()}
        return self

    def repeat(self, repeat_times: int = 2, interleave: bool = True) -> "DataProto":
        """``interleave``: a a b b (several samples per prompt, neighbours); otherwise a b a b."""
        if interleave:
            b = {k: v.repeat_interleave(repeat_times, dim=0) for k, v in self.batch.items()}
            n = {k: np.repeat(v, repeat_times, axis=0) for k, v in self.non_tensor_batch.items()}
        else:
            b = {k: v.repeat(repeat_times, *([1] * (v.dim() - 1))) for k, v in self.batch.items()}
            n = {k: np.tile(v, (repeat_times,) + (1,) * (v.ndim - 1)) for k, v in self.non_tensor_batch.items()}
        return DataProto(b, n, self.meta_info)

    def pad_to_divisor(self, divisor: int):
        """(padded batch, number of padding rows): rows from the start are repeated until the size divides."""
        pad = (-len(self)) % divisor
        if pad == 0:
            return self, 0
        reps = [self[i % len(self):i % len(self) + 1] for i in range(pad)]
        return DataProto.concat([self] + reps), pad

    def unpad(self, pad: int) -> "DataProto":
        return self[:len(self) - pad] if pad else self

    def make_iterator(self, mini_batch_size: int, epochs: int = 1, seed: Optional[int] = None) -> Iterator["DataProto"]:
        if len(self) % mini_batch_size:
            raise ValueError(f"batch size {len(self)} is not divisible by the mini-batch size {mini_batch_size}")
        g = torch.Generator()
        if seed is not None:
            g.manual_seed(seed)
        for _ in range(epochs):
            order = torch.randperm(len(self), generator=g) if seed is not None else torch.arange(len(self))
            for lo in range(0, len(self), mini_batch_size):
                idx = order[lo:lo + mini_batch_size]
                yield DataProto({k: v[idx.to(v.device)] for k, v in self.batch.items()},
                                {k: v[idx.numpy()] for k, v in self.non_tensor_batch.items()}, self.meta_info)
