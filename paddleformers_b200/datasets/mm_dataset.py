"""Multimodal SFT examples: chat messages with ``<image>`` markers plus image files -> token ids with one placeholder
token per merged patch, labels, pixel patches and grids (the job of the reference's multimodal plugins,
paddleformers/datasets/template/mm_plugin.py, and ``mm_collate_fn``, paddleformers/datasets/collate.py:755).

Every ``<image>`` in a message is replaced by ``vision_start + image_pad * n + vision_end`` where n is the number of
merged patches of the corresponding image after pre-processing; the expansion is done on token ids, so the tokenizer
only has to know the three special tokens.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch
from torch.utils.data import Dataset

from .sft_dataset import IGNORE_INDEX, read_examples, to_messages
from .template import get_template

IMAGE_MARKER = "<image>"


def _load_image(path_or_array) -> np.ndarray:
    if isinstance(path_or_array, np.ndarray):
        return path_or_array
    from PIL import Image

    return np.asarray(Image.open(path_or_array).convert("RGB"))


class MMSFTDataset(Dataset):
    def __init__(self, path_or_examples, tokenizer, image_processor, template: Optional[str], max_seq_len: int,
                 image_token: str = "<|image_pad|>", vision_start_token: Optional[str] = "<|vision_start|>",
                 vision_end_token: Optional[str] = "<|vision_end|>", emit_token_types: bool = False, pretrain: bool = False):
        self.examples = list(read_examples(path_or_examples)) if isinstance(path_or_examples, str) else list(path_or_examples)
        self.tok, self.proc, self.template, self.max_seq_len = tokenizer, image_processor, get_template(template), max_seq_len
        ids = [None if t is None else tokenizer.convert_tokens_to_ids(t) for t in (image_token, vision_start_token, vision_end_token)]
        if any(t is not None and (i is None or i == tokenizer.unk_token_id)
               for t, i in zip((image_token, vision_start_token, vision_end_token), ids)):
            raise ValueError("the tokenizer must know the image placeholder and vision start / end tokens")
        self.image_id, self.start_id, self.end_id = ids               # families without start / end tokens pass None for them
        self.pretrain = pretrain                                       # VL-PT: {"text": "... <image> ...", "images": [...]}, every text token a target
        self.emit_token_types = emit_token_types                       # prefix-LM families: 0 on context tokens, 1 on answer tokens
        self.marker_ids = tokenizer.encode(IMAGE_MARKER, add_special_tokens=False)

    def __len__(self):
        return len(self.examples)

    def _expand(self, ids: List[int], mask: List[int], counts: List[int]):
        """Replace every occurrence of the marker's token sequence by the placeholder run of the next image."""
        out_ids, out_mask, k, i, m = [], [], 0, 0, len(self.marker_ids)
        while i < len(ids):
            if m and ids[i:i + m] == self.marker_ids and k < len(counts):
                run = ([self.start_id] if self.start_id is not None else []) + [self.image_id] * counts[k] \
                    + ([self.end_id] if self.end_id is not None else [])
                out_ids += run
                out_mask += [0] * len(run)            # image tokens are context, never targets
                k += 1
                i += m
            else:
                out_ids.append(ids[i])
                out_mask.append(mask[i])
                i += 1
        if k != len(counts):
            raise ValueError(f"{len(counts)} images but {k} {IMAGE_MARKER} markers in the conversation")
        return out_ids, out_mask

    def _images(self, ex):
        """(tensor fields of the example's images, placeholder count per image)."""
        images = [_load_image(p) for p in ex.get("images", [])]
        item, counts = {}, []
        if images:
            pre = self.proc(images)
            item["pixel_values"] = pre["pixel_values"]
            if "image_grid_thw" in pre:                 # variable-resolution towers: one grid per image
                item["image_grid_thw"] = pre["image_grid_thw"]
                counts = [self.proc.num_image_tokens(g) for g in pre["image_grid_thw"].tolist()]
            else:                                       # fixed-size towers: the same number of tokens for every image
                counts = [self.proc.num_image_tokens()] * len(images)
        return item, counts

    def _encode(self, ex, counts):
        """(token ids, target mask) of one conversation (or, for pre-training, of one text) with the image runs expanded."""
        ids, mask = [], []
        if self.pretrain or ("messages" not in ex and "text" in ex):
            ids = self.tok.encode(ex["text"], add_special_tokens=False)
            if self.tok.eos_token_id is not None:
                ids = ids + [self.tok.eos_token_id]
            mask = [1] * len(ids)
        else:
            norm = to_messages(ex)
            for p_ids, r_ids in self.template.encode_multiturn(self.tok, norm["messages"], norm["system"], norm["tools"]):
                ids += p_ids + r_ids
                mask += [0] * len(p_ids) + [1] * len(r_ids)
        return self._expand(ids, mask, counts)

    def __getitem__(self, i):
        ex = self.examples[i]
        item, counts = self._images(ex)
        ids, mask = self._encode(ex, counts)
        if len(ids) > self.max_seq_len + 1:
            raise ValueError(f"example {i} needs {len(ids)} tokens (images are not truncated); raise max_seq_len")
        item["input_ids"] = torch.tensor(ids[:-1])
        item["labels"] = torch.tensor([t if m else IGNORE_INDEX for t, m in zip(ids[1:], mask[1:])])
        if self.emit_token_types:
            item["token_type_ids"] = torch.tensor(mask[:-1])
        return item


class MMDPODataset(MMSFTDataset):
    """Preference pairs over images: {"messages" | "prompt", "images", "chosen", "rejected"}. Every example yields two
    sequences that share the prompt and its images, one ending in the chosen and one in the rejected response; targets are
    the response tokens only (the multimodal side of paddleformers/cli/train/dpo/workflow.py:65)."""

    def __getitem__(self, i):
        ex = self.examples[i]
        item, counts = self._images(ex)
        if "messages" in ex:
            msgs = list(ex["messages"])
        else:
            prompt = ex.get("prompt", ex.get("src"))
            msgs = [{"role": "user", "content": prompt[-1] if isinstance(prompt, list) else prompt}]
        rows = []
        for key in ("chosen", "rejected"):
            resp = ex[key]["content"] if isinstance(ex[key], dict) else ex[key]
            ids, mask = self._encode(dict(ex, messages=msgs + [{"role": "assistant", "content": resp}]), counts)
            # only the final response is scored
            last = max((j for j in range(len(mask)) if mask[j] == 0), default=-1)
            mask = [0] * (last + 1) + mask[last + 1:]
            if len(ids) > self.max_seq_len + 1:
                raise ValueError(f"example {i} needs {len(ids)} tokens (images are not truncated); raise max_seq_len")
            rows.append((torch.tensor(ids[:-1]), torch.tensor([t if m else IGNORE_INDEX for t, m in zip(ids[1:], mask[1:])])))
        item["input_ids"], item["labels"] = [r[0] for r in rows], [r[1] for r in rows]
        return item


def mm_dpo_collate_fn(examples: List[dict], pad_token_id: int = 0, ignore_index: int = IGNORE_INDEX) -> dict:
    """Rows 2b / 2b + 1 hold example b's chosen / rejected sequence; the example's image patches (and grids) appear once per
    row, in row order, so that the placeholders of both rows find their features."""
    flat = []
    for e in examples:
        for k in range(2):
            row = {"input_ids": e["input_ids"][k], "labels": e["labels"][k]}
            for key in ("pixel_values", "image_grid_thw"):
                if e.get(key) is not None:
                    row[key] = e[key]
            flat.append(row)
    from ..models.vision_language import mm_collate_fn

    out = mm_collate_fn(flat, pad_token_id=pad_token_id, ignore_index=ignore_index)
    out["preference_pairs"] = torch.tensor(len(examples))
    return out
