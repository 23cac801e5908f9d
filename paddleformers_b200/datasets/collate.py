"""Collators: packed samples -> model inputs with O(S) mask descriptions.

Same contract as paddleformers/datasets/collate.py (``collate_fn`` :572, ``dpo_collate_fn`` :168,
``gen_attn_mask_startend_row_indices`` :1185, ``calc_padding_size`` :123):

* every sample is a list of ``Sequence`` objects packed into one row; token ids, (already shifted) labels and position
  ids are concatenated and padded to ``max_seq_len`` rounded up to the parallel padding multiple;
* ``padding_free`` flattens the whole batch into ONE row so that no pad tokens are computed at all;
* the attention mask is described column-wise: ``attn_mask_startend_row_indices[b, j]`` = first query row that may
  NOT see key j = end of the document containing j (pad keys get their own index, so nobody sees them); a dense
  [B, 1, S, S] boolean mask can be produced instead for the eager / sdpa backends.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence as Seq

import numpy as np
import torch

from .sft_dataset import IGNORE_INDEX, Sequence


def calc_padding_size(seq_len: int, training_args) -> int:
    cp = getattr(training_args, "context_parallel_size", 1) or 1
    sp = (getattr(training_args, "tensor_model_parallel_size", 1) or 1) if getattr(training_args, "sequence_parallel", False) else 1
    mult = 2 if cp * sp > 1 else 1
    if getattr(training_args, "fp8", None):
        mult = (mult + 3) // 4 * 4
    mult *= cp * sp
    return int(math.ceil(seq_len / mult) * mult)


def gen_attn_mask_startend_row_indices(doc_lens: Seq[int], max_seq_len: int, use_global_causal_attn: bool = False) -> np.ndarray:
    idx: List[int] = []
    offset = 0
    if use_global_causal_attn:
        total = sum(doc_lens)
        idx.extend([total] * total)
        offset = total
    else:
        for n in doc_lens:
            idx.extend([offset + n] * n)
            offset += n
    if offset < max_seq_len:
        idx.extend(range(offset, max_seq_len))
    return np.asarray(idx[:max_seq_len], dtype=np.int32)


def gen_self_attn_mask(doc_lens: Seq[int], max_seq_len: int, use_global_causal_attn: bool = False) -> np.ndarray:
    """Dense boolean [1, S, S] block-causal mask (True = attend) equivalent to the row indices above."""
    kend = gen_attn_mask_startend_row_indices(doc_lens, max_seq_len, use_global_causal_attn)
    i = np.arange(max_seq_len)[:, None]
    j = np.arange(max_seq_len)[None, :]
    return ((j <= i) & (i < kend[None, :]))[None]


def _pad(values: List[int], n: int, pad: int) -> List[int]:
    return values[:n] + [pad] * max(0, n - len(values))


def collate_fn(batch: List[List[Sequence]], tokenizer=None, training_args=None, max_seq_len: Optional[int] = None,
               padding_free: bool = False, use_attn_mask_startend_row_indices: bool = True,
               use_global_causal_attn: bool = False, pad_token_id: Optional[int] = None) -> Dict[str, torch.Tensor]:
    if pad_token_id is None:
        pad_token_id = getattr(tokenizer, "pad_token_id", None)
        if pad_token_id is None:
            pad_token_id = 0
    if padding_free:
        batch = [[s for sample in batch for s in sample]]
        max_seq_len = sum(len(s) for s in batch[0])
    if not max_seq_len:
        max_seq_len = max(sum(len(s) for s in sample) for sample in batch)
    if training_args is not None:
        max_seq_len = calc_padding_size(max_seq_len, training_args)
    out: Dict[str, List[Any]] = {"input_ids": [], "labels": [], "position_ids": []}
    masks = []
    for sample in batch:
        ids = [t for s in sample for t in s.token_ids]
        lab = [t for s in sample for t in s.labels]
        pos = [t for s in sample for t in s.position_ids]
        # the last label of a packed document must not predict the first token of the next document
        off = 0
        for s in sample[:-1]:
            off += len(s)
            if off - 1 < len(lab):
                lab[off - 1] = IGNORE_INDEX if s.labels[-1] == IGNORE_INDEX else lab[off - 1]
        out["input_ids"].append(_pad(ids, max_seq_len, pad_token_id))
        out["labels"].append(_pad(lab, max_seq_len, IGNORE_INDEX))
        out["position_ids"].append(_pad(pos, max_seq_len, 0))
        lens = [len(s) for s in sample]
        # truncate the document list to max_seq_len
        tot, kept = 0, []
        for n in lens:
            if tot >= max_seq_len:
                break
            kept.append(min(n, max_seq_len - tot))
            tot += kept[-1]
        if use_attn_mask_startend_row_indices:
            masks.append(gen_attn_mask_startend_row_indices(kept, max_seq_len, use_global_causal_attn))
        else:
            masks.append(gen_self_attn_mask(kept, max_seq_len, use_global_causal_attn))
    res = {k: torch.tensor(v, dtype=torch.long) for k, v in out.items()}
    if use_attn_mask_startend_row_indices:
        res["attn_mask_startend_row_indices"] = torch.from_numpy(np.stack(masks))
    else:
        res["attention_mask"] = torch.from_numpy(np.stack(masks))
    return res


def dpo_collate_fn(batch: List[dict], tokenizer=None, training_args=None, max_seq_len: Optional[int] = None,
                   pad_token_id: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """Each example carries a prompt with a chosen and a rejected response, packed into ONE row
    ``prompt + chosen + prompt + rejected`` as two documents (so a single forward scores both), plus
    ``response_indexs`` = [row, chosen start, chosen end, rejected start, rejected end] used by the loss to sum
    log-probabilities (paddleformers/nn/criterion/dpo_loss.py:56-245)."""
    if pad_token_id is None:
        pad_token_id = getattr(tokenizer, "pad_token_id", None) or 0
    rows_ids, rows_lab_c, rows_lab_r, rows_pos, masks, ridx = [], [], [], [], [], []
    if not max_seq_len:
        max_seq_len = max(2 * len(ex["prompt_ids"]) + len(ex["chosen_ids"]) + len(ex["rejected_ids"]) for ex in batch)
    if training_args is not None:
        max_seq_len = calc_padding_size(max_seq_len, training_args)
    for b, ex in enumerate(batch):
        p, c, r = list(ex["prompt_ids"]), list(ex["chosen_ids"]), list(ex["rejected_ids"])
        doc1, doc2 = p + c, p + r
        ids = (doc1 + doc2)[:max_seq_len]
        lab_c = [IGNORE_INDEX] * len(ids)
        lab_r = [IGNORE_INDEX] * len(ids)
        # next-token targets inside each response span
        c0, c1 = len(p) - 1, len(doc1) - 1
        r0, r1 = len(doc1) + len(p) - 1, len(doc1) + len(doc2) - 1
        for t in range(c0, min(c1, len(ids) - 1)):
            lab_c[t] = ids[t + 1]
        for t in range(r0, min(r1, len(ids) - 1)):
            lab_r[t] = ids[t + 1]
        rows_ids.append(_pad(ids, max_seq_len, pad_token_id))
        rows_lab_c.append(_pad(lab_c, max_seq_len, IGNORE_INDEX))
        rows_lab_r.append(_pad(lab_r, max_seq_len, IGNORE_INDEX))
        rows_pos.append(_pad(list(range(len(doc1))) + list(range(len(doc2))), max_seq_len, 0))
        kept = [min(len(doc1), max_seq_len), max(0, min(len(doc2), max_seq_len - len(doc1)))]
        masks.append(gen_attn_mask_startend_row_indices([k for k in kept if k > 0], max_seq_len))
        ridx.append([b, c0, min(c1, max_seq_len), min(r0, max_seq_len), min(r1, max_seq_len)])
    return {
        "input_ids": torch.tensor(rows_ids, dtype=torch.long),
        "chosen_labels": torch.tensor(rows_lab_c, dtype=torch.long),
        "rejected_labels": torch.tensor(rows_lab_r, dtype=torch.long),
        "position_ids": torch.tensor(rows_pos, dtype=torch.long),
        "attn_mask_startend_row_indices": torch.from_numpy(np.stack(masks)),
        "response_indexs": torch.tensor(ridx, dtype=torch.long),
    }


def mm_collate_fn(batch: List[dict], tokenizer=None, training_args=None, max_seq_len: Optional[int] = None, **kw):
    """Multimodal collate: text fields go through ``collate_fn``; per-sample ``pixel_values`` / ``image_grid_thw``
    tensors are concatenated along their first dimension (the layout Qwen2-VL style processors produce)."""
    text = collate_fn([ex["sequences"] for ex in batch], tokenizer, training_args, max_seq_len, **kw)
    for key in ("pixel_values", "image_grid_thw", "pixel_values_videos", "video_grid_thw"):
        vals = [ex[key] for ex in batch if ex.get(key) is not None]
        if vals:
            text[key] = torch.cat([torch.as_tensor(v) for v in vals], dim=0)
    return text
