"""Synthetic token datasets for benchmarks and tests: uniform-random ids, optional packed documents with
document-causal mask bounds."""
from __future__ import annotations

from typing import Dict, Optional

import torch
from torch.utils.data import Dataset


class SyntheticCausalLMDataset(Dataset):
    """``num_samples`` sequences of ``seq_len`` uniform-random token ids; labels are the ids shifted by one.

    With ``doc_len_range=(lo, hi)`` each sequence is a pack of documents with random lengths in [lo, hi]: position ids
    restart per document, ``attn_mask_startend_row_indices`` holds for every key position the end of its document
    (FlashMask start row, paddleformers/datasets/collate.py:1185-1215) and the label at each document's last token
    is ignored."""

    def __init__(self, vocab_size: int, seq_len: int, num_samples: int, seed: int = 0,
                 doc_len_range: Optional[tuple] = None, ignore_index: int = -100):
        self.vocab_size, self.seq_len, self.num_samples, self.seed = vocab_size, seq_len, num_samples, seed
        self.doc_len_range = doc_len_range
        self.ignore_index = ignore_index

    def __len__(self):
        return self.num_samples

    def __getitem__(self, i: int) -> Dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(self.seed * 1000003 + i)
        toks = torch.randint(0, self.vocab_size, (self.seq_len + 1,), generator=g)
        item = {"input_ids": toks[:-1].clone(), "labels": toks[1:].clone()}
        if self.doc_len_range is not None:
            lo, hi = self.doc_len_range
            S = self.seq_len
            kend = torch.empty(S, dtype=torch.int32)
            pos = torch.empty(S, dtype=torch.int64)
            p = 0
            while p < S:
                ln = int(torch.randint(lo, hi + 1, (1,), generator=g))
                e = min(S, p + ln)
                kend[p:e] = e
                pos[p:e] = torch.arange(e - p)
                item["labels"][e - 1] = self.ignore_index
                p = e
            item["attn_mask_startend_row_indices"] = kend
            item["position_ids"] = pos
        return item
