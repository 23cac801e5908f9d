"""Preference datasets: {"prompt"/"src", "chosen", "rejected"} or chat ``messages`` + chosen / rejected responses ->
token ids for ``dpo_collate_fn`` (paddleformers/datasets/DPODataset.py role)."""
from __future__ import annotations

from typing import List, Optional

from torch.utils.data import Dataset

from .sft_dataset import read_examples
from .template import get_template


class DPODataset(Dataset):
    def __init__(self, examples: List[dict]):
        self.examples = examples

    def __len__(self):
        return len(self.examples)

    def __getitem__(self, i):
        return self.examples[i]


def create_dpo_dataset(path: str, tokenizer, max_seq_len: int, template: Optional[str] = None) -> DPODataset:
    tpl = get_template(template)
    out = []
    for p in [x.strip() for x in path.split(",") if x.strip()]:
        for ex in read_examples(p):
            if "messages" in ex:
                msgs = ex["messages"]
                chosen, rejected = ex["chosen"], ex["rejected"]
            else:
                prompt = ex.get("prompt", ex.get("src"))
                prompt = prompt[-1] if isinstance(prompt, list) else prompt
                msgs = [{"role": "user", "content": prompt}]
                chosen, rejected = ex.get("chosen", ex.get("response", [None, None])[0] if isinstance(ex.get("response"), list) else None), ex.get("rejected")
                if chosen is None and isinstance(ex.get("response"), list):
                    order = ex.get("sort", [1, 0])
                    chosen = ex["response"][0 if order[0] > order[1] else 1]
                    rejected = ex["response"][1 if order[0] > order[1] else 0]
            if isinstance(chosen, dict):
                chosen = chosen.get("content", "")
            if isinstance(rejected, dict):
                rejected = rejected.get("content", "")
            p_ids, c_ids = tpl.encode_oneturn(tokenizer, msgs + [{"role": "assistant", "content": chosen}])
            _, r_ids = tpl.encode_oneturn(tokenizer, msgs + [{"role": "assistant", "content": rejected}])
            budget = max_seq_len - 2 * len(p_ids)
            if budget < 4:
                continue
            c_ids, r_ids = c_ids[: budget // 2], r_ids[: budget // 2]
            if c_ids and r_ids:
                out.append({"prompt_ids": p_ids, "chosen_ids": c_ids, "rejected_ids": r_ids})
    return DPODataset(out)
