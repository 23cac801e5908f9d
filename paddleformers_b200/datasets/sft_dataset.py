"""Online SFT / pretraining dataflow: readers, multi-source mixing, tokenisation, packing.

Roles of paddleformers/datasets/SFTDataset.py (``BaseSFTDataset`` :65, ``_generate_sequences`` :340, ``MapSFTDataset``
:1000) and paddleformers/datasets/loader.py:21 (``create_dataset``): examples come from jsonl / json / csv / parquet /
txt files in "messages" (chat), "erniekit" (src / tgt lists), alpaca or plain-text schemas, several sources are mixed
by concatenation, random sampling with probabilities or interleaving, every example becomes a ``Sequence`` (token ids,
labels with the prompt masked, position ids) and sequences are packed up to ``max_seq_len`` with one of three
strategies: truncate (no packing), greedy (first come first packed) or bin packing (first-fit decreasing over a
look-ahead window).
"""
from __future__ import annotations

import csv
import json
import os
import random
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, Iterator, List, Optional, Sequence as Seq

import torch
from torch.utils.data import Dataset, IterableDataset

from .template import Template, get_template

IGNORE_INDEX = -100


@dataclass
class Sequence:
    token_ids: List[int]
    labels: List[int]
    position_ids: List[int]
    source: str = ""

    def __len__(self):
        return len(self.token_ids)


# ---------------------------------------------------------------------------------------------------------------
# readers
# ---------------------------------------------------------------------------------------------------------------
def read_examples(path: str) -> Iterator[dict]:
    ext = os.path.splitext(path)[1].lower()
    if ext == ".jsonl":
        with open(path, encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if line:
                    yield json.loads(line)
    elif ext == ".json":
        with open(path, encoding="utf-8") as f:
            data = json.load(f)
        for ex in (data if isinstance(data, list) else data.get("data", [])):
            yield ex
    elif ext == ".csv":
        with open(path, newline="", encoding="utf-8") as f:
            for row in csv.DictReader(f):
                yield dict(row)
    elif ext == ".parquet":
        import pyarrow.parquet as pq

        for row in pq.read_table(path).to_pylist():
            yield row
    elif ext == ".txt":
        with open(path, encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    yield {"text": line.rstrip("\n")}
    else:
        raise ValueError(f"unsupported dataset file type: {path}")


def to_messages(ex: dict) -> Dict[str, Any]:
    """Normalise the supported schemas to {"messages": [...], "system": str|None, "tools": [...]|None, "text": str|None}."""
    if "messages" in ex:
        return {"messages": ex["messages"], "system": ex.get("system"), "tools": ex.get("tools"), "text": None}
    if "conversations" in ex:  # sharegpt
        role_map = {"human": "user", "gpt": "assistant", "system": "system", "function_call": "function", "observation": "observation"}
        msgs = [{"role": role_map.get(m.get("from"), m.get("from")), "content": m.get("value", "")} for m in ex["conversations"]]
        tools = ex.get("tools")
        if isinstance(tools, str) and tools:
            tools = json.loads(tools)
        return {"messages": msgs, "system": ex.get("system"), "tools": tools, "text": None}
    if "src" in ex and "tgt" in ex:  # erniekit
        src, tgt = ex["src"], ex["tgt"]
        src = [src] if isinstance(src, str) else src
        tgt = [tgt] if isinstance(tgt, str) else tgt
        msgs = []
        for s, t in zip(src, tgt):
            msgs += [{"role": "user", "content": s}, {"role": "assistant", "content": t}]
        return {"messages": msgs, "system": ex.get("system"), "tools": None, "text": None}
    if "instruction" in ex:  # alpaca
        q = ex["instruction"] + ("\n" + ex["input"] if ex.get("input") else "")
        return {"messages": [{"role": "user", "content": q}, {"role": "assistant", "content": ex.get("output", "")}],
                "system": ex.get("system"), "tools": None, "text": None}
    if "prompt" in ex and ("response" in ex or "completion" in ex):
        return {"messages": [{"role": "user", "content": ex["prompt"]},
                             {"role": "assistant", "content": ex.get("response", ex.get("completion", ""))}],
                "system": None, "tools": None, "text": None}
    if "text" in ex:
        return {"messages": None, "system": None, "tools": None, "text": ex["text"]}
    raise ValueError(f"unrecognised example schema with keys {sorted(ex)}")


# ---------------------------------------------------------------------------------------------------------------
# tokenisation
# ---------------------------------------------------------------------------------------------------------------
def encode_example(ex: dict, tokenizer, template: Template, max_seq_len: int, train_on_prompt: bool = False,
                   source: str = "") -> Optional[Sequence]:
    """Labels are next-token targets aligned with the inputs (already shifted): label[t] = token[t+1] where that token
    belongs to a trained span, IGNORE_INDEX elsewhere."""
    norm = to_messages(ex)
    if norm["text"] is not None:
        ids = tokenizer.encode(norm["text"], add_special_tokens=False)
        if tokenizer.eos_token_id is not None:
            ids = ids + [tokenizer.eos_token_id]
        mask = [1] * len(ids)
    else:
        ids, mask = [], []
        for p_ids, r_ids in template.encode_multiturn(tokenizer, norm["messages"], norm["system"], norm["tools"]):
            ids += p_ids
            mask += [1 if train_on_prompt else 0] * len(p_ids)
            ids += r_ids
            mask += [1] * len(r_ids)
    if len(ids) < 2:
        return None
    ids, mask = ids[: max_seq_len + 1], mask[: max_seq_len + 1]
    inputs = ids[:-1]
    labels = [t if m else IGNORE_INDEX for t, m in zip(ids[1:], mask[1:])]
    if all(l == IGNORE_INDEX for l in labels):
        return None
    return Sequence(inputs, labels, list(range(len(inputs))), source)


# ---------------------------------------------------------------------------------------------------------------
# packing
# ---------------------------------------------------------------------------------------------------------------
def pack_greedy(seqs: Iterable[Sequence], max_seq_len: int) -> Iterator[List[Sequence]]:
    cur, cur_len = [], 0
    for s in seqs:
        if cur and cur_len + len(s) > max_seq_len:
            yield cur
            cur, cur_len = [], 0
        cur.append(s)
        cur_len += len(s)
    if cur:
        yield cur


def pack_binpacking(seqs: Iterable[Sequence], max_seq_len: int, window: int = 512) -> Iterator[List[Sequence]]:
    """First-fit decreasing over windows of ``window`` sequences (the reference uses the ``binpacking`` package for the
    same purpose)."""
    buf: List[Sequence] = []

    def flush(items):
        bins: List[List[Sequence]] = []
        space: List[int] = []
        for s in sorted(items, key=len, reverse=True):
            for i, free in enumerate(space):
                if len(s) <= free:
                    bins[i].append(s)
                    space[i] -= len(s)
                    break
            else:
                bins.append([s])
                space.append(max_seq_len - len(s))
        return bins

    for s in seqs:
        buf.append(s)
        if len(buf) >= window:
            yield from flush(buf)
            buf = []
    if buf:
        yield from flush(buf)


def pack_sequences(seqs: Iterable[Sequence], max_seq_len: int, strategy: str = "greedy", window: int = 512):
    if strategy in ("truncate", "none", None):
        return ([s] for s in seqs)
    if strategy == "greedy":
        return pack_greedy(seqs, max_seq_len)
    if strategy in ("binpacking", "bin_packing"):
        return pack_binpacking(seqs, max_seq_len, window)
    raise ValueError(f"unknown packing strategy {strategy!r}")


# ---------------------------------------------------------------------------------------------------------------
# datasets
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class DataSource:
    path: str
    prob: float = 1.0
    template: Optional[str] = None
    name: str = ""


class IterableSFTDataset(IterableDataset):
    """Streams packed samples (lists of ``Sequence``); mixes sources by ``mix_strategy``."""

    def __init__(self, sources: Seq[DataSource], tokenizer, max_seq_len: int, template: Optional[str] = None,
                 packing: str = "greedy", mix_strategy: str = "concat", seed: int = 0, train_on_prompt: bool = False,
                 num_epochs: int = 1, shuffle: bool = False):
        self.sources, self.tokenizer, self.max_seq_len = list(sources), tokenizer, max_seq_len
        self.template_name, self.packing, self.mix, self.seed = template, packing, mix_strategy, seed
        self.train_on_prompt, self.num_epochs, self.shuffle = train_on_prompt, num_epochs, shuffle
        self.epoch = 0

    def set_epoch(self, epoch):
        self.epoch = epoch

    def _source_iter(self, src: DataSource) -> Iterator[Sequence]:
        tpl = get_template(src.template or self.template_name)
        for ex in read_examples(src.path):
            s = encode_example(ex, self.tokenizer, tpl, self.max_seq_len, self.train_on_prompt, src.name or src.path)
            if s is not None:
                yield s

    def _mixed(self) -> Iterator[Sequence]:
        rng = random.Random(self.seed + self.epoch)
        if self.mix == "concat" or len(self.sources) == 1:
            for src in self.sources:
                yield from self._source_iter(src)
            return
        iters = [self._source_iter(s) for s in self.sources]
        alive = list(range(len(iters)))
        if self.mix == "interleave":
            while alive:
                for i in list(alive):
                    try:
                        yield next(iters[i])
                    except StopIteration:
                        alive.remove(i)
            return
        if self.mix == "random":
            probs = [s.prob for s in self.sources]
            while alive:
                i = rng.choices(alive, weights=[probs[a] for a in alive])[0]
                try:
                    yield next(iters[i])
                except StopIteration:
                    alive.remove(i)
            return
        raise ValueError(f"unknown mix strategy {self.mix!r}")

    def __iter__(self):
        for _ in range(self.num_epochs):
            yield from pack_sequences(self._mixed(), self.max_seq_len, self.packing)
            self.epoch += 1


class MapSFTDataset(Dataset):
    """Materialised (tokenised and packed once) version of the same dataflow, addressable by index."""

    def __init__(self, *args, **kw):
        it = IterableSFTDataset(*args, **kw)
        self.samples: List[List[Sequence]] = list(iter(it))
        if kw.get("shuffle"):
            random.Random(kw.get("seed", 0)).shuffle(self.samples)

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i):
        return self.samples[i]


def create_dataset(dataset_path: str, tokenizer, max_seq_len: int, dataset_prob: Optional[str] = None,
                   template: Optional[str] = None, packing: str = "greedy", mix_strategy: str = "concat",
                   streaming: bool = False, **kw):
    """``dataset_path`` and ``dataset_prob`` are comma-separated lists, as in the reference's YAML configs."""
    paths = [p.strip() for p in dataset_path.split(",") if p.strip()]
    probs = [float(x) for x in dataset_prob.split(",")] if dataset_prob else [1.0] * len(paths)
    if len(probs) != len(paths):
        raise ValueError("dataset_prob must have one entry per dataset_path")
    sources = [DataSource(p, pr, name=os.path.basename(p)) for p, pr in zip(paths, probs)]
    cls = IterableSFTDataset if streaming else MapSFTDataset
    return cls(sources, tokenizer, max_seq_len, template=template, packing=packing, mix_strategy=mix_strategy, **kw)
