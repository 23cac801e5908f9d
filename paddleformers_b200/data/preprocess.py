"""Tokenise raw text into the memory-mapped ``.bin`` / ``.idx`` corpus format read by ``GPTDataset``.

    python -m paddleformers_b200.data.preprocess --input corpus.jsonl --tokenizer <dir> --output-prefix data/corpus \\
        [--json-key text] [--append-eos] [--workers 8] [--dtype auto]

Input: a ``.jsonl`` file (one object per line, the text under ``--json-key``) or a ``.txt`` file (one document per line;
with ``--split-sentences`` every line is a sentence and blank lines end documents). Output: ``<prefix>.bin`` (token ids)
and ``<prefix>.idx`` (document and sequence boundaries), the layout of the reference's pre-training data tools
(paddleformers/data/indexed_dataset.py:360 reader; ``create_pretraining_data`` style writers).
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import sys
import time
from typing import Iterator, List

import numpy as np

from .indexed_dataset import MMapIndexedDatasetBuilder

_TOK = None
_ARGS = None


def _init(tokenizer_dir: str, args_dict: dict):
    global _TOK, _ARGS
    from ..transformers.auto import AutoTokenizer

    _TOK = AutoTokenizer.from_pretrained(tokenizer_dir)
    _ARGS = args_dict


def _encode(text: str) -> List[int]:
    ids = _TOK.encode(text, add_special_tokens=False)
    if _ARGS["append_eos"] and _TOK.eos_token_id is not None:
        ids = ids + [_TOK.eos_token_id]
    return ids


def _documents(path: str, key: str) -> Iterator[str]:
    if path.endswith(".jsonl"):
        with open(path, encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if line:
                    text = json.loads(line).get(key)
                    if text:
                        yield text
    else:
        with open(path, encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    yield line.rstrip("\n")


def preprocess(input_path: str, tokenizer_dir: str, output_prefix: str, json_key: str = "text", append_eos: bool = True,
               workers: int = 1, dtype: str = "auto", log_every: int = 10000) -> dict:
    args_dict = {"append_eos": append_eos}
    _init(tokenizer_dir, args_dict)
    vocab = len(_TOK)
    np_dtype = {"auto": np.uint16 if vocab < 65536 else np.int32, "uint16": np.uint16, "int32": np.int32}[dtype]
    os.makedirs(os.path.dirname(os.path.abspath(output_prefix)), exist_ok=True)
    builder = MMapIndexedDatasetBuilder(output_prefix, dtype=np_dtype)
    docs = _documents(input_path, json_key)
    t0, n_docs, n_tok = time.time(), 0, 0
    if workers > 1:
        pool = mp.get_context("spawn").Pool(workers, initializer=_init, initargs=(tokenizer_dir, args_dict))
        stream = pool.imap(_encode, docs, chunksize=64)
    else:
        pool, stream = None, map(_encode, docs)
    for ids in stream:
        if not ids:
            continue
        builder.add_document(np.asarray(ids, dtype=np_dtype))
        n_docs += 1
        n_tok += len(ids)
        if log_every and n_docs % log_every == 0:
            print(f"{n_docs} documents, {n_tok} tokens, {n_tok / max(time.time() - t0, 1e-9):.0f} tokens/s", file=sys.stderr)
    if pool is not None:
        pool.close()
        pool.join()
    builder.finalize()
    return {"documents": n_docs, "tokens": n_tok, "dtype": np.dtype(np_dtype).name, "prefix": output_prefix}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--input", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--output-prefix", required=True)
    ap.add_argument("--json-key", default="text")
    ap.add_argument("--append-eos", action="store_true")
    ap.add_argument("--workers", type=int, default=1)
    ap.add_argument("--dtype", default="auto", choices=["auto", "uint16", "int32"])
    a = ap.parse_args(argv)
    print(json.dumps(preprocess(a.input, a.tokenizer, a.output_prefix, a.json_key, a.append_eos, a.workers, a.dtype)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
