"""Memory-mapped token datasets in the Megatron ``.bin`` / ``.idx`` format and the GPT sample index.

Same on-disk format and index semantics as paddleformers/data/indexed_dataset.py:360 (``MMapIndexedDataset``) and
paddleformers/data/causal_dataset.py:350-523 (``GPTDataset``: document order, sample boundaries that may span
documents, shuffled sample order; blends of several datasets by weight). The sample index is built with vectorised
numpy instead of the reference's compiled ``fast_dataindex`` helper.
"""
from __future__ import annotations

import os
import struct
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.utils.data import Dataset

_HDR_MAGIC = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}
_CODES = {np.dtype(v).name: k for k, v in _DTYPES.items()}


def index_file_path(prefix: str) -> str:
    return prefix + ".idx"


def data_file_path(prefix: str) -> str:
    return prefix + ".bin"


class MMapIndexedDatasetBuilder:
    def __init__(self, prefix: str, dtype=np.int32):
        self.prefix = prefix
        self.dtype = np.dtype(dtype)
        self._bin = open(data_file_path(prefix), "wb")
        self._sizes: List[int] = []
        self._doc_idx: List[int] = [0]

    def add_item(self, tokens) -> None:
        arr = np.asarray(tokens, dtype=self.dtype)
        self._bin.write(arr.tobytes(order="C"))
        self._sizes.append(arr.size)

    def end_document(self) -> None:
        self._doc_idx.append(len(self._sizes))

    def add_document(self, tokens) -> None:
        self.add_item(tokens)
        self.end_document()

    def finalize(self) -> None:
        self._bin.close()
        sizes = np.asarray(self._sizes, dtype=np.int32)
        pointers = np.zeros(len(sizes), dtype=np.int64)
        if len(sizes) > 1:
            np.cumsum(sizes[:-1].astype(np.int64) * self.dtype.itemsize, out=pointers[1:])
        with open(index_file_path(self.prefix), "wb") as f:
            f.write(_HDR_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", _CODES[self.dtype.name]))
            f.write(struct.pack("<Q", len(sizes)))
            f.write(struct.pack("<Q", len(self._doc_idx)))
            f.write(sizes.tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(self._doc_idx, dtype=np.int64).tobytes(order="C"))


class MMapIndexedDataset(Dataset):
    def __init__(self, prefix: str):
        self.prefix = prefix
        with open(index_file_path(prefix), "rb") as f:
            magic = f.read(9)
            if magic != _HDR_MAGIC:
                raise ValueError(f"{index_file_path(prefix)} is not an mmap index file")
            (version,) = struct.unpack("<Q", f.read(8))
            (code,) = struct.unpack("<B", f.read(1))
            (n,) = struct.unpack("<Q", f.read(8))
            (ndoc,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self.dtype = np.dtype(_DTYPES[code])
        idx = np.memmap(index_file_path(prefix), mode="r", order="C")
        self.sizes = np.frombuffer(idx, dtype=np.int32, count=n, offset=offset)
        self.pointers = np.frombuffer(idx, dtype=np.int64, count=n, offset=offset + self.sizes.nbytes)
        self.doc_idx = np.frombuffer(idx, dtype=np.int64, count=ndoc, offset=offset + self.sizes.nbytes + self.pointers.nbytes)
        self._bin = np.memmap(data_file_path(prefix), mode="r", order="C")

    def __len__(self):
        return len(self.sizes)

    def get(self, i: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        size = int(self.sizes[i])
        length = size - offset if length is None else length
        ptr = int(self.pointers[i]) + offset * self.dtype.itemsize
        return np.frombuffer(self._bin, dtype=self.dtype, count=length, offset=ptr)

    def __getitem__(self, i):
        return self.get(i)


_HOST = None


def _host():
    """The compiled index helpers (``csrc_host/data_index.cpp``), built on first use; None if no compiler is there."""
    global _HOST
    if _HOST is None:
        import ctypes

        from ..ops import _build

        try:
            _build.build_host_library()
            lib = _build.load_host_library()
            i64p, i32p, f64p = (ctypes.POINTER(t) for t in (ctypes.c_int64, ctypes.c_int32, ctypes.c_double))
            lib.pfb_build_sample_index.restype = ctypes.c_int64
            lib.pfb_build_sample_index.argtypes = [i32p, i64p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, i64p]
            lib.pfb_build_blend_index.restype = None
            lib.pfb_build_blend_index.argtypes = [f64p, ctypes.c_int32, ctypes.c_int64, i32p, i64p]
            lib.pfb_build_doc_bounds.restype = None
            lib.pfb_build_doc_bounds.argtypes = [i64p, ctypes.c_int64, ctypes.c_int64, i32p, i64p]
            _HOST = lib
        except Exception:  # noqa: BLE001 - no compiler / read-only tree: the numpy paths below are equivalent
            _HOST = False
    return _HOST or None


def _ptr(a: np.ndarray, ctype):
    import ctypes

    return a.ctypes.data_as(ctypes.POINTER(ctype))


def build_sample_index(sizes: np.ndarray, doc_order: np.ndarray, seq_length: int, num_samples: int,
                       use_native: bool = True) -> np.ndarray:
    """sample_idx[k] = (position in doc_order, token offset in that document) where sample k starts; sample k covers
    seq_length + 1 tokens (inputs + shifted labels) and may span documents."""
    lib = _host() if use_native else None
    if lib is not None and len(doc_order) > 0:
        import ctypes

        sz = np.ascontiguousarray(sizes, dtype=np.int32)
        order = np.ascontiguousarray(doc_order, dtype=np.int64)
        out = np.zeros((num_samples + 1, 2), dtype=np.int64)
        n = lib.pfb_build_sample_index(_ptr(sz, ctypes.c_int32), _ptr(order, ctypes.c_int64), len(order), seq_length,
                                       num_samples, _ptr(out, ctypes.c_int64))
        return out[:n + 1]
    lens = sizes[doc_order].astype(np.int64)
    cum = np.concatenate([[0], np.cumsum(lens)])
    total = cum[-1]
    max_samples = int((total - 1) // seq_length)
    n = min(num_samples, max_samples)
    starts = np.arange(n + 1, dtype=np.int64) * seq_length
    doc_pos = np.searchsorted(cum, starts, side="right") - 1
    doc_pos = np.minimum(doc_pos, len(lens) - 1)
    offs = starts - cum[doc_pos]
    return np.stack([doc_pos, offs], axis=1)


class GPTDataset(Dataset):
    """Fixed-length causal-LM samples over a token stream of shuffled documents."""

    def __init__(self, indexed: MMapIndexedDataset, documents: Optional[np.ndarray], num_samples: int, seq_length: int,
                 seed: int = 1234, shuffle: bool = True, eos_token_id: Optional[int] = None, build_masks: bool = False,
                 cache_dir: Optional[str] = None, name: str = "train"):
        self.ds, self.seq_length, self.eos, self.build_masks = indexed, seq_length, eos_token_id, build_masks
        documents = np.arange(len(indexed), dtype=np.int64) if documents is None else np.asarray(documents, dtype=np.int64)
        tokens_per_epoch = int(indexed.sizes[documents].astype(np.int64).sum())
        epochs = max(1, int(np.ceil((num_samples * seq_length + 1) / max(tokens_per_epoch, 1))))
        cache = None
        if cache_dir:
            os.makedirs(cache_dir, exist_ok=True)
            cache = os.path.join(cache_dir, f"{name}_{len(documents)}d_{num_samples}ns_{seq_length}sl_{seed}s.npz")
        if cache and os.path.exists(cache):
            z = np.load(cache)
            self.doc_order, self.sample_idx, self.shuffle_idx = z["doc"], z["sample"], z["shuffle"]
        else:
            rng = np.random.RandomState(seed)
            order = np.tile(documents, epochs)
            if shuffle:
                rng.shuffle(order)
            self.doc_order = order
            self.sample_idx = build_sample_index(indexed.sizes, order, seq_length, num_samples)
            n = len(self.sample_idx) - 1
            self.shuffle_idx = rng.permutation(n) if shuffle else np.arange(n)
            if cache:
                np.savez(cache, doc=self.doc_order, sample=self.sample_idx, shuffle=self.shuffle_idx)

    def __len__(self):
        return len(self.shuffle_idx)

    def _tokens(self, k: int) -> np.ndarray:
        (d0, o0), (d1, o1) = self.sample_idx[k], self.sample_idx[k + 1]
        need = self.seq_length + 1
        parts, got, d, o = [], 0, int(d0), int(o0)
        while got < need and d < len(self.doc_order):
            doc = int(self.doc_order[d])
            take = min(int(self.ds.sizes[doc]) - o, need - got)
            if take > 0:
                parts.append(self.ds.get(doc, o, take))
                got += take
            d, o = d + 1, 0
        out = np.concatenate(parts) if parts else np.zeros(0, dtype=self.ds.dtype)
        if got < need:
            out = np.concatenate([out, np.zeros(need - got, dtype=out.dtype)])
        return out.astype(np.int64)

    def __getitem__(self, i):
        toks = self._tokens(int(self.shuffle_idx[i]))
        item = {"input_ids": torch.from_numpy(toks[:-1].copy()), "labels": torch.from_numpy(toks[1:].copy())}
        if self.build_masks and self.eos is not None:
            # document-causal packing: a document ends after every eos token
            ids = toks[:-1]
            S = len(ids)
            lib = _host()
            if lib is not None:
                import ctypes

                ids_c = np.ascontiguousarray(ids, dtype=np.int64)
                kend, pos = np.empty(S, dtype=np.int32), np.empty(S, dtype=np.int64)
                lib.pfb_build_doc_bounds(_ptr(ids_c, ctypes.c_int64), S, int(self.eos), _ptr(kend, ctypes.c_int32),
                                         _ptr(pos, ctypes.c_int64))
                item["attn_mask_startend_row_indices"] = torch.from_numpy(kend)
                item["position_ids"] = torch.from_numpy(pos)
                return item
            ends = np.nonzero(ids == self.eos)[0] + 1
            bounds = np.concatenate([ends[ends < S], [S]])
            kend = np.empty(S, dtype=np.int32)
            pos = np.empty(S, dtype=np.int64)
            lo = 0
            for e in bounds:
                kend[lo:e] = e
                pos[lo:e] = np.arange(e - lo)
                lo = e
            item["attn_mask_startend_row_indices"] = torch.from_numpy(kend)
            item["position_ids"] = torch.from_numpy(pos)
        return item


class BlendableDataset(Dataset):
    """Weighted mixture of datasets with a deterministic interleaving that keeps each dataset's share close to its
    weight at every prefix (greedy largest-deficit rule)."""

    def __init__(self, datasets: Sequence[Dataset], weights: Sequence[float], size: int, use_native: bool = True):
        w = np.asarray(weights, dtype=np.float64)
        w = np.ascontiguousarray(w / w.sum())
        self.datasets = list(datasets)
        self.dataset_index = np.zeros(size, dtype=np.int32)
        self.sample_index = np.zeros(size, dtype=np.int64)
        lib = _host() if use_native else None
        if lib is not None:
            import ctypes

            lib.pfb_build_blend_index(_ptr(w, ctypes.c_double), len(w), size, _ptr(self.dataset_index, ctypes.c_int32),
                                      _ptr(self.sample_index, ctypes.c_int64))
            return
        counts = np.zeros(len(w), dtype=np.int64)
        for i in range(size):
            deficit = w * (i + 1) - counts
            d = int(np.argmax(deficit))
            self.dataset_index[i] = d
            self.sample_index[i] = counts[d]
            counts[d] += 1

    def __len__(self):
        return len(self.dataset_index)

    def __getitem__(self, i):
        d = int(self.dataset_index[i])
        ds = self.datasets[d]
        return ds[int(self.sample_index[i]) % len(ds)]


def get_train_valid_test_split(split: str, n: int) -> List[Tuple[int, int]]:
    """``"949,50,1"`` -> document index ranges of the three splits."""
    parts = [float(x) for x in split.replace("/", ",").split(",")]
    parts = (parts + [0.0, 0.0])[:3]
    tot = sum(parts)
    bounds, acc = [0], 0.0
    for p in parts:
        acc += p / tot
        bounds.append(int(round(acc * n)))
    bounds[-1] = n
    return [(bounds[i], bounds[i + 1]) for i in range(3)]


def build_train_valid_test_datasets(data_prefix: Sequence[str], split: str, seq_length: int, num_samples: Sequence[int],
                                    seed: int = 1234, eos_token_id: Optional[int] = None, build_masks: bool = False,
                                    cache_dir: Optional[str] = None):
    """``data_prefix`` is either [prefix] or [w1, prefix1, w2, prefix2, ...] like the reference's ``input_dir``."""
    if len(data_prefix) == 1:
        weights, prefixes = [1.0], list(data_prefix)
    else:
        weights = [float(x) for x in data_prefix[0::2]]
        prefixes = list(data_prefix[1::2])
    out = []
    for split_i, name in enumerate(("train", "valid", "test")):
        parts = []
        for w, pre in zip(weights, prefixes):
            ds = MMapIndexedDataset(pre)
            lo, hi = get_train_valid_test_split(split, len(ds))[split_i]
            if hi <= lo or num_samples[split_i] <= 0:
                continue
            share = int(np.ceil(num_samples[split_i] * w / sum(weights) * 1.005))
            parts.append((w, GPTDataset(ds, np.arange(lo, hi), share, seq_length, seed, True, eos_token_id, build_masks,
                                        cache_dir, f"{name}_{os.path.basename(pre)}")))
        if not parts:
            out.append(None)
        elif len(parts) == 1:
            out.append(parts[0][1])
        else:
            out.append(BlendableDataset([p[1] for p in parts], [p[0] for p in parts], num_samples[split_i]))
    return tuple(out)
