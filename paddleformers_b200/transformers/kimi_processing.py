"""Kimi-K2.5 inputs: the native-resolution image / video-chunk processor, the tiktoken-based tokenizer and the processor that
joins them (the jobs of paddleformers/transformers/kimi_k25/{vision_processor,media_utils,tokenizer,processor}.py; the
reference has this family's processors and no model, and so does this package). Videos come in as decoded frames
[frames, H, W, 3] with their frame rate: no video decoder is bundled."""
from __future__ import annotations

import base64
import json
import math
import os
from datetime import datetime, timezone
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from .image_processing import _resize
from .tool_declaration import sort_keys_deep, tools_to_typescript

DEFAULT_MEDIA_CONFIG = dict(patch_size=14, merge_kernel_size=2, temporal_merge_kernel_size=4, in_patch_limit=16384,
                            in_patch_limit_each_frame=4096, in_patch_limit_video=None, patch_limit_on_one_side=512,
                            fixed_output_tokens=None, sample_fps=2.0, max_num_frames_each_video=None,
                            timestamp_mode="hh:mm:ss.fff", image_mean=(0.5, 0.5, 0.5), image_std=(0.5, 0.5, 0.5))


def timestamp_text(seconds: float, mode: str = "hh:mm:ss.fff") -> str:
    clock = datetime.fromtimestamp(seconds, tz=timezone.utc)
    millis = f".{int((seconds % 1) * 1000):03d}"
    if mode == "hh:mm:ss.fff":
        return clock.strftime("%H:%M:%S") + millis
    if mode == "mm:ss.fff":
        return clock.strftime("%M:%S") + millis
    if mode == "mm:ss":
        return clock.strftime("%M:%S")
    raise ValueError(f"unknown timestamp mode: {mode}")


def native_resolution_geometry(width: int, height: int, patch_size: int, merge: int, patch_limit: int, side_limit: int,
                               fixed_tokens: Optional[int] = None) -> Dict[str, int]:
    """Size an image keeps in a native-resolution (NaViT-style) tower: it is only ever shrunk, so that the patch count stays
    within ``patch_limit`` and neither side exceeds ``side_limit`` patches, then padded at the right / bottom to a multiple of
    ``patch_size * merge``. ``num_tokens`` is the row count after the merge."""
    shrink = min(1.0, math.sqrt(patch_limit / (max(1.0, width // patch_size) * max(1.0, height // patch_size))),
                 side_limit * patch_size / width, side_limit * patch_size / height)
    new_w = min(max(1, int(width * shrink)), side_limit * patch_size)
    new_h = min(max(1, int(height * shrink)), side_limit * patch_size)
    block = merge * patch_size
    pad_w, pad_h = -new_w % block, -new_h % block
    rows, cols = (new_h + pad_h) // block, (new_w + pad_w) // block
    if fixed_tokens is None and max(rows, cols) * merge > side_limit:
        raise ValueError(f"{rows} x {cols} merged patches exceed the limit of {side_limit} patches on one side")
    return {"num_tokens": rows * cols if fixed_tokens is None else fixed_tokens, "new_width": new_w, "new_height": new_h,
            "pad_width": pad_w, "pad_height": pad_h, "sampled_nframes": 1}


def patchify(pixels: torch.Tensor, patch_size: int):
    """[B, T, C, H, W] -> (patches [B * T * H/P * W/P, C, P, P] in frame, row, column order, grid [B, 3] = (T, H/P, W/P))."""
    B, T, C, H, W = pixels.shape
    x = pixels.reshape(B * T, C, H // patch_size, patch_size, W // patch_size, patch_size).permute(0, 2, 4, 1, 3, 5)
    return x.reshape(-1, C, patch_size, patch_size), torch.tensor([[T, H // patch_size, W // patch_size]] * B)


class KimiVisionProcessor:
    """``preprocess(medias)``: ``{"type": "image", "image": uint8 [H, W, 3] or PIL}`` and ``{"type": "video_chunk",
    "video_chunk": uint8 [T, H, W, 3]}`` items -> ``pixel_values`` [patches, 3, P, P] and ``grid_thws`` [items, 3]."""

    def __init__(self, media_proc_cfg: Optional[dict] = None):
        self.cfg = {**DEFAULT_MEDIA_CONFIG, **(media_proc_cfg or {})}
        self.frames_per_chunk = self.cfg["temporal_merge_kernel_size"]

    @classmethod
    def from_pretrained(cls, path: str):
        with open(os.path.join(path, "preprocessor_config.json")) as f:
            return cls(json.load(f).get("media_proc_cfg"))

    def save_pretrained(self, path: str):
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "preprocessor_config.json"), "w") as f:
            json.dump({"image_processor_type": "KimiK25VisionProcessor", "media_proc_cfg": self.cfg}, f, indent=1, sort_keys=True)

    @staticmethod
    def chunk_prompt(stamp: str) -> str:
        return f"{stamp}<|media_begin|>video<|media_content|><|media_pad|><|media_end|>"

    def split_video_chunks(self, frames: np.ndarray, fps: float) -> List[dict]:
        """Sample the clip at ``sample_fps`` (a whole number of chunks, at least none), cut it into chunks of
        ``temporal_merge_kernel_size`` frames and give every chunk a prompt that opens with its start time."""
        c, total = self.cfg, len(frames)
        rate = min(c["sample_fps"], fps)
        k = self.frames_per_chunk
        n = max(round(total * rate / fps), 1) // k * k
        picks = np.linspace(0, total - 1, n).round().astype(int)
        return [{"type": "video_chunk", "video_chunk": np.asarray(frames)[picks[i:i + k]],
                 "prompt": self.chunk_prompt(timestamp_text(picks[i] / float(fps), c["timestamp_mode"]))} for i in range(0, n, k)]

    def geometry(self, media: dict) -> Dict[str, int]:
        c = self.cfg
        if media["type"] == "image":
            h, w = np.asarray(media["image"]).shape[:2]
            return native_resolution_geometry(w, h, c["patch_size"], c["merge_kernel_size"], c["in_patch_limit"],
                                              c["patch_limit_on_one_side"], c["fixed_output_tokens"])
        if media["type"] == "video_chunk":
            frames = np.asarray(media["video_chunk"])
            per_frame = c["in_patch_limit_each_frame"] or c["in_patch_limit"]
            if c["in_patch_limit_video"] is not None:               # a chunk's frames share the clip budget
                per_frame = min(round(c["in_patch_limit_video"] / len(frames)), per_frame)
            g = native_resolution_geometry(frames.shape[2], frames.shape[1], c["patch_size"], c["merge_kernel_size"], per_frame,
                                           c["patch_limit_on_one_side"], c["fixed_output_tokens"])
            g["sampled_nframes"] = len(frames)
            return g
        raise ValueError(f"unsupported media type: {media['type']}")

    get_resize_config = geometry

    def media_tokens(self, media: dict) -> int:
        return self.geometry(media)["num_tokens"]

    def preprocess(self, medias: Sequence[dict]) -> Dict[str, torch.Tensor]:
        medias = [medias] if isinstance(medias, dict) else list(medias)
        if not medias:
            return {}
        c = self.cfg
        mean, std = (torch.tensor(c[k], dtype=torch.float32).view(1, 3, 1, 1) for k in ("image_mean", "image_std"))
        patches, grids = [], []
        for item in medias:
            g = self.geometry(item)
            frames = np.asarray(item["image"])[None] if item["type"] == "image" else np.asarray(item["video_chunk"])
            sized = np.stack([_resize(np.ascontiguousarray(f), g["new_height"], g["new_width"]) for f in frames])
            sized = np.pad(sized, ((0, 0), (0, g["pad_height"]), (0, g["pad_width"]), (0, 0)))
            x = (torch.from_numpy(sized).permute(0, 3, 1, 2).float() / 255.0 - mean) / std
            p, grid = patchify(x[None], c["patch_size"])
            patches.append(p)
            grids.append(grid)
        return {"pixel_values": torch.cat(patches), "grid_thws": torch.cat(grids)}

    __call__ = preprocess


class TikTokenTokenizer:
    """Byte-pair tokenizer over a tiktoken rank file (one ``base64(token bytes) rank`` pair per line) with 256 special-token
    slots after the base vocabulary; ``special_tokens`` names some of them (id -> text), the rest read
    ``<|reserved_token_{id}|>``. Special-token text inside a prompt encodes to its id. ``apply_chat_template`` renders the
    Jinja template with ``tools_ts_str``, the tools in TypeScript-like notation."""

    num_reserved_special_tokens = 256
    pat_str = "|".join([
        r"""[\p{Han}]+""",
        r"""[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]*[\p{Ll}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?""",
        r"""[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]+[\p{Ll}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?""",
        r"""\p{N}{1,3}""",
        r""" ?[^\s\p{L}\p{N}]+[\r\n]*""",
        r"""\s*[\r\n]+""",
        r"""\s+(?!\S)""",
        r"""\s+""",
    ])
    MAX_ENCODE_CHARS, MAX_RUN_CHARS = 400_000, 25_000          # tiktoken's limits on one call / one run without a break

    def __init__(self, vocab_file: str, special_tokens: Optional[Dict[int, str]] = None, bos_token: str = "[BOS]",
                 eos_token: str = "[EOS]", pad_token: Optional[str] = None, unk_token: Optional[str] = None,
                 chat_template: Optional[str] = None):
        import tiktoken

        self.vocab_file = vocab_file
        with open(vocab_file, "rb") as f:
            ranks = {base64.b64decode(tok): int(rank) for tok, rank in (line.split() for line in f.read().splitlines() if line)}
        base = len(ranks)
        named = {int(k): v for k, v in (special_tokens or {}).items()}
        self.special_tokens = {named.get(i, f"<|reserved_token_{i}|>"): i for i in range(base, base + self.num_reserved_special_tokens)}
        self.model = tiktoken.Encoding(name=os.path.basename(vocab_file), pat_str=self.pat_str, mergeable_ranks=ranks,
                                       special_tokens=self.special_tokens)
        self.named_special_tokens = named
        self.bos_token, self.eos_token, self.pad_token, self.unk_token = bos_token, eos_token, pad_token, unk_token
        self.bos_token_id, self.eos_token_id = self.special_tokens[bos_token], self.special_tokens[eos_token]
        self.pad_token_id = self.special_tokens[pad_token] if pad_token else None
        self.unk_token_id = self.special_tokens[unk_token] if unk_token else None
        self.chat_template = chat_template

    @property
    def vocab_size(self) -> int:
        return self.model.n_vocab

    def get_vocab(self) -> Dict[str, int]:
        out = {self.model.decode_single_token_bytes(i).decode("latin-1"): i for i in range(self.vocab_size - len(self.special_tokens))}
        out.update(self.special_tokens)
        return out

    @staticmethod
    def _bounded_runs(s: str, limit: int):
        """Pieces of ``s`` in which no run of whitespace, or of anything else, is longer than ``limit``."""
        start, run, space = 0, 0, s[:1].isspace()
        for i, ch in enumerate(s):
            if ch.isspace() != space:
                run, space = 1, not space
            else:
                run += 1
                if run > limit:
                    yield s[start:i]
                    start, run = i, 1
        yield s[start:]

    def encode(self, text: str, allow_special_tokens: bool = True, add_special_tokens: bool = False) -> List[int]:
        ids: List[int] = []
        for lo in range(0, max(len(text), 1), self.MAX_ENCODE_CHARS):
            for piece in self._bounded_runs(text[lo:lo + self.MAX_ENCODE_CHARS], self.MAX_RUN_CHARS):
                ids.extend(self.model.encode(piece, allowed_special="all") if allow_special_tokens
                           else self.model.encode(piece, disallowed_special=()))
        return ids

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        ids = [int(ids)] if isinstance(ids, (int, np.integer)) else [int(i) for i in ids]
        if skip_special_tokens:
            first = self.vocab_size - len(self.special_tokens)
            ids = [i for i in ids if i < first]
        return self.model.decode(ids)

    def batch_decode(self, sequences, skip_special_tokens: bool = False) -> List[str]:
        return [self.decode(s, skip_special_tokens) for s in sequences]

    def __call__(self, text, add_special_tokens: bool = False) -> Dict[str, torch.Tensor]:
        ids = self.encode(text)
        return {"input_ids": torch.tensor([ids]), "attention_mask": torch.ones(1, len(ids), dtype=torch.long)}

    def apply_chat_template(self, conversation, tools: Optional[List[dict]] = None, tokenize: bool = False,
                            add_generation_prompt: bool = True, thinking: bool = True, **kw):
        if not self.chat_template:
            raise ValueError("this tokenizer has no chat template")
        from jinja2.sandbox import ImmutableSandboxedEnvironment

        tools = sort_keys_deep(tools)
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.filters["tojson"] = lambda x, **k: json.dumps(x, ensure_ascii=False, **k)
        text = env.from_string(self.chat_template).render(
            messages=conversation, tools=tools, tools_ts_str=tools_to_typescript(tools) if tools else None,
            add_generation_prompt=add_generation_prompt, thinking=thinking, bos_token=self.bos_token, eos_token=self.eos_token, **kw)
        return self.encode(text) if tokenize else text

    def save_pretrained(self, path: str):
        os.makedirs(path, exist_ok=True)
        target = os.path.join(path, "tiktoken.model")
        if os.path.abspath(target) != os.path.abspath(self.vocab_file):
            with open(self.vocab_file, "rb") as src, open(target, "wb") as dst:
                dst.write(src.read())
        with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
            json.dump({"tokenizer_class": "TikTokenTokenizer", "bos_token": self.bos_token, "eos_token": self.eos_token,
                       "pad_token": self.pad_token, "unk_token": self.unk_token, "chat_template": self.chat_template,
                       "added_tokens_decoder": {str(i): {"content": t} for i, t in sorted(self.named_special_tokens.items())}},
                      f, indent=1, ensure_ascii=False)

    @classmethod
    def from_pretrained(cls, path: str):
        with open(os.path.join(path, "tokenizer_config.json")) as f:
            c = json.load(f)
        named = {int(i): (t["content"] if isinstance(t, dict) else t) for i, t in (c.get("added_tokens_decoder") or {}).items()}
        template = c.get("chat_template")
        jinja = os.path.join(path, "chat_template.jinja")
        if template is None and os.path.isfile(jinja):
            with open(jinja) as f:
                template = f.read()
        text = lambda t: t["content"] if isinstance(t, dict) else t
        return cls(os.path.join(path, "tiktoken.model"), named, text(c.get("bos_token") or "[BOS]"), text(c.get("eos_token") or "[EOS]"),
                   text(c.get("pad_token")), text(c.get("unk_token")), template)


class KimiProcessor:
    """``processor(messages=...)`` or ``processor(text=..., medias=...)`` -> ``input_ids``, ``attention_mask``,
    ``pixel_values``, ``grid_thws``. A video (``{"type": "video", "video": frames, "fps": f}``) becomes a run of chunk items,
    and the ``video_placeholder`` that stands for it in the text becomes the chunks' prompts. Each image or chunk keeps ONE
    ``<|media_pad|>`` in the text: the model repeats it per feature row."""

    video_placeholder = "<|kimi_k25_video_placeholder|>"
    model_input_names = ["input_ids", "attention_mask", "pixel_values", "grid_thws"]

    def __init__(self, image_processor: KimiVisionProcessor, tokenizer):
        self.image_processor = self.media_processor = image_processor
        self.tokenizer = tokenizer

    @classmethod
    def from_pretrained(cls, path: str):
        return cls(KimiVisionProcessor.from_pretrained(path), TikTokenTokenizer.from_pretrained(path))

    def save_pretrained(self, path: str):
        self.image_processor.save_pretrained(path)
        self.tokenizer.save_pretrained(path)

    def expand_videos(self, medias: Sequence[dict]):
        items, prompts = [], []
        for m in medias:
            if m["type"] == "image":
                items.append(m)
            elif m["type"] == "video":
                chunks = self.media_processor.split_video_chunks(m["video"], m.get("fps", 1.0))
                items.extend(chunks)
                prompts.append("".join(c["prompt"] for c in chunks))
            else:
                raise ValueError(f"unsupported media type: {m['type']}")
        return items, prompts

    def insert_video_prompts(self, text: str, prompts: Sequence[str]) -> str:
        parts = text.split(self.video_placeholder)
        if len(parts) == 1:
            return text
        if len(parts) != len(prompts) + 1:
            raise ValueError(f"{len(parts) - 1} video placeholders in the text for {len(prompts)} videos")
        return "".join(a + b for a, b in zip(parts, list(prompts) + [""]))

    @staticmethod
    def medias_of(messages: Sequence[dict]) -> List[dict]:
        out = []
        for msg in messages:
            if msg.get("role") != "user" or not isinstance(msg.get("content"), list):
                continue
            for part in msg["content"]:
                kind = part.get("type") if isinstance(part, dict) else None
                if kind in ("video", "video_url"):
                    src = part["video_url"]
                    out.append({"type": "video", "video": src["url"] if isinstance(src, dict) else src, "fps": part.get("fps", 1.0)})
                elif kind in ("image", "image_url"):
                    out.append({"type": "image", "image": part["image_url"]})
        return out

    def __call__(self, messages: Optional[List[dict]] = None, medias: Optional[List[dict]] = None, text: Optional[str] = None,
                 **template_kwargs) -> Dict[str, Any]:
        if messages is None and (medias is None or text is None):
            raise ValueError("give either `messages` or both `medias` and `text`")
        if medias is None:
            medias = self.medias_of(messages)
        items, prompts = self.expand_videos(medias)
        if text is None:
            text = self.tokenizer.apply_chat_template(messages, **template_kwargs)
        text = self.insert_video_prompts(text, prompts)
        return {**self.tokenizer(text, add_special_tokens=False), **self.media_processor.preprocess(items)}

    def apply_chat_template(self, messages, **kw):
        return self.tokenizer.apply_chat_template(messages, **kw)

    def decode(self, *a, **kw):
        return self.tokenizer.decode(*a, **kw)

    def batch_decode(self, *a, **kw):
        return self.tokenizer.batch_decode(*a, **kw)
