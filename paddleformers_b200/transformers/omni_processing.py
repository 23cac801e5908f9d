"""Prompt assembly for Qwen3-Omni: text with image, video and audio tags -> token ids plus the pixel / mel inputs, every tag
repeated once per feature row its input will occupy (the job of paddleformers/transformers/qwen3_omni_moe/processor.py; the
reference has this family's processor and no model, and so does this package). With ``use_audio_in_video`` the audio rows of
a clip's sound track are interleaved with its video rows by time stamp."""
from __future__ import annotations

import re
from typing import List, Optional, Sequence

import numpy as np
import torch

from .audio_processing import LogMelFeatureExtractor
from .image_processing import Qwen2VLImageProcessor, Qwen2VLVideoProcessor


def audio_encoder_output_lengths(frames):
    """Rows the audio encoder returns for ``frames`` mel frames: the encoder works on windows of 100 frames, each of which
    three stride-2 convolutions turn into 13 rows; the ragged last window shrinks by the same three halvings."""
    frames = np.asarray(frames, dtype=np.int64)
    tail = frames % 100
    rows = (tail - 1) // 2 + 1
    rows = ((rows - 1) // 2 + 1 - 1) // 2 + 1
    return rows + (frames // 100) * 13


def interleave_by_time(video_times: np.ndarray, audio_rows: int) -> List[bool]:
    """Merge order of a clip's video rows (time stamp ``video_times[i]``, non-decreasing, in audio-row units) and its
    ``audio_rows`` audio rows (time stamp = row index): True = next video row, False = next audio row. A video row goes first
    when the stamps are equal."""
    order, v, a = [], 0, 0
    while v < len(video_times) and a < audio_rows:
        if video_times[v] <= a:
            order.append(True)
            v += 1
        else:
            order.append(False)
            a += 1
    return order + [True] * (len(video_times) - v) + [False] * (audio_rows - a)


class Qwen3OmniProcessor:
    """``processor(text, images=, videos=, audio=)`` -> ``input_ids``, ``attention_mask`` and the modality inputs
    (``pixel_values`` + ``image_grid_thw``, ``pixel_values_videos`` + ``video_grid_thw`` + ``video_second_per_grid``,
    ``input_features`` + ``feature_attention_mask``). ``tokenizer`` needs ``encode`` and must know the tag strings."""

    def __init__(self, tokenizer, image_processor=None, video_processor=None, feature_extractor=None,
                 image_token: str = "<|image_pad|>", video_token: str = "<|video_pad|>", audio_token: str = "<|audio_pad|>",
                 vision_bos_token: str = "<|vision_start|>", vision_eos_token: str = "<|vision_end|>",
                 audio_bos_token: str = "<|audio_start|>", audio_eos_token: str = "<|audio_end|>",
                 position_id_per_seconds: float = 13.0):
        self.tokenizer = tokenizer
        self.image_processor = image_processor or Qwen2VLImageProcessor(patch_size=16)
        self.video_processor = video_processor or Qwen2VLVideoProcessor(patch_size=16)
        self.feature_extractor = feature_extractor or LogMelFeatureExtractor(feature_size=128)
        self.image_token, self.video_token, self.audio_token = image_token, video_token, audio_token
        self.vision_bos_token, self.vision_eos_token = vision_bos_token, vision_eos_token
        self.audio_bos_token, self.audio_eos_token = audio_bos_token, audio_eos_token
        self.position_id_per_seconds = position_id_per_seconds

    def expand_tags(self, text: str, audio_lengths: Sequence[int], image_grids, video_grids, video_second_per_grid: Sequence[float],
                    use_audio_in_video: bool = False) -> str:
        """One prompt with every tag repeated for its input. Inputs are consumed in prompt order per kind; with
        ``use_audio_in_video`` a video tag (wrapped in the vision begin / end tags) takes the next audio length too and becomes
        ``vision-begin audio-begin <rows merged by time> audio-end vision-end``."""
        audio, images, videos, seconds = iter(audio_lengths), iter(image_grids), iter(video_grids), iter(video_second_per_grid)
        m_img, m_vid = self.image_processor.merge_size ** 2, self.video_processor.merge_size ** 2
        tags = "|".join(re.escape(t) for t in (self.audio_token, self.image_token, self.video_token))
        wrapped = re.escape(self.vision_bos_token + self.video_token + self.vision_eos_token)
        pattern = re.compile(f"{wrapped}|{tags}" if use_audio_in_video else tags)

        def one(match):
            tag = match.group()
            if tag == self.audio_token:
                return self.audio_token * int(next(audio))
            if tag == self.image_token:
                return self.image_token * (int(np.prod(np.asarray(next(images)))) // m_img)
            if not use_audio_in_video:
                return self.video_token * (int(np.prod(np.asarray(next(videos)))) // m_vid)
            if tag == self.video_token:
                raise ValueError("with use_audio_in_video every video tag must be wrapped in the vision begin / end tags")
            t, h, w = (int(v) for v in np.asarray(next(videos)))
            m = self.video_processor.merge_size
            times = np.repeat(np.arange(t), (h // m) * (w // m)) * next(seconds) * self.position_id_per_seconds
            rows = "".join(self.video_token if is_video else self.audio_token for is_video in interleave_by_time(times, int(next(audio))))
            return self.vision_bos_token + self.audio_bos_token + rows + self.audio_eos_token + self.vision_eos_token

        try:
            text = pattern.sub(one, text)
        except (StopIteration, RuntimeError) as e:
            raise ValueError("the prompt has more tags of one kind than inputs of that kind") from e
        for left, kind in ((audio, "audio"), (images, "image"), (videos, "video")):
            if next(left, None) is not None:
                raise ValueError(f"more {kind} inputs than tags of that kind in the prompt")
        return text

    def __call__(self, text, images=None, videos=None, audio=None, sampling_rate: Optional[int] = None, fps: float = 1.0,
                 use_audio_in_video: bool = False, video_kwargs: Optional[dict] = None) -> dict:
        texts = [text] if isinstance(text, str) else list(text)
        out, audio_lengths, image_grids, video_grids, seconds = {}, [], [], [], []
        if audio is not None:
            pre = self.feature_extractor(list(audio), sampling_rate=sampling_rate, padding="longest", truncation=False,
                                         return_attention_mask=True)
            out["input_features"], out["feature_attention_mask"] = pre["input_features"], pre["attention_mask"]
            audio_lengths = audio_encoder_output_lengths(pre["attention_mask"].sum(-1).numpy()).tolist()
        if images is not None:
            pre = self.image_processor(list(images))
            out.update(pre)
            image_grids = pre["image_grid_thw"].tolist()
        if videos is not None:
            pre = self.video_processor(list(videos), **(video_kwargs or {}))
            out.update(pre)
            video_grids = pre["video_grid_thw"].tolist()
            seconds = [self.video_processor.temporal_patch_size / fps] * len(video_grids)
            out["video_second_per_grid"] = torch.tensor(seconds)
        # the inputs are listed for the whole batch in prompt order: hand every prompt the ones its tags consume
        a, i, v = iter(audio_lengths), iter(image_grids), iter(video_grids)
        ids = []
        for t in texts:
            n_i, n_v = t.count(self.image_token), t.count(self.video_token)
            n_a = t.count(self.audio_token) + (n_v if use_audio_in_video else 0)
            take = lambda it, n: [next(it) for _ in range(n)]
            try:
                vg = take(v, n_v)
                expanded = self.expand_tags(t, take(a, n_a), take(i, n_i), vg, seconds[:len(vg)], use_audio_in_video)
            except (StopIteration, RuntimeError) as e:
                raise ValueError("the prompts have more tags of one kind than inputs of that kind") from e
            ids.append(self.tokenizer.encode(expanded, add_special_tokens=False))
        for left, kind in ((a, "audio"), (i, "image"), (v, "video")):
            if next(left, None) is not None:
                raise ValueError(f"more {kind} inputs than tags of that kind in the prompts")
        width = max(len(x) for x in ids)
        pad = getattr(self.tokenizer, "pad_token_id", None) or 0
        out["input_ids"] = torch.tensor([[pad] * (width - len(x)) + x for x in ids])          # left padding, as for generation
        out["attention_mask"] = torch.tensor([[0] * (width - len(x)) + [1] * len(x) for x in ids])
        return out

    def batch_decode(self, sequences, skip_special_tokens: bool = True):
        return [self.tokenizer.decode(list(map(int, s)), skip_special_tokens=skip_special_tokens) for s in sequences]
