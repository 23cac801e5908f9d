"""Audio front end: log-mel spectrograms for speech models (the role of paddleformers/transformers/audio_processing_utils.py,
audio_utils.py and the Whisper feature extractor).

``LogMelFeatureExtractor`` pads or cuts every waveform to ``chunk_length`` seconds, takes a Hann-windowed STFT, applies a
triangular mel filter bank on the Slaney scale with area normalisation, and compresses: log10, floor at (max - 8), then
(x + 4) / 4. The STFT and the filter bank run as tensor operations on the device the waveform lives on, so a data worker with
a GPU stream can extract features without a host round trip.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence, Union

import numpy as np
import torch


def hertz_to_mel_slaney(f: torch.Tensor) -> torch.Tensor:
    """Linear below 1 kHz (3 mel per 200 Hz), logarithmic above."""
    f = f.to(torch.float64)
    lin = 3.0 * f / 200.0
    log = 15.0 + torch.log(f.clamp(min=1e-10) / 1000.0) * (27.0 / math.log(6.4))
    return torch.where(f >= 1000.0, log, lin)


def mel_to_hertz_slaney(m: torch.Tensor) -> torch.Tensor:
    m = m.to(torch.float64)
    lin = 200.0 * m / 3.0
    log = 1000.0 * torch.exp((math.log(6.4) / 27.0) * (m - 15.0))
    return torch.where(m >= 15.0, log, lin)


def mel_filter_bank(num_frequency_bins: int, num_mel_filters: int, min_frequency: float, max_frequency: float,
                    sampling_rate: int) -> torch.Tensor:
    """[num_frequency_bins, num_mel_filters] triangular filters, Slaney scale, each normalised to unit area."""
    edges = torch.linspace(float(hertz_to_mel_slaney(torch.tensor(min_frequency))), float(hertz_to_mel_slaney(torch.tensor(max_frequency))),
                           num_mel_filters + 2, dtype=torch.float64)
    centres = mel_to_hertz_slaney(edges)                                           # [M + 2] in Hz
    freqs = torch.linspace(0, sampling_rate // 2, num_frequency_bins, dtype=torch.float64)
    widths = centres[1:] - centres[:-1]
    slopes = centres[None, :] - freqs[:, None]                                      # [F, M + 2]
    down = -slopes[:, :-2] / widths[:-1]
    up = slopes[:, 2:] / widths[1:]
    bank = torch.clamp(torch.minimum(down, up), min=0.0)
    bank = bank * (2.0 / (centres[2:] - centres[:-2]))[None]
    return bank.to(torch.float32)


class LogMelFeatureExtractor:
    """``extractor(waveforms, sampling_rate=16000)`` -> ``{"input_features": float32 [B, feature_size, frames]}``."""

    def __init__(self, feature_size: int = 80, sampling_rate: int = 16000, hop_length: int = 160, chunk_length: int = 30,
                 n_fft: int = 400, padding_value: float = 0.0, **unused):
        self.feature_size, self.sampling_rate, self.hop_length = feature_size, sampling_rate, hop_length
        self.chunk_length, self.n_fft, self.padding_value = chunk_length, n_fft, padding_value
        self.n_samples = chunk_length * sampling_rate
        self.nb_max_frames = self.n_samples // hop_length
        self.mel_filters = mel_filter_bank(1 + n_fft // 2, feature_size, 0.0, 8000.0, sampling_rate)

    @classmethod
    def from_pretrained(cls, path: str):
        with open(os.path.join(path, "preprocessor_config.json")) as f:
            return cls(**json.load(f))

    def save_pretrained(self, path: str):
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "preprocessor_config.json"), "w") as f:
            json.dump({"feature_extractor_type": "WhisperFeatureExtractor", "feature_size": self.feature_size,
                       "sampling_rate": self.sampling_rate, "hop_length": self.hop_length, "chunk_length": self.chunk_length,
                       "n_fft": self.n_fft, "padding_value": self.padding_value}, f, indent=1)

    def log_mel(self, waveform: torch.Tensor) -> torch.Tensor:
        """[B, samples] -> [B, feature_size, samples / hop]."""
        window = torch.hann_window(self.n_fft, device=waveform.device)
        stft = torch.stft(waveform.float(), self.n_fft, self.hop_length, window=window, return_complex=True)
        power = stft[..., :-1].abs() ** 2
        mel = self.mel_filters.to(waveform.device).T @ power
        log_spec = torch.clamp(mel, min=1e-10).log10()
        peak = log_spec.amax(dim=(1, 2), keepdim=True)
        return (torch.maximum(log_spec, peak - 8.0) + 4.0) / 4.0

    def __call__(self, raw_speech: Union[np.ndarray, torch.Tensor, Sequence], sampling_rate: int = None, device: str = "cpu",
                 padding="max_length", truncation: bool = True, return_attention_mask: bool = False) -> Dict[str, torch.Tensor]:
        """``padding="max_length"`` pads (and with ``truncation`` cuts) every clip to ``chunk_length`` seconds, the Whisper
        encoder's fixed input; ``padding="longest"`` (or True) pads to the longest clip of the batch, for encoders that take
        clips of any length. ``return_attention_mask`` adds ``attention_mask`` [B, frames]: 1 for frames that start inside
        the clip."""
        if sampling_rate is not None and sampling_rate != self.sampling_rate:
            raise ValueError(f"the model expects audio sampled at {self.sampling_rate} Hz, got {sampling_rate} Hz: resample first")
        if isinstance(raw_speech, (np.ndarray, torch.Tensor)) and getattr(raw_speech, "ndim", 1) == 1:
            raw_speech = [raw_speech]
        clips = [torch.as_tensor(np.asarray(w) if not isinstance(w, torch.Tensor) else w, dtype=torch.float32) for w in raw_speech]
        if truncation:
            clips = [w[: self.n_samples] for w in clips]
        width = self.n_samples if padding == "max_length" else max(w.numel() for w in clips)
        batch = torch.full((len(clips), width), self.padding_value, dtype=torch.float32, device=device)
        for i, w in enumerate(clips):
            batch[i, : w.numel()] = w.to(device)
        out = {"input_features": self.log_mel(batch)}
        if return_attention_mask:
            frames = out["input_features"].shape[-1]
            starts = torch.arange(frames, device=device) * self.hop_length
            out["attention_mask"] = (starts[None, :] < torch.tensor([w.numel() for w in clips], device=device)[:, None]).to(torch.int32)
        return out


WhisperFeatureExtractor = LogMelFeatureExtractor


def kaldi_mel_filter_bank(num_frequency_bins: int, num_mel_filters: int, min_frequency: float, max_frequency: float,
                          sampling_rate: int) -> torch.Tensor:
    """[num_frequency_bins, num_mel_filters] triangular filters on the Kaldi (HTK-formula) mel scale, mel = 1127 ln(1 + f / 700),
    with the triangles drawn in MEL space (a bin's weight is linear in its mel value, not in its frequency) and no area
    normalisation: the filter bank of Kaldi-compatible front ends."""
    def to_mel(f):
        return 1127.0 * torch.log(1.0 + f / 700.0)

    edges = torch.linspace(float(to_mel(torch.tensor(float(min_frequency), dtype=torch.float64))),
                           float(to_mel(torch.tensor(float(max_frequency), dtype=torch.float64))), num_mel_filters + 2, dtype=torch.float64)
    bins = to_mel(torch.linspace(0, sampling_rate // 2, num_frequency_bins, dtype=torch.float64))          # bin centres in mel
    widths = edges[1:] - edges[:-1]
    slopes = edges[None, :] - bins[:, None]
    down, up = -slopes[:, :-2] / widths[:-1], slopes[:, 2:] / widths[1:]
    return torch.clamp(torch.minimum(down, up), min=0.0).to(torch.float32)


class KaldiFbankFeatureExtractor:
    """Log-mel features of the Phi-4-multimodal audio branch (paddleformers/transformers/phi4_multimodal/feature_extraction.py):
    25 ms frames every 10 ms without padding at the edges, per-frame pre-emphasis (the first sample of a frame is paired with
    its successor), 16-bit amplitude scale, symmetric Hamming window, 512-point power spectrum, 80 Kaldi-scale mel filters up
    to 7690 Hz, natural log floored at 0. ``extractor(waveforms)`` returns ``audio_input_features`` [B, frames, 80],
    ``audio_embed_sizes`` [B] (placeholders per clip: frames / compression rate, rounded up, then / downsample rate, rounded
    up) and, for a batch of clips of different lengths, ``audio_attention_mask`` [B, frames]."""

    def __init__(self, feature_size: int = 80, sampling_rate: int = 16000, hop_length: int = 160, n_fft: int = 512,
                 win_length: int = 400, preemphasis: float = 0.97, audio_compression_rate: int = 8, audio_downsample_rate: int = 1,
                 audio_feat_stride: int = 1, mel_min_frequency: float = 0.0, mel_max_frequency: float = 7690.0, **unused):
        self.feature_size, self.sampling_rate, self.hop_length, self.n_fft, self.win_length = feature_size, sampling_rate, hop_length, n_fft, win_length
        self.preemphasis, self.rate, self.down, self.stride = preemphasis, audio_compression_rate, audio_downsample_rate, audio_feat_stride
        self.mel_filters = kaldi_mel_filter_bank(n_fft // 2 + 1, feature_size, mel_min_frequency, mel_max_frequency, sampling_rate)

    @classmethod
    def from_pretrained(cls, path: str):
        with open(os.path.join(path, "preprocessor_config.json")) as f:
            return cls(**json.load(f))

    def num_frames(self, num_samples: int) -> int:
        return ((num_samples - self.win_length) // self.hop_length + 1) * self.stride

    def num_placeholders(self, frames: int) -> int:
        return -(-(-(-frames // self.rate)) // self.down)

    def features(self, wave: torch.Tensor) -> torch.Tensor:
        """wave [samples] -> [frames, feature_size]."""
        frames = wave.to(torch.float32).unfold(-1, self.win_length, self.hop_length)
        prev = torch.roll(frames, 1, dims=-1)
        prev[:, 0] = prev[:, 1]
        frames = (frames - self.preemphasis * prev) * 32768
        window = torch.hamming_window(self.win_length, periodic=False, dtype=torch.float64, device=wave.device)
        spec = torch.fft.rfft(window * frames, n=self.n_fft, dim=1).to(torch.complex64).abs() ** 2
        return torch.log(torch.clamp(spec @ self.mel_filters.to(wave.device), min=1.0))

    def __call__(self, raw_speech, sampling_rate: int = None, **unused) -> Dict[str, torch.Tensor]:
        if sampling_rate is not None and sampling_rate != self.sampling_rate:
            raise ValueError(f"expected audio sampled at {self.sampling_rate} Hz, got {sampling_rate}")
        clips = raw_speech if isinstance(raw_speech, (list, tuple)) else (list(raw_speech) if getattr(raw_speech, "ndim", 1) > 1 else [raw_speech])
        feats = [self.features(torch.as_tensor(np.asarray(c) if not isinstance(c, torch.Tensor) else c)) for c in clips]
        n = torch.tensor([f.shape[0] for f in feats])
        out = torch.zeros(len(feats), int(n.max()), self.feature_size)
        for i, f in enumerate(feats):
            out[i, :f.shape[0]] = f
        data = {"audio_input_features": out, "audio_embed_sizes": torch.tensor([self.num_placeholders(int(x)) for x in n])}
        if len(feats) > 1:
            data["audio_attention_mask"] = torch.arange(int(n.max()))[None] < n[:, None]
        return data
