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

    def __call__(self, raw_speech: Union[np.ndarray, torch.Tensor, Sequence], sampling_rate: int = None, device: str = "cpu") -> Dict[str, torch.Tensor]:
        if sampling_rate is not None and sampling_rate != self.sampling_rate:
            raise ValueError(f"the model expects audio sampled at {self.sampling_rate} Hz, got {sampling_rate} Hz: resample first")
        if isinstance(raw_speech, (np.ndarray, torch.Tensor)) and getattr(raw_speech, "ndim", 1) == 1:
            raw_speech = [raw_speech]
        batch = torch.full((len(raw_speech), self.n_samples), self.padding_value, dtype=torch.float32, device=device)
        for i, w in enumerate(raw_speech):
            w = torch.as_tensor(np.asarray(w) if not isinstance(w, torch.Tensor) else w, dtype=torch.float32)[: self.n_samples]
            batch[i, : w.numel()] = w.to(device)
        return {"input_features": self.log_mel(batch)}


WhisperFeatureExtractor = LogMelFeatureExtractor
