"""Whisper: encoder-decoder speech recognition (paddleformers/transformers/whisper).

Encoder: two 1-D convolutions over the log-mel spectrogram (the second with stride 2), fixed sinusoidal positions, pre-LayerNorm
blocks with full attention. Decoder: token + learned position embeddings, pre-LayerNorm blocks with causal self-attention and
cross-attention over the encoder states, output projection tied to the token embedding. Self-attention goes through the flash
attention entry point (non-causal in the encoder, causal in the decoder); cross-attention has different query and key lengths
and runs as a library call. Tensor names are the checkpoint's own, under ``model.``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from ..transformers.configuration_utils import PretrainedConfig
from ..transformers.conversion_utils import Rule, WeightMap
from ..transformers.model_utils import PretrainedModel
from .modeling import CausalLMOutput


class WhisperConfig(PretrainedConfig):
    model_type = "whisper"

    def __init__(self, vocab_size=51865, num_mel_bins=80, encoder_layers=4, encoder_attention_heads=6, decoder_layers=4,
                 decoder_attention_heads=6, decoder_ffn_dim=1536, encoder_ffn_dim=1536, d_model=384, max_source_positions=1500,
                 max_target_positions=448, activation_function="gelu", scale_embedding=False, decoder_start_token_id=50257,
                 pad_token_id=50256, bos_token_id=50256, eos_token_id=50256, **kwargs):
        kwargs.pop("model_type", None)
        kwargs.setdefault("tie_word_embeddings", True)
        super().__init__(vocab_size=vocab_size, hidden_size=d_model, num_hidden_layers=decoder_layers,
                         num_attention_heads=decoder_attention_heads, pad_token_id=pad_token_id, bos_token_id=bos_token_id,
                         eos_token_id=eos_token_id, **kwargs)
        self.num_mel_bins, self.d_model = num_mel_bins, d_model
        self.encoder_layers, self.encoder_attention_heads, self.encoder_ffn_dim = encoder_layers, encoder_attention_heads, encoder_ffn_dim
        self.decoder_layers, self.decoder_attention_heads, self.decoder_ffn_dim = decoder_layers, decoder_attention_heads, decoder_ffn_dim
        self.max_source_positions, self.max_target_positions = max_source_positions, max_target_positions
        self.activation_function, self.scale_embedding = activation_function, scale_embedding
        self.decoder_start_token_id = decoder_start_token_id

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            for k in ("hidden_size", "num_hidden_layers", "num_attention_heads"):
                d.pop(k, None)
            d["is_encoder_decoder"] = True
        return d


def sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    """Fixed encoder positions: sines in the first half of the channels, cosines in the second."""
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2, dtype=torch.float32))
    t = torch.arange(length, dtype=torch.float32)[:, None] * inv[None]
    return torch.cat([t.sin(), t.cos()], dim=1)


class _Attention(nn.Module):
    def __init__(self, d: int, heads: int, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.heads, self.hd = heads, d // heads
        self.q_proj, self.v_proj, self.out_proj = nn.Linear(d, d, **kw), nn.Linear(d, d, **kw), nn.Linear(d, d, **kw)
        self.k_proj = nn.Linear(d, d, bias=False, **kw)

    def forward(self, x, memory=None, causal=False):
        B, S, d = x.shape
        src = x if memory is None else memory
        T = src.shape[1]
        q = self.q_proj(x).view(B, S, self.heads, self.hd)
        k = self.k_proj(src).view(B, T, self.heads, self.hd)
        v = self.v_proj(src).view(B, T, self.heads, self.hd)
        if memory is None:
            o = F.flash_attention(q, k, v, causal=causal)
        else:
            o = TF.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
        return self.out_proj(o.reshape(B, S, d))


class _Layer(nn.Module):
    def __init__(self, d: int, heads: int, ffn: int, cross: bool, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.self_attn = _Attention(d, heads, **kw)
        self.self_attn_layer_norm = nn.LayerNorm(d, **kw)
        if cross:
            self.encoder_attn = _Attention(d, heads, **kw)
            self.encoder_attn_layer_norm = nn.LayerNorm(d, **kw)
        self.cross = cross
        self.fc1, self.fc2 = nn.Linear(d, ffn, **kw), nn.Linear(ffn, d, **kw)
        self.final_layer_norm = nn.LayerNorm(d, **kw)

    def forward(self, x, memory=None):
        x = x + self.self_attn(self.self_attn_layer_norm(x), causal=self.cross)
        if self.cross:
            x = x + self.encoder_attn(self.encoder_attn_layer_norm(x), memory=memory)
        return x + self.fc2(TF.gelu(self.fc1(self.final_layer_norm(x))))


class WhisperEncoder(nn.Module):
    def __init__(self, cfg: WhisperConfig, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        d = cfg.d_model
        self.conv1 = nn.Conv1d(cfg.num_mel_bins, d, kernel_size=3, padding=1, **kw)
        self.conv2 = nn.Conv1d(d, d, kernel_size=3, stride=2, padding=1, **kw)
        self.embed_positions = nn.Embedding(cfg.max_source_positions, d, **kw)
        self.embed_positions.weight.requires_grad_(False)
        self.layers = nn.ModuleList([_Layer(d, cfg.encoder_attention_heads, cfg.encoder_ffn_dim, False, **kw) for _ in range(cfg.encoder_layers)])
        self.layer_norm = nn.LayerNorm(d, **kw)

    def forward(self, input_features):                       # [B, mel bins, frames]
        x = TF.gelu(self.conv1(input_features.to(self.conv1.weight.dtype)))
        x = TF.gelu(self.conv2(x)).transpose(1, 2)
        x = x + self.embed_positions.weight[None, :x.shape[1]]
        for layer in self.layers:
            x = layer(x)
        return self.layer_norm(x)


class WhisperDecoder(nn.Module):
    def __init__(self, cfg: WhisperConfig, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        d = cfg.d_model
        self.scale = math.sqrt(d) if cfg.scale_embedding else 1.0
        self.embed_tokens = nn.Embedding(cfg.vocab_size, d, **kw)
        self.embed_positions = nn.Embedding(cfg.max_target_positions, d, **kw)
        self.layers = nn.ModuleList([_Layer(d, cfg.decoder_attention_heads, cfg.decoder_ffn_dim, True, **kw) for _ in range(cfg.decoder_layers)])
        self.layer_norm = nn.LayerNorm(d, **kw)

    def forward(self, input_ids, memory):
        x = self.embed_tokens(input_ids) * self.scale + self.embed_positions.weight[None, :input_ids.shape[1]]
        for layer in self.layers:
            x = layer(x, memory)
        return self.layer_norm(x)


class _Body(nn.Module):
    def __init__(self, cfg, dtype=None, device=None):
        super().__init__()
        self.encoder = WhisperEncoder(cfg, dtype=dtype, device=device)
        self.decoder = WhisperDecoder(cfg, dtype=dtype, device=device)


def shift_tokens_right(labels: torch.Tensor, pad_token_id: int, start_token_id: int) -> torch.Tensor:
    """Decoder inputs for teacher forcing: the labels moved one step right behind the start token; ignored labels become padding."""
    out = labels.new_full(labels.shape, pad_token_id)
    out[:, 1:] = labels[:, :-1]
    out[:, 0] = start_token_id
    return out.masked_fill(out == -100, pad_token_id)


class WhisperForConditionalGeneration(PretrainedModel):
    config_class = WhisperConfig

    def __init__(self, config: WhisperConfig, dtype=None, device=None):
        super().__init__(config)
        self.model = _Body(config, dtype=dtype, device=device)
        self.post_init()
        with torch.no_grad():
            self.model.encoder.embed_positions.weight.copy_(sinusoids(config.max_source_positions, config.d_model))

    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, (nn.Linear, nn.Conv1d)):
            nn.init.normal_(module.weight, 0.0, std)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, 0.0, std)

    def forward(self, input_features=None, decoder_input_ids=None, labels=None, encoder_outputs=None,
                return_logits: Optional[bool] = None, **unused):
        """``labels`` are aligned with the decoder outputs (position t predicts labels[:, t]); without ``decoder_input_ids`` the
        decoder is fed the labels shifted right behind ``decoder_start_token_id``."""
        cfg = self.config
        memory = encoder_outputs if encoder_outputs is not None else self.model.encoder(input_features)
        if decoder_input_ids is None:
            decoder_input_ids = shift_tokens_right(labels, cfg.pad_token_id, cfg.decoder_start_token_id)
        hidden = self.model.decoder(decoder_input_ids, memory)
        out = CausalLMOutput(hidden_states=memory)
        logits = TF.linear(hidden, self.model.decoder.embed_tokens.weight)
        if return_logits if return_logits is not None else labels is None:
            out.logits = logits
        if labels is not None:
            count = (labels != -100).sum()
            out.loss = TF.cross_entropy(logits.float().view(-1, logits.shape[-1]), labels.reshape(-1), ignore_index=-100, reduction="sum") \
                / count.clamp(min=1)
            out.num_tokens = count
        return out

    @torch.no_grad()
    def generate(self, input_features, decoder_input_ids=None, max_new_tokens: int = 64, eos_token_id: Optional[int] = None):
        """Greedy transcription: the encoder runs once, the decoder re-reads its own prefix at every step."""
        cfg = self.config
        eos = cfg.eos_token_id if eos_token_id is None else eos_token_id
        memory = self.model.encoder(input_features)
        B = memory.shape[0]
        ids = decoder_input_ids if decoder_input_ids is not None else \
            torch.full((B, 1), cfg.decoder_start_token_id, dtype=torch.long, device=memory.device)
        done = torch.zeros(B, dtype=torch.bool, device=memory.device)
        for _ in range(min(max_new_tokens, cfg.max_target_positions - ids.shape[1])):
            hidden = self.model.decoder(ids, memory)[:, -1]
            nxt = TF.linear(hidden, self.model.decoder.embed_tokens.weight).argmax(-1)
            nxt = torch.where(done, torch.full_like(nxt, cfg.pad_token_id), nxt)
            ids = torch.cat([ids, nxt[:, None]], dim=1)
            done |= nxt == eos
            if bool(done.all()):
                break
        return ids

    def weight_map(self) -> WeightMap:
        return WeightMap([Rule(name, [name]) for name, _ in self.named_parameters()])
