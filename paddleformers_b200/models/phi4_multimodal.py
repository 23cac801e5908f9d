"""Phi-4-multimodal: a Phi-3 style decoder fed by an image branch and an audio branch
(paddleformers/transformers/phi4_multimodal/modeling.py:1-2000, configuration.py).

* Image branch: a SigLIP-style tower over 448 x 448 crops whose learned position table is addressed by the FRACTIONAL
  position of each patch inside the valid part of its crop (bucketised, so crops that are only partly filled reuse the table),
  with attention restricted to valid patches. The hidden states of layer ``feature_layer`` are average-pooled 2 x 2 (after a
  one-patch reflection pad when the grid is odd), arranged per image as [sub-crops tiled into one grid, a learned separator at
  the end of every row | a learned separator | the global crop, same row separators], and projected by a two-layer GELU MLP.
* Audio branch: global mean / variance normalisation of the log-mel frames, a strided convolution stack (time / 8) + linear,
  conformer blocks (half-step feed-forward with a gated linear unit, self-attention with a learned relative-position bias per
  head, a gated point-wise + causal depth-wise convolution module, a second half-step feed-forward, LayerNorm); sequences longer
  than 500 frames are cut into windows of 500. The result goes through one of two GELU MLP projectors: "speech" for audio-only
  prompts, "vision" when the prompt also has images.
* The features replace the image / audio placeholder tokens of the prompt; the decoder is the unified decoder (fused qkv and
  gate-up projections, partial rotary, long-rope scaling).

Checkpoint tensors keep their published names (``model.embed_tokens_extend.image_embed.*`` / ``.audio_embed.*``).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..transformers.configuration_utils import PretrainedConfig
from ..transformers.conversion_utils import Rule, WeightMap
from ..transformers.model_utils import PretrainedModel
from .configuration import Phi3Config
from .modeling import BatchContext, CausalLMOutput, DecoderForCausalLM, build_weight_map

_ACT = {"swish": TF.silu, "silu": TF.silu, "relu": TF.relu, "gelu": TF.gelu,
        "gelu_pytorch_tanh": lambda x: TF.gelu(x, approximate="tanh"), "sigmoid": torch.sigmoid}

_VISION = dict(hidden_size=1152, intermediate_size=4304, num_hidden_layers=27, num_attention_heads=16, num_channels=3,
               image_size=448, patch_size=14, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6, crop_size=448,
               image_token_id=200010, feature_layer=-2)
_AUDIO = dict(hidden_size=1024, intermediate_size=1536, num_blocks=24, num_attention_heads=16, activation="swish", chunk_size=-1,
              left_chunk=18, ext_pw_out_channel=1024, depthwise_separable_out_channel=1024, depthwise_multiplier=1, kernel_size=3,
              conv_activation="swish", input_size=80, conv_glu_type="swish", time_reduction=8, bias_max_distance=1000,
              bias_symmetric=False, nemo_activation="relu", nemo_conv_channels=1024, downsample_rate=1, audio_token_id=200011,
              feature_layer=-2, nemo_final_size=10)


class Phi4MultimodalConfig(PretrainedConfig):
    model_type = "phi4_multimodal"

    def __init__(self, vision_config=None, audio_config=None, **text):
        text.pop("model_type", None)
        text.setdefault("vocab_size", 200064)
        text.setdefault("hidden_size", 3072)
        text.setdefault("intermediate_size", 8192)
        text.setdefault("num_hidden_layers", 32)
        text.setdefault("num_attention_heads", 32)
        text.setdefault("num_key_value_heads", 8)
        text.setdefault("rms_norm_eps", 1e-5)
        text.setdefault("max_position_embeddings", 131072)
        text.setdefault("tie_word_embeddings", False)
        self.text_config = Phi3Config(**text)
        self.vision_config = dict(_VISION, **{k: v for k, v in (vision_config or {}).items() if k in _VISION})
        self.audio_config = dict(_AUDIO, **{k: v for k, v in (audio_config or {}).items() if k in _AUDIO})
        t = self.text_config
        super().__init__(vocab_size=t.vocab_size, hidden_size=t.hidden_size, num_hidden_layers=t.num_hidden_layers,
                         num_attention_heads=t.num_attention_heads, tie_word_embeddings=t.tie_word_embeddings,
                         bos_token_id=t.bos_token_id, eos_token_id=t.eos_token_id, pad_token_id=t.pad_token_id, dtype=t.dtype)

    @property
    def image_token_id(self):
        return self.vision_config["image_token_id"]

    @property
    def audio_token_id(self):
        return self.audio_config["audio_token_id"]

    def to_dict(self, saving: bool = False):
        d = self.text_config.to_dict(saving)           # the decoder's fields live at the top level of config.json
        d["model_type"] = self.model_type
        d["vision_config"] = dict(self.vision_config, model_type="phi4_multimodal_vision")
        d["audio_config"] = dict(self.audio_config, model_type="phi4_multimodal_audio")
        return d


# ---------------------------------------------------------------------------------------------------------------------
# image branch
# ---------------------------------------------------------------------------------------------------------------------
class _VisionLayer(nn.Module):
    def __init__(self, vc, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        H = vc["hidden_size"]
        self.heads = vc["num_attention_heads"]
        self.layer_norm1, self.layer_norm2 = nn.LayerNorm(H, eps=vc["layer_norm_eps"], **kw), nn.LayerNorm(H, eps=vc["layer_norm_eps"], **kw)
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (nn.Linear(H, H, **kw) for _ in range(4))
        self.fc1, self.fc2 = nn.Linear(H, vc["intermediate_size"], **kw), nn.Linear(vc["intermediate_size"], H, **kw)
        self.act = _ACT[vc["hidden_act"]]

    def forward(self, x, key_mask):
        """x [N, P, H]; key_mask [N, P] bool: patches that exist."""
        N, P, H = x.shape
        h = self.layer_norm1(x)
        q, k, v = (p(h).view(N, P, self.heads, -1).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        a = TF.scaled_dot_product_attention(q, k, v, attn_mask=key_mask[:, None, None, :])
        x = x + self.out_proj(a.transpose(1, 2).reshape(N, P, H))
        return x + self.fc2(self.act(self.fc1(self.layer_norm2(x))))


class _PoolingHeadWeights(nn.Module):
    def __init__(self, vc, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        H = vc["hidden_size"]
        self.probe = nn.Parameter(torch.zeros(1, 1, H, **kw))
        self.attention = nn.MultiheadAttention(H, vc["num_attention_heads"], batch_first=True, **kw)
        self.layernorm = nn.LayerNorm(H, eps=vc["layer_norm_eps"], **kw)
        self.fc1, self.fc2 = nn.Linear(H, vc["intermediate_size"], **kw), nn.Linear(vc["intermediate_size"], H, **kw)


class Phi4VisionTower(nn.Module):
    """Crops [N, 3, S, S] + valid-patch masks [N, S/p, S/p] -> hidden states of layer ``feature_layer`` [N, (S/p)^2, H]."""

    def __init__(self, vc, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.vc = vc
        self.side = vc["image_size"] // vc["patch_size"]
        self.patch_embedding = nn.Conv2d(vc["num_channels"], vc["hidden_size"], vc["patch_size"], vc["patch_size"], **kw)
        self.position_embedding = nn.Embedding(self.side ** 2, vc["hidden_size"], **kw)
        # hidden_states[feature_layer] of an L-layer tower (index 0 = the embeddings): the output of layer L + feature_layer
        n_run = vc["num_hidden_layers"] + 1 + vc["feature_layer"] if vc["feature_layer"] < 0 else vc["feature_layer"]
        self.layers = nn.ModuleList([_VisionLayer(vc, **kw) for _ in range(vc["num_hidden_layers"])])
        self.n_run = n_run
        # the checkpoint also carries the tower's last layers, final norm and pooling head; the language model reads an
        # earlier layer, so they only travel with the weights
        self.post_layernorm = nn.LayerNorm(vc["hidden_size"], eps=vc["layer_norm_eps"], **kw)
        self.head = _PoolingHeadWeights(vc, **kw)

    def position_ids(self, mask: torch.Tensor) -> torch.Tensor:
        """Table row of every patch: its fractional (row, column) inside the valid part of the crop, bucketised to the
        table's side; patches outside the valid part use row 0."""
        N, Ph, Pw = mask.shape
        side = self.side
        bounds = torch.arange(1 / side, 1.0, 1 / side, device=mask.device)
        nh, nw = mask[:, :, 0].sum(1), mask[:, 0, :].sum(1)
        fh = (torch.arange(Ph, device=mask.device, dtype=torch.float32)[None] / nh[:, None]).clamp(max=1.0 - 1e-6)
        fw = (torch.arange(Pw, device=mask.device, dtype=torch.float32)[None] / nw[:, None]).clamp(max=1.0 - 1e-6)
        bh, bw = torch.bucketize(fh, bounds, right=True), torch.bucketize(fw, bounds, right=True)
        ids = (bh[:, :, None] * side + bw[:, None, :]).reshape(N, -1)
        return torch.where(mask.reshape(N, -1), ids, torch.zeros_like(ids))

    def forward(self, pixels: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        x = self.patch_embedding(pixels.to(self.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        x = x + self.position_embedding(self.position_ids(mask))
        key_mask = mask.reshape(mask.shape[0], -1)
        for layer in self.layers[:self.n_run]:
            x = layer(x, key_mask)
        return x


class Phi4ImageEmbedding(nn.Module):
    def __init__(self, config: Phi4MultimodalConfig, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        vc = config.vision_config
        self.crop, self.dim = vc["crop_size"], vc["hidden_size"]
        self.odd = (vc["image_size"] // vc["patch_size"]) % 2 != 0
        self.img_processor = Phi4VisionTower(vc, **kw)
        self.img_projection_up = nn.Linear(self.dim, config.hidden_size, **kw)
        self.img_projection_down = nn.Linear(config.hidden_size, config.hidden_size, **kw)
        self.global_img_feature_extensor = nn.Parameter(torch.zeros(1, 1, self.dim, **kw))
        self.sub_img_feature_extensor = nn.Parameter(torch.zeros(1, 1, 1, self.dim, **kw))

    def crop_features(self, pixels, mask):
        """[crops, 3, S, S] -> [crops, f, f, dim]: tower features pooled 2 x 2."""
        x = self.img_processor(pixels, mask)
        w = int(math.sqrt(x.shape[1]))
        x = x.view(-1, w, w, x.shape[-1]).permute(0, 3, 1, 2)
        if self.odd:
            x = TF.pad(x, (0, 1, 0, 1), mode="reflect")
        return TF.avg_pool2d(x, 2, 2).permute(0, 2, 3, 1)

    def forward(self, image_pixel_values, image_sizes, image_attention_mask) -> torch.Tensor:
        """image_pixel_values [B, 1 + crops, 3, S, S] (the global view first), image_sizes [B, 2] (height, width of the resized
        image: multiples of the crop size), image_attention_mask [B, 1 + crops, S/p, S/p]. Returns the rows that replace the
        placeholders, image after image."""
        B = image_pixel_values.shape[0]
        feats = self.crop_features(image_pixel_values.flatten(0, 1), image_attention_mask.flatten(0, 1).bool())
        f = feats.shape[1]
        feats = feats.view(B, -1, f, f, self.dim)
        rows = []
        for b in range(B):
            hr, wr = int(image_sizes[b, 0]) // self.crop, int(image_sizes[b, 1]) // self.crop
            sep = self.sub_img_feature_extensor
            glob = torch.cat([feats[b, :1], sep.expand(1, f, 1, self.dim)], dim=2).reshape(-1, self.dim)
            sub = feats[b, 1:1 + hr * wr].reshape(hr, wr, f, f, self.dim).transpose(1, 2).reshape(1, hr * f, wr * f, self.dim)
            m = image_attention_mask[b, 1:1 + hr * wr, 0::2, 0::2].reshape(hr, wr, f, f).transpose(1, 2).reshape(hr * f, wr * f)
            uh, uw = int(m[:, 0].sum()), int(m[0, :].sum())          # the part of the tiled grid that shows the image
            sub = torch.cat([sub[:, :uh, :uw], sep.expand(1, uh, 1, self.dim)], dim=2).reshape(-1, self.dim)
            rows.append(torch.cat([sub, self.global_img_feature_extensor[0], glob], dim=0))
        x = torch.cat(rows, dim=0)
        return self.img_projection_down(TF.gelu(self.img_projection_up(x)))


# ---------------------------------------------------------------------------------------------------------------------
# audio branch
# ---------------------------------------------------------------------------------------------------------------------
class _AudioMLP(nn.Module):
    def __init__(self, ac, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.layer_norm = nn.LayerNorm(ac["hidden_size"], **kw)
        self.gate_up_proj = nn.Linear(ac["hidden_size"], 2 * ac["intermediate_size"], **kw)
        self.down_proj = nn.Linear(ac["intermediate_size"], ac["hidden_size"], **kw)
        self.act = _ACT[ac["activation"]]

    def forward(self, x):
        up, gate = self.gate_up_proj(self.layer_norm(x)).chunk(2, dim=-1)
        return self.down_proj(up * self.act(gate))


class _AudioConv(nn.Module):
    """LayerNorm -> point-wise conv to 2C with a gated linear unit (own biases) -> causal depth-wise + point-wise conv ->
    activation -> point-wise conv."""

    def __init__(self, ac, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        H, C, K = ac["hidden_size"], ac["ext_pw_out_channel"], ac["kernel_size"]
        self.K, self.C = K, C
        self.layer_norm = nn.LayerNorm(H, **kw)
        self.glu_conv = nn.Conv1d(H, 2 * C, 1, **kw)
        self.b1, self.b2 = nn.Parameter(torch.zeros(1, C, 1, **kw)), nn.Parameter(torch.zeros(1, C, 1, **kw))
        self.dw_conv = nn.Conv1d(H, H * ac["depthwise_multiplier"], K, 1, padding=K - 1, groups=H, **kw)
        self.pw_conv = nn.Conv1d(H * ac["depthwise_multiplier"], ac["depthwise_separable_out_channel"], 1, **kw)
        self.ext_pw_conv_1d = nn.Conv1d(H, C, 1, **kw)
        self.glu_act, self.act = _ACT[ac["conv_glu_type"]], _ACT[ac["conv_activation"]]

    def forward(self, x):
        h = self.glu_conv(self.layer_norm(x).transpose(1, 2))
        h = (h[:, :self.C] + self.b1) * self.glu_act(h[:, self.C:] + self.b2)
        h = self.pw_conv(self.dw_conv(h))
        if self.K > 1:
            h = h[:, :, :-(self.K - 1)]                 # the padding on the right is cut: position t sees t - K + 1 .. t
        return self.ext_pw_conv_1d(self.act(h)).transpose(1, 2)


class _ConformerLayer(nn.Module):
    def __init__(self, ac, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        H = ac["hidden_size"]
        self.heads = ac["num_attention_heads"]
        self.feed_forward_in, self.feed_forward_out = _AudioMLP(ac, **kw), _AudioMLP(ac, **kw)
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = (nn.Linear(H, H, **kw) for _ in range(4))
        self.conv = _AudioConv(ac, **kw)
        self.layer_norm_att, self.layer_norm = nn.LayerNorm(H, **kw), nn.LayerNorm(H, **kw)

    def forward(self, x, bias):
        """x [N, T, H]; bias [N or 1, heads, T, T] additive (relative-position bias, -inf on hidden keys)."""
        N, T, H = x.shape
        x = x + 0.5 * self.feed_forward_in(x)
        h = self.layer_norm_att(x)
        q, k, v = (p(h).view(N, T, self.heads, -1).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        a = TF.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype))
        x = x + self.o_proj(a.transpose(1, 2).reshape(N, T, H))
        x = x + self.conv(x)
        x = x + 0.5 * self.feed_forward_out(x)
        return self.layer_norm(x)


def streaming_visibility(T: int, chunk: int, left_chunks: int, device) -> torch.Tensor:
    """bool [T, T]: frame i sees the frames of its own chunk of ``chunk`` frames and of ``left_chunks`` chunks before it
    (``chunk`` <= 0 or >= T: everything)."""
    if chunk <= 0 or chunk >= T:
        return torch.ones(T, T, dtype=torch.bool, device=device)
    c = torch.arange(T, device=device) // chunk
    return (c[None, :] <= c[:, None]) & (c[None, :] >= c[:, None] - left_chunks)


class Phi4AudioEncoder(nn.Module):
    WINDOW = 500            # frames (after the time reduction) that one pass of the blocks sees

    def __init__(self, ac, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.ac = ac
        self.register_buffer("global_mean", torch.zeros(ac["input_size"], **kw))
        self.register_buffer("global_invstd", torch.ones(ac["input_size"], **kw))
        C = ac["nemo_conv_channels"]
        self.act = _ACT[ac["nemo_activation"]]
        n_sub = int(math.log2(ac["time_reduction"]))
        self.conv_in = nn.Conv2d(1, C, 3, 2, 1, **kw)
        self.conv_dw = nn.ModuleList([nn.Conv2d(C, C, 3, 2, 1, groups=C, **kw) for _ in range(n_sub - 1)])
        self.conv_pw = nn.ModuleList([nn.Conv2d(C, C, 1, **kw) for _ in range(n_sub - 1)])
        self.out = nn.Linear(C * ac["nemo_final_size"], ac["hidden_size"], **kw)
        buckets = ac["bias_max_distance"] * (1 if ac["bias_symmetric"] else 2)
        self.bias_values = nn.Embedding(buckets, ac["num_attention_heads"], **kw)
        self.encoders = nn.ModuleList([_ConformerLayer(ac, **kw) for _ in range(ac["num_blocks"])])

    def relative_bias(self, T: int, device) -> torch.Tensor:
        D = self.ac["bias_max_distance"]
        rel = (torch.arange(T, device=device)[None, :] - torch.arange(T, device=device)[:, None]).clamp(-D, D - 1)
        idx = rel.abs() if self.ac["bias_symmetric"] else rel + self.bias_values.num_embeddings // 2
        return self.bias_values(idx).permute(2, 0, 1)[None]                  # [1, heads, T, T]

    def forward(self, feats: torch.Tensor, frame_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """feats [N, frames, mel]; frame_mask [N, frames] bool (valid frames). Returns [N, ceil(frames / r), H]."""
        ac = self.ac
        x = ((feats - self.global_mean) * self.global_invstd)[:, None]
        x = self.act(self.conv_in(x))
        for dw, pw in zip(self.conv_dw, self.conv_pw):
            x = self.act(pw(dw(x)))
        N, _, T, _ = x.shape
        x = self.out(x.transpose(1, 2).reshape(N, T, -1))
        valid = None
        if frame_mask is not None:
            n = torch.ceil(frame_mask.sum(1) / ac["time_reduction"])
            valid = torch.arange(T, device=x.device)[None] < n[:, None]                     # [N, T]
        W, pad = self.WINDOW, 0
        if T > W:                                        # long audio: windows of W frames, each attended on its own
            pad = (-T) % W
            x = TF.pad(x, (0, 0, 0, pad)).reshape(N * ((T + pad) // W), W, -1)
            if valid is not None:
                valid = TF.pad(valid, (0, pad)).reshape(-1, W)
        Tw = x.shape[1]
        vis = streaming_visibility(Tw, ac["chunk_size"], ac["left_chunk"], x.device)[None]    # [1, Tw, Tw]
        if valid is not None:
            vis = vis & valid[:, None, :]
        bias = self.relative_bias(Tw, x.device).float() + torch.zeros_like(vis, dtype=torch.float32).masked_fill(~vis, float("-inf"))[:, None]
        for layer in self.encoders:
            x = layer(x, bias)
        if T > W:
            x = x.reshape(N, -1, x.shape[-1])[:, :T]
        return x


class Phi4AudioEmbedding(nn.Module):
    def __init__(self, config: Phi4MultimodalConfig, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        ac, H = config.audio_config, config.hidden_size
        self.encoder = Phi4AudioEncoder(ac, **kw)
        width = ac["hidden_size"] * ac["downsample_rate"]
        self.up_proj_for_speech, self.down_proj_for_speech = nn.Linear(width, H, **kw), nn.Linear(H, H, **kw)
        self.up_proj_for_vision_speech, self.down_proj_for_vision_speech = nn.Linear(width, H, **kw), nn.Linear(H, H, **kw)

    def forward(self, audio_input_features, audio_embed_sizes, audio_attention_mask=None, mode: str = "speech") -> torch.Tensor:
        h = self.encoder(audio_input_features.to(self.up_proj_for_speech.weight.dtype), audio_attention_mask)
        up, down = (self.up_proj_for_speech, self.down_proj_for_speech) if mode == "speech" else \
            (self.up_proj_for_vision_speech, self.down_proj_for_vision_speech)
        h = down(TF.gelu(up(h)))
        return torch.cat([h[i, :int(n)] for i, n in enumerate(audio_embed_sizes)], dim=0)


# ---------------------------------------------------------------------------------------------------------------------
class _FeatureEmbedding(nn.Module):
    def __init__(self, config, dtype=None, device=None):
        super().__init__()
        self.image_embed = Phi4ImageEmbedding(config, dtype=dtype, device=device)
        self.audio_embed = Phi4AudioEmbedding(config, dtype=dtype, device=device)


class Phi4MultimodalForCausalLM(PretrainedModel):
    config_class = Phi4MultimodalConfig

    def __init__(self, config: Phi4MultimodalConfig, dtype=None, device=None):
        super().__init__(config)
        self.embed_tokens_extend = _FeatureEmbedding(config, dtype=dtype, device=device)
        self.language = DecoderForCausalLM(config.text_config, dtype=dtype, device=device)

    def forward(self, input_ids, image_pixel_values=None, image_sizes=None, image_attention_mask=None, audio_input_features=None,
                audio_embed_sizes=None, audio_attention_mask=None, labels=None, position_ids=None,
                return_logits: Optional[bool] = None, **unused):
        cfg, lm = self.config, self.language
        h = lm.model.embed(input_ids, whole=True)
        flat = input_ids.reshape(-1)
        for tok, feats in ((cfg.image_token_id, None if image_pixel_values is None else
                            self.embed_tokens_extend.image_embed(image_pixel_values, image_sizes, image_attention_mask)),
                           (cfg.audio_token_id, None if audio_input_features is None else
                            self.embed_tokens_extend.audio_embed(audio_input_features, audio_embed_sizes, audio_attention_mask,
                                                                 "vision" if image_pixel_values is not None else "speech"))):
            if feats is not None:
                mask = flat == tok
                assert int(mask.sum()) == feats.shape[0], "one placeholder token per image / audio feature row is required"
                h = h.masked_scatter(mask[:, None], feats.to(h.dtype))
        ctx = lm.model.make_context(input_ids, position_ids)
        hidden, residual = lm.model.run_layers(lm.model.token_slice(h), None, ctx)
        hidden = lm.model.norm(hidden, residual)[0] if residual is not None else lm.model.norm(hidden)
        out = CausalLMOutput()
        if return_logits if return_logits is not None else labels is None:
            out.logits = lm.full_logits(hidden).view(ctx.B, ctx.S, -1)
        if labels is not None:
            lab = labels.reshape(-1)
            count = (lab != lm.ignore_index).sum()
            scale = 1.0 / (count.clamp(min=1).to(torch.float32) * float(lm.loss_accumulation_steps))
            out.loss, _ = lm._loss(hidden, lab, scale)
            out.num_tokens = count
        return out

    @property
    def loss_accumulation_steps(self):
        return self.language.loss_accumulation_steps

    @loss_accumulation_steps.setter
    def loss_accumulation_steps(self, v):
        self.language.loss_accumulation_steps = v

    def weight_map(self) -> WeightMap:
        rules = []
        for r in build_weight_map(self.config.text_config).rules.values():
            rules.append(Rule("language." + r.target, list(r.sources), r.op, r.dim, r.num_experts, r.expert_pairs, r.sizes,
                              r.rope_deinterleave, r.flatten, fn=r.fn))
        known = {r.target for r in rules}
        for name, _ in self.language.named_parameters():
            if "language." + name not in known:
                rules.append(Rule("language." + name, [name]))
        img, aud = "model.embed_tokens_extend.image_embed.", "model.embed_tokens_extend.audio_embed."
        tower = {"patch_embedding.": "embeddings.patch_embedding.", "position_embedding.": "embeddings.position_embedding."}
        attn = ("q_proj", "k_proj", "v_proj", "out_proj")
        names = [n for n, _ in self.embed_tokens_extend.named_parameters()] + [n for n, _ in self.embed_tokens_extend.named_buffers()]
        for name in names:
            src = name
            if name.startswith("image_embed.img_processor."):
                rest = name[len("image_embed.img_processor."):]
                for a, b in tower.items():
                    if rest.startswith(a):
                        rest = b + rest[len(a):]
                if rest.startswith(("head.fc1.", "head.fc2.")):
                    rest = rest.replace("head.", "head.mlp.", 1)
                if rest.startswith("layers."):
                    parts = rest.split(".")
                    if parts[2] in attn:
                        parts.insert(2, "self_attn")
                    elif parts[2] in ("fc1", "fc2"):
                        parts.insert(2, "mlp")
                    rest = "encoder." + ".".join(parts)
                src = img + "img_processor." + rest
            elif name.startswith("image_embed."):
                src = img + name[len("image_embed."):]
            elif name.startswith("audio_embed.encoder."):
                rest = name[len("audio_embed.encoder."):]
                parts = rest.split(".")
                if rest.startswith(("global_mean", "global_invstd")):
                    rest = "encoder_embedding." + rest
                elif rest.startswith("conv_in."):
                    rest = "embed.conv.0." + parts[-1]
                elif rest.startswith("conv_dw."):
                    rest = f"embed.conv.{2 + 3 * int(parts[1])}." + parts[-1]
                elif rest.startswith("conv_pw."):
                    rest = f"embed.conv.{3 + 3 * int(parts[1])}." + parts[-1]
                elif rest.startswith("out."):
                    rest = "embed." + rest
                elif rest.startswith("bias_values."):
                    rest = "relative_attention_bias_layer." + rest
                elif rest.startswith("encoders."):
                    if parts[2] in ("q_proj", "k_proj", "v_proj", "o_proj"):
                        parts.insert(2, "self_attn")
                    elif parts[2] == "conv":
                        sub = {"glu_conv": "glu.ext_pw_conv_1d", "b1": "glu.b1", "b2": "glu.b2", "dw_conv": "dw_sep_conv_1d.dw_conv",
                               "pw_conv": "dw_sep_conv_1d.pw_conv"}
                        if parts[3] in sub:
                            parts[3] = sub[parts[3]]
                    rest = ".".join(parts)
                src = aud + "encoder." + rest
            elif name.startswith("audio_embed."):
                src = aud + name[len("audio_embed."):]
            rules.append(Rule("embed_tokens_extend." + name, [src]))
        return WeightMap(rules)


class Phi4MultimodalProcessor:
    """Prompt + images + audio clips -> model inputs: every image tag of the prompt is repeated once per feature row of the
    corresponding image, every audio tag once per row of the corresponding clip (the job of
    paddleformers/transformers/phi4_multimodal/processor.py). ``tokenizer`` must map ``image_token`` / ``audio_token`` to the
    placeholder ids of the model configuration."""

    def __init__(self, tokenizer, image_processor=None, audio_processor=None, image_token: str = "<|image|>", audio_token: str = "<|audio|>"):
        from ..transformers.audio_processing import KaldiFbankFeatureExtractor
        from ..transformers.image_processing import DynamicHDImageProcessor

        self.tokenizer = tokenizer
        self.image_processor = image_processor or DynamicHDImageProcessor()
        self.audio_processor = audio_processor or KaldiFbankFeatureExtractor()
        self.image_token, self.audio_token = image_token, audio_token

    def __call__(self, text: str, images=None, audio=None, sampling_rate: Optional[int] = None) -> dict:
        import re

        out = {}
        counts = {self.image_token: [], self.audio_token: []}
        if images is not None:
            pre = self.image_processor(list(images))
            counts[self.image_token] = list(pre.pop("num_img_tokens"))
            out.update(pre)
        if audio is not None:
            pre = self.audio_processor(list(audio), sampling_rate=sampling_rate)
            counts[self.audio_token] = [int(n) for n in pre["audio_embed_sizes"]]
            out.update(pre)
        for tag, per in counts.items():
            if text.count(tag) != len(per):
                raise ValueError(f"the prompt has {text.count(tag)} {tag} tags for {len(per)} inputs of that kind")
            it = iter(per)
            text = re.sub(re.escape(tag), lambda _m, tag=tag, it=it: tag * next(it), text)
        out["input_ids"] = torch.tensor([self.tokenizer.encode(text, add_special_tokens=False)])
        return out
