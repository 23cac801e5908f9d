"""Llama 4 with images (paddleformers/transformers/llama4: multimodal.py, modeling.py vision classes).

The vision tower is a ViT over fixed-size tiles: an unfold + linear patch projection, a class token appended after the patches,
learned positions, LayerNorm before and after the encoder, pre-LayerNorm blocks whose queries and keys are rotated in
interleaved pairs by the patch's column (first half of the pairs) and row (second half), and an adapter that folds 2 x 2
neighbouring patches into the channels (ratio 0.5 per side) before a two-layer GELU MLP. One bias-free linear layer maps the
adapter output to the decoder width. The decoder is the Llama 4 text model; image tokens are ordinary causal context.
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
from .modeling import DecoderForCausalLM
from .paligemma import PaliGemmaForConditionalGeneration

_VISION_DEFAULTS = dict(hidden_size=768, hidden_act="gelu", num_hidden_layers=34, num_attention_heads=16, num_channels=3, intermediate_size=5632,
                        vision_output_dim=7680, image_size=448, patch_size=14, norm_eps=1e-5, pixel_shuffle_ratio=0.5, projector_input_dim=4096,
                        projector_output_dim=4096, rope_theta=10000.0)


class Llama4Config(PretrainedConfig):
    model_type = "llama4"

    def __init__(self, text_config=None, vision_config=None, image_token_index=200092, boi_token_index=200080, eoi_token_index=200081, **kwargs):
        from .configuration import Llama4TextConfig

        kwargs.pop("model_type", None)
        text = text_config
        if not isinstance(text, PretrainedConfig):
            text = dict(text_config or {})
            text.pop("model_type", None)
            text = Llama4TextConfig(**text)
        kwargs.setdefault("tie_word_embeddings", bool(text.tie_word_embeddings))
        super().__init__(**{k: v for k, v in kwargs.items() if k != "vocab_size"})
        self.text_config = text
        vis = dict(vision_config or {})
        vis.pop("model_type", None)
        rp = vis.pop("rope_parameters", None) or {}
        if "rope_theta" in rp:
            vis["rope_theta"] = rp["rope_theta"]
        self.vision_config = {**_VISION_DEFAULTS, **vis}
        self.image_token_id = int(kwargs.get("image_token_id", image_token_index))
        self.boi_token_index, self.eoi_token_index = boi_token_index, eoi_token_index
        self.vocab_size = text.vocab_size

    @property
    def num_image_tokens(self) -> int:
        vc = self.vision_config
        return int((vc["image_size"] // vc["patch_size"]) ** 2 * vc["pixel_shuffle_ratio"] ** 2)

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        text = self.text_config.to_dict(saving)
        text["model_type"] = "llama4_text"
        vis = dict(self.vision_config, model_type="llama4_vision_model")
        vis["rope_parameters"] = {"rope_type": "default", "rope_theta": vis.pop("rope_theta")}
        d.update(text_config=text, vision_config=vis, image_token_index=self.image_token_id)
        d.pop("image_token_id", None)
        return d


class _Block(nn.Module):
    def __init__(self, vc: dict, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        H = vc["hidden_size"]
        self.heads, self.hd = vc["num_attention_heads"], H // vc["num_attention_heads"]
        self.input_layernorm, self.post_attention_layernorm = nn.LayerNorm(H, **kw), nn.LayerNorm(H, **kw)
        self.qkv = nn.Linear(H, 3 * H, **kw)
        self.o_proj = nn.Linear(H, H, **kw)
        self.fc1, self.fc2 = nn.Linear(H, vc["intermediate_size"], **kw), nn.Linear(vc["intermediate_size"], H, **kw)

    def forward(self, x, cos, sin):                       # cos / sin: [tokens, head_dim / 2]
        B, N, H = x.shape
        q, k, v = self.qkv(self.input_layernorm(x)).view(B, N, 3, self.heads, self.hd).unbind(2)

        def rot(t):                                       # pairs (2i, 2i + 1) rotate together
            a, b = t.float()[..., 0::2], t.float()[..., 1::2]
            c, s = cos[None, :, None, :], sin[None, :, None, :]
            return torch.stack([a * c - b * s, a * s + b * c], dim=-1).flatten(-2).to(t.dtype)

        o = F.flash_attention(rot(q), rot(k), v.contiguous(), causal=False).reshape(B, N, H)
        x = x + self.o_proj(o)
        return x + self.fc2(TF.gelu(self.fc1(self.post_attention_layernorm(x))))


class Llama4VisionModel(nn.Module):
    def __init__(self, vc: dict, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.vc = vc
        H, P = vc["hidden_size"], vc["patch_size"]
        self.side = vc["image_size"] // P
        self.patch_embedding = nn.Linear(vc["num_channels"] * P * P, H, bias=False, **kw)
        self.class_embedding = nn.Parameter(H ** -0.5 * torch.randn(H, **kw))
        self.positional_embedding_vlm = nn.Parameter(H ** -0.5 * torch.randn(self.side ** 2 + 1, H, **kw))
        self.layernorm_pre, self.layernorm_post = nn.LayerNorm(H, **kw), nn.LayerNorm(H, **kw)
        self.layers = nn.ModuleList([_Block(vc, **kw) for _ in range(vc["num_hidden_layers"])])
        self.adapter_fc1 = nn.Linear(vc["intermediate_size"], vc["projector_input_dim"], bias=False, **kw)
        self.adapter_fc2 = nn.Linear(vc["projector_output_dim"], vc["projector_output_dim"], bias=False, **kw)

    def angles(self, device) -> torch.Tensor:
        """[patches + 1, head_dim / 2]: the first half of the pairs turns with (column + 1), the second with (row + 1); the class
        token (last) is not rotated."""
        hd = self.vc["hidden_size"] // self.vc["num_attention_heads"]
        freq_dim = hd // 2
        inv = 1.0 / (self.vc["rope_theta"] ** (torch.arange(0, freq_dim, 2, device=device)[: freq_dim // 2].float() / freq_dim))
        idx = torch.arange(self.side ** 2, device=device)
        ang = torch.cat([((idx % self.side) + 1)[:, None] * inv[None], ((idx // self.side) + 1)[:, None] * inv[None]], dim=-1)
        return torch.cat([ang, torch.zeros(1, ang.shape[1], device=device)], dim=0)

    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """[tiles, C, H, W] -> [tiles, folded patches, projector_output_dim]."""
        B, C, Hh, Ww = pixel_values.shape
        P = self.vc["patch_size"]
        x = pixel_values.to(self.patch_embedding.weight.dtype).view(B, C, Hh // P, P, Ww // P, P).permute(0, 2, 4, 1, 3, 5)
        x = self.patch_embedding(x.reshape(B, -1, C * P * P))
        x = torch.cat([x, self.class_embedding.expand(B, 1, -1)], dim=1) + self.positional_embedding_vlm
        x = self.layernorm_pre(x)
        ang = self.angles(x.device)
        cos, sin = ang.cos(), ang.sin()
        for layer in self.layers:
            x = layer(x, cos, sin)
        x = self.layernorm_post(x)[:, :-1]
        # fold 2 x 2 neighbours into the channels, in the element order of the published checkpoints
        r = self.vc["pixel_shuffle_ratio"]
        n, ch = self.side, x.shape[-1]
        x = x.view(B, n, int(n * r), int(ch / r)).permute(0, 2, 1, 3).contiguous()
        x = x.view(B, int(n * r), int(n * r), int(ch / (r * r))).permute(0, 2, 1, 3).reshape(B, -1, int(ch / (r * r)))
        return TF.gelu(self.adapter_fc2(TF.gelu(self.adapter_fc1(x))))

    def weight_map(self) -> WeightMap:
        rules = [Rule("patch_embedding.weight", ["patch_embedding.linear.weight"]), Rule("class_embedding", ["class_embedding"]),
                 Rule("positional_embedding_vlm", ["positional_embedding_vlm"]),
                 Rule("adapter_fc1.weight", ["vision_adapter.mlp.fc1.weight"]), Rule("adapter_fc2.weight", ["vision_adapter.mlp.fc2.weight"])]
        for n in ("layernorm_pre", "layernorm_post"):
            rules += [Rule(f"{n}.{leaf}", [f"{n}.{leaf}"]) for leaf in ("weight", "bias")]
        for i in range(len(self.layers)):
            a, b = f"layers.{i}.", f"model.layers.{i}."
            for leaf in ("weight", "bias"):
                rules.append(Rule(a + f"qkv.{leaf}", [b + f"self_attn.{n}_proj.{leaf}" for n in "qkv"], "concat", 0))
                for mine, theirs in (("o_proj", "self_attn.o_proj"), ("input_layernorm", "input_layernorm"), ("fc1", "mlp.fc1"), ("fc2", "mlp.fc2"),
                                     ("post_attention_layernorm", "post_attention_layernorm")):
                    rules.append(Rule(a + f"{mine}.{leaf}", [b + f"{theirs}.{leaf}"]))
        return WeightMap(rules)


class Llama4ForConditionalGeneration(PaliGemmaForConditionalGeneration):
    config_class = Llama4Config
    _vision_name = "vision_model."
    _LAYOUTS = {"legacy": ("language_model.model.", "")}

    def __init__(self, config: Llama4Config, dtype=None, device=None):
        PretrainedModel.__init__(self, config)
        self.vision_tower = Llama4VisionModel(config.vision_config, dtype=dtype, device=device)
        self.projector = nn.Linear(config.vision_config["vision_output_dim"], config.text_config.hidden_size, bias=False, dtype=dtype, device=device)
        self.language = DecoderForCausalLM(config.text_config, dtype=dtype, device=device)
        self._layout = "legacy"
        self.post_init()

    def _init_weights(self, module):
        std = self.config.text_config.initializer_range
        if module is self.projector or (isinstance(module, nn.Linear) and any(module is m for m in self.vision_tower.modules())):
            nn.init.normal_(module.weight, 0.0, std)
            if module.bias is not None:
                nn.init.zeros_(module.bias)

    def image_features(self, pixel_values: torch.Tensor) -> torch.Tensor:
        feats = self.vision_tower(pixel_values)
        return self.projector(feats.reshape(-1, feats.shape[-1]))

    def two_way_tokens(self, input_ids, token_type_ids):
        return None

    def generation_token_types(self, prompt_len, total_len, batch, device):
        return None

    def projector_rules(self, prefix: str):
        return [Rule("projector.weight", [prefix + "multi_modal_projector.linear_1.weight"])]
