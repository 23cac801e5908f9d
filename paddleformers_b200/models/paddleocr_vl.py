"""PaddleOCR-VL (paddleformers/transformers/paddleocr_vl): a variable-resolution SigLIP-style encoder in front of an ERNIE-4.5
style dense decoder with multimodal rotary sections.

Vision: patches in raster order, the learned position table resampled bilinearly to every image's own grid, pre-LayerNorm blocks
with biased projections whose queries and keys carry a 2-D rotary embedding (rows on the first quarter of the frequencies,
columns on the second), full attention inside each image; then a LayerNorm, 2 x 2 neighbouring patches joined into one token and
a two-layer GELU MLP to the decoder width. Text: Llama-shaped blocks with half-split rotary pairs; the three position streams
(time, row, column) select the rotary angle per frequency section, as in Qwen2-VL, whose forward pass this model reuses.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from ..transformers.configuration_utils import PretrainedConfig
from ..transformers.conversion_utils import Rule, WeightMap
from ..transformers.model_utils import PretrainedModel
from .modeling import DecoderForCausalLM, build_weight_map
from .vision_language import Qwen2VLForConditionalGeneration


class PaddleOCRVLConfig(PretrainedConfig):
    model_type = "paddleocr_vl"

    def __init__(self, text_config=None, vision_config=None, image_token_id=100295, video_token_id=100296, vision_start_token_id=101305,
                 vision_end_token_id=101306, **kwargs):
        from .configuration import LlamaConfig

        kwargs.pop("model_type", None)
        text = dict(text_config or {})
        text.pop("model_type", None)
        rp = dict(text.get("rope_parameters") or {})
        rs = dict(text.pop("rope_scaling", None) or {})
        self_section = list(rp.pop("mrope_section", None) or rs.get("mrope_section") or [16, 24, 24])
        if "rope_parameters" in text:
            text["rope_parameters"] = rp
        bias = bool(text.pop("use_bias", False))
        text.setdefault("attention_bias", bias)
        text.setdefault("mlp_bias", bias)
        text.setdefault("tie_word_embeddings", bool(kwargs.get("tie_word_embeddings", True)))
        text.setdefault("rms_norm_eps", 1e-5)
        kwargs.setdefault("tie_word_embeddings", bool(text["tie_word_embeddings"]))
        super().__init__(**{k: v for k, v in kwargs.items() if k != "vocab_size"})
        self.text_config = LlamaConfig(**text)
        self.mrope_section = self_section
        vis = dict(vision_config or {})
        vis.pop("model_type", None)
        self.vision_config = {"hidden_size": 1152, "intermediate_size": 4304, "num_hidden_layers": 27, "num_attention_heads": 16,
                              "num_channels": 3, "image_size": 384, "patch_size": 14, "hidden_act": "gelu_pytorch_tanh", "layer_norm_eps": 1e-6,
                              "spatial_merge_size": 2, **vis}
        self.image_token_id, self.video_token_id = image_token_id, video_token_id
        self.vision_start_token_id, self.vision_end_token_id = vision_start_token_id, vision_end_token_id
        self.vocab_size = self.text_config.vocab_size

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        text = self.text_config.to_dict(saving)
        text["model_type"] = "paddleocr_vl_text"
        text["use_bias"] = bool(self.text_config.attention_bias)
        scaling = text.pop("rope_scaling", None) or {}
        text["rope_parameters"] = {"rope_type": "default", **scaling, "rope_theta": text.pop("rope_theta", self.text_config.rope_theta),
                                   "mrope_section": self.mrope_section}
        d["text_config"] = text
        d["vision_config"] = dict(self.vision_config, model_type="paddleocr_vl_vision")
        d.pop("mrope_section", None)
        return d


class _Block(nn.Module):
    def __init__(self, vc: dict, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        H = vc["hidden_size"]
        self.heads, self.hd = vc["num_attention_heads"], H // vc["num_attention_heads"]
        self.layer_norm1 = nn.LayerNorm(H, eps=vc["layer_norm_eps"], **kw)
        self.layer_norm2 = nn.LayerNorm(H, eps=vc["layer_norm_eps"], **kw)
        self.qkv, self.out_proj = nn.Linear(H, 3 * H, **kw), nn.Linear(H, H, **kw)
        self.fc1, self.fc2 = nn.Linear(H, vc["intermediate_size"], **kw), nn.Linear(vc["intermediate_size"], H, **kw)
        self.tanh_gelu = vc["hidden_act"] == "gelu_pytorch_tanh"

    def forward(self, x, cos, sin, lengths: List[int]):          # x [N, H]; cos / sin [N, head_dim / 2]
        N = x.shape[0]
        q, k, v = self.qkv(self.layer_norm1(x)).view(N, 3, self.heads, self.hd).unbind(1)
        half = self.hd // 2

        def rot(t):
            a, b = t[..., :half].float(), t[..., half:].float()
            c, s = cos[:, None, :], sin[:, None, :]
            return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(t.dtype)

        q, k = rot(q), rot(k)
        outs, off = [], 0
        for n in lengths:
            sl = slice(off, off + n)
            outs.append(F.flash_attention(q[sl][None], k[sl][None], v[sl][None].contiguous(), causal=False)[0])
            off += n
        x = x + self.out_proj(torch.cat(outs, dim=0).reshape(N, -1))
        h = self.fc1(self.layer_norm2(x))
        return x + self.fc2(TF.gelu(h, approximate="tanh") if self.tanh_gelu else TF.gelu(h))


class PaddleOCRVisionTower(nn.Module):
    def __init__(self, vc: dict, text_hidden: int, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.vc = vc
        H, P, ms = vc["hidden_size"], vc["patch_size"], vc["spatial_merge_size"]
        self.patch_embedding = nn.Linear(vc["num_channels"] * P * P, H, **kw)
        self.side = vc["image_size"] // P
        self.position_embedding = nn.Embedding(self.side ** 2, H, **kw)
        self.layers = nn.ModuleList([_Block(vc, **kw) for _ in range(vc["num_hidden_layers"])])
        self.post_layernorm = nn.LayerNorm(H, eps=vc["layer_norm_eps"], **kw)
        self.pre_norm = nn.LayerNorm(H, eps=1e-5, **kw)
        self.linear_1 = nn.Linear(H * ms * ms, H * ms * ms, **kw)
        self.linear_2 = nn.Linear(H * ms * ms, text_hidden, **kw)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """pixel_values [patches, C, P, P] (or flattened), patches of every image in raster order -> [merged patches, text hidden]."""
        vc, ms = self.vc, self.vc["spatial_merge_size"]
        x = self.patch_embedding(pixel_values.reshape(pixel_values.shape[0], -1).to(self.patch_embedding.weight.dtype))
        table = self.position_embedding.weight.view(1, self.side, self.side, -1).permute(0, 3, 1, 2).float()
        hd = vc["hidden_size"] // vc["num_attention_heads"]
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, device=x.device, dtype=torch.float32) / (hd // 2)))
        pos, angles, lengths = [], [], []
        for t, h, w in grid_thw.tolist():
            p = TF.interpolate(table, size=(h, w), mode="bilinear", align_corners=False).permute(0, 2, 3, 1).reshape(h * w, -1)
            pos.append(p.to(x.dtype).repeat(t, 1))
            idx = torch.arange(h * w, device=x.device)
            ang = torch.cat([(idx // w)[:, None] * inv[None], (idx % w)[:, None] * inv[None]], dim=-1)       # rows, then columns
            angles.append(ang.repeat(t, 1))
            lengths += [h * w] * t
        x = x + torch.cat(pos, dim=0)
        ang = torch.cat(angles, dim=0)
        cos, sin = ang.cos(), ang.sin()
        for layer in self.layers:
            x = layer(x, cos, sin, lengths)
        x = self.pre_norm(self.post_layernorm(x))
        out, off = [], 0
        for t, h, w in grid_thw.tolist():                      # join every 2 x 2 block of the raster into one token
            n = t * h * w
            f = x[off:off + n].view(t, h // ms, ms, w // ms, ms, -1).transpose(2, 3).reshape(t * (h // ms) * (w // ms), -1)
            out.append(self.linear_2(TF.gelu(self.linear_1(f))))
            off += n
        return torch.cat(out, dim=0)


class PaddleOCRVLForConditionalGeneration(Qwen2VLForConditionalGeneration):
    config_class = PaddleOCRVLConfig

    def __init__(self, config: PaddleOCRVLConfig, dtype=None, device=None):
        PretrainedModel.__init__(self, config)
        self.visual = PaddleOCRVisionTower(config.vision_config, config.text_config.hidden_size, dtype=dtype, device=device)
        self.language = DecoderForCausalLM(config.text_config, dtype=dtype, device=device)
        self.post_init()

    def _init_weights(self, module):
        if isinstance(module, (nn.Linear, nn.Embedding)) and any(module is m for m in self.visual.modules()):
            nn.init.normal_(module.weight, 0.0, self.config.text_config.initializer_range)
            if getattr(module, "bias", None) is not None:
                nn.init.zeros_(module.bias)

    def load_hf_checkpoint(self, directory: str, strict: bool = False) -> None:
        PretrainedModel.load_hf_checkpoint(self, directory, strict)

    def weight_map(self) -> WeightMap:
        vc = self.config.vision_config
        H, C, P = vc["hidden_size"], vc["num_channels"], vc["patch_size"]
        text_map = build_weight_map(self.config.text_config)
        rules = [Rule("language." + r.target, list(r.sources), r.op, r.dim, sizes=r.sizes) for r in text_map.rules.values()]
        known = {r.target for r in rules}
        rules += [Rule("language." + n, [text_map.translate(n)]) for n, _ in self.language.named_parameters() if "language." + n not in known]
        v = "model.visual.vision_model."
        rules += [Rule("visual.patch_embedding.weight", [v + "embeddings.patch_embedding.weight"], reshape=[H, -1], source_shape=[H, C, P, P]),
                  Rule("visual.patch_embedding.bias", [v + "embeddings.patch_embedding.bias"]),
                  Rule("visual.position_embedding.weight", [v + "embeddings.position_embedding.weight"])]
        for leaf in ("weight", "bias"):
            rules += [Rule(f"visual.post_layernorm.{leaf}", [v + f"post_layernorm.{leaf}"])]
            rules += [Rule(f"visual.{n}.{leaf}", [f"mlp_AR.{n}.{leaf}"]) for n in ("pre_norm", "linear_1", "linear_2")]
            for i in range(vc["num_hidden_layers"]):
                a, b = f"visual.layers.{i}.", v + f"encoder.layers.{i}."
                rules.append(Rule(a + f"qkv.{leaf}", [b + f"self_attn.{n}_proj.{leaf}" for n in "qkv"], "concat", 0))
                rules += [Rule(a + f"{mine}.{leaf}", [b + f"{theirs}.{leaf}"]) for mine, theirs in
                          (("out_proj", "self_attn.out_proj"), ("layer_norm1", "layer_norm1"), ("layer_norm2", "layer_norm2"),
                           ("fc1", "mlp.fc1"), ("fc2", "mlp.fc2"))]
        return WeightMap(rules)
