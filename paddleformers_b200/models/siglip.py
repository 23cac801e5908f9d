"""SigLIP vision encoder: the image tower used on its own for embeddings and as the vision side of several
vision-language families (paddleformers/transformers/siglip_vision_model).

A plain ViT: non-overlapping patch convolution (run as one GEMM over flattened patches), learned absolute position
embeddings, pre-LayerNorm blocks with biased fused q | k | v attention (full, non-causal) and a tanh-GELU MLP, a final
LayerNorm, and an optional pooling head (one learned probe attends over all patch tokens, then LayerNorm + MLP with a
residual). Attention runs on the flash attention path (``causal=False``); q / k / v of the checkpoint are fused into one
projection by the weight map.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from ..transformers.configuration_utils import PretrainedConfig
from ..transformers.conversion_utils import Rule, WeightMap
from ..transformers.model_utils import PretrainedModel


class SiglipVisionConfig(PretrainedConfig):
    model_type = "siglip_vision_model"

    def __init__(self, hidden_size=768, intermediate_size=3072, num_hidden_layers=12, num_attention_heads=12, num_channels=3,
                 image_size=224, patch_size=16, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6, vision_use_head=True, **kwargs):
        kwargs.pop("model_type", None)
        kwargs.pop("attention_dropout", None)
        super().__init__(hidden_size=hidden_size, num_hidden_layers=num_hidden_layers, num_attention_heads=num_attention_heads,
                         **{k: v for k, v in kwargs.items() if k != "vocab_size"})
        self.intermediate_size, self.num_channels = intermediate_size, num_channels
        self.image_size, self.patch_size = image_size, patch_size
        self.hidden_act, self.layer_norm_eps, self.vision_use_head = hidden_act, layer_norm_eps, vision_use_head

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            d.pop("vocab_size", None)
            d.pop("tie_word_embeddings", None)
        return d


def _act(name: str):
    if name == "gelu_pytorch_tanh":
        return lambda x: TF.gelu(x, approximate="tanh")
    if name == "quick_gelu":
        return lambda x: x * torch.sigmoid(1.702 * x)
    return getattr(TF, name)


class _Block(nn.Module):
    def __init__(self, cfg: SiglipVisionConfig, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        H = cfg.hidden_size
        self.heads, self.hd = cfg.num_attention_heads, H // cfg.num_attention_heads
        self.layer_norm1 = nn.LayerNorm(H, eps=cfg.layer_norm_eps, **kw)
        self.layer_norm2 = nn.LayerNorm(H, eps=cfg.layer_norm_eps, **kw)
        self.qkv = nn.Linear(H, 3 * H, **kw)
        self.out_proj = nn.Linear(H, H, **kw)
        self.fc1 = nn.Linear(H, cfg.intermediate_size, **kw)
        self.fc2 = nn.Linear(cfg.intermediate_size, H, **kw)
        self.act = _act(cfg.hidden_act)

    def forward(self, x):                                  # [B, N, H]
        B, N, H = x.shape
        q, k, v = self.qkv(self.layer_norm1(x)).view(B, N, 3, self.heads, self.hd).unbind(2)
        a = F.flash_attention(q, k, v, causal=False).reshape(B, N, H)
        x = x + self.out_proj(a)
        return x + self.fc2(self.act(self.fc1(self.layer_norm2(x))))


class _PoolingHead(nn.Module):
    """One learned query ("probe") attends over all tokens; LayerNorm + MLP with a residual on the pooled vector."""

    def __init__(self, cfg: SiglipVisionConfig, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        H = cfg.hidden_size
        self.heads = cfg.num_attention_heads
        self.probe = nn.Parameter(torch.randn(1, 1, H, **kw))
        self.in_proj_weight = nn.Parameter(torch.empty(3 * H, H, **kw))
        self.in_proj_bias = nn.Parameter(torch.zeros(3 * H, **kw))
        nn.init.xavier_uniform_(self.in_proj_weight)
        self.out_proj = nn.Linear(H, H, **kw)
        self.layernorm = nn.LayerNorm(H, eps=cfg.layer_norm_eps, **kw)
        self.fc1 = nn.Linear(H, cfg.intermediate_size, **kw)
        self.fc2 = nn.Linear(cfg.intermediate_size, H, **kw)
        self.act = _act(cfg.hidden_act)

    def forward(self, x):
        B, N, H = x.shape
        hd = H // self.heads
        wq, wk, wv = self.in_proj_weight.chunk(3, dim=0)
        bq, bk, bv = self.in_proj_bias.chunk(3, dim=0)
        q = TF.linear(self.probe.expand(B, 1, H), wq, bq).view(B, 1, self.heads, hd).transpose(1, 2)
        k = TF.linear(x, wk, bk).view(B, N, self.heads, hd).transpose(1, 2)
        v = TF.linear(x, wv, bv).view(B, N, self.heads, hd).transpose(1, 2)
        p = torch.softmax((q.float() @ k.float().transpose(-1, -2)) * hd ** -0.5, dim=-1)
        pooled = self.out_proj((p @ v.float()).to(x.dtype).transpose(1, 2).reshape(B, 1, H))
        pooled = pooled + self.fc2(self.act(self.fc1(self.layernorm(pooled))))
        return pooled[:, 0]


class SiglipVisionModel(PretrainedModel):
    config_class = SiglipVisionConfig

    def __init__(self, config: SiglipVisionConfig, dtype=None, device=None):
        super().__init__(config)
        kw = dict(dtype=dtype, device=device)
        H, P = config.hidden_size, config.patch_size
        self.patch_embedding = nn.Linear(config.num_channels * P * P, H, **kw)          # the patch convolution as a GEMM
        self.position_embedding = nn.Embedding((config.image_size // P) ** 2, H, **kw)
        self.layers = nn.ModuleList([_Block(config, **kw) for _ in range(config.num_hidden_layers)])
        self.post_layernorm = nn.LayerNorm(H, eps=config.layer_norm_eps, **kw)
        self.head = _PoolingHead(config, **kw) if config.vision_use_head else None
        self.post_init()

    def _init_weights(self, module):
        if isinstance(module, (nn.Linear, nn.Embedding)):
            nn.init.normal_(module.weight, 0.0, self.config.initializer_range)
            if getattr(module, "bias", None) is not None:
                nn.init.zeros_(module.bias)

    def patches(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """[B, C, H, W] -> [B, (H / P)(W / P), C P P] in the convolution's weight layout (channel, row, column)."""
        B, C, Hh, Ww = pixel_values.shape
        P = self.config.patch_size
        x = pixel_values.view(B, C, Hh // P, P, Ww // P, P).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(B, (Hh // P) * (Ww // P), C * P * P)

    def forward(self, pixel_values: torch.Tensor, feature_layer: Optional[int] = None):
        """Returns (last_hidden_state [B, N, H], pooled [B, H] or None). With ``feature_layer`` (an index into [embeddings,
        block 1, ..., block N], negative from the end) the first element is that intermediate state, without the final
        LayerNorm, and nothing is pooled."""
        x = self.patch_embedding(self.patches(pixel_values.to(self.patch_embedding.weight.dtype)))
        x = x + self.position_embedding.weight[None, :x.shape[1]]
        if feature_layer is not None:
            stop = feature_layer if feature_layer >= 0 else len(self.layers) + 1 + feature_layer
            for blk in self.layers[:stop]:
                x = blk(x)
            return x, None
        for blk in self.layers:
            x = blk(x)
        x = self.post_layernorm(x)
        return x, (self.head(x) if self.head is not None else None)

    def weight_map(self) -> WeightMap:
        cfg = self.config
        P, H, C = cfg.patch_size, cfg.hidden_size, cfg.num_channels
        v = "vision_model."
        rules = [Rule("patch_embedding.weight", [v + "embeddings.patch_embedding.weight"], reshape=[H, -1], source_shape=[H, C, P, P]),
                 Rule("patch_embedding.bias", [v + "embeddings.patch_embedding.bias"]),
                 Rule("position_embedding.weight", [v + "embeddings.position_embedding.weight"]),
                 Rule("post_layernorm.weight", [v + "post_layernorm.weight"]), Rule("post_layernorm.bias", [v + "post_layernorm.bias"])]
        for i in range(cfg.num_hidden_layers):
            a, b = f"layers.{i}.", v + f"encoder.layers.{i}."
            for leaf in ("weight", "bias"):
                rules.append(Rule(a + f"qkv.{leaf}", [b + f"self_attn.{n}_proj.{leaf}" for n in "qkv"], "concat", 0))
                for mine, theirs in (("out_proj", "self_attn.out_proj"), ("layer_norm1", "layer_norm1"), ("layer_norm2", "layer_norm2"),
                                     ("fc1", "mlp.fc1"), ("fc2", "mlp.fc2")):
                    rules.append(Rule(a + f"{mine}.{leaf}", [b + f"{theirs}.{leaf}"]))
        if self.head is not None:
            h = v + "head."
            rules += [Rule("head.probe", [h + "probe"]), Rule("head.in_proj_weight", [h + "attention.in_proj_weight"]),
                      Rule("head.in_proj_bias", [h + "attention.in_proj_bias"])]
            for leaf in ("weight", "bias"):
                for mine, theirs in (("out_proj", "attention.out_proj"), ("layernorm", "layernorm"), ("fc1", "mlp.fc1"), ("fc2", "mlp.fc2")):
                    rules.append(Rule(f"head.{mine}.{leaf}", [h + f"{theirs}.{leaf}"]))
        return WeightMap(rules)
