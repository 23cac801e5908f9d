"""Molmo: a CLIP-style image tower whose multi-crop patch features are pooled and ADDED to the token embeddings of a
post-norm (or pre-norm) decoder (paddleformers/transformers/molmo/modeling.py:154-365 decoder, :379-701 vision backbone,
:943-1170 embedding and model, :716-830 checkpoint names; configuration.py).

* Tower: patches arrive already flattened ([crops, patches, 3 * p * p]); linear patch embedding without bias, class token,
  learned positions (bicubically resized when the grid differs), LayerNorm, pre-LayerNorm blocks with quick-GELU MLPs. The
  outputs of the layers listed in ``vit_layers`` are concatenated along the features; crops that are all padding (-1) are
  zeroed.
* Padding embeddings: one learned vector is added to patches that are all padding, another to patches that are partly padding
  (``image_masks`` holds the valid fraction of every patch).
* Pooling: every 2 x 2 block of patches is reduced to one row by attention whose query is the block's mean; a SwiGLU MLP
  projects to the decoder width.
* The rows are added at the sequence positions given by ``image_input_idx`` (-1: unused row).
* Decoder: the unified decoder with norms after each branch (``norm_after``) or before, one RMSNorm over all heads' query / key
  features (``attention_layer_norm``), optionally clamped projections (``clip_qkv``); the vocabulary is the base table followed
  by ``additional_vocab_size`` extra rows, the output head covers the base table only.

Checkpoint tensors keep the published names (``model.transformer.wte.embedding``, ``blocks.N.att_proj`` ...,
``model.vision_backbone.*``); the fused ``ff_proj`` stores [up | gate], which is swapped into the kernels' [gate | up] order.
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
from .configuration import DecoderConfig
from .modeling import CausalLMOutput, DecoderForCausalLM

_VISION = {"image_default_input_size": (336, 336), "image_patch_size": 14, "image_pos_patch_size": 14, "image_emb_dim": 1024,
           "image_num_heads": 16, "image_num_key_value_heads": 16, "image_num_layers": 23, "image_head_dim": 64,
           "image_mlp_dim": 4096, "image_mlp_activations": "quick_gelu", "image_num_pos": 577, "image_norm_eps": 1e-5}


class MolmoTextConfig(DecoderConfig):
    model_type = "molmo_text"

    def __init__(self, norm_after=True, attention_layer_norm=True, clip_qkv=None, **kw):
        super().__init__(**kw)
        self.block_style = "post" if norm_after else "pre"
        self.qk_norm_full = bool(attention_layer_norm)
        self.clip_qkv = clip_qkv


class MolmoConfig(PretrainedConfig):
    model_type = "molmo"

    def __init__(self, vocab_size=100278, embedding_size=100352, hidden_size=4096, intermediate_size=22016, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=None, attention_layer_norm=True, norm_after=True, layer_norm_type="rms",
                 layer_norm_eps=1e-6, additional_vocab_size=128, qkv_bias=False, clip_qkv=None, rope_theta=500000.0, rope_impl="llama",
                 max_position_embeddings=4096, weight_tying=False, head_dim=None, vision_backbone=None,
                 image_padding_embed="pad_and_partial_pad", vit_layers=(-2, -9), image_pooling_h=2, image_pooling_w=2,
                 image_pooling_2d="attention-meanq", image_projector="mlp", activation_type="swiglu", **kwargs):
        if layer_norm_type != "rms" or activation_type != "swiglu" or image_pooling_2d != "attention-meanq" or image_projector != "mlp":
            raise NotImplementedError("Molmo: RMSNorm, SwiGLU, attention-meanq pooling and the MLP projector are implemented")
        if rope_impl not in ("llama", "half"):
            raise NotImplementedError("Molmo: the half-split rotary layout (rope_impl llama) is implemented")
        if image_padding_embed not in (None, "pad_and_partial_pad"):
            raise NotImplementedError(f"Molmo: image_padding_embed {image_padding_embed!r}")
        kwargs["tie_word_embeddings"] = bool(kwargs.get("tie_word_embeddings", weight_tying) or weight_tying)
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, num_hidden_layers=num_hidden_layers,
                         num_attention_heads=num_attention_heads, **kwargs)
        self.embedding_size = embedding_size if embedding_size is not None else vocab_size
        self.additional_vocab_size = int(additional_vocab_size or 0)
        self.intermediate_size, self.num_key_value_heads = intermediate_size, num_key_value_heads or num_attention_heads
        self.attention_layer_norm, self.norm_after, self.layer_norm_type, self.layer_norm_eps = attention_layer_norm, norm_after, layer_norm_type, layer_norm_eps
        self.qkv_bias, self.clip_qkv, self.rope_theta, self.rope_impl = qkv_bias, clip_qkv, rope_theta, rope_impl
        self.max_position_embeddings, self.weight_tying = max_position_embeddings, self.tie_word_embeddings
        self.head_dim = head_dim or hidden_size // num_attention_heads
        self.activation_type = activation_type
        vb = None
        if vision_backbone is not False:
            vb = dict(_VISION, **(vision_backbone or {}))
            vb["image_default_input_size"] = tuple(vb["image_default_input_size"])
        self.vision_backbone = vb
        self.image_padding_embed, self.vit_layers = image_padding_embed, tuple(vit_layers) if vit_layers is not None else None
        self.image_pooling_h, self.image_pooling_w = image_pooling_h, image_pooling_w
        self.image_pooling_2d, self.image_projector = image_pooling_2d, image_projector

    @property
    def image_num_patch(self):
        size, p = self.vision_backbone["image_default_input_size"], self.vision_backbone["image_patch_size"]
        return size[0] // p, size[1] // p

    def llm_patches_per_crop(self):
        h, w = self.image_num_patch
        return (h + self.image_pooling_h - 1) // self.image_pooling_h, (w + self.image_pooling_w - 1) // self.image_pooling_w

    def text_config(self) -> MolmoTextConfig:
        """The decoder as the unified decoder sees it: one embedding table of base + extra rows, the fused MLP width halved."""
        return MolmoTextConfig(
            vocab_size=self.embedding_size + self.additional_vocab_size, hidden_size=self.hidden_size,
            intermediate_size=self.intermediate_size // 2, num_hidden_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads, num_key_value_heads=self.num_key_value_heads, head_dim=self.head_dim,
            rms_norm_eps=self.layer_norm_eps, rope_theta=self.rope_theta, attention_bias=self.qkv_bias,
            max_position_embeddings=self.max_position_embeddings, norm_after=self.norm_after,
            attention_layer_norm=self.attention_layer_norm, clip_qkv=self.clip_qkv, tie_word_embeddings=True, dtype=self.dtype,
            rope_scaling=getattr(self, "rope_scaling", None))


def _quick_gelu(x):
    return x * torch.sigmoid(1.702 * x)


class _VisionAttention(nn.Module):
    def __init__(self, vc, in_dim: int, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.heads, self.kv_heads, self.hd = vc["image_num_heads"], vc["image_num_key_value_heads"], vc["image_head_dim"]
        self.wq = nn.Linear(in_dim, self.heads * self.hd, **kw)
        self.wk = nn.Linear(in_dim, self.kv_heads * self.hd, **kw)
        self.wv = nn.Linear(in_dim, self.kv_heads * self.hd, **kw)
        self.wo = nn.Linear(self.heads * self.hd, vc["image_emb_dim"], **kw)

    def forward(self, xq, xkv=None):
        xkv = xq if xkv is None else xkv
        N, Q, _ = xq.shape
        q = self.wq(xq).view(N, Q, self.heads, self.hd).transpose(1, 2)
        k = self.wk(xkv).view(N, -1, self.kv_heads, self.hd).transpose(1, 2)
        v = self.wv(xkv).view(N, -1, self.kv_heads, self.hd).transpose(1, 2)
        if self.heads != self.kv_heads:
            k, v = (t.repeat_interleave(self.heads // self.kv_heads, dim=1) for t in (k, v))
        a = TF.scaled_dot_product_attention(q.float(), k.float(), v.float()).to(xq.dtype)       # scores and softmax in fp32
        return self.wo(a.transpose(1, 2).reshape(N, Q, self.heads * self.hd))


class _VisionBlock(nn.Module):
    def __init__(self, vc, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        D = vc["image_emb_dim"]
        self.attention = _VisionAttention(vc, D, **kw)
        self.feed_forward = nn.ModuleDict({"w1": nn.Linear(D, vc["image_mlp_dim"], **kw), "w2": nn.Linear(vc["image_mlp_dim"], D, **kw)})
        self.attention_norm, self.ffn_norm = nn.LayerNorm(D, eps=vc["image_norm_eps"], **kw), nn.LayerNorm(D, eps=vc["image_norm_eps"], **kw)
        self.act = _quick_gelu if vc.get("image_mlp_activations", "quick_gelu") == "quick_gelu" else TF.gelu

    def forward(self, x):
        x = x + self.attention(self.attention_norm(x))
        return x + self.feed_forward["w2"](self.act(self.feed_forward["w1"](self.ffn_norm(x))))


class _Resblocks(nn.Module):
    def __init__(self, vc, dtype=None, device=None):
        super().__init__()
        self.resblocks = nn.ModuleList([_VisionBlock(vc, dtype=dtype, device=device) for _ in range(vc["image_num_layers"])])


class MolmoVisionTransformer(nn.Module):
    def __init__(self, vc, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        D, p = vc["image_emb_dim"], vc["image_patch_size"]
        self.class_embedding = nn.Parameter(torch.zeros(D, **kw))
        self.positional_embedding = nn.Parameter(torch.zeros(vc["image_num_pos"], D, **kw))
        self.patch_embedding = nn.Linear(p * p * 3, D, bias=False, **kw)
        self.pre_ln = nn.LayerNorm(D, eps=vc["image_norm_eps"], **kw)
        self.transformer = _Resblocks(vc, **kw)

    def positions(self, grid) -> torch.Tensor:
        cls, pos = self.positional_embedding[:1], self.positional_embedding[1:]
        side = int(math.sqrt(pos.shape[0]))
        pos = pos.reshape(side, side, -1)
        if (side, side) != tuple(grid):
            pos = TF.interpolate(pos.permute(2, 0, 1)[None].float(), size=tuple(grid), mode="bicubic", align_corners=False)[0]
            pos = pos.permute(1, 2, 0).to(cls.dtype)
        return torch.cat([cls, pos.reshape(-1, pos.shape[-1])], dim=0)

    def forward(self, patches, grid):
        """patches [N, P, 3 p p] -> the output of every block, each [N, 1 + P, D]."""
        x = self.patch_embedding(patches)
        x = torch.cat([self.class_embedding.view(1, 1, -1).expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1)
        x = x + self.positions(grid).to(x.dtype)
        x = TF.layer_norm(x.float(), x.shape[-1:], self.pre_ln.weight.float(), self.pre_ln.bias.float(), self.pre_ln.eps).to(x.dtype)
        outs = []
        for blk in self.transformer.resblocks:
            x = blk(x)
            outs.append(x)
        return outs


class MolmoVisionBackbone(nn.Module):
    def __init__(self, config: MolmoConfig, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.config = config
        vc = config.vision_backbone
        self.image_vit = MolmoVisionTransformer(vc, **kw)
        n = len(config.vit_layers) if config.vit_layers is not None else 1
        dim = vc["image_emb_dim"] * n
        self.pad_embed = nn.Parameter(torch.zeros(2, dim, **kw)) if config.image_padding_embed else None
        self.image_pooling_2d = _VisionAttention(vc, dim, **kw)
        hidden = config.intermediate_size // 2
        self.image_projector = nn.ModuleDict({"w1": nn.Linear(vc["image_emb_dim"], hidden, bias=False, **kw),
                                              "w2": nn.Linear(hidden, config.hidden_size, bias=False, **kw),
                                              "w3": nn.Linear(vc["image_emb_dim"], hidden, bias=False, **kw)})

    def forward(self, images: torch.Tensor, image_masks: torch.Tensor) -> torch.Tensor:
        """images [B, crops, patches, 3 p p] (all -1: an unused crop), image_masks [B, crops, patches] (valid fraction of every
        patch) -> [B, crops, pooled patches, hidden]."""
        cfg = self.config
        B, C, P, px = images.shape
        flat = images.reshape(B * C, P, px)
        used = ~(flat == -1).all(dim=2).all(dim=1)
        outs = self.image_vit(flat.to(self.image_vit.patch_embedding.weight.dtype), cfg.image_num_patch)
        feats = torch.cat([outs[i] for i in cfg.vit_layers], dim=-1) if cfg.vit_layers is not None else outs[-1]
        feats = feats[:, 1:] * used[:, None, None].to(feats.dtype)                       # the class token is dropped
        feats = feats.reshape(B, C, P, -1)
        if self.pad_embed is not None:
            all_pad = (image_masks == 0)
            partial = (image_masks < 1) & ~all_pad
            feats = feats + self.pad_embed[0] * all_pad[..., None].to(feats.dtype) + self.pad_embed[1] * partial[..., None].to(feats.dtype)
        h, w = cfg.image_num_patch
        ph, pw = cfg.image_pooling_h, cfg.image_pooling_w
        feats = feats.reshape(B, C, h, w, -1)
        feats = TF.pad(feats, (0, 0, 0, (-w) % pw, 0, (-h) % ph))                         # zero rows / columns up to whole blocks
        hb, wb = feats.shape[2] // ph, feats.shape[3] // pw
        blocks = feats.reshape(B, C, hb, ph, wb, pw, -1).permute(0, 1, 2, 4, 3, 5, 6).reshape(B * C * hb * wb, ph * pw, -1)
        pooled = self.image_pooling_2d(blocks.mean(dim=1, keepdim=True), blocks).reshape(B, C, hb * wb, -1)
        pr = self.image_projector
        return pr["w2"](TF.silu(pr["w1"](pooled)) * pr["w3"](pooled))


class _Body(nn.Module):
    def __init__(self, config, dtype=None, device=None):
        super().__init__()
        self.vision_backbone = MolmoVisionBackbone(config, dtype=dtype, device=device) if config.vision_backbone else None


class MolmoForCausalLM(PretrainedModel):
    config_class = MolmoConfig

    def __init__(self, config: MolmoConfig, dtype=None, device=None):
        super().__init__(config)
        self.model = _Body(config, dtype=dtype, device=device)
        self.language = DecoderForCausalLM(config.text_config(), dtype=dtype, device=device)
        E = config.embedding_size
        self.lm_head = None if config.tie_word_embeddings else nn.Linear(config.hidden_size, E, bias=False, dtype=dtype, device=device)
        if self.lm_head is not None:
            nn.init.normal_(self.lm_head.weight, 0.0, config.initializer_range)

    def head_weight(self):
        if self.lm_head is not None:
            return self.lm_head.weight
        return self.language.model.embed_tokens.weight[:self.config.embedding_size]       # the head covers the base table only

    def forward(self, input_ids, images=None, image_masks=None, image_input_idx=None, labels=None, position_ids=None,
                attn_mask_startend_row_indices=None, return_logits: Optional[bool] = None, **unused):
        lm = self.language
        B, S = input_ids.shape
        h = lm.model.embed(input_ids, whole=True)                                                      # [B * S, H]
        if images is not None:
            if self.model.vision_backbone is None:
                raise ValueError("this Molmo configuration has no vision backbone")
            if image_masks is None or image_input_idx is None:
                raise ValueError("images need image_masks and image_input_idx")
            feats = self.model.vision_backbone(images, image_masks)
            C, Pp = feats.shape[1:3]
            if tuple(image_input_idx.shape) != (B, C, Pp):
                raise ValueError(f"image_input_idx {tuple(image_input_idx.shape)} does not match (batch {B}, crops {C}, rows {Pp})")
            idx = image_input_idx.reshape(B, C * Pp)
            valid = idx >= 0
            rows = (torch.arange(B, device=idx.device)[:, None] * S + idx.clamp(min=0)).reshape(-1)
            add = (feats.reshape(B * C * Pp, -1) * valid.reshape(-1, 1)).to(h.dtype)
            h = h.index_add(0, rows, add)
        kend = attn_mask_startend_row_indices.reshape(B, -1) if attn_mask_startend_row_indices is not None else None
        ctx = lm.model.make_context(input_ids, position_ids, kend)
        hidden, residual = lm.model.run_layers(lm.model.token_slice(h), None, ctx)
        hidden = lm.model.norm(hidden, residual)[0] if residual is not None else lm.model.norm(hidden)
        out = CausalLMOutput()
        if return_logits if return_logits is not None else labels is None:
            out.logits = TF.linear(hidden, self.head_weight()).view(B, S, -1)
        if labels is not None:
            lab = labels.reshape(-1)
            count = (lab != lm.ignore_index).sum()
            scale = 1.0 / (count.clamp(min=1).to(torch.float32) * float(lm.loss_accumulation_steps))
            out.loss, _ = F.fused_linear_cross_entropy(hidden, self.head_weight(), lab, lm.ignore_index, 2048, scale)
            out.num_tokens = count
        return out

    @property
    def loss_accumulation_steps(self):
        return self.language.loss_accumulation_steps

    @loss_accumulation_steps.setter
    def loss_accumulation_steps(self, v):
        self.language.loss_accumulation_steps = v

    def weight_map(self) -> WeightMap:
        cfg = self.config
        T, Lm = "model.transformer.", "language.model."
        E, A = cfg.embedding_size, cfg.additional_vocab_size
        swap = (lambda t: torch.cat(t.chunk(2, dim=0)[::-1], dim=0),) * 2               # [up | gate] <-> [gate | up]; its own inverse
        rules = [Rule(Lm + "norm.weight", [T + "ln_f.weight"])]
        if A:
            rules.append(Rule(Lm + "embed_tokens.weight", [T + "wte.embedding", T + "wte.new_embedding"], "concat", 0, sizes=[E, A]))
        else:
            rules.append(Rule(Lm + "embed_tokens.weight", [T + "wte.embedding"]))
        if self.lm_head is not None:
            rules.append(Rule("lm_head.weight", [T + "ff_out.weight"]))
        first, second = ("post_attention_layernorm", "post_feedforward_layernorm") if cfg.norm_after else ("input_layernorm", "post_attention_layernorm")
        for i in range(cfg.num_hidden_layers):
            a, b = f"{Lm}layers.{i}.", f"{T}blocks.{i}."
            rules += [Rule(a + "self_attn.qkv_proj.weight", [b + "att_proj.weight"]), Rule(a + "self_attn.o_proj.weight", [b + "attn_out.weight"]),
                      Rule(a + "mlp.gate_up_proj.weight", [b + "ff_proj.weight"], fn=swap), Rule(a + "mlp.down_proj.weight", [b + "ff_out.weight"]),
                      Rule(a + first + ".weight", [b + "attn_norm.weight"]), Rule(a + second + ".weight", [b + "ff_norm.weight"])]
            if cfg.qkv_bias:
                rules.append(Rule(a + "self_attn.qkv_proj.bias", [b + "att_proj.bias"]))
            if cfg.attention_layer_norm:
                rules += [Rule(a + "self_attn.q_norm.weight", [b + "q_norm.weight"]), Rule(a + "self_attn.k_norm.weight", [b + "k_norm.weight"])]
        if self.model.vision_backbone is not None:
            for name, _ in self.model.vision_backbone.named_parameters():
                rules.append(Rule("model.vision_backbone." + name, ["model.vision_backbone." + name]))
        return WeightMap(rules)


class MolmoProcessor:
    """Prompt + images -> ``input_ids`` (start token, the images' token blocks, the prompt), ``images``, ``image_masks`` and
    ``image_input_idx`` with positions counted in the final sequence (paddleformers/transformers/molmo/processing.py:99-190).
    ``tokenizer`` must encode ``<im_start>``, ``<im_end>``, ``<im_patch>`` and ``<im_col>`` as single tokens."""

    TOKENS = ("<im_start>", "<im_end>", "<im_patch>", "<im_col>")

    def __init__(self, tokenizer, image_processor=None):
        from ..transformers.image_processing import MolmoImageProcessor

        self.tokenizer = tokenizer
        self.image_processor = image_processor or MolmoImageProcessor()
        ids = [tokenizer.encode(t, add_special_tokens=False) for t in self.TOKENS]
        if any(len(i) != 1 for i in ids):
            raise ValueError("the tokenizer must encode the Molmo image tokens as single tokens")
        self.start_id, self.end_id, self.patch_id, self.col_id = (i[0] for i in ids)

    def __call__(self, text: str, images=None, message_format: str = "role") -> dict:
        import numpy as np

        prompt = "" if text is None else text
        if message_format == "role":
            prompt = "User: " + prompt + " Assistant:"
        ids = [self.tokenizer.bos_token_id if self.tokenizer.bos_token_id is not None else self.tokenizer.eos_token_id]
        out = {}
        if images:
            crops, masks, idx = [], [], []
            for img in images:
                c, m, toks, ix = self.image_processor.preprocess_one(np.asarray(img), self.patch_id, self.col_id, self.start_id, self.end_id)
                idx.append(np.where(ix >= 0, ix + len(ids), -1))
                ids += toks.tolist()
                crops.append(c)
                masks.append(m)
            out = {"images": torch.from_numpy(np.concatenate(crops))[None], "image_masks": torch.from_numpy(np.concatenate(masks))[None],
                   "image_input_idx": torch.from_numpy(np.concatenate(idx))[None]}
        ids += self.tokenizer.encode(" " + prompt, add_special_tokens=False)
        out["input_ids"] = torch.tensor([ids])
        return out
