"""PaliGemma and Gemma 3 with images. PaliGemma: a SigLIP image encoder, one linear projector and a Gemma decoder that reads the image tokens and the prompt
with two-way attention and writes the answer causally (paddleformers/transformers/paligemma).

The prefix (image placeholders + prompt, ``token_type_ids == 0``) attends to itself in both directions; the suffix
(``token_type_ids == 1``) is causal and sees the whole prefix. This is expressed as a per-key lower bound ``kstart[j]`` = first
row of j's prefix block (j itself for suffix keys), next to the per-key upper bound used for packed documents; the attention
runs through the tensor-operation back-ends, because the flash kernels take the upper bound only. Without ``token_type_ids``
the whole input is one prefix (a prompt being encoded for generation).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch
import torch.nn as nn

from ..transformers.configuration_utils import PretrainedConfig
from ..transformers.conversion_utils import Rule, WeightMap
from ..transformers.model_utils import PretrainedModel
from .modeling import BatchContext, CausalLMOutput, DecoderForCausalLM, build_weight_map
from .siglip import SiglipVisionConfig, SiglipVisionModel


def two_way_block_starts(two_way: torch.Tensor) -> torch.Tensor:
    """two_way: bool [B, S], True on tokens of blocks that attend in both directions (runs of True are one block each).
    Returns int32 [B, S]: for a key inside a block, the first position of its block; for any other key, its own position."""
    B, S = two_way.shape
    idx = torch.arange(S, device=two_way.device)[None].expand(B, S)
    prev = torch.nn.functional.pad(two_way, (1, 0), value=False)[:, :-1]
    start_here = torch.where(two_way & ~prev, idx, torch.zeros_like(idx))      # block starts carry their index
    block_start = torch.cummax(start_here, dim=1).values
    return torch.where(two_way, block_start, idx).to(torch.int32).contiguous()


def two_way_block_ends(two_way: torch.Tensor) -> torch.Tensor:
    """int32 [B, S]: for a key inside a two-way block, one past the last position of its block; 0 for any other key. Layers
    with a sliding window keep a block whole: the upper bound of a block key is at least this."""
    B, S = two_way.shape
    rev = torch.flip(two_way, dims=[1])
    starts_rev = two_way_block_starts(rev).long()                     # first position of the block in the reversed order
    ends = S - torch.flip(starts_rev, dims=[1])
    return torch.where(two_way, ends, torch.zeros_like(ends)).to(torch.int32).contiguous()


class PaliGemmaConfig(PretrainedConfig):
    model_type = "paligemma"

    def __init__(self, text_config=None, vision_config=None, image_token_id=None, image_token_index=None, projection_dim=None,
                 hidden_size=None, **kwargs):
        from ..transformers.auto import AutoConfig

        kwargs.pop("model_type", None)
        text = dict(text_config or {}) if not isinstance(text_config, PretrainedConfig) else text_config
        if isinstance(text, dict):
            text.setdefault("tie_word_embeddings", True)
            text.pop("use_bidirectional_attention", None)
            text = AutoConfig.for_model(text.pop("model_type", "gemma"), **text)
        kwargs.setdefault("tie_word_embeddings", bool(text.tie_word_embeddings))
        super().__init__(**{k: v for k, v in kwargs.items() if k != "vocab_size"})
        self.text_config = text
        vis = dict(vision_config or {}) if not isinstance(vision_config, PretrainedConfig) else vision_config.to_dict()
        vis.pop("model_type", None)
        self.projection_dim = int(projection_dim or vis.get("projection_dim") or text.hidden_size)
        vis.pop("projection_dim", None)
        vis["vision_use_head"] = False
        self.vision_config = SiglipVisionConfig(**vis)
        tok = image_token_id if image_token_id is not None else image_token_index
        self.image_token_id = int(tok if tok is not None else 257152)
        self.hidden_size = int(hidden_size or text.hidden_size)
        self.vocab_size = text.vocab_size

    @property
    def num_image_tokens(self) -> int:
        return (self.vision_config.image_size // self.vision_config.patch_size) ** 2

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        text = self.text_config.to_dict(saving)
        text["model_type"] = self.text_config.model_type
        text["num_image_tokens"] = self.num_image_tokens
        vis = self.vision_config.to_dict(saving)
        vis.update(model_type="siglip_vision_model", projection_dim=self.projection_dim)
        d.update(text_config=text, vision_config=vis, image_token_index=self.image_token_id)
        d.pop("image_token_id", None)
        return d


class PaliGemma2Config(PaliGemmaConfig):
    """The same composite with the Gemma 2 decoder as the default text model (paddleformers/transformers/paligemma2)."""

    model_type = "paligemma2"

    def __init__(self, text_config=None, **kwargs):
        if not isinstance(text_config, PretrainedConfig):
            text_config = dict(text_config or {})
            text_config.setdefault("model_type", "gemma2")
        super().__init__(text_config=text_config, **kwargs)


class PaliGemmaForConditionalGeneration(PretrainedModel):
    config_class = PaliGemmaConfig

    def __init__(self, config: PaliGemmaConfig, dtype=None, device=None):
        super().__init__(config)
        self.vision_tower = SiglipVisionModel(config.vision_config, dtype=dtype, device=device)
        self.build_projector(config, dtype, device)
        self.language = DecoderForCausalLM(config.text_config, dtype=dtype, device=device)
        self._layout = "nested"                     # tensor-name generation of the checkpoint being read / written
        self.post_init()

    def build_projector(self, config, dtype, device):
        self.projector = nn.Linear(config.vision_config.hidden_size, config.projection_dim, dtype=dtype, device=device)

    def _init_weights(self, module):
        if module is getattr(self, "projector", None):
            nn.init.normal_(module.weight, 0.0, self.config.text_config.initializer_range)
            nn.init.zeros_(module.bias)

    def image_features(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """[B, C, H, W] -> [B * tokens, text hidden]. The decoder multiplies embeddings by sqrt(hidden) when it looks tokens
        up; image rows enter after that step and therefore stay unscaled."""
        hidden, _ = self.vision_tower(pixel_values)
        return self.project(hidden)

    def project(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.projector(hidden).reshape(-1, self.config.projection_dim)

    def two_way_tokens(self, input_ids, token_type_ids) -> torch.Tensor:
        """bool [B, S]: tokens inside blocks that attend in both directions. Here: the prefix (type 0); everything when no types
        are given."""
        return (token_type_ids == 0) if token_type_ids is not None else torch.ones_like(input_ids, dtype=torch.bool)

    def projector_rules(self, prefix: str):
        return [Rule("projector.weight", [prefix + "multi_modal_projector.linear.weight"]),
                Rule("projector.bias", [prefix + "multi_modal_projector.linear.bias"])]

    def forward(self, input_ids, pixel_values=None, token_type_ids=None, labels=None, kend=None,
                return_logits: Optional[bool] = None, image_embeds=None, **unused):
        cfg, lm = self.config, self.language
        B, S = input_ids.shape
        is_image = input_ids == cfg.image_token_id
        ids = input_ids.masked_fill(is_image, 0) if cfg.image_token_id >= cfg.text_config.vocab_size else input_ids
        h = lm.model.embed(ids, whole=True)
        if pixel_values is not None or image_embeds is not None:
            feats = (image_embeds if image_embeds is not None else self.image_features(pixel_values)).to(h.dtype)
            assert int(is_image.sum()) == feats.shape[0], "one placeholder token per image patch is required"
            h = h.masked_scatter(is_image.reshape(-1)[:, None], feats)
        two_way = self.two_way_tokens(input_ids, token_type_ids)
        ctx = lm.model.make_context(input_ids, None, kend)
        if two_way is not None:
            ctx.kstart = two_way_block_starts(two_way)
            if ctx.kend_window is not None:           # a window never cuts through a two-way block
                ctx.kend_window = torch.maximum(ctx.kend_window, two_way_block_ends(two_way))
        hidden, residual = lm.model.run_layers(lm.model.token_slice(h), None, ctx)
        hidden = lm.model.norm(hidden, residual)[0] if residual is not None else lm.model.norm(hidden)
        out = CausalLMOutput()
        if return_logits if return_logits is not None else labels is None:
            out.logits = lm.full_logits(hidden).view(B, S, -1)
        if labels is not None:
            lab = labels.reshape(-1)
            count = (lab != lm.ignore_index).sum()
            scale = 1.0 / (count.clamp(min=1).to(torch.float32) * float(lm.loss_accumulation_steps))
            out.loss, _ = lm._loss(hidden, lab, scale)
            out.num_tokens = count
        return out

    def generation_token_types(self, prompt_len: int, total_len: int, batch: int, device) -> Optional[torch.Tensor]:
        """Token types while decoding: the prompt stays a two-way prefix, generated tokens are causal."""
        types = torch.ones(batch, total_len, dtype=torch.long, device=device)
        types[:, :prompt_len] = 0
        return types

    @torch.no_grad()
    def generate(self, input_ids, pixel_values=None, max_new_tokens: int = 32, eos_token_id: Optional[int] = None):
        """Greedy decoding. Every step re-reads the whole sequence (no key / value cache): the image features are computed once
        and the decoder sees the same masks as in training, so the result equals cached decoding."""
        cfg, lm = self.config, self.language
        eos = eos_token_id if eos_token_id is not None else getattr(cfg.text_config, "eos_token_id", None)
        eos_ids = set(eos) if isinstance(eos, (list, tuple)) else ({eos} if eos is not None else set())
        feats = self.image_features(pixel_values) if pixel_values is not None else None
        ids, prompt_len = input_ids, input_ids.shape[1]
        done = torch.zeros(ids.shape[0], dtype=torch.bool, device=ids.device)
        pad = getattr(cfg.text_config, "pad_token_id", None) or 0
        for _ in range(max_new_tokens):
            types = self.generation_token_types(prompt_len, ids.shape[1], ids.shape[0], ids.device)
            logits = self.forward(ids, token_type_ids=types, image_embeds=feats).logits[:, -1]
            nxt = torch.where(done, torch.full_like(logits.argmax(-1), pad), logits.argmax(-1))
            ids = torch.cat([ids, nxt[:, None]], dim=1)
            for e in eos_ids:
                done |= nxt == e
            if bool(done.all()):
                break
        return ids

    @property
    def loss_accumulation_steps(self):
        return self.language.loss_accumulation_steps

    @loss_accumulation_steps.setter
    def loss_accumulation_steps(self, v):
        self.language.loss_accumulation_steps = v

    # ------------------------------------------------------------------ checkpoint names
    _vision_name = "vision_tower."
    _LAYOUTS = {                                   # (decoder "model." ->, vision / projector prefix)
        "legacy": ("language_model.model.", ""),                   # published checkpoints
        "flat": ("model.language_model.", "model."),
        "nested": ("model.language_model.model.", "model."),
    }

    def load_hf_checkpoint(self, directory: str, strict: bool = False) -> None:
        from ..transformers.model_utils import _CheckpointReader

        reader = _CheckpointReader(directory)
        saved = self._layout
        for name, (text, _) in self._LAYOUTS.items():
            if reader.has(text + "embed_tokens.weight"):
                self._layout = name
                break
        try:
            super().load_hf_checkpoint(directory, strict)
        finally:
            self._layout = saved

    def weight_map(self) -> WeightMap:
        text_prefix, other = self._LAYOUTS[self._layout]

        def text_name(s: str) -> str:
            if s.startswith("lm_head."):                       # beside the decoder's "model." in every layout
                return (text_prefix if self._layout == "legacy" else other)[:-len("model.")] + s
            return text_prefix + s[len("model."):] if s.startswith("model.") else s

        rules = []
        text_map = build_weight_map(self.config.text_config)
        for r in text_map.rules.values():
            rules.append(dataclasses.replace(r, target="language." + r.target, sources=[text_name(s) for s in r.sources]))
        known = {r.target for r in rules}
        for name, _ in self.language.named_parameters():                 # parameters without a fusion rule: renamed only
            if "language." + name not in known:
                rules.append(Rule("language." + name, [text_name(text_map.translate(name))]))
        for r in self.vision_tower.weight_map().rules.values():
            rules.append(dataclasses.replace(r, target="vision_tower." + r.target, sources=[other + self._vision_name + s for s in r.sources]))
        return WeightMap(rules + self.projector_rules(other))


class Gemma3Config(PaliGemmaConfig):
    """Gemma 3 with images (paddleformers/transformers/gemma3): the SigLIP patch grid is average-pooled to
    ``mm_tokens_per_image`` tokens per image, normalised and projected by one matrix; the tokens of one image attend to each
    other in both directions inside the otherwise causal Gemma 3 text decoder."""

    model_type = "gemma3"

    def __init__(self, text_config=None, vision_config=None, mm_tokens_per_image=256, boi_token_index=255999, eoi_token_index=256000,
                 image_token_index=262144, **kwargs):
        text = text_config
        if not isinstance(text, PretrainedConfig):
            text = dict(text_config or {})
            text["model_type"] = "gemma3_text"
        super().__init__(text_config=text, vision_config=vision_config, image_token_index=kwargs.pop("image_token_id", image_token_index),
                         **kwargs)
        self.mm_tokens_per_image = int(mm_tokens_per_image)
        self.boi_token_index, self.eoi_token_index = boi_token_index, eoi_token_index
        self.projection_dim = self.text_config.hidden_size

    @property
    def num_image_tokens(self) -> int:
        return self.mm_tokens_per_image

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        d["text_config"].pop("num_image_tokens", None)
        d["vision_config"].pop("projection_dim", None)
        d.pop("projection_dim", None)
        return d


class Gemma3ForConditionalGeneration(PaliGemmaForConditionalGeneration):
    config_class = Gemma3Config

    def build_projector(self, config, dtype, device):
        kw = dict(dtype=dtype, device=device)
        self.mm_input_projection_weight = nn.Parameter(torch.zeros(config.vision_config.hidden_size, config.text_config.hidden_size, **kw))
        self.mm_soft_emb_norm = nn.Parameter(torch.zeros(config.vision_config.hidden_size, **kw))    # stored as (scale - 1)

    def _init_weights(self, module):
        if module is self:
            nn.init.normal_(self.mm_input_projection_weight, 0.0, self.config.text_config.initializer_range)

    def project(self, hidden: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        B, N, H = hidden.shape
        side = int(N ** 0.5)
        out_side = int(cfg.mm_tokens_per_image ** 0.5)
        k = side // out_side
        pooled = hidden.view(B, out_side, k, out_side, k, H).float().mean(dim=(2, 4)).reshape(B, out_side * out_side, H)
        normed = pooled * torch.rsqrt(pooled.pow(2).mean(-1, keepdim=True) + cfg.vision_config.layer_norm_eps)
        normed = (normed * (1.0 + self.mm_soft_emb_norm.float())).to(hidden.dtype)
        return (normed @ self.mm_input_projection_weight).reshape(-1, cfg.text_config.hidden_size)

    def generation_token_types(self, prompt_len, total_len, batch, device):
        return None                                    # the image blocks are found from the placeholder tokens

    def two_way_tokens(self, input_ids, token_type_ids) -> torch.Tensor:
        """The tokens of each image (type 1, or the image placeholder when no types are given); consecutive images are told
        apart by the end-of-image / begin-of-image tokens between them."""
        return (token_type_ids == 1) if token_type_ids is not None else (input_ids == self.config.image_token_id)

    def projector_rules(self, prefix: str):
        return [Rule("mm_input_projection_weight", [prefix + "multi_modal_projector.mm_input_projection_weight"]),
                Rule("mm_soft_emb_norm", [prefix + "multi_modal_projector.mm_soft_emb_norm.weight"])]


class AyaVisionConfig(PaliGemmaConfig):
    """Aya Vision (paddleformers/transformers/aya_vision): SigLIP features of one encoder layer, neighbouring patches folded
    into the channel dimension (``downsample_factor`` per side), LayerNorm + SwiGLU projector, Cohere 2 decoder; causal."""

    model_type = "aya_vision"

    def __init__(self, text_config=None, vision_config=None, downsample_factor=2, alignment_intermediate_size=36864,
                 adapter_layer_norm_eps=1e-6, vision_feature_layer=-1, vision_feature_select_strategy="full", image_token_index=255036,
                 **kwargs):
        text = text_config
        if not isinstance(text, PretrainedConfig):
            text = dict(text_config or {})
            text.setdefault("model_type", "cohere2")
        super().__init__(text_config=text, vision_config=vision_config, image_token_index=kwargs.pop("image_token_id", image_token_index),
                         **kwargs)
        self.downsample_factor, self.alignment_intermediate_size = int(downsample_factor), int(alignment_intermediate_size)
        self.adapter_layer_norm_eps, self.vision_feature_layer = adapter_layer_norm_eps, int(vision_feature_layer)
        self.vision_feature_select_strategy = vision_feature_select_strategy
        self.projection_dim = self.text_config.hidden_size

    @property
    def num_image_tokens(self) -> int:
        return (self.vision_config.image_size // self.vision_config.patch_size // self.downsample_factor) ** 2

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        d["text_config"].pop("num_image_tokens", None)
        d["vision_config"].pop("projection_dim", None)
        d.pop("projection_dim", None)
        return d


class AyaVisionForConditionalGeneration(PaliGemmaForConditionalGeneration):
    config_class = AyaVisionConfig

    def build_projector(self, config, dtype, device):
        kw = dict(dtype=dtype, device=device)
        width = config.vision_config.hidden_size * config.downsample_factor ** 2
        self.layernorm = nn.LayerNorm(width, eps=config.adapter_layer_norm_eps, **kw)
        self.linear_1 = nn.Linear(width, config.alignment_intermediate_size, **kw)
        self.linear_2 = nn.Linear(config.alignment_intermediate_size // 2, config.text_config.hidden_size, **kw)

    def _init_weights(self, module):
        if module is getattr(self, "linear_1", None) or module is getattr(self, "linear_2", None):
            nn.init.normal_(module.weight, 0.0, self.config.text_config.initializer_range)
            nn.init.zeros_(module.bias)

    def image_features(self, pixel_values: torch.Tensor) -> torch.Tensor:
        hidden, _ = self.vision_tower(pixel_values, feature_layer=self.config.vision_feature_layer)
        return self.project(hidden)

    def project(self, hidden: torch.Tensor) -> torch.Tensor:
        B, N, C = hidden.shape
        side, f = int(N ** 0.5), self.config.downsample_factor
        # fold f x f neighbouring patches into the channels; the element order follows the published checkpoints: first f
        # neighbours along the second grid axis, then f along the first, and the folded grid is stored second axis first
        x = hidden.reshape(B, side, side // f, C * f).permute(0, 2, 1, 3)
        x = x.reshape(B, side // f, side // f, C * f * f).permute(0, 2, 1, 3)
        x = self.linear_1(self.layernorm(x))
        val, gate = x.chunk(2, dim=-1)
        return self.linear_2(torch.nn.functional.silu(gate) * val).reshape(-1, self.config.text_config.hidden_size)

    def two_way_tokens(self, input_ids, token_type_ids):
        return None

    def generation_token_types(self, prompt_len, total_len, batch, device):
        return None

    def projector_rules(self, prefix: str):
        return [Rule(f"{m}.{leaf}", [prefix + f"multi_modal_projector.{m}.{leaf}"])
                for m in ("layernorm", "linear_1", "linear_2") for leaf in ("weight", "bias")]


class ShieldGemma2Config(Gemma3Config):
    model_type = "shieldgemma2"

    def __init__(self, yes_token_index=10784, no_token_index=3771, **kwargs):
        super().__init__(**kwargs)
        self.yes_token_index, self.no_token_index = int(yes_token_index), int(no_token_index)


@dataclasses.dataclass
class ImageClassifierOutput:
    logits: torch.Tensor            # [B, 2]: the "yes" and "no" logits at the last position
    probabilities: torch.Tensor     # softmax over the two


class ShieldGemma2ForImageClassification(Gemma3ForConditionalGeneration):
    """Image policy classifier (paddleformers/transformers/shieldgemma2): Gemma 3 reads the image and a policy prompt; the
    answer is the probability of "yes" against "no" as the next token."""

    config_class = ShieldGemma2Config
    _LAYOUTS = {
        "legacy": ("model.language_model.model.", "model."),
        "flat": ("model.model.language_model.", "model.model."),
        "nested": ("model.model.language_model.model.", "model.model."),
    }

    def forward(self, input_ids, pixel_values=None, token_type_ids=None, **kw):
        out = super().forward(input_ids, pixel_values=pixel_values, token_type_ids=token_type_ids, return_logits=True)
        picked = out.logits[:, -1, [self.config.yes_token_index, self.config.no_token_index]].float()
        return ImageClassifierOutput(picked, torch.softmax(picked, dim=-1))
