"""ERNIE-4.5-VL: vision tower + variable-resolution resampler + an ERNIE-4.5 MoE decoder whose experts are isolated per
modality (paddleformers/transformers/ernie4_5_moe_vl/model/modeling_moe_vl.py, model/dfnrope/modeling.py,
model/configuration.py:488).

* Vision tower: one GEMM over flattened patches, pre-LayerNorm blocks with 2-D rotary attention inside every frame
  (the Qwen2-VL block of ``vision_language.py``), a final LayerNorm. No merger of its own.
* Resampler: 2 x 2 neighbouring patches folded into channels -> MLP + LayerNorm; then frames paired in time (even frame
  beside odd frame; a still image is paired with itself) -> MLP + LayerNorm; projection to the decoder width; RMSNorm.
* Decoder: the unified decoder with ERNIE's interleaved rotary rows (permuted on load) and three-axis positions: of the
  ``s0 + s1`` lowest frequency pairs the even ones rotate with the row position and the odd ones with the column position,
  the remaining ``s2`` pairs with the temporal position (``mrope_section = [s0, s1, s2]``); text tokens advance all three
  together. MoE layers hold a text and a vision expert group with separate routers and widths
  (``nn.moe.ModalityMoELayer``): image / video placeholders and their start / end markers are routed to the vision group,
  everything else to the text group; shared experts see every token.

Checkpoint tensors keep the published names: the decoder under ``model.``, experts numbered text first then vision, both
routers transposed (``gate.weight`` / ``gate.weight_1``), both correction biases as the rows of one tensor, the tower under
``model.vision_model.``, the resampler's MLPs as numbered sequential entries.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..transformers.configuration_utils import PretrainedConfig
from ..transformers.conversion_utils import Rule, WeightMap
from .configuration import Ernie4_5MoeConfig
from .modeling import BatchContext, CausalLMOutput, DecoderForCausalLM, RMSNorm, build_weight_map
from .vision_language import Qwen2VLForConditionalGeneration, VisionTower, _VisionBlock, multimodal_position_ids


class Ernie4_5VLTextConfig(Ernie4_5MoeConfig):
    model_type = "ernie4_5_vl_moe_text"

    def __init__(self, moe_intermediate_size=(1536, 512), mlp_layer_types=None, rope_parameters=None, **kw):
        sizes = list(moe_intermediate_size) if isinstance(moe_intermediate_size, (list, tuple)) else [moe_intermediate_size] * 2
        rope_parameters = dict(rope_parameters or {"rope_theta": 500000.0, "rope_type": "default"})
        kw.setdefault("rope_theta", rope_parameters.get("rope_theta", 500000.0))
        super().__init__(moe_intermediate_size=int(sizes[0]), **kw)
        self.moe_vision_intermediate_size = int(sizes[-1])
        self.mrope_section = list(rope_parameters.get("mrope_section", [22, 22, 20]))
        self.rope_parameters = rope_parameters
        L = self.num_hidden_layers
        if mlp_layer_types is None:
            mlp_layer_types = ["sparse" if self.is_moe_layer(i) else "dense" for i in range(L)]
        self.mlp_layer_types = list(mlp_layer_types)
        self.moe_layers = [i for i, t in enumerate(self.mlp_layer_types) if t == "sparse"]
        self.moe_modality_isolated = True

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            d["moe_intermediate_size"] = [self.moe_intermediate_size, self.moe_vision_intermediate_size]
            for k in ("moe_vision_intermediate_size", "moe_layers", "moe_modality_isolated", "mrope_section",
                      "num_experts", "num_experts_per_tok", "n_shared_experts", "first_k_dense_replace", "decoder_sparse_step"):
                d.pop(k, None)
        return d


_VISION_DEFAULTS = dict(depth=32, hidden_size=1280, hidden_act="quick_gelu", num_heads=16, in_channels=3, patch_size=14,
                        spatial_merge_size=2, intermediate_size=5120, temporal_merge_size=2, rms_norm_eps=1e-6)


class Ernie4_5VLConfig(PretrainedConfig):
    model_type = "ernie4_5_vl_moe"

    def __init__(self, text_config=None, vision_config=None, image_token_id=100295, video_token_id=103367,
                 image_start_token_id=101304, image_end_token_id=101305, video_start_token_id=101306, video_end_token_id=101307,
                 **kwargs):
        kwargs.setdefault("tie_word_embeddings", True)
        if isinstance(text_config, dict):
            text_config = dict(text_config)
            text_config.setdefault("tie_word_embeddings", kwargs["tie_word_embeddings"])
            text_config = Ernie4_5VLTextConfig(**{k: v for k, v in text_config.items() if k != "model_type"})
        self.text_config = text_config or Ernie4_5VLTextConfig()
        vc = dict(_VISION_DEFAULTS)
        vc.update({k: v for k, v in (vision_config or {}).items() if k in _VISION_DEFAULTS})
        self.vision_config = vc
        super().__init__(vocab_size=self.text_config.vocab_size, hidden_size=self.text_config.hidden_size,
                         num_hidden_layers=self.text_config.num_hidden_layers,
                         num_attention_heads=self.text_config.num_attention_heads, **kwargs)
        self.image_token_id, self.video_token_id = image_token_id, video_token_id
        self.image_start_token_id, self.image_end_token_id = image_start_token_id, image_end_token_id
        self.video_start_token_id, self.video_end_token_id = video_start_token_id, video_end_token_id

    # the names the data pipeline uses for the markers around an image
    @property
    def vision_start_token_id(self):
        return self.image_start_token_id

    @property
    def vision_end_token_id(self):
        return self.image_end_token_id

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        d["text_config"] = self.text_config.to_dict(saving)
        d["vision_config"] = dict(self.vision_config, model_type="ernie4_5_vl_moe_vision")
        if saving:
            for k in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads"):
                d.pop(k, None)
        return d


class ErnieVisionTower(VisionTower):
    """Patch GEMM -> rotary blocks -> LayerNorm; returns one row per patch (merging is the resampler's job)."""

    def __init__(self, vc: dict, dtype=None, device=None):
        nn.Module.__init__(self)
        kw = dict(dtype=dtype, device=device)
        self.vc = vc
        dim = vc["hidden_size"]
        self.patch_embed = nn.Linear(vc["in_channels"] * vc["patch_size"] ** 2, dim, bias=False, **kw)
        self.blocks = nn.ModuleList([_VisionBlock(dim, vc["num_heads"], vc["intermediate_size"], vc["hidden_act"],
                                                  eps=vc["rms_norm_eps"], **kw) for _ in range(vc["depth"])])
        self.ln = nn.LayerNorm(dim, eps=vc["rms_norm_eps"], **kw)
        self.head_dim = dim // vc["num_heads"]

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        x = self.patch_embed(pixel_values.to(self.patch_embed.weight.dtype))
        cos, sin = self.rotary(grid_thw, x.device)
        lengths = [h * w for t, h, w in grid_thw.tolist() for _ in range(t)]
        for blk in self.blocks:
            x = blk(x, cos, sin, lengths)
        return self.ln(x)


class _ResamplerMLP(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, eps: float, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.fc1, self.fc2 = nn.Linear(in_dim, out_dim, **kw), nn.Linear(out_dim, out_dim, **kw)
        self.ln = nn.LayerNorm(out_dim, eps=eps, **kw)

    def forward(self, x):
        return self.ln(self.fc2(TF.gelu(self.fc1(x))))


class VariableResolutionResampler(nn.Module):
    def __init__(self, config: Ernie4_5VLConfig, dtype=None, device=None):
        super().__init__()
        vc, kw = config.vision_config, dict(dtype=dtype, device=device)
        self.merge, self.tmerge = vc["spatial_merge_size"], vc["temporal_merge_size"]
        assert self.tmerge == 2, "frames are paired (temporal_merge_size 2)"
        sdim = vc["hidden_size"] * self.merge ** 2
        self.spatial_linear = _ResamplerMLP(sdim, sdim, vc["rms_norm_eps"], **kw)
        self.temporal_linear = _ResamplerMLP(sdim * self.tmerge, sdim, vc["rms_norm_eps"], **kw)
        self.mlp = nn.Linear(sdim, config.text_config.hidden_size, **kw)
        self.after_norm = RMSNorm(config.text_config.hidden_size, config.text_config.rms_norm_eps, **kw)

    def forward(self, x: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        m = self.merge ** 2
        x = self.spatial_linear(x.reshape(-1, x.shape[-1] * m))
        first, second, off = [], [], 0
        for t, h, w in grid_thw.tolist():
            n = h * w // m                                  # merged patches per frame
            odd_start = 1 if t > 1 else 0                   # a still image is its own partner
            for a, b in zip(range(0, t, 2), range(odd_start, t, 2)):
                first.append(torch.arange(off + a * n, off + (a + 1) * n))
                second.append(torch.arange(off + b * n, off + (b + 1) * n))
            off += t * n
        first, second = torch.cat(first).to(x.device), torch.cat(second).to(x.device)
        x = torch.cat([x.index_select(0, first), x.index_select(0, second)], dim=-1)
        return self.after_norm(self.mlp(self.temporal_linear(x)))


class Ernie4_5VLForConditionalGeneration(Qwen2VLForConditionalGeneration):
    config_class = Ernie4_5VLConfig

    def __init__(self, config: Ernie4_5VLConfig, dtype=None, device=None):
        from ..transformers.model_utils import PretrainedModel

        PretrainedModel.__init__(self, config)
        self.visual = ErnieVisionTower(config.vision_config, dtype=dtype, device=device)
        self.resampler = VariableResolutionResampler(config, dtype=dtype, device=device)
        self.language = DecoderForCausalLM(config.text_config, dtype=dtype, device=device)
        D = config.text_config.head_dim
        s = config.text_config.mrope_section
        assert sum(s) == D // 2 and s[0] == s[1], "mrope_section must cover half the head size with equal row / column parts"
        i = torch.arange(D // 2)
        self.register_buffer("rope_axis", torch.where(i < s[0] + s[1], 1 + i % 2, torch.zeros_like(i)), persistent=False)

    def _context(self, input_ids, position_ids3) -> BatchContext:
        B, S = input_ids.shape
        D = self.config.text_config.head_dim
        cos_t, sin_t = self.language.model.rope(input_ids.device, int(position_ids3.max().item()) + 1)
        sel = position_ids3.reshape(3, B * S)[self.rope_axis.to(input_ids.device)]                    # [D / 2, B * S]
        col = torch.arange(D // 2, device=input_ids.device)[:, None]
        return BatchContext(B, S, torch.arange(B * S, device=input_ids.device), None,
                            cos_t[sel, col].t().contiguous(), sin_t[sel, col].t().contiguous())

    def vision_rows(self, input_ids: torch.Tensor) -> torch.Tensor:
        """bool [B, S]: tokens served by the vision experts (placeholders and the markers around them)."""
        cfg = self.config
        ids = [cfg.image_token_id, cfg.video_token_id, cfg.image_start_token_id, cfg.image_end_token_id,
               cfg.video_start_token_id, cfg.video_end_token_id]
        return torch.isin(input_ids, torch.tensor([i for i in ids if i is not None], device=input_ids.device))

    def forward(self, input_ids, pixel_values=None, image_grid_thw=None, pixel_values_videos=None, video_grid_thw=None, labels=None,
                position_ids=None, moe_mm_token_type_ids=None, return_logits: Optional[bool] = None, **unused):
        cfg, lm = self.config, self.language
        if lm.model.sp:
            raise NotImplementedError("the vision rows of the modality-isolated experts are whole-sequence positions: this model "
                                      "runs without sequence parallelism")
        h = lm.model.embed(input_ids, whole=True)
        for pv, grid, tok in ((pixel_values, image_grid_thw, cfg.image_token_id), (pixel_values_videos, video_grid_thw, cfg.video_token_id)):
            if pv is not None:
                feats = self.resampler(self.visual(pv, grid), grid).to(h.dtype)
                mask = (input_ids.reshape(-1) == tok)
                assert int(mask.sum()) == feats.shape[0], "one placeholder token per resampled patch is required"
                h = h.masked_scatter(mask[:, None], feats)
        if position_ids is None:
            vgrid = video_grid_thw
            if vgrid is not None:                       # paired frames: half as many temporal steps reach the decoder
                vgrid = vgrid.clone()
                vgrid[:, 0] = vgrid[:, 0] // cfg.vision_config["temporal_merge_size"]
            position_ids = multimodal_position_ids(input_ids, cfg.image_token_id, cfg.video_token_id, image_grid_thw, vgrid,
                                                   cfg.vision_config["spatial_merge_size"])
        elif position_ids.dim() == 2:
            position_ids = position_ids[None].expand(3, -1, -1)
        ctx = self._context(input_ids, position_ids)
        vis = (moe_mm_token_type_ids != 0) if moe_mm_token_type_ids is not None else self.vision_rows(input_ids)
        vis = vis.reshape(-1)
        from ..nn.moe import ModalityMoELayer

        moes = [m.mlp for m in lm.model.layers.values() if isinstance(m.mlp, ModalityMoELayer)]
        for m in moes:
            m.vision_rows = vis
        try:
            hidden, residual = lm.model.run_layers(lm.model.token_slice(h), None, ctx)
        finally:
            for m in moes:
                m.vision_rows = None
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

    def load_hf_checkpoint(self, directory: str, strict: bool = False) -> None:
        from ..transformers.model_utils import PretrainedModel

        PretrainedModel.load_hf_checkpoint(self, directory, strict)

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
                              r.rope_deinterleave, r.flatten, fn=r.fn, expert_base=r.expert_base))
        known = {r.target for r in rules}
        for name, _ in self.language.named_parameters():
            if "language." + name not in known:
                rules.append(Rule("language." + name, [name]))
        vis = "model.vision_model."
        rules.append(Rule("visual.patch_embed.weight", [vis + "patch_embed.proj.weight"]))
        for i in range(self.config.vision_config["depth"]):
            a, b = f"visual.blocks.{i}.", vis + f"blocks.{i}."
            for mine, theirs in (("norm1", "norm1"), ("norm2", "norm2"), ("qkv", "attn.qkv"), ("proj", "attn.proj"),
                                 ("fc1", "mlp.fc1"), ("fc2", "mlp.fc2")):
                for leaf in ("weight", "bias"):
                    rules.append(Rule(a + f"{mine}.{leaf}", [b + f"{theirs}.{leaf}"]))
        for leaf in ("weight", "bias"):
            rules.append(Rule(f"visual.ln.{leaf}", [vis + f"ln.{leaf}"]))
        seq = {"fc1": "0", "fc2": "2", "ln": "3"}
        for name, _ in self.resampler.named_parameters():
            parts = name.split(".")
            if parts[0] in ("spatial_linear", "temporal_linear"):
                parts[1] = seq[parts[1]]
            rules.append(Rule("resampler." + name, ["model.resampler_model." + ".".join(parts)]))
        return WeightMap(rules)

    def hf_state_dict_items(self, tensor_for=None):
        """The text and the vision router's correction biases are written as the two rows of one tensor."""
        pending = {}
        for name, t in super().hf_state_dict_items(tensor_for):
            if name.endswith("moe_statics.e_score_correction_bias"):
                if name in pending:
                    yield name, torch.cat([pending.pop(name), t], dim=0)       # text_moe is registered before vision_moe
                else:
                    pending[name] = t
                continue
            yield name, t
