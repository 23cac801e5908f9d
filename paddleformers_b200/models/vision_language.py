"""Qwen2-VL style vision-language model: a ViT with 2-D rotary embedding and a 2x2 patch merger in front of the unified
decoder, multimodal rotary positions (temporal / height / width sections of the rotary frequencies) in the decoder.

Roles of paddleformers/transformers/qwen2_vl (vision tower, merger, ``get_rope_index``) and of the multimodal collator
(paddleformers/datasets/collate.py:755 ``mm_collate_fn``). The language model is the ordinary ``DecoderForCausalLM`` with
Qwen2 settings; multimodal rotary embedding needs no new kernel: the three position streams are folded into one
per-token cos / sin table, which the rotary kernels index by token number.

Inputs follow the Hugging Face processor: ``pixel_values`` [patches, C * T * P * P] with the patches of every image
ordered merge-block by merge-block, ``image_grid_thw`` [images, 3], and ``input_ids`` holding one ``image_token_id`` per
merged patch.
"""
from __future__ import annotations

import itertools
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from ..transformers.configuration_utils import PretrainedConfig
from ..transformers.conversion_utils import Rule, WeightMap
from ..transformers.model_utils import PretrainedModel
from .configuration import Qwen2Config
from .modeling import BatchContext, CausalLMOutput, DecoderForCausalLM, build_weight_map


class Qwen2VLConfig(PretrainedConfig):
    model_type = "qwen2_vl"

    def __init__(self, text_config=None, vision_config=None, image_token_id=151655, video_token_id=151656,
                 vision_start_token_id=151652, vision_end_token_id=151653, **kwargs):
        text = dict(text_config or {})
        # older checkpoints keep the text fields at the top level
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "max_position_embeddings", "rms_norm_eps", "rope_theta", "rope_scaling",
                  "rope_parameters", "tie_word_embeddings", "hidden_act"):
            if k in kwargs and k not in text:
                text[k] = kwargs.pop(k)
        tie = bool(text.get("tie_word_embeddings", kwargs.get("tie_word_embeddings", False)))
        kwargs.setdefault("tie_word_embeddings", tie)
        kwargs.pop("model_type", None)
        super().__init__(**{k: v for k, v in kwargs.items() if k not in ("text_config", "vision_config")})
        text.pop("model_type", None)
        text.setdefault("tie_word_embeddings", tie)
        self.text_config = text if isinstance(text, Qwen2Config) else Qwen2Config(**text)
        rs = self.text_config.rope_scaling or {}
        rp = text.get("rope_parameters") or {}
        self.mrope_section = list(rs.get("mrope_section") or rp.get("mrope_section") or [])
        if rs.get("rope_type", rs.get("type")) in ("mrope", "default"):
            self.text_config.rope_scaling = None           # the sections only select positions; frequencies are plain
        v = dict(vision_config or {})
        v.pop("model_type", None)
        self.vision_config = {"depth": 32, "embed_dim": 1280, "hidden_size": self.text_config.hidden_size, "hidden_act": "quick_gelu",
                              "mlp_ratio": 4, "num_heads": 16, "in_channels": 3, "patch_size": 14, "spatial_merge_size": 2,
                              "temporal_patch_size": 2, **v}
        self.image_token_id, self.video_token_id = image_token_id, video_token_id
        self.vision_start_token_id, self.vision_end_token_id = vision_start_token_id, vision_end_token_id

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        text = self.text_config.to_dict(saving)
        text["model_type"] = "qwen2_vl_text"
        text["rope_scaling"] = {"type": "mrope", "mrope_section": self.mrope_section}
        d["text_config"] = text
        d["vision_config"] = dict(self.vision_config, model_type="qwen2_vl")
        d.pop("mrope_section", None)
        return d


class Qwen2_5_VLConfig(Qwen2VLConfig):
    """Qwen2.5-VL: the vision blocks use RMSNorm and a biased SwiGLU MLP, most of them attend inside windows of
    ``window_size`` pixels (``fullatt_block_indexes`` lists the blocks that see the whole image), and the merger normalises
    with RMSNorm (paddleformers/transformers/qwen2_5_vl)."""

    model_type = "qwen2_5_vl"

    def __init__(self, vision_config=None, **kwargs):
        v = dict(vision_config or {})
        if "in_chans" in v:
            v.setdefault("in_channels", v.pop("in_chans"))
        defaults = {"depth": 32, "hidden_size": 1280, "intermediate_size": 3420, "num_heads": 16, "in_channels": 3, "out_hidden_size": 3584,
                    "patch_size": 14, "spatial_merge_size": 2, "temporal_patch_size": 2, "window_size": 112,
                    "fullatt_block_indexes": [7, 15, 23, 31], "hidden_act": "silu", "tokens_per_second": 4}
        super().__init__(vision_config={}, **kwargs)
        self.vision_config = {**defaults, **{k: v[k] for k in v if k != "model_type"}}

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        d["text_config"]["model_type"] = "qwen2_5_vl_text"
        d["vision_config"]["model_type"] = "qwen2_5_vl"
        return d


def _quick_gelu(x):
    return x * torch.sigmoid(1.702 * x)


class _RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, self.weight, self.eps)


class _VisionBlock(nn.Module):
    def __init__(self, dim: int, heads: int, mlp_hidden: int, act: str, dtype=None, device=None, rms_norm: bool = False,
                 swiglu: bool = False, bias: bool = True, eps: float = 1e-6, mlp_bias: Optional[bool] = None, qk_norm: bool = False):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        if qk_norm:                                    # per-head RMSNorm on queries and keys before the rotary embedding
            self.q_norm, self.k_norm = _RMSNorm(dim // heads, eps, **kw), _RMSNorm(dim // heads, eps, **kw)
        self.qk_norm = qk_norm
        mlp_bias = bias if mlp_bias is None else mlp_bias
        norm = (lambda: _RMSNorm(dim, eps, **kw)) if rms_norm else (lambda: nn.LayerNorm(dim, eps=eps, **kw))
        self.norm1, self.norm2 = norm(), norm()
        self.qkv = nn.Linear(dim, 3 * dim, bias=bias, **kw)
        self.proj = nn.Linear(dim, dim, bias=bias, **kw)
        self.swiglu = swiglu
        if swiglu:
            self.gate_proj = nn.Linear(dim, mlp_hidden, bias=mlp_bias, **kw)
            self.up_proj = nn.Linear(dim, mlp_hidden, bias=mlp_bias, **kw)
            self.down_proj = nn.Linear(mlp_hidden, dim, bias=mlp_bias, **kw)
        else:
            self.fc1 = nn.Linear(dim, mlp_hidden, **kw)
            self.fc2 = nn.Linear(mlp_hidden, dim, **kw)
        self.heads, self.hd = heads, dim // heads
        self.act = _quick_gelu if act == "quick_gelu" else (lambda x: TF.gelu(x, approximate="tanh")) if act == "gelu_pytorch_tanh" \
            else getattr(TF, act)

    def mlp(self, x):
        if self.swiglu:
            return self.down_proj(self.act(self.gate_proj(x)) * self.up_proj(x))
        return self.fc2(self.act(self.fc1(x)))

    def forward(self, x, cos, sin, lengths: List[int]):
        N = x.shape[0]
        q, k, v = self.qkv(self.norm1(x)).view(N, 3, self.heads, self.hd).unbind(1)
        half = self.hd // 2

        def rot(t):                                    # 2-D rotary: first half of the pairs from the row, second from the column
            t1, t2 = t[..., :half].float(), t[..., half:].float()
            return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], dim=-1).to(t.dtype)

        if self.qk_norm:
            q, k = self.q_norm(q.contiguous()), self.k_norm(k.contiguous())
        q, k = rot(q), rot(k)
        outs, off = [], 0
        for n in lengths:                              # full (non-causal) attention inside each image / frame
            sl = slice(off, off + n)
            outs.append(F.flash_attention(q[sl][None], k[sl][None], v[sl][None], causal=False)[0])
            off += n
        a = torch.cat(outs, dim=0).reshape(N, -1)
        x = x + self.proj(a)
        return x + self.mlp(self.norm2(x))


class VisionTower(nn.Module):
    def __init__(self, vc: dict, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.vc = vc
        dim = vc["embed_dim"]
        self.patch_dim = vc["in_channels"] * vc["temporal_patch_size"] * vc["patch_size"] ** 2
        self.patch_embed = nn.Linear(self.patch_dim, dim, bias=False, **kw)      # the strided Conv3d as one GEMM
        self.blocks = nn.ModuleList([_VisionBlock(dim, vc["num_heads"], int(dim * vc["mlp_ratio"]), vc["hidden_act"], **kw)
                                     for _ in range(vc["depth"])])
        m = vc["spatial_merge_size"] ** 2
        self.ln_q = nn.LayerNorm(dim, eps=1e-6, **kw)
        self.merge_fc1 = nn.Linear(dim * m, dim * m, **kw)
        self.merge_fc2 = nn.Linear(dim * m, vc["hidden_size"], **kw)
        self.head_dim = dim // vc["num_heads"]

    def rotary(self, grid_thw: torch.Tensor, device):
        """cos / sin [patches, head_dim / 2]: row position drives the first quarter of the frequencies, column position
        the second, in the merge-block patch order of the processor."""
        ms = self.vc["spatial_merge_size"]
        quarter = self.head_dim // 4
        inv = 1.0 / (10000.0 ** (torch.arange(0, self.head_dim // 2, 2, dtype=torch.float32, device=device) / (self.head_dim // 2)))
        out = []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h, device=device)[:, None].expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(w, device=device)[None, :].expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).flatten()
            ang = torch.cat([hp[:, None].float() * inv[None], wp[:, None].float() * inv[None]], dim=-1)
            assert ang.shape[1] == 2 * quarter
            out.append(ang.repeat(t, 1))
        ang = torch.cat(out, dim=0)[:, None, :]
        return ang.cos(), ang.sin()

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        x = self.patch_embed(pixel_values.to(self.patch_embed.weight.dtype))
        cos, sin = self.rotary(grid_thw, x.device)
        lengths = [h * w for t, h, w in grid_thw.tolist() for _ in range(t)]
        for blk in self.blocks:
            x = blk(x, cos, sin, lengths)
        m = self.vc["spatial_merge_size"] ** 2
        x = self.ln_q(x).view(-1, x.shape[-1] * m)
        return self.merge_fc2(TF.gelu(self.merge_fc1(x)))


class WindowedVisionTower(VisionTower):
    """Qwen2.5-VL tower: merged-patch groups are re-ordered window by window so that windowed blocks attend inside
    contiguous runs; full-attention blocks use the per-image runs on the same ordering; the merged output is put back
    into the processor's order."""

    def __init__(self, vc: dict, dtype=None, device=None):
        nn.Module.__init__(self)
        kw = dict(dtype=dtype, device=device)
        self.vc = vc
        dim = vc["hidden_size"]
        self.patch_dim = vc["in_channels"] * vc["temporal_patch_size"] * vc["patch_size"] ** 2
        self.patch_embed = nn.Linear(self.patch_dim, dim, bias=False, **kw)
        self.blocks = nn.ModuleList([_VisionBlock(dim, vc["num_heads"], vc["intermediate_size"], vc["hidden_act"], rms_norm=True,
                                                  swiglu=True, **kw) for _ in range(vc["depth"])])
        m = vc["spatial_merge_size"] ** 2
        self.ln_q = _RMSNorm(dim, 1e-6, **kw)
        self.merge_fc1 = nn.Linear(dim * m, dim * m, **kw)
        self.merge_fc2 = nn.Linear(dim * m, vc["out_hidden_size"], **kw)
        self.head_dim = dim // vc["num_heads"]

    def window_order(self, grid_thw: torch.Tensor):
        ms, unit = self.vc["spatial_merge_size"], self.vc["spatial_merge_size"] ** 2
        win = self.vc["window_size"] // ms // self.vc["patch_size"]
        index, lengths, base = [], [], 0
        for t, h, w in grid_thw.tolist():
            gh, gw = h // ms, w // ms
            idx = torch.arange(t * gh * gw).reshape(t, gh, gw)
            ph, pw = win - gh % win, win - gw % win                 # (a full extra window of padding when already aligned)
            nh, nw = (gh + ph) // win, (gw + pw) // win
            padded = TF.pad(idx, (0, pw, 0, ph), value=-100).reshape(t, nh, win, nw, win).permute(0, 1, 3, 2, 4)
            padded = padded.reshape(t, nh * nw, win, win)
            per_window = (padded != -100).sum([2, 3]).reshape(-1)
            flat = padded.reshape(-1)
            index.append(flat[flat != -100] + base)
            lengths += [int(n) * unit for n in per_window.tolist() if n > 0]
            base += t * gh * gw
        return torch.cat(index), lengths

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        unit = self.vc["spatial_merge_size"] ** 2
        x = self.patch_embed(pixel_values.to(self.patch_embed.weight.dtype))
        cos, sin = self.rotary(grid_thw, x.device)
        order, window_lengths = self.window_order(grid_thw)
        order = order.to(x.device)
        N = x.shape[0]

        def regroup(t):
            return t.reshape(N // unit, unit, *t.shape[1:])[order].reshape(N, *t.shape[1:])

        x, cos, sin = regroup(x), regroup(cos), regroup(sin)
        image_lengths = [h * w for t, h, w in grid_thw.tolist() for _ in range(t)]
        full = set(self.vc["fullatt_block_indexes"])
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, image_lengths if i in full else window_lengths)
        x = self.ln_q(x).view(-1, x.shape[-1] * unit)
        x = self.merge_fc2(TF.gelu(self.merge_fc1(x)))
        return x[torch.argsort(order)]


def multimodal_position_ids(input_ids: torch.Tensor, image_token_id: int, video_token_id: int, image_grid_thw, video_grid_thw,
                            merge: int) -> torch.Tensor:
    """[3, B, S] temporal / height / width positions: text tokens advance all three together; the tokens of an image keep
    the temporal position fixed and count rows and columns of the merged grid; the next text token continues after the
    larger of the two extents (the rule of the published Qwen2-VL model code)."""
    B, S = input_ids.shape
    pos = torch.zeros(3, B, S, dtype=torch.long, device=input_ids.device)
    grids = {image_token_id: iter(image_grid_thw.tolist()) if image_grid_thw is not None else iter(()),
             video_token_id: iter(video_grid_thw.tolist()) if video_grid_thw is not None else iter(())}
    for b in range(B):
        row = input_ids[b].tolist()
        cur, parts = 0, []
        for is_vis, group in itertools.groupby(range(S), key=lambda i: row[i] if row[i] in grids else -1):
            idx = list(group)
            if is_vis == -1:
                parts.append(torch.arange(cur, cur + len(idx))[None].expand(3, -1))
                cur += len(idx)
                continue
            done = 0
            while done < len(idx):                     # consecutive images without text in between
                t, h, w = next(grids[is_vis])
                gh, gw = h // merge, w // merge
                n = t * gh * gw
                wpos = torch.arange(cur, cur + gw).repeat(gh * t)
                hpos = torch.arange(cur, cur + gh).repeat_interleave(gw * t)
                tpos = torch.full((n,), cur, dtype=torch.long)
                parts.append(torch.stack([tpos, hpos, wpos]))
                cur += max(gh, gw)
                done += n
        pos[:, b] = torch.cat(parts, dim=1).to(pos.device)
    return pos


class Qwen2VLForConditionalGeneration(PretrainedModel):
    """Qwen2-VL and (with a ``Qwen2_5_VLConfig``) Qwen2.5-VL."""

    config_class = Qwen2VLConfig

    def __init__(self, config: Qwen2VLConfig, dtype=None, device=None):
        super().__init__(config)
        tower = WindowedVisionTower if isinstance(config, Qwen2_5_VLConfig) else VisionTower
        self.visual = tower(config.vision_config, dtype=dtype, device=device)
        self.language = DecoderForCausalLM(config.text_config, dtype=dtype, device=device)
        # tensor names differ between generations of checkpoints: the vision tower is stored as "visual.*" or
        # "model.visual.*", the decoder as "model.*" or "model.language_model.*"; both are probed on load, and the writer
        # uses "model.visual.*" + "model.*", which current and older readers of the format accept
        self._vision_prefix, self._text_nested = "model.visual.", False

    # ------------------------------------------------------------------ rotary tables
    def _context(self, input_ids, position_ids3) -> BatchContext:
        B, S = input_ids.shape
        lm = self.language.model
        D = self.config.text_config.head_dim
        cos_t, sin_t = lm.rope(input_ids.device, int(position_ids3.max().item()) + 1)
        sections = self.config.mrope_section or [D // 2]
        axis = torch.repeat_interleave(torch.arange(len(sections), device=input_ids.device) % 3,
                                       torch.tensor(sections, device=input_ids.device))           # [D / 2] -> t / h / w
        flat = position_ids3.reshape(3, B * S)
        sel = flat[axis]                                                                            # [D / 2, B * S]
        col = torch.arange(D // 2, device=input_ids.device)[:, None]
        cos = cos_t[sel, col].t().contiguous()                                                      # [B * S, D / 2]
        sin = sin_t[sel, col].t().contiguous()
        return BatchContext(B, S, torch.arange(B * S, device=input_ids.device), None, cos, sin)

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids, pixel_values=None, image_grid_thw=None, pixel_values_videos=None, video_grid_thw=None, labels=None,
                position_ids=None, return_logits: Optional[bool] = None, **unused):
        cfg, lm = self.config, self.language
        h = lm.model.embed(input_ids, whole=True)
        for pv, grid, tok in ((pixel_values, image_grid_thw, cfg.image_token_id), (pixel_values_videos, video_grid_thw, cfg.video_token_id)):
            if pv is not None:
                feats = self.visual(pv, grid).to(h.dtype)
                mask = (input_ids.reshape(-1) == tok)
                assert int(mask.sum()) == feats.shape[0], "one placeholder token per merged patch is required"
                h = h.masked_scatter(mask[:, None], feats)
        if position_ids is None:
            position_ids = multimodal_position_ids(input_ids, cfg.image_token_id, cfg.video_token_id, image_grid_thw, video_grid_thw,
                                                   cfg.vision_config["spatial_merge_size"])
        ctx = self._context(input_ids, position_ids)
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

    # ------------------------------------------------------------------ checkpoint names
    def load_hf_checkpoint(self, directory: str, strict: bool = False) -> None:
        from ..transformers.model_utils import _CheckpointReader

        reader = _CheckpointReader(directory)
        saved = (self._vision_prefix, self._text_nested)
        self._vision_prefix = "visual." if reader.has("visual.patch_embed.proj.weight") else "model.visual."
        self._text_nested = reader.has("model.language_model.embed_tokens.weight")
        try:
            super().load_hf_checkpoint(directory, strict)
        finally:
            self._vision_prefix, self._text_nested = saved

    def weight_map(self) -> WeightMap:
        vis = self._vision_prefix

        def text_name(s: str) -> str:
            if s.startswith("lm_head.") or not self._text_nested:
                return s
            return s.replace("model.", "model.language_model.", 1)

        rules = []
        for r in build_weight_map(self.config.text_config).rules.values():
            rules.append(Rule("language." + r.target, [text_name(s) for s in r.sources], r.op, r.dim, r.num_experts, r.expert_pairs,
                              r.sizes, r.rope_deinterleave, r.flatten))
        known = {r.target for r in rules}
        for name, _ in self.language.named_parameters():                 # parameters without a fusion rule: renamed only
            t = "language." + name
            if t not in known:
                rules.append(Rule(t, [text_name(name)]))
        vc = self.config.vision_config
        windowed = isinstance(self.config, Qwen2_5_VLConfig)
        width = vc["hidden_size"] if windowed else vc["embed_dim"]
        conv_shape = [width, vc["in_channels"], vc["temporal_patch_size"], vc["patch_size"], vc["patch_size"]]
        rules.append(Rule("visual.patch_embed.weight", [vis + "patch_embed.proj.weight"], reshape=[width, -1], source_shape=conv_shape))
        mlp_names = (("gate_proj", "mlp.gate_proj"), ("up_proj", "mlp.up_proj"), ("down_proj", "mlp.down_proj")) if windowed else \
            (("fc1", "mlp.fc1"), ("fc2", "mlp.fc2"))
        own = dict(self.visual.named_parameters())
        for i in range(vc["depth"]):
            a, b = f"visual.blocks.{i}.", vis + f"blocks.{i}."
            for mine, theirs in (("norm1", "norm1"), ("norm2", "norm2"), ("qkv", "attn.qkv"), ("proj", "attn.proj")) + mlp_names:
                for leaf in ("weight", "bias"):
                    if f"blocks.{i}.{mine}.{leaf}" in own:              # RMSNorm has no bias
                        rules.append(Rule(a + f"{mine}.{leaf}", [b + f"{theirs}.{leaf}"]))
        for mine, theirs in (("ln_q", "merger.ln_q"), ("merge_fc1", "merger.mlp.0"), ("merge_fc2", "merger.mlp.2")):
            for leaf in ("weight", "bias"):
                if f"{mine}.{leaf}" in own:
                    rules.append(Rule(f"visual.{mine}.{leaf}", [vis + f"{theirs}.{leaf}"]))
        return WeightMap(rules)


def mm_collate_fn(examples: List[dict], pad_token_id: int = 0, ignore_index: int = -100) -> dict:
    """Batch multimodal examples: ``input_ids`` / ``labels`` are padded to the longest row, the patch tensors of all
    images are concatenated in example order with their grids (the layout ``Qwen2VLForConditionalGeneration`` expects)."""
    S = max(len(e["input_ids"]) for e in examples)
    ids = torch.full((len(examples), S), pad_token_id, dtype=torch.long)
    labels = torch.full((len(examples), S), ignore_index, dtype=torch.long)
    for i, e in enumerate(examples):
        n = len(e["input_ids"])
        ids[i, :n] = torch.as_tensor(e["input_ids"])
        if "labels" in e:
            labels[i, :n] = torch.as_tensor(e["labels"])
    out = {"input_ids": ids, "labels": labels}
    pv = [torch.as_tensor(e["pixel_values"]) for e in examples if e.get("pixel_values") is not None]
    if pv:
        out["pixel_values"] = torch.cat(pv, dim=0)
        grids = [torch.as_tensor(e["image_grid_thw"]).reshape(-1, 3) for e in examples if e.get("image_grid_thw") is not None]
        if grids:                                      # fixed-size towers have no grids
            out["image_grid_thw"] = torch.cat(grids, dim=0)
    if any("token_type_ids" in e for e in examples):   # prefix-LM families; padding counts as (causal) answer positions
        types = torch.ones((len(examples), S), dtype=torch.long)
        for i, e in enumerate(examples):
            types[i, :len(e["token_type_ids"])] = torch.as_tensor(e["token_type_ids"])
        out["token_type_ids"] = types
    return out


class Qwen2_5_VLForConditionalGeneration(Qwen2VLForConditionalGeneration):
    config_class = Qwen2_5_VLConfig



# ---------------------------------------------------------------------------------------------------------------
# Qwen3-VL
# ---------------------------------------------------------------------------------------------------------------
class Qwen3VLConfig(Qwen2VLConfig):
    """Qwen3-VL: a Qwen3 decoder (per-head QK norm) whose rotary frequencies take the temporal / height / width position in
    an interleaved pattern, a vision tower with learned position embeddings interpolated to the image grid, and "deepstack":
    features of intermediate vision blocks are added to the visual tokens after the first decoder layers
    (paddleformers/transformers/qwen3_vl)."""

    model_type = "qwen3_vl"
    text_model_type = "qwen3_vl_text"

    def _text_class(self):
        from .configuration import Qwen3Config

        return Qwen3Config

    def __init__(self, text_config=None, vision_config=None, **kwargs):

        text = dict(text_config or {})
        text.pop("model_type", None)
        rp = dict(text.get("rope_parameters") or text.get("rope_scaling") or {})
        section = list(rp.pop("mrope_section", None) or [24, 20, 20])
        rp.pop("mrope_interleaved", None)
        if "rope_parameters" in text:
            text["rope_parameters"] = rp
        elif "rope_scaling" in text:
            text["rope_scaling"] = rp if rp.get("rope_type", rp.get("type", "default")) not in ("default", "mrope") else None
        tie = bool(text.get("tie_word_embeddings", kwargs.get("tie_word_embeddings", False)))
        text.setdefault("tie_word_embeddings", tie)
        text.setdefault("use_qk_norm", True)
        text.setdefault("rope_theta", 5000000.0)
        super().__init__(text_config={"num_hidden_layers": 1}, vision_config={}, **{**kwargs, "tie_word_embeddings": tie})
        self.text_config = self._text_class()(**text)
        self.mrope_section, self.mrope_interleaved = section, True
        v = dict(vision_config or {})
        v.pop("model_type", None)
        self.vision_config = {"depth": 27, "hidden_size": 1152, "hidden_act": "gelu_pytorch_tanh", "intermediate_size": 4304,
                              "num_heads": 16, "in_channels": 3, "patch_size": 16, "spatial_merge_size": 2, "temporal_patch_size": 2,
                              "out_hidden_size": self.text_config.hidden_size, "num_position_embeddings": 2304,
                              "deepstack_visual_indexes": [8, 16, 24], **v}

    def to_dict(self, saving: bool = False):
        d = PretrainedConfig.to_dict(self, saving)
        text = self.text_config.to_dict(saving)
        text["model_type"] = self.text_model_type
        scaling = text.pop("rope_scaling", None) or {}
        text["rope_parameters"] = {"rope_type": "default", **scaling, "rope_theta": text.pop("rope_theta", self.text_config.rope_theta),
                                   "mrope_section": self.mrope_section, "mrope_interleaved": True}
        d["text_config"] = text
        d["vision_config"] = dict(self.vision_config, model_type=self.model_type)
        d.pop("mrope_section", None)
        d.pop("mrope_interleaved", None)
        return d


class Qwen3VLMoeConfig(Qwen3VLConfig):
    """Qwen3-VL with the Qwen3-MoE decoder (paddleformers/transformers/qwen3_vl_moe)."""

    model_type = "qwen3_vl_moe"
    text_model_type = "qwen3_vl_moe_text"

    def _text_class(self):
        from .configuration import Qwen3MoeConfig

        def make(**kw):
            cfg = Qwen3MoeConfig(**kw)
            cfg.hf_fused_experts = True        # this family's checkpoints hold the experts as stacked tensors
            return cfg

        return make

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving and "num_experts" in d["text_config"]:
            d["text_config"]["num_local_experts"] = d["text_config"]["num_experts"]
        return d


class _Merger(nn.Module):
    """LayerNorm (before or after the merge-block shuffle) -> linear -> GELU -> linear to the decoder width."""

    def __init__(self, dim: int, unit: int, out_dim: int, post_shuffle_norm: bool, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.width, self.post = dim * unit, post_shuffle_norm
        self.norm = nn.LayerNorm(self.width if post_shuffle_norm else dim, eps=1e-6, **kw)
        self.fc1 = nn.Linear(self.width, self.width, **kw)
        self.fc2 = nn.Linear(self.width, out_dim, **kw)

    def forward(self, x):
        x = self.norm(x.view(-1, self.width)) if self.post else self.norm(x).view(-1, self.width)
        return self.fc2(TF.gelu(self.fc1(x)))


class Qwen3VisionTower(VisionTower):
    def __init__(self, vc: dict, dtype=None, device=None):
        nn.Module.__init__(self)
        kw = dict(dtype=dtype, device=device)
        self.vc = vc
        dim = vc["hidden_size"]
        self.patch_dim = vc["in_channels"] * vc["temporal_patch_size"] * vc["patch_size"] ** 2
        self.patch_embed = nn.Linear(self.patch_dim, dim, bias=True, **kw)
        self.pos_embed = nn.Embedding(vc["num_position_embeddings"], dim, **kw)
        self.side = int(vc["num_position_embeddings"] ** 0.5)
        self.blocks = nn.ModuleList([_VisionBlock(dim, vc["num_heads"], vc["intermediate_size"], vc["hidden_act"], **kw)
                                     for _ in range(vc["depth"])])
        unit = vc["spatial_merge_size"] ** 2
        self.merger = _Merger(dim, unit, vc["out_hidden_size"], False, **kw)
        self.deepstack_indexes = list(vc["deepstack_visual_indexes"])
        self.deepstack_mergers = nn.ModuleList([_Merger(dim, unit, vc["out_hidden_size"], True, **kw) for _ in self.deepstack_indexes])
        self.head_dim = dim // vc["num_heads"]

    def position_embeddings(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """The learned side x side table, bilinearly interpolated to every image's patch grid (corners aligned), repeated
        over frames and put in the processor's merge-block patch order."""
        ms, side = self.vc["spatial_merge_size"], self.side
        table = self.pos_embed.weight
        out = []
        for t, h, w in grid_thw.tolist():
            hs = torch.linspace(0, side - 1, h, device=table.device)
            ws = torch.linspace(0, side - 1, w, device=table.device)
            h0, w0 = hs.long(), ws.long()
            h1, w1 = (h0 + 1).clamp(max=side - 1), (w0 + 1).clamp(max=side - 1)
            dh, dw = (hs - h0)[:, None].to(table.dtype), (ws - w0)[None, :].to(table.dtype)

            def at(r, c):
                return table[(r[:, None] * side + c[None, :]).reshape(-1)].view(h, w, -1)

            e = at(h0, w0) * ((1 - dh) * (1 - dw))[..., None] + at(h0, w1) * ((1 - dh) * dw)[..., None] \
                + at(h1, w0) * (dh * (1 - dw))[..., None] + at(h1, w1) * (dh * dw)[..., None]
            e = e.view(h // ms, ms, w // ms, ms, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(e.repeat(t, 1))
        return torch.cat(out, dim=0)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor):
        x = self.patch_embed(pixel_values.to(self.patch_embed.weight.dtype))
        x = x + self.position_embeddings(grid_thw).to(x.dtype)
        cos, sin = self.rotary(grid_thw, x.device)
        lengths = [h * w for t, h, w in grid_thw.tolist() for _ in range(t)]
        deep = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, lengths)
            if i in self.deepstack_indexes:
                deep.append(self.deepstack_mergers[self.deepstack_indexes.index(i)](x))
        return self.merger(x), deep


class Qwen3VLForConditionalGeneration(Qwen2VLForConditionalGeneration):
    config_class = Qwen3VLConfig

    def __init__(self, config: Qwen3VLConfig, dtype=None, device=None):
        PretrainedModel.__init__(self, config)
        self.visual = Qwen3VisionTower(config.vision_config, dtype=dtype, device=device)
        self.language = DecoderForCausalLM(config.text_config, dtype=dtype, device=device)
        self._vision_prefix, self._text_nested = "model.visual.", True

    def _context(self, input_ids, position_ids3) -> BatchContext:
        B, S = input_ids.shape
        lm = self.language.model
        D = self.config.text_config.head_dim
        cos_t, sin_t = lm.rope(input_ids.device, int(position_ids3.max().item()) + 1)
        # interleaved sections: frequency i follows the temporal position unless i = 1 (mod 3) below 3 * section[1] (height)
        # or i = 2 (mod 3) below 3 * section[2] (width)
        axis = torch.zeros(D // 2, dtype=torch.long, device=input_ids.device)
        sec = self.config.mrope_section
        axis[1:sec[1] * 3:3] = 1
        axis[2:sec[2] * 3:3] = 2
        flat = position_ids3.reshape(3, B * S)
        sel = flat[axis]
        col = torch.arange(D // 2, device=input_ids.device)[:, None]
        return BatchContext(B, S, torch.arange(B * S, device=input_ids.device), None, cos_t[sel, col].t().contiguous(),
                            sin_t[sel, col].t().contiguous())

    def forward(self, input_ids, pixel_values=None, image_grid_thw=None, pixel_values_videos=None, video_grid_thw=None, labels=None,
                position_ids=None, return_logits: Optional[bool] = None, **unused):
        cfg, lm = self.config, self.language
        if lm.model.sp:
            raise NotImplementedError("deepstack features are added to whole-sequence hidden states: this model runs without "
                                      "sequence parallelism")
        h = lm.model.embed(input_ids)
        flat_ids = input_ids.reshape(-1)
        visual_rows, deep_feats = [], None
        frames_grid = None
        if video_grid_thw is not None:          # every frame of a video is placed like an image (text may sit between frames)
            frames_grid = torch.repeat_interleave(video_grid_thw, video_grid_thw[:, 0], dim=0).clone()
            frames_grid[:, 0] = 1
        for pv, grid, tok in ((pixel_values, image_grid_thw, cfg.image_token_id), (pixel_values_videos, video_grid_thw, cfg.video_token_id)):
            if pv is None:
                continue
            feats, deep = self.visual(pv, grid)
            rows = (flat_ids == tok).nonzero(as_tuple=True)[0]
            assert rows.numel() == feats.shape[0], "one placeholder token per merged patch is required"
            h = h.index_copy(0, rows, feats.to(h.dtype))
            visual_rows.append(rows)
            deep_feats = deep if deep_feats is None else [torch.cat([a, b], dim=0) for a, b in zip(deep_feats, deep)]
        if position_ids is None:
            position_ids = multimodal_position_ids(input_ids, cfg.image_token_id, cfg.video_token_id, image_grid_thw, frames_grid,
                                                   cfg.vision_config["spatial_merge_size"])
        ctx = self._context(input_ids, position_ids)
        hidden, residual = h, None
        rows = torch.cat(visual_rows) if visual_rows else None
        for i, layer in enumerate(lm.model.layers.values()):
            hidden, residual = layer(hidden, residual, ctx)
            if deep_feats is not None and i < len(deep_feats):
                # the layer's output is hidden + residual (the add runs inside the next norm): adding to either term adds to it
                add = deep_feats[i].to(hidden.dtype)
                if residual is None:
                    hidden = hidden.index_add(0, rows, add)
                else:
                    residual = residual.index_add(0, rows, add)
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
        PretrainedModel.load_hf_checkpoint(self, directory, strict)

    def weight_map(self) -> WeightMap:
        vis = "model.visual."
        rules = []
        for r in build_weight_map(self.config.text_config).rules.values():
            src = [s if s.startswith("lm_head.") else s.replace("model.", "model.language_model.", 1) for s in r.sources]
            rules.append(Rule("language." + r.target, src, r.op, r.dim, r.num_experts, r.expert_pairs, r.sizes, r.rope_deinterleave,
                              r.flatten, r.reshape, r.source_shape, r.offset, fn=r.fn, qkv_groups=r.qkv_groups))
        known = {r.target for r in rules}
        for name, _ in self.language.named_parameters():
            if "language." + name not in known:
                rules.append(Rule("language." + name, [name if name.startswith("lm_head.") else name.replace("model.", "model.language_model.", 1)]))
        vc = self.config.vision_config
        width = vc["hidden_size"]
        conv_shape = [width, vc["in_channels"], vc["temporal_patch_size"], vc["patch_size"], vc["patch_size"]]
        rules.append(Rule("visual.patch_embed.weight", [vis + "patch_embed.proj.weight"], reshape=[width, -1], source_shape=conv_shape))
        rules.append(Rule("visual.patch_embed.bias", [vis + "patch_embed.proj.bias"]))
        rules.append(Rule("visual.pos_embed.weight", [vis + "pos_embed.weight"]))
        for i in range(vc["depth"]):
            a, b = f"visual.blocks.{i}.", vis + f"blocks.{i}."
            for mine, theirs in (("norm1", "norm1"), ("norm2", "norm2"), ("qkv", "attn.qkv"), ("proj", "attn.proj"),
                                 ("fc1", "mlp.linear_fc1"), ("fc2", "mlp.linear_fc2")):
                for leaf in ("weight", "bias"):
                    rules.append(Rule(a + f"{mine}.{leaf}", [b + f"{theirs}.{leaf}"]))
        mergers = [("visual.merger.", vis + "merger.")] + [(f"visual.deepstack_mergers.{k}.", vis + f"deepstack_merger_list.{k}.")
                                                           for k in range(len(vc["deepstack_visual_indexes"]))]
        for a, b in mergers:
            for mine, theirs in (("norm", "norm"), ("fc1", "linear_fc1"), ("fc2", "linear_fc2")):
                for leaf in ("weight", "bias"):
                    rules.append(Rule(a + f"{mine}.{leaf}", [b + f"{theirs}.{leaf}"]))
        return WeightMap(rules)


class Qwen3VLMoeForConditionalGeneration(Qwen3VLForConditionalGeneration):
    config_class = Qwen3VLMoeConfig


# ---------------------------------------------------------------------------------------------------------------
# GLM-4.5V
# ---------------------------------------------------------------------------------------------------------------
class Glm4vMoeConfig(Qwen2VLConfig):
    """GLM-4.5V: the GLM-4.5 MoE decoder with multimodal rotary sections on its rotated half of each head, and a vision tower
    with RMSNorm / bias-free SwiGLU blocks, bicubically interpolated position embeddings, a strided-convolution merge of
    2 x 2 patches and a gated merger MLP (paddleformers/transformers/glm4v_moe)."""

    model_type = "glm4v_moe"

    def __init__(self, text_config=None, vision_config=None, image_token_id=151363, video_token_id=151364, image_start_token_id=151339,
                 image_end_token_id=151340, **kwargs):
        text = dict(text_config or {})
        text.pop("model_type", None)
        rp = dict(text.get("rope_parameters") or {})
        section = list(rp.pop("mrope_section", None) or [8, 12, 12])
        if "rope_parameters" in text:
            text["rope_parameters"] = rp
        tie = bool(text.get("tie_word_embeddings", kwargs.get("tie_word_embeddings", False)))
        text.setdefault("tie_word_embeddings", tie)
        for k, v in self._text_defaults.items():
            text.setdefault(k, v)
        for k in ("video_start_token_id", "video_end_token_id"):
            kwargs.pop(k, None)
        super().__init__(text_config={"num_hidden_layers": 1}, vision_config={}, image_token_id=image_token_id,
                         video_token_id=video_token_id, vision_start_token_id=image_start_token_id,
                         vision_end_token_id=image_end_token_id, **{**kwargs, "tie_word_embeddings": tie})
        self.text_config = self._text_class()(**text)
        self.mrope_section = section
        self.image_start_token_id, self.image_end_token_id = image_start_token_id, image_end_token_id
        v = dict(vision_config or {})
        v.pop("model_type", None)
        self.vision_config = {"depth": 24, "hidden_size": 1536, "hidden_act": "silu", "attention_bias": False, "num_heads": 12,
                              "in_channels": 3, "image_size": 336, "patch_size": 14, "rms_norm_eps": 1e-5, "spatial_merge_size": 2,
                              "temporal_patch_size": 2, "out_hidden_size": self.text_config.hidden_size, "intermediate_size": 13696,
                              **self._vision_defaults, **v}

    _text_defaults = {"attention_bias": True, "use_qk_norm": False}
    _vision_defaults: dict = {}
    _text_type, _vision_type = "glm4v_moe_text", "glm4v_moe_vision"

    @staticmethod
    def _text_class():
        from .configuration import Glm4MoeConfig

        return Glm4MoeConfig

    def to_dict(self, saving: bool = False):
        d = PretrainedConfig.to_dict(self, saving)
        text = self.text_config.to_dict(saving)
        text["model_type"] = self._text_type
        scaling = text.pop("rope_scaling", None) or {}
        text["rope_parameters"] = {"rope_type": "default", **scaling, "rope_theta": text.pop("rope_theta", self.text_config.rope_theta),
                                   "partial_rotary_factor": self.text_config.partial_rotary_factor, "mrope_section": self.mrope_section}
        d["text_config"] = text
        d["vision_config"] = dict(self.vision_config, model_type=self._vision_type)
        for k in ("mrope_section", "vision_start_token_id", "vision_end_token_id"):
            d.pop(k, None)
        return d


class Glm4vVisionTower(VisionTower):
    def __init__(self, vc: dict, dtype=None, device=None):
        nn.Module.__init__(self)
        kw = dict(dtype=dtype, device=device)
        self.vc = vc
        dim, out, eps, ms = vc["hidden_size"], vc["out_hidden_size"], vc["rms_norm_eps"], vc["spatial_merge_size"]
        self.patch_dim = vc["in_channels"] * vc["temporal_patch_size"] * vc["patch_size"] ** 2
        self.patch_embed = nn.Linear(self.patch_dim, dim, bias=True, **kw)
        self.post_conv_layernorm = _RMSNorm(dim, eps, **kw)
        self.side = vc["image_size"] // vc["patch_size"]
        self.position_embedding = nn.Embedding(self.side ** 2, dim, **kw)
        # the blocks' MLP width is the OUTPUT width of the tower; ``intermediate_size`` belongs to the merger
        self.blocks = nn.ModuleList([_VisionBlock(dim, vc["num_heads"], out, vc["hidden_act"], rms_norm=True, swiglu=True,
                                                  bias=bool(vc.get("attention_bias", False)), mlp_bias=False, eps=eps, **kw) for _ in range(vc["depth"])])
        self.post_layernorm = _RMSNorm(dim, eps, **kw)
        self.downsample = nn.Linear(dim * ms * ms, out, bias=True, **kw)          # the stride-ms convolution over one merge block
        self.merge_proj = nn.Linear(out, out, bias=False, **kw)
        self.merge_norm = nn.LayerNorm(out, **kw)
        self.merge_gate = nn.Linear(out, vc["intermediate_size"], bias=False, **kw)
        self.merge_up = nn.Linear(out, vc["intermediate_size"], bias=False, **kw)
        self.merge_down = nn.Linear(vc["intermediate_size"], out, bias=False, **kw)
        self.head_dim = dim // vc["num_heads"]

    def position_embeddings(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """Bicubic samples of the learned side x side table at the centre of every patch (coordinates relative to the image's own
        grid), in the processor's merge-block patch order."""
        ms, side = self.vc["spatial_merge_size"], self.side
        table = self.position_embedding.weight
        table2d = table.view(side, side, -1).permute(2, 0, 1)[None].float()
        out = []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h, device=table.device)[:, None].expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(w, device=table.device)[None, :].expand(h, w).reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).flatten()
            grid = torch.stack([(wp.float() + 0.5) / w * 2 - 1, (hp.float() + 0.5) / h * 2 - 1], dim=-1)[None, :, None, :]
            e = TF.grid_sample(table2d, grid, mode="bicubic", align_corners=False, padding_mode="border")[0, :, :, 0].t()
            out.append(e.to(table.dtype).repeat(t, 1))
        return torch.cat(out, dim=0)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        ms = self.vc["spatial_merge_size"]
        x = self.post_conv_layernorm(self.patch_embed(pixel_values.to(self.patch_embed.weight.dtype)))
        x = x + self.position_embeddings(grid_thw).to(x.dtype)
        cos, sin = self.rotary(grid_thw, x.device)
        lengths = [h * w for t, h, w in grid_thw.tolist() for _ in range(t)]
        for blk in self.blocks:
            x = blk(x, cos, sin, lengths)
        x = self.post_layernorm(x)
        # a merge block's ms x ms patches are consecutive rows: channel-major flattening matches the convolution's weight layout
        x = x.view(-1, ms, ms, x.shape[-1]).permute(0, 3, 1, 2).reshape(-1, x.shape[-1] * ms * ms)
        x = self.merge_proj(self.downsample(x))
        x = TF.gelu(self.merge_norm(x))
        return self.merge_down(TF.silu(self.merge_gate(x)) * self.merge_up(x))


class Glm4vMoeForConditionalGeneration(Qwen2VLForConditionalGeneration):
    config_class = Glm4vMoeConfig

    def __init__(self, config: Glm4vMoeConfig, dtype=None, device=None):
        PretrainedModel.__init__(self, config)
        self.visual = Glm4vVisionTower(config.vision_config, dtype=dtype, device=device)
        self.language = DecoderForCausalLM(config.text_config, dtype=dtype, device=device)
        self._vision_prefix, self._text_nested = "model.visual.", True

    def _context(self, input_ids, position_ids3) -> BatchContext:
        B, S = input_ids.shape
        lm = self.language.model
        half = int(self.config.text_config.head_dim * self.config.text_config.partial_rotary_factor) // 2     # rotated frequencies
        cos_t, sin_t = lm.rope(input_ids.device, int(position_ids3.max().item()) + 1)
        sections = self.config.mrope_section
        assert sum(sections) == half, "mrope sections must cover the rotated half of the head"
        axis = torch.repeat_interleave(torch.arange(len(sections), device=input_ids.device) % 3,
                                       torch.tensor(sections, device=input_ids.device))
        sel = position_ids3.reshape(3, B * S)[axis]
        col = torch.arange(half, device=input_ids.device)[:, None]
        return BatchContext(B, S, torch.arange(B * S, device=input_ids.device), None, cos_t[sel, col].t().contiguous(),
                            sin_t[sel, col].t().contiguous())

    def load_hf_checkpoint(self, directory: str, strict: bool = False) -> None:
        PretrainedModel.load_hf_checkpoint(self, directory, strict)

    def weight_map(self) -> WeightMap:
        vis = "model.visual."
        rules = []
        text_map = build_weight_map(self.config.text_config)
        for r in text_map.rules.values():
            src = [x if x.startswith("lm_head.") else x.replace("model.", "model.language_model.", 1) for x in r.sources]
            rules.append(Rule("language." + r.target, src, r.op, r.dim, r.num_experts, r.expert_pairs, r.sizes, r.rope_deinterleave,
                              r.flatten, r.reshape, r.source_shape, r.offset, fn=r.fn, qkv_groups=r.qkv_groups))
        known = {r.target for r in rules}
        for name, _ in list(self.language.named_parameters()) + [(k, None) for k, _ in self.language.named_buffers()]:
            if "language." + name not in known and (name in dict(self.language.named_parameters()) or name in self.language.state_dict()):
                theirs = text_map.translate(name)            # the text family's own spelling of plainly renamed tensors
                rules.append(Rule("language." + name, [theirs if theirs.startswith("lm_head.") else theirs.replace("model.", "model.language_model.", 1)]))
        vc = self.config.vision_config
        dim, out, ms = vc["hidden_size"], vc["out_hidden_size"], vc["spatial_merge_size"]
        conv_shape = [dim, vc["in_channels"], vc["temporal_patch_size"], vc["patch_size"], vc["patch_size"]]
        rules += [Rule("visual.patch_embed.weight", [vis + "patch_embed.proj.weight"], reshape=[dim, -1], source_shape=conv_shape),
                  Rule("visual.patch_embed.bias", [vis + "patch_embed.proj.bias"]),
                  Rule("visual.post_conv_layernorm.weight", [vis + "post_conv_layernorm.weight"]),
                  Rule("visual.position_embedding.weight", [vis + "embeddings.position_embedding.weight"]),
                  Rule("visual.post_layernorm.weight", [vis + "post_layernorm.weight"]),
                  Rule("visual.downsample.weight", [vis + "downsample.weight"], reshape=[out, -1], source_shape=[out, dim, ms, ms]),
                  Rule("visual.downsample.bias", [vis + "downsample.bias"]),
                  Rule("visual.merge_proj.weight", [vis + "merger.proj.weight"]),
                  Rule("visual.merge_norm.weight", [vis + "merger.post_projection_norm.weight"]),
                  Rule("visual.merge_norm.bias", [vis + "merger.post_projection_norm.bias"]),
                  Rule("visual.merge_gate.weight", [vis + "merger.gate_proj.weight"]),
                  Rule("visual.merge_up.weight", [vis + "merger.up_proj.weight"]),
                  Rule("visual.merge_down.weight", [vis + "merger.down_proj.weight"])]
        own = dict(self.visual.named_parameters())
        for i in range(vc["depth"]):
            a, b = f"visual.blocks.{i}.", vis + f"blocks.{i}."
            for mine, theirs in (("norm1", "norm1"), ("norm2", "norm2"), ("qkv", "attn.qkv"), ("proj", "attn.proj"),
                                 ("gate_proj", "mlp.gate_proj"), ("up_proj", "mlp.up_proj"), ("down_proj", "mlp.down_proj")):
                for leaf in ("weight", "bias"):
                    if f"blocks.{i}.{mine}.{leaf}" in own:
                        rules.append(Rule(a + f"{mine}.{leaf}", [b + f"{theirs}.{leaf}"]))
        return WeightMap(rules)


class GlmOcrConfig(Glm4vMoeConfig):
    """GLM-OCR (paddleformers/transformers/glm_ocr): the dense GLM-4 decoder with multimodal rotary sections, and the GLM-4.5V
    vision tower without learned position embeddings, with per-head RMSNorm on queries and keys, biased projections and a
    merger three times the output width."""

    model_type = "glm_ocr"
    _text_defaults = {"attention_bias": False}
    _vision_defaults = {"hidden_size": 1024, "attention_bias": True, "num_heads": 16, "out_hidden_size": 1536, "intermediate_size": 4096}
    _text_type, _vision_type = "glm_ocr_text", "glm_ocr_vision"

    def __init__(self, image_token_id=59280, video_token_id=59281, image_start_token_id=59256, image_end_token_id=59257, **kwargs):
        super().__init__(image_token_id=image_token_id, video_token_id=video_token_id, image_start_token_id=image_start_token_id,
                         image_end_token_id=image_end_token_id, **kwargs)

    @staticmethod
    def _text_class():
        from .configuration import Glm4Config

        return Glm4Config


class GlmOcrVisionTower(Glm4vVisionTower):
    def __init__(self, vc: dict, dtype=None, device=None):
        nn.Module.__init__(self)
        kw = dict(dtype=dtype, device=device)
        self.vc = vc
        dim, out, eps, ms = vc["hidden_size"], vc["out_hidden_size"], vc["rms_norm_eps"], vc["spatial_merge_size"]
        bias = bool(vc.get("attention_bias", True))
        self.patch_dim = vc["in_channels"] * vc["temporal_patch_size"] * vc["patch_size"] ** 2
        self.patch_embed = nn.Linear(self.patch_dim, dim, bias=True, **kw)
        self.blocks = nn.ModuleList([_VisionBlock(dim, vc["num_heads"], vc["intermediate_size"], vc["hidden_act"], rms_norm=True, swiglu=True,
                                                  bias=bias, mlp_bias=bias, eps=eps, qk_norm=True, **kw) for _ in range(vc["depth"])])
        self.post_layernorm = _RMSNorm(dim, eps, **kw)
        self.downsample = nn.Linear(dim * ms * ms, out, bias=True, **kw)
        wide = out * vc["in_channels"]
        self.merge_proj = nn.Linear(out, out, bias=False, **kw)
        self.merge_norm = nn.LayerNorm(out, **kw)
        self.merge_gate = nn.Linear(out, wide, bias=False, **kw)
        self.merge_up = nn.Linear(out, wide, bias=False, **kw)
        self.merge_down = nn.Linear(wide, out, bias=False, **kw)
        self.head_dim = dim // vc["num_heads"]

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        ms = self.vc["spatial_merge_size"]
        x = self.patch_embed(pixel_values.to(self.patch_embed.weight.dtype))
        cos, sin = self.rotary(grid_thw, x.device)
        lengths = [h * w for t, h, w in grid_thw.tolist() for _ in range(t)]
        for blk in self.blocks:
            x = blk(x, cos, sin, lengths)
        x = self.post_layernorm(x)
        x = x.view(-1, ms, ms, x.shape[-1]).permute(0, 3, 1, 2).reshape(-1, x.shape[-1] * ms * ms)
        x = self.merge_proj(self.downsample(x))
        x = TF.gelu(self.merge_norm(x))
        return self.merge_down(TF.silu(self.merge_gate(x)) * self.merge_up(x))


class GlmOcrForConditionalGeneration(Glm4vMoeForConditionalGeneration):
    config_class = GlmOcrConfig

    def __init__(self, config: GlmOcrConfig, dtype=None, device=None):
        PretrainedModel.__init__(self, config)
        self.visual = GlmOcrVisionTower(config.vision_config, dtype=dtype, device=device)
        self.language = DecoderForCausalLM(config.text_config, dtype=dtype, device=device)
        self._vision_prefix, self._text_nested = "model.visual.", True

    def weight_map(self) -> WeightMap:
        base = super().weight_map()
        own = dict(self.named_parameters())
        rules = [r for r in base.rules.values() if r.target in own]        # no position table, no norm after the patch projection
        for i in range(self.config.vision_config["depth"]):
            for n in ("q_norm", "k_norm"):
                rules.append(Rule(f"visual.blocks.{i}.{n}.weight", [f"model.visual.blocks.{i}.attn.{n}.weight"]))
        return WeightMap(rules)
