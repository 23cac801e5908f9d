"""Text generation: greedy, sampling (temperature / top-k / top-p / repetition penalty), beam search and diverse
(group) beam search, with a key/value cache, stopping criteria and a streamer hook.

Counterpart: paddleformers/generation/utils.py:347 (``GenerationMixin``), :818 (``generate``), the logits processors
and stopping criteria of paddleformers/generation/.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Callable, List, Optional

import torch
import torch.nn.functional as TF


@dataclass
class GenerationConfig:
    max_new_tokens: int = 64
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    num_beams: int = 1
    num_beam_groups: int = 1
    diversity_penalty: float = 0.0
    num_return_sequences: int = 1
    length_penalty: float = 1.0
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None
    stop_token_ids: List[int] = field(default_factory=list)

    def save_pretrained(self, d: str):
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, "generation_config.json"), "w") as f:
            json.dump(asdict(self), f, indent=2)

    @classmethod
    def from_pretrained(cls, d: str):
        p = os.path.join(d, "generation_config.json")
        if not os.path.exists(p):
            return cls()
        with open(p) as f:
            raw = json.load(f)
        return cls(**{k: v for k, v in raw.items() if k in cls.__dataclass_fields__})


class KVCache:
    """Per-layer key / value store for incremental decoding (GQA layers of the unified decoder)."""

    def __init__(self):
        self.k: Optional[torch.Tensor] = None   # [B, S, Hkv, D]
        self.v: Optional[torch.Tensor] = None

    def attend(self, attn, qkv2d, ctx):
        B, S, Hq, Hkv, D = ctx.B, ctx.S, attn.Hq, attn.Hkv, attn.D
        q = qkv2d[:, : Hq * D].reshape(B, S, Hq, D)
        k = qkv2d[:, Hq * D:(Hq + Hkv) * D].reshape(B, S, Hkv, D)
        v = qkv2d[:, (Hq + Hkv) * D:].reshape(B, S, Hkv, D)
        self.k = k if self.k is None else torch.cat([self.k, k], 1)
        self.v = v if self.v is None else torch.cat([self.v, v], 1)
        Sk = self.k.shape[1]
        qf = q.permute(0, 2, 1, 3).float()
        kf = self.k.permute(0, 2, 1, 3).float().repeat_interleave(Hq // Hkv, 1)
        vf = self.v.permute(0, 2, 1, 3).float().repeat_interleave(Hq // Hkv, 1)
        s = qf @ kf.transpose(-1, -2) * attn.scale
        cap = float(getattr(attn, "softcap", 0.0) or 0.0)
        if cap:
            s = torch.tanh(s / cap) * cap
        i = torch.arange(Sk - S, Sk, device=q.device)[:, None]
        j = torch.arange(Sk, device=q.device)[None]
        vis = j <= i
        w = int(getattr(attn, "window", 0) or 0)
        if w:
            vis = vis & (i - j < w)           # sliding-window layer: only the last ``w`` keys
        c = int(getattr(attn, "chunk", 0) or 0)
        if c:
            vis = vis & (i // c == j // c)    # chunked layer: keys of the query's own chunk
        s = s.masked_fill(~vis[None, None], float("-inf"))
        sinks = getattr(attn, "sinks", None)
        if sinks is not None:             # one extra logit per head in the softmax denominator
            sink = sinks.float().view(1, -1, 1, 1).expand(s.shape[0], -1, s.shape[2], 1)
            o = torch.softmax(torch.cat([s, sink], -1), -1)[..., :-1] @ vf
            return o.permute(0, 2, 1, 3).reshape(B * S, Hq * D).to(qkv2d.dtype)
        o = torch.softmax(s, -1) @ vf
        return o.permute(0, 2, 1, 3).reshape(B * S, Hq * D).to(qkv2d.dtype)

    def reorder(self, idx):
        self.k, self.v = self.k.index_select(0, idx), self.v.index_select(0, idx)


def _process_logits(logits, generated, cfg: GenerationConfig):
    if cfg.repetition_penalty != 1.0 and generated.numel():
        score = logits.gather(1, generated)
        score = torch.where(score < 0, score * cfg.repetition_penalty, score / cfg.repetition_penalty)
        logits = logits.scatter(1, generated, score)
    if cfg.do_sample:
        if cfg.temperature != 1.0:
            logits = logits / max(cfg.temperature, 1e-5)
        if cfg.top_k > 0:
            kth = logits.topk(min(cfg.top_k, logits.shape[-1]), dim=-1)[0][:, -1:]
            logits = logits.masked_fill(logits < kth, float("-inf"))
        if cfg.top_p < 1.0:
            sl, si = logits.sort(dim=-1, descending=True)
            cp = torch.softmax(sl, -1).cumsum(-1)
            remove = cp - torch.softmax(sl, -1) > cfg.top_p
            sl = sl.masked_fill(remove, float("-inf"))
            logits = torch.full_like(logits, float("-inf")).scatter(1, si, sl)
    return logits


@torch.no_grad()
def generate(model, input_ids: torch.Tensor, generation_config: Optional[GenerationConfig] = None,
             streamer: Optional[Callable[[torch.Tensor], None]] = None, logits_processor=None, stopping_criteria=None,
             **kw) -> torch.Tensor:
    """Greedy / sampling / beam decoding with a KV cache. ``logits_processor`` (a ``LogitsProcessorList``) runs before the
    built-in repetition penalty and sampling warpers; ``stopping_criteria`` (a ``StoppingCriteriaList``) adds to the
    end-of-sequence and stop-token checks."""
    cfg = generation_config or GenerationConfig()
    for k, v in kw.items():
        setattr(cfg, k, v)
    if cfg.eos_token_id is None:
        cfg.eos_token_id = getattr(model.config, "eos_token_id", None)
    if cfg.num_beams > 1:
        return _beam_search(model, input_ids, cfg)
    stops = set(cfg.stop_token_ids) | ({cfg.eos_token_id} if cfg.eos_token_id is not None else set())
    layers = list(model.model.layer_range)
    use_cache = not model.config.is_mla and not getattr(model.config, "no_kv_cache", False)
    caches = {i: KVCache() for i in layers} if use_cache else None
    B = input_ids.shape[0]
    seq = input_ids
    done = torch.zeros(B, dtype=torch.bool, device=input_ids.device)
    cur, past = input_ids, 0
    for _ in range(cfg.max_new_tokens):
        pos = torch.arange(past, past + cur.shape[1], device=cur.device)[None].expand(B, -1)
        out = model(cur if use_cache else seq, position_ids=pos if use_cache else None, caches=caches, return_logits=True)
        logits = out.logits[:, -1].float()
        if logits_processor is not None:
            logits = logits_processor(seq, logits)
        logits = _process_logits(logits, seq, cfg)
        nxt = torch.multinomial(torch.softmax(logits, -1), 1) if cfg.do_sample else logits.argmax(-1, keepdim=True)
        if cfg.pad_token_id is not None:
            nxt = torch.where(done[:, None], torch.full_like(nxt, cfg.pad_token_id), nxt)
        seq = torch.cat([seq, nxt], 1)
        if streamer is not None:
            (streamer.put if hasattr(streamer, "put") else streamer)(nxt)
        for s in stops:
            done |= nxt[:, 0] == s
        if stopping_criteria is not None:
            done |= stopping_criteria(seq, logits)
        if bool(done.all()):
            break
        past += cur.shape[1]
        cur = nxt
    if streamer is not None and hasattr(streamer, "end"):
        streamer.end()
    return seq


def _beam_search(model, input_ids, cfg: GenerationConfig):
    """Beam search; with ``num_beam_groups`` > 1 the beams are split into groups that are advanced one after the other
    inside every step, and a token already chosen by an earlier group in that step costs ``diversity_penalty`` per use
    (Hamming diversity), so that the groups explore different continuations
    (paddleformers/generation/utils.py: ``group_beam_search``). ``num_return_sequences`` best hypotheses are returned per
    input, [B * num_return_sequences, L]."""
    B, nb = input_ids.shape[0], cfg.num_beams
    ng = max(int(getattr(cfg, "num_beam_groups", 1) or 1), 1)
    if nb % ng != 0:
        raise ValueError(f"num_beams {nb} must be a multiple of num_beam_groups {ng}")
    if ng > 1 and float(getattr(cfg, "diversity_penalty", 0.0) or 0.0) <= 0.0:
        raise ValueError("group beam search needs diversity_penalty > 0 (otherwise every group finds the same beams)")
    gs = nb // ng
    nret = max(int(getattr(cfg, "num_return_sequences", 1) or 1), 1)
    if nret > nb:
        raise ValueError("num_return_sequences must not exceed num_beams")
    dev = input_ids.device
    seq = input_ids.repeat_interleave(nb, 0)
    scores = torch.full((B, nb), -1e9, device=dev)
    scores[:, ::gs] = 0.0                           # one live beam per group at the start
    finished: List[List] = [[] for _ in range(B)]
    L0 = input_ids.shape[1]
    for step in range(cfg.max_new_tokens):
        out = model(seq, return_logits=True)
        lp_all = torch.log_softmax(out.logits[:, -1].float(), -1).view(B, nb, -1)
        V = lp_all.shape[-1]
        new_seq = [[None] * nb for _ in range(B)]
        new_scores = [[-1e9] * nb for _ in range(B)]
        chosen = torch.zeros(B, V, device=dev)       # tokens taken by earlier groups in this step
        for g in range(ng):
            lo = g * gs
            lp = lp_all[:, lo:lo + gs]
            if g > 0:
                lp = lp - cfg.diversity_penalty * chosen[:, None, :]
            cand = (scores[:, lo:lo + gs, None] + lp).reshape(B, gs * V)
            top, idx = cand.topk(2 * gs, dim=-1)
            beam, tok = idx // V, idx % V
            for b in range(B):
                keep = []
                for sc, bm, tk in zip(top[b].tolist(), beam[b].tolist(), tok[b].tolist()):
                    cand_seq = torch.cat([seq[b * nb + lo + bm], torch.tensor([tk], device=dev)])
                    if cfg.eos_token_id is not None and tk == cfg.eos_token_id:
                        finished[b].append((sc / ((cand_seq.numel() - L0) ** cfg.length_penalty), cand_seq))
                    else:
                        keep.append((sc, cand_seq))
                    if len(keep) == gs:
                        break
                while len(keep) < gs:
                    keep.append((-1e9, keep[-1][1] if keep else torch.cat([seq[b * nb + lo], seq.new_zeros(1)])))
                for i, (sc, cs) in enumerate(keep):
                    new_seq[b][lo + i], new_scores[b][lo + i] = cs, sc
                    if sc > -1e8:
                        chosen[b, cs[-1]] += 1
        seq = torch.stack([x for row in new_seq for x in row])
        scores = torch.tensor(new_scores, device=dev)
        if all(len(f) >= nb for f in finished):
            break
    outs = []
    for b in range(B):
        pool = finished[b] + [(scores[b, i].item() / max(seq.shape[1] - L0, 1) ** cfg.length_penalty, seq[b * nb + i])
                              for i in range(nb) if scores[b, i].item() > -1e8]
        pool.sort(key=lambda x: -x[0])
        uniq = []
        for sc, cs in pool:                           # groups may converge on one hypothesis: return distinct ones first
            if not any(cs.numel() == u.numel() and torch.equal(cs, u) for u in uniq):
                uniq.append(cs)
        uniq += [p[1] for p in pool]
        outs += uniq[:nret]
    n = max(o.numel() for o in outs)
    pad = cfg.pad_token_id if cfg.pad_token_id is not None else (cfg.eos_token_id or 0)
    return torch.stack([torch.cat([o, o.new_full((n - o.numel(),), pad)]) for o in outs])


class GenerationMixin:
    def generate(self, input_ids, generation_config=None, **kw):
        return generate(self, input_ids, generation_config, **kw)
