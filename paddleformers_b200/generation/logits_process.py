"""Logits processors, stopping criteria and streamers for ``generate`` (the composable pieces of
paddleformers/generation/logits_process.py, stopping_criteria.py and streamers.py). Every processor maps
(input_ids [B, L], scores [B, V]) -> scores; every criterion maps (input_ids, scores) -> bool tensor [B]."""
from __future__ import annotations

import queue
from typing import Iterable, List, Optional, Sequence

import torch


class LogitsProcessor:
    def __call__(self, input_ids: torch.Tensor, scores: torch.Tensor) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError


class LogitsProcessorList(list):
    def __call__(self, input_ids, scores):
        for p in self:
            scores = p(input_ids, scores)
        return scores


class MinLengthLogitsProcessor(LogitsProcessor):
    """Forbid the end-of-sequence tokens until the sequence holds ``min_length`` tokens."""

    def __init__(self, min_length: int, eos_token_id):
        self.min_length = min_length
        self.eos = [eos_token_id] if isinstance(eos_token_id, int) else list(eos_token_id)

    def __call__(self, input_ids, scores):
        if input_ids.shape[1] < self.min_length:
            scores = scores.clone()
            scores[:, self.eos] = float("-inf")
        return scores


class RepetitionPenaltyLogitsProcessor(LogitsProcessor):
    def __init__(self, penalty: float):
        self.penalty = penalty

    def __call__(self, input_ids, scores):
        s = scores.gather(1, input_ids)
        s = torch.where(s < 0, s * self.penalty, s / self.penalty)
        return scores.scatter(1, input_ids, s)


class NoRepeatNGramLogitsProcessor(LogitsProcessor):
    """Ban every token that would complete an n-gram already present in the sequence."""

    def __init__(self, ngram_size: int):
        assert ngram_size > 0
        self.n = ngram_size

    def __call__(self, input_ids, scores):
        n = self.n
        if input_ids.shape[1] + 1 < n:
            return scores
        scores = scores.clone()
        for b, row in enumerate(input_ids.tolist()):
            prefix = tuple(row[len(row) - n + 1:]) if n > 1 else ()
            banned = [row[i + n - 1] for i in range(len(row) - n + 1) if tuple(row[i:i + n - 1]) == prefix]
            if banned:
                scores[b, banned] = float("-inf")
        return scores


class TemperatureLogitsWarper(LogitsProcessor):
    def __init__(self, temperature: float):
        self.t = max(float(temperature), 1e-5)

    def __call__(self, input_ids, scores):
        return scores / self.t


class TopKLogitsWarper(LogitsProcessor):
    def __init__(self, top_k: int, min_tokens_to_keep: int = 1):
        self.k = max(top_k, min_tokens_to_keep)

    def __call__(self, input_ids, scores):
        kth = scores.topk(min(self.k, scores.shape[-1]), dim=-1)[0][:, -1:]
        return scores.masked_fill(scores < kth, float("-inf"))


class TopPLogitsWarper(LogitsProcessor):
    def __init__(self, top_p: float, min_tokens_to_keep: int = 1):
        self.p, self.keep = top_p, min_tokens_to_keep

    def __call__(self, input_ids, scores):
        sl, si = scores.sort(dim=-1, descending=True)
        probs = torch.softmax(sl, -1)
        remove = probs.cumsum(-1) - probs > self.p
        remove[:, :self.keep] = False
        sl = sl.masked_fill(remove, float("-inf"))
        return torch.full_like(scores, float("-inf")).scatter(1, si, sl)


class ForcedEOSTokenLogitsProcessor(LogitsProcessor):
    """At the last allowed position only the end-of-sequence token is possible."""

    def __init__(self, max_length: int, eos_token_id: int):
        self.max_length, self.eos = max_length, eos_token_id

    def __call__(self, input_ids, scores):
        if input_ids.shape[1] == self.max_length - 1:
            forced = torch.full_like(scores, float("-inf"))
            forced[:, self.eos] = 0.0
            return forced
        return scores


class SuppressTokensLogitsProcessor(LogitsProcessor):
    def __init__(self, tokens: Iterable[int]):
        self.tokens = list(tokens)

    def __call__(self, input_ids, scores):
        scores = scores.clone()
        scores[:, self.tokens] = float("-inf")
        return scores


# ---------------------------------------------------------------------------------------------------------------
class StoppingCriteria:
    def __call__(self, input_ids: torch.Tensor, scores: Optional[torch.Tensor] = None) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class StoppingCriteriaList(list):
    def __call__(self, input_ids, scores=None):
        done = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
        for c in self:
            done |= c(input_ids, scores)
        return done


class MaxLengthCriteria(StoppingCriteria):
    def __init__(self, max_length: int):
        self.max_length = max_length

    def __call__(self, input_ids, scores=None):
        return torch.full((input_ids.shape[0],), input_ids.shape[1] >= self.max_length, dtype=torch.bool, device=input_ids.device)


class EosTokenCriteria(StoppingCriteria):
    def __init__(self, eos_token_id):
        self.eos = [eos_token_id] if isinstance(eos_token_id, int) else list(eos_token_id)

    def __call__(self, input_ids, scores=None):
        last = input_ids[:, -1]
        return torch.isin(last, torch.tensor(self.eos, device=input_ids.device))


class StopSequenceCriteria(StoppingCriteria):
    """Stop a row once it ends with any of the given token sequences (stop words tokenised by the caller)."""

    def __init__(self, sequences: Sequence[Sequence[int]]):
        self.sequences = [list(s) for s in sequences if len(s)]

    def __call__(self, input_ids, scores=None):
        done = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
        for s in self.sequences:
            if input_ids.shape[1] >= len(s):
                tail = input_ids[:, -len(s):]
                done |= (tail == torch.tensor(s, device=input_ids.device)[None]).all(-1)
        return done


# ---------------------------------------------------------------------------------------------------------------
class TextStreamer:
    """Decodes tokens of the first sequence as they arrive and hands complete text pieces to ``on_text``."""

    def __init__(self, tokenizer, skip_prompt: bool = True, on_text=None, **decode_kwargs):
        self.tok, self.skip_prompt, self.kw = tokenizer, skip_prompt, decode_kwargs
        self.on_text = on_text or (lambda s, end=False: print(s, end="" if not end else "\n", flush=True))
        self.ids: List[int] = []
        self.printed = 0

    def put(self, tokens: torch.Tensor):
        self.ids.extend(tokens.reshape(tokens.shape[0], -1)[0].tolist())
        text = self.tok.decode(self.ids, **self.kw)
        # hold back a trailing partial character / word piece
        if text.endswith("\n") or (text and not text.endswith("�")):
            new = text[self.printed:]
            if new:
                self.on_text(new)
                self.printed = len(text)

    __call__ = put

    def end(self):
        text = self.tok.decode(self.ids, **self.kw)
        self.on_text(text[self.printed:], end=True)
        self.ids, self.printed = [], 0


class TextIteratorStreamer(TextStreamer):
    """Iterator flavour: ``for piece in streamer`` from another thread while ``generate`` runs."""

    def __init__(self, tokenizer, timeout: Optional[float] = None, **kw):
        self.q: "queue.Queue" = queue.Queue()
        self.timeout = timeout
        super().__init__(tokenizer, on_text=self._push, **kw)

    def _push(self, s, end=False):
        if s:
            self.q.put(s)
        if end:
            self.q.put(None)

    def __iter__(self):
        return self

    def __next__(self):
        v = self.q.get(timeout=self.timeout)
        if v is None:
            raise StopIteration
        return v
