"""Optimizer variants over the flat sharded buffers of ``ShardedAdamW``.

* ``AdamWCustom`` - AdamW with the options of the reference's custom optimizer (paddleformers/utils/optimizer.py:268):
  moments kept in bf16 (``moment_dtype``), moments kept in host memory and streamed through the device in chunks
  (``offload_moments``), and an update whose floating-point operation order is that of ``torch.optim.AdamW``, so that a
  single-process run reproduces a Hugging Face / PyTorch run bit for bit (``hf_bitexact``; the reference's
  ``_hf_bitexact_adamw_step`` :54 and ``HFBitexactClipGradByGlobalNorm``, paddleformers/utils/hf_bitexact_clip.py).
* ``AdamWMini`` - one second-moment value per block instead of one per element (a row of a matrix, a whole vector), as in
  the reference's ``AdamWMini`` (paddleformers/utils/optimizer.py): the second-moment memory shrinks by the row length.

Both reuse the gradient reduction (reduce-scatter in the sharding group, all-reduce over data parallel), the MoE-aware
global-norm clipping and the parameter all-gather of the base class; only the per-shard update differs. These updates are
written with tensor operations, not with the fused AdamW kernel, and read the skip flag on the host once per step.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

from ..parallel.sharding import ShardedAdamW, _Domain


class AdamWCustom(ShardedAdamW):
    custom_update = True

    def __init__(self, *args, moment_dtype: torch.dtype = torch.float32, offload_moments: bool = False,
                 offload_chunk_numel: int = 1 << 26, hf_bitexact: bool = False, **kw):
        self.moment_dtype = moment_dtype
        self.offload_moments = bool(offload_moments)
        self.offload_chunk_numel = int(offload_chunk_numel)
        self.hf_bitexact = bool(hf_bitexact)
        super().__init__(*args, **kw)
        if self.hf_bitexact and any(d.shard_size > 1 for d in self.domains):
            raise ValueError("hf_bitexact reproduces a single-process run: optimizer sharding must be off")

    def _build_domain(self, dom: _Domain, dtype):
        super()._build_domain(dom, dtype)
        for k in ("exp_avg", "exp_avg_sq"):
            t = getattr(dom, k).to(self.moment_dtype)
            if self.offload_moments:
                t = t.cpu()
                if torch.cuda.is_available():
                    t = t.pin_memory()
            setattr(dom, k, t)

    # ------------------------------------------------------------------ clipping in torch's operation order
    def _global_grad_norm(self, shards) -> torch.Tensor:
        if not self.hf_bitexact:
            return super()._global_grad_norm(shards)
        # torch.nn.utils.clip_grad_norm_: 2-norm of the per-parameter 2-norms, parameters in model order
        order = {id(p): i for i, p in enumerate(self.model.parameters())}
        grads = sorted(((order[id(p)], p.main_grad) for dom in self.domains for _, p in dom.params), key=lambda x: x[0])
        norms = [torch.linalg.vector_norm(g, 2.0) for _, g in grads]
        return torch.linalg.vector_norm(torch.stack(norms), 2.0)

    # ------------------------------------------------------------------ update
    def _chunks(self, n: int):
        step = self.offload_chunk_numel if self.offload_moments else n
        for lo in range(0, n, max(step, 1)):
            yield lo, min(lo + step, n)

    def _update(self, dom, g, pslice, sc):
        if float(sc[4]) != 0.0:          # non-finite gradient norm: leave weights and moments alone
            return
        b1, b2 = self.betas
        lr = float(self.lr)
        bc1, bc2 = 1.0 - b1 ** self.step_count, 1.0 - b2 ** self.step_count
        dev = dom.master.device
        clip = sc[1]
        for lo, hi in self._chunks(dom.master.numel()):
            m_store, v_store = dom.exp_avg[lo:hi], dom.exp_avg_sq[lo:hi]
            m = m_store.to(dev, torch.float32, non_blocking=True)
            v = v_store.to(dev, torch.float32, non_blocking=True)
            if m.data_ptr() == m_store.data_ptr():           # fp32 moments on the compute device: update in place
                m, v = m_store, v_store
            w = dom.master[lo:hi]
            gr = g[lo:hi] * clip if (self.max_grad_norm and self.max_grad_norm > 0) else g[lo:hi]
            if self.hf_bitexact:
                # operation order of torch.optim.AdamW (single tensor, foreach off): decay, lerp, addcmul, sqrt / sqrt(bc2) + eps
                w.mul_(1.0 - lr * dom.weight_decay)
                m.lerp_(gr, 1.0 - b1)
                v.mul_(b2).addcmul_(gr, gr, value=1.0 - b2)
                denom = (v.sqrt() / math.sqrt(bc2)).add_(self.eps)
                w.addcdiv_(m, denom, value=-(lr / bc1))
            else:
                m.mul_(b1).add_(gr, alpha=1.0 - b1)
                v.mul_(b2).addcmul_(gr, gr, value=1.0 - b2)
                w.mul_(1.0 - lr * dom.weight_decay)
                w.addcdiv_(m / bc1, (v / bc2).sqrt_().add_(self.eps), value=-lr)
            if m is not m_store:
                m_store.copy_(m.to(m_store.dtype), non_blocking=True)
                v_store.copy_(v.to(v_store.dtype), non_blocking=True)
        if self.offload_moments and dev.type == "cuda":
            torch.cuda.current_stream(dev).synchronize()     # the host copies must land before the next step reads them
        pslice.copy_(dom.master)

    def load_state_dict(self, sd) -> None:
        for dom in self.domains:                             # the base class copies into the moment tensors: dtypes convert
            s = sd["domains"][dom.name]
            s["exp_avg"], s["exp_avg_sq"] = s["exp_avg"].to(dom.exp_avg.dtype), s["exp_avg_sq"].to(dom.exp_avg_sq.dtype)
        super().load_state_dict(sd)

    def memory_bytes(self) -> int:
        n = 0
        for dom in self.domains:
            for t in (dom.master, dom.exp_avg, dom.exp_avg_sq, dom.flat_grad, dom.flat_param):
                if t.device.type != "cpu" or not self.offload_moments or t is dom.master:
                    n += t.numel() * t.element_size()
        return n


class AdamWMini(ShardedAdamW):
    """AdamW whose second moment is one value per block: mean(g^2) over a row of a matrix (the fan-in of one output unit; for
    stacked expert weights a row of one expert's matrix) or over a whole vector. First moments stay per element. A row that
    a shard boundary cuts is treated as two blocks, one on either side; a checkpoint therefore resumes only with the
    sharding degree it was written with."""

    custom_update = True

    def _build_domain(self, dom: _Domain, dtype):
        super()._build_domain(dom, dtype)
        n = dom.shard_numel
        lo = dom.shard_rank * n
        starts: List[int] = []
        for name, p in dom.params:                       # block boundaries inside this rank's slice, in flat order
            off, cnt = dom.offsets[name]
            row = p.shape[-1] if p.dim() >= 2 else cnt
            a, b = max(off, lo), min(off + cnt, lo + n)
            if b <= a:
                continue
            first = off + (a - off) // row * row
            pts = list(range(first, b, row))
            pts[0] = a
            if b == off + cnt and b < lo + n:
                pts.append(b)                            # alignment padding after the parameter is a block of its own
            starts.extend(x - lo for x in pts)
        if not starts or starts[0] != 0:
            starts.insert(0, 0)                          # leading padding (cannot happen) or an empty slice
        dev = dom.master.device
        st = torch.tensor(sorted(set(starts)), dtype=torch.int64, device=dev)
        ends = torch.cat([st[1:], torch.tensor([n], dtype=torch.int64, device=dev)])
        dom.block_len = (ends - st)
        dom.block_id = torch.repeat_interleave(torch.arange(st.numel(), device=dev), dom.block_len)   # [shard numel]
        dom.exp_avg_sq = torch.zeros(st.numel(), dtype=torch.float32, device=dev)

    def _update(self, dom, g, pslice, sc):
        if float(sc[4]) != 0.0:
            return
        b1, b2 = self.betas
        lr = float(self.lr)
        bc1, bc2 = 1.0 - b1 ** self.step_count, 1.0 - b2 ** self.step_count
        gr = g * sc[1] if (self.max_grad_norm and self.max_grad_norm > 0) else g
        dom.exp_avg.mul_(b1).add_(gr, alpha=1.0 - b1)
        sq = torch.zeros_like(dom.exp_avg_sq).index_add_(0, dom.block_id, gr * gr) / dom.block_len.to(torch.float32)
        dom.exp_avg_sq.mul_(b2).add_(sq, alpha=1.0 - b2)
        denom = (dom.exp_avg_sq / bc2).sqrt_().add_(self.eps)
        dom.master.mul_(1.0 - lr * dom.weight_decay)
        dom.master.addcdiv_(dom.exp_avg / bc1, denom[dom.block_id], value=-lr)
        pslice.copy_(dom.master)

    def second_moment_numel(self) -> int:
        return sum(int(d.exp_avg_sq.numel()) for d in self.domains)
