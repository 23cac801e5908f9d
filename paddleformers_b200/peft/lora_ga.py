"""LoRA-GA: initialise the adapters from the gradient of the full weights, so that the first adapter steps follow the
direction full fine-tuning would take.

Procedure (paddleformers/peft/lora/loraga_utils.py:36-320): estimate dL/dW of every adapted linear layer on a few batches
(averaged over batches and data-parallel ranks, gathered over tensor-parallel ranks), take a truncated SVD
G = U S V^T, set B to the first r left singular vectors and A to singular vectors r .. 2r of the input side, both scaled by
in_features^(1/4) / sqrt(stable_gamma) (or by 1 / scaling when ``stable_gamma`` is -1), and subtract scaling * B A from the
frozen weight so that the model's function is unchanged at step 0. Weights here are [out, in], so G is [out, in], U spans
outputs and V inputs.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional

import torch
import torch.distributed as dist

from ..transformers.model_utils import param_shard_spec
from .lora import LoRALinear, LoRAModel


def estimate_gradients(model: LoRAModel, batches: Iterable[dict], loss_fn: Optional[Callable] = None,
                       dp_group=None) -> Dict[str, torch.Tensor]:
    """Mean gradient of the frozen base weight of every ``LoRALinear`` over ``batches`` (fp32, this rank's shard). The
    adapters are switched off meanwhile, so the gradient is that of the unmodified model. ``loss_fn(model, batch)``
    defaults to ``model(**batch).loss``."""
    layers = {n: m for n, m in model.named_modules() if isinstance(m, LoRALinear)}
    saved = {}
    for n, m in layers.items():
        w = m.base.weight
        saved[n] = (w.requires_grad, m.disabled, w.grad, getattr(w, "main_grad", None))
        w.requires_grad_(True)
        w.grad = None
        if hasattr(w, "main_grad"):
            del w.main_grad                      # gradients must come back through autograd, not an accumulation buffer
        m.disabled = True
    was_training = model.training
    model.train()
    acc = {n: torch.zeros_like(m.base.weight, dtype=torch.float32) for n, m in layers.items()}
    count = 0
    try:
        for batch in batches:
            loss = loss_fn(model, batch) if loss_fn is not None else model(**batch).loss
            loss.backward()
            for n, m in layers.items():
                if m.base.weight.grad is not None:
                    acc[n] += m.base.weight.grad.float()
                    m.base.weight.grad = None
            for p in model.parameters():
                p.grad = None
            count += 1
    finally:
        for n, m in layers.items():
            req, dis, grad, mg = saved[n]
            m.base.weight.requires_grad_(req)
            m.base.weight.grad = grad
            if mg is not None:
                m.base.weight.main_grad = mg
            m.disabled = dis
        model.train(was_training)
    world = dist.get_world_size(dp_group) if (dist.is_initialized() and dp_group is not None) else 1
    for n in acc:
        acc[n] /= max(count, 1)
        if world > 1:
            dist.all_reduce(acc[n], group=dp_group)
            acc[n] /= world
    return acc


def _full_matrix(layer: LoRALinear, shard: torch.Tensor) -> torch.Tensor:
    tp = int(getattr(layer.base, "tp", 1) or 1)
    if tp <= 1:
        return shard
    parts = [torch.empty_like(shard) for _ in range(tp)]
    dist.all_gather(parts, shard.contiguous(), group=layer.base.group)
    return param_shard_spec(layer.base.weight).unshard(parts, tp)


def _my_shard(p: torch.Tensor, full: torch.Tensor, layer: LoRALinear) -> torch.Tensor:
    tp = int(getattr(layer.base, "tp", 1) or 1)
    if tp <= 1 or getattr(p, "shard_spec", None) is None:
        return full
    return param_shard_spec(p).shard(full, dist.get_rank(layer.base.group), tp)


@torch.no_grad()
def lora_ga_reinit(model: LoRAModel, grads: Dict[str, torch.Tensor], stable_gamma: float = 16.0, niter: int = 4) -> Dict[str, torch.Tensor]:
    """Re-initialise every adapter from its layer's gradient and fold the initial product out of the base weight. Returns
    the new adapter tensors by parameter name (the reference keeps them to rebuild the shifted base weights on resume)."""
    out = {}
    for name, layer in model.named_modules():
        if not isinstance(layer, LoRALinear) or name not in grads:
            continue
        r = layer.cfg.r
        G = _full_matrix(layer, grads[name].float())
        n_out, n_in = G.shape
        q = min(4 * r, n_out, n_in)
        if q < 2 * r:
            raise ValueError(f"{name}: LoRA-GA needs min(out, in) >= 2 r (got {n_out} x {n_in}, r = {r})")
        gen_state = torch.random.get_rng_state()
        torch.manual_seed(0)                      # the randomised range finder must give every rank the same factors
        try:
            U, S, V = torch.svd_lowrank(G, q=q, niter=niter)
        finally:
            torch.random.set_rng_state(gen_state)
        B = U[:, :r].contiguous()                 # [out, r]
        A = V[:, r:2 * r].t().contiguous()        # [r, in]
        if stable_gamma != -1:
            s = n_in ** 0.25 / float(stable_gamma) ** 0.5
            A, B = A * s, B * s
        else:
            A, B = A / layer.scaling, B / layer.scaling
        A_loc = _my_shard(layer.lora_A, A.to(G.device), layer).to(layer.lora_A.dtype)
        B_loc = _my_shard(layer.lora_B, B.to(G.device), layer).to(layer.lora_B.dtype)
        layer.lora_A.copy_(A_loc)
        layer.lora_B.copy_(B_loc)
        # subtract the product of the adapters as stored (after rounding to their dtype), cut like the base weight
        delta = (B.to(layer.lora_B.dtype).float() @ A.to(layer.lora_A.dtype).float()) * layer.scaling
        w = layer.base.weight
        w.sub_(_my_shard(w, delta, layer).to(w.dtype))
        out[name + ".lora_A"], out[name + ".lora_B"] = A_loc.clone(), B_loc.clone()
    model.loraga_init_dict = out
    return out


def lora_ga_init(model: LoRAModel, batches: Iterable[dict], stable_gamma: float = 16.0, loss_fn: Optional[Callable] = None,
                 dp_group=None) -> Dict[str, torch.Tensor]:
    """``estimate_gradients`` followed by ``lora_ga_reinit``."""
    return lora_ga_reinit(model, estimate_gradients(model, batches, loss_fn, dp_group), stable_gamma)
