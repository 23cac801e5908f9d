"""Layer factories with tensor-parallel plans: ``Linear.create(in, out, tp_plan="colwise" | "rowwise" | None)``,
``Embedding.create``, ``Norm.create``, ``MLP``, ``LMHead`` (paddleformers/nn/linear.py:29-93, nn/embedding.py:24-29,
nn/norm.py:54-83, nn/mlp.py:113-130, nn/lm_head.py:27-99). They return the modules the unified decoder is built from,
so user-defined models get the fused kernels, the fused collectives and the sharding annotations by construction."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding
from ..parallel.topology import get_parallel_state
from .general import GeneralInterface


class Linear(GeneralInterface):
    @classmethod
    def create(cls, in_features: int, out_features: int, has_bias: bool = False, tp_plan: Optional[str] = None,
               sequence_parallel: bool = False, sections: Optional[List[int]] = None, epilogue: Optional[str] = None,
               dtype=None, device=None) -> nn.Module:
        """``tp_plan``: "colwise" (split the output features), "rowwise" (split the input features) or None (replicated).
        With tensor-parallel degree 1 every plan degenerates to a plain linear layer."""
        tp = get_parallel_state().degrees.mp
        key = "default" if (tp == 1 or tp_plan is None) else tp_plan
        return cls.get(key)(in_features, out_features, has_bias, sequence_parallel, sections, epilogue, dtype, device)


Linear.register("default", lambda i, o, b, sp, sec, epi, dt, dev: nn.Linear(i, o, bias=b, dtype=dt, device=dev))
Linear.register("colwise", lambda i, o, b, sp, sec, epi, dt, dev: ColumnParallelLinear(i, o, bias=b, sections=sec, sequence_parallel=sp,
                                                                                       epilogue=epi, dtype=dt, device=dev))
Linear.register("rowwise", lambda i, o, b, sp, sec, epi, dt, dev: RowParallelLinear(i, o, bias=b, sequence_parallel=sp, dtype=dt, device=dev))


class Embedding(GeneralInterface):
    @classmethod
    def create(cls, num_embeddings: int, embedding_dim: int, sequence_parallel: bool = False, dtype=None, device=None) -> nn.Module:
        if get_parallel_state().degrees.mp > 1:
            return VocabParallelEmbedding(num_embeddings, embedding_dim, sequence_parallel, dtype=dtype, device=device)
        return nn.Embedding(num_embeddings, embedding_dim, dtype=dtype, device=device)


class Norm(GeneralInterface):
    @classmethod
    def create(cls, hidden_size: int, eps: float = 1e-6, norm_type: str = "rms_norm", sequence_parallel: bool = False, dtype=None,
               device=None) -> nn.Module:
        return cls.get(norm_type)(hidden_size, eps, sequence_parallel, dtype, device)


def _rms(hidden, eps, sp, dtype, device):
    from ..models.modeling import RMSNorm

    return RMSNorm(hidden, eps, sp, dtype=dtype, device=device)


Norm.register("rms_norm", _rms)
Norm.register("layer_norm", lambda h, eps, sp, dt, dev: nn.LayerNorm(h, eps=eps, dtype=dt, device=dev))


class MLP(GeneralInterface):
    """SwiGLU MLP with the fused gate|up projection (and the SwiGLU GEMM epilogue on the GPU)."""

    @classmethod
    def create(cls, config, hidden_size: Optional[int] = None, intermediate_size: Optional[int] = None, has_bias: bool = False,
               dtype=None, device=None) -> nn.Module:
        from .moe import DenseMLP

        return DenseMLP(hidden_size or config.hidden_size, intermediate_size or config.intermediate_size, config, bias=has_bias,
                        dtype=dtype, device=device)


class LMHead(GeneralInterface):
    """Vocabulary projection; under tensor parallelism the weight is split along the vocabulary and meant to be used with
    the vocabulary-parallel fused loss (``parallel.vocab_parallel_loss``), which never materialises full logits."""

    @classmethod
    def create(cls, config, sequence_parallel: bool = False, dtype=None, device=None) -> nn.Module:
        if get_parallel_state().degrees.mp > 1:
            return ColumnParallelLinear(config.hidden_size, config.vocab_size, bias=False, sequence_parallel=sequence_parallel,
                                        dtype=dtype, device=device)
        return nn.Linear(config.hidden_size, config.vocab_size, bias=False, dtype=dtype, device=device)
