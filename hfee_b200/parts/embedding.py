"""Token embedding and the output head."""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Part, register_part


class TokenEmbedding(Part):
    """``x[i,:] = table[token_i,:] * scale`` (hostfog/hfee internal/llm/forward.go:75-77 has no scale).
    spec: ``vocab``, ``width``, ``scale`` (default 1), ``sinusoid_base`` (default None; a base b adds the token's
    position p as ``sin(p * b^(-2i/width))`` to entry 2i and the cosine of the same angle to entry 2i + 1)."""
    category = "embedding"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"table": TensorNeed((spec.vocab, spec.width), role="table")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.table = tensors["table"]
        self.scale = float(spec.get("scale", 1.0))
        base = spec.get("sinusoid_base")
        self.sinusoid_base = None if base is None else float(base)

    def forward(self, step: Any, residual: torch.Tensor) -> None:
        ops.tag("embed")
        ops.embed(self.table, step.token_ids, residual, step.slot_of_token, getattr(step, "feedback", None),
                  scale=self.scale)
        if self.sinusoid_base is not None:
            ops.add_sinusoid(residual, step.positions, self.sinusoid_base)


class BigramTokenEmbedding(Part):
    """``x[i,:] = table[token_i,:] + pairs[r_i,:]`` with ``r_i = (previous token * mul_prev + token_i * mul_cur) mod buckets``
    and, for a request's first token, ``r_i = buckets`` (the last row of ``pairs`` [buckets + 1, width]).
    spec: ``vocab``, ``width``, ``buckets``, ``mul_prev``, ``mul_cur``.  The previous token of a portion's first token
    belongs to the request: one int32 per request slot, which the model asks of the cache manager
    (:meth:`cache_need`) and hands to ``forward`` as ``cache.state``."""
    category = "embedding"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"table": TensorNeed((spec.vocab, spec.width), role="table"),
                "pairs": TensorNeed((spec.buckets + 1, spec.width), role="table")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.table, self.pairs = tensors["table"], tensors["pairs"]
        self.buckets, self.mul_prev, self.mul_cur = int(spec.buckets), int(spec.mul_prev), int(spec.mul_cur)
        if self.buckets < 1 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError(f"bigram embedding: buckets {self.buckets} must be positive and the multipliers non-negative")

    def cache_need(self):
        from ..cache.needs import FixedState
        return FixedState((1,), "int32")

    def forward(self, step: Any, residual: torch.Tensor, cache: Any = None) -> None:
        if cache is None or cache.state is None:
            raise ValueError("the bigram embedding needs its per-request state (the request's last token)")
        ops.tag("embed")
        ops.embed_bigram(self.table, self.pairs, step, cache.state, residual, self.buckets, self.mul_prev, self.mul_cur)


class LinearHead(Part):
    """``logits = x . W^T * scale`` in float32 (internal/llm/forward.go:132-141).  spec: ``vocab``,
    ``width``, ``tied`` (use the embedding table as W, internal/llm/model.go:118-121), ``scale``
    (default 1: no scaling pass), ``softcap`` (default None; a cap c turns the logits into ``c * tanh(logits / c)``)."""
    category = "head"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        # tied: the checkpoint need not hold a head; if it does, that tensor is used, as the
        # reference uses output.weight whenever the file has one (internal/llm/model.go:118-121)
        return {"weight": TensorNeed((spec.vocab, spec.width), optional=bool(spec.get("tied", False)))}

    def __init__(self, spec, tensors, rt, embedding: TokenEmbedding = None):
        super().__init__(spec, tensors, rt)
        if "weight" in tensors:
            self.weight = tensors["weight"]
        elif spec.get("tied", False):
            if embedding is None:
                raise ValueError("a tied head needs the embedding part")
            self.weight = embedding.table
        else:
            raise ValueError("the head has no weight and is not tied to the embedding")
        self.scale = float(spec.get("scale", 1.0))
        cap = spec.get("softcap")
        self.softcap = None if cap is None else float(cap)

    accepts_lazy_input = True        # the final norm may be fused into the product

    def forward(self, xn, logits: torch.Tensor) -> None:
        if isinstance(xn, torch.Tensor):
            ops.tag("head")
            ops.linear(xn, self.weight, logits)
        else:
            ops.tag("head")
            ops.linear_normed(xn, self.weight, logits)
        if self.scale != 1.0:
            ops.scale_(logits, self.scale)
        if self.softcap is not None:
            ops.softcap_(logits, self.softcap)


register_part("embedding", "token", TokenEmbedding)
register_part("embedding", "token_bigram", BigramTokenEmbedding)
register_part("head", "linear", LinearHead)
