"""Grouped-query softmax attention over a window of the paged cache, with the options a design may switch on:

* ``value_dim``: a value's size need not be the key's;
* ``biases``: which of the projections q, k, v, o add a bias (``"q.b"`` ... in the part's tensors);
* ``qk_norm`` = ``"whole"``: an RMS norm with a weight over the whole query projection and over the whole key
  projection (all heads at once, before they are split into heads and before the rotation), eps ``qk_norm_eps``;
* ``position``: a rotary part; its ``rope_dim`` leading dimensions of every head are rotated, in either pairing;
* ``window``: a query sees itself and the ``window - 1`` positions before it (None: all earlier positions);
* ``sink``: the softmax's denominator also holds exp(sink_h), one learned number per query head that has no key and
  no value and is not scaled.

score(i, j) = q_i . k_j * ``scale``.  A *split mixer* (see :mod:`hfee_b200.parts.recurrent`): ``mix`` leaves the
concatenated heads, times ``out_scale``, for W_o, so it runs alone or as a branch of a parallel mixer.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.needs import PagedKV
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import build_part, register_part
from .recurrent import SplitMixer


class SoftmaxAttention(SplitMixer):
    """spec: ``width``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim``, ``scale``, ``window``, ``position``,
    ``biases`` (a tuple out of "q", "k", "v", "o"), ``qk_norm`` (None or "whole"), ``qk_norm_eps``, ``sink`` (bool)."""

    @property
    def graph_safe(self) -> bool:
        return bool(self.position.graph_safe)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        q, k, v = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim, spec.kv_heads * spec.value_dim
        rows = {"q": q, "k": k, "v": v, "o": spec.width}
        needs = {"q": TensorNeed((q, spec.width)), "k": TensorNeed((k, spec.width)), "v": TensorNeed((v, spec.width)),
                 "o": TensorNeed((spec.width, spec.heads * spec.value_dim))}
        for b in spec.get("biases") or ():
            if b not in rows:
                raise ValueError(f"softmax attention: no projection {b!r} to put a bias on")
            needs[b + ".b"] = TensorNeed((rows[b],), role="vector")
        if spec.get("qk_norm") == "whole":
            needs["q.norm"] = TensorNeed((q,), role="scale")
            needs["k.norm"] = TensorNeed((k,), role="scale")
        elif spec.get("qk_norm") is not None:
            raise ValueError(f"softmax attention: unknown qk_norm {spec.get('qk_norm')!r} (known: 'whole')")
        if spec.get("sink"):
            needs["sink"] = TensorNeed((spec.heads,), role="vector")
        return needs

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.heads, self.kv_heads = int(spec.heads), int(spec.kv_heads)
        self.head_dim, self.value_dim = int(spec.head_dim), int(spec.value_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} must be a multiple of kv_heads {self.kv_heads}")
        self.scale = float(spec.scale)
        self.window = spec.get("window")
        if self.window is not None and int(self.window) < 1:
            raise ValueError(f"a window holds at least the token itself, got {self.window}")
        self.position = build_part("position", spec.position, {}, rt)
        self.q_cols, self.k_cols = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.v_cols = self.kv_heads * self.value_dim
        self.in_weight = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        self.biases = tuple(tensors.get(b + ".b") for b in ("q", "k", "v"))
        self.out_bias = tensors.get("o.b")
        self.norm_weights = (tensors.get("q.norm"), tensors.get("k.norm"))
        self.norm_eps = float(spec.get("qk_norm_eps") or 0.0)
        self.sink = tensors.get("sink")
        self.w_o = tensors["o"]
        self.inner_cols, self.in_rows = self.heads * self.value_dim, self.q_cols + self.k_cols + self.v_cols
        # partial results of a decode step whose keys are split among CTAs (tensor-core kernel only)
        tile = ops.distance_attention_tile(self.head_dim, self.value_dim) if rt.dtype == torch.bfloat16 else 0
        self.split_scratch = rt.scratch("attn_partials", (rt.max_requests * self.heads * ops.MAX_SPLITS * (tile + 2),),
                                        torch.float32) if tile else None

    def cache_need(self) -> PagedKV:
        return PagedKV(self.kv_heads, self.head_dim, None if self.window is None else int(self.window), None, self.value_dim)

    def mix(self, proj, step, cache, writes_cache, into, out_scale: float = 1.0) -> None:
        rt, n = self.rt, step.n
        cs = self.position.table(step)
        q = rt.scratch("attn_q", (rt.max_tokens, self.q_cols))[:n]
        ops.tag("rope")
        ops.attention_prepare(proj, 0, self.q_cols, self.q_cols + self.k_cols, self.heads, self.kv_heads, self.head_dim,
                              self.value_dim, step, q, cache.k if writes_cache else None, cache.v if writes_cache else None,
                              cache.block_table, cache.page_size, cs, self.position.rope_dim, self.position.interleaved,
                              self.biases, self.norm_weights, self.norm_eps)
        ops.tag("attention")
        ops.softmax_attention(q, cache.k, cache.v, cache.block_table, cache.page_size, step, into, self.heads, self.kv_heads,
                              self.head_dim, self.value_dim, self.scale, int(self.window or 0), self.sink, out_scale,
                              self.split_scratch)


register_part("mixer", "softmax_attention", SoftmaxAttention)
