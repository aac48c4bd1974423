"""Grouped-query softmax attention without a rotation, whose scores lose a logarithmic penalty on distance:

    score(i, j) = q_i . k_j * scale - r1_h * ln(1 + r2_h * (i - j))        (j <= i; r1, r2 per query head)

Key and value sizes are independent; keys and values are cached as they leave their projections.  A *split mixer*
(see :mod:`hfee_b200.parts.recurrent`): ``mix`` leaves the concatenated heads, times ``out_scale``, for W_o.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.needs import PagedKV
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import register_part
from .recurrent import SplitMixer


class DistanceAttention(SplitMixer):
    """spec: ``width``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim``, ``scale``, ``window`` (optional)."""

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        q, k, v = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim, spec.kv_heads * spec.value_dim
        return {"q": TensorNeed((q, spec.width)), "k": TensorNeed((k, spec.width)), "v": TensorNeed((v, spec.width)),
                "o": TensorNeed((spec.width, spec.heads * spec.value_dim)),
                "r1": TensorNeed((spec.heads,), role="positive"), "r2": TensorNeed((spec.heads,), role="positive")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.heads, self.kv_heads = int(spec.heads), int(spec.kv_heads)
        self.head_dim, self.value_dim = int(spec.head_dim), int(spec.value_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} must be a multiple of kv_heads {self.kv_heads}")
        self.scale = float(spec.scale)
        self.window = spec.get("window")
        self.q_cols, self.k_cols = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.v_cols = self.kv_heads * self.value_dim
        self.in_weight = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        self.r1, self.r2 = tensors["r1"], tensors["r2"]
        self.w_o = tensors["o"]
        self.inner_cols, self.in_rows = self.heads * self.value_dim, self.q_cols + self.k_cols + self.v_cols
        # partial results of a decode step whose keys are split among CTAs (tensor-core kernel only)
        tile = ops.distance_attention_tile(self.head_dim, self.value_dim) if rt.dtype == torch.bfloat16 else 0
        self.split_scratch = rt.scratch("attn_partials", (rt.max_requests * self.heads * ops.MAX_SPLITS * (tile + 2),),
                                        torch.float32) if tile else None

    def cache_need(self) -> PagedKV:
        return PagedKV(self.kv_heads, self.head_dim, self.window, None, self.value_dim)

    def mix(self, proj, step, cache, writes_cache, into, out_scale: float = 1.0) -> None:
        d, vd = self.head_dim, self.value_dim
        if writes_cache:
            ops.tag("rope")
            ops.rope_norm_cache(proj, None, 0, None, step.positions, step.slot_of_token, cache.block_table, cache.page_size,
                                k=(self.kv_heads, self.q_cols, d, d, 0, cache.k, 0),
                                v=(self.q_cols + self.k_cols, vd, vd, cache.v))
        ops.tag("attention")
        ops.distance_attention(proj[:, :self.q_cols], cache.k, cache.v, cache.block_table, cache.page_size, step, into,
                               self.heads, self.kv_heads, d, vd, self.scale, self.r1, self.r2, out_scale, int(self.window or 0),
                               self.split_scratch)


register_part("mixer", "distance_attention", DistanceAttention)
