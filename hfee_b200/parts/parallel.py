"""Several split mixers side by side on one input: ``out = sum_b scale_b * mixer_b(h)``.

The branches' input projections run as one product, every branch leaves what its output projection reads (already
times its scale) in its columns of one buffer, and one product with the branches' output weights side by side
adds them up.  Each branch keeps the cache it asks for: pages from (at most) one branch, and every branch's named
states under ``<branch>.<name>``.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..cache.manager import CacheView
from ..cache.needs import CacheBundle, FixedState, PagedKV
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Mixer, part_class, register_part
from .gated_attention import pad8
from .recurrent import SplitMixer

BRANCHES = ("left", "right")


class ParallelMixer(Mixer):
    """spec: ``width``, ``left``, ``right`` (PartSpecs of split mixers), ``left_scale``, ``right_scale``."""
    graph_safe = True
    can_overwrite = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        needs = {}
        for b in BRANCHES:
            sub = getattr(spec, b)
            for key, need in part_class("mixer", sub.kind).tensor_needs(sub).items():
                needs[f"{b}.{key}"] = need
        return needs

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.branches, self.scales = [], []
        for b in BRANCHES:
            sub = getattr(spec, b)
            own = {k[len(b) + 1:]: t for k, t in tensors.items() if k.startswith(b + ".")}
            part = part_class("mixer", sub.kind)(sub, own, rt)
            if not isinstance(part, SplitMixer):
                raise ValueError(f"a parallel mixer runs split mixers; {sub.kind!r} is none")
            self.branches.append((b, part))
            self.scales.append(float(getattr(spec, b + "_scale")))
        self.w_in = torch.cat([p.in_weight for _, p in self.branches], dim=0).contiguous()
        self.w_o = torch.cat([p.w_o for _, p in self.branches], dim=1).contiguous()
        self.in_cols, self.inner_cols = self.w_in.shape[0], self.w_o.shape[1]
        for _, p in self.branches:          # the branches' own copies are not used again
            p.in_weight = p.w_o = None
        self.out_bias = None
        for (_, p), scale in zip(self.branches, self.scales):
            if p.out_bias is not None:
                b = p.out_bias * scale
                self.out_bias = b if self.out_bias is None else self.out_bias + b

    def cache_need(self) -> CacheBundle:
        paged, states = None, {}
        for b, part in self.branches:
            need = part.cache_need()
            if isinstance(need, PagedKV):
                need = CacheBundle.of(need)
            elif isinstance(need, FixedState):
                need = CacheBundle.of(None, state=need)
            if need is None:
                continue
            if need.paged is not None:
                if paged is not None:
                    raise ValueError("only one branch of a parallel mixer may keep pages")
                paged = need.paged
            for name, state in need.states:
                states[f"{b}.{name}"] = state
        return CacheBundle(paged, tuple(sorted(states.items())))

    def _view(self, cache: Any, branch: str) -> CacheView:
        own = {k[len(branch) + 1:]: t for k, t in cache.states.items() if k.startswith(branch + ".")}
        return CacheView(k=cache.k, v=cache.v, block_table=cache.block_table, page_size=cache.page_size,
                         state=own.get("state"), states=own)

    def forward(self, h, out: torch.Tensor, step: Any, cache: Any, writes_cache: bool, accumulate: bool = True) -> None:
        n, rt = step.n, self.rt
        h = h if isinstance(h, torch.Tensor) else h.tensor()
        proj = rt.scratch("split_proj", (rt.max_tokens, pad8(self.in_cols)))[:n, :self.in_cols]
        ops.tag("qkv")
        ops.linear(h, self.w_in, proj)
        inner = rt.scratch("split_inner", (rt.max_tokens, pad8(self.inner_cols)))[:n, :self.inner_cols]
        at_in = at_out = 0
        for (b, part), scale in zip(self.branches, self.scales):
            rows, cols = part_rows(part), part.inner_cols
            extra = {"h": h} if part.needs_input else {}
            part.mix(proj[:, at_in:at_in + rows], step, self._view(cache, b), writes_cache, inner[:, at_out:at_out + cols], scale,
                     **extra)
            at_in, at_out = at_in + rows, at_out + cols
        ops.tag("o")
        ops.linear(inner, self.w_o, out, accumulate=accumulate)
        if self.out_bias is not None:
            ops.add_bias(out, self.out_bias)


def part_rows(part: SplitMixer) -> int:
    """Rows of a branch's input projection (its ``in_weight`` may have been handed over already)."""
    return int(part.in_rows)


register_part("mixer", "parallel", ParallelMixer)
