"""Arrangement of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from typing import Any

import torch

from ..kernels import ops
from .base import Block, register_part
from .norm import LazyNormed


class PreNormBlock(Block):
    """``x += mixer(norm(x)); x += feed_forward(norm(x))`` on the float32 residual
    stream (hostfog/hfee internal/llm/forward.go:82-114).  Built by the model with
    its parts already constructed; ``ffn`` with ``ffn_norm`` is optional (a layer may have no
    feed-forward).  ``forward(..., residual_add=e)`` first adds ``e`` to the stream, inside the
    mixer norm's kernel when that norm can (``takes_residual_add``)."""
    needs = ("mixer", "mixer_norm")
    graph_safe = True

    def __init__(self, spec, tensors, rt, parts):
        super().__init__(spec, tensors, rt, parts)
        self.mixer, self.feed_forward = parts["mixer"], parts.get("ffn")
        self.mixer_norm, self.ffn_norm = parts["mixer_norm"], parts.get("ffn_norm")
        if (self.feed_forward is None) != (self.ffn_norm is None):
            raise ValueError("a feed-forward and its input norm come together")
        self.width = int(spec.width)
        import inspect
        self.takes_residual_add = "residual_add" in inspect.signature(self.mixer_norm.forward).parameters

    def forward(self, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool, residual_add=None) -> None:
        xn = self.rt.scratch("block_normed", (self.rt.max_tokens, self.width))[:step.n]
        if residual_add is not None:
            self.mixer_norm.forward(residual, xn, residual_add=residual_add)
            self.mixer.forward(xn, residual, step, cache, writes_cache)
        else:
            self.mixer.forward(self._normed(self.mixer, self.mixer_norm, residual, xn), residual, step, cache, writes_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(self._normed(self.feed_forward, self.ffn_norm, residual, xn), residual, step)

    @staticmethod
    def _normed(consumer, norm, residual, buffer):
        """The consumer's input: a lazily normed one if it says it can take it (and may fuse the
        norm into its first product), else the normed tensor."""
        lazy = LazyNormed(norm, residual, buffer)
        return lazy if getattr(consumer, "accepts_lazy_input", False) else lazy.tensor()


class OutputNormBlock(Block):
    """``x += norm(mixer(conv_in(x))); x += norm(feed_forward(x))``: the norms sit on the sublayers'
    outputs and the sublayers read the residual stream itself.  Optional parts: ``mixer_conv`` (a short
    convolution over time added to what the mixer reads: the mixer gets ``x + conv(x)``), ``ffn`` with
    ``ffn_norm`` (a layer may have no feed-forward).  The layer's cache is a bundle: the mixer's pages
    or its state (named ``recurrent``) and the convolution's history (``conv``)."""
    needs = ("mixer", "mixer_norm")
    graph_safe = True

    def __init__(self, spec, tensors, rt, parts):
        super().__init__(spec, tensors, rt, parts)
        self.mixer, self.mixer_norm = parts["mixer"], parts["mixer_norm"]
        self.conv = parts.get("mixer_conv")
        self.feed_forward, self.ffn_norm = parts.get("ffn"), parts.get("ffn_norm")
        if (self.feed_forward is None) != (self.ffn_norm is None):
            raise ValueError("a feed-forward and its output norm come together")
        self.width = int(spec.width)

    def cache_need(self):
        from ..cache.needs import CacheBundle, FixedState, PagedKV
        need = self.mixer.cache_need()
        if self.conv is None:
            return need
        states = {"conv": self.conv.cache_need()}
        if isinstance(need, FixedState):
            states["recurrent"] = need
        elif need is not None and not isinstance(need, PagedKV):
            raise TypeError(f"an output-norm block cannot bundle a mixer cache of type {type(need).__name__}")
        return CacheBundle.of(need if isinstance(need, PagedKV) else None, **states)

    def forward(self, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool) -> None:
        rt, n = self.rt, step.n
        y = rt.scratch("block_sublayer_out", (rt.max_tokens, self.width), torch.float32)[:n]
        if self.conv is not None:
            h = rt.scratch("block_normed", (rt.max_tokens, self.width))[:n]
            self.conv.forward(residual, h, step, cache.states["conv"], writes_cache)
        else:
            h = self._as_input(residual, n)
        self._run(self.mixer, y, h, step, cache, writes_cache)
        if self.feed_forward is None:
            self.mixer_norm.forward_add(y, residual)
            return
        if rt.dtype == torch.float32:
            self.mixer_norm.forward_add(y, residual)
            x = residual
        else:       # the norm kernel also leaves the new residual in the feed-forward's input dtype
            x = rt.scratch("block_normed", (rt.max_tokens, self.width))[:n]
            self.mixer_norm.forward_add(y, residual, cast_out=x)
        self._run(self.feed_forward, y, x, step)
        self.ffn_norm.forward_add(y, residual)

    def _as_input(self, residual: torch.Tensor, n: int) -> torch.Tensor:
        """The residual stream in the dtype the matrix products read."""
        if self.rt.dtype == torch.float32:
            return residual
        x = self.rt.scratch("block_normed", (self.rt.max_tokens, self.width))[:n]
        ops.tag("norm")
        ops.cast_rows(residual, x)
        return x

    @staticmethod
    def _run(part, y, x, step, *cache_args):
        """``y = part(x)``: parts that can store their output do; others add into a cleared buffer."""
        if getattr(part, "can_overwrite", False):
            part.forward(x, y, step, *cache_args, accumulate=False)
        else:
            y.zero_()
            part.forward(x, y, step, *cache_args)


class SandwichNormBlock(Block):
    """``x += norm_out(mixer(norm_in(x))); x += norm_out'(feed_forward(norm_in'(x)))``: a norm in front of every
    sublayer and another on its output.  ``ffn`` with ``ffn_norm`` and ``ffn_out_norm`` is optional (a layer may have
    no feed-forward).  The layer's cache is whatever the mixer asks for."""
    needs = ("mixer", "mixer_norm", "mixer_out_norm")
    graph_safe = True

    def __init__(self, spec, tensors, rt, parts):
        super().__init__(spec, tensors, rt, parts)
        self.mixer, self.mixer_norm, self.mixer_out_norm = parts["mixer"], parts["mixer_norm"], parts["mixer_out_norm"]
        self.feed_forward = parts.get("ffn")
        self.ffn_norm, self.ffn_out_norm = parts.get("ffn_norm"), parts.get("ffn_out_norm")
        if (self.feed_forward is None) != (self.ffn_norm is None) or (self.feed_forward is None) != (self.ffn_out_norm is None):
            raise ValueError("a feed-forward comes with its input norm and its output norm")
        self.width = int(spec.width)

    def forward(self, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool) -> None:
        rt, n = self.rt, step.n
        xn = rt.scratch("block_normed", (rt.max_tokens, self.width))[:n]
        y = rt.scratch("block_sublayer_out", (rt.max_tokens, self.width), torch.float32)[:n]
        self.mixer_norm.forward(residual, xn)
        OutputNormBlock._run(self.mixer, y, xn, step, cache, writes_cache)
        if self.feed_forward is None:
            self.mixer_out_norm.forward_add(y, residual)
            return
        # the output norm's kernel also leaves the next sublayer's normed input
        self.mixer_out_norm.forward_add(y, residual, then=self.ffn_norm, then_out=xn)
        OutputNormBlock._run(self.feed_forward, y, xn, step)
        self.ffn_out_norm.forward_add(y, residual)


class ScaledPreNormBlock(Block):
    """``y = x + m * mixer(norm(x)); r = y + m * feed_forward(norm(y))`` with one multiplier ``m`` on every
    sublayer's output (spec ``residual_scale``), and an optional ``merge`` part that turns the layer's result r into
    what the next layer reads.  ``ffn`` with ``ffn_norm`` is optional.  The scaled sum and the next norm leave in one
    kernel; the last sum is the merge's, when there is one."""
    needs = ("mixer", "mixer_norm")
    graph_safe = True

    def __init__(self, spec, tensors, rt, parts):
        super().__init__(spec, tensors, rt, parts)
        self.mixer, self.mixer_norm = parts["mixer"], parts["mixer_norm"]
        self.feed_forward, self.ffn_norm = parts.get("ffn"), parts.get("ffn_norm")
        if (self.feed_forward is None) != (self.ffn_norm is None):
            raise ValueError("a feed-forward and its input norm come together")
        self.merge = parts.get("merge")
        self.width, self.scale = int(spec.width), float(spec.residual_scale)

    def forward(self, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool) -> None:
        rt, n = self.rt, step.n
        xn = rt.scratch("block_normed", (rt.max_tokens, self.width))[:n]
        y = rt.scratch("block_sublayer_out", (rt.max_tokens, self.width), torch.float32)[:n]
        if self.merge is not None:
            self.merge.begin(residual, step)
        self.mixer_norm.forward(residual, xn)
        OutputNormBlock._run(self.mixer, y, xn, step, cache, writes_cache)
        if self.feed_forward is not None:
            ops.tag("norm")
            ops.scaled_add_norm(y, self.scale, residual, self.ffn_norm.weight, self.ffn_norm.eps, xn)
            OutputNormBlock._run(self.feed_forward, y, xn, step)
        if self.merge is not None:
            self.merge.forward(residual, y, self.scale, step)
        else:
            ops.tag("norm")
            ops.scaled_add(y, self.scale, residual)


register_part("block", "scaled_pre_norm", ScaledPreNormBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
register_part("block", "pre_norm", PreNormBlock)
register_part("block", "output_norm", OutputNormBlock)
