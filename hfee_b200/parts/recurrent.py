"""Mixers built on an elementwise linear recurrence S_t = a_t S_(t-1) + b_t with a float32 state per request.

``mingru``: the gates read only the current token.  With h the mixer's input::

    z = sigmoid(W_z h + b_z)      u = W_x h + b_x      c = u + 1/2 where u >= 0, sigmoid(u) where u < 0
    S_t = (1 - z) S_(t-1) + z c   (per channel)        out = W_o (S_t * silu(W_g h))

``selective_scan``: a state-space scan whose step size, input and read-out vectors depend on the token, behind a
short causal convolution::

    [x | z] = W_in h              x = silu(conv(x) + b_conv)          [dt | B | C] = W_x x
    dt = softplus(W_dt dt + b_dt) A = -exp(A_log)
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n              y_c = sum_n S[c, n] C_n + D_c x_c
    out = W_o (y * silu(z))

States start at zero and belong to the request (as do the convolution's last ``taps - 1`` inputs), so a prompt may be
cut anywhere.  Gates, step sizes, decays and states are float32; the projections are the activations' dtype.

Both are *split mixers*: ``in_weight`` (the rows of their input projection), ``inner_cols`` and ``w_o`` are public and
``mix(proj, step, cache, writes_cache, into, out_scale)`` leaves what W_o reads, times ``out_scale``, in ``into``, so
that a mixer that runs several of them side by side can project once in and once out.  A split mixer may also carry
``out_bias`` (added after W_o) and set ``needs_input`` (its ``mix`` then gets the mixer's input as ``h=`` for a small
product of its own).
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..cache.needs import CacheBundle, FixedState
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Mixer, register_part
from .gated_attention import pad8


class SplitMixer(Mixer):
    """A mixer of the form ``W_o f(W_in h)``; see the module's text."""
    graph_safe = True
    can_overwrite = True
    in_weight: torch.Tensor
    w_o: torch.Tensor
    inner_cols: int
    in_rows: int
    out_bias = None          # float32 [width] added to the mixer's output, or None
    needs_input = False      # True: ``mix`` also takes the mixer's input itself, as ``h=``

    def mix(self, proj: torch.Tensor, step: Any, cache: Any, writes_cache: bool, into: torch.Tensor, out_scale: float = 1.0) -> None:
        raise NotImplementedError

    def forward(self, h, out: torch.Tensor, step: Any, cache: Any, writes_cache: bool, accumulate: bool = True) -> None:
        n, rt = step.n, self.rt
        h = h if isinstance(h, torch.Tensor) else h.tensor()
        rows = self.in_weight.shape[0]
        proj = rt.scratch("split_proj", (rt.max_tokens, pad8(rows)))[:n, :rows]
        ops.tag("qkv")
        ops.linear(h, self.in_weight, proj)
        inner = rt.scratch("split_inner", (rt.max_tokens, pad8(self.inner_cols)))[:n, :self.inner_cols]
        if self.needs_input:
            self.mix(proj, step, cache, writes_cache, inner, h=h)
        else:
            self.mix(proj, step, cache, writes_cache, inner)
        ops.tag("o")
        ops.linear(inner, self.w_o, out, accumulate=accumulate)
        if self.out_bias is not None:
            ops.add_bias(out, self.out_bias)


class MinGRU(SplitMixer):
    """spec: ``width``, ``channels`` (size of the recurrence)."""

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        c, w = spec.channels, spec.width
        return {"z": TensorNeed((c, w)), "x": TensorNeed((c, w)), "g": TensorNeed((c, w)), "o": TensorNeed((w, c)),
                "z_bias": TensorNeed((c,), role="vector"), "x_bias": TensorNeed((c,), role="vector")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.channels = int(spec.channels)
        self.in_weight = torch.cat([tensors["z"], tensors["x"], tensors["g"]], dim=0).contiguous()
        self.z_bias, self.x_bias = tensors["z_bias"], tensors["x_bias"]
        self.w_o = tensors["o"]
        self.inner_cols, self.in_rows = self.channels, 3 * self.channels

    def cache_need(self) -> FixedState:
        return FixedState((self.channels,), "float32")

    def mix(self, proj, step, cache, writes_cache, into, out_scale: float = 1.0) -> None:
        if out_scale != 1.0:
            raise ValueError("the minGRU mixer has no output scale")
        c = self.channels
        ops.tag("scan")
        ops.mingru(proj, 0, c, 2 * c, self.z_bias, self.x_bias, cache.state, step, into, c, writes_cache)


class SelectiveScan(SplitMixer):
    """spec: ``width``, ``inner`` (channels), ``state`` (entries per channel), ``dt_rank``, ``taps``."""

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        c, n, r, w = spec.inner, spec.state, spec.dt_rank, spec.width
        return {"in": TensorNeed((2 * c, w)), "conv": TensorNeed((c, spec.taps), role="vector"),
                "conv_bias": TensorNeed((c,), role="vector"), "x": TensorNeed((r + 2 * n, c)), "dt": TensorNeed((c, r)),
                "dt_bias": TensorNeed((c,), role="vector"), "A_log": TensorNeed((c, n), role="vector"),
                "D": TensorNeed((c,), role="vector"), "o": TensorNeed((w, c))}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.inner, self.n_state, self.dt_rank, self.taps = int(spec.inner), int(spec.state), int(spec.dt_rank), int(spec.taps)
        if self.taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {self.taps}")
        self.in_weight = tensors["in"]
        self.conv_weight, self.conv_bias = tensors["conv"], tensors["conv_bias"]
        self.w_x, self.w_dt = tensors["x"], tensors["dt"]
        self.dt_bias, self.a_log, self.d_skip = tensors["dt_bias"], tensors["A_log"], tensors["D"]
        self.w_o = tensors["o"]
        self.inner_cols, self.in_rows = self.inner, 2 * self.inner
        self.low_cols = self.dt_rank + 2 * self.n_state

    def cache_need(self) -> CacheBundle:
        return CacheBundle.of(None, conv=FixedState((self.taps - 1, self.inner), "float32"),
                              recurrent=FixedState((self.inner, self.n_state), "float32"))

    def mix(self, proj, step, cache, writes_cache, into, out_scale: float = 1.0) -> None:
        n, rt, c = step.n, self.rt, self.inner
        xc = rt.scratch("scan_conv", (rt.max_tokens, pad8(c)))[:n, :c]
        ops.tag("conv")
        ops.conv_act(proj[:, :c], self.conv_weight, cache.states["conv"], step, xc, "silu", writes_cache, bias=self.conv_bias)
        low = rt.scratch("scan_low", (rt.max_tokens, pad8(self.low_cols)))[:n, :self.low_cols]
        ops.tag("scan_proj")
        ops.linear(xc, self.w_x, low)
        dt = rt.scratch("scan_dt", (rt.max_tokens, c), torch.float32)[:n]
        ops.linear(low[:, :self.dt_rank], self.w_dt, dt)
        ops.tag("scan")
        ops.selective_scan(xc, dt, low, self.dt_rank, self.dt_rank + self.n_state, proj[:, c:2 * c], self.a_log, self.d_skip,
                           self.dt_bias, cache.states["recurrent"], step, into, out_scale, writes_cache)


register_part("mixer", "mingru", MinGRU)
register_part("mixer", "selective_scan", SelectiveScan)
