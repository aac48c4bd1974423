"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))`` added to the residual
stream; ``act`` is SiLU (hostfog/hfee internal/llm/forward.go:110-114, internal/ggml/ops.go:160-165)
or the tanh form of GELU."""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Part, register_part


class SwiGLUFeedForward(Part):
    """spec: ``width``, ``inner`` (intermediate size), ``activation`` (``"silu"``, the default, or
    ``"gelu_tanh"``).  ``forward(..., accumulate=False)`` stores the output instead of adding it."""
    can_overwrite = True
    category = "feed_forward"
    graph_safe = True
    accepts_lazy_input = True        # the input norm may be fused into the gate/up projection

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"gate": TensorNeed((spec.inner, spec.width)), "up": TensorNeed((spec.inner, spec.width)),
                "down": TensorNeed((spec.width, spec.inner))}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.inner = int(spec.inner)
        self.activation = str(spec.get("activation", "silu"))
        if self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"unknown feed-forward activation {self.activation!r} (known: {sorted(ops.GATE_ACTIVATIONS)})")
        # one fused projection.  bfloat16: rows in groups of 4 gate rows then 4 up rows, so a
        # kernel that owns 8 consecutive rows can apply SwiGLU in its epilogue; else [gate | up].
        gate, up = tensors["gate"], tensors["up"]
        g = ops.SWIGLU_GRANULE
        if gate.dtype == torch.bfloat16 and self.inner % g == 0:
            self.granule = g
            w = torch.stack([gate.reshape(self.inner // g, g, -1), up.reshape(self.inner // g, g, -1)], dim=1)
            self.w_gate_up = w.reshape(2 * self.inner, -1).contiguous()
        else:
            self.granule = self.inner
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors["down"]

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step: Any, accumulate: bool = True) -> None:
        n, rt = step.n, self.rt
        gu = rt.scratch("ffn_gate_up", (rt.max_tokens, 2 * self.inner))[:n]
        h = rt.scratch("ffn_hidden", (rt.max_tokens, self.inner))[:n]
        ops.tag("gate_up")
        if self.activation == "silu":
            ops.linear_swiglu_normed(xn, self.w_gate_up, h, self.granule, gu)
        else:
            ops.linear_gated_normed(xn, self.w_gate_up, h, self.granule, gu, self.activation)
        ops.tag("down")
        ops.linear(h, self.w_down, residual, accumulate=accumulate)


class DenseFeedForward(Part):
    """``down(act(up(x)))`` without a gate.  spec: ``width``, ``inner``, ``activation`` (``"relu2"``: the square of
    relu).  ``forward(..., accumulate=False)`` stores the output instead of adding it."""
    can_overwrite = True
    category = "feed_forward"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"up": TensorNeed((spec.inner, spec.width)), "down": TensorNeed((spec.width, spec.inner))}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.inner = int(spec.inner)
        self.activation = str(spec.activation)
        if self.activation not in ops.UNARY_ACTIVATIONS:
            raise ValueError(f"unknown feed-forward activation {self.activation!r} (known: {sorted(ops.UNARY_ACTIVATIONS)})")
        self.w_up, self.w_down = tensors["up"], tensors["down"]

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step: Any, accumulate: bool = True) -> None:
        n, rt = step.n, self.rt
        xn = xn if isinstance(xn, torch.Tensor) else xn.tensor()
        h = rt.scratch("ffn_hidden", (rt.max_tokens, self.inner))[:n]
        ops.tag("up")
        ops.linear_act(xn, self.w_up, h, self.activation)
        ops.tag("down")
        ops.linear(h, self.w_down, residual, accumulate=accumulate)


class ClampedGluFeedForward(Part):
    """``down(g * sigmoid(alpha * g) * (u + shift))`` with ``g = min(gate(x), limit)``, ``u = clamp(up(x), -limit, limit)``.
    spec: ``width``, ``inner``, ``limit``, ``alpha``, ``shift`` (default 1).  ``forward(..., accumulate=False)`` stores the
    output instead of adding it.  In bfloat16 the activation runs in the epilogue of the gate/up product for prompt
    portions (gate and up rows stored in runs of four)."""
    can_overwrite = True
    category = "feed_forward"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"gate": TensorNeed((spec.inner, spec.width)), "up": TensorNeed((spec.inner, spec.width)),
                "down": TensorNeed((spec.width, spec.inner))}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.inner, self.limit, self.alpha = int(spec.inner), float(spec.limit), float(spec.alpha)
        self.shift = float(spec.get("shift", 1.0))
        if self.limit <= 0:
            raise ValueError(f"the limit must be positive, got {self.limit}")
        gate, up = tensors["gate"], tensors["up"]
        g = ops.SWIGLU_GRANULE
        if gate.dtype == torch.bfloat16 and self.inner % g == 0:
            self.granule, self.w_gate_up = g, ops.interleave_gate_up(gate, up, g)
        else:
            self.granule, self.w_gate_up = self.inner, torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors["down"]

    def forward(self, xn, residual: torch.Tensor, step: Any, accumulate: bool = True) -> None:
        from .gated_attention import pad8
        n, rt = step.n, self.rt
        xn = xn if isinstance(xn, torch.Tensor) else xn.tensor()
        gu = rt.scratch("ffn_gate_up", (rt.max_tokens, pad8(2 * self.inner)))[:n, :2 * self.inner]
        h = rt.scratch("ffn_hidden", (rt.max_tokens, pad8(self.inner)))[:n, :self.inner]
        ops.tag("gate_up")
        ops.linear_clamped_glu(xn, self.w_gate_up, h, self.granule, gu, self.limit, self.alpha, self.shift)
        ops.tag("down")
        ops.linear(h, self.w_down, residual, accumulate=accumulate)


register_part("feed_forward", "clamped_glu", ClampedGluFeedForward)
register_part("feed_forward", "dense", DenseFeedForward)
register_part("feed_forward", "swiglu", SwiGLUFeedForward)
register_part("feed_forward", "gated", SwiGLUFeedForward)       # the same part named for its general form
