"""Norm parts.  RMS norm, formula of hostfog/hfee internal/ggml/ops.go:125-134:
``dst = x * 1/sqrt(mean(x^2) + eps) * weight`` per row, with the sum in float32
here (float64 in the reference); and layer norm with a weight and no bias:
``dst = (x - mean) / sqrt(mean((x - mean)^2) + eps) * weight``."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Part, register_part


class RMSNorm(Part):
    """spec: ``width``, ``eps``, ``add_unit`` (scale by 1+w instead of w; default False)."""
    category = "norm"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"weight": TensorNeed((spec.width,), role="scale")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.weight = tensors["weight"]
        self.eps = float(spec.eps)
        self.add_unit = bool(spec.get("add_unit", False))

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        before = ops.tag("norm")
        ops.rmsnorm(x, self.weight, out, self.eps, rows=rows, add_unit=self.add_unit)
        ops.tag(before)


    def forward_add(self, y: torch.Tensor, residual: torch.Tensor, cast_out: Optional[torch.Tensor] = None,
                    then: Optional["RMSNorm"] = None, then_out: Optional[torch.Tensor] = None) -> None:
        """``residual += norm(y)``: the norm on a sublayer's output (both float32); ``cast_out`` also takes
        the new residual in the dtype the next matrix product reads.  With ``then`` (another norm) the new
        residual, normed by it, goes to ``then_out``: the input of the sublayer that follows."""
        before = ops.tag("norm")
        if then is not None and cast_out is None and residual.shape[1] <= ops.RMSNORM_ADD_NORM_MAX_WIDTH:
            ops.rmsnorm_add_norm(y, self.weight, residual, self.eps, then.weight, then.eps, then_out,
                                 add_unit=self.add_unit, add_unit2=then.add_unit)
        else:
            ops.rmsnorm_add(y, self.weight, residual, self.eps, add_unit=self.add_unit, cast_out=cast_out)
            if then is not None:
                ops.rmsnorm(residual, then.weight, then_out, then.eps, add_unit=then.add_unit)
        ops.tag(before)

    def fused_params(self):
        """(weight, eps, add_unit): what a kernel needs to apply this norm itself."""
        return self.weight, self.eps, self.add_unit


class LayerNorm(Part):
    """spec: ``width``, ``eps``.  Mean and variance (the mean of the squared deviations) per row in float32; a weight
    per column, no bias."""
    category = "norm"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"weight": TensorNeed((spec.width,), role="scale")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.weight = tensors["weight"]
        self.eps = float(spec.eps)

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None,
                residual_add: Optional[torch.Tensor] = None) -> None:
        """``residual_add`` (float32, like ``x``): the row normed is ``x + residual_add``, and ``x`` keeps that sum."""
        before = ops.tag("norm")
        ops.layernorm(x, self.weight, out, self.eps, rows=rows, residual_add=residual_add)
        ops.tag(before)


class LazyNormed:
    """The normed input of a mixer, feed-forward or head that has not been computed yet.

    A part that can fuse the norm into its first matrix product hands this object to
    ``ops.linear_normed``; any other use calls :meth:`tensor`, which runs the norm once into
    ``buffer`` and returns it.  ``rows`` gathers source rows (the head norms only the rows whose
    logits are wanted)."""

    def __init__(self, norm, source: torch.Tensor, buffer: torch.Tensor, rows: Optional[torch.Tensor] = None):
        self.norm, self.source, self.buffer, self.rows = norm, source, buffer, rows
        self.n = buffer.shape[0]
        self.out_dtype = buffer.dtype
        self._done = False

    def fused_params(self):
        f = getattr(self.norm, "fused_params", None)
        return f() if f is not None else None

    def tensor(self) -> torch.Tensor:
        if not self._done:
            self.norm.forward(self.source, self.buffer, rows=self.rows)
            self._done = True
        return self.buffer


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "layer_norm", LayerNorm)
