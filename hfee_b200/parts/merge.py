"""What a layer hands on, when that is more than its own result.

``depth_average``: with X_0 the embedding's output and X_(i+1) the result of layer i, the stream that leaves layer i
is ``sum_(j <= i+1) a_i[j] X_j`` with the layer's own i + 2 weights.  The X_j of the step's tokens are kept in one
scratch buffer of the engine (they belong to the step, not to a request: nothing is cached), so the layers of a
model share it by name.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Part, register_part


class DepthAverage(Part):
    """spec: ``width``, ``index`` (the layer's place i, from 0), ``depth`` (number of layers in the model)."""
    category = "merge"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"weights": TensorNeed((spec.index + 2,), role="average")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.index, self.depth, self.width = int(spec.index), int(spec.depth), int(spec.width)
        if not 0 <= self.index < self.depth:
            raise ValueError(f"layer index {self.index} is outside a model of {self.depth} layers")
        self.weights = tensors["weights"]

    def _history(self) -> torch.Tensor:
        return self.rt.scratch("depth_history", (self.depth + 1, self.rt.max_tokens, self.width), torch.float32)

    def begin(self, residual: torch.Tensor, step: Any) -> None:
        """In front of the layer's sublayers: the first layer keeps the stream it was given as X_0."""
        if self.index == 0:
            self._history()[0, :step.n].copy_(residual)

    def forward(self, residual: torch.Tensor, y: Optional[torch.Tensor], scale: float, step: Any) -> None:
        """``residual`` (+ ``scale * y``) is the layer's result; it is kept, and ``residual`` becomes the average."""
        before = ops.tag("norm")
        ops.depth_average(residual, y, scale, self._history(), self.weights, self.index)
        ops.tag(before)


register_part("merge", "depth_average", DepthAverage)
