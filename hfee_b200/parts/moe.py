"""Routed mixture of small gated experts, with an optional expert that every token uses.

    s = softmax(W_router h)  (float32, over all experts)         chosen = the ``top`` largest s
    out = sum_(e in chosen) router_scale * s_e * expert_e(h)  +  shared(h)
    expert(h) = W_down (g * sigmoid(alpha * g) * (u + shift)),  g = min(W_gate h, limit),  u = clamp(W_up h, -limit, limit)

The chosen weights are not renormalised.  ``router`` = ``"sigmoid_groups"`` is another router: s = sigmoid(W_router h);
the experts form ``groups`` equal groups of neighbours, a group's score is the sum of its two largest s, only experts of the
``keep`` best groups can be chosen, and the chosen s are divided by their sum (+ 1e-20) before the scale.  ``limit`` None
means no clamp (with alpha = 1 and shift = 0 the expert is silu(gate) * up), and ``shared_gate`` multiplies the shared
expert's output by sigmoid(W_sg h), one number per token.  The experts' tensors are stacked at load time (``[experts, 2 * inner, width]``,
each expert's gate rows and then its up rows, and ``[experts, width, inner]``); the (token, choice) pairs are ordered by
expert on the device, so the launches of a step depend on its token count alone and the step replays from a CUDA graph.
In bfloat16 with rows of whole 16-byte pieces the two products run on the tensor cores as grouped products over tiles of
128 places that never span two experts, the activation in the first one's epilogue (gate and up rows stored in runs of
four); otherwise (float32) on the CUDA cores in tiles of 32 places.  The shared expert's activation runs in the epilogue
of its gate/up product for prompt portions in bfloat16.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .gated_attention import pad8


class RoutedExperts(Part):
    """spec: ``width``, ``experts``, ``top``, ``router_scale``, ``inner``, ``limit``, ``alpha``, ``shared_inner`` and
    ``shared_limit`` (``shared_inner`` None: no shared expert); optional: ``shift`` (default 1), ``router`` (``"softmax"``,
    the default, or ``"sigmoid_groups"`` with ``groups`` and ``keep``), ``shared_gate`` (default False; tensor
    ``shared.sg`` [1, width]).  ``forward(..., accumulate=False)`` stores the output."""
    category = "feed_forward"
    graph_safe = True
    can_overwrite = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        w, f = spec.width, spec.inner
        needs = {"router": TensorNeed((spec.experts, w))}
        for e in range(spec.experts):
            needs[f"e{e}.gate"] = TensorNeed((f, w))
            needs[f"e{e}.up"] = TensorNeed((f, w))
            needs[f"e{e}.down"] = TensorNeed((w, f))
        if spec.get("shared_inner") is not None:
            s = spec.shared_inner
            needs.update({"shared.gate": TensorNeed((s, w)), "shared.up": TensorNeed((s, w)), "shared.down": TensorNeed((w, s))})
            if spec.get("shared_gate"):
                needs["shared.sg"] = TensorNeed((1, w))
        return needs

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.width, self.experts, self.top = int(spec.width), int(spec.experts), int(spec.top)
        self.inner, self.alpha = int(spec.inner), float(spec.alpha)
        self.limit = float("inf") if spec.get("limit") is None else float(spec.limit)
        self.shift = float(spec.get("shift", 1.0))
        self.router_scale = float(spec.router_scale)
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"top {self.top} is outside 1..{self.experts}")
        self.router = str(spec.get("router", "softmax"))
        if self.router == "sigmoid_groups":
            self.groups, self.keep = int(spec.groups), int(spec.keep)
            if self.groups < 1 or self.experts % self.groups or not 1 <= self.keep <= self.groups:
                raise ValueError(f"{self.experts} experts do not form {self.groups} equal groups of which {self.keep} are kept")
            if self.top > self.keep * (self.experts // self.groups):
                raise ValueError(f"top {self.top} exceeds the {self.keep * (self.experts // self.groups)} experts of the kept groups")
        elif self.router != "softmax":
            raise ValueError(f"unknown router {self.router!r} (known: softmax, sigmoid_groups)")
        self.w_router = tensors["router"]
        self.shared_gate = spec.get("shared_inner") is not None and bool(spec.get("shared_gate", False))
        if self.shared_gate:
            # the shared expert's gate rides in the router's product as one more row; the grouped router reads its rows
            # with a stride, the softmax router does not
            if self.router != "sigmoid_groups":
                raise ValueError("a gated shared expert goes with the sigmoid_groups router")
            self.w_router = torch.cat([tensors["router"], tensors["shared.sg"]], dim=0).contiguous()
        pairs = rt.max_tokens * self.top
        self.grouped = ops.moe_experts_grouped_ok(rt.dtype, self.width, self.inner)
        self.tiles = ops.moe_tiles_grouped(pairs, self.experts) if self.grouped else ops.moe_max_tiles(pairs, self.experts)
        g = ops.SWIGLU_GRANULE
        gates = torch.stack([tensors[f"e{e}.gate"] for e in range(self.experts)])
        ups = torch.stack([tensors[f"e{e}.up"] for e in range(self.experts)])
        # grouped products: gate and up rows in runs of four, so that the first product's epilogue applies the activation
        self.fused_act = self.grouped and self.inner % g == 0
        if self.fused_act:
            self.w_gate_up = ops.interleave_gate_up(gates, ups, g)
        else:
            self.w_gate_up = torch.cat([gates, ups], dim=1).contiguous()
            self.w_gate, self.w_up = self.w_gate_up[:, :self.inner], self.w_gate_up[:, self.inner:]
        del gates, ups
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]).contiguous()
        self.shared_inner = spec.get("shared_inner")
        if self.shared_inner is not None:
            self.shared_inner = int(self.shared_inner)
            self.shared_limit = float("inf") if spec.get("shared_limit") is None else float(spec.shared_limit)
            gate, up = tensors["shared.gate"], tensors["shared.up"]
            if gate.dtype == torch.bfloat16 and self.shared_inner % g == 0:
                self.shared_granule, self.w_shared_in = g, ops.interleave_gate_up(gate, up, g)
            else:
                self.shared_granule, self.w_shared_in = self.shared_inner, torch.cat([gate, up], dim=0).contiguous()
            self.w_shared_down = tensors["shared.down"]

    def forward(self, xn, out: torch.Tensor, step: Any, accumulate: bool = True) -> None:
        n, rt, top = step.n, self.rt, self.top
        xn = xn if isinstance(xn, torch.Tensor) else xn.tensor()
        i32 = torch.int32
        logits = rt.scratch("moe_logits", (rt.max_tokens, self.w_router.shape[0]), torch.float32)[:n]
        choice = rt.scratch("moe_choice", (rt.max_tokens, top), i32)[:n]
        weight = rt.scratch("moe_weight", (rt.max_tokens, top), torch.float32)[:n]
        ops.tag("router")
        ops.linear(xn, self.w_router, logits)
        if self.router == "sigmoid_groups":
            ops.moe_route_grouped(logits, self.experts, top, self.groups, self.keep, self.router_scale, choice, weight)
        else:
            ops.moe_route(logits, top, self.router_scale, choice, weight)
        gate_col = logits[:, self.experts:] if self.shared_gate else None
        place = None
        if self.grouped:
            rows = self.tiles * ops.GROUPED_TILE_ROWS
            place = rt.scratch("moe_place", (rt.max_tokens * top,), i32)
            row_pair = rt.scratch("moe_row_pair", (rows,), i32)
            tile_group = rt.scratch("moe_tile_group", (self.tiles,), i32)
            rows_in = rt.scratch("moe_rows_in", (rows, self.width))
            gate_up = None if self.fused_act else rt.scratch("moe_gate_up", (rows, 2 * self.inner))
            hidden = rt.scratch("moe_hidden_rows", (rows, self.inner))
            pair_out = rt.scratch("moe_rows_out", (rows, self.width), torch.float32)
            ops.tag("experts")
            ops.moe_experts_grouped(xn, top, choice, self.w_gate_up, self.w_down, self.limit, place, row_pair, tile_group,
                                    rows_in, gate_up, hidden, pair_out, self.alpha, self.shift)
        else:
            offsets = rt.scratch("moe_offsets", (self.experts + 1,), i32)
            order = rt.scratch("moe_order", (rt.max_tokens * top,), i32)
            tile_expert = rt.scratch("moe_tile_expert", (self.tiles,), i32)
            tile_row = rt.scratch("moe_tile_row", (self.tiles,), i32)
            hidden = rt.scratch("moe_hidden", (rt.max_tokens * top, pad8(self.inner)))[:n * top, :self.inner]
            pair_out = rt.scratch("moe_pair_out", (rt.max_tokens * top, self.width), torch.float32)[:n * top]
            ops.moe_plan(choice, self.experts, offsets, order, tile_expert, tile_row)
            ops.tag("experts")
            ops.moe_experts(xn, top, self.w_gate, self.w_up, self.w_down, self.limit, offsets, order, tile_expert, tile_row,
                            hidden, pair_out, self.alpha, self.shift)
        extra = None
        if self.shared_inner is not None:
            s = self.shared_inner
            gu = rt.scratch("ffn_gate_up", (rt.max_tokens, pad8(2 * s)))[:n, :2 * s]
            h = rt.scratch("ffn_hidden", (rt.max_tokens, pad8(s)))[:n, :s]
            ops.tag("gate_up")
            ops.linear_clamped_glu(xn, self.w_shared_in, h, self.shared_granule, gu, self.shared_limit, self.alpha, self.shift)
            ops.tag("down")
            if gate_col is None:
                ops.linear(h, self.w_shared_down, out, accumulate=accumulate)
                accumulate = True
            else:           # the gated shared expert joins the routed ones in the weighted sum
                extra = rt.scratch("moe_shared_out", (rt.max_tokens, self.width), torch.float32)[:n]
                ops.linear(h, self.w_shared_down, extra)
        ops.tag("experts")
        ops.moe_combine(pair_out, weight, out, accumulate, place, extra, gate_col)


register_part("feed_forward", "routed_experts", RoutedExperts)
