"""Linear attention whose matrix state is gated by the token.  With q, k of size ``key_dim`` and v of size
``value_dim`` per head (projections of the mixer's input h, q times key_dim^(-1/2)) and a float32 state per request:

``channel_decay_attention`` (gated linear attention): a decay per key channel from a low-rank projection,

    a_t = sigmoid(W_a2 (W_a1 h) + b_a2)^(1/tau)        S_t = diag(a_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t

each head's o RMS-normed over value_dim with one weight [value_dim] for all heads, times silu(W_g h), then W_o.

``matrix_memory`` (the matrix memory of an xLSTM): exponential input and forget gates per head, capped smoothly,

    i_t = c tanh((W_i h + b_i) / c)    f_t = logsigmoid(c tanh((W_f h + b_f) / c))    m_t = max(f_t + m_(t-1), i_t)
    S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T       n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)

(S, n and m start at zero); each head's o divided by its root mean square, times a weight [heads * value_dim], times
sigmoid(W_g h), then W_o.

Gates, decays, their logarithms and exponentials, the states and the norms are float32; the gates' pre-activations
leave their products in float32.  Both are *split mixers* (see :mod:`hfee_b200.parts.recurrent`).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.needs import CacheBundle, FixedState
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import register_part
from .gated_attention import pad8
from .recurrent import SplitMixer


def _workspace(part, step):
    """The chunked path's workspace, sized once for the engine's limits, for steps that take that path."""
    if step.max_new < ops.RECURRENCE_CHUNKED_MIN:
        return None
    rt = part.rt
    return rt.scratch("recurrence_runs", (ops.gated_recurrence_workspace(rt.max_requests, rt.max_tokens, part.heads, part.key_dim,
                                                                         part.value_dim),), torch.float32)


class ChannelDecayAttention(SplitMixer):
    """spec: ``width``, ``heads``, ``key_dim``, ``value_dim``, ``decay_rank`` (rows of W_a1), ``tau``, ``eps`` (of the
    output norm).  Tensors: ``q``, ``k`` [heads * key_dim, width], ``v``, ``g`` [heads * value_dim, width], ``a1``
    [decay_rank, width], ``a2`` [heads * key_dim, decay_rank], ``a2.b``, ``norm`` [value_dim], ``o``."""

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        qk, vg, w = spec.heads * spec.key_dim, spec.heads * spec.value_dim, spec.width
        return {"q": TensorNeed((qk, w)), "k": TensorNeed((qk, w)), "v": TensorNeed((vg, w)), "g": TensorNeed((vg, w)),
                "a1": TensorNeed((spec.decay_rank, w)), "a2": TensorNeed((qk, spec.decay_rank)),
                "a2.b": TensorNeed((qk,), role="vector"), "norm": TensorNeed((spec.value_dim,), role="scale"),
                "o": TensorNeed((w, vg))}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.heads, self.key_dim, self.value_dim = int(spec.heads), int(spec.key_dim), int(spec.value_dim)
        self.rank, self.tau, self.eps = int(spec.decay_rank), float(spec.tau), float(spec.eps)
        if self.tau <= 0:
            raise ValueError(f"tau must be positive, got {self.tau}")
        self.qk_cols, self.vg_cols = self.heads * self.key_dim, self.heads * self.value_dim
        # one fused projection: rows [q | k | v | g | a1]
        self.in_weight = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"], tensors["a1"]], dim=0).contiguous()
        self.w_a2, self.a2_bias = tensors["a2"], tensors["a2.b"]
        self.norm_weight = tensors["norm"]
        self.w_o = tensors["o"]
        self.inner_cols, self.in_rows = self.vg_cols, 2 * self.qk_cols + 2 * self.vg_cols + self.rank

    def cache_need(self) -> FixedState:
        return FixedState((self.heads, self.key_dim, self.value_dim), "float32")

    def mix(self, proj, step, cache, writes_cache, into, out_scale: float = 1.0) -> None:
        n, rt = step.n, self.rt
        a, b = self.qk_cols, 2 * self.qk_cols
        c, d = b + self.vg_cols, b + 2 * self.vg_cols
        state = cache.state if cache.state is not None else cache.states["state"]
        z = rt.scratch("gla_decay_pre", (rt.max_tokens, self.qk_cols), torch.float32)[:n]
        ops.tag("scan_proj")
        ops.linear(proj[:, d:d + self.rank], self.w_a2, z)
        o = rt.scratch("linattn_out", (rt.max_tokens, self.vg_cols), torch.float32)[:n]
        ops.tag("linear_attention")
        ops.gated_recurrence(ops.RECURRENCE_CHANNEL_DECAY, proj[:, :a], proj[:, a:b], proj[:, b:c], z, self.a2_bias,
                             1.0 / self.tau, self.key_dim ** -0.5, state, step, o, self.heads, self.key_dim, self.value_dim,
                             writes_cache, workspace=_workspace(self, step))
        ops.tag("gate")
        ops.head_norm_gate_scaled(o, self.norm_weight, self.eps, proj[:, c:d], into, self.heads, self.value_dim, "silu", out_scale)


class MatrixMemory(SplitMixer):
    """spec: ``width``, ``heads``, ``key_dim``, ``value_dim``, ``gate_cap``, ``eps`` (of the output norm).  Tensors: ``q``,
    ``k`` [heads * key_dim, width], ``v``, ``g`` [heads * value_dim, width], ``i``, ``f`` [heads, width], ``i.b``, ``f.b``
    [heads], ``norm`` [heads * value_dim], ``o``."""

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        qk, vg, w, h = spec.heads * spec.key_dim, spec.heads * spec.value_dim, spec.width, spec.heads
        return {"q": TensorNeed((qk, w)), "k": TensorNeed((qk, w)), "v": TensorNeed((vg, w)), "g": TensorNeed((vg, w)),
                "i": TensorNeed((h, w)), "f": TensorNeed((h, w)), "i.b": TensorNeed((h,), role="vector"),
                "f.b": TensorNeed((h,), role="vector"), "norm": TensorNeed((vg,), role="scale"), "o": TensorNeed((w, vg))}

    # the gates read the mixer's input itself, in a product of their own with a float32 result
    needs_input = True

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.heads, self.key_dim, self.value_dim = int(spec.heads), int(spec.key_dim), int(spec.value_dim)
        self.cap, self.eps = float(spec.gate_cap), float(spec.eps)
        if self.cap <= 0:
            raise ValueError(f"gate_cap must be positive, got {self.cap}")
        self.qk_cols, self.vg_cols = self.heads * self.key_dim, self.heads * self.value_dim
        self.in_weight = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0).contiguous()
        self.w_gates = torch.cat([tensors["i"], tensors["f"]], dim=0).contiguous()          # rows [i | f]
        self.gate_bias = torch.cat([tensors["i.b"], tensors["f.b"]]).contiguous()
        self.norm_weight = tensors["norm"]
        self.w_o = tensors["o"]
        self.inner_cols, self.in_rows = self.vg_cols, 2 * self.qk_cols + 2 * self.vg_cols

    def cache_need(self) -> CacheBundle:
        h, d, dv = self.heads, self.key_dim, self.value_dim
        return CacheBundle.of(None, memory=FixedState((h, d, dv), "float32"), normalizer=FixedState((h, d), "float32"),
                              maximum=FixedState((h,), "float32"))

    def mix(self, proj, step, cache, writes_cache, into, out_scale: float = 1.0, h=None) -> None:
        if h is None:
            raise ValueError("the matrix memory's gates need the mixer's input")
        n, rt = step.n, self.rt
        a, b = self.qk_cols, 2 * self.qk_cols
        c, d = b + self.vg_cols, b + 2 * self.vg_cols
        gates = rt.scratch("memory_gates", (rt.max_tokens, pad8(2 * self.heads)), torch.float32)[:n, :2 * self.heads]
        ops.tag("scan_proj")
        ops.linear(h, self.w_gates, gates)
        o = rt.scratch("linattn_out", (rt.max_tokens, self.vg_cols), torch.float32)[:n]
        ops.tag("linear_attention")
        ops.gated_recurrence(ops.RECURRENCE_EXP_GATES, proj[:, :a], proj[:, a:b], proj[:, b:c], gates, self.gate_bias, self.cap,
                             self.key_dim ** -0.5, cache.states["memory"], step, o, self.heads, self.key_dim, self.value_dim,
                             writes_cache, cache.states["normalizer"], cache.states["maximum"], _workspace(self, step))
        ops.tag("gate")
        ops.head_norm_gate_scaled(o, self.norm_weight, self.eps, proj[:, c:d], into, self.heads, self.value_dim, "sigmoid", out_scale)


register_part("mixer", "channel_decay_attention", ChannelDecayAttention)
register_part("mixer", "matrix_memory", MatrixMemory)
