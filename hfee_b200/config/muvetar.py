"""Typed configuration of the Muvetar decoder, read from its config.json.

A Muvetar model adds sines and cosines of the position to its embedding, runs a list of layers, each with one
of two mixers (``mingru``: an elementwise gated recurrence; ``parallel``: softmax attention with a logarithmic
penalty on distance beside a selective state-space scan) and an optional mixture-of-experts feed-forward, scales
every sublayer's output by ``residual_mult``, hands each layer a learned average of all earlier layers' results,
and caps its logits.  Every size and every constant that differs between models comes from config.json; nothing
here has a default that a model could silently fall back on.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .dobelix import _get, _int, _num
from .llama import ConfigError


@dataclass(frozen=True)
class MinGruMixer:
    width: int


@dataclass(frozen=True)
class DistanceAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float


@dataclass(frozen=True)
class SelectiveScan:
    inner: int
    state: int
    dt_rank: int
    taps: int


@dataclass(frozen=True)
class ParallelMixer:
    left: DistanceAttention
    right: SelectiveScan
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class Expert:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    router_scale: float
    expert: Expert
    shared: Optional[Expert]


@dataclass(frozen=True)
class MuvetarLayer:
    type: str
    mixer: Any
    mlp: Optional[MoeMlp]


@dataclass(frozen=True)
class MuvetarConfig:
    vocab: int
    width: int
    layers: Tuple[MuvetarLayer, ...]
    eps: float
    residual_mult: float
    logit_softcap: float
    max_positions: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MuvetarConfig":
        layers = _get(d, "layers", "config")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            m = _get(entry, "mixer", where)
            mw = where + ".mixer"
            if kind == "mingru":
                mixer = MinGruMixer(_int(m, "width", mw))
            elif kind == "parallel":
                left, right = _get(m, "left", mw), _get(m, "right", mw)
                lw, rw = mw + ".left", mw + ".right"
                heads, kv = _int(left, "heads", lw), _int(left, "kv_heads", lw)
                if heads % kv:
                    raise ConfigError(f"config.json: {lw}.heads {heads} must be a multiple of kv_heads {kv}")
                mixer = ParallelMixer(
                    DistanceAttention(heads, kv, _int(left, "dim", lw), _int(left, "vdim", lw), _num(left, "scale", lw)),
                    SelectiveScan(_int(right, "inner", rw), _int(right, "state", rw), _int(right, "dt_rank", rw),
                                  _int(right, "conv", rw)),
                    _num(m, "left_scale", mw), _num(m, "right_scale", mw))
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design (known: mingru, parallel)")
            out.append(MuvetarLayer(kind, mixer, _mlp(entry.get("mlp") if isinstance(entry, Mapping) else None, where + ".mlp")))
        max_positions = d.get("max_positions", d.get("max_position_embeddings", 1 << 20))
        cap = _num(d, "logit_softcap", "config")
        if cap <= 0:
            raise ConfigError(f"config.json: logit_softcap must be positive, got {cap}")
        return cls(vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"), layers=tuple(out),
                   eps=_num(_get(d, "norm", "config"), "eps", "norm"), residual_mult=_num(d, "residual_mult", "config"),
                   logit_softcap=cap, max_positions=int(max_positions))


def _expert(e: Mapping[str, Any], where: str) -> Expert:
    limit = _num(e, "limit", where)
    if limit <= 0:
        raise ConfigError(f"config.json: {where}.limit must be positive, got {limit}")
    return Expert(_int(e, "ff", where), limit)


def _mlp(mlp: Optional[Mapping[str, Any]], where: str) -> Optional[MoeMlp]:
    if mlp is None:
        return None
    kind = _get(mlp, "kind", where)
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design (known: moe)")
    router = _get(mlp, "router", where)
    experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router.top {top} exceeds its {experts} experts")
    shared = mlp.get("shared")
    return MoeMlp(experts, top, _num(router, "scale", where + ".router"), _expert(_get(mlp, "expert", where), where + ".expert"),
                  None if shared is None else _expert(shared, where + ".shared"))
