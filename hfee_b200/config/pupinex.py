"""Typed configuration of the Pupinex decoder, read from its config.json.

A Pupinex model adds a hashed embedding of (previous token, token) to its token embedding, runs a list of pre-norm
layers (layer norms with a weight and no bias), of which a stretch may run several times over with the same weights
(``loop``; the embedding's output is added again in front of every further pass), and ties its head to the embedding
table.  Each layer has one of three mixers (``attention``: windowed grouped-query softmax attention with biases, an
interleaved partial rotation and a sink; ``gla``: linear attention with a decay per key channel; ``parallel``: windowed
attention with normed queries and keys beside a matrix memory with exponential gates) and an optional feed-forward
(``dense``: a clamped gated one; ``moe``: routed experts with sigmoid scores and a choice limited to groups, plus an
optional gated shared expert).  Every size and every constant that differs between models comes from config.json or a
tensor's shape; nothing here has a default that a model could silently fall back on.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .dobelix import _get, _int, _num
from .llama import ConfigError


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    factor: float            # every frequency is divided by it (1: no scaling)


@dataclass(frozen=True)
class WindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot: Rotation


@dataclass(frozen=True)
class ChannelDecay:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int                # rows of the decay's low-rank projection (from the tensor's shape)


@dataclass(frozen=True)
class MatrixMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ParallelMixer:
    left: WindowAttention
    right: MatrixMemory
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DenseMlp:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    groups: int
    keep: int
    router_scale: float
    ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class PupinexLayer:
    type: str
    mixer: Any
    mlp: Any                 # DenseMlp, MoeMlp or None


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class PupinexConfig:
    vocab: int
    width: int
    layers: Tuple[PupinexLayer, ...]
    loop: Optional[Loop]
    eps: float
    buckets: int
    mul_prev: int
    mul_cur: int
    max_positions: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "PupinexConfig":
        layers = _get(d, "layers", "config")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            m = _get(entry, "mixer", where)
            mw = where + ".mixer"
            if kind == "attention":
                mixer = _attention(m, mw)
            elif kind == "gla":
                rank = m.get("rank") if isinstance(m, Mapping) else None
                if rank is None:
                    raise ConfigError(f"config.json: {mw}: the decay's rank is neither given nor known from the tensor l{i}.mix.a1")
                mixer = ChannelDecay(_int(m, "heads", mw), _int(m, "dim", mw), _int(m, "vdim", mw), _positive(m, "tau", mw), int(rank))
            elif kind == "parallel":
                right = _get(m, "right", mw)
                rw = mw + ".right"
                mixer = ParallelMixer(_attention(_get(m, "left", mw), mw + ".left"),
                                      MatrixMemory(_int(right, "heads", rw), _int(right, "dim", rw), _int(right, "vdim", rw),
                                                   _positive(right, "gate_cap", rw)),
                                      _num(m, "left_scale", mw), _num(m, "right_scale", mw))
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design (known: attention, gla, parallel)")
            out.append(PupinexLayer(kind, mixer, _mlp(entry.get("mlp") if isinstance(entry, Mapping) else None, where + ".mlp")))
        loop = d.get("loop")
        if loop is not None:
            loop = Loop(_count(loop, "start", "loop"), _count(loop, "stop", "loop"), _int(loop, "times", "loop"))
            if not (0 <= loop.start <= loop.stop <= len(out)) or loop.times < 1:
                raise ConfigError(f"config.json: loop {loop.start}..{loop.stop} x {loop.times} does not fit {len(out)} layers")
        bigram = _get(_get(d, "embedding", "config"), "bigram", "embedding")
        buckets = _int(bigram, "buckets", "embedding.bigram")
        if buckets < 1:
            raise ConfigError(f"config.json: embedding.bigram.buckets must be positive, got {buckets}")
        max_positions = d.get("max_positions", d.get("max_position_embeddings", 1 << 20))
        return cls(vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"), layers=tuple(out), loop=loop,
                   eps=_num(_get(d, "norm", "config"), "eps", "norm"), buckets=buckets,
                   mul_prev=_int(bigram, "mul_prev", "embedding.bigram"), mul_cur=_int(bigram, "mul_cur", "embedding.bigram"),
                   max_positions=int(max_positions))


def _count(d: Mapping[str, Any], key: str, where: str) -> int:
    """An integer that may be zero."""
    v = _get(d, key, where)
    if not isinstance(v, int) or isinstance(v, bool) or v < 0:
        raise ConfigError(f"config.json: {where}.{key} must be a non-negative integer, got {v!r}")
    return v


def _positive(d: Mapping[str, Any], key: str, where: str) -> float:
    v = _num(d, key, where)
    if v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


def _attention(m: Mapping[str, Any], where: str) -> WindowAttention:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if kv < 1 or heads % kv:
        raise ConfigError(f"config.json: {where}.heads {heads} must be a multiple of kv_heads {kv}")
    dim = _int(m, "dim", where)
    rot = m.get("rot")
    if rot is None:                      # no rotation at all
        rotation = Rotation(0, 1.0, 1.0)
    else:
        dims = _count(rot, "dims", where + ".rot")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most dim {dim}")
        scaling = rot.get("scaling")
        factor = 1.0 if scaling is None else _positive(scaling, "factor", where + ".rot.scaling")
        rotation = Rotation(dims, _positive(rot, "base", where + ".rot") if dims else 1.0, factor)
    mask = m.get("mask")
    window = None if mask is None else _int(mask, "size", where + ".mask")       # no mask: every earlier position
    return WindowAttention(heads, kv, dim, _int(m, "vdim", where), _num(m, "scale", where), window, rotation)


def _mlp(mlp: Optional[Mapping[str, Any]], where: str):
    if mlp is None:
        return None
    kind = _get(mlp, "kind", where)
    if kind == "dense":
        return DenseMlp(_int(mlp, "ff", where), _positive(mlp, "limit", where))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design (known: dense, moe)")
    router = _get(mlp, "router", where)
    rw = where + ".router"
    experts, top = _int(router, "experts", rw), _int(router, "top", rw)
    groups = router.get("groups")
    count, keep = (1, 1) if groups is None else (_int(groups, "count", rw + ".groups"), _int(groups, "keep", rw + ".groups"))
    if count < 1 or experts % count or not 1 <= keep <= count:
        raise ConfigError(f"config.json: {rw}: {experts} experts do not form {count} equal groups of which {keep} are kept")
    if not 1 <= top <= keep * (experts // count):
        raise ConfigError(f"config.json: {rw}.top {top} is outside 1..{keep * (experts // count)} (the experts of the kept groups)")
    shared = mlp.get("shared")
    return MoeMlp(experts, top, count, keep, _num(router, "scale", rw), _int(_get(mlp, "expert", where), "ff", where + ".expert"),
                  None if shared is None else _int(shared, "ff", where + ".shared"))


def fill_from_tensors(config_json: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Mapping[str, Any]:
    """config.json does not name the rank of a ``gla`` layer's decay projection: it is the row count of the layer's
    ``mix.a1`` tensor."""
    layers = config_json.get("layers")
    if not isinstance(layers, (list, tuple)):
        return config_json
    out = dict(config_json)
    new_layers = []
    for i, entry in enumerate(layers):
        if isinstance(entry, Mapping) and entry.get("type") == "gla" and isinstance(entry.get("mixer"), Mapping) \
                and "rank" not in entry["mixer"] and f"l{i}.mix.a1" in shapes:
            entry = dict(entry)
            entry["mixer"] = dict(entry["mixer"], rank=int(shapes[f"l{i}.mix.a1"][0]))
        new_layers.append(entry)
    out["layers"] = new_layers
    return out
