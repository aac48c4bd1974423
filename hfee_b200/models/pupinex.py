"""The Pupinex decoder as an arrangement of parts.

    E = table[token] + pairs[hash(previous token, token)]
    layer run (input x):  y = x + mixer(LN_1(x));  x = y + ffn(LN_2(y))          (the second only with a feed-forward)
    layers loop.start .. loop.stop - 1 run loop.times times in a row with the same weights, a cache of its own per
    pass, and x += E right in front of every pass but the first
    logits = table . LN_final(x)

Layer i's tensors are named ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*`` and ``l<i>.mlp.*``; model level: ``embed``,
``bigram``, ``final.norm``.
"""
from __future__ import annotations

from ..config.llama import LinearRopeScaling
from ..config.pupinex import PupinexConfig, fill_from_tensors
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunSpec

SWISH_ALPHA = 1.702          # fixed by the design: g * sigmoid(1.702 g) in the dense feed-forward


def _attention(cfg: PupinexConfig, a, pairing: str, **options) -> PartSpec:
    scaling = LinearRopeScaling(a.rot.factor) if a.rot.factor != 1.0 else None
    position = (PartSpec("rotary", head_dim=a.dim, rope_dim=a.rot.dims, theta=a.rot.base, scaling=scaling, pairing=pairing)
                if a.rot.dims > 0 else PartSpec("none"))
    return PartSpec("softmax_attention", width=cfg.width, heads=a.heads, kv_heads=a.kv_heads, head_dim=a.dim, value_dim=a.vdim,
                    scale=a.scale, window=a.window, position=position, **options)


def _mixer(cfg: PupinexConfig, layer, p: str):
    m = layer.mixer
    if layer.type == "attention":
        spec = _attention(cfg, m, "interleaved", biases=("q", "k", "v", "o"), sink=True)
        keys = ("q", "q.b", "k", "k.b", "v", "v.b", "o", "o.b", "sink")
        return spec, {"mixer." + k: p + "mix." + k for k in keys}
    if layer.type == "gla":
        spec = PartSpec("channel_decay_attention", width=cfg.width, heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
                        decay_rank=m.rank, tau=m.tau, eps=cfg.eps)
        return spec, {"mixer." + k: p + "mix." + k for k in ("q", "k", "v", "g", "a1", "a2", "a2.b", "norm", "o")}
    left = _attention(cfg, m.left, "half", biases=("q", "k", "v"), qk_norm="whole", qk_norm_eps=cfg.eps)
    right = PartSpec("matrix_memory", width=cfg.width, heads=m.right.heads, key_dim=m.right.dim, value_dim=m.right.vdim,
                     gate_cap=m.right.gate_cap, eps=cfg.eps)
    spec = PartSpec("parallel", width=cfg.width, left=left, right=right, left_scale=m.left_scale, right_scale=m.right_scale)
    names = {"mixer.left." + k: p + "mix.left." + k for k in ("q", "q.b", "k", "k.b", "v", "v.b", "q.norm", "k.norm", "o")}
    names.update({"mixer.right." + k: p + "mix.right." + k for k in ("q", "k", "v", "g", "i", "i.b", "f", "f.b", "norm", "o")})
    return spec, names


def _feed_forward(cfg: PupinexConfig, f, p: str):
    from ..config.pupinex import DenseMlp
    if isinstance(f, DenseMlp):
        spec = PartSpec("clamped_glu", width=cfg.width, inner=f.ff, limit=f.limit, alpha=SWISH_ALPHA, shift=1.0)
        return spec, {"ffn." + k: p + "mlp." + k for k in ("gate", "up", "down")}
    # experts: silu(gate) * up, the clamped gated form without a clamp, alpha = 1 and no shift
    spec = PartSpec("routed_experts", width=cfg.width, experts=f.experts, top=f.top, router_scale=f.router_scale, inner=f.ff,
                    limit=None, alpha=1.0, shift=0.0, router="sigmoid_groups", groups=f.groups, keep=f.keep,
                    shared_inner=f.shared_ff, shared_limit=None, shared_gate=f.shared_ff is not None)
    names = {"ffn.router": p + "mlp.router"}
    for e in range(f.experts):
        for k in ("gate", "up", "down"):
            names[f"ffn.e{e}.{k}"] = f"{p}mlp.e{e}.{k}"
    if f.shared_ff is not None:
        for k in ("gate", "up", "down", "sg"):
            names[f"ffn.shared.{k}"] = f"{p}mlp.shared.{k}"
    return spec, names


def run_order(cfg: PupinexConfig):
    """The schedule: every layer in order, the looped stretch ``times`` times with a cache of its own per pass; the
    first run of every pass but the first takes the embedding's output on top."""
    n = len(cfg.layers)
    loop = cfg.loop
    if loop is None or loop.stop == loop.start:
        return ModelSpec.sequential(n)
    runs = [(i, False) for i in range(loop.start)]
    for r in range(loop.times):
        runs += [(i, r > 0 and i == loop.start) for i in range(loop.start, loop.stop)]
    runs += [(i, False) for i in range(loop.stop, n)]
    return tuple(RunSpec(layer=i, cache=j, adds_embedding=add) for j, (i, add) in enumerate(runs))


def pupinex_spec(cfg: PupinexConfig) -> ModelSpec:
    norm = PartSpec("layer_norm", width=cfg.width, eps=cfg.eps)
    block = PartSpec("pre_norm", width=cfg.width)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mixer, names = _mixer(cfg, layer, p)
        names["mixer_norm.weight"] = p + "norm1"
        parts = {"mixer": ("mixer", mixer), "mixer_norm": ("norm", norm)}
        if layer.mlp is not None:
            ffn, ffn_names = _feed_forward(cfg, layer.mlp, p)
            parts["ffn"], parts["ffn_norm"] = ("feed_forward", ffn), ("norm", norm)
            names.update(ffn_names)
            names["ffn_norm.weight"] = p + "norm2"
        layers.append(LayerSpec(block, parts, names))
    return ModelSpec(
        width=cfg.width, vocab=cfg.vocab,
        embedding=PartSpec("token_bigram", vocab=cfg.vocab, width=cfg.width, buckets=cfg.buckets, mul_prev=cfg.mul_prev,
                           mul_cur=cfg.mul_cur),
        layers=tuple(layers), schedule=run_order(cfg), final_norm=norm,
        head=PartSpec("linear", vocab=cfg.vocab, width=cfg.width, tied=True),
        names={"embedding.table": "embed", "embedding.pairs": "bigram", "final_norm.weight": "final.norm"},
        max_positions=cfg.max_positions)


register_architecture("Pupinex", PupinexConfig.from_dict, pupinex_spec, fill_from_tensors)
