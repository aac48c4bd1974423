"""The Muvetar decoder as an arrangement of parts.

    X_0 = table[token] + sinusoid(position)
    layer i (input x):  y = x + m * mixer(norm1(x));  X_(i+1) = y + m * ffn(norm2(y))   (the second only with a feed-forward)
                        x = sum_(j <= i+1) a_i[j] X_j
    logits = cap * tanh(head(norm(x)) / cap)

Layer i's tensors are named ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*`` and ``l<i>.dwa`` (the i + 2
weights a_i); model level: ``embed``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.muvetar import MuvetarConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec

SINUSOID_BASE = 10000.0      # fixed by the design
SWISH_ALPHA = 1.702          # fixed by the design: g * sigmoid(1.702 g)


def _mixer(cfg: MuvetarConfig, layer, p: str):
    m = layer.mixer
    if layer.type == "mingru":
        spec = PartSpec("mingru", width=cfg.width, channels=m.width)
        return spec, {"mixer." + k: p + "mix." + s for k, s in
                      (("z", "z"), ("z_bias", "z.b"), ("x", "x"), ("x_bias", "x.b"), ("g", "g"), ("o", "o"))}
    left = PartSpec("distance_attention", width=cfg.width, heads=m.left.heads, kv_heads=m.left.kv_heads, head_dim=m.left.dim,
                    value_dim=m.left.vdim, scale=m.left.scale)
    right = PartSpec("selective_scan", width=cfg.width, inner=m.right.inner, state=m.right.state, dt_rank=m.right.dt_rank,
                     taps=m.right.taps)
    spec = PartSpec("parallel", width=cfg.width, left=left, right=right, left_scale=m.left_scale, right_scale=m.right_scale)
    names = {"mixer.left." + k: p + "mix.left." + k for k in ("q", "k", "v", "r1", "r2", "o")}
    names.update({"mixer.right." + k: p + "mix.right." + s for k, s in
                  (("in", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("x", "x"), ("dt", "dt"), ("dt_bias", "dt.b"),
                   ("A_log", "A_log"), ("D", "D"), ("o", "o"))})
    return spec, names


def muvetar_spec(cfg: MuvetarConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", width=cfg.width, eps=cfg.eps)
    block = PartSpec("scaled_pre_norm", width=cfg.width, residual_scale=cfg.residual_mult)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mixer, names = _mixer(cfg, layer, p)
        names.update({"mixer_norm.weight": p + "norm1", "merge.weights": p + "dwa"})
        parts = {"mixer": ("mixer", mixer), "mixer_norm": ("norm", norm),
                 "merge": ("merge", PartSpec("depth_average", width=cfg.width, index=i, depth=len(cfg.layers)))}
        if layer.mlp is not None:
            f = layer.mlp
            shared = f.shared
            parts["ffn"] = ("feed_forward", PartSpec(
                "routed_experts", width=cfg.width, experts=f.experts, top=f.top, router_scale=f.router_scale, inner=f.expert.ff,
                limit=f.expert.limit, alpha=SWISH_ALPHA, shared_inner=None if shared is None else shared.ff,
                shared_limit=None if shared is None else shared.limit))
            parts["ffn_norm"] = ("norm", norm)
            names["ffn_norm.weight"] = p + "norm2"
            names["ffn.router"] = p + "mlp.router"
            for e in range(f.experts):
                for k in ("gate", "up", "down"):
                    names[f"ffn.e{e}.{k}"] = f"{p}mlp.e{e}.{k}"
            if shared is not None:
                for k in ("gate", "up", "down"):
                    names[f"ffn.shared.{k}"] = f"{p}mlp.shared.{k}"
        layers.append(LayerSpec(block, parts, names))
    return ModelSpec(
        width=cfg.width, vocab=cfg.vocab,
        embedding=PartSpec("token", vocab=cfg.vocab, width=cfg.width, sinusoid_base=SINUSOID_BASE),
        layers=tuple(layers), schedule=ModelSpec.sequential(len(layers)), final_norm=norm,
        head=PartSpec("linear", vocab=cfg.vocab, width=cfg.width, tied=False, softcap=cfg.logit_softcap),
        names={"embedding.table": "embed", "final_norm.weight": "final.norm", "head.weight": "head"},
        max_positions=cfg.max_positions)


register_architecture("Muvetar", MuvetarConfig.from_dict, muvetar_spec)
