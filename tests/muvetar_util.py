"""Small Muvetar configurations and helpers shared by the Muvetar tests."""
import json
import os

import numpy as np
import torch

from dobelix_util import make_runner, sequences  # noqa: F401  (the same engine settings and token draws)


def moe(experts, top, ff, limit, scale, shared_ff=None, shared_limit=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff, "limit": limit}}
    if shared_ff is not None:
        m["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return m


def mingru(width, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def parallel(heads, kv_heads, dim, vdim, scale, inner, state, dt_rank, conv, left_scale=1.0, right_scale=1.0, mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale},
                      "right": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv},
                      "left_scale": left_scale, "right_scale": right_scale}}


def config(width, vocab, layers, eps=1e-5, residual_mult=0.5, softcap=15.0):
    return {"architecture": "Muvetar", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
            "residual_mult": residual_mult, "logit_softcap": softcap}


# Two configurations that differ from each other in every size and option: B has a layer without feed-forward, experts
# without a shared one, one chosen expert, as many key/value heads as query heads, a convolution of one tap and of
# five, values smaller than keys, a residual multiplier of 1 and other constants everywhere.
MUV_A = config(64, 200, [parallel(4, 2, 16, 24, 0.25, 48, 6, 5, 3, 1.3, 0.8, mlp=moe(8, 2, 24, 1.0, 2.0, 40, 1.5)),
                         mingru(80, mlp=moe(8, 2, 24, 1.0, 2.0, 40, 1.5)),
                         mingru(40),
                         parallel(2, 1, 32, 16, 0.2, 72, 16, 4, 4, 0.7, 1.2, mlp=moe(5, 3, 16, 2.0, 1.0))],
               eps=1e-5, residual_mult=0.5, softcap=15.0)
MUV_B = config(96, 310, [mingru(96, mlp=moe(4, 1, 40, 0.7, 1.5, 24, 3.0)),
                         parallel(3, 3, 24, 8, 0.3, 64, 3, 9, 1, 1.0, 1.0),
                         parallel(6, 2, 16, 16, 0.11, 100, 20, 2, 5, 2.0, 0.5, mlp=moe(12, 4, 8, 1.2, 3.0)),
                         mingru(56, mlp=moe(3, 3, 32, 5.0, 0.5, 8, 0.4)),
                         mingru(120)],
               eps=1e-6, residual_mult=1.0, softcap=4.0)
STD = 0.15
MARK_A, MARK_B, MARK_LATER = 0, 1, 2      # embedding dimensions that mark the tokens of the far-token tests
ROUTE_AT = 3                              # first of the embedding dimensions that name a token's experts


def clear_routes(tensors, cfg, loud=6.0):
    """Make every router's choice a clear call, so that rounding cannot flip one.  Every layer with experts gets
    embedding dimensions of its own, one per expert, which its router reads with weight 1 (and everything else with
    a tenth of its random weight); token t is loud in the dimensions of the ``top`` experts from t % experts on
    (cyclically), and no sublayer's output projection writes into those dimensions.  Which experts are chosen is then
    settled; positions, mixers and earlier layers still move the scores, so the chosen experts' weights differ from
    token to token."""
    emb = tensors["embed"]
    at = ROUTE_AT
    for i, layer in enumerate(cfg["layers"]):
        if not layer.get("mlp"):
            continue
        r = layer["mlp"]["router"]
        experts, top = r["experts"], r["top"]
        assert at + experts <= emb.shape[1], "the width has no room for every layer's marks"
        w = tensors[f"l{i}.mlp.router"]
        w.mul_(0.1)
        emb[:, at:at + experts] = 0.0
        for e in range(experts):
            w[e, at:at + experts] = 0.0
            w[e, at + e] = 1.0
        for t in range(emb.shape[0]):
            for k in range(top):
                emb[t, at + (t + k) % experts] = loud
        at += experts
    for name, t in tensors.items():          # no sublayer writes into the marks: they reach every router as the embedding left them
        if name.endswith((".o", ".down")):
            t[ROUTE_AT:at] = 0.0


def write_model(path, cfg, seed, dtype="bfloat16", edit=None, routes=True):
    """A model folder with random weights (stored in ``dtype``); ``edit(tensors)`` may change them first.  Decays, step
    sizes and distance penalties get values that spread over their useful ranges."""
    from hfee_b200.config.registry import resolve
    from hfee_b200.parts.model import model_tensor_needs
    from hfee_b200.weights.random_init import random_tensors
    from hfee_b200.weights.safetensors_io import write_file
    arch, typed = resolve(cfg)
    needs = model_tensor_needs(arch.build_spec(typed))
    tensors = random_tensors(needs, seed, torch.float32, STD)
    g = torch.Generator().manual_seed(seed)
    for name, t in tensors.items():
        if name.endswith("right.A_log"):
            t.copy_(torch.empty(t.shape).uniform_(-4.0, 1.0, generator=g))
        elif name.endswith("right.dt.b"):
            t.copy_(torch.empty(t.shape).uniform_(-3.0, 1.0, generator=g))
        elif name.endswith("left.r1"):
            t.copy_(torch.empty(t.shape).uniform_(0.1, 1.5, generator=g))
        elif name.endswith("left.r2"):
            t.copy_(torch.empty(t.shape).uniform_(0.02, 2.0, generator=g))
        elif name.endswith(".dwa"):
            t.copy_(torch.empty(t.shape).uniform_(0.1, 0.9, generator=g))
    if routes and any(l.get("mlp") for l in cfg["layers"]):
        clear_routes(tensors, cfg)
    if edit is not None:
        edit(tensors)
    store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(path, "model.safetensors"), {k: v.to(store).contiguous() for k, v in tensors.items()})
    return path


def mark_first_tokens(tensors, size=1.0):
    """Tokens 0 and 1 (which the far-token tests put at the start of a sequence only) carry a large entry in a dimension
    of their own, every other token in a third one, and nothing else: a projection can pick out "first token A",
    "first token B" and "any later token" by one column of its weight each."""
    emb = tensors["embed"]
    emb[:, [MARK_A, MARK_B, MARK_LATER]] = 0.0
    emb[0, MARK_A] = size
    emb[1, MARK_B] = size
    emb[2:, MARK_LATER] = size


def smallest_route_margin(plain, cfg, weights, seqs):
    """The smallest gap, over all tokens and layers, between a chosen expert's router logit and the best one left out."""
    del plain.ROUTE_MARGINS[:]
    for s in seqs:
        plain.forward(cfg, weights, s)
    return min(plain.ROUTE_MARGINS) if plain.ROUTE_MARGINS else float("inf")
