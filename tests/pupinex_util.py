"""Small Pupinex configurations and helpers shared by the Pupinex tests."""
import json
import os

import numpy as np
import torch

from dobelix_util import make_runner, sequences  # noqa: F401  (the same engine settings and token draws)


def attn(heads, kv_heads, dim, vdim, scale, window, rot_dims, base, factor=None):
    rot = {"dims": rot_dims, "base": base}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}, "rot": rot}


def attention(heads, kv_heads, dim, vdim, scale, window, rot_dims, base, mlp=None):
    return {"type": "attention", "mixer": attn(heads, kv_heads, dim, vdim, scale, window, rot_dims, base), "mlp": mlp}


def gla(heads, dim, vdim, tau, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def parallel(left, heads, dim, vdim, gate_cap, left_scale=1.0, right_scale=1.0, mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap},
                      "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, groups, keep, ff, scale, shared_ff=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}},
         "expert": {"ff": ff}}
    if shared_ff is not None:
        m["shared"] = {"ff": shared_ff}
    return m


def config(width, vocab, layers, loop=None, eps=1e-5, buckets=97, mul_prev=31, mul_cur=7):
    c = {"architecture": "Pupinex", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
         "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


RANK = 6            # rows of a gla layer's decay projection in the test models (the file's tensor decides)

# Two configurations that differ from each other in every size and option.  A: a loop over the middle layers run three
# times, values wider than keys, a window shorter than a page, experts in three groups of which two are kept.  B: no
# loop, a layer without feed-forward, as many key/value heads as query heads, a whole head rotated, no frequency
# scaling, experts without a shared one, one group, one chosen expert, a window longer than the sequences.
PUP_A = config(64, 200, [
    parallel(attn(4, 2, 16, 24, 0.3, 21, 8, 1000.0, factor=2.0), 2, 16, 24, 8.0, 0.7, 1.2, mlp=dense(80, 1.5)),
    attention(4, 2, 24, 16, 0.25, 13, 12, 500.0, mlp=moe(6, 2, 3, 2, 24, 1.8, shared_ff=40)),
    gla(2, 16, 32, 8.0, mlp=dense(72, 0.9)),
    attention(2, 1, 32, 32, 0.2, 40, 32, 10000.0, mlp=moe(4, 1, 2, 1, 16, 2.5, shared_ff=24))],
    loop=(1, 3, 3), eps=1e-5, buckets=97, mul_prev=31, mul_cur=7)
PUP_B = config(96, 310, [
    gla(3, 24, 16, 3.0),
    attention(3, 3, 16, 40, 0.35, 500, 16, 77.0, mlp=moe(5, 3, 1, 1, 40, 0.9)),
    parallel(attn(6, 2, 16, 16, 0.2, 33, 16, 2.0e5), 3, 8, 48, 15.0, 1.5, 0.4),
    gla(1, 40, 56, 20.0, mlp=dense(64, 4.0))],
    loop=None, eps=1e-6, buckets=1, mul_prev=5, mul_cur=3)
STD = 0.15
MARK_A, MARK_B, MARK_LATER = 0, 1, 2      # embedding dimensions that mark the tokens of the far-token tests
ROUTE_AT = 3                              # first of the embedding dimensions that name a token's experts


def clear_routes(tensors, cfg, loud=8.0):
    """Make every router's choice a clear call, so that rounding cannot flip one.  Every layer with experts gets embedding
    dimensions of its own, one per expert, which its router reads with weight 1 (and everything else with a tenth of its
    random weight); token t is loud in the dimensions of ``top`` experts that lie in ``keep`` groups (which ones depends
    on t), and nothing else writes into those dimensions (no output projection, no bigram row).  Which experts are chosen
    is then settled; the norm in front and the other dimensions still move the scores, so the weights differ from token
    to token."""
    emb = tensors["embed"]
    at = ROUTE_AT
    for i, layer in enumerate(cfg["layers"]):
        if not layer.get("mlp") or layer["mlp"]["kind"] != "moe":
            continue
        r = layer["mlp"]["router"]
        experts, top, groups, keep = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"]
        size = experts // groups
        assert at + experts <= emb.shape[1], "the width has no room for every layer's marks"
        w = tensors[f"l{i}.mlp.router"]
        w.mul_(0.1)
        emb[:, at:at + experts] = 0.0
        for e in range(experts):
            w[e, at:at + experts] = 0.0
            w[e, at + e] = 1.0
        for t in range(emb.shape[0]):
            kept = [(t + j) % groups for j in range(keep)]
            for k in range(top):
                e = kept[k % keep] * size + (t + k // keep) % size
                emb[t, at + e] = loud
        at += experts
    tensors["bigram"][:, ROUTE_AT:at] = 0.0
    for name, t in tensors.items():          # no sublayer writes into the marks: they reach every router as the embedding left them
        if name.endswith((".o", ".down")):
            t[ROUTE_AT:at] = 0.0
        elif name.endswith(".o.b"):
            t[ROUTE_AT:at] = 0.0


def write_model(path, cfg, seed, dtype="bfloat16", edit=None, routes=True):
    """A model folder with random weights (stored in ``dtype``); ``edit(tensors)`` may change them first.  Gate biases,
    decay biases and sinks get values that spread over their useful ranges."""
    from hfee_b200.config.registry import resolve
    from hfee_b200.parts.model import model_tensor_needs
    from hfee_b200.weights.random_init import random_tensors
    from hfee_b200.weights.safetensors_io import write_file
    cfg_full = json.loads(json.dumps(cfg))
    for layer in cfg_full["layers"]:          # the registry learns the rank from the file; here there is no file yet
        if layer["type"] == "gla":
            layer["mixer"]["rank"] = RANK
    arch, typed = resolve(cfg_full)
    needs = model_tensor_needs(arch.build_spec(typed))
    tensors = random_tensors(needs, seed, torch.float32, STD)
    g = torch.Generator().manual_seed(seed)
    for name, t in tensors.items():
        if name.endswith(".sink"):
            t.copy_(torch.empty(t.shape).uniform_(-1.0, 3.0, generator=g))
        elif name.endswith(".a2.b"):
            t.copy_(torch.empty(t.shape).uniform_(-1.0, 5.0, generator=g))
        elif name.endswith(".f.b"):
            t.copy_(torch.empty(t.shape).uniform_(0.0, 5.0, generator=g))
        elif name.endswith(".i.b"):
            t.copy_(torch.empty(t.shape).uniform_(-2.0, 2.0, generator=g))
        elif name.endswith((".q.b", ".k.b", ".v.b", ".o.b")):
            t.copy_(torch.empty(t.shape).uniform_(-0.3, 0.3, generator=g))
        elif name.endswith((".a2", ".i", ".f")):
            t.mul_(4.0)                       # gates that move with the token
    if routes and any((l.get("mlp") or {}).get("kind") == "moe" for l in cfg["layers"]):
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
    """Tokens 0 and 1 (which the far-token tests put at chosen places only) carry a large entry in a dimension of their
    own, every other token in a third one, and nothing else: a projection can pick out "token A", "token B" and "any
    other token" by one column of its weight each.  The bigram rows are cleared so that nothing else enters the stream."""
    emb = tensors["embed"]
    emb[:, [MARK_A, MARK_B, MARK_LATER]] = 0.0
    emb[0, MARK_A] = size
    emb[1, MARK_B] = size
    emb[2:, MARK_LATER] = size
    tensors["bigram"].zero_()


def smallest_route_margin(plain, cfg, weights, seqs):
    """The smallest gap, over all routed tokens and layers, between a chosen expert's score and the best one left out."""
    del plain.ROUTE_MARGINS[:]
    for s in seqs:
        plain.forward(cfg, weights, s)
    return min(plain.ROUTE_MARGINS) if plain.ROUTE_MARGINS else float("inf")
