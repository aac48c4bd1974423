"""Plain, slow Pupinex decoder used as the oracle of the test-suite.

Whole sequences only, no cache, no batching, one function per mechanism, numpy float64 throughout, loops over
tokens where the definition is a recurrence.  It shares no code with the ``hfee_b200`` package: its own safetensors
reader and its own reading of config.json.

The design, in the notation used below (x: residual stream [T, width]; LN_*: layer norms with a weight and no bias):

    E = table[token] + bigram[hash(previous token, token)]              (the embedding output)
    per layer run (input x):  y = x + mixer(LN_1(x));  x = y + ffn(LN_2(y))   (the second only with a feed-forward)
    a stretch of layers runs several times over with the same weights; x += E in front of every pass but the first
    logits = table . LN_final(x)

Three mixers: ``attention`` (grouped-query softmax attention over a sliding window, with biases, an interleaved
partial rotation and a sink in the denominator), ``gla`` (linear attention whose state decays per key channel by a
gate computed from the token) and ``parallel`` (windowed softmax attention with normed queries and keys beside a
matrix memory with exponential gates).  Two feed-forwards: a clamped gated one, and routed experts whose router
scores are sigmoids and whose choice is limited to the best groups of experts, plus a gated shared expert.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

SWISH_ALPHA = 1.702
ROUTE_MARGINS = []           # per routed token: lowest chosen score minus the highest score left out (tests read it)


def read_safetensors(path):
    """name -> float64 (or integer) ndarray; bfloat16 is widened by a 16-bit shift."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    kinds = {"F64": "<f8", "F32": "<f4", "F16": "<f2", "I32": "<i4", "I64": "<i8"}
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = blob[lo:hi]
        if meta["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(raw, dtype=kinds[meta["dtype"]])
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float64)
        out[name] = arr.reshape(meta["shape"])
    return out


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# --------------------------------------------------------------------------
# one function per mechanism
# --------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def layer_norm(x, w, eps):
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: a hash of (previous, current); the first token takes the last row."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return np.asarray(rows)


def embed(tokens, table, bigram, bg):
    return table[np.asarray(tokens)] + bigram[bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])]


def rotate(x, dims, base, pairing, factor=1.0):
    """x: [T, heads, dim]; the first ``dims`` dimensions of each head are rotated by the token's position.
    ``interleaved`` pairs (2i, 2i+1), ``half`` pairs (i, i + dims/2); every frequency is divided by ``factor``."""
    T = x.shape[0]
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)]) / factor
    a = np.arange(T)[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    out = x.copy()
    if pairing == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def windowed_softmax_attention(q, k, v, scale, window, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Token i sees j with 0 <= i - j < window.  ``sink``
    [H]: one more term exp(sink_h) in the denominator that has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = s.max() if sink is None else max(s.max(), sink[h])
            e = np.exp(s - m)
            den = e.sum() + (0.0 if sink is None else math.exp(sink[h] - m))
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def sink_attention_mixer(h, T_, p, m):
    """The ``attention`` mixer: biases on q, k, v and o, interleaved partial rotation, window, sink."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ T_[p + "q"].T + T_[p + "q.b"]).reshape(T, H, d)
    k = (h @ T_[p + "k"].T + T_[p + "k.b"]).reshape(T, G, d)
    v = (h @ T_[p + "v"].T + T_[p + "v.b"]).reshape(T, G, dv)
    rot = m["rot"]
    q = rotate(q, rot["dims"], rot["base"], "interleaved")
    k = rotate(k, rot["dims"], rot["base"], "interleaved")
    o = windowed_softmax_attention(q, k, v, m["scale"], m["mask"]["size"], sink=T_[p + "sink"])
    return o.reshape(T, H * dv) @ T_[p + "o"].T + T_[p + "o.b"]


def normed_attention_branch(h, T_, p, m, eps):
    """The parallel mixer's left branch: biases on q, k, v; RMS norm with a weight over the whole q and the whole k
    projection before the rotation; rotate-half partial rotation with linearly scaled frequencies; window."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ T_[p + "q"].T + T_[p + "q.b"]
    k = h @ T_[p + "k"].T + T_[p + "k.b"]
    v = (h @ T_[p + "v"].T + T_[p + "v.b"]).reshape(T, G, dv)
    q = (unit_rms(q, eps) * T_[p + "q.norm"]).reshape(T, H, d)
    k = (unit_rms(k, eps) * T_[p + "k.norm"]).reshape(T, G, d)
    rot = m["rot"]
    factor = (rot.get("scaling") or {}).get("factor", 1.0)
    q = rotate(q, rot["dims"], rot["base"], "half", factor)
    k = rotate(k, rot["dims"], rot["base"], "half", factor)
    o = windowed_softmax_attention(q, k, v, m["scale"], m["mask"]["size"])
    return o.reshape(T, H * dv) @ T_[p + "o"].T


def channel_decay_recurrence(q, k, v, alpha):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t.  q, k, alpha [T, H, d], v [T, H, dv]."""
    T, H, d = q.shape
    dv = v.shape[2]
    o = np.zeros((T, H, dv))
    for h in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = alpha[t, h][:, None] * S + np.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ q[t, h]
    return o


def gla_mixer(h, T_, p, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ T_[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ T_[p + "k"].T).reshape(T, H, d)
    v = (h @ T_[p + "v"].T).reshape(T, H, dv)
    z = (h @ T_[p + "a1"].T) @ T_[p + "a2"].T + T_[p + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, d)
    o = channel_decay_recurrence(q, k, v, alpha)
    o = unit_rms(o, eps) * T_[p + "norm"]                      # per head, over vdim; one weight for all heads
    return (o.reshape(T, H * dv) * silu(h @ T_[p + "g"].T)) @ T_[p + "o"].T


def matrix_memory(q, k, v, i_gate, f_gate):
    """Exponentially gated matrix memory with a running maximum that starts at 0.  q, k [T, H, d], v [T, H, dv],
    i_gate, f_gate [T, H] (logarithms of the input and forget gates)."""
    T, H, d = q.shape
    dv = v.shape[2]
    o = np.zeros((T, H, dv))
    for h in range(H):
        S, n, m = np.zeros((d, dv)), np.zeros(d), 0.0
        for t in range(T):
            m_new = max(f_gate[t, h] + m, i_gate[t, h])
            a, b = math.exp(f_gate[t, h] + m - m_new), math.exp(i_gate[t, h] - m_new)
            S = a * S + b * np.outer(k[t, h], v[t, h])
            n = a * n + b * k[t, h]
            m = m_new
            o[t, h] = S.T @ q[t, h] / (max(abs(n @ q[t, h]), math.exp(-m)) + 1e-6)
    return o


def matrix_memory_branch(h, T_, p, m, eps):
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ T_[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ T_[p + "k"].T).reshape(T, H, d)
    v = (h @ T_[p + "v"].T).reshape(T, H, dv)
    i_gate = cap * np.tanh((h @ T_[p + "i"].T + T_[p + "i.b"]) / cap)
    f_gate = log_sigmoid(cap * np.tanh((h @ T_[p + "f"].T + T_[p + "f.b"]) / cap))
    o = unit_rms(matrix_memory(q, k, v, i_gate, f_gate), eps).reshape(T, H * dv)
    return (o * T_[p + "norm"] * sigmoid(h @ T_[p + "g"].T)) @ T_[p + "o"].T


def parallel_mixer(h, T_, p, m, eps):
    return (m["left_scale"] * normed_attention_branch(h, T_, p + "left.", m["left"], eps)
            + m["right_scale"] * matrix_memory_branch(h, T_, p + "right.", m["right"], eps))


def clamped_ffn(h, T_, p, limit):
    g = np.minimum(h @ T_[p + "gate"].T, limit)
    u = np.clip(h @ T_[p + "up"].T, -limit, limit)
    return (g * sigmoid(SWISH_ALPHA * g) * (u + 1.0)) @ T_[p + "down"].T


def silu_expert(h, T_, p):
    return (silu(h @ T_[p + "gate"].T) * (h @ T_[p + "up"].T)) @ T_[p + "down"].T


def group_limited_choice(s, top, groups, keep):
    """s [experts] -> indices of the ``top`` largest among the experts of the ``keep`` best groups (a group's score
    is the sum of its two largest).  Ties go to the lower index."""
    E = len(s)
    size = E // groups
    gs = []
    for g in range(groups):
        part = np.sort(s[g * size:(g + 1) * size])[::-1]
        gs.append(part[:2].sum())
    best = sorted(range(groups), key=lambda g: (-gs[g], g))[:keep]
    allowed = [e for e in range(E) if e // size in best]
    return sorted(allowed, key=lambda e: (-s[e], e))[:top]


def routed_ffn(h, T_, p, f):
    r = f["router"]
    T = h.shape[0]
    z = h @ T_[p + "router"].T
    s = sigmoid(z)
    out = np.zeros((T, T_[p + "e0.down"].shape[0]))
    for t in range(T):
        groups = r.get("groups") or {"count": 1, "keep": 1}
        chosen = group_limited_choice(s[t], r["top"], groups["count"], groups["keep"])
        left_out = [s[t, e] for e in range(len(s[t])) if e not in chosen]
        ROUTE_MARGINS.append(min(s[t, chosen]) - max(left_out) if left_out else 1.0)
        w = s[t, chosen] / (s[t, chosen].sum() + 1e-20) * r["scale"]
        for e, we in zip(chosen, w):
            out[t] += we * silu_expert(h[t:t + 1], T_, f"{p}e{e}.")[0]
    if f.get("shared") is not None:
        out += silu_expert(h, T_, p + "shared.") * sigmoid(h @ T_[p + "shared.sg"].T)
    return out


def feed_forward(h, T_, p, f):
    if f["kind"] == "dense":
        return clamped_ffn(h, T_, p, f["limit"])
    return routed_ffn(h, T_, p, f)


def run_order(cfg):
    """Layer indices in the order they run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for r in range(times):
        order += [(i, r > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg, T_, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence; ``layers_out`` (a list) receives the residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    e0 = embed(tokens, T_["embed"], T_["bigram"], cfg["embedding"]["bigram"])
    x = e0.copy()
    for i, add_embedding in run_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        if add_embedding:
            x = x + e0
        h = layer_norm(x, T_[p + "norm1"], eps)
        if layer["type"] == "attention":
            x = x + sink_attention_mixer(h, T_, p + "mix.", layer["mixer"])
        elif layer["type"] == "gla":
            x = x + gla_mixer(h, T_, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            x = x + parallel_mixer(h, T_, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + feed_forward(layer_norm(x, T_[p + "norm2"], eps), T_, p + "mlp.", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.copy())
    return layer_norm(x, T_["final.norm"], eps) @ T_["embed"].T


def greedy(cfg, T_, prompt, n):
    """``n`` tokens after ``prompt``, each the argmax (lowest id on ties) of the logits at the last position."""
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(np.argmax(forward(cfg, T_, seq)[-1])))
    return seq[len(prompt):]
