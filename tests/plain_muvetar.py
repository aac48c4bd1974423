"""Plain, slow Muvetar decoder used as the oracle of the test-suite.

Whole sequences only, no cache, no batching, one function per mechanism, numpy
float64 throughout, loops over tokens where the definition is a recurrence.  It
shares no code with the ``hfee_b200`` package: its own safetensors reader and its own
reading of config.json.

The design, in the notation used below (x: residual stream [T, width]; N_* RMS norms with a weight):

    X_0 = table[token] + sinusoid(position)
    per layer i (input x):  y = x + m * mixer(N_1(x));  X_(i+1) = y + m * moe(N_2(y))
                            x = sum_(j <= i+1) a_i[j] X_j            (what the next layer, or the output, reads)
    logits = cap * tanh(W_head N_final(x) / cap)

Two mixers: ``mingru`` (an elementwise gated recurrence with an output gate) and ``parallel`` (softmax
attention with a logarithmic distance penalty beside a selective state-space scan behind a short
convolution, their outputs added with one weight each).  The feed-forward is a routed mixture of small
clamped gated experts plus one shared expert.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


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
def rms_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def sinusoid(T, width, first=0):
    """[T, width]: column 2i is sin(p * 10000^(-2i/width)), column 2i+1 the cosine of the same angle."""
    out = np.zeros((T, width))
    p = np.arange(first, first + T, dtype=np.float64)[:, None]
    for c in range(width):
        i = c // 2
        angle = p[:, 0] * 10000.0 ** (-2.0 * i / width)
        out[:, c] = np.sin(angle) if c % 2 == 0 else np.cos(angle)
    return out


def mingru(h, W, p, m):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t per channel; out = W_o (S_t * silu(W_g h_t))."""
    z = sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    gate = silu(h @ W[p + "g"].T)
    S = np.zeros(m["width"])
    out = np.zeros((h.shape[0], m["width"]))
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out[t] = S * gate[t]
    return out @ W[p + "o"].T


def distance_attention(h, W, p, m):
    """Causal grouped-query softmax attention; the score of key j for query i is
    q.k * scale - r1_h * ln(1 + r2_h * (i - j))."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, d)
    k = (h @ W[p + "k"].T).reshape(T, G, d)
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    r1, r2 = W[p + "r1"], W[p + "r2"]
    out = np.zeros((T, H, dv))
    dist = np.arange(T)[:, None] - np.arange(T)[None, :]
    visible = dist >= 0
    far = np.where(visible, dist, 0).astype(np.float64)
    for hd in range(H):
        g = hd // (H // G)
        s = q[:, hd] @ k[:, g].T * m["scale"] - r1[hd] * np.log(1.0 + r2[hd] * far)
        s = np.where(visible, s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        w = np.exp(s)
        w /= w.sum(axis=1, keepdims=True)
        out[:, hd] = w @ v[:, g]
    return out.reshape(T, H * dv) @ W[p + "o"].T


def causal_conv(x, w, b):
    """y[t, c] = b[c] + sum_j w[c, j] x[t - taps + 1 + j, c], zeros in front of the sequence."""
    T, taps = x.shape[0], w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, x.shape[1])), x], axis=0)
    y = np.zeros_like(x)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j]
    return y + b


def selective_scan(h, W, p, m):
    """x, z = W_in h; x = silu(conv(x)); dt, B, C = W_x x; dt = softplus(W_dt dt + b);
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n; y_c = sum_n S[c, n] C_n + D_c x_c; out = W_o (y * silu(z))."""
    T = h.shape[0]
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ W[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    low = x @ W[p + "x"].T
    dt, B, C = low[:, :R], low[:, R:R + N], low[:, R + N:]
    dt = softplus(dt @ W[p + "dt"].T + W[p + "dt.b"])
    A = -np.exp(W[p + "A_log"])
    S = np.zeros((inner, N))
    y = np.zeros((T, inner))
    for t in range(T):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + W[p + "D"] * x[t]
    return (y * silu(z)) @ W[p + "o"].T


def parallel_mixer(h, W, p, m):
    return (m["left_scale"] * distance_attention(h, W, p + "left.", m["left"])
            + m["right_scale"] * selective_scan(h, W, p + "right.", m["right"]))


def clamped_expert(h, W, p, limit):
    """W_down (g * sigmoid(1.702 g) * (u + 1)) with g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit)."""
    g = np.minimum(h @ W[p + "gate"].T, limit)
    u = np.clip(h @ W[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


ROUTE_MARGINS = []       # per call of route(): the smallest gap between the last chosen logit and the best one left out


def route(h, W_router, top, scale):
    """(chosen experts [T, top], their weights [T, top]): softmax over all experts, the ``top`` largest,
    times ``scale``, not renormalised."""
    z = h @ W_router.T
    if top < z.shape[1]:
        ranked = -np.sort(-z, axis=1)
        ROUTE_MARGINS.append(float(np.min(ranked[:, top - 1] - ranked[:, top])))
    z = z - z.max(axis=1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=1, keepdims=True)
    chosen = np.argsort(-s, axis=1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, axis=1) * scale


def moe(h, W, p, mlp):
    r = mlp["router"]
    chosen, weight = route(h, W[p + "router"], r["top"], r["scale"])
    out = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weight[t]):
            out[t] += w * clamped_expert(h[t:t + 1], W, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared") is not None:
        out += clamped_expert(h, W, p + "shared.", mlp["shared"]["limit"])
    return out


# --------------------------------------------------------------------------
def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] (float64) for one whole sequence; with ``return_layers`` also the residual stream
    after every layer, [layers, T, width]."""
    tokens = np.asarray(tokens)
    T, width, eps, m = len(tokens), cfg["width"], cfg["norm"]["eps"], cfg["residual_mult"]
    x = W["embed"][tokens] + sinusoid(T, width)
    history, streams = [x], []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "mingru":
            y = mingru(h, W, p + "mix.", layer["mixer"])
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, W, p + "mix.", layer["mixer"])
        else:
            raise ValueError(f"unknown mixer {layer['type']!r}")
        x = x + m * y
        if layer.get("mlp") is not None:
            x = x + m * moe(rms_norm(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
        history.append(x)
        a = W[p + "dwa"]
        x = sum(a[j] * history[j] for j in range(i + 2))
        streams.append(x)
    cap = cfg["logit_softcap"]
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(streams)) if return_layers else logits


def greedy(cfg, W, prompt, n):
    """``n`` tokens after ``prompt``, each the argmax of the last position's logits (ties: the lowest id)."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(np.argmax(forward(cfg, W, tokens)[-1])))
    return tokens[len(prompt):]
