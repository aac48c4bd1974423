"""Times one kernel of the library in isolation with CUDA events, on inputs larger than L2
where that matters, and prints what it achieved against the roofline that bounds it.

    python -m hfee_b200.kernels.microbench gemm_tcgen05 --m 2048 --n 16384 --k 2048 [--epilogue swiglu]
    python -m hfee_b200.kernels.microbench gemm_pair    --m 2048 --n 16384 --k 2048 --epilogue swiglu
    python -m hfee_b200.kernels.microbench gemm_stream  --m 8 --n 16384 --k 2048 [--epilogue swiglu]
    python -m hfee_b200.kernels.microbench gemm_ring    --m 8 --n 2048 --k 8192 --epilogue accum
    python -m hfee_b200.kernels.microbench gemm_skinny  --m 64 --n 2048 --k 8192 --epilogue accum
    python -m hfee_b200.kernels.microbench attention_decode  --batch 8 --context 2048 --heads 32 --kv-heads 8 --head-dim 64
    python -m hfee_b200.kernels.microbench attention_prefill --tokens 2048 --heads 32 --kv-heads 8 --head-dim 64
    python -m hfee_b200.kernels.microbench sigmoid_attention --tokens 2048 --heads 32 --kv-heads 8 --head-dim 64 --chunk 128
    python -m hfee_b200.kernels.microbench linear_attention  --tokens 2048 --heads 32 --head-dim 64 [--batch 8 for a decode step]
    python -m hfee_b200.kernels.microbench delta_rule        --tokens 2048 --heads 32 --kv-heads 8 --head-dim 64 [--decode --batch 8]
    python -m hfee_b200.kernels.microbench conv_act          --tokens 2048 --heads 32 --kv-heads 8 --head-dim 64
    python -m hfee_b200.kernels.microbench latent_attention  --tokens 2048 --heads 32 --head-dim 64 --rank 256 --window 512 [--decode --batch 8]
    python -m hfee_b200.kernels.microbench head_linear       --tokens 2048 --heads 32 --head-dim 64 --rank 256
    python -m hfee_b200.kernels.microbench rope_norm_cache   --tokens 2048 --heads 32 --kv-heads 8 --head-dim 64
    python -m hfee_b200.kernels.microbench mingru            --tokens 2048 --channels 2048 [--decode --batch 8]
    python -m hfee_b200.kernels.microbench selective_scan    --tokens 2048 --channels 2048 --state 16 [--decode --batch 8]
    python -m hfee_b200.kernels.microbench distance_attention --tokens 2048 --heads 32 --kv-heads 8 --head-dim 64 [--value-dim 128] [--decode --batch 8]
    python -m hfee_b200.kernels.microbench moe_experts       --tokens 2048 --k 2048 --inner 2048 --experts 16 --top 2
    python -m hfee_b200.kernels.microbench row_ops           --tokens 2048 --k 2048 --inner 4096 --depth 6

``--iters`` timed launches follow ``--warmup`` untimed ones; ``--rotate`` distinct weight
buffers are cycled so that a weight-streaming kernel never finds its weights in L2.  The
same command line under ``ncu`` gives the counters summarised in ``profiles/``.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch

from . import ops

DEV = "cuda:0"
EPI = {"store": ops.EPI_STORE, "accum": ops.EPI_ACCUM, "swiglu": ops.EPI_SWIGLU}


GRAPH = False


def _time(fn, warmup: int, iters: int) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if GRAPH:          # device time without host launch overhead: the timed launches replay from a CUDA graph
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(warmup + i)
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters * 1e-3
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(warmup + i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def _gemm(args, kind: str) -> dict:
    m, n, k = args.m, args.n, args.k
    epi = EPI[args.epilogue]
    a = (torch.randn(m, k, device=DEV) * 0.5).to(torch.bfloat16)
    ws = [(torch.randn(n, k, device=DEV) * 0.05).to(torch.bfloat16) for _ in range(args.rotate)]
    if epi == ops.EPI_ACCUM:
        out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    elif epi == ops.EPI_SWIGLU:
        out = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
    else:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    if kind == "gemm_tcgen05":
        fn = lambda i: ops.gemm_tcgen05(a, ws[i % len(ws)], out, epi, args.block_n)
    elif kind == "gemm_skinny":
        fn = lambda i: ops.gemm_skinny(a, ws[i % len(ws)], out, epi)
    elif kind == "gemm_pair":
        fn = lambda i: ops.gemm_tcgen05_pair(a, ws[i % len(ws)], out, epi)
    elif kind == "gemm_ring":
        fn = lambda i: ops.gemm_ring(a, ws[i % len(ws)], out, epi)
    else:
        fn = lambda i: ops.gemm_stream(a, ws[i % len(ws)], out, epi)
    sec = _time(fn, args.warmup, args.iters)
    ops.check_status()
    flops = 2.0 * m * n * k
    bytes_ = 2.0 * (n * k + m * k) + out.numel() * out.element_size()
    return {"kernel": kind, "m": m, "n": n, "k": k, "epilogue": args.epilogue, "us": round(sec * 1e6, 2),
            "tflops": round(flops / sec / 1e12, 1), "gbs": round(bytes_ / sec / 1e9, 1)}


class _Batch:
    pass


def _attention(args, decode: bool) -> dict:
    heads, kv, hd, page = args.heads, args.kv_heads, args.head_dim, args.page_size
    if decode:
        before, new = [args.context] * args.batch, [1] * args.batch
    else:
        before, new = [args.context_before], [args.tokens]
    r = len(before)
    total = [b + n for b, n in zip(before, new)]
    max_pages = max(-(-t // page) for t in total)
    n_pages = r * max_pages
    table = torch.randperm(n_pages).reshape(r, max_pages).to(torch.int32).to(DEV)
    kp = torch.randn(n_pages, kv, page, hd, device=DEV).to(torch.bfloat16)
    vp = torch.randn(n_pages, kv, page, hd, device=DEV).to(torch.bfloat16)
    n = sum(new)
    q = torch.randn(n, heads * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    b = _Batch()
    cu = [0]
    for x in new:
        cu.append(cu[-1] + x)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    b.cu_tokens, b.slots, b.context_before = i32(cu), i32(list(range(r))), i32(before)
    b.n, b.r, b.max_new, b.max_context = n, r, max(new), max(total)
    b.planning_context = b.max_context
    b.attention_splits = args.splits or None
    pos = i32([p for s, c in zip(before, new) for p in range(s, s + c)])
    sot = i32([i for i, c in enumerate(new) for _ in range(c)])
    scratch = torch.empty(r * heads * ops.MAX_SPLITS * (hd + 2), dtype=torch.float32, device=DEV) if decode else None
    scale = 1.0 / math.sqrt(hd)
    fn = lambda i: ops.paged_attention(q, kp, vp, table, page, pos, sot, out, heads, kv, hd, scale, 0, step=b, scratch=scratch)
    sec = _time(fn, args.warmup, args.iters)
    kv_bytes = sum(total) * kv * hd * 2 * 2
    flops = sum(4.0 * heads * hd * (c * s + c * (c + 1) / 2) for s, c in zip(before, new))
    return {"kernel": "attention_decode" if decode else "attention_prefill", "heads": heads, "kv_heads": kv,
            "head_dim": hd, "requests": r, "context": max(total), "us": round(sec * 1e6, 2),
            "kv_gbs": round(kv_bytes / sec / 1e9, 1), "tflops": round(flops / sec / 1e12, 1)}


def _batch_of(before, new):
    b = _Batch()
    cu = [0]
    for x in new:
        cu.append(cu[-1] + x)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    b.cu_tokens, b.slots, b.context_before = i32(cu), i32(list(range(len(new)))), i32(before)
    b.n, b.r, b.max_new, b.max_context = sum(new), len(new), max(new), max(s + c for s, c in zip(before, new))
    b.positions = i32([p for s, c in zip(before, new) for p in range(s, s + c)])
    b.slot_of_token = i32([i for i, c in enumerate(new) for _ in range(c)])
    return b


def _sigmoid_attention(args) -> dict:
    """Chunked sigmoid attention of one prompt portion (``--batch 0``) or of a decode step of ``--batch`` requests."""
    heads, kv, hd, page, chunk = args.heads, args.kv_heads, args.head_dim, args.page_size, args.chunk
    before, new = ([args.context] * args.batch, [1] * args.batch) if args.decode else ([args.context_before], [args.tokens])
    b = _batch_of(before, new)
    max_pages = -(-b.max_context // page)
    table = torch.randperm(b.r * max_pages).reshape(b.r, max_pages).to(torch.int32).to(DEV)
    kp = torch.randn(b.r * max_pages, kv, page, hd, device=DEV).to(torch.bfloat16)
    vp = torch.randn(b.r * max_pages, kv, page, hd, device=DEV).to(torch.bfloat16)
    q = torch.randn(b.n, heads * hd, device=DEV).to(torch.bfloat16)
    gate = torch.randn(b.n, heads * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    temp = torch.ones(heads, device=DEV)
    bias = torch.zeros(heads, device=DEV)
    ops.USE_SIGMOID_MMA = not args.no_tc_attention
    fn = lambda i: ops.sigmoid_attention(q, kp, vp, table, page, b, out, heads, kv, hd, hd ** -0.5, 0, chunk, temp, bias, gate)
    sec = _time(fn, args.warmup, args.iters)
    keys = sum(p - (p // chunk) * chunk + 1 if chunk else p + 1 for s, c in zip(before, new) for p in range(s, s + c))
    flops = 4.0 * heads * hd * keys
    moved = 3 * b.n * heads * hd * 2 + 2 * sum(min(s + c, (chunk or s + c) + c) for s, c in zip(before, new)) * kv * hd * 2
    return {"kernel": "sigmoid_attention", "heads": heads, "kv_heads": kv, "head_dim": hd, "chunk": chunk, "requests": b.r,
            "tokens": b.n, "us": round(sec * 1e6, 2), "tflops": round(flops / sec / 1e12, 2), "gbs": round(moved / sec / 1e9, 1)}


def _linear_attention(args) -> dict:
    """Linear attention with decay: one prompt portion through the chunked kernels, or a decode step of ``--batch``
    requests through the token-by-token kernel (key and value size ``--head-dim``)."""
    heads, d = args.heads, args.head_dim
    before, new = ([args.context] * args.batch, [1] * args.batch) if args.decode else ([0], [args.tokens])
    b = _batch_of(before, new)
    proj = (torch.randn(b.n, 4 * heads * d, device=DEV) * 0.5).to(torch.bfloat16)
    q, k, v = proj[:, :heads * d], proj[:, heads * d:2 * heads * d], proj[:, 2 * heads * d:3 * heads * d]
    decay = torch.linspace(0.5, 0.999, heads, device=DEV)
    state = torch.zeros(b.r, heads, d, d, device=DEV)
    out = torch.empty(b.n, heads * d, dtype=torch.float32, device=DEV)
    ws = torch.empty(ops.linear_attention_workspace(b.r, b.n, heads, d, d), dtype=torch.float32, device=DEV)
    fn = lambda i: ops.linear_attention(q, k, v, decay, state, b, out, heads, d, d, "silu", True, ws,
                                        tensor_cores=not args.no_tc_attention)
    sec = _time(fn, args.warmup, args.iters)
    state_bytes = b.r * heads * d * d * 4
    moved = 3 * b.n * heads * d * 2 + b.n * heads * d * 4 + 2 * state_bytes        # q, k, v in; o out; the state in and out
    flops = b.n * heads * 4.0 * d * d if args.decode else b.n * heads * (4.0 * d * d + 4.0 * d * 32)
    return {"kernel": "linear_attention", "heads": heads, "dim": d, "requests": b.r, "tokens": b.n,
            "us": round(sec * 1e6, 2), "tflops": round(flops / sec / 1e12, 2), "gbs": round(moved / sec / 1e9, 1)}


def _delta_rule(args) -> dict:
    """The gated delta rule: one prompt portion or a decode step of ``--batch`` requests (key and value size ``--head-dim``,
    ``--kv-heads`` query/key heads)."""
    heads, g, d = args.heads, args.kv_heads, args.head_dim
    before, new = ([args.context] * args.batch, [1] * args.batch) if args.decode else ([0], [args.tokens])
    b = _batch_of(before, new)
    qkv = (torch.randn(b.n, 2 * g * d + heads * d, device=DEV) * 0.5).to(torch.bfloat16)
    ba = torch.randn(b.n, 2 * heads, device=DEV).to(torch.bfloat16)
    a_log, dt_bias = torch.linspace(-4.0, 1.0, heads, device=DEV), torch.linspace(-3.0, 1.0, heads, device=DEV)
    state = torch.zeros(b.r, heads, d, d, device=DEV)
    out = torch.empty(b.n, heads * d, dtype=torch.float32, device=DEV)
    ws = torch.empty(ops.delta_rule_workspace(b.r, b.n, heads, g, d), dtype=torch.float32, device=DEV)
    fn = lambda i: ops.delta_rule(qkv, 0, g * d, 2 * g * d, ba, 0, heads, a_log, dt_bias, state, b, out, heads, g, d, d, True, ws)
    sec = _time(fn, args.warmup, args.iters)
    moved = b.n * (2 * g * d + heads * d) * 2 + b.n * heads * d * 4 + 2 * b.r * heads * d * d * 4
    flops = b.n * heads * 6.0 * d * d
    return {"kernel": "delta_rule", "heads": heads, "qk_heads": g, "dim": d, "requests": b.r, "tokens": b.n,
            "us": round(sec * 1e6, 2), "tflops": round(flops / sec / 1e12, 3), "gbs": round(moved / sec / 1e9, 1)}


def _conv_act(args) -> dict:
    heads, g, d = args.heads, args.kv_heads, args.head_dim
    b = _batch_of([0], [args.tokens])
    width = 2 * g * d + heads * d
    x = torch.randn(b.n, width + 8, device=DEV).to(torch.bfloat16)[:, :width]
    w = torch.randn(width, 4, device=DEV)
    state = torch.zeros(1, 3, width, device=DEV)
    out = torch.empty(b.n, width, dtype=torch.bfloat16, device=DEV)
    sec = _time(lambda i: ops.conv_act(x, w, state, b, out, "silu", True), args.warmup, args.iters)
    return {"kernel": "conv_act", "width": width, "tokens": b.n, "us": round(sec * 1e6, 2),
            "gbs": round(2 * b.n * width * 2 / sec / 1e9, 1)}


def _latent_attention(args) -> dict:
    """Attention over one cached vector per token of ``--rank`` + ``--head-dim``/2 dimensions whose first ``--rank`` are the values."""
    heads, rank, page, window = args.heads, args.rank, args.page_size, args.window
    dk = rank + args.head_dim // 2
    before, new = ([args.context] * args.batch, [1] * args.batch) if args.decode else ([args.context_before], [args.tokens])
    b = _batch_of(before, new)
    max_pages = -(-b.max_context // page)
    table = torch.randperm(b.r * max_pages).reshape(b.r, max_pages).to(torch.int32).to(DEV)
    pool = torch.randn(b.r * max_pages, 1, page, dk, device=DEV).to(torch.bfloat16)
    q = (torch.randn(b.n, heads * dk, device=DEV) * 0.3).to(torch.bfloat16)
    out = torch.empty(b.n, heads * rank, dtype=torch.bfloat16, device=DEV)
    ops.USE_LATENT_MMA = not args.no_tc_attention
    fn = lambda i: ops.latent_attention(q, pool, table, page, b, out, heads, dk, rank, dk ** -0.5, window)
    sec = _time(fn, args.warmup, args.iters)
    keys = sum(min(p + 1, window) if window else p + 1 for s, c in zip(before, new) for p in range(s, s + c))
    flops = 2.0 * heads * (dk + rank) * keys
    moved = b.n * heads * (dk + rank) * 2 + sum(min(s + c, (window or s + c) + c) for s, c in zip(before, new)) * dk * 2
    return {"kernel": "latent_attention", "heads": heads, "key_dim": dk, "value_dim": rank, "window": window, "requests": b.r,
            "tokens": b.n, "us": round(sec * 1e6, 2), "tflops": round(flops / sec / 1e12, 2), "gbs": round(moved / sec / 1e9, 1)}


def _head_linear(args) -> dict:
    """The two per-head products of a latent attention: queries folded onto the latent (head_dim -> rank) and the attended
    latent expanded to values (rank -> head_dim)."""
    heads, d, rank, n = args.heads, args.head_dim, args.rank, args.tokens
    r = d // 2
    qh = torch.randn(n, heads * (d + r), device=DEV).to(torch.bfloat16)
    w_fold = (torch.randn(heads, rank, d, device=DEV) * 0.1).to(torch.bfloat16)
    qf = torch.empty(n, heads * (rank + r), dtype=torch.bfloat16, device=DEV)
    ol = torch.randn(n, heads * rank, device=DEV).to(torch.bfloat16)
    w_uv = (torch.randn(heads, d, rank, device=DEV) * 0.1).to(torch.bfloat16)
    att = torch.empty(n, heads * d, dtype=torch.bfloat16, device=DEV)
    gate = torch.randn(n, heads, device=DEV).to(torch.bfloat16)
    fold = _time(lambda i: ops.head_linear(qh, 0, d + r, w_fold, qf, 0, rank + r), args.warmup, args.iters)
    expand = _time(lambda i: ops.head_linear(ol, 0, rank, w_uv, att, 0, d, gate), args.warmup, args.iters)
    flops = 2.0 * n * heads * d * rank
    return {"kernel": "head_linear", "heads": heads, "head_dim": d, "rank": rank, "tokens": n,
            "fold_us": round(fold * 1e6, 2), "fold_tflops": round(flops / fold / 1e12, 1),
            "fold_gbs": round(n * heads * (d + rank) * 2 / fold / 1e9, 1),
            "expand_us": round(expand * 1e6, 2), "expand_tflops": round(flops / expand / 1e12, 1),
            "expand_gbs": round(n * heads * (d + rank) * 2 / expand / 1e9, 1)}


def _rope_norm_cache(args) -> dict:
    heads, kv, d, page = args.heads, args.kv_heads, args.head_dim, args.page_size
    b = _batch_of([0], [args.tokens])
    max_pages = -(-b.n // page)
    table = torch.randperm(max_pages).reshape(1, max_pages).to(torch.int32).to(DEV)
    kp = torch.empty(max_pages, kv, page, d, dtype=torch.bfloat16, device=DEV)
    vp = torch.empty_like(kp)
    cols = (heads + 2 * kv) * d
    proj = torch.randn(b.n, cols, device=DEV).to(torch.bfloat16)
    cs = torch.rand(b.n, d // 2, 2, device=DEV)
    q = torch.empty(b.n, heads * d, dtype=torch.bfloat16, device=DEV)
    fn = lambda i: ops.rope_norm_cache(proj, cs, d, 1e-5, b.positions, b.slot_of_token, table, page, q=(heads, 0, d, d, 0, q, 0, d),
                                       k=(kv, heads * d, d, d, 0, kp, 0), v=((heads + kv) * d, d, d, vp))
    sec = _time(fn, args.warmup, args.iters)
    return {"kernel": "rope_norm_cache", "tokens": b.n, "us": round(sec * 1e6, 2), "gbs": round(2 * b.n * cols * 2 / sec / 1e9, 1)}


def _mingru(args) -> dict:
    """minGRU over ``--channels`` channels: one prompt portion, or a decode step of ``--batch`` requests."""
    c = args.channels
    before, new = ([args.context] * args.batch, [1] * args.batch) if args.decode else ([0], [args.tokens])
    b = _batch_of(before, new)
    proj = torch.randn(b.n, 3 * c, device=DEV).to(torch.bfloat16)
    zb, xb = torch.randn(c, device=DEV), torch.randn(c, device=DEV)
    state = torch.zeros(b.r, c, device=DEV)
    out = torch.empty(b.n, c, dtype=torch.bfloat16, device=DEV)
    sec = _time(lambda i: ops.mingru(proj, 0, c, 2 * c, zb, xb, state, b, out, c, True), args.warmup, args.iters)
    moved = b.n * 4 * c * 2 + 2 * b.r * c * 4
    return {"kernel": "mingru", "channels": c, "requests": b.r, "tokens": b.n, "us": round(sec * 1e6, 2),
            "gbs": round(moved / sec / 1e9, 1)}


def _selective_scan(args) -> dict:
    """Selective scan over ``--channels`` channels of ``--state`` entries: one prompt portion, or a decode step of ``--batch``."""
    c, ns = args.channels, args.state
    before, new = ([args.context] * args.batch, [1] * args.batch) if args.decode else ([0], [args.tokens])
    b = _batch_of(before, new)
    xz = (torch.randn(b.n, 2 * c, device=DEV) * 0.5).to(torch.bfloat16)
    bc = (torch.randn(b.n, 2 * ns, device=DEV) * 0.5).to(torch.bfloat16)
    dt = torch.randn(b.n, c, device=DEV) - 2.0
    a_log = torch.log(torch.arange(1, ns + 1, device=DEV, dtype=torch.float32)).repeat(c, 1).contiguous()
    d_skip, dt_bias = torch.ones(c, device=DEV), torch.zeros(c, device=DEV)
    state = torch.zeros(b.r, c, ns, device=DEV)
    out = torch.empty(b.n, c, dtype=torch.bfloat16, device=DEV)
    fn = lambda i: ops.selective_scan(xz[:, :c], dt, bc, 0, ns, xz[:, c:], a_log, d_skip, dt_bias, state, b, out, 1.0, True)
    sec = _time(fn, args.warmup, args.iters)
    moved = b.n * (3 * c * 2 + c * 4 + 2 * ns * 2) + 2 * b.r * c * ns * 4
    return {"kernel": "selective_scan", "channels": c, "state": ns, "requests": b.r, "tokens": b.n, "us": round(sec * 1e6, 2),
            "gbs": round(moved / sec / 1e9, 1), "exp_per_s_e12": round(b.n * c * ns / sec / 1e12, 3)}


def _distance_attention(args) -> dict:
    """Softmax attention with the logarithmic distance penalty: one prompt portion, or a decode step of ``--batch`` requests."""
    heads, kv, hd, vd, page = args.heads, args.kv_heads, args.head_dim, args.value_dim or args.head_dim, args.page_size
    before, new = ([args.context] * args.batch, [1] * args.batch) if args.decode else ([args.context_before], [args.tokens])
    b = _batch_of(before, new)
    b.planning_context, b.attention_splits = b.max_context, args.splits or None
    max_pages = -(-b.max_context // page)
    table = torch.randperm(b.r * max_pages).reshape(b.r, max_pages).to(torch.int32).to(DEV)
    kp = torch.randn(b.r * max_pages, kv, page, hd, device=DEV).to(torch.bfloat16)
    vp = torch.randn(b.r * max_pages, kv, page, vd, device=DEV).to(torch.bfloat16)
    q = torch.randn(b.n, heads * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty(b.n, heads * vd, dtype=torch.bfloat16, device=DEV)
    r1, r2 = torch.linspace(0.5, 2.0, heads, device=DEV), torch.linspace(0.1, 1.0, heads, device=DEV)
    tile = ops.distance_attention_tile(hd, vd)
    scratch = torch.empty(b.r * heads * ops.MAX_SPLITS * (tile + 2), dtype=torch.float32, device=DEV) if args.decode and tile else None
    fn = lambda i: ops.distance_attention(q, kp, vp, table, page, b, out, heads, kv, hd, vd, hd ** -0.5, r1, r2, 1.0, 0, scratch)
    sec = _time(fn, args.warmup, args.iters)
    total = [s + c for s, c in zip(before, new)]
    kv_bytes = sum(total) * kv * (hd + vd) * 2
    flops = sum(2.0 * heads * (hd + vd) * (c * s + c * (c + 1) / 2) for s, c in zip(before, new))
    return {"kernel": "distance_attention", "heads": heads, "kv_heads": kv, "head_dim": hd, "value_dim": vd, "requests": b.r,
            "context": b.max_context, "us": round(sec * 1e6, 2), "kv_gbs": round(kv_bytes / sec / 1e9, 1),
            "tflops": round(flops / sec / 1e12, 1)}


def _moe_experts(args) -> dict:
    """The routed experts of ``--tokens`` tokens (``--experts`` of inner size ``--inner``, ``--top`` a token, width ``--k``):
    plan, gather, both grouped products and the activation between them, and the weighted sum."""
    n, w, f, e, top = args.tokens, args.k, args.inner, args.experts, args.top
    x = torch.randn(n, w, device=DEV).to(torch.bfloat16)
    w_gu = (torch.randn(e, 2 * f, w, device=DEV) * w ** -0.5).to(torch.bfloat16)      # rows in runs of [4 gate | 4 up]
    w_d = (torch.randn(e, w, f, device=DEV) * f ** -0.5).to(torch.bfloat16)
    logits = torch.randn(n, e, device=DEV)
    choice = torch.empty(n, top, dtype=torch.int32, device=DEV)
    weight = torch.empty(n, top, dtype=torch.float32, device=DEV)
    ops.moe_route(logits, top, 1.0, choice, weight)
    tiles = ops.moe_tiles_grouped(n * top, e)
    rows = tiles * ops.GROUPED_TILE_ROWS
    i32 = lambda k: torch.empty(k, dtype=torch.int32, device=DEV)
    place, row_pair, tile_group = i32(n * top), i32(rows), i32(tiles)
    bf = lambda c: torch.empty(rows, c, dtype=torch.bfloat16, device=DEV)
    rows_in, gate_up, hidden = bf(w), (bf(2 * f) if args.unfused else None), bf(f)
    rows_out = torch.empty(rows, w, dtype=torch.float32, device=DEV)
    y = torch.zeros(n, w, dtype=torch.float32, device=DEV)

    def fn(i):
        ops.moe_experts_grouped(x, top, choice, w_gu, w_d, 7.0, place, row_pair, tile_group, rows_in, gate_up, hidden, rows_out)
        ops.moe_combine(rows_out, weight, y, False, place)
    sec = _time(fn, args.warmup, args.iters)
    flops = 2.0 * n * top * 3 * f * w
    return {"kernel": "moe_experts_grouped", "tokens": n, "width": w, "inner": f, "experts": e, "top": top, "tiles": tiles,
            "us": round(sec * 1e6, 2), "tflops": round(flops / sec / 1e12, 1)}


def _row_ops(args) -> dict:
    """The row kernels of the scaled pre-norm block with a depth average, the clamped gated activation and the sinusoid, on
    ``--tokens`` rows of width ``--k`` (activation: inner size ``--inner``): microseconds and GB/s each."""
    n, w, f, depth = args.tokens, args.k, args.inner, args.depth
    res = {"kernel": "row_ops", "tokens": n, "width": w}
    x, y = torch.randn(n, w, device=DEV), torch.randn(n, w, device=DEV)
    hist = torch.randn(depth + 1, n, w, device=DEV)
    wts = torch.full((depth + 1,), 1.0 / (depth + 1), device=DEV)
    sec = _time(lambda i: ops.depth_average(x, y, 0.5, hist, wts, depth - 1), args.warmup, args.iters)
    res["depth_average"] = {"entries": depth + 1, "us": round(sec * 1e6, 2), "gbs": round(n * w * 4 * (depth + 4) / sec / 1e9, 1)}
    nw, out = torch.ones(w, device=DEV), torch.empty(n, w, dtype=torch.bfloat16, device=DEV)
    sec = _time(lambda i: ops.scaled_add_norm(y, 0.5, x, nw, 1e-5, out), args.warmup, args.iters)
    res["scaled_add_norm"] = {"us": round(sec * 1e6, 2), "gbs": round(n * w * 14 / sec / 1e9, 1)}
    gu, h = torch.randn(n, 2 * f, device=DEV).to(torch.bfloat16), torch.empty(n, f, dtype=torch.bfloat16, device=DEV)
    sec = _time(lambda i: ops.clamped_glu(gu, h, 7.0), args.warmup, args.iters)
    res["clamped_glu"] = {"inner": f, "us": round(sec * 1e6, 2), "gbs": round(n * f * 6 / sec / 1e9, 1)}
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    sec = _time(lambda i: ops.add_sinusoid(x, pos), args.warmup, args.iters)
    res["add_sinusoid"] = {"us": round(sec * 1e6, 2), "gbs": round(n * w * 8 / sec / 1e9, 1)}
    return res


def _softmax_attention(args) -> dict:
    """Windowed softmax attention with a sink (``--window``, 0: none): one prompt portion, or a decode step of ``--batch``."""
    heads, kv, hd, vd, page = args.heads, args.kv_heads, args.head_dim, args.value_dim or args.head_dim, args.page_size
    before, new = ([args.context] * args.batch, [1] * args.batch) if args.decode else ([args.context_before], [args.tokens])
    b = _batch_of(before, new)
    b.planning_context, b.attention_splits = b.max_context, args.splits or None
    max_pages = -(-b.max_context // page)
    table = torch.randperm(b.r * max_pages).reshape(b.r, max_pages).to(torch.int32).to(DEV)
    kp = torch.randn(b.r * max_pages, kv, page, hd, device=DEV).to(torch.bfloat16)
    vp = torch.randn(b.r * max_pages, kv, page, vd, device=DEV).to(torch.bfloat16)
    q = torch.randn(b.n, heads * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty(b.n, heads * vd, dtype=torch.bfloat16, device=DEV)
    sink = torch.linspace(-1.0, 2.0, heads, device=DEV)
    tile = ops.distance_attention_tile(hd, vd)
    scratch = torch.empty(b.r * heads * ops.MAX_SPLITS * (tile + 2), dtype=torch.float32, device=DEV) if args.decode and tile else None
    fn = lambda i: ops.softmax_attention(q, kp, vp, table, page, b, out, heads, kv, hd, vd, hd ** -0.5, args.window, sink, 1.0, scratch)
    sec = _time(fn, args.warmup, args.iters)
    w = args.window or (1 << 30)
    seen = lambda s, c: sum(min(w, s + j + 1) for j in range(c))          # keys each new token reads
    kv_bytes = sum(min(s + c, w + c) for s, c in zip(before, new)) * kv * (hd + vd) * 2
    flops = sum(2.0 * heads * (hd + vd) * seen(s, c) for s, c in zip(before, new))
    return {"kernel": "softmax_attention", "heads": heads, "kv_heads": kv, "head_dim": hd, "value_dim": vd, "requests": b.r,
            "context": b.max_context, "window": args.window, "us": round(sec * 1e6, 2), "kv_gbs": round(kv_bytes / sec / 1e9, 1),
            "tflops": round(flops / sec / 1e12, 1)}


def _gated_recurrence(args, mode: int) -> dict:
    """The gated matrix-state recurrences (``gla``: a decay per key channel; ``matrix_memory``: exponential gates) of
    ``--heads`` heads with keys of ``--head-dim`` and values of ``--value-dim``: one prompt portion of ``--tokens`` tokens
    (walked as runs side by side), or a decode step of ``--batch`` requests."""
    heads, d, vd = args.heads, args.head_dim, args.value_dim or args.head_dim
    before, new = ([args.context] * args.batch, [1] * args.batch) if args.decode else ([0], [args.tokens])
    b = _batch_of(before, new)
    qk, vc = heads * d, heads * vd
    proj = (torch.randn(b.n, 2 * qk + vc, device=DEV) * 0.5).to(torch.bfloat16)
    pre = torch.randn(b.n, qk if mode == 0 else 2 * heads, device=DEV)
    keep = pre.clone()
    bias = torch.full((pre.shape[1],), 2.0, device=DEV)
    S = torch.zeros(b.r, heads, d, vd, device=DEV)
    N, M = torch.zeros(b.r, heads, d, device=DEV), torch.zeros(b.r, heads, device=DEV)
    out = torch.empty(b.n, vc, device=DEV)
    ws = torch.empty(ops.gated_recurrence_workspace(b.r, b.n, heads, d, vd), device=DEV)

    def fn(i):
        if mode == 0 and b.max_new >= ops.RECURRENCE_CHUNKED_MIN:
            pre.copy_(keep)                # the chunked path turns the gates into decays in place
        ops.gated_recurrence(mode, proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:], pre, bias, 1.0 / 16 if mode == 0 else 15.0,
                             d ** -0.5, S, b, out, heads, d, vd, True, N if mode else None, M if mode else None, ws)
    sec = _time(fn, args.warmup, args.iters)
    chunked = b.max_new >= ops.RECURRENCE_CHUNKED_MIN
    flops = (2 if chunked else 1) * b.n * heads * d * vd * (5.0 if mode == 0 else 5.0)      # a chunked walk visits a token twice
    io = b.n * ((2 * qk + vc) * 2 + pre.shape[1] * 4 + vc * 4) + 2 * b.r * heads * d * vd * 4
    return {"kernel": "gla" if mode == 0 else "matrix_memory", "heads": heads, "key_dim": d, "value_dim": vd, "tokens": b.n,
            "requests": b.r, "chunked": chunked, "us": round(sec * 1e6, 2), "fp32_tflops": round(flops / sec / 1e12, 2),
            "io_gbs": round(io / sec / 1e9, 1)}


def _pupinex_rows(args) -> dict:
    """Row kernels of the Pupinex parts on ``--tokens`` rows of width ``--k``: layer norm, the bigram embedding, the bias,
    the step between the q/k/v projection and the attention, and the per-head norm with its gate."""
    n, w = args.tokens, args.k
    res = {"kernel": "pupinex_rows", "tokens": n, "width": w}
    x, nw = torch.randn(n, w, device=DEV), torch.ones(w, device=DEV)
    out = torch.empty(n, w, dtype=torch.bfloat16, device=DEV)
    sec = _time(lambda i: ops.layernorm(x, nw, out, 1e-5), args.warmup, args.iters)
    res["layernorm"] = {"us": round(sec * 1e6, 2), "gbs": round(n * w * 6 / sec / 1e9, 1)}
    sec = _time(lambda i: ops.rmsnorm(x, nw, out, 1e-5), args.warmup, args.iters)
    res["rmsnorm"] = {"us": round(sec * 1e6, 2), "gbs": round(n * w * 6 / sec / 1e9, 1)}
    sec = _time(lambda i: ops.add_bias(x, nw), args.warmup, args.iters)
    res["add_bias"] = {"us": round(sec * 1e6, 2), "gbs": round(n * w * 8 / sec / 1e9, 1)}
    b = _batch_of([0], [n])
    b.token_ids = torch.randint(0, 32768, (n,), dtype=torch.int32, device=DEV)
    b.feedback = None
    table = torch.randn(32768, w, device=DEV).to(torch.bfloat16)
    pairs = torch.randn(65522, w, device=DEV).to(torch.bfloat16)
    last = torch.zeros(b.r, 1, dtype=torch.int32, device=DEV)
    sec = _time(lambda i: ops.embed_bigram(table, pairs, b, last, x, 65521, 1000003, 31), args.warmup, args.iters)
    res["embed_bigram"] = {"us": round(sec * 1e6, 2), "gbs": round(n * w * 8 / sec / 1e9, 1)}
    heads, kv, hd, page = args.heads, args.kv_heads, args.head_dim, args.page_size
    cols = (heads + 2 * kv) * hd
    proj = torch.randn(n, cols, device=DEV).to(torch.bfloat16)
    max_pages = -(-n // page)
    tbl = torch.arange(max_pages, dtype=torch.int32, device=DEV).reshape(1, max_pages)
    kp = torch.zeros(max_pages, kv, page, hd, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    q = torch.empty(n, heads * hd, dtype=torch.bfloat16, device=DEV)
    cs = torch.rand(n, hd // 4, 2, device=DEV)
    bias = [torch.zeros(c, device=DEV) for c in (heads * hd, kv * hd, kv * hd)]
    norms = (torch.ones(heads * hd, device=DEV), torch.ones(kv * hd, device=DEV))
    sec = _time(lambda i: ops.attention_prepare(proj, 0, heads * hd, (heads + kv) * hd, heads, kv, hd, hd, b, q, kp, vp, tbl, page, cs,
                                                hd // 2, False, tuple(bias), norms, 1e-5), args.warmup, args.iters)
    res["attention_prepare"] = {"us": round(sec * 1e6, 2), "gbs": round(n * cols * 4 / sec / 1e9, 1)}
    o, g = torch.randn(n, w, device=DEV), torch.randn(n, w, device=DEV).to(torch.bfloat16)
    sec = _time(lambda i: ops.head_norm_gate_scaled(o, nw, 1e-5, g, out, 8, w // 8, "sigmoid", 0.5), args.warmup, args.iters)
    res["head_norm_gate"] = {"us": round(sec * 1e6, 2), "gbs": round(n * w * 8 / sec / 1e9, 1)}
    return res


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["delta_rule", "conv_act", "latent_attention", "head_linear", "rope_norm_cache",
                                       "gemm_tcgen05", "gemm_stream", "gemm_skinny", "gemm_ring", "gemm_pair", "attention_decode", "attention_prefill",
                                      "sigmoid_attention", "linear_attention", "mingru", "selective_scan",
                                       "distance_attention", "moe_experts", "row_ops", "softmax_attention", "gla", "matrix_memory",
                                       "pupinex_rows"])
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--epilogue", default="store", choices=list(EPI))
    ap.add_argument("--block-n", type=int, default=None)
    ap.add_argument("--rotate", type=int, default=4, help="distinct weight buffers cycled between launches")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--context-before", type=int, default=0)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--rank", type=int, default=256, help="latent_attention / head_linear: size of the key/value latent")
    ap.add_argument("--window", type=int, default=512, help="latent_attention: sliding window (0: all earlier positions)")
    ap.add_argument("--chunk", type=int, default=128, help="sigmoid_attention: positions per block of the mask")
    ap.add_argument("--decode", action="store_true", help="sigmoid_attention / linear_attention: a decode step of --batch requests")
    ap.add_argument("--channels", type=int, default=2048, help="mingru / selective_scan: channels of the recurrence")
    ap.add_argument("--state", type=int, default=16, help="selective_scan: state entries per channel")
    ap.add_argument("--value-dim", type=int, default=0, help="distance_attention: value size per head (0: the key size)")
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--top", type=int, default=2)
    ap.add_argument("--inner", type=int, default=2048, help="moe_experts / row_ops: inner size of an expert")
    ap.add_argument("--unfused", action="store_true", help="moe_experts: the activation as a pass of its own")
    ap.add_argument("--depth", type=int, default=6, help="row_ops: layers in front of the depth average")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tc-attention", action="store_true", help="attention_prefill: the tcgen05 kernel (the default)")
    ap.add_argument("--no-tc-attention", action="store_true", help="attention_prefill: the mma.sync kernel")
    ap.add_argument("--graph", action="store_true", help="replay the timed launches from a CUDA graph (no host launch cost)")
    args = ap.parse_args(argv)
    global GRAPH
    GRAPH = args.graph
    ops.USE_TC_ATTENTION = args.tc_attention or not args.no_tc_attention
    torch.manual_seed(0)
    if args.kernel.startswith("gemm"):
        res = _gemm(args, args.kernel)
    elif args.kernel == "sigmoid_attention":
        res = _sigmoid_attention(args)
    elif args.kernel == "linear_attention":
        res = _linear_attention(args)
    elif args.kernel in ("delta_rule", "conv_act", "latent_attention", "head_linear", "rope_norm_cache"):
        res = {"delta_rule": _delta_rule, "conv_act": _conv_act, "latent_attention": _latent_attention,
               "head_linear": _head_linear, "rope_norm_cache": _rope_norm_cache}[args.kernel](args)
    elif args.kernel in ("mingru", "selective_scan", "distance_attention", "moe_experts", "row_ops"):
        res = {"mingru": _mingru, "selective_scan": _selective_scan, "distance_attention": _distance_attention,
               "moe_experts": _moe_experts, "row_ops": _row_ops}[args.kernel](args)
    elif args.kernel == "softmax_attention":
        res = _softmax_attention(args)
    elif args.kernel in ("gla", "matrix_memory"):
        res = _gated_recurrence(args, 0 if args.kernel == "gla" else 1)
    elif args.kernel == "pupinex_rows":
        res = _pupinex_rows(args)
    else:
        res = _attention(args, args.kernel == "attention_decode")
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
