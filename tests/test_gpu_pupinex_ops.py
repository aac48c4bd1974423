"""The kernels behind the Pupinex parts, each against a few lines of plain float64 arithmetic."""
import numpy as np
import pytest
import torch

import plain_pupinex as plain
from test_gpu_dobelix_ops import DEV, make_step

pytestmark = pytest.mark.gpu


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def close(got, want, tol):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return np.max(np.abs(got - want)) <= tol * max(np.max(np.abs(want)), 1e-30)


def token_step(entries, lengths, max_requests=4):
    """entries: [(slot, tokens)]; lengths: tokens each slot holds already."""
    from hfee_b200.engine.batch import Step, StepBuffers, StepEntry
    buffers = StepBuffers(max(64, sum(len(t) for _, t in entries)), max_requests, DEV)
    return Step([StepEntry(s, t, []) for s, t in entries], lengths, buffers)


@pytest.mark.parametrize("width", [6, 64, 1500, 5000])
def test_layer_norm(width):
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(width)
    n = 9
    x, w, e = rng.normal(size=(n, width)) * 3 + 1.5, rng.normal(size=width) + 1.0, rng.normal(size=(n, width))
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 8e-3)):
        out = torch.empty((n, width), dtype=dtype, device=DEV)
        ops.layernorm(dev(x), dev(w), out, 1e-5)
        assert close(out.float().cpu().numpy(), plain.layer_norm(x, w, 1e-5), tol)
    rows = [7, 0, 3]
    out = torch.empty((3, width), device=DEV)
    ops.layernorm(dev(x), dev(w), out, 1e-3, rows=dev(rows, torch.int32))
    assert close(out.cpu().numpy(), plain.layer_norm(x[rows], w, 1e-3), 3e-6)
    xd, out = dev(x), torch.empty((n, width), device=DEV)
    ops.layernorm(xd, dev(w), out, 1e-5, residual_add=dev(e))          # the sum stays in x, its norm goes out
    assert close(xd.cpu().numpy(), x + e, 1e-6) and close(out.cpu().numpy(), plain.layer_norm(x + e, w, 1e-5), 3e-6)
    b = rng.normal(size=width)
    ops.add_bias(xd, dev(b))
    assert close(xd.cpu().numpy(), x + e + b, 1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bigram_embedding_remembers_each_request_last_token(dtype):
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(1)
    vocab, width, buckets, mp, mc = 50, 24, 7, 12345, 678
    table, pairs = dev(rng.normal(size=(vocab, width)), dtype), dev(rng.normal(size=(buckets + 1, width)), dtype)
    tf, pf = table.float().cpu().numpy().astype(np.float64), pairs.float().cpu().numpy().astype(np.float64)
    seqs = {2: rng.integers(0, vocab, 30).tolist(), 0: rng.integers(0, vocab, 11).tolist(), 3: rng.integers(0, vocab, 5).tolist()}
    want = {s: plain.embed(t, tf, pf, {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}) for s, t in seqs.items()}
    last = torch.full((4, 1), 49, dtype=torch.int32, device=DEV)              # stale content of the slots' earlier users
    lengths = [0, 0, 0, 0]
    got = {s: [] for s in seqs}
    for sizes in ({2: 1, 0: 4}, {2: 1, 3: 5}, {0: 1, 2: 17}, {2: 11, 0: 6}):
        entries = [(s, seqs[s][lengths[s]:lengths[s] + n]) for s, n in sizes.items()]
        step = token_step(entries, lengths)
        out = torch.empty((step.n, width), device=DEV)
        ops.embed_bigram(table, pairs, step, last, out, buckets, mp, mc)
        o, at = out.cpu().numpy(), 0
        for s, n in sizes.items():
            got[s].append(o[at:at + n]); at += n; lengths[s] += n
    for s in seqs:
        assert close(np.concatenate(got[s]), want[s], 1e-6), s
    assert last[1, 0].item() == 49 and last[2, 0].item() == seqs[2][-1]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,rope,interleaved,normed,biased", [
    (4, 2, 16, 24, 8, True, False, True), (3, 3, 10, 6, 10, False, True, True), (2, 1, 32, 32, 0, False, True, False),
    (6, 2, 64, 16, 32, False, False, False), (1, 1, 6, 14, 2, True, True, True)])
def test_attention_prepare(dtype, heads, kv, dim, vdim, rope, interleaved, normed, biased):
    """Biases, the norm over whole projections, either pairing of a partial rotation, and the cache write."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(heads * dim)
    page, n0, n = 16, 21, 13                                  # 13 new tokens behind 21 cached ones, across a page's edge
    qc, kc, vc = heads * dim, kv * dim, kv * vdim
    src = dev(rng.normal(size=(n, qc + kc + vc + 3)), dtype)[:, :qc + kc + vc]
    x = src.float().cpu().numpy().astype(np.float64)
    bq, bk, bv = (rng.normal(size=c) if biased else None for c in (qc, kc, vc))
    wq, wk = (rng.normal(size=c) + 1.0 if normed else None for c in (qc, kc))
    eps = 1e-4
    q, k, v = x[:, :qc], x[:, qc:qc + kc], x[:, qc + kc:]
    if biased:
        q, k, v = q + bq, k + bk, v + bv
    if normed:
        q, k = plain.unit_rms(q, eps) * wq, plain.unit_rms(k, eps) * wk
    pos = np.arange(n0, n0 + n)

    def rotated(t, h):
        full = np.zeros((n0 + n, h, dim)); full[n0:] = t.reshape(n, h, dim)
        return plain.rotate(full, rope, 300.0, "interleaved" if interleaved else "half")[n0:] if rope else t.reshape(n, h, dim)
    want_q, want_k = rotated(q, heads).reshape(n, qc), rotated(k, kv)
    step = make_step([n], lengths=[n0], slots=[1])
    table = torch.tensor([[5, 2, 7, -1], [3, 0, 6, 4], [-1] * 4, [-1] * 4], dtype=torch.int32, device=DEV)
    k_pool, v_pool = torch.zeros((8, kv, page, dim), dtype=dtype, device=DEV), torch.zeros((8, kv, page, vdim), dtype=dtype, device=DEV)
    cs = None
    if rope:
        inv = torch.tensor([300.0 ** (-2.0 * i / rope) for i in range(rope // 2)], dtype=torch.float64, device=DEV)
        cs = torch.empty((n, rope // 2, 2), device=DEV)
        ops.rope_table(step.positions, inv, cs)
    q_out = torch.empty((n, qc), dtype=dtype, device=DEV)
    f = lambda a: None if a is None else dev(a)
    ops.attention_prepare(src, 0, qc, qc + kc, heads, kv, dim, vdim, step, q_out, k_pool, v_pool, table, page, cs, rope, interleaved,
                          (f(bq), f(bk), f(bv)), (f(wq), f(wk)), eps)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert close(q_out.float().cpu().numpy(), want_q, tol)
    pages = [3, 0, 6, 4]
    for t, p in enumerate(pos):
        kk = k_pool[pages[p // page], :, p % page].float().cpu().numpy()
        vv = v_pool[pages[p // page], :, p % page].float().cpu().numpy()
        assert close(kk, want_k[t], tol) and close(vv, v[t].reshape(kv, vdim), tol)
    assert torch.count_nonzero(k_pool[5]) == 0 and torch.count_nonzero(k_pool[3][:, :n0 % page]) == 0     # other requests' pages, earlier rows
    q_only = torch.empty((n, qc), dtype=dtype, device=DEV)
    ops.attention_prepare(src, 0, qc, qc + kc, heads, kv, dim, vdim, step, q_only, None, None, table, page, cs, rope, interleaved,
                          (f(bq), None, None), (f(wq), None), eps)
    assert torch.equal(q_only, q_out)


def _paged(seq_k, seq_v, page, dtype, order):
    """Pools and a block table row holding one request's keys and values on the pages ``order``."""
    T, G, d = seq_k.shape
    dv = seq_v.shape[2]
    pages = max(order) + 2
    k_pool = torch.full((pages, G, page, d), 9.0, dtype=dtype, device=DEV)          # stale content everywhere else
    v_pool = torch.full((pages, G, page, dv), -9.0, dtype=dtype, device=DEV)
    for t in range(T):
        k_pool[order[t // page], :, t % page] = dev(seq_k[t], dtype)
        v_pool[order[t // page], :, t % page] = dev(seq_v[t], dtype)
    return k_pool, v_pool


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,window", [(4, 2, 16, 24, 21), (2, 2, 64, 64, 200), (6, 1, 32, 8, 1), (3, 3, 12, 10, 40),
                                                      (8, 2, 128, 64, 77)])
def test_softmax_attention_with_sink_and_window(dtype, heads, kv, dim, vdim, window):
    """A prompt portion behind cached tokens, single decoded tokens (keys split among thread blocks where the kernel
    does that) and the two mixed, against the plain softmax with a sink."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(heads + dim)
    page, T = 16, 150
    q = rng.normal(size=(T, heads, dim))
    k, v = rng.normal(size=(T, kv, dim)), rng.normal(size=(T, kv, vdim))
    sink = rng.uniform(-2.0, 4.0, size=heads)
    rd = lambda a: dev(a, dtype).float().cpu().numpy().astype(np.float64)
    want = plain.windowed_softmax_attention(rd(q), rd(k), rd(v), 0.2, window, sink)
    want_plain = plain.windowed_softmax_attention(rd(q), rd(k), rd(v), 0.2, window)
    order = [4, 1, 7, 0, 9, 3, 8, 2, 6, 5]
    k_pool, v_pool = _paged(k, v, page, dtype, order)
    table = torch.full((4, 12), -1, dtype=torch.int32, device=DEV)
    table[2, :10] = dev(order, torch.int32)
    tile = ops.distance_attention_tile(dim, vdim)
    scratch = torch.empty((4 * heads * ops.MAX_SPLITS * (tile + 2),), device=DEV) if tile else None
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for lo, hi in ((0, T), (0, 37), (37, 149), (149, 150), (100, 101), (16, 18)):
        step = make_step([hi - lo], lengths=[lo], slots=[2])
        step.attention_splits = 3 if hi - lo == 1 else None
        qd = dev(q[lo:hi].reshape(hi - lo, heads * dim), dtype)
        for s, w in ((sink, want), (None, want_plain)):
            out = torch.empty((hi - lo, heads * vdim), dtype=dtype, device=DEV)
            ops.softmax_attention(qd, k_pool, v_pool, table, page, step, out, heads, kv, dim, vdim, 0.2, window,
                                  None if s is None else dev(s), 0.5, scratch)
            assert close(out.float().cpu().numpy(), 0.5 * w[lo:hi].reshape(hi - lo, -1), tol), (lo, hi, s is None)


def plain_recurrence(mode, q, k, v, pre, bias, p0, state):
    """One request, token by token; returns outputs and the new state (S, n, m)."""
    T, H, d = q.shape
    S, nrm, m = (a.copy() for a in state)
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        for h in range(H):
            if mode == 0:
                a = plain.sigmoid(pre[t, h * d:(h + 1) * d] + bias[h * d:(h + 1) * d]) ** p0
                S[h] = a[:, None] * S[h] + np.outer(k[t, h], v[t, h])
                out[t, h] = S[h].T @ q[t, h]
            else:
                i = p0 * np.tanh((pre[t, h] + bias[h]) / p0)
                f = plain.log_sigmoid(p0 * np.tanh((pre[t, H + h] + bias[H + h]) / p0))
                m_new = max(f + m[h], i)
                a, b = np.exp(f + m[h] - m_new), np.exp(i - m_new)
                S[h] = a * S[h] + b * np.outer(k[t, h], v[t, h])
                nrm[h] = a * nrm[h] + b * k[t, h]
                m[h] = m_new
                out[t, h] = S[h].T @ q[t, h] / (max(abs(nrm[h] @ q[t, h]), np.exp(-m_new)) + 1e-6)
    return out, (S, nrm, m)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("heads,dim,vdim", [(2, 16, 24), (1, 70, 40), (3, 5, 33), (2, 128, 64)])
def test_gated_recurrence_continues_across_portions(dtype, mode, heads, dim, vdim):
    """Portions longer than a stage, of one and two tokens, several requests in slots out of order, against the
    recurrence written out; a slot that is not in the batch keeps its state."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(heads * dim + mode)
    lens, slots = [45, 1, 19], [2, 0, 3]
    qk, vc = heads * dim, heads * vdim
    proj = [dev(rng.normal(size=(n, 2 * qk + vc + 5)) * 0.7, dtype) for n in lens]
    pre_cols = qk if mode == 0 else 2 * heads
    pre = [rng.normal(size=(n, pre_cols)) * 2.0 for n in lens]
    bias = rng.normal(size=pre_cols) + (2.0 if mode == 0 else 0.0)
    p0, q_scale = (1.0 / 3.0, dim ** -0.5) if mode == 0 else (4.0, dim ** -0.5)
    S = torch.full((4, heads, dim, vdim), 7.0, device=DEV)
    N, M = torch.full((4, heads, dim), 7.0, device=DEV), torch.full((4, heads), 7.0, device=DEV)
    for s in slots:
        S[s].zero_(); N[s].zero_(); M[s].zero_()
    want = []
    for x, z in zip(proj, pre):
        xf = x.float().cpu().numpy().astype(np.float64)
        n = xf.shape[0]
        o, _ = plain_recurrence(mode, xf[:, :qk].reshape(n, heads, dim) * q_scale, xf[:, qk:2 * qk].reshape(n, heads, dim),
                                xf[:, 2 * qk:2 * qk + vc].reshape(n, heads, vdim), z, bias, p0,
                                (np.zeros((heads, dim, vdim)), np.zeros((heads, dim)), np.zeros(heads)))
        want.append(o.reshape(n, vc))
    got, at = [[] for _ in lens], [0, 0, 0]
    for sizes in ([17, 1, 2], [1, 0, 16], [2, 0, 1], [25, 0, 0]):
        live = [i for i, n in enumerate(sizes) if n]
        x = torch.cat([proj[i][at[i]:at[i] + sizes[i]] for i in live])
        z = dev(np.concatenate([pre[i][at[i]:at[i] + sizes[i]] for i in live]))
        step = make_step([sizes[i] for i in live], slots=[slots[i] for i in live])
        out = torch.empty((x.shape[0], vc), device=DEV)
        ops.gated_recurrence(mode, x[:, :qk], x[:, qk:2 * qk], x[:, 2 * qk:2 * qk + vc], z, dev(bias), p0, q_scale, S, step, out,
                             heads, dim, vdim, True, N if mode else None, M if mode else None)
        o, j = out.cpu().numpy(), 0
        for i in live:
            got[i].append(o[j:j + sizes[i]]); j += sizes[i]; at[i] += sizes[i]
    for g, w in zip(got, want):
        assert close(np.concatenate(g), w, 2e-5)
    assert torch.all(S[1] == 7.0) and torch.all(N[1] == 7.0) and torch.all(M[1] == 7.0)
    before = S.clone()
    step = make_step([3], slots=[2])
    ops.gated_recurrence(mode, proj[0][:3, :qk], proj[0][:3, qk:2 * qk], proj[0][:3, 2 * qk:2 * qk + vc], dev(pre[0][:3]), dev(bias), p0,
                         q_scale, S, step, torch.empty((3, vc), device=DEV), heads, dim, vdim, False, N if mode else None,
                         M if mode else None)
    assert torch.equal(S, before)                                  # a run that must not write the state does not


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("heads,dim,vdim", [(2, 16, 24), (1, 70, 40), (2, 128, 64)])
def test_gated_recurrence_in_runs_of_tokens(mode, heads, dim, vdim):
    """Long portions are walked as runs of 64 tokens side by side: portions that end inside a run, at its edge and one
    behind it, next to a single token and a short portion, continue the same states as the walk token by token."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(heads * dim + mode + 7)
    lens, slots = [64 + 130 + 65, 1 + 1 + 3, 9 + 128 + 1], [1, 3, 0]
    qk, vc = heads * dim, heads * vdim
    proj = [dev(rng.normal(size=(n, 2 * qk + vc)) * 0.7) for n in lens]
    pre_cols = qk if mode == 0 else 2 * heads
    pre = [rng.normal(size=(n, pre_cols)) * 2.0 for n in lens]
    bias = rng.normal(size=pre_cols) + (2.0 if mode == 0 else 0.0)
    p0, q_scale = (0.5, dim ** -0.5) if mode == 0 else (6.0, dim ** -0.5)
    S, N, M = torch.zeros((4, heads, dim, vdim), device=DEV), torch.zeros((4, heads, dim), device=DEV), torch.zeros((4, heads), device=DEV)
    want = []
    for x, z in zip(proj, pre):
        xf, n = x.cpu().numpy().astype(np.float64), x.shape[0]
        o, _ = plain_recurrence(mode, xf[:, :qk].reshape(n, heads, dim) * q_scale, xf[:, qk:2 * qk].reshape(n, heads, dim),
                                xf[:, 2 * qk:].reshape(n, heads, vdim), z, bias, p0,
                                (np.zeros((heads, dim, vdim)), np.zeros((heads, dim)), np.zeros(heads)))
        want.append(o.reshape(n, vc))
    ws = torch.empty((ops.gated_recurrence_workspace(4, 512, heads, dim, vdim),), device=DEV)
    got, at = [[] for _ in lens], [0, 0, 0]
    for sizes in ([64, 1, 9], [130, 1, 128], [65, 3, 1]):
        x = torch.cat([proj[i][at[i]:at[i] + sizes[i]] for i in range(3)])
        z = dev(np.concatenate([pre[i][at[i]:at[i] + sizes[i]] for i in range(3)]))
        step = make_step(sizes, slots=slots)
        out = torch.empty((x.shape[0], vc), device=DEV)
        ops.gated_recurrence(mode, x[:, :qk], x[:, qk:2 * qk], x[:, 2 * qk:], z, dev(bias), p0, q_scale, S, step, out, heads, dim, vdim,
                             True, N if mode else None, M if mode else None, ws if max(sizes) >= ops.RECURRENCE_CHUNKED_MIN else None)
        o, j = out.cpu().numpy(), 0
        for i in range(3):
            got[i].append(o[j:j + sizes[i]]); j += sizes[i]; at[i] += sizes[i]
    for g, w in zip(got, want):
        assert close(np.concatenate(g), w, 3e-5)
    assert float(S[2].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,head_dim,per_head,act", [(3, 24, False, "silu"), (2, 40, True, "sigmoid"), (1, 7, True, "silu"), (5, 64, False, "sigmoid")])
def test_head_norm_gate_with_weights_per_head_and_a_scale(dtype, heads, head_dim, per_head, act):
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(head_dim)
    n, cols = 11, heads * head_dim
    x, g = rng.normal(size=(n, cols)) * 3, dev(rng.normal(size=(n, cols)), dtype)
    w = rng.normal(size=cols if per_head else head_dim) + 1.0
    out = torch.empty((n, cols), dtype=dtype, device=DEV)
    ops.head_norm_gate_scaled(dev(x), dev(w), 1e-5, g, out, heads, head_dim, act, 0.7)
    gf = g.float().cpu().numpy().astype(np.float64)
    normed = plain.unit_rms(x.reshape(n, heads, head_dim), 1e-5)
    normed = normed * (w.reshape(heads, head_dim) if per_head else w)
    want = 0.7 * normed.reshape(n, cols) * (plain.silu(gf) if act == "silu" else plain.sigmoid(gf))
    assert close(out.float().cpu().numpy(), want, 2e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("experts,top,groups,keep", [(16, 2, 2, 1), (6, 2, 3, 2), (5, 3, 1, 1), (4, 2, 4, 3), (1, 1, 1, 1), (64, 6, 8, 3),
                                                     (40, 40, 4, 4)])
def test_group_limited_router(experts, top, groups, keep):
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(experts)
    n = 50
    logits = rng.normal(size=(n, experts + 3)) * 2.0
    logits[3, :experts] = 0.25                                     # ties everywhere: lower groups and lower experts win
    ld = dev(logits)
    choice = torch.empty((n, top), dtype=torch.int32, device=DEV)
    weight = torch.empty((n, top), device=DEV)
    ops.moe_route_grouped(ld, experts, top, groups, keep, 2.5, choice, weight)
    z = ld.cpu().numpy().astype(np.float64)[:, :experts]
    s = plain.sigmoid(z)
    for t in range(n):
        chosen = plain.group_limited_choice(s[t], top, groups, keep)
        assert choice[t].tolist() == chosen, t
        assert close(weight[t].cpu().numpy(), s[t, chosen] / (s[t, chosen].sum() + 1e-20) * 2.5, 3e-6)


def test_weighted_sum_with_a_gated_extra_term():
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(5)
    n, top, width = 19, 3, 50
    pair_out, w = rng.normal(size=(n * top, width)), rng.normal(size=(n, top))
    extra, logits, y0 = rng.normal(size=(n, width)), rng.normal(size=(n, 7)), rng.normal(size=(n, width))
    base = np.einsum("tk,tkc->tc", w, pair_out.reshape(n, top, width))
    ld = dev(logits)
    for accumulate in (False, True):
        y = dev(y0)
        ops.moe_combine(dev(pair_out), dev(w), y, accumulate, None, dev(extra), ld[:, 6:])
        want = base + plain.sigmoid(logits[:, 6:7]) * extra + (y0 if accumulate else 0.0)
        assert close(y.cpu().numpy(), want, 3e-6)
    y = dev(y0)
    ops.moe_combine(dev(pair_out), dev(w), y, False, None, dev(extra))
    assert close(y.cpu().numpy(), base + extra, 3e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("limit,alpha,shift", [(1.5, 1.702, 1.0), (float("inf"), 1.0, 0.0), (0.4, 0.5, -0.25)])
def test_gated_activation_family(dtype, limit, alpha, shift):
    """g sigmoid(alpha g) (u + shift) with both clamped: alone, behind a small product and in the epilogue of a large one;
    without a limit, alpha = 1 and no shift it is silu(gate) * up."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(3)
    inner, width = 64, 96
    wg, wu = dev(rng.normal(size=(inner, width)) * 0.2, dtype), dev(rng.normal(size=(inner, width)) * 0.2, dtype)
    w_cat = torch.cat([wg, wu]).contiguous()
    w_int = ops.interleave_gate_up(wg, wu, 4)

    def want(x):
        xf, g, u = (t.float().cpu().numpy().astype(np.float64) for t in (x, wg, wu))
        gate, up = np.minimum(xf @ g.T, limit), np.clip(xf @ u.T, -limit, limit)
        return gate * plain.sigmoid(alpha * gate) * (up + shift)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    for n in (5, 200):
        x = dev(rng.normal(size=(n, width)), dtype)
        for w, granule in ((w_cat, inner), (w_int, 4)):
            out, gu = torch.empty((n, inner), dtype=dtype, device=DEV), torch.empty((n, 2 * inner), dtype=dtype, device=DEV)
            ops.linear_clamped_glu(x, w, out, granule, gu, limit, alpha, shift)
            assert close(out.float().cpu().numpy(), want(x), tol), (n, granule)
    if limit == float("inf"):
        x = dev(rng.normal(size=(7, width)), dtype)
        xf, g, u = (t.float().cpu().numpy().astype(np.float64) for t in (x, wg, wu))
        assert close(want(x), plain.silu(xf @ g.T) * (xf @ u.T), 1e-12)
