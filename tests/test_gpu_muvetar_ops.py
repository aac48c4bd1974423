"""The kernels behind the Muvetar parts, each against a few lines of plain float64 arithmetic."""
import numpy as np
import pytest
import torch

import plain_muvetar as plain
from test_gpu_dobelix_ops import DEV, make_step

pytestmark = pytest.mark.gpu


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def close(got, want, tol):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return np.max(np.abs(got - want)) <= tol * max(np.max(np.abs(want)), 1e-30)


@pytest.mark.parametrize("width", [6, 64, 250])
def test_sinusoid_softcap_scaled_sum_and_depth_average(width):
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(width)
    n = 37
    pos = rng.integers(0, 5000, size=n)
    x = rng.normal(size=(n, width))
    xd = dev(x)
    ops.add_sinusoid(xd, dev(pos, torch.int32), 10000.0)
    want = x.copy()
    for t, p in enumerate(pos):
        want[t] += plain.sinusoid(1, width, first=int(p))[0]
    assert close(xd.cpu().numpy(), want, 2e-6)
    logits = rng.normal(size=(n, width)) * 9.0
    ld = dev(logits)
    ops.softcap_(ld, 4.0)
    assert close(ld.cpu().numpy(), 4.0 * np.tanh(logits / 4.0), 2e-6)
    # residual += m * y, and the norm of the sum
    y, r, w = rng.normal(size=(n, width)), rng.normal(size=(n, width)), rng.normal(size=width) + 1.0
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 8e-3)):
        rd, out = dev(r), torch.empty((n, width), dtype=dtype, device=DEV)
        ops.scaled_add_norm(dev(y), 0.3, rd, dev(w), 1e-5, out)
        assert close(rd.cpu().numpy(), r + 0.3 * y, 2e-6)
        assert close(out.float().cpu().numpy(), plain.rms_norm(r + 0.3 * y, w, 1e-5), tol)
    rd = dev(r)
    ops.scaled_add(dev(y), -1.5, rd)
    assert close(rd.cpu().numpy(), r - 1.5 * y, 2e-6)
    # the depth average over a history of more rows than the step has
    hist = rng.normal(size=(5, n + 3, width))
    a = rng.normal(size=4)
    for with_y in (True, False):
        hd, rd = dev(hist), dev(r)
        ops.depth_average(rd, dev(y) if with_y else None, 0.5, hd, dev(a), 2)
        result = r + 0.5 * y if with_y else r
        assert close(hd[3, :n].cpu().numpy(), result, 2e-6) and torch.equal(hd[4], dev(hist[4])) and torch.equal(hd[3, n:], dev(hist[3, n:]))
        assert close(rd.cpu().numpy(), a[0] * hist[0, :n] + a[1] * hist[1, :n] + a[2] * hist[2, :n] + a[3] * result, 4e-6)


def plain_mingru_states(pz, px, pg, bz, bx, S):
    out = np.zeros(pz.shape)
    for t in range(pz.shape[0]):
        z = plain.sigmoid(pz[t] + bz)
        u = px[t] + bx
        S = (1 - z) * S + z * np.where(u >= 0, u + 0.5, plain.sigmoid(u))
        out[t] = S * plain.silu(pg[t])
    return out, S


@pytest.mark.parametrize("channels", [5, 64, 200])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mingru_continues_across_portions(channels, dtype):
    """Portions longer than one warp's run, of one and two tokens, several requests in slots out of order."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(channels)
    lens, slots = [150, 1, 40], [2, 0, 3]
    cols = 3 * channels + 4
    proj = [dev(rng.normal(size=(n, cols)) * 1.5, dtype) for n in lens]
    bz, bx = rng.normal(size=channels), rng.normal(size=channels)
    state = torch.full((4, channels), 7.0, device=DEV)
    for s in slots:
        state[s].zero_()
    want, final = [], []
    for p in proj:
        p = p.double().cpu().numpy()
        o, S = plain_mingru_states(p[:, 2:2 + channels], p[:, 2 + channels:2 + 2 * channels], p[:, 4 + 2 * channels:], bz, bx, np.zeros(channels))
        want.append(o); final.append(S)
    got, at = [[] for _ in lens], [0, 0, 0]
    for sizes in ([97, 1, 2], [1, 0, 17], [2, 0, 1], [50, 0, 20]):
        live = [i for i, n in enumerate(sizes) if n]
        x = torch.cat([proj[i][at[i]:at[i] + sizes[i]] for i in live])
        step = make_step([sizes[i] for i in live], slots=[slots[i] for i in live])
        out = torch.empty((x.shape[0], channels), dtype=dtype, device=DEV)
        ops.mingru(x, 2, 2 + channels, 4 + 2 * channels, dev(bz), dev(bx), state, step, out, channels)
        o, k = out.float().cpu().numpy(), 0
        for i in live:
            got[i].append(o[k:k + sizes[i]]); k += sizes[i]; at[i] += sizes[i]
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    for i in range(3):
        assert close(np.concatenate(got[i]), want[i], tol)
        assert close(state[slots[i]].cpu().numpy(), final[i], 2e-5)
    assert torch.all(state[1] == 7.0)
    # a run that does not keep its state (a reader of another run's cache) leaves the slot as it was
    before = state.clone()
    ops.mingru(proj[0][:9], 2, 2 + channels, 4 + 2 * channels, dev(bz), dev(bx), state, make_step([9], slots=[2]),
               torch.empty((9, channels), dtype=dtype, device=DEV), channels, write_state=False)
    assert torch.equal(state, before)


def plain_scan(x, dtp, B, C, z, a_log, D, bias, S, out_scale):
    A = -np.exp(a_log)
    out = np.zeros(x.shape)
    for t in range(x.shape[0]):
        dt = plain.softplus(dtp[t] + bias)
        S = np.exp(dt[:, None] * A) * S + (dt * x[t])[:, None] * B[t][None, :]
        out[t] = (S @ C[t] + D * x[t]) * plain.silu(z[t]) * out_scale
    return out, S


@pytest.mark.parametrize("channels,n_state", [(6, 1), (40, 3), (64, 16), (33, 24), (16, 130)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selective_scan_continues_across_portions(channels, n_state, dtype):
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(channels + n_state)
    lens, slots = [130, 1, 35], [1, 3, 0]
    r = 3                                   # columns in front of B in the rows that hold B and C
    x = [dev(rng.normal(size=(n, channels)), dtype) for n in lens]
    z = [dev(rng.normal(size=(n, channels)), dtype) for n in lens]
    bc = [dev(rng.normal(size=(n, r + 2 * n_state)) * 0.5, dtype) for n in lens]
    dtp = [dev(rng.normal(size=(n, channels)) - 1.0) for n in lens]
    a_log, D, bias = rng.uniform(-3.0, 1.0, size=(channels, n_state)), rng.normal(size=channels), rng.normal(size=channels)
    state = torch.full((4, channels, n_state), 7.0, device=DEV)
    for s in slots:
        state[s].zero_()
    f64 = lambda t: t.double().cpu().numpy()
    want, final = [], []
    for i in range(3):
        b = f64(bc[i])
        o, S = plain_scan(f64(x[i]), f64(dtp[i]), b[:, r:r + n_state], b[:, r + n_state:], f64(z[i]), a_log, D, bias,
                          np.zeros((channels, n_state)), 0.7)
        want.append(o); final.append(S)
    got, at = [[] for _ in lens], [0, 0, 0]
    for sizes in ([70, 1, 2], [1, 0, 17], [2, 0, 1], [57, 0, 15]):
        live = [i for i, n in enumerate(sizes) if n]
        cut = lambda ts: torch.cat([ts[i][at[i]:at[i] + sizes[i]] for i in live])
        step = make_step([sizes[i] for i in live], slots=[slots[i] for i in live])
        xs = cut(x)
        out = torch.empty_like(xs)
        ops.selective_scan(xs, cut(dtp), cut(bc), r, r + n_state, cut(z), dev(a_log), dev(D), dev(bias), state, step, out, 0.7)
        o, k = out.float().cpu().numpy(), 0
        for i in live:
            got[i].append(o[k:k + sizes[i]]); k += sizes[i]; at[i] += sizes[i]
    tol = 3e-5 if dtype == torch.float32 else 1.5e-2
    for i in range(3):
        assert close(np.concatenate(got[i]), want[i], tol)
        assert close(state[slots[i]].cpu().numpy(), final[i], 3e-5)
    assert torch.all(state[2] == 7.0)


@pytest.mark.parametrize("experts,top", [(1, 1), (5, 3), (16, 2), (64, 8), (130, 4), (7, 7)])
def test_router_takes_the_largest_scores_and_the_plan_orders_every_pair(experts, top):
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(experts)
    n = 77
    logits = rng.normal(size=(n, experts)) * 2.0
    logits[5, :] = 0.25                              # a tie everywhere: the lowest experts win
    choice = torch.empty((n, top), dtype=torch.int32, device=DEV)
    weight = torch.empty((n, top), dtype=torch.float32, device=DEV)
    ops.moe_route(dev(logits), top, 1.7, choice, weight)
    s = np.exp(logits - logits.max(axis=1, keepdims=True))
    s /= s.sum(axis=1, keepdims=True)
    order = np.argsort(-s, axis=1, kind="stable")[:, :top]
    assert np.array_equal(choice.cpu().numpy(), order)
    assert close(weight.cpu().numpy(), np.take_along_axis(s, order, axis=1) * 1.7, 1e-5)
    assert choice[5].tolist() == list(range(top))
    tiles = ops.moe_max_tiles(n * top, experts)
    i32 = lambda k: torch.full((k,), -7, dtype=torch.int32, device=DEV)
    offsets, places, tile_expert, tile_row = i32(experts + 1), i32(n * top), i32(tiles), i32(tiles)
    ops.moe_plan(choice, experts, offsets, places, tile_expert, tile_row)
    off, pl = offsets.cpu().numpy(), places.cpu().numpy()
    flat = order.reshape(-1)
    assert off[0] == 0 and off[-1] == n * top and sorted(pl.tolist()) == list(range(n * top))
    for e in range(experts):
        assert off[e + 1] - off[e] == int((flat == e).sum()) and all(flat[p] == e for p in pl[off[e]:off[e + 1]])
    rows = ops.moe_tile_rows()
    covered = []
    for e, r0 in zip(tile_expert.tolist(), tile_row.tolist()):
        if e >= 0:
            assert off[e] <= r0 < off[e + 1] and (r0 - off[e]) % rows == 0
            covered.extend(range(r0, min(r0 + rows, off[e + 1])))
    assert sorted(covered) == list(range(n * top))


@pytest.mark.parametrize("n,experts,top,inner,width", [(1, 4, 2, 24, 40), (70, 5, 3, 20, 36), (200, 16, 2, 64, 128), (33, 3, 3, 72, 264)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_against_a_loop_over_tokens(n, experts, top, inner, width, dtype):
    """Every (token, chosen expert) pair through the expert's two products and its clamped gate, weighted and summed;
    limits small enough that both clamps are at work; one expert gets no token at all."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(n + experts)
    limit, alpha = 0.8, 1.702
    x = dev(rng.normal(size=(n, width)), dtype)
    wg, wu = (dev(rng.normal(size=(experts, inner, width)) * 0.2, dtype) for _ in range(2))
    wd = dev(rng.normal(size=(experts, width, inner)) * 0.2, dtype)
    logits = rng.normal(size=(n, experts))
    if experts > top:
        logits[:, experts - 1] = -50.0
    choice = torch.empty((n, top), dtype=torch.int32, device=DEV)
    weight = torch.empty((n, top), dtype=torch.float32, device=DEV)
    ops.moe_route(dev(logits), top, 2.0, choice, weight)
    tiles = ops.moe_max_tiles(n * top, experts)
    i32 = lambda k: torch.zeros((k,), dtype=torch.int32, device=DEV)
    offsets, places, tile_expert, tile_row = i32(experts + 1), i32(n * top), i32(tiles), i32(tiles)
    ops.moe_plan(choice, experts, offsets, places, tile_expert, tile_row)
    hidden = torch.empty((n * top, inner), dtype=dtype, device=DEV)
    pair_out = torch.empty((n * top, width), dtype=torch.float32, device=DEV)
    ops.moe_experts(x, top, wg, wu, wd, limit, offsets, places, tile_expert, tile_row, hidden, pair_out, alpha)
    y0 = rng.normal(size=(n, width))
    f64 = lambda t: t.double().cpu().numpy()
    X, G, U, Dn, ch, wt = f64(x), f64(wg), f64(wu), f64(wd), choice.cpu().numpy(), f64(weight)
    want = np.zeros((n, width))
    clamped = 0
    for t in range(n):
        for k in range(top):
            e = ch[t, k]
            g, u = G[e] @ X[t], U[e] @ X[t]
            clamped += int((g > limit).sum() + (np.abs(u) > limit).sum())
            g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
            want[t] += wt[t, k] * (Dn[e] @ (g / (1 + np.exp(-alpha * g)) * (u + 1)))
    assert clamped > 0
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    for accumulate in (False, True):
        y = dev(y0)
        ops.moe_combine(pair_out, weight, y, accumulate)
        assert close(y.cpu().numpy(), want + (y0 if accumulate else 0.0), tol)


@pytest.mark.parametrize("inner", [8, 100])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gate(inner, dtype):
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(inner)
    gu = dev(rng.normal(size=(19, 2 * inner)) * 3.0, dtype)
    out = torch.empty((19, inner), dtype=dtype, device=DEV)
    ops.clamped_glu(gu, out, 1.5, 1.702)
    v = gu.double().cpu().numpy()
    g, u = np.minimum(v[:, :inner], 1.5), np.clip(v[:, inner:], -1.5, 1.5)
    assert close(out.float().cpu().numpy(), g / (1 + np.exp(-1.702 * g)) * (u + 1), 2e-6 if dtype == torch.float32 else 8e-3)


class DistanceBatch:
    """A paged cache with shuffled pages, keys of ``d`` and values of ``dv`` elements, stale content in the unused places,
    and a step of ``new[i]`` tokens for request i with ``before[i]`` tokens cached."""

    def __init__(self, dtype, heads, kv, d, dv, page, before, new, seed=0):
        g = torch.Generator().manual_seed(seed)
        r = len(before)
        total = [b + n for b, n in zip(before, new)]
        max_pages = max(-(-t // page) for t in total) + 1
        n_pages = r * max_pages + 2
        perm = torch.randperm(n_pages, generator=g)[:r * max_pages].reshape(r, max_pages)
        self.block_table = perm.to(torch.int32).to(DEV)
        self.kp = (torch.randn(n_pages, kv, page, d, generator=g) * 30).to(dtype).to(DEV)
        self.vp = (torch.randn(n_pages, kv, page, dv, generator=g) * 30).to(dtype).to(DEV)
        self.k = [torch.randn(t, kv, d, generator=g).to(dtype) for t in total]
        self.v = [torch.randn(t, kv, dv, generator=g).to(dtype) for t in total]
        for i in range(r):
            for first in range(0, total[i], page):
                pg, m = int(perm[i, first // page]), min(page, total[i] - first)
                self.kp[pg, :, :m] = self.k[i][first:first + m].transpose(0, 1).to(DEV)
                self.vp[pg, :, :m] = self.v[i][first:first + m].transpose(0, 1).to(DEV)
        self.n, self.r, self.before, self.new = sum(new), r, before, new
        self.q = (torch.randn(self.n, heads * d, generator=g) * 1.5).to(dtype).to(DEV)
        i32 = lambda x: torch.tensor(np.asarray(x), dtype=torch.int32, device=DEV)
        self.cu_tokens, self.slots, self.context_before = i32(np.concatenate([[0], np.cumsum(new)])), i32(np.arange(r)), i32(before)
        self.positions = i32(np.concatenate([np.arange(b, b + k) for b, k in zip(before, new)]))
        self.slot_of_token = i32(np.concatenate([np.full(k, i) for i, k in enumerate(new)]))
        self.max_new, self.max_context, self.attention_splits = max(new), max(total), None
        self.heads, self.kv, self.d, self.dv = heads, kv, d, dv

    def reference(self, scale, r1, r2):
        out = np.zeros((self.n, self.heads, self.dv))
        q = self.q.double().cpu().numpy().reshape(self.n, self.heads, self.d)
        group, at = self.heads // self.kv, 0
        for i in range(self.r):
            k, v = self.k[i].double().numpy(), self.v[i].double().numpy()
            for t in range(self.new[i]):
                pos = self.before[i] + t
                far = pos - np.arange(pos + 1)
                for h in range(self.heads):
                    s = k[:pos + 1, h // group] @ q[at, h] * scale - r1[h] * np.log(1.0 + r2[h] * far)
                    w = np.exp(s - s.max())
                    out[at, h] = (w / w.sum()) @ v[:pos + 1, h // group]
                at += 1
        return out.reshape(self.n, -1)


@pytest.mark.parametrize("heads,kv,d,dv,page", [(4, 2, 16, 16, 16), (6, 2, 24, 8, 16), (3, 1, 40, 72, 32), (8, 8, 64, 64, 64),
                                                (16, 2, 64, 128, 64), (2, 1, 136, 104, 16), (5, 5, 8, 200, 16)])
@pytest.mark.parametrize("before,new", [([0, 3, 40, 129], [37, 1, 17, 2]), ([0, 63, 64, 700], [1, 1, 1, 1])])
def test_distance_attention_on_the_tensor_cores(heads, kv, d, dv, page, before, new):
    """Key and value sizes that differ and are not the tile's size; portions beside single tokens; decode steps with and
    without their keys split among CTAs; the float32 kernel on the CUDA cores beside it."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(heads + d)
    r1, r2 = rng.uniform(0.2, 1.5, size=heads), rng.uniform(0.05, 2.0, size=heads)
    scale, out_scale = 0.4 / np.sqrt(d), 0.7
    assert ops.distance_attention_tile(d, dv) >= max(d, dv)
    for dtype, tol in ((torch.bfloat16, 1.5e-2), (torch.float32, 2e-5)):
        b = DistanceBatch(dtype, heads, kv, d, dv, page, before, new, seed=d)
        want = b.reference(scale, r1, r2) * out_scale
        tile = ops.distance_attention_tile(d, dv)
        for splits in ((None, 3, 7) if max(new) == 1 and dtype == torch.bfloat16 else (None,)):
            b.attention_splits = splits
            scratch = torch.full((b.n * heads * (splits or 1) * (tile + 2),), float("nan"), dtype=torch.float32, device=DEV) if splits else None
            out = torch.full((b.n, heads * dv), float("nan"), dtype=dtype, device=DEV)
            ops.distance_attention(b.q, b.kp, b.vp, b.block_table, page, b, out, heads, kv, d, dv, scale, dev(r1), dev(r2), out_scale,
                                   0, scratch)
            assert close(out.float().cpu().numpy(), want, tol), (dtype, splits)


def test_distance_penalty_decides_between_a_near_and_a_far_key():
    """Two keys with the same score, one at distance 1 and one at distance 300: the weights follow (1 + r2 * distance)^-r1
    alone, on both kernels."""
    from hfee_b200.kernels import ops
    heads, kv, d, dv, page, ctx = 2, 1, 16, 16, 16, 302
    r1, r2 = np.array([1.0, 0.5]), np.array([0.5, 2.0])
    for dtype, tol in ((torch.bfloat16, 1e-2), (torch.float32, 1e-5)):
        b = DistanceBatch(dtype, heads, kv, d, dv, page, [ctx - 1], [1], seed=1)
        k = torch.zeros(ctx, kv, d)
        v = torch.zeros(ctx, kv, dv)
        k[:, 0, 0] = -40.0                                  # every other key is out of the question
        k[ctx - 2, 0, 0] = k[ctx - 1 - 300, 0, 0] = 0.0
        k[ctx - 1, 0, 0] = -40.0
        v[ctx - 2, 0, 0], v[ctx - 1 - 300, 0, 1] = 1.0, 1.0
        for first in range(0, ctx, page):
            pg, m = int(b.block_table[0, first // page]), min(page, ctx - first)
            b.kp[pg, :, :m] = k[first:first + m].transpose(0, 1).to(dtype).to(DEV)
            b.vp[pg, :, :m] = v[first:first + m].transpose(0, 1).to(dtype).to(DEV)
        q = torch.zeros(1, heads * d)
        q[0, 0] = q[0, d] = 1.0
        out = torch.empty((1, heads * dv), dtype=dtype, device=DEV)
        ops.distance_attention(q.to(dtype).to(DEV), b.kp, b.vp, b.block_table, page, b, out, heads, kv, d, dv, 1.0, dev(r1), dev(r2))
        got = out.float().cpu().numpy().reshape(heads, dv)
        for h in range(heads):
            near, far = (1 + r2[h] * 1) ** -r1[h], (1 + r2[h] * 300) ** -r1[h]
            assert abs(got[h, 0] - near / (near + far)) < tol and abs(got[h, 1] - far / (near + far)) < tol


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("n,experts,top,inner,width", [(1, 4, 2, 16, 32), (9, 3, 3, 24, 40), (300, 5, 2, 72, 64), (700, 2, 1, 136, 264)])
def test_experts_on_the_tensor_cores(n, experts, top, inner, width, fused):
    """The grouped products over tiles of 128 places against a loop over tokens: experts with no token, with fewer than a
    tile and with several tiles; NaN in the scratch rows that hold no pair.  ``fused``: gate and up rows in runs of four
    and the activation in the first product's epilogue."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(n)
    dtype, limit, alpha = torch.bfloat16, 0.8, 1.702
    assert ops.moe_experts_grouped_ok(dtype, width, inner)
    x = dev(rng.normal(size=(n, width)), dtype)
    wgu = dev(rng.normal(size=(experts, 2 * inner, width)) * 0.2, dtype)
    wd = dev(rng.normal(size=(experts, width, inner)) * 0.2, dtype)
    logits = rng.normal(size=(n, experts))
    if experts > top:
        logits[:, experts - 1] = -50.0
    choice = torch.empty((n, top), dtype=torch.int32, device=DEV)
    weight = torch.empty((n, top), dtype=torch.float32, device=DEV)
    ops.moe_route(dev(logits), top, 2.0, choice, weight)
    tiles = ops.moe_tiles_grouped(n * top, experts)
    rows = tiles * ops.GROUPED_TILE_ROWS
    i32 = lambda k: torch.full((k,), 12345, dtype=torch.int32, device=DEV)
    nan = lambda c, dt: torch.full((rows, c), float("nan"), dtype=dt, device=DEV)
    place, row_pair, tile_group = i32(n * top), i32(rows), i32(tiles)
    rows_out = nan(width, torch.float32)
    if fused:
        ops.moe_experts_grouped(x, top, choice, ops.interleave_gate_up(wgu[:, :inner], wgu[:, inner:]), wd, limit, place, row_pair,
                                tile_group, nan(width, dtype), None, nan(inner, dtype), rows_out, alpha)
    else:
        ops.moe_experts_grouped(x, top, choice, wgu, wd, limit, place, row_pair, tile_group, nan(width, dtype), nan(2 * inner, dtype),
                                nan(inner, dtype), rows_out, alpha)
    ops.check_status()
    pl, rp, tg, ch = place.cpu().numpy(), row_pair.cpu().numpy(), tile_group.cpu().numpy(), choice.cpu().numpy()
    assert len(set(pl)) == n * top                                  # every pair has a row of its own, in a tile of its expert
    for pair, row in enumerate(pl):
        assert rp[row] == pair and tg[row // ops.GROUPED_TILE_ROWS] == ch[pair // top, pair % top]
    f64 = lambda t: t.double().cpu().numpy()
    X, GU, Dn, wt = f64(x), f64(wgu), f64(wd), f64(weight)
    want = np.zeros((n, width))
    for t in range(n):
        for k in range(top):
            e = ch[t, k]
            g, u = np.minimum(GU[e, :inner] @ X[t], limit), np.clip(GU[e, inner:] @ X[t], -limit, limit)
            want[t] += wt[t, k] * (Dn[e] @ (g / (1 + np.exp(-alpha * g)) * (u + 1)))
    y0 = rng.normal(size=(n, width))
    for accumulate in (False, True):
        y = dev(y0)
        ops.moe_combine(rows_out, weight, y, accumulate, place)
        assert close(y.cpu().numpy(), want + (y0 if accumulate else 0.0), 2e-2)


@pytest.mark.parametrize("n,inner,width,limit", [(65, 8, 16, 0.5), (200, 72, 64, 0.8), (300, 520, 264, 7.0), (2, 24, 40, 0.8)])
def test_gate_up_product_with_the_clamped_activation(n, inner, width, limit):
    """The gate/up product whose epilogue applies the clamped gated activation (prompt portions) and its route through
    a buffer (few tokens), against float64; the limit is low enough to cut some gates and ups."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(inner)
    dtype, alpha = torch.bfloat16, 1.702
    x = dev(rng.normal(size=(n, width)), dtype)
    wg, wu = dev(rng.normal(size=(inner, width)) * 0.3, dtype), dev(rng.normal(size=(inner, width)) * 0.3, dtype)
    out = torch.full((n, inner), float("nan"), dtype=dtype, device=DEV)
    scratch = torch.empty((n, 2 * inner), dtype=dtype, device=DEV)
    ops.linear_clamped_glu(x, ops.interleave_gate_up(wg, wu), out, ops.SWIGLU_GRANULE, scratch, limit, alpha)
    ops.check_status()
    X = x.double().cpu().numpy()
    g = np.minimum(X @ wg.double().cpu().numpy().T, limit)
    u = np.clip(X @ wu.double().cpu().numpy().T, -limit, limit)
    assert (g == limit).any() and (np.abs(u) == limit).any()
    assert close(out.float().cpu().numpy(), g / (1 + np.exp(-alpha * g)) * (u + 1), 2e-2)
