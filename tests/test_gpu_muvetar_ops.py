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
