"""Muvetar without a GPU: reading config.json, tensor names and shapes, what the mixers ask of the cache manager, and the
plain implementation's own consistency (each mechanism against a closed form or a second way of computing it)."""
import json

import numpy as np
import pytest

import muvetar_util as mu
import plain_muvetar as plain


def test_config_reads_every_size_and_refuses_what_it_does_not_know():
    from hfee_b200.config import ConfigError, resolve
    arch, cfg = resolve(mu.MUV_A)
    assert arch.name == "Muvetar" and cfg.width == 64 and cfg.vocab == 200 and cfg.eps == 1e-5
    assert cfg.residual_mult == 0.5 and cfg.logit_softcap == 15.0
    assert [l.type for l in cfg.layers] == ["parallel", "mingru", "mingru", "parallel"]
    p0, p3 = cfg.layers[0].mixer, cfg.layers[3].mixer
    assert (p0.left.heads, p0.left.kv_heads, p0.left.dim, p0.left.vdim, p0.left.scale) == (4, 2, 16, 24, 0.25)
    assert (p0.right.inner, p0.right.state, p0.right.dt_rank, p0.right.taps) == (48, 6, 5, 3)
    assert (p0.left_scale, p0.right_scale, p3.left_scale, p3.right_scale) == (1.3, 0.8, 0.7, 1.2)
    assert cfg.layers[1].mixer.width == 80 and cfg.layers[2].mlp is None
    m0, m3 = cfg.layers[0].mlp, cfg.layers[3].mlp
    assert (m0.experts, m0.top, m0.router_scale, m0.expert.ff, m0.expert.limit) == (8, 2, 2.0, 24, 1.0)
    assert (m0.shared.ff, m0.shared.limit) == (40, 1.5) and m3.shared is None and (m3.experts, m3.top) == (5, 3)
    with pytest.raises(ConfigError, match="not a mixer"):
        resolve(dict(mu.MUV_A, layers=[{"type": "attention", "mixer": {}, "mlp": None}]))
    for key in ("norm", "residual_mult", "logit_softcap", "vocab", "width"):
        with pytest.raises(ConfigError, match=key):
            resolve({k: v for k, v in mu.MUV_A.items() if k != key})
    with pytest.raises(ConfigError, match="multiple of kv_heads"):
        resolve(mu.config(32, 50, [mu.parallel(3, 2, 8, 8, 0.3, 16, 4, 2, 2)]))
    with pytest.raises(ConfigError, match="not a feed-forward"):
        resolve(mu.config(32, 50, [dict(mu.mingru(16), mlp={"kind": "dense", "ff": 8})]))
    with pytest.raises(ConfigError, match="exceeds"):
        resolve(mu.config(32, 50, [mu.mingru(16, mlp=mu.moe(3, 4, 8, 1.0, 1.0))]))
    with pytest.raises(ConfigError, match="state"):
        bad = mu.parallel(2, 1, 8, 8, 0.3, 16, 4, 2, 2)
        del bad["mixer"]["right"]["state"]
        resolve(mu.config(32, 50, [bad]))


def test_layout_names_and_cache_needs():
    from hfee_b200 import CacheBundle, FixedState, PagedKV
    from hfee_b200.config import resolve
    from hfee_b200.parts.model import model_tensor_needs
    arch, cfg = resolve(mu.MUV_B)
    spec = arch.build_spec(cfg)
    needs = model_tensor_needs(spec)
    assert needs["embed"].shape == (310, 96) and needs["head"].shape == (310, 96) and needs["final.norm"].shape == (96,)
    assert needs["l0.mix.z"].shape == (96, 96) and needs["l0.mix.z.b"].shape == (96,) and needs["l0.mix.o"].shape == (96, 96)
    assert needs["l3.mix.g"].shape == (56, 96) and needs["l3.mix.o"].shape == (96, 56)
    assert needs["l1.mix.left.q"].shape == (72, 96) and needs["l1.mix.left.v"].shape == (24, 96)
    assert needs["l2.mix.left.k"].shape == (32, 96) and needs["l2.mix.left.o"].shape == (96, 96) and needs["l2.mix.left.r1"].shape == (6,)
    assert needs["l2.mix.right.in"].shape == (200, 96) and needs["l2.mix.right.conv"].shape == (100, 5)
    assert needs["l2.mix.right.x"].shape == (2 + 40, 100) and needs["l2.mix.right.dt"].shape == (100, 2)
    assert needs["l2.mix.right.A_log"].shape == (100, 20) and needs["l2.mix.right.D"].shape == (100,)
    assert needs["l1.mix.right.conv"].shape == (64, 1) and needs["l1.mix.right.conv.b"].shape == (64,)
    assert [needs[f"l{i}.dwa"].shape for i in range(5)] == [(2,), (3,), (4,), (5,), (6,)]
    assert "l1.norm2" not in needs and "l4.mlp.router" not in needs and "l2.mlp.shared.gate" not in needs
    assert needs["l0.mlp.router"].shape == (4, 96) and needs["l0.mlp.e3.down"].shape == (96, 40) and "l0.mlp.e4.gate" not in needs
    assert needs["l3.mlp.shared.up"].shape == (8, 96) and needs["l2.mlp.e11.gate"].shape == (8, 96)
    # what the mixers ask of the cache manager: pages for the attention branch with values of their own size, the scan's
    # state and its convolution's last inputs, the minGRU's one state row; built without a device
    mixers = [layer.parts["mixer"][1] for layer in spec.layers]
    assert [m.kind for m in mixers] == ["mingru", "parallel", "parallel", "mingru", "mingru"]
    assert PagedKV(2, 16, None, None, 16) != PagedKV(2, 16, None, None, 8)
    bundle = CacheBundle.of(PagedKV(3, 24, None, None, 8), **{"right.conv": FixedState((0, 64)), "right.recurrent": FixedState((64, 3))})
    assert bundle.state_map()["right.recurrent"].shape == (64, 3) and bundle.paged.value_dim == 8


def test_cache_manager_holds_pages_and_states_of_a_parallel_mixer_and_zeroes_a_reused_slot():
    import torch
    from hfee_b200 import CacheBundle, CacheManager, FixedState, PagedKV
    needs = {0: CacheBundle.of(PagedKV(2, 16, None, None, 24), **{"right.conv": FixedState((2, 48), "float32"),
                                                                     "right.recurrent": FixedState((48, 6), "float32")}),
             1: FixedState((80,), "float32"),
             2: CacheBundle.of(PagedKV(1, 32, None, None, 16), **{"right.conv": FixedState((3, 72), "float32"),
                                                                     "right.recurrent": FixedState((72, 16), "float32")})}
    m = CacheManager(needs, page_size=16, num_pages=6, max_requests=2, max_context=96, dtype=torch.float32)
    v0, v1, v2 = m.view(0), m.view(1), m.view(2)
    assert v0.k.shape == (6, 2, 16, 16) and v0.v.shape == (6, 2, 16, 24) and v2.v.shape == (6, 1, 16, 16)
    assert v0.states["right.conv"].shape == (2, 2, 48) and v2.states["right.recurrent"].shape == (2, 72, 16)
    assert v1.state.shape == (2, 80) and v1.state.dtype == torch.float32
    a = m.open()
    m.reserve(a, 40); m.commit(a, 40)
    v1.state[a].fill_(2.0); v0.states["right.recurrent"][a].fill_(1.0); v2.states["right.conv"][a].fill_(4.0)
    assert m.free_pages() == 6 - 3
    b = m.open()
    m.reserve(b, 48); m.commit(b, 48)
    from hfee_b200 import OutOfPages
    with pytest.raises(OutOfPages):
        m.reserve(a, 49)                      # would need a fourth page; nothing is taken
    m.check_invariants()
    m.close(a)
    assert m.free_pages() == 3 and m.open() == a
    assert float(v1.state[a].abs().max()) == 0 and float(v0.states["right.recurrent"][a].abs().max()) == 0
    assert float(v2.states["right.conv"][a].abs().max()) == 0


def _random_weights(cfg, seed):
    from hfee_b200.config import resolve
    from hfee_b200.parts.model import model_tensor_needs
    arch, typed = resolve(cfg)
    rng = np.random.default_rng(seed)
    w = {}
    for name, need in model_tensor_needs(arch.build_spec(typed)).items():
        w[name] = rng.normal(size=need.shape) * 0.3 + (1.0 if need.role == "scale" else 0.0)
        if name.endswith((".r1", ".r2")):
            w[name] = np.abs(w[name]) + 0.1
    return w


def test_plain_implementation_is_causal_and_every_earlier_token_matters():
    cfg = mu.config(16, 30, [mu.parallel(2, 1, 8, 4, 0.5, 12, 3, 2, 3, mlp=mu.moe(4, 2, 8, 1.0, 2.0, 6, 1.0)), mu.mingru(10)])
    w = _random_weights(cfg, 0)
    a = [3, 7, 1, 9, 4, 4, 2, 8, 5]
    b = list(a); b[2] = 11
    la, lb = plain.forward(cfg, w, a), plain.forward(cfg, w, b)
    assert np.allclose(la[:2], lb[:2]) and all(not np.allclose(la[t], lb[t]) for t in range(2, 9))
    logits, streams = plain.forward(cfg, w, a, return_layers=True)
    assert streams.shape == (2, 9, 16) and np.all(np.abs(logits) < 15.0)


def test_plain_mingru_against_its_closed_form():
    """With z constant the state is a geometric average of the candidates; the candidate's two branches meet at 1/2."""
    W = {"m.z": np.zeros((3, 2)), "m.z.b": np.full(3, np.log(3.0)),            # z = 3/4
         "m.x": np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]), "m.x.b": np.zeros(3),
         "m.g": np.zeros((3, 2)), "m.o": np.eye(3)}
    W["m.g"][:, 0] = 50.0                                                        # silu(50 * 1) = 50 when h[0] = 1
    h = np.array([[1.0, -2.0], [1.0, 0.0], [1.0, 3.0]])
    out = plain.mingru(h, W, "m.", {"width": 3}) / 50.0
    cand = lambda u: u + 0.5 if u >= 0 else 1.0 / (1.0 + np.exp(-u))
    c = np.array([[cand(1.0), cand(-2.0), cand(-1.0)], [cand(1.0), cand(0.0), cand(1.0)], [cand(1.0), cand(3.0), cand(4.0)]])
    S = np.zeros(3)
    for t in range(3):
        S = 0.25 * S + 0.75 * c[t]
        assert np.allclose(out[t], S)
    assert np.isclose(cand(0.0), 0.5) and np.isclose(cand(-1e-9), 0.5)


def test_plain_selective_scan_against_a_sum_over_the_past():
    """One tap and no bias: y_t = sum_(s <= t) exp(A (dt_(s+1) + ... + dt_t)) dt_s x_s B_s . C_t + D x_t."""
    rng = np.random.default_rng(1)
    m = {"inner": 3, "state": 2, "dt_rank": 1, "conv": 1}
    W = {"s.in": rng.normal(size=(6, 4)), "s.conv": np.ones((3, 1)), "s.conv.b": np.zeros(3), "s.x": rng.normal(size=(5, 3)),
         "s.dt": rng.normal(size=(3, 1)), "s.dt.b": rng.normal(size=3), "s.A_log": rng.normal(size=(3, 2)), "s.D": rng.normal(size=3),
         "s.o": np.eye(3)}
    h = rng.normal(size=(6, 4))
    got = plain.selective_scan(h, W, "s.", m)
    xz = h @ W["s.in"].T
    x, z = plain.silu(xz[:, :3]), xz[:, 3:]
    low = x @ W["s.x"].T
    dt = np.log1p(np.exp(low[:, :1] @ W["s.dt"].T + W["s.dt.b"]))
    B, C, A = low[:, 1:3], low[:, 3:5], -np.exp(W["s.A_log"])
    for t in range(6):
        y = W["s.D"] * x[t]
        for s in range(t + 1):
            decay = np.exp(A * dt[s + 1:t + 1].sum(axis=0)[:, None])
            y = y + ((decay * (dt[s] * x[s])[:, None] * B[s][None, :]) @ C[t])
        assert np.allclose(got[t], y * plain.silu(z[t]))
    conv = plain.causal_conv(np.arange(1.0, 6.0)[:, None], np.array([[1.0, 10.0, 100.0]]), np.array([0.5]))
    assert conv[:, 0].tolist() == [100.5, 210.5, 321.5, 432.5, 543.5]


def test_plain_distance_penalty_and_routing():
    """Equal keys: the attention weights fall with distance as (1 + r2 d)^(-r1); the router takes the largest scores,
    scales them and does not renormalise; the expert's clamps hold."""
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 3, "scale": 1.0}
    W = {"a.q": np.zeros((2, 3)), "a.k": np.zeros((2, 3)), "a.v": np.eye(3), "a.o": np.eye(3), "a.r1": np.array([2.0]), "a.r2": np.array([0.5])}
    h = np.eye(3)
    out = plain.distance_attention(h, W, "a.", m)
    wts = np.array([(1 + 0.5 * 2) ** -2.0, (1 + 0.5 * 1) ** -2.0, 1.0])
    assert np.allclose(out[2], wts / wts.sum()) and np.allclose(out[0], [1, 0, 0])
    choice, weight = plain.route(np.array([[1.0, 0.0]]), np.array([[0.0, 0.0], [1.0, 0.0], [3.0, 0.0], [2.0, 0.0]]), 2, 1.5)
    s = np.exp([0.0, 1.0, 3.0, 2.0]); s /= s.sum()
    assert sorted(choice[0].tolist()) == [2, 3] and np.allclose(sorted(weight[0]), sorted([1.5 * s[2], 1.5 * s[3]]))
    E = {"e.gate": np.array([[5.0], [-5.0]]), "e.up": np.array([[9.0], [-9.0]]), "e.down": np.eye(2)}
    y = plain.clamped_expert(np.array([[1.0]]), E, "e.", 2.0)[0]
    assert np.isclose(y[0], 2.0 / (1 + np.exp(-1.702 * 2.0)) * 3.0) and np.isclose(y[1], -5.0 / (1 + np.exp(1.702 * 5.0)) * -1.0)


def test_depth_average_reads_every_earlier_result():
    """What leaves layer i is the weighted sum of the embedding's output and of every layer's own result so far; a layer's
    own result is built on the average that the layer before handed on."""
    cfg = mu.config(16, 30, [mu.mingru(8), mu.mingru(12), mu.mingru(6)], residual_mult=1.0)
    w = _random_weights(cfg, 3)
    seq = [1, 5, 9, 2]
    _, streams = plain.forward(cfg, w, seq, return_layers=True)
    x0 = w["embed"][seq] + plain.sinusoid(4, 16)
    X1 = x0 + plain.mingru(plain.rms_norm(x0, w["l0.norm1"], 1e-5), w, "l0.mix.", {"width": 8})
    x1 = w["l0.dwa"][0] * x0 + w["l0.dwa"][1] * X1
    assert np.allclose(streams[0], x1)
    X2 = x1 + plain.mingru(plain.rms_norm(x1, w["l1.norm1"], 1e-5), w, "l1.mix.", {"width": 12})
    a = w["l1.dwa"]
    assert np.allclose(streams[1], a[0] * x0 + a[1] * X1 + a[2] * X2)


def test_command_line_creates_and_shows_a_model_folder(tmp_path, capsys):
    from hfee_b200 import cli
    from hfee_b200.config import resolve_model_dir
    from hfee_b200.parts.model import model_tensor_needs
    from hfee_b200.weights import Checkpoint
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(mu.MUV_B))
    model = tmp_path / "model"
    assert cli.main(["create", str(model), str(cfg_path), "--seed", "2"]) == 0
    arch, cfg = resolve_model_dir(str(model))
    assert arch.name == "Muvetar" and cfg.layers[2].mlp.top == 4
    needs = model_tensor_needs(arch.build_spec(cfg))
    Checkpoint(str(model)).check(needs)                 # everything asked for is there, nothing else
    c, w = plain.load(str(model))                       # and the plain reader finds every tensor it wants
    assert plain.forward(c, w, [1, 2, 3]).shape == (3, 310)
    capsys.readouterr()
    assert cli.main(["show", str(model)]) == 0
    out = capsys.readouterr().out
    assert "Muvetar" in out and f"{sum(int(np.prod(n.shape)) for n in needs.values()):,}" in out
