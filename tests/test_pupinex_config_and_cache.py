"""Pupinex on the CPU: configuration and its errors, the run order, what each layer asks of the cache manager, and the
plain implementation's own consistency (a recurrence against its closed form, a window against a mask, the router's
groups)."""
import ast
import copy
import os

import numpy as np
import pytest

import plain_pupinex as plain
import pupinex_util as pu


def resolved(cfg):
    from hfee_b200.config.registry import resolve
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer["type"] == "gla":
            layer["mixer"].setdefault("rank", pu.RANK)
    return resolve(cfg)


def test_config_reads_every_size_and_constant():
    arch, c = resolved(pu.PUP_A)
    assert arch.name == "Pupinex" and (c.vocab, c.width, c.eps, c.buckets, c.mul_prev, c.mul_cur) == (200, 64, 1e-5, 97, 31, 7)
    assert (c.loop.start, c.loop.stop, c.loop.times) == (1, 3, 3)
    left = c.layers[0].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.scale, left.window) == (4, 2, 16, 24, 0.3, 21)
    assert (left.rot.dims, left.rot.base, left.rot.factor) == (8, 1000.0, 2.0) and c.layers[1].mixer.rot.factor == 1.0
    right = c.layers[0].mixer.right
    assert (right.heads, right.dim, right.vdim, right.gate_cap) == (2, 16, 24, 8.0)
    assert (c.layers[0].mixer.left_scale, c.layers[0].mixer.right_scale) == (0.7, 1.2)
    m = c.layers[1].mlp
    assert (m.experts, m.top, m.groups, m.keep, m.router_scale, m.ff, m.shared_ff) == (6, 2, 3, 2, 1.8, 24, 40)
    assert (c.layers[2].mixer.tau, c.layers[2].mixer.rank, c.layers[2].mlp.ff, c.layers[2].mlp.limit) == (8.0, pu.RANK, 72, 0.9)
    _, b = resolved(pu.PUP_B)
    assert b.loop is None and b.layers[0].mlp is None and b.layers[1].mlp.shared_ff is None


def test_run_order_gives_every_pass_a_cache_of_its_own():
    arch, c = resolved(pu.PUP_A)
    spec = arch.build_spec(c)
    runs = [(r.layer, r.cache, r.adds_embedding) for r in spec.schedule]
    assert runs == [(0, 0, False), (1, 1, False), (2, 2, False), (1, 3, True), (2, 4, False), (1, 5, True), (2, 6, False), (3, 7, False)]
    assert [i for i, _ in plain.run_order(pu.PUP_A)] == [r[0] for r in runs]
    assert [a for _, a in plain.run_order(pu.PUP_A)] == [r[2] for r in runs]
    for loop, want in (((0, 4, 2), [0, 1, 2, 3, 0, 1, 2, 3]), ((3, 4, 3), [0, 1, 2, 3, 3, 3]), ((2, 2, 5), [0, 1, 2, 3]), ((0, 1, 1), [0, 1, 2, 3])):
        arch, c = resolved({**pu.PUP_A, "loop": {"start": loop[0], "stop": loop[1], "times": loop[2]}})
        sched = arch.build_spec(c).schedule
        assert [r.layer for r in sched] == want and [r.cache for r in sched] == list(range(len(want)))


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "not a mixer of this design"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "not a feed-forward of this design"),
    (lambda c: c["layers"][1]["mixer"].update(heads=5), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=26), "at most dim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "must be even"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "experts of the kept groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][2]["mixer"].update(tau=0.0), "must be positive"),
    (lambda c: c["layers"][2]["mlp"].update(limit=-1.0), "must be positive"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["loop"].update(stop=9), "does not fit"),
    (lambda c: c["embedding"]["bigram"].pop("mul_prev"), "mul_prev"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_errors_name_the_key(change, message):
    from hfee_b200.config.llama import ConfigError
    cfg = copy.deepcopy(pu.PUP_A)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        resolved(cfg)


def test_the_decay_rank_comes_from_the_tensor():
    from hfee_b200.config.llama import ConfigError
    from hfee_b200.config.registry import resolve
    with pytest.raises(ConfigError, match="rank"):
        resolve(pu.PUP_A)
    _, c = resolve(pu.PUP_A, {"l2.mix.a1": (11, 64), "l0.mix.left.q": (64, 64)})
    assert c.layers[2].mixer.rank == 11


def test_tensor_names_and_shapes():
    from hfee_b200.parts.model import model_tensor_needs
    arch, c = resolved(pu.PUP_A)
    needs = model_tensor_needs(arch.build_spec(c))
    shape = lambda n: tuple(needs[n].shape)
    assert shape("embed") == (200, 64) and shape("bigram") == (98, 64) and shape("final.norm") == (64,) and "head" not in needs
    assert shape("l0.mix.left.q") == (64, 64) and shape("l0.mix.left.v") == (48, 64) and shape("l0.mix.left.k.norm") == (32,)
    assert shape("l0.mix.left.o") == (64, 96) and "l0.mix.left.o.b" not in needs and "l0.mix.left.sink" not in needs
    assert shape("l0.mix.right.i") == (2, 64) and shape("l0.mix.right.f.b") == (2,) and shape("l0.mix.right.norm") == (48,)
    assert shape("l1.mix.o.b") == (64,) and shape("l1.mix.sink") == (4,) and shape("l1.mix.v.b") == (32,)
    assert shape("l1.mlp.router") == (6, 64) and shape("l1.mlp.e5.down") == (64, 24) and shape("l1.mlp.shared.sg") == (1, 64)
    assert shape("l2.mix.a1") == (pu.RANK, 64) and shape("l2.mix.a2") == (32, pu.RANK) and shape("l2.mix.norm") == (32,)
    assert shape("l2.mlp.gate") == (72, 64) and needs["l1.mix.sink"].role == "vector" and needs["l0.norm1"].role == "scale"


def test_cache_needs_per_run():
    """The model asks for pages where a layer attends (windowed), for float32 states where it recurs, and for one
    integer per request for the embedding; every pass of a looped layer asks again."""
    import torch
    from hfee_b200.cache import CacheManager
    from hfee_b200.cache.needs import CacheBundle, FixedState, PagedKV
    from hfee_b200.parts.base import part_class
    arch, c = resolved(pu.PUP_A)
    spec = arch.build_spec(c)
    needs = {}
    for run in spec.schedule:
        mixer = spec.layers[run.layer].parts["mixer"][1]
        cls = part_class("mixer", mixer.kind)
        needs[run.cache] = (mixer.kind, cls)
    assert [k for k, _ in needs.values()] == ["parallel", "softmax_attention", "channel_decay_attention", "softmax_attention",
                                              "channel_decay_attention", "softmax_attention", "channel_decay_attention", "softmax_attention"]
    as_needs = {0: CacheBundle.of(PagedKV(2, 16, 21, None, 24), **{"right.memory": FixedState((2, 16, 24)), "right.normalizer": FixedState((2, 16)),
                                                                   "right.maximum": FixedState((2,))}),
                1: PagedKV(2, 24, 13, None, 16), 2: FixedState((2, 16, 32)), 3: PagedKV(2, 24, 13, None, 16), 4: FixedState((2, 16, 32)),
                -1: FixedState((1,), "int32")}
    m = CacheManager(as_needs, 16, 12, 3, 96, torch.float32)
    assert m.view(-1).state.dtype == torch.int32 and tuple(m.view(-1).state.shape) == (3, 1)
    assert m.view(1).k.shape == m.view(3).k.shape == (12, 2, 16, 24) and m.view(1).v.shape[-1] == 16
    assert m.view(1).k.data_ptr() != m.view(3).k.data_ptr() and m.view(2).state.data_ptr() != m.view(4).state.data_ptr()
    assert tuple(m.view(0).states["right.memory"].shape) == (3, 2, 16, 24) and tuple(m.view(0).states["right.maximum"].shape) == (3, 2)
    s = m.open()
    m.reserve(s, 60); m.commit(s, 60)
    m.check_invariants()
    held = [int((g.table[s] >= 0).sum()) for g in m.paged]
    assert sorted(held) == [1, 2]            # windows of 13 and 21 tokens: one and two pages of 16 still hold keys a later token reads
    m.view(2).state[s].fill_(3.0); m.view(-1).state[s].fill_(5)
    m.close(s)
    assert m.open() == s and float(m.view(2).state[s].abs().sum()) == 0.0 and int(m.view(-1).state[s]) == 0


def test_every_kernel_call_passes_as_many_arguments_as_its_signature_names():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "hfee_b200", "kernels", "ops.py")
    tree = ast.parse(open(path).read())
    sigs = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.Assign) and getattr(node.targets[0], "id", None) == "_SIGNATURES":
            sigs = {k.value: len(v.elts) for k, v in zip(node.value.keys, node.value.values)}
    assert len(sigs) > 60
    for node in ast.walk(tree):
        if (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and isinstance(node.func.value, ast.Name)
                and node.func.value.id == "lib" and node.func.attr in sigs):
            assert len(node.args) == sigs[node.func.attr], f"{node.func.attr} at line {node.lineno}"


# ------------------------------------------------------------------ the plain implementation against itself
def test_channel_decay_recurrence_equals_its_closed_form():
    rng = np.random.default_rng(0)
    T, H, d, dv = 9, 2, 3, 4
    q, k, v = rng.normal(size=(T, H, d)), rng.normal(size=(T, H, d)), rng.normal(size=(T, H, dv))
    a = rng.uniform(0.5, 1.0, size=(T, H, d))
    o = plain.channel_decay_recurrence(q, k, v, a)
    for h in range(H):
        for t in range(T):
            want = np.zeros(dv)
            for s in range(t + 1):
                decay = np.prod(a[s + 1:t + 1, h], axis=0)
                want += ((q[t, h] * decay) @ k[s, h]) * v[s, h]
            assert np.allclose(o[t, h], want)


def test_matrix_memory_equals_unstabilised_gates_where_those_are_tame():
    rng = np.random.default_rng(1)
    T, H, d, dv = 12, 2, 3, 4
    q, k, v = rng.normal(size=(T, H, d)), rng.normal(size=(T, H, d)), rng.normal(size=(T, H, dv))
    ig, fg = rng.normal(size=(T, H)), -rng.uniform(0.0, 0.5, size=(T, H))
    o = plain.matrix_memory(q, k, v, ig, fg)
    for h in range(H):
        C, n, m = np.zeros((d, dv)), np.zeros(d), 0.0
        for t in range(T):
            C = np.exp(fg[t, h]) * C + np.exp(ig[t, h]) * np.outer(k[t, h], v[t, h])
            n = np.exp(fg[t, h]) * n + np.exp(ig[t, h]) * k[t, h]
            m = max(fg[t, h] + m, ig[t, h])
            want = C.T @ q[t, h] * np.exp(-m) / (max(abs(n @ q[t, h]) * np.exp(-m), np.exp(-m)) + 1e-6)
            assert np.allclose(o[t, h], want)


def test_window_and_sink_against_a_masked_matrix():
    rng = np.random.default_rng(2)
    T, H, G, d, dv, window = 14, 4, 2, 5, 3, 4
    q, k, v = rng.normal(size=(T, H, d)), rng.normal(size=(T, G, d)), rng.normal(size=(T, G, dv))
    sink = rng.normal(size=H)
    o = plain.windowed_softmax_attention(q, k, v, 0.7, window, sink)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = (i - j >= 0) & (i - j < window)
    for h in range(H):
        s = np.where(seen, (q[:, h] @ k[:, h // 2].T) * 0.7, -np.inf)
        e = np.exp(s)
        assert np.allclose(o[:, h], (e / (e.sum(1, keepdims=True) + np.exp(sink[h]))) @ v[:, h // 2])
    assert np.allclose(plain.windowed_softmax_attention(q, k, v, 0.7, T + 5, sink - 80.0), plain.windowed_softmax_attention(q, k, v, 0.7, T))


def test_pairings_of_the_rotation_are_one_rotation_in_two_layouts():
    rng = np.random.default_rng(3)
    x = rng.normal(size=(7, 2, 12))
    dims = 8
    perm = [2 * i for i in range(dims // 2)] + [2 * i + 1 for i in range(dims // 2)] + list(range(dims, 12))
    a = plain.rotate(x, dims, 50.0, "interleaved", 3.0)
    b = plain.rotate(x[..., perm], dims, 50.0, "half", 3.0)
    assert np.allclose(a[..., perm], b) and np.allclose(a[0], x[0]) and np.allclose(a[..., dims:], x[..., dims:])
    y = x.copy()
    y[1] = x[3]                               # position 3 with every frequency divided by 3 turns as position 1 does
    assert np.allclose(plain.rotate(x, dims, 50.0, "half", 3.0)[3], plain.rotate(y, dims, 50.0, "half", 1.0)[1])


def test_group_limited_choice():
    s = np.array([0.9, 0.1, 0.5, 0.6, 0.55, 0.56, 0.95, 0.0])
    assert plain.group_limited_choice(s, 2, 4, 1) == [5, 4]            # the groups score 1.0, 1.1, 1.11, 0.95: the third wins by its pair
    assert plain.group_limited_choice(s, 2, 1, 1) == [6, 0]            # without groups the two largest scores
    assert plain.group_limited_choice(s, 3, 2, 1) == [6, 5, 4] and plain.group_limited_choice(s, 3, 2, 2) == [6, 0, 3]
    assert plain.group_limited_choice(np.full(6, 0.3), 2, 3, 2) == [0, 1]


def test_bigram_rows_and_greedy():
    assert plain.bigram_rows([5, 9, 9, 0], 7, 3, 2).tolist() == [7, (15 + 18) % 7, (27 + 18) % 7, 27 % 7]
    import tempfile
    d = pu.write_model(tempfile.mkdtemp(), pu.config(32, 30, [pu.gla(1, 8, 8, 4.0)]), seed=1)
    c, w = plain.load(d)
    out = plain.greedy(c, w, [3, 4], 4)
    assert len(out) == 4 and out[0] == int(np.argmax(plain.forward(c, w, [3, 4])[-1]))
