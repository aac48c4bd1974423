"""The Pupinex decoder on the GPU against the plain implementation of tests/plain_pupinex.py: each mixer and feed-forward
alone, whole prompts, prefill then token by token, portions down to two tokens, mixed batches over few pages and slots,
window and page edges, far keys and far writes, the first tokens, long decoding, other sizes, and greedy generation
through the engine's entry point."""
import numpy as np
import pytest

import plain_pupinex as plain
import pupinex_util as pu
import replay_util as ru

pytestmark = pytest.mark.gpu

# Largest |difference| relative to the largest |logit| of the plain float64 result on the same stored weights,
# and the root mean square of the differences relative to that of the logits.  float32: rounding of float32
# sums only.  bfloat16: activations between kernels are rounded to 8 bits of mantissa.
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
RMS_TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}
LENGTHS = (5, 17, 33, 100, 1, 71, 40, 9)


def rms_err(got, ref):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.sqrt(np.mean((got - ref) ** 2)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg, seed in (("A", pu.PUP_A, 3), ("B", pu.PUP_B, 4)):
        d = pu.write_model(str(tmp_path_factory.mktemp("pupinex" + name)), cfg, seed)
        c, w = plain.load(d)
        seqs = pu.sequences(cfg["vocab"], LENGTHS, seed=11)
        assert pu.smallest_route_margin(plain, c, w, seqs) > 0.1          # no router's choice is a close call
        out[name] = (d, cfg, seqs, [plain.forward(c, w, s) for s in seqs])
    return out


def check(got, ref, dtype, what="", rms_tol=None):
    assert sorted(got) == list(range(len(ref)))
    for i in range(len(ref)):
        assert got[i].shape == ref[i].shape
        err, rms = ru.rel_err(got[i], ref[i]), rms_err(got[i], ref[i])
        assert err < TOL[dtype] and rms < (rms_tol or RMS_TOL[dtype]), f"{what} request {i}: relative error {err:.3g}, rms {rms:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("scheme", ["whole", "prefill_then_decode", "portions", "mixed"])
def test_replay(models, name, dtype, scheme):
    d, cfg, seqs, ref = models[name]
    if scheme == "mixed":
        steps = ru.mixed(seqs, live=4, seed=2)
        # the four longest at once need 100+71+40+33 -> 17 pages of 16 with rounding; slots and pages are used again
        runner = pu.make_runner(d, dtype, max_tokens=17 * 16, context=112)
    else:
        steps = {"whole": ru.whole, "prefill_then_decode": lambda s: ru.prefill_then_decode(s, tail=20),
                 "portions": ru.portions}[scheme](seqs)
        runner = pu.make_runner(d, dtype, max_tokens=112, max_requests=1)
    check(ru.run_in_process(runner, steps), ref, dtype, scheme)


def test_batch_of_unequal_requests_equals_each_alone(models):
    """float32: a row's sums run in one order whatever else is in the batch."""
    d, cfg, seqs, ref = models["A"]
    alone = ru.run_in_process(pu.make_runner(d, "float32", 112, max_requests=1), ru.whole(seqs))
    runner = pu.make_runner(d, "float32", max_tokens=512, max_requests=8, context=112)
    steps = [{"entries": [(i, s, list(range(len(s)))) for i, s in enumerate(seqs)], "end": list(range(len(seqs)))}]
    together = ru.run_in_process(runner, steps)
    for i in range(len(seqs)):
        assert ru.rel_err(together[i], alone[i]) < 2e-6


A = pu.attn
ALONE = {
    "attention": pu.attention(4, 2, 16, 24, 0.3, 11, 8, 100.0),
    "attention_one_head_whole_rotation": pu.attention(1, 1, 40, 8, 0.2, 7, 40, 1.0e4),
    "attention_no_rotation_window_one": pu.attention(2, 2, 16, 16, 0.3, 1, 0, 1.0e4),
    "attention_tensor_core_sizes": pu.attention(4, 1, 64, 64, 0.15, 30, 32, 5.0e4),
    "attention_wide_values_long_window": pu.attention(6, 3, 64, 128, 0.12, 1000, 16, 300.0),
    "gla": pu.gla(2, 16, 24, 8.0),
    "gla_one_head_many_rows": pu.gla(1, 72, 40, 1.0),
    "gla_odd_sizes": pu.gla(3, 5, 33, 30.0),
    "left_alone": pu.parallel(A(4, 2, 16, 8, 0.4, 9, 16, 50.0, factor=4.0), 1, 8, 8, 5.0, left_scale=1.3, right_scale=0.0),
    "memory_alone": pu.parallel(A(1, 1, 8, 8, 0.3, 5, 2, 10.0), 3, 16, 24, 15.0, left_scale=0.0, right_scale=0.8),
    "memory_many_rows_small_cap": pu.parallel(A(1, 1, 8, 8, 0.3, 5, 2, 10.0), 1, 70, 40, 1.5, left_scale=0.0, right_scale=1.0),
    "both_branches": pu.parallel(A(2, 1, 24, 16, 0.25, 17, 12, 1000.0, factor=1.5), 2, 16, 16, 10.0, left_scale=0.6, right_scale=0.5),
    "dense": pu.gla(1, 8, 8, 4.0, mlp=pu.dense(40, 0.7)),
    "experts_with_shared": pu.gla(1, 8, 8, 4.0, mlp=pu.moe(6, 2, 3, 2, 20, 2.5, shared_ff=28)),
    "experts_all_of_the_kept_groups": pu.gla(1, 8, 8, 4.0, mlp=pu.moe(6, 3, 2, 1, 12, 0.7)),
    "one_expert_of_one": pu.gla(1, 8, 8, 4.0, mlp=pu.moe(1, 1, 1, 1, 12, 1.0, shared_ff=12)),
    "groups_of_one_expert": pu.gla(1, 8, 8, 4.0, mlp=pu.moe(4, 2, 4, 3, 16, 1.0)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", list(ALONE.values()), ids=list(ALONE))
def test_each_mechanism_alone(tmp_path, layer, dtype):
    """One layer (a mixer without feed-forward, or a small mixer with a feed-forward): whole, and in portions through
    the cache or state."""
    cfg = pu.config(48, 90, [layer])
    d = pu.write_model(str(tmp_path), cfg, seed=7)
    c, w = plain.load(d)
    seqs = pu.sequences(90, (37, 3, 64), seed=5)
    ref = [plain.forward(c, w, s) for s in seqs]
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(2, 9, 1, 1, 30, 2))):
        check(ru.run_in_process(pu.make_runner(d, dtype, 64, max_requests=1), steps), ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_fit_no_vector_access(tmp_path, dtype):
    """Width, vocabulary, ranks and head sizes that are multiples of neither 8 nor 4: every kernel takes its scalar path."""
    layers = [pu.parallel(A(3, 1, 12, 10, 0.3, 6, 6, 20.0, factor=3.0), 3, 6, 14, 4.0, 0.9, 1.2, mlp=pu.moe(5, 2, 1, 1, 14, 1.5, shared_ff=18)),
              pu.gla(2, 10, 7, 2.0, mlp=pu.dense(22, 1.3)),
              pu.attention(2, 2, 6, 14, 0.4, 19, 2, 9.0)]
    cfg = pu.config(50, 77, layers, loop=(0, 2, 2), eps=3e-6, buckets=11, mul_prev=1, mul_cur=1)
    d = pu.write_model(str(tmp_path), cfg, seed=13)
    c, w = plain.load(d)
    seqs = pu.sequences(77, (41, 2, 19), seed=6)
    ref = [plain.forward(c, w, s) for s in seqs]
    rms_tol = 2.5e-2 if dtype == "bfloat16" else None       # short sums average less of the rounding than wider models' do
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(3, 2, 17, 1, 5)), ru.mixed(seqs, live=2, seed=1)):
        check(ru.run_in_process(pu.make_runner(d, dtype, 96, max_requests=2, context=48), steps), ref, dtype, rms_tol=rms_tol)


@pytest.mark.parametrize("loop", [None, (0, 1, 2), (1, 2, 4), (0, 3, 2), (2, 3, 1), (1, 1, 3)])
def test_loops(tmp_path, loop):
    """A stretch of layers run several times over: at the start, in the middle, the whole model, once, and an empty one.
    Every pass has a state of its own (a shared one would show at once), and the embedding comes on top again."""
    layers = [pu.gla(2, 8, 8, 6.0, mlp=pu.dense(24, 1.0)), pu.attention(2, 1, 8, 8, 0.4, 5, 4, 30.0),
              pu.parallel(A(2, 2, 8, 8, 0.3, 4, 8, 70.0), 1, 8, 16, 6.0, 1.0, 1.0)]
    cfg = pu.config(32, 60, layers, loop=loop)
    d = pu.write_model(str(tmp_path), cfg, seed=17)
    c, w = plain.load(d)
    seqs = pu.sequences(60, (23, 6), seed=9)
    ref = [plain.forward(c, w, s) for s in seqs]
    if loop is not None and loop[2] > 1 and loop[1] > loop[0]:
        no_loop = plain.forward({**c, "loop": None}, w, seqs[0])
        assert ru.rel_err(no_loop, ref[0]) > 1e-2
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(2, 5, 1, 9, 2)), ru.mixed(seqs, live=2, seed=3)):
        check(ru.run_in_process(pu.make_runner(d, "float32", 64, max_requests=2, context=32), steps), ref, "float32", str(loop))


def test_bigram_needs_the_token_before_a_portion(tmp_path):
    """The token in front of a portion's first token belongs to the request: with a bigram table that dwarfs the token
    table, a lost or stale previous token (a slot's earlier user, the batch's neighbour) would change every logit."""
    cfg = pu.config(32, 40, [pu.gla(1, 8, 8, 4.0)], buckets=13, mul_prev=3, mul_cur=5)

    def loud(tensors):
        tensors["bigram"].mul_(20.0)
    d = pu.write_model(str(tmp_path), cfg, seed=19, edit=loud)
    c, w = plain.load(d)
    seqs = pu.sequences(40, (30, 21, 9, 14), seed=2)
    ref = [plain.forward(c, w, s) for s in seqs]
    shuffled = plain.forward(c, {**w, "bigram": w["bigram"][::-1].copy()}, seqs[0])
    assert ru.rel_err(shuffled, ref[0]) > 0.05
    for steps in (ru.portions(seqs, sizes=(1, 1, 2, 7, 1, 3)), ru.mixed(seqs, live=2, seed=5), ru.prefill_then_decode(seqs, tail=8)):
        check(ru.run_in_process(pu.make_runner(d, "float32", 64, max_requests=2, context=32), steps), ref, "float32")


MARK = 6.0          # the marks' size: the norm in front leaves them large


def _marked_sequence(length, at, vocab=50, seed=8):
    """Tokens 2.. at random with token 0 at the places ``at`` (token 1 nowhere); and the same with token 1 there."""
    base = [2 + t % (vocab - 2) for t in pu.sequences(vocab, (length,), seed=seed)[0]]
    a, b = list(base), list(base)
    for p in at:
        a[p], b[p] = 0, 1
    return a, b


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "left"])
def test_keys_just_inside_and_just_outside_the_window(tmp_path, dtype, kind):
    """One key is made to stand out for every later query, and it carries a value of its own: the logits of the query
    window - 1 places behind it (the last that sees it) and of the next one (the first that does not) differ a lot, and
    both must match the plain implementation: in whole prompts, in portions that end or begin at the edge, for decoded
    tokens, and where the window's edge lies on, before or behind a page's."""
    window, page = 37, 16
    if kind == "attention":
        layer = pu.attention(2, 1, 16, 8, 1.0, window, 8, 1.0e4)
        p = "l0.mix."
    else:
        layer = pu.parallel(A(2, 2, 16, 8, 1.0, window, 8, 1.0e4, factor=2.0), 1, 8, 8, 5.0, left_scale=1.0, right_scale=0.0)
        p = "l0.mix.left."
    cfg = pu.config(32, 50, [layer])

    def marked(tensors):
        pu.mark_first_tokens(tensors, MARK)
        wq, wk, wv = tensors[p + "q"], tensors[p + "k"], tensors[p + "v"]
        # the unrotated dimensions 8..15 of every head carry the mark: rotation cannot turn the loud score away
        wq.mul_(0.2); wk.mul_(0.2)
        for h0 in range(0, wk.shape[0], 16):
            wk[h0 + 8:h0 + 16, pu.MARK_A] = wk[h0 + 8:h0 + 16, pu.MARK_B] = 1.0
            wk[h0 + 8:h0 + 16, pu.MARK_LATER] = 0.0
        for h0 in range(0, wq.shape[0], 16):
            wq[h0 + 8:h0 + 16, pu.MARK_LATER] = 1.0
        wv[:, pu.MARK_A], wv[:, pu.MARK_B] = 1.0, -1.0
        for b in ("q.b", "k.b", "v.b"):
            tensors[p + b].zero_()
        if kind == "attention":
            tensors[p + "sink"].fill_(0.5)
    d = pu.write_model(str(tmp_path), cfg, seed=33, edit=marked)
    c, w = plain.load(d)
    for place in (0, 11, page - 1, page, 27):
        seq, other = _marked_sequence(place + window + 12, [place])
        ref, ref_other = plain.forward(c, w, seq), plain.forward(c, w, other)
        inside, outside = place + window - 1, place + window
        effect = ru.rel_err(ref_other[inside], ref[inside])
        assert effect > 0.05 and ru.rel_err(ref_other[outside:], ref[outside:]) < 1e-9       # seen, then gone for good
        limit = TOL[dtype] if dtype == "float32" else max(TOL[dtype], effect / 10)
        n = len(seq)
        cuts = [(n,), (inside, 1, 1, n), (inside + 1, n), (inside - 1, 2, n), (place + 1,) + (1,) * (n - place - 1), (2, 2, place + 5, 3, n)]
        for sizes in cuts:
            for s, r in ((seq, ref), (other, ref_other)):
                got = ru.run_in_process(pu.make_runner(d, dtype, 96, page_size=page, max_requests=1), ru.portions([s], sizes=sizes))
                assert ru.rel_err(got[0], r) < limit, f"marked key at {place}, cut {sizes[:5]}"


def _far_check(d, dtype, places, length=400):
    c, w = plain.load(d)
    seq, other = _marked_sequence(length, places)
    ref, ref_other = plain.forward(c, w, seq), plain.forward(c, w, other)
    effect = ru.rel_err(ref_other[-8:], ref[-8:])
    assert effect > 5 * TOL[dtype]                                       # the far token matters
    # float32: rounding of sums.  bfloat16: every logit here hangs on a handful of rounded numbers (one layer, weights
    # made so that one key or a few writes decide), so the largest difference is held to a tenth of what the far
    # token changes, and the root mean square to the usual bound.
    limit = TOL[dtype] if dtype == "float32" else max(TOL[dtype], effect / 10)
    runner = pu.make_runner(d, dtype, 416, page_size=32, max_requests=1)
    for s, r in ((other, ref_other), (seq, ref)):                        # the same slot and pages twice
        steps = ru.portions([s], sizes=(130, 2, 67, 1, 1, 100, 64)) if s is seq else ru.prefill_then_decode([s], tail=40)
        got = ru.run_in_process(runner, steps)
        assert ru.rel_err(got[0], r) < limit and rms_err(got[0], r) < RMS_TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(tmp_path, dtype):
    """A window of 395 positions: the marked key at position 7 is seen by the last tokens of 400, across many pages, next
    to a sink that would swallow the weight of ordinary keys."""
    cfg = pu.config(32, 50, [pu.attention(2, 2, 16, 8, 1.0, 395, 8, 1.0e4)])

    def marked(tensors):
        pu.mark_first_tokens(tensors, MARK)
        wq, wk, wv = tensors["l0.mix.q"], tensors["l0.mix.k"], tensors["l0.mix.v"]
        wq.mul_(0.2); wk.mul_(0.2)
        for h0 in (0, 16):
            wk[h0 + 8:h0 + 16, pu.MARK_A] = wk[h0 + 8:h0 + 16, pu.MARK_B] = 1.0
            wk[h0 + 8:h0 + 16, pu.MARK_LATER] = 0.0
            wq[h0 + 8:h0 + 16, pu.MARK_LATER] = 1.0
        wv[:, pu.MARK_A], wv[:, pu.MARK_B] = 1.0, -1.0
        for b in ("q.b", "k.b", "v.b"):
            tensors["l0.mix." + b].zero_()
        tensors["l0.mix.sink"].fill_(4.0)
    _far_check(pu.write_model(str(tmp_path), cfg, seed=33, edit=marked), dtype, places=[7])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_takes_its_share(tmp_path, dtype):
    """Sinks far above the scores shrink every head's output, sinks far below change nothing: the plain implementation
    says so, and the kernels agree for prompts, portions and decoded tokens (whose keys are split among thread blocks)."""
    cfg = pu.config(32, 50, [pu.attention(4, 2, 16, 16, 0.3, 300, 8, 1.0e3)])
    seqs = pu.sequences(50, (330,), seed=3)
    refs = {}
    for level in (-30.0, 0.0, 6.0):
        d = pu.write_model(str(tmp_path / f"s{level}"), cfg, seed=5, edit=lambda t: t["l0.mix.sink"].copy_(level + 0.1 * t["l0.mix.sink"]))
        c, w = plain.load(d)
        refs[level] = plain.forward(c, w, seqs[0])
        runner = pu.make_runner(d, dtype, 352, page_size=32, max_requests=1)
        for steps in (ru.whole(seqs), ru.prefill_then_decode(seqs, tail=25), ru.portions(seqs, sizes=(100, 2, 31, 1, 1, 200))):
            check(ru.run_in_process(runner, steps), [refs[level]], dtype, f"sink {level}")
    assert ru.rel_err(refs[0.0], refs[-30.0]) > 0.02 and ru.rel_err(refs[6.0], refs[0.0]) > 0.02


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_write_reaches_through_the_decaying_state(tmp_path, dtype):
    """Decays next to 1 for every channel: what the marked tokens wrote still shows hundreds of tokens later, after
    portions, decoded tokens, and a slot that another request used before."""
    cfg = pu.config(32, 50, [pu.gla(2, 8, 8, 16.0)])

    def slow(tensors):
        pu.mark_first_tokens(tensors, MARK)
        t = lambda k: tensors["l0.mix." + k]
        t("a2").mul_(0.1)
        t("a2.b").fill_(7.0)
        t("k").mul_(0.05)
        t("k")[:, pu.MARK_A] = t("k")[:, pu.MARK_B] = 1.0                     # the marked tokens write loudly
        t("k")[:, pu.MARK_LATER] = 0.0
        t("v")[:, pu.MARK_A], t("v")[:, pu.MARK_B] = 1.0, -1.0                # and opposite values
        t("q")[:, pu.MARK_LATER] = 1.0
        t("o").mul_(4.0)                                                      # the mixer's output weighs in the logits
    _far_check(pu.write_model(str(tmp_path), cfg, seed=35, edit=slow), dtype, places=[0, 1, 2])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_write_reaches_through_the_matrix_memory(tmp_path, dtype):
    """Forget gates next to 1, an input gate that is wide open for the marked tokens and nearly shut for every other one."""
    cfg = pu.config(32, 50, [pu.parallel(A(1, 1, 8, 8, 0.3, 4, 2, 10.0), 2, 8, 8, 12.0, left_scale=0.0, right_scale=1.0)])

    def slow(tensors):
        pu.mark_first_tokens(tensors, MARK)
        t = lambda k: tensors["l0.mix.right." + k]
        t("f").mul_(0.02); t("f.b").fill_(9.0)
        t("i").mul_(0.02); t("i.b").fill_(0.0)
        t("i")[:, pu.MARK_A] = t("i")[:, pu.MARK_B] = 1.0
        t("i")[:, pu.MARK_LATER] = -1.0
        t("k").mul_(0.3)
        t("v")[:, pu.MARK_A], t("v")[:, pu.MARK_B] = 1.0, -1.0
    _far_check(pu.write_model(str(tmp_path), cfg, seed=37, edit=slow), dtype, places=[0, 1, 2])


def test_the_running_maximum_starts_at_zero_and_gates_are_capped(tmp_path):
    """Very negative input gates: with a maximum that started at minus infinity the first tokens' outputs would be of
    order one, with zero they are tiny.  Pre-activations far beyond the cap: tanh holds them there.  The plain
    implementation shows both effects and the kernels follow it, also in the first portion of one token."""
    cfg = pu.config(32, 50, [pu.parallel(A(1, 1, 8, 8, 0.3, 4, 2, 10.0), 2, 8, 8, 3.0, left_scale=0.0, right_scale=1.0)])

    def edit(tensors):
        tensors["l0.mix.right.i.b"].fill_(-40.0)
        tensors["l0.mix.right.f.b"].fill_(40.0)
    d = pu.write_model(str(tmp_path), cfg, seed=39, edit=edit)
    c, w = plain.load(d)
    seqs = pu.sequences(50, (30, 1, 2), seed=4)
    ref = [plain.forward(c, w, s) for s in seqs]
    c2 = {**c, "layers": [{**c["layers"][0], "mixer": {**c["layers"][0]["mixer"], "right": {**c["layers"][0]["mixer"]["right"], "gate_cap": 50.0}}}]}
    assert ru.rel_err(plain.forward(c2, w, seqs[0]), ref[0]) > 1e-3
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(1, 1, 2, 5, 30))):
        check(ru.run_in_process(pu.make_runner(d, "float32", 32, max_requests=1), steps), ref, "float32")


def test_variants_of_the_plain_implementation_show_in_the_logits(tmp_path):
    """What a wrong reading would compute gives other logits, so the comparison would see it."""
    layers = [pu.attention(2, 1, 16, 16, 0.3, 9, 8, 100.0, mlp=pu.moe(6, 2, 3, 2, 16, 2.0, shared_ff=12)),
              pu.parallel(A(2, 1, 16, 16, 0.3, 9, 8, 100.0, factor=4.0), 1, 8, 8, 6.0, 0.7, 1.1, mlp=pu.dense(24, 0.5))]
    cfg = pu.config(48, 40, layers, loop=(0, 2, 2))
    d = pu.write_model(str(tmp_path), cfg, seed=5, routes=False)      # random routers: the limit to groups decides choices
    c, w = plain.load(d)
    seq = pu.sequences(40, (30,), seed=3)[0]
    ref = plain.forward(c, w, seq)

    def with_mixer(i, **changes):
        layers = [dict(l) for l in c["layers"]]
        layers[i]["mixer"] = {**layers[i]["mixer"], **changes}
        return {**c, "layers": layers}
    a0, left = c["layers"][0]["mixer"], c["layers"][1]["mixer"]["left"]
    variants = {
        "window one longer": (with_mixer(0, mask={"size": 10}), w),
        "no sink": (c, {**w, "l0.mix.sink": w["l0.mix.sink"] - 100.0}),
        "rotate-half in the attention layer": (c, None),
        "no frequency scaling": (with_mixer(1, left={**left, "rot": {"dims": 8, "base": 100.0}}), w),
        "no query norm weight": (c, {**w, "l1.mix.left.q.norm": np.ones_like(w["l1.mix.left.q.norm"])}),
        "no output bias": (c, {**w, "l0.mix.o.b": 0 * w["l0.mix.o.b"]}),
        "no limit": ({**c, "layers": [c["layers"][0], {**c["layers"][1], "mlp": pu.dense(24, 50.0)}]}, w),
        "ungated shared expert": (c, {**w, "l0.mlp.shared.sg": 0 * w["l0.mlp.shared.sg"]}),
        "all groups kept": ({**c, "layers": [{**c["layers"][0], "mlp": pu.moe(6, 2, 3, 3, 16, 2.0, shared_ff=12)}, c["layers"][1]]}, w),
        "no loop": ({**c, "loop": None}, w),
    }
    for what, (cv, wv) in variants.items():
        if wv is None:
            old = plain.sink_attention_mixer
            plain.sink_attention_mixer = lambda h, T_, p, m, old=old: _half_rotated(h, T_, p, m)
            try:
                out = plain.forward(cv, w, seq)
            finally:
                plain.sink_attention_mixer = old
        else:
            out = plain.forward(cv, wv, seq)
        assert ru.rel_err(out, ref) > 1e-3, what
    got = ru.run_in_process(pu.make_runner(d, "float32", 32, max_requests=1), ru.whole([seq]))
    assert ru.rel_err(got[0], ref) < TOL["float32"]


def _half_rotated(h, T_, p, m):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = plain.rotate((h @ T_[p + "q"].T + T_[p + "q.b"]).reshape(T, H, d), m["rot"]["dims"], m["rot"]["base"], "half")
    k = plain.rotate((h @ T_[p + "k"].T + T_[p + "k.b"]).reshape(T, G, d), m["rot"]["dims"], m["rot"]["base"], "half")
    v = (h @ T_[p + "v"].T + T_[p + "v.b"]).reshape(T, G, dv)
    o = plain.windowed_softmax_attention(q, k, v, m["scale"], m["mask"]["size"], sink=T_[p + "sink"])
    return o.reshape(T, H * dv) @ T_[p + "o"].T + T_[p + "o.b"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_graphs(models, dtype):
    """300 tokens one by one behind a short prompt, replayed from CUDA graphs, two requests side by side."""
    d, cfg, _, _ = models["B"]
    c, w = plain.load(d)
    seqs = pu.sequences(cfg["vocab"], (330, 317), seed=4)
    ref = [plain.forward(c, w, s) for s in seqs]
    runner = pu.make_runner(d, dtype, 704, page_size=16, max_requests=2, graphs=True, context=352)
    assert runner.model.graph_safe
    steps = ru.batched_decode(seqs, tails=[300, 300])
    got = ru.run_in_process(runner, steps)
    assert runner.graph_replays > 250
    check(got, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_binary(models, tmp_path, dtype):
    d, cfg, seqs, ref = models["A"]
    steps = ru.mixed(seqs, live=4, seed=5)
    got = ru.run_trace_binary(d, dtype, steps, str(tmp_path), max_tokens=5 * 64, vocab=cfg["vocab"])
    check(got, ref, dtype)


def test_greedy_generation_through_the_engine(models):
    """Engine.generate (scheduler, sampler, pipelined decode) gives the plain implementation's greedy tokens."""
    from hfee_b200 import Engine, SamplingOptions
    d, cfg, seqs, _ = models["A"]
    c, w = plain.load(d)
    prompts = [seqs[0], seqs[1], seqs[7], seqs[2], seqs[6]]
    want = [plain.greedy(c, w, p, 12) for p in prompts]
    eng = Engine(d, dtype="float32", page_size=16, max_context=128, max_requests=3, max_batch_tokens=48, prefill_chunk=11)
    got = [r.token_ids for r in eng.generate(prompts, SamplingOptions.greedy(num_predict=12))]
    assert got == want


def test_command_line_generates(models):
    """``bin/hfee-b200 run`` on a Pupinex folder: greedy tokens of the plain implementation, and a seeded draw through
    the sampling chain that repeats."""
    import os, subprocess, sys
    d, cfg, seqs, _ = models["B"]
    c, w = plain.load(d)
    toks = plain.greedy(c, w, [5, 6, 7], 6)
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "hfee-b200")
    base = [sys.executable, exe, "run", d, "--prompt-ids", "5,6,7", "--num-predict", "6", "--dtype", "float32", "--num-ctx", "256"]
    p = subprocess.run(base + ["--temperature", "0", "--repeat-penalty", "1"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    assert p.stdout.split("\n")[0].split() == [str(t) for t in toks]
    draws = [subprocess.run(base + ["--temperature", "0.9", "--top-k", "20", "--seed", "7"], capture_output=True, text=True,
                            timeout=300).stdout.split("\n")[0] for _ in range(2)]
    assert draws[0] == draws[1] and len(draws[0].split()) == 6
