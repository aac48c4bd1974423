"""The Muvetar decoder on the GPU against the plain implementation of tests/plain_muvetar.py: each mixer and the routed
feed-forward alone, whole prompts, prefill then token by token, portions down to two tokens, mixed batches over few
pages and slots, page edges, far keys and far writes, the first tokens, long decoding, other sizes, and greedy
generation through the engine's entry point."""
import numpy as np
import pytest

import muvetar_util as mu
import plain_muvetar as plain
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
    for name, cfg, seed in (("A", mu.MUV_A, 3), ("B", mu.MUV_B, 4)):
        d = mu.write_model(str(tmp_path_factory.mktemp("muvetar" + name)), cfg, seed)
        c, w = plain.load(d)
        seqs = mu.sequences(cfg["vocab"], LENGTHS, seed=11)
        assert mu.smallest_route_margin(plain, c, w, seqs) > 0.5          # no router's choice is a close call
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
        runner = mu.make_runner(d, dtype, max_tokens=17 * 16, context=112)
    else:
        steps = {"whole": ru.whole, "prefill_then_decode": lambda s: ru.prefill_then_decode(s, tail=20),
                 "portions": ru.portions}[scheme](seqs)
        runner = mu.make_runner(d, dtype, max_tokens=112, max_requests=1)
    check(ru.run_in_process(runner, steps), ref, dtype, scheme)


def test_batch_of_unequal_requests_equals_each_alone(models):
    """float32: a row's sums run in one order whatever else is in the batch."""
    d, cfg, seqs, ref = models["A"]
    alone = ru.run_in_process(mu.make_runner(d, "float32", 112, max_requests=1), ru.whole(seqs))
    runner = mu.make_runner(d, "float32", max_tokens=512, max_requests=8, context=112)
    steps = [{"entries": [(i, s, list(range(len(s)))) for i, s in enumerate(seqs)], "end": list(range(len(seqs)))}]
    together = ru.run_in_process(runner, steps)
    for i in range(len(seqs)):
        assert ru.rel_err(together[i], alone[i]) < 2e-6


ALONE = {
    "mingru": mu.mingru(40),
    "mingru_odd_width": mu.mingru(37),
    "attention_alone": mu.parallel(4, 2, 16, 24, 0.3, 8, 2, 1, 2, left_scale=1.4, right_scale=0.0),
    "attention_one_head_small_values": mu.parallel(1, 1, 40, 8, 0.2, 8, 2, 1, 2, left_scale=0.9, right_scale=0.0),
    "attention_tensor_core_sizes": mu.parallel(4, 1, 64, 64, 0.15, 8, 2, 1, 2, left_scale=1.0, right_scale=0.0),
    "attention_wide_values": mu.parallel(6, 3, 64, 128, 0.12, 8, 2, 1, 2, left_scale=1.0, right_scale=0.0),
    "scan_alone": mu.parallel(1, 1, 8, 8, 0.3, 56, 12, 4, 4, left_scale=0.0, right_scale=1.3),
    "scan_one_state_one_tap": mu.parallel(1, 1, 8, 8, 0.3, 30, 1, 1, 1, left_scale=0.0, right_scale=0.6),
    "scan_large_state": mu.parallel(1, 1, 8, 8, 0.3, 24, 40, 7, 2, left_scale=0.0, right_scale=1.0),
    "both_branches": mu.parallel(2, 1, 24, 16, 0.25, 44, 5, 3, 3, left_scale=0.8, right_scale=1.1),
    "experts_with_shared": mu.mingru(16, mlp=mu.moe(6, 2, 20, 0.6, 2.5, 28, 0.9)),
    "experts_all_chosen_no_shared": mu.mingru(16, mlp=mu.moe(3, 3, 36, 1.5, 0.7)),
    "one_expert_of_one": mu.mingru(16, mlp=mu.moe(1, 1, 12, 1.0, 1.0, 12, 1.0)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", list(ALONE.values()), ids=list(ALONE))
def test_each_mechanism_alone(tmp_path, layer, dtype):
    """One layer (a mixer without feed-forward, or a small mixer with the routed feed-forward): whole, and in portions
    through the cache or state."""
    cfg = mu.config(48, 90, [layer], residual_mult=1.0)
    d = mu.write_model(str(tmp_path), cfg, seed=7)
    c, w = plain.load(d)
    seqs = mu.sequences(90, (37, 3, 64), seed=5)
    ref = [plain.forward(c, w, s) for s in seqs]
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(2, 9, 1, 1, 30, 2))):
        check(ru.run_in_process(mu.make_runner(d, dtype, 64, max_requests=1), steps), ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_fit_no_vector_access(tmp_path, dtype):
    """Width, vocabulary, ranks and head sizes that are multiples of neither 8 nor 4: every kernel takes its scalar path."""
    layers = [mu.parallel(3, 1, 12, 10, 0.3, 22, 3, 5, 3, 0.9, 1.2, mlp=mu.moe(5, 2, 14, 0.8, 1.5, 18, 1.1)),
              mu.mingru(26, mlp=mu.moe(3, 1, 10, 1.3, 2.0)),
              mu.parallel(2, 2, 6, 14, 0.4, 10, 7, 1, 2, 1.0, 0.5)]
    cfg = mu.config(50, 77, layers, eps=3e-6, residual_mult=0.8, softcap=6.0)
    d = mu.write_model(str(tmp_path), cfg, seed=13)
    c, w = plain.load(d)
    seqs = mu.sequences(77, (41, 2, 19), seed=6)
    ref = [plain.forward(c, w, s) for s in seqs]
    rms_tol = 2.5e-2 if dtype == "bfloat16" else None       # short sums average less of the rounding than wider models' do
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(3, 2, 17, 1, 5)), ru.mixed(seqs, live=2, seed=1)):
        check(ru.run_in_process(mu.make_runner(d, dtype, 96, max_requests=2, context=48), steps), ref, dtype, rms_tol=rms_tol)


@pytest.mark.parametrize("taps", [1, 2, 5])
def test_convolution_taps_and_first_tokens(tmp_path, taps):
    """The first tokens of a sequence see zeros in front of it; a portion of one or two tokens is shorter than the
    convolution's history; with one tap there is no history at all."""
    cfg = mu.config(40, 70, [mu.parallel(2, 1, 8, 8, 0.3, 24, 4, 2, taps, 0.5, 1.5)])
    d = mu.write_model(str(tmp_path), cfg, seed=9)
    c, w = plain.load(d)
    seqs = mu.sequences(70, (9, 2, 1, 30), seed=1)
    ref = [plain.forward(c, w, s) for s in seqs]
    runner = mu.make_runner(d, "float32", 32, max_requests=1)
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(1, 1, 2, 1, 3, 17, 2)), ru.prefill_then_decode(seqs, tail=6)):
        check(ru.run_in_process(runner, steps), ref, "float32", f"taps={taps}")
    if taps > 1:        # and the history matters: without the earlier taps the second token's logits differ
        w2 = dict(w)
        w2["l0.mix.right.conv"] = w["l0.mix.right.conv"].copy()
        w2["l0.mix.right.conv"][:, :-1] = 0.0
        assert ru.rel_err(plain.forward(c, w2, seqs[0])[1:], ref[0][1:]) > 20 * TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_distance_penalty_and_page_edges(tmp_path, dtype):
    """A large score scale makes single keys dominate, so a key that is lost, read twice or taken at the wrong distance
    shows: portions that start at, before and after a page's edge, single decoded tokens across edges, and the
    first tokens.  The penalty itself shows: other r1 or r2, or a distance off by one, give other logits."""
    page = 16
    layer = mu.parallel(2, 1, 16, 16, 1.5, 8, 2, 1, 2, left_scale=1.0, right_scale=0.0)
    cfg = mu.config(32, 60, [layer], residual_mult=1.0)
    d = mu.write_model(str(tmp_path), cfg, seed=21)
    c, w = plain.load(d)
    seq = mu.sequences(60, (100,), seed=2)[0]
    ref = plain.forward(c, w, seq)
    for name, change in (("l0.mix.left.r1", lambda v: v * 1.05), ("l0.mix.left.r2", lambda v: v * 1.1), ("l0.mix.left.r1", lambda v: v * 0.0)):
        assert ru.rel_err(plain.forward(c, {**w, name: change(w[name])}, seq)[1:], ref[1:]) > 5 * TOL["float32"]
    cuts = [(100,), (page, page, 100), (page - 1, 2, page - 1, 2, 100), (page + 1, page - 1, 2, 100),
            (47,) + (1,) * 53, (15,) + (1,) * 85, (2, 2, 100), (1, 1, 1, 100)]
    for sizes in cuts:
        steps = ru.portions([seq], sizes=sizes)
        got = ru.run_in_process(mu.make_runner(d, dtype, 112, page_size=page, max_requests=1), steps)
        assert ru.rel_err(got[0], ref) < TOL[dtype], f"cut {sizes[:5]}"


def _far_sequences(first):
    """Two sequences of 400 tokens that differ in their first ``first`` tokens only (tokens 0 and 1 stand nowhere else)."""
    later = [2 + t % 48 for t in mu.sequences(50, (400 - first,), seed=8)[0]]
    return [t % 2 for t in range(first)] + later, [(t + 1) % 2 for t in range(first)] + later


def _far_check(d, dtype, first=1):
    c, w = plain.load(d)
    seq, other = _far_sequences(first)
    ref, ref_other = plain.forward(c, w, seq), plain.forward(c, w, other)
    effect = ru.rel_err(ref_other[-8:], ref[-8:])
    assert effect > 5 * TOL[dtype]                                       # the far token matters
    # float32: rounding of sums.  bfloat16: every logit here hangs on a handful of rounded numbers (one layer, weights
    # made so that one key or a few writes decide), so the largest difference is held to a tenth of what the far
    # token changes, and the root mean square to the usual bound.
    limit = TOL[dtype] if dtype == "float32" else max(TOL[dtype], effect / 10)
    runner = mu.make_runner(d, dtype, 416, page_size=32, max_requests=1)
    for s, r in ((other, ref_other), (seq, ref)):                        # the same slot and pages twice
        steps = ru.portions([s], sizes=(130, 2, 67, 1, 1, 100, 64)) if s is seq else ru.prefill_then_decode([s], tail=40)
        got = ru.run_in_process(runner, steps)
        assert ru.rel_err(got[0], r) < limit and rms_err(got[0], r) < RMS_TOL[dtype]


MARK = 6.0          # the marks' size: well above the position vector's entries, so the norm leaves them large


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(tmp_path, dtype):
    """The first token's key is made to stand out for every later query, by more than the distance penalty takes off
    400 positions away, so its value shows hundreds of tokens later, across pages, after portions and for decoded
    tokens."""
    cfg = mu.config(32, 50, [mu.parallel(2, 2, 16, 8, 0.05, 8, 2, 1, 2, left_scale=1.0, right_scale=0.0)], residual_mult=1.0)

    def marked(tensors):
        mu.mark_first_tokens(tensors, MARK)
        wq, wk = tensors["l0.mix.left.q"], tensors["l0.mix.left.k"]
        wk[:, mu.MARK_A] = wk[:, mu.MARK_B] = 1.0                          # both first tokens: the same loud key
        wk[:, mu.MARK_LATER] = 0.0
        wq[:, mu.MARK_LATER] = 1.0                                         # every later query points at it
        wv = tensors["l0.mix.left.v"]
        wv[:, mu.MARK_A], wv[:, mu.MARK_B] = 1.0, -1.0                      # and the two first tokens carry opposite values
        tensors["l0.mix.left.r1"].fill_(0.5)
        tensors["l0.mix.left.r2"].fill_(1.0)
    _far_check(mu.write_model(str(tmp_path), cfg, seed=33, edit=marked), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_write_reaches_through_the_mingru_state(tmp_path, dtype):
    """Update gates near 1 for the first tokens and near 0 for every later one: what the first tokens wrote still shows
    hundreds of tokens later, after portions, decoded tokens, and a slot that another request used before."""
    cfg = mu.config(32, 50, [mu.mingru(24)], residual_mult=1.0)

    def slow(tensors):
        mu.mark_first_tokens(tensors, MARK)
        wz, wx = tensors["l0.mix.z"], tensors["l0.mix.x"]
        wz.mul_(0.1)
        wz[:, mu.MARK_A] = wz[:, mu.MARK_B] = 2.0
        wz[:, mu.MARK_LATER] = -3.0
        wx[:, mu.MARK_A], wx[:, mu.MARK_B] = 1.0, -1.0                      # the two first tokens write opposite candidates
        tensors["l0.mix.z.b"].zero_()
    _far_check(mu.write_model(str(tmp_path), cfg, seed=35, edit=slow), dtype, first=3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_write_reaches_through_the_scan_state(tmp_path, dtype):
    """A scan that hardly forgets (A near 0), a large step for the first tokens and a tiny one for every later token."""
    cfg = mu.config(32, 50, [mu.parallel(1, 1, 8, 8, 0.3, 24, 6, 2, 2, left_scale=0.0, right_scale=1.0)], residual_mult=1.0)

    def slow(tensors):
        mu.mark_first_tokens(tensors, MARK)
        t = lambda k: tensors["l0.mix.right." + k]
        t("A_log").fill_(-9.0)
        t("in")[0].zero_()                                                  # channel 0 of x carries "this is a first token"
        t("in")[0, mu.MARK_A] = t("in")[0, mu.MARK_B] = 1.0
        t("in")[1:24, mu.MARK_A], t("in")[1:24, mu.MARK_B] = 0.5, -0.5      # the other channels tell the two first tokens apart
        t("conv")[0, :] = 0.0
        t("conv")[0, -1] = 1.0
        t("conv.b")[0] = 0.0
        t("x")[:2].zero_()
        t("x")[0, 0] = 1.5                                                  # the step-size projection reads that channel
        t("dt").zero_()
        t("dt")[:, 0] = 1.0
        t("dt.b").fill_(-6.0)
    _far_check(mu.write_model(str(tmp_path), cfg, seed=37, edit=slow), dtype, first=3)


def test_variants_of_the_plain_implementation_show_in_the_logits(tmp_path):
    """What a wrong reading would compute gives other logits, so the comparison would see it: no residual multiplier on
    the feed-forward, renormalised router weights, a candidate without its two branches, no depth average."""
    cfg = mu.config(48, 40, [mu.mingru(20, mlp=mu.moe(4, 2, 16, 0.8, 2.0, 12, 1.2)), mu.mingru(12)], residual_mult=0.5)
    d = mu.write_model(str(tmp_path), cfg, seed=5)
    c, w = plain.load(d)
    seq = mu.sequences(40, (30,), seed=3)[0]
    ref = plain.forward(c, w, seq)
    assert ru.rel_err(plain.forward({**c, "residual_mult": 1.0}, w, seq), ref) > 1e-3
    w2 = dict(w); w2["l1.dwa"] = np.array([0.0, 0.0, 1.0])                     # the last layer's own result alone
    assert ru.rel_err(plain.forward(c, w2, seq), ref) > 1e-3
    c2 = {**c, "layers": [dict(c["layers"][0], mlp=dict(c["layers"][0]["mlp"], router={"experts": 4, "top": 2, "scale": 1.0})), c["layers"][1]]}
    assert ru.rel_err(plain.forward(c2, w, seq), ref) > 1e-3
    w3 = dict(w); w3["l0.mix.x.b"] = w["l0.mix.x.b"] - 100.0                   # every candidate on the sigmoid branch
    assert ru.rel_err(plain.forward(c, w3, seq), ref) > 1e-3
    got = ru.run_in_process(mu.make_runner(d, "float32", 32, max_requests=1), ru.whole([seq]))
    assert ru.rel_err(got[0], ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_graphs(models, dtype):
    """300 tokens one by one behind a short prompt, replayed from CUDA graphs, two requests side by side."""
    d, cfg, _, _ = models["B"]
    c, w = plain.load(d)
    seqs = mu.sequences(cfg["vocab"], (330, 317), seed=4)
    ref = [plain.forward(c, w, s) for s in seqs]
    runner = mu.make_runner(d, dtype, 704, page_size=16, max_requests=2, graphs=True, context=352)
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
    """``bin/hfee-b200 run`` on a Muvetar folder: greedy tokens of the plain implementation, and a seeded draw
    through the sampling chain that repeats."""
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
