#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on the Llama-3.2-1B shape with random
bfloat16 weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 1b|8b|13b] [--layers L] [--dtype bfloat16|float32] [--breakdown]

A "step" is one decode step of a batch of 8 requests whose prompts of 2,048 tokens
are already cached (context limit 4,096).  The JSON line carries: ``value`` (decoded
tokens a second, timed on the device over exactly K steps), ``e2e`` (the same through
``Engine.generate``: host tokens in, host tokens out), ``prefill`` (one prompt of
2,048 tokens), ``roofline`` (bytes a decode step must read over its time, against the
measured HBM copy bandwidth), ``points`` (decode at batch 1 and 64), ``clocks`` and
``gpu_launches``.  Weights (2.5 GB) and the cache of the live requests are far larger
than the 126 MB L2, so no L2 flush is needed between steps.

``--shape 8b`` / ``13b`` run the layer sizes of Llama-3.1-8B / Llama-2-13B (by default with fewer
layers, named beside the full number in ``config``), ``--dtype float32`` the true 32-bit path.
``--design dobelix`` prints, instead of the line above, prompt and decode times of a Dobelix model (linear
attention with decay, chunked sigmoid attention, short convolutions, norms on the sublayers' outputs) beside a
Llama model of the same width, heads, feed-forward and number of layers, with what each class of kernels costs;
``--design bamipel`` the same for a Bamipel model (gated delta rule, latent attention under a sliding window, gated
grouped-query attention, norms on both sides of every sublayer, a relu^2 feed-forward); ``--design muvetar`` for a
Muvetar model (minGRU layers in turn with softmax attention under a logarithmic distance penalty beside a selective
scan; routed experts with a shared one whose active sizes add up to the dense feed-forward; depth averaging);
``--design pupinex`` for a Pupinex model (windowed attention with normed queries and keys beside a matrix memory, windowed
attention with a sink, gated linear attention with a decay per key channel; a clamped gated feed-forward in turn with
group-limited routed experts and a gated shared one; a hashed bigram embedding and layer norms).
``--breakdown`` prints, instead of the line above, what each class of kernels costs inside the decode
step at batch 1, 8 and 64 and inside the prompt pass: the step is timed again with that class's
launches left out (results wrong, timing not), and the difference is the class's cost in place.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: the Llama-3.2-1B shape.
MODEL = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 16, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": True,
}
# BASELINE.json configs[3] and configs[4]: the Llama-3.1-8B and Llama-2-13B shapes.
SHAPES = {
    "1b": (MODEL, "llama-3.2-1b-shape", 16),
    "8b": ({
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
        "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": False,
    }, "llama-3.1-8b-shape", 8),
    "13b": ({
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 40,
        "head_dim": 128, "intermediate_size": 13824, "vocab_size": 32000, "rope_theta": 10000.0,
        "rope_scaling": None, "rms_norm_eps": 1e-5, "max_position_embeddings": 4096, "tie_word_embeddings": False,
    }, "llama-2-13b-shape", 8),
}
E2E_MIN_STEPS = 128                               # the wall-clock window of the end-to-end number never shrinks below this
PROMPT = 2048
CONTEXT = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PUBLISHED_TOK_S = 7.0      # "about 7" tokens/s for llama3.2:1b on a 2-core VPS, the reference's README


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in list(out) + ["sm_max_mhz"]:
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi sampling SM clocks and throttle reasons while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.proc = None

    def summary(self):
        self.stop()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, layers, elem=2):
    """Sizes a decode step reads: every matrix once (the embedding table only as the head, or the
    head of its own), ``elem`` bytes per weight and cache element."""
    d, h, kv, hd, i, v = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                          cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    layer_params = d * (h + 2 * kv) * hd + h * hd * d + 3 * d * i
    return {"layer_params": layer_params, "head_params": v * d,
            "weight_bytes": elem * (layers * layer_params + v * d) + 4 * (2 * layers + 1) * d,
            "kv_bytes_per_token": 2 * layers * kv * hd * elem}


def prefill_flops(cfg, layers, t):
    n = model_numbers(cfg, layers)
    attn = 4 * layers * cfg["num_attention_heads"] * cfg["head_dim"] * t * (t + 1) // 2
    return 2 * t * layers * n["layer_params"] + attn + 2 * n["head_params"]


def dobelix_like(model, layers, chunk=128):
    """A Dobelix configuration of the layer sizes of the Llama configuration ``model``: every third layer
    chunked sigmoid attention (from the second on), the others linear attention with as many heads."""
    h, kv, hd = model["num_attention_heads"], model["num_key_value_heads"], model["head_dim"]
    ff = {"kind": "dense", "ff": model["intermediate_size"]}
    decay = [1.0 - 2.0 ** (-1 - 7 * i / max(1, h - 1)) for i in range(h)]
    out = []
    for i in range(layers):
        if i % 3 == 1:
            out.append({"type": "attention", "mlp": ff,
                        "mixer": {"heads": h, "kv_heads": kv, "dim": hd, "vdim": hd, "mask": {"size": chunk},
                                  "rot": {"dims": hd, "base": 10000.0}, "scale": hd ** -0.5}})
        else:
            out.append({"type": "lightning", "mlp": ff, "mixer": {"heads": h, "dim": hd, "vdim": hd, "decay": decay}})
    return {"architecture": "Dobelix", "vocab": model["vocab_size"], "width": model["hidden_size"], "layers": out,
            "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "embedding": {"scale": 1.0}, "logit_scale": 1.0}


def bamipel_like(model, layers, window=512):
    """A Bamipel configuration of the layer sizes of the Llama configuration ``model``: in turn the gated delta rule
    (as many value heads, a query/key head per key/value head), latent attention (a key/value latent of four head
    sizes, a rotated part of half a head, a query latent of three eighths of the width, a sliding window) and gated
    grouped-query attention."""
    h, kv, hd = model["num_attention_heads"], model["num_key_value_heads"], model["head_dim"]
    ff = {"kind": "dense", "ff": model["intermediate_size"]}
    width = model["hidden_size"]
    out = []
    for i in range(layers):
        if i % 3 == 0:
            out.append({"type": "delta", "mlp": ff, "mixer": {"heads": h, "kv_heads": kv, "dim": hd, "vdim": hd, "conv": 4}})
        elif i % 3 == 1:
            out.append({"type": "latent_attention", "mlp": ff,
                        "mixer": {"heads": h, "dim": hd, "rot_dim": hd // 2, "vdim": hd, "q_rank": 3 * width // 8,
                                  "kv_rank": 4 * hd, "mask": {"size": window}, "rot": {"dims": hd // 2, "base": 10000.0},
                                  "scale": (hd + hd // 2) ** -0.5}})
        else:
            out.append({"type": "attention", "mlp": ff,
                        "mixer": {"heads": h, "kv_heads": kv, "dim": hd, "vdim": hd, "scale": 1.0 / hd,
                                  "rot": {"dims": hd, "base": 500000.0,
                                          "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}})
    return {"architecture": "Bamipel", "vocab": model["vocab_size"], "width": width, "layers": out, "norm": {"eps": 1e-5}}


def muvetar_like(model, layers, experts=16, top=2):
    """A Muvetar configuration of the layer sizes of the Llama configuration ``model``: in turn a parallel mixer
    (distance attention with the Llama heads beside a selective scan of the model's width, 16 state entries per channel, a
    step-size rank of a sixteenth of the width, four taps) and a minGRU of the model's width; every layer with ``experts``
    routed experts of a quarter of the dense feed-forward each (``top`` chosen) and a shared one of half of it, so that a
    token passes as many feed-forward weights as in the dense model."""
    h, kv, hd = model["num_attention_heads"], model["num_key_value_heads"], model["head_dim"]
    width, ff = model["hidden_size"], model["intermediate_size"]
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": 1.0},
           "expert": {"ff": ff // 4, "limit": 7.0}, "shared": {"ff": ff // 2, "limit": 7.0}}
    out = []
    for i in range(layers):
        if i % 2 == 0:
            out.append({"type": "parallel", "mlp": mlp,
                        "mixer": {"left": {"heads": h, "kv_heads": kv, "dim": hd, "vdim": hd, "scale": hd ** -0.5},
                                  "right": {"inner": width, "state": 16, "dt_rank": width // 16, "conv": 4},
                                  "left_scale": 1.0, "right_scale": 1.0}})
        else:
            out.append({"type": "mingru", "mlp": mlp, "mixer": {"width": width}})
    return {"architecture": "Muvetar", "vocab": model["vocab_size"], "width": width, "layers": out, "norm": {"eps": 1e-5},
            "residual_mult": 1.0, "logit_softcap": 30.0}


def pupinex_like(model, layers, experts=16, top=2):
    """A Pupinex configuration of the layer sizes of the Llama configuration ``model``, layer types in turn: a parallel
    mixer (windowed attention with the Llama heads, normed queries and keys, beside a matrix memory with as many heads as
    the model has key/value heads, keys of the head size and values that fill the width), windowed attention with a sink,
    gated linear attention (the same heads, keys of twice the head size, values that fill the width, a decay projection of
    rank 16), and attention again; windows of 1,024 positions, half of every head rotated.  The attention layers carry
    ``experts`` routed experts of a quarter of the dense feed-forward each (``top`` chosen, two groups of which one is
    kept) and a gated shared one of half of it, the other layers the dense clamped feed-forward, so that a token passes
    as many feed-forward weights as in the dense model.  No stretch of layers is looped."""
    h, kv, hd = model["num_attention_heads"], model["num_key_value_heads"], model["head_dim"]
    width, ff = model["hidden_size"], model["intermediate_size"]
    moe = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": 2, "keep": 1}},
           "expert": {"ff": ff // 4}, "shared": {"ff": ff // 2}}
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    attn = lambda **more: dict({"heads": h, "kv_heads": kv, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "mask": {"size": 1024}}, **more)
    kinds = [
        {"type": "parallel", "mlp": dense,
         "mixer": {"left": attn(rot={"dims": hd // 2, "base": 500000.0, "scaling": {"factor": 4.0}}),
                   "right": {"heads": kv, "dim": hd, "vdim": width // kv, "gate_cap": 15.0}, "left_scale": 1.0, "right_scale": 1.0}},
        {"type": "attention", "mlp": moe, "mixer": attn(rot={"dims": hd // 2, "base": 500000.0})},
        {"type": "gla", "mlp": dense, "mixer": {"heads": kv, "dim": 2 * hd, "vdim": width // kv, "tau": 16.0, "rank": 16}},
        {"type": "attention", "mlp": moe, "mixer": attn(rot={"dims": hd // 2, "base": 500000.0})},
    ]
    return {"architecture": "Pupinex", "vocab": model["vocab_size"], "width": width, "layers": [kinds[i % 4] for i in range(layers)],
            "norm": {"eps": 1e-5}, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}}}


DESIGNS = {"dobelix": dobelix_like, "bamipel": bamipel_like, "muvetar": muvetar_like, "pupinex": pupinex_like}
# kernel classes (the names the parts tag their launches with) that only some layers of a design have: class -> the layer
# types that have it; every other class is counted once per layer ("head": once per model)
DESIGN_CLASSES = {
    "dobelix": {"conv": ("lightning", "attention"), "gate": ("lightning",), "linear_attention": ("lightning",),
                "rope": ("attention",), "attention": ("attention",)},
    "bamipel": {"conv": ("delta",), "delta_rule": ("delta",), "gate": ("delta",), "rope": ("attention", "latent_attention"),
                "attention": ("attention", "latent_attention"), "fold": ("latent_attention",), "expand": ("latent_attention",)},
    "muvetar": {"conv": ("parallel",), "scan_proj": ("parallel",), "scan": ("parallel", "mingru"), "rope": ("parallel",),
                "attention": ("parallel",), "router": ("parallel", "mingru"), "experts": ("parallel", "mingru")},
    "pupinex": {"rope": ("parallel", "attention"), "attention": ("parallel", "attention"), "scan_proj": ("parallel", "gla"),
                "linear_attention": ("parallel", "gla"), "gate": ("parallel", "gla"), "router": ("attention",), "experts": ("attention",)},
}
CLASS_ORDER = ("conv", "norm", "qkv", "rope", "fold", "attention", "expand", "linear_attention", "delta_rule", "scan_proj", "scan",
               "gate", "o", "router", "experts", "gate_up", "up", "down", "head")


def design_comparison(args):
    """Prompt pass and decode step of a model of the named design and of the Llama model of equal layer sizes, and the cost
    of each class of kernels inside them (step time minus step time with the class's launches left out)."""
    import shutil
    import numpy as np
    import torch
    from hfee_b200 import Engine, StepEntry, write_random_model
    from hfee_b200.kernels import ops

    pk = peaks()
    base, base_name, _ = SHAPES[args.shape]
    layers = args.layers or 6
    base = dict(base, num_hidden_layers=layers, vocab_size=32768, tie_word_embeddings=True,
                max_position_embeddings=max(base["max_position_embeddings"], 2 * args.prompt))
    designs = {"llama": base, args.design: DESIGNS[args.design](base, layers)}
    rng = np.random.default_rng(0)
    out = {"design_comparison": f"{base_name} layer sizes, {layers} layers, vocabulary 32768, bf16, random weights",
           "prompt_tokens": args.prompt, "decode_batch": args.batch,
           "classes": "us per layer that has the class: step time minus step time with the class left out"}
    clocks = ClockSampler()
    clocks.start()
    for name, cfg in designs.items():
        tmp = tempfile.mkdtemp(prefix="hfee_bench_")
        write_random_model(tmp, cfg, seed=0, dtype="bfloat16")
        engine = Engine(tmp, dtype=args.dtype, page_size=64, max_requests=args.batch, max_context=2 * args.prompt,
                        max_batch_tokens=args.prompt, max_cache_tokens=args.batch * 2 * args.prompt,
                        use_cuda_graphs=not args.no_graphs)
        shutil.rmtree(tmp, ignore_errors=True)
        runner = engine.runner
        vocab = 32768

        def timed(fn, iters):
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(iters):
                fn(i)
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / iters

        def prefill_ms(tokens, iters=3):
            prompt = rng.integers(0, vocab, size=tokens).tolist()

            def once(_):
                s = runner.open()
                runner.step([StepEntry(s, prompt, [tokens - 1])])
                runner.close(s)
            for _ in range(3):
                once(0)
            return timed(once, iters)

        def decode_ms(batch, steps=48):
            slots = [runner.open() for _ in range(batch)]
            for s in slots:
                runner.step([StepEntry(s, rng.integers(0, vocab, size=args.prompt).tolist(), [])])
            feed = rng.integers(0, vocab, size=(steps + 4, batch)).tolist()
            one = lambda i: runner.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            for i in range(4):
                one(i)
            ms = timed(lambda i: one(4 + i), steps)
            for s in slots:
                runner.close(s)
            return ms

        def forget_graphs():
            runner._graphs.clear()
            runner._graph_seen.clear()

        if name == "llama":
            having = {"rope": layers, "attention": layers, "gate_up": layers, "up": 0}
            having.update({c: 0 for cs in DESIGN_CLASSES.values() for c in cs if c not in having})
        else:
            kinds = [l["type"] for l in cfg["layers"]]
            having = {c: sum(kinds.count(k) for k in types) for c, types in DESIGN_CLASSES[name].items()}
            having.update({c: 0 for cs in DESIGN_CLASSES.values() for c in cs if c not in having})
            having.update({"gate_up": 0, "up": layers} if name == "bamipel" else {"gate_up": layers, "up": 0})

        def classes_of(measure, rounds=3):
            res = {}
            for c in CLASS_ORDER:
                n = having.get(c, 1 if c == "head" else layers)
                if n == 0:
                    continue
                diffs = []
                for _ in range(rounds):
                    ops.leave_out([])
                    forget_graphs()
                    whole = measure()
                    ops.leave_out([c])
                    forget_graphs()
                    diffs.append(whole - measure())
                res[c] = round(statistics.median(diffs) * 1e3 / n, 2)
            ops.leave_out([])
            forget_graphs()
            return res

        r = {"prefill_ms": {str(t): round(prefill_ms(t), 3) for t in sorted({512, args.prompt})},
             "decode_ms": {str(b): round(decode_ms(b), 4) for b in sorted({1, args.batch})}}
        r["prefill_tok_s"] = round(args.prompt / (r["prefill_ms"][str(args.prompt)] / 1e3), 1)
        r["decode_tok_s"] = round(args.batch / (r["decode_ms"][str(args.batch)] / 1e3), 1)
        if not args.no_points:
            r["prefill_classes_us"] = classes_of(lambda: prefill_ms(args.prompt, 2))
            r["decode_classes_us"] = classes_of(lambda: decode_ms(args.batch, 32))
        out[name] = r
        del engine, runner
        torch.cuda.empty_cache()
    out["clocks"] = clocks.summary()
    out["peaks"] = {k: pk[k] for k in ("hbm_gbs", "bf16_tflops", "source") if k in pk}
    print(json.dumps(out))
    return 0


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "hostfog/hfee is a Go program with no Python package (pip: 'neither setup.py nor "
                      "pyproject.toml found') and no Go toolchain is installed, so it cannot be built or run here"}))
    return 0


def main():
    global PROMPT, CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="layer sizes: Llama-3.2-1B (the headline), 3.1-8B, 2-13B")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers of the same sizes, if memory or time needs it (config names both numbers)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--breakdown", action="store_true", help="cost of each class of kernels inside the steps, instead of the bench line")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="profiling aid: run just one of the measurements (the JSON line is then partial)")
    ap.add_argument("--prompt", type=int, default=PROMPT,
                    help="tokens of the prompts (other context lengths than the headline's 2,048; the cache holds twice as many per request)")
    ap.add_argument("--no-graphs", action="store_true", help="profiling aid: launch decode kernels one by one")
    ap.add_argument("--design", default=None, choices=sorted(DESIGNS),
                    help="instead of the bench line: this design beside the Llama model of equal layer sizes "
                         "(--shape, --layers, --prompt, --batch apply; --no-points skips the cost per class of kernels)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.design:
        return design_comparison(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.prompt != PROMPT:
        PROMPT, CONTEXT = args.prompt, max(CONTEXT, 2 * args.prompt)

    import numpy as np
    import torch
    from hfee_b200 import Engine, SamplingOptions, StepEntry, write_random_model
    from hfee_b200.kernels import ops

    pk = peaks()
    model, model_name, default_layers = SHAPES[args.shape]
    full_layers = model["num_hidden_layers"]
    layers = args.layers or default_layers
    f32 = args.dtype == "float32"
    elem = 4 if f32 else 2
    cfg = dict(model, num_hidden_layers=layers)
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], CONTEXT)
    nums = model_numbers(cfg, layers, elem)
    context = min(CONTEXT, cfg["max_position_embeddings"])
    if f32:      # no tensor cores on this path: FFMA rate of this device at its highest clock
        props = torch.cuda.get_device_properties(0)
        compute_peak = props.multi_processor_count * 128 * 2 * (pk.get("sm_max_mhz") or 1965.0) * 1e6
    else:
        compute_peak = pk["bf16_tflops"] * 1e12
    rng = np.random.default_rng(0)
    tmp = tempfile.mkdtemp(prefix="hfee_bench_")
    t0 = time.time()
    write_random_model(tmp, cfg, seed=0, dtype="bfloat16")
    print(f"[bench] random model written in {time.time() - t0:.0f}s", file=sys.stderr, flush=True)

    if args.only != "all":
        args.no_points = args.no_e2e = True
    max_b = 64 if (args.breakdown or not args.no_points) else args.batch
    max_b = max(max_b, args.batch)
    engine = Engine(tmp, dtype=args.dtype, page_size=64, max_requests=max_b, max_context=context,
                    max_batch_tokens=PROMPT, max_cache_tokens=max_b * context, use_cuda_graphs=not args.no_graphs)
    runner = engine.runner
    import shutil
    shutil.rmtree(tmp, ignore_errors=True)
    vocab = cfg["vocab_size"]
    sample_out = torch.zeros(max_b, dtype=torch.int32, device=runner.device)
    argmax_scratch = engine.sampler.argmax_scratch

    def timed(fn, iters):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(iters):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    prompt = rng.integers(0, vocab, size=PROMPT).tolist()

    def prefill_once(_):
        s = runner.open()
        runner.step([StepEntry(s, prompt, [PROMPT - 1])])
        runner.close(s)

    def decode_point(batch, steps, warmup, quiet=False):
        """Time ``steps`` decode steps of ``batch`` requests with prompts of PROMPT tokens cached."""
        slots = [runner.open() for _ in range(batch)]
        for s in slots:
            runner.step([StepEntry(s, rng.integers(0, vocab, size=PROMPT).tolist(), [])])
        start = PROMPT
        feed = rng.integers(0, vocab, size=(warmup + steps, batch)).tolist()

        def one(i):
            logits = runner.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            ops.tag("sample")
            ops.argmax(logits, sample_out[:batch], argmax_scratch)

        for i in range(warmup):
            one(i)
        before = ops.launch_count()
        if not quiet:
            print(f"[bench] timed decode (batch {batch}) starts after {before} launches", file=sys.stderr, flush=True)
        ms = timed(lambda i: one(warmup + i), steps)
        launches = ops.launch_count() - before
        ctx = start + warmup + (steps - 1) / 2.0 + 1
        for s in slots:
            runner.close(s)
        return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
                "bytes": nums["weight_bytes"] + batch * ctx * nums["kv_bytes_per_token"], "context": ctx}

    config = {"model": model_name, "global_batch": args.batch, "seq_len": context,
              "prompt_len": PROMPT, "parallelism": "single_gpu", "layers": layers,
              "layers_full": full_layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
              "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
              "intermediate": cfg["intermediate_size"], "vocab": vocab, "tied_embeddings": bool(cfg["tie_word_embeddings"]),
              "page_size": 64, "weights": "random bf16 seed 0", "l2": "inputs larger than L2",
              "peaks": pk["source"] + (", float32 against the FFMA rate" if f32 else "")}

    # ---------------------------------------------------------------- cost of each class of kernels
    if args.breakdown:
        per_layer = ["norm", "qkv", "rope", "attention", "o", "gate_up", "down"]
        once = ["embed", "head", "sample"]
        out = {"breakdown": "step time minus step time with the class left out; us per layer for layer classes, us per step for the rest",
               "config": config, "dtype": "bf16" if not f32 else "fp32"}

        def forget_graphs():
            runner._graphs.clear()
            runner._graph_seen.clear()

        def classes_of(measure, rounds=3):
            """Whole step and step without a class back to back, ``rounds`` times; the class costs the median
            of the differences of such pairs (the clocks move under the power cap during a run this long,
            and the two halves of a pair see the same clocks)."""
            whole_all = []
            res = {}
            for c in per_layer + once:
                diffs = []
                for _ in range(rounds):
                    ops.leave_out([])
                    forget_graphs()
                    whole = measure()
                    ops.leave_out([c])
                    forget_graphs()
                    diffs.append(whole - measure())
                    whole_all.append(whole)
                res[c] = round(statistics.median(diffs) * 1e3 / (layers if c in per_layer else 1), 2)
            ops.leave_out([])
            forget_graphs()
            res["step_ms"] = round(statistics.median(whole_all), 4)
            res["step_ms_spread"] = round(max(whole_all) - min(whole_all), 4)
            res["sum_ms"] = round(sum(res[c] * (layers if c in per_layer else 1) for c in per_layer + once) / 1e3, 4)
            return res

        clocks = ClockSampler()
        clocks.start()
        for b in (1, 8, 64):            # every measurement on freshly read prompts: the same context each time
            out[f"decode_b{b}"] = classes_of(lambda: decode_point(b, 64, 4, quiet=True)["ms_per_step"])
        for _ in range(args.warmup):
            prefill_once(0)
        out["prefill_2048"] = classes_of(lambda: timed(prefill_once, 2) / 2, rounds=7)
        out["clocks"] = clocks.summary()
        print(json.dumps(out))
        return 0

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    clocks = ClockSampler()
    prefill = None
    if args.only in ("all", "prefill"):
        for _ in range(args.warmup):
            prefill_once(0)
        clocks.start()
        p_iters = 5 if args.only == "all" else 1
        print(f"[bench] timed prefill starts after {ops.launch_count()} launches", file=sys.stderr, flush=True)
        p_ms = timed(prefill_once, p_iters) / p_iters
        p_flops = prefill_flops(cfg, layers, PROMPT)
        prefill = {"value": round(PROMPT / (p_ms / 1e3), 1), "tokens": PROMPT, "ms": round(p_ms, 3),
                   "frac": round(p_flops / (p_ms / 1e3) / compute_peak, 4)}
    else:
        clocks.start()
    if args.only == "prefill":
        print(json.dumps({"prefill": prefill, "clocks": clocks.summary()}))
        return 0

    # ---------------------------------------------------------------- decode
    main_pt = decode_point(args.batch, args.steps, args.warmup)
    clock_summary = clocks.summary()
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(decode_point(b, min(args.steps, 64), args.warmup)["tok_s"], 1)

    # ---------------------------------------------------------------- end to end through generate()
    # Host tokens in, host tokens out: every step copies its token ids and positions from pinned
    # host memory and reads the sampled ids back.  Prompts are read first; the timed window opens
    # when every request has produced `warmup` tokens (all are decoding by then) and closes when
    # the first one ends, so it holds decode steps of the full batch only.  It is a wall-clock
    # window, so it never holds fewer than E2E_MIN_STEPS steps, whatever --steps is.
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(args.steps, E2E_MIN_STEPS)
        e2e_warm = max(args.warmup, 8)         # the decode step's CUDA graph is captured in the first few steps
        prompts = [rng.integers(0, vocab, size=PROMPT).tolist() for _ in range(args.batch)]
        opts = SamplingOptions.greedy(num_predict=e2e_warm + e2e_steps)
        counts = [0] * args.batch
        marks = {}

        def on_token(i, tok):
            counts[i] += 1
            if "start" not in marks and min(counts) >= e2e_warm:
                marks["start"] = (time.perf_counter(), sum(counts), engine.h2d_bytes, engine.d2h_bytes, runner.steps_run)
            if "start" in marks and "end" not in marks and max(counts) >= e2e_warm + e2e_steps:
                marks["end"] = (time.perf_counter(), sum(counts), engine.h2d_bytes, engine.d2h_bytes, runner.steps_run)

        engine.generate(prompts, opts, on_token=on_token)
        (t0_, n0_, h0, d0, s0), (t1_, n1_, h1, d1, s1) = marks["start"], marks["end"]
        n_steps = max(1, s1 - s0)
        e2e = {"value": round((n1_ - n0_) / (t1_ - t0_), 1), "unit": "tokens/s",
               "h2d_bytes_per_step": round((h1 - h0) / n_steps, 1),
               "d2h_bytes_per_step": round((d1 - d0) / n_steps, 1), "steps": n_steps}

    achieved = main_pt["bytes"] / (main_pt["ms_per_step"] / 1e3) / 1e9
    # The reference publishes one figure: "about 7" tokens/s for one conversation with llama3.2:1b (a
    # 2-core CPU, quantised weights).  The like-for-like point here is decode at batch 1 of the 1B shape.
    single = points.get("decode_b1") if args.shape == "1b" and not f32 else None
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({model_name.replace('-shape', '').replace('llama', 'Llama')} shape)",
        "value": round(main_pt["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_pt["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(single / PUBLISHED_TOK_S, 1) if single else None,
        "vs_baseline_of": "decode_b1 over the reference's published single-conversation rate (CPU, quantised weights)",
        "dtype": "fp32" if f32 else "bf16", "data": "synthetic",
        "impl": "ours",
        "config": config,
        "e2e": e2e,
        "gpu_launches": int(main_pt["launches"]),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
