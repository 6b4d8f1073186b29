#!/usr/bin/env python3
"""Measurement of the library's headline metric on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl own|reference]

A "step" is one decode step of the batch.  The default run has the layer sizes
of SmolLM2-1.7B (random weights, bfloat16), a batch of 8 and sequences that end
at a context of 8192 tokens.  It prints ONE JSON line:

  value      decoded tokens a second, device time of K replayed decode steps
             (the sampled tokens feed the next step on the device)
  e2e        the same through the public entry point DecodeBatch.step_host:
             every step uploads the tokens it feeds from pinned host memory and
             downloads the tokens it sampled
  prefill    one prompt of 2,048 tokens through step(), its token ids handed over
             as an array (the figure reported; `ms_from_list` is the same with a
             Python list of ints): tokens a second, and the step's flops / time /
             the bfloat16 matrix peak
  roofline   the decode step against HBM: bytes it has to read (every weight
             once, the cache of the live sequences) / its time / the copy peak
  points     decode tokens a second at batch 1 and 64 (same context), and
             decode_b{1,8,64}_u2048: batches whose prompts, of lengths drawn
             uniformly from [128, 2048] (seeded), were really prefilled through
             step() before the timed decode steps; points_ms and points_roofline
             give every point's milliseconds per step and its fraction of the
             HBM roofline at its own context lengths
  cpu_baseline  for context only: the plain NumPy implementation of tests/ on the
             host, tiny-llama-A, tokens a second

Peaks come from MEASURED_PEAKS.json beside this file if present, else from the
fallback figures of an earlier measurement on the same pool.  Inputs are larger
than L2 (3.4 GB of weights and 1.6 GB of cache per sequence against 126 MB), so
no flush is needed between steps.  For --gpus N > 1 it prints a line that says
so and exits with 2: this library runs on one GPU.
"""
import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SMOLLM2_1P7B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 32,
    "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 49152,
    "rope_theta": 130000.0, "rope_scaling": None, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 8192,
}
LLAMA3_SCALING = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                  "original_max_position_embeddings": 8192}
# The other shapes the reference's engine names, for measurements beside the default.
LLAMA_3P2_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 16, "hidden_size": 2048, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0, "rope_scaling": dict(LLAMA3_SCALING, factor=32.0), "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 131072,
}
LLAMA_3P1_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "rope_theta": 500000.0, "rope_scaling": dict(LLAMA3_SCALING, factor=8.0), "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 131072,
}
SHAPES = {"smollm2-1.7b": ("SmolLM2-1.7B", SMOLLM2_1P7B), "llama-3.2-1b": ("Llama-3.2-1B", LLAMA_3P2_1B),
          "llama-3.1-8b": ("Llama-3.1-8B", LLAMA_3P1_8B)}
FULL_LAYERS = SMOLLM2_1P7B["num_hidden_layers"]
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs.  The
    query polls every 20 ms from before the warm-up on; `mark()` at the start of the
    timed region separates the samples.  The summary is taken over the timed region
    when it is long enough to hold three samples, else over warm-up and timed region
    together (`window` says which)."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.proc = None
        self.marked_at = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def mark(self):
        """The timed region begins now (samples carry nvidia-smi's own time stamps)."""
        self.marked_at = datetime.datetime.now()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.03)                        # let the sample that covers the region's end be taken
        ended_at = datetime.datetime.now()
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        rows = []
        for line in out.splitlines():
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 7:
                continue
            try:
                when = datetime.datetime.strptime(cells[0], "%Y/%m/%d %H:%M:%S.%f")
                rows.append((when, float(cells[1]), float(cells[2]),
                             [n for n, c in zip(self.NAMES, cells[3:7]) if c.lower().startswith("active")]))
            except ValueError:
                continue
        timed = [r for r in rows if self.marked_at is not None and self.marked_at <= r[0] <= ended_at]
        window = "timed region"
        if len(timed) < 3:
            timed, window = rows, "warm-up and timed region"
        sm, mx = [r[1] for r in timed], [r[2] for r in timed]
        reasons = sorted({n for r in timed for n in r[3]})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "window": window, "poll_ms": 20}


def decode_bytes(cfg, n_layers, batch, context):
    """Bytes a decode step has to read: every weight it uses once (bfloat16) and
    the keys and values of the live sequences."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * H + H * q + 3 * H * I + 2 * H
    # a tied head reads the embedding table; a separate one is read instead of it (a
    # decode step reads only a few rows of the table itself)
    weights = 2 * (n_layers * per_layer + V * H + H)
    cache = batch * context * n_layers * 2 * kv * 2
    return weights + cache, weights, cache


def prefill_flops(cfg, n_layers, T):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, hd = cfg["num_attention_heads"], cfg["head_dim"]
    q, kv = nh * hd, cfg["num_key_value_heads"] * hd
    gemm = 2 * T * ((q + 2 * kv) * H + H * q + 3 * H * I)
    attn = 2 * T * T * hd * nh          # causal: half of QK^T and half of PV
    return n_layers * (gemm + attn) + 2 * V * H


def kernel_breakdown(run, repeats, what, n_layers):
    """Where a step's time goes: for every kernel the time it ADDS to the step (its end
    minus the end of the kernel before it; kernels of a step overlap their starts under
    programmatic dependent launch, so durations would count some time twice), summed per
    kernel name; a kernel launched several times per layer (the products) is split by
    its position among those launches (#0, #1, ... in launch order)."""
    import collections
    import torch
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(repeats):
            run()
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                    key=lambda e: e.time_range.start)
    def short(name):
        name = name.replace("(anonymous namespace)::", "").replace("void ", "")
        return name.split("(")[0][:60]
    per_step = collections.Counter(short(e.name) for e in events)
    per_layer = {k: (v // repeats) // n_layers if (v // repeats) % n_layers == 0 else 1 for k, v in per_step.items()}
    seen = collections.Counter()
    added = collections.defaultdict(lambda: [0, 0.0])
    last_end = None
    for e in events:
        begin, end = e.time_range.start, e.time_range.end
        name = short(e.name)
        if per_layer[name] > 1:
            k = seen[name]
            seen[name] = k + 1
            name = f"{name} #{k % per_layer[name]}"
        if last_end is not None:
            gain = max(0.0, end - last_end) if begin - last_end < 50 else end - begin   # a gap: another step begins
            row = added[name]
            row[0] += 1
            row[1] += gain
        last_end = end if last_end is None else max(last_end, end)
    total = sum(t for _, t in added.values())
    print(f"# {what}: time added per kernel, microseconds per step (sum {total / repeats:.1f})")
    for name, (count, t) in sorted(added.items(), key=lambda kv: -kv[1][1]):
        print(f"# {t / repeats:9.1f} us  {100 * t / total:5.1f} %  {count / repeats:6.1f} launches  {name}")


def prefill_only(args, model, cache, vocab, gen):
    """For profilers: `warmup` + `steps` prefills of one 2,048-token prompt."""
    import torch
    from go_tinygrad_b200.engine import StepEntry, step
    prompt = torch.randint(0, vocab, (2048,), generator=gen).tolist()
    times = []
    for i in range(args.warmup + args.steps):
        slot = cache.open_sequence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step(model, cache, [StepEntry(slot, prompt, [2047])])
        b.record()
        torch.cuda.synchronize()
        if i >= args.warmup:
            times.append(a.elapsed_time(b))
        cache.close_sequence(slot)
    if args.breakdown:
        def once():
            slot = cache.open_sequence()
            step(model, cache, [StepEntry(slot, prompt, [2047])])
            cache.close_sequence(slot)
        kernel_breakdown(once, 3, "prefill of 2,048 tokens", args.layers)
    print(json.dumps({"only": "prefill", "ms": round(statistics.median(times), 3)}))
    return 0


def run_own(args):
    import torch
    import go_tinygrad_b200 as lib
    from go_tinygrad_b200.engine import StepEntry, step
    from go_tinygrad_b200.engine.decode import DecodeBatch
    from go_tinygrad_b200.kernels import ops

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    shape_name, shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    cfg = dict(shape, num_hidden_layers=args.layers)
    pk = peaks()
    model = lib.Model.random(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02)
    context, vocab = args.context, cfg["vocab_size"]
    if args.only != "all":
        args.points = False
    biggest = max([args.batch] + ([1, 64] if args.points else []))
    cache = model.new_cache(max_tokens=biggest * context + 64 * 40, max_slots=biggest + 1)
    for grp in cache.groups:                       # synthetic keys and values of unit scale
        grp.storage.normal_(0.0, 1.0)
    gen = torch.Generator().manual_seed(0)

    kv_row = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * args.layers     # cache bytes of one token, all layers
    weight_bytes = decode_bytes(cfg, args.layers, 0, 0)[1]
    # at least this much untimed device work before a timed region (not in the --only modes,
    # which are for profilers and want few launches before the captured ones)
    WARM_MS = 300.0 if args.only == "all" else 0.0

    def decode_run(batch, steps, warmup, host, prompts=None):
        """`steps` timed decode steps of `batch` sequences.  Without `prompts` the
        sequences are equal and end at `context` tokens over synthetic keys and values;
        with them (token lists) every sequence is really prefilled through step(),
        eight prompts a step, and decoding goes on from what the model sampled.
        Returns tokens a second, ms per step, the clock record, launches per step and
        the bytes a timed step reads on average."""
        slots = [cache.open_sequence() for _ in range(batch)]
        if prompts is not None:
            prompts = sorted(prompts, key=len, reverse=True)     # longest first, as the generation loop orders a batch
        if prompts is None:
            starts = [context] * batch
            est_ms = (weight_bytes + batch * context * kv_row) / (pk["hbm_gbs"] * 1e6)
        else:
            starts = [len(p) for p in prompts]
            est_ms = (weight_bytes + sum(starts) * kv_row) / (pk["hbm_gbs"] * 1e6)
        # the clocks settle under load: warm up for `warmup` steps and for WARM_MS at least
        warm = max(warmup, int(WARM_MS / est_ms) + 1)
        if prompts is None:
            warm = max(warmup, min(warm, context - steps - 8))
        total = warm + steps + (6 if args.breakdown else 0)
        sampler = ClockSampler()
        sampler.start()
        if prompts is None:
            for s in slots:
                cache.reserve(s, context)
                cache.advance(s, context - total)
            cache.flush_tables()
            tokens = torch.randint(0, vocab, (batch,), generator=gen).tolist()
        else:
            tokens = []
            for lo in range(0, batch, 8):
                part = list(zip(slots[lo:lo + 8], prompts[lo:lo + 8]))
                logits = step(model, cache, [StepEntry(s, p, [len(p) - 1]) for s, p in part])
                tokens += logits.argmax(dim=1).tolist()
            for s, n in zip(slots, starts):
                cache.reserve(s, n + total)
            cache.flush_tables()
        db = DecodeBatch(model, cache, slots, list(range(batch)), lib.Sampler(0.0, 0),
                         use_graph=not args.eager, chained=not args.no_chain)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches_before = ops.launch_count()
        if host:
            out = db.step_host(tokens, [0] * batch)      # eager: loads and configures kernels
            per_step = ops.launch_count() - launches_before
            for i in range(1, warm):
                out = db.step_host(out, [i] * batch)
            torch.cuda.synchronize()
            first = [cache.length(s) for s in slots]
            sampler.mark()
            start.record()
            for i in range(steps):
                out = db.step_host(out, [warm + i] * batch)
            stop.record()
        else:
            db.set_state(tokens, [0] * batch)
            db._launch()                                 # eager: loads and configures kernels
            per_step = ops.launch_count() - launches_before
            for _ in range(warm - 1):
                db.step_device()
            torch.cuda.synchronize()
            first = [cache.length(s) for s in slots]
            sampler.mark()
            start.record()
            for _ in range(steps):
                db.step_device()
            stop.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = start.elapsed_time(stop) / steps
        # a timed step attends over its sequences' keys: their lengths at the middle of the region
        read_bytes = weight_bytes + sum(n + steps // 2 for n in first) * kv_row
        if args.breakdown and not host:
            kernel_breakdown(db.step_device, 6, f"decode step, batch {batch}, mean context {sum(first) / batch:.0f}", args.layers)
        for s in slots:
            cache.close_sequence(s)
        return {"value": batch / (ms * 1e-3), "ms": ms, "clocks": clocks, "launches": per_step + 1,   # +1: the kernel that feeds tokens back
                "bytes": read_bytes, "mean_context": sum(first) / batch + steps / 2}

    def u2048_prompts(n):
        """The decode workload as the benchmark description words it: prompts of lengths
        uniform in [128, 2048], ids uniform in the vocabulary (seeded)."""
        g = torch.Generator().manual_seed(1)
        lengths = torch.randint(128, 2049, (64,), generator=g).tolist()
        prompts = [torch.randint(0, vocab, (k,), generator=g).tolist() for k in lengths]
        if n > 64:                      # more sequences than the named points use: the same draw goes on
            more = torch.randint(128, 2049, (n - 64,), generator=g).tolist()
            prompts += [torch.randint(0, vocab, (k,), generator=g).tolist() for k in more]
        return prompts[:n]

    if args.only == "decode":          # for profilers: the decode steps and nothing else
        r = decode_run(args.batch, args.steps, args.warmup, host=False,
                       prompts=u2048_prompts(args.batch) if args.workload == "u2048" else None)
        print(json.dumps({"only": "decode", "value": round(r["value"], 1), "ms_per_step": round(r["ms"], 4),
                          "launches_per_step": r["launches"], "eager": args.eager}))
        return 0
    if args.only == "prefill":
        return prefill_only(args, model, cache, vocab, gen)
    main_run = decode_run(args.batch, args.steps, args.warmup, host=False)
    e2e_run = decode_run(args.batch, args.steps, args.warmup, host=True)
    points, points_ms, points_roofline, points_context = {}, {}, {}, {}

    def point(name, r):
        points[name] = round(r["value"], 1)
        points_ms[name] = round(r["ms"], 4)
        points_roofline[name] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        points_context[name] = round(r["mean_context"], 1)
    if args.points:
        few = max(3, args.steps // 2)
        for b in (1, 64):
            point(f"decode_b{b}", decode_run(b, few, args.warmup, host=False))
        prompts = u2048_prompts(64)            # really prefilled, then decoded
        for b in (1, 8, 64):
            point(f"decode_b{b}_u2048", decode_run(b, few if b != args.batch else args.steps, args.warmup,
                                                   host=False, prompts=prompts[:b]))

    # prefill of one 2,048-token prompt through the step function: its ids as an array
    # (the figure reported) and as a Python list of ints (what build_context then converts)
    T = 2048
    prompt = torch.randint(0, vocab, (T,), generator=gen)
    pre = {}
    for kind, tokens in (("array", prompt.numpy()), ("list", prompt.tolist())):
        times = []
        for i in range(3 + 5):
            slot = cache.open_sequence()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            step(model, cache, [StepEntry(slot, tokens, [T - 1])])
            b.record()
            torch.cuda.synchronize()
            if i >= 3:
                times.append(a.elapsed_time(b))
            cache.close_sequence(slot)
        pre[kind] = statistics.median(times)
    pre_ms = pre["array"]
    flops = prefill_flops(cfg, args.layers, T)

    ms = main_run["ms"]
    achieved = main_run["bytes"] / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch}, context {context} ({shape_name} shape)",
        "value": round(main_run["value"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "model": f"{shape_name} shape, random weights", "layers": args.layers,
            "layers_of_model": full_layers, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "rope_theta": cfg["rope_theta"], "tied_head": bool(cfg["tie_word_embeddings"]),
            "global_batch": args.batch, "seq_len": context,
            "prefill_tokens": T, "parallelism": "single GPU", "l2": "inputs larger than L2",
            "peaks": pk["source"], "graph": "decode step replayed as a CUDA graph",
            "warmup_floor_ms": WARM_MS,
        },
        "clocks": main_run["clocks"],
        "e2e": {"value": round(e2e_run["value"], 1), "unit": "tokens/s", "ms_per_step": round(e2e_run["ms"], 4),
                "h2d_bytes_per_step": 3 * 4 * args.batch, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": main_run["launches"] * args.steps,
        "prefill": {"value": round(T / (pre_ms * 1e-3), 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "tokens_given_as": "array", "ms_from_list": round(pre["list"], 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                     "weight_gb": round(weight_bytes / 1e9, 3),
                     "cache_gb": round((main_run["bytes"] - weight_bytes) / 1e9, 3)},
        "points": points, "points_ms": points_ms, "points_roofline": points_roofline,
        "points_context": points_context,
        "cpu_baseline": cpu_baseline(),
    }
    print(json.dumps(line))
    return 0


def cpu_baseline():
    """For context only: the plain NumPy implementation that the tests use as their
    oracle, on the host, at tiny-llama-A (three prompts of 5, 17 and 32 tokens, 16
    greedy tokens each; it recomputes the whole sequence for every token).  The
    reference itself is a Go program that cannot be built here; it reports tokens a
    second the same way, new tokens over wall time (cmd/llmgen/main.go:121-133)."""
    import tempfile
    import numpy as np
    import go_tinygrad_b200 as lib
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    try:
        import plain_llama
    except ImportError:
        return {"unavailable": "tests/plain_llama.py not found"}
    tiny = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2,
            "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
            "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
            "tie_word_embeddings": True, "max_position_embeddings": 128}
    with tempfile.TemporaryDirectory() as folder:
        lib.write_random_model(folder, tiny, seed=0, dtype="float32", std=0.02, norm_std=0.01)
        cfg, w = plain_llama.read_model(folder)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 256, n).tolist() for n in (5, 17, 32)]
    t0 = time.time()
    new = sum(len(plain_llama.generate(cfg, w, p, 16)) for p in prompts)
    elapsed = time.time() - t0
    return {"what": "plain NumPy implementation on the host CPU, tiny-llama-A, float32, no cache",
            "value": round(new / elapsed, 1), "unit": "tokens/s", "tokens": new}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=SMOLLM2_1P7B["max_position_embeddings"])
    ap.add_argument("--shape", default="smollm2-1.7b", choices=sorted(SHAPES),
                    help="the model shape; the default is the one the headline numbers are quoted on")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the model has, where memory or time needs it")
    ap.add_argument("--no-points", dest="points", action="store_false",
                    help="skip the batch-1 and batch-64 decode points")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only and print a short line (for profilers)")
    ap.add_argument("--workload", default="context", choices=["context", "u2048"],
                    help="with --only decode: equal sequences at --context over synthetic keys, or prompts of "
                         "lengths uniform in [128, 2048] that are really prefilled")
    ap.add_argument("--breakdown", action="store_true",
                    help="with --only: also print, as comment lines, the time each kernel adds to a step")
    ap.add_argument("--eager", action="store_true",
                    help="launch the decode step kernel by kernel instead of replaying a graph")
    ap.add_argument("--no-chain", action="store_true",
                    help="decode kernels wait for their predecessor to finish before they are launched")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Go program (go.mod, purego); no Go toolchain is installed "
                          "and pip cannot build it, so it cannot be run here"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"--gpus {args.gpus}: this library runs on one GPU; "
                                   f"there is no multi-GPU path to measure", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    return run_own(args)


if __name__ == "__main__":
    sys.exit(main())
