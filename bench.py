"""Decode and prefill throughput of the Qwen3-4B layer sizes with random bfloat16 weights
on one B200.  A "step" is one decode step of the whole batch.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second of K CUDA-graph decode steps
at the given batch (device time, CUDA events); ``e2e`` is the same through
``Engine.generate`` (host token lists in, host token lists out); ``prefill`` is one
2,048-token prompt; ``roofline`` compares the bytes a decode step has to read (every
weight once, the cache of the live requests) with the measured HBM copy bandwidth;
``points`` holds batch 1 and 64; ``workloads`` the reference's three public workloads
(batch x prompt x new tokens) as tokens per second of whole ``generate`` calls, prefill
included.  Only N=1 is supported.

``--impl reference`` runs the unmodified reference engine (a copy of its ``engine/`` folder
under ``baseline/_ref/``) through its own ``Engine(model_path).generate`` on the same
configuration, batch, prompt length and step counts, and prints the same line with
``"impl": "reference"``.  ``--workload 8b|14b`` runs the two larger workloads: batch 16 with
prompts of 64 to 2,048 tokens and 128 greedy steps at the Qwen3-8B sizes; batch 64 with
1,024-token prompts and 256 steps, half of the sequences sampling at temperature 0.8, at the
Qwen3-14B sizes.

``--design lanilix`` measures the Lanilix decoder instead (named configurations
``lanilix-w2048`` and ``lanilix-w4096``: eight layers, three gated-delta-rule layers to one
windowed-attention layer) beside a Qwen3 decoder of the same width, feed-forward, heads, head
size, depth and vocabulary: prefill of one 2,048-token prompt and decode steps at ``--batch``,
and every kernel of the new design alone (cold caches) beside the like kernel of the Qwen3
path, each with the fraction of its roofline.  ``--design bunudra`` does the same for the Bunudra
decoder (``bunudra-w2048``, ``bunudra-w4096``: matrix-memory, chunked-attention and
latent-attention layers with routed experts) beside a Lanilix decoder of the same width, depth,
heads and feed-forward weights, its closest relative here.  ``--design ditilix`` measures the
Ditilix decoder (``ditilix-w2048``, ``ditilix-w4096``: attention over all keys with a score cap and a
query temperature, every other layer reading the keys of the layer before it, one dense
feed-forward with a polynomial of norms and seven routed ones) beside a Qwen3 decoder of the same
width, depth, heads and feed-forward products.  ``--design dubazen`` measures the Dubazen decoder
(``dubazen-w2048``, ``dubazen-w4096``: four copies of the stream joined by hyper-connections, selective
scans, pairs of softmax attention with sinks and linear attention, gated linear attention, routed
experts weighted at their output) beside a Bunudra decoder of the same width, depth, heads and
experts, its closest relative here.  The default run is untouched by all four.
"""

from __future__ import annotations

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

SIZES = {"4b": "qwen3-4b", "8b": "qwen3-8b", "14b": "qwen3-14b"}     # named configurations of the package


def config_json(sizes):
    """The config.json of the package's named configuration (data under config/presets)."""
    with open(os.path.join(ROOT, "thing_htn_2026_b200", "config", "presets", SIZES[sizes] + ".json")) as handle:
        return json.load(handle)


CONTEXT = 4096
PROMPT = 512
PREFILL_TOKENS = 2048
WORKLOADS = ((1, 512, 32), (4, 2048, 32), (16, 512, 128))     # AGENTS.md:56-60 of the reference
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PREFILL_WARM, PREFILL_TIMED, PREFILL_MORE = 2, 3, 5
PREFILL_SETTLE_S = 3.0        # both arms repeat the prefill this long before the figure is taken


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(path) as handle:
            data = json.load(handle)
        for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if key in data:
                out[key] = float(data[key])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
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
        self.file.flush()
        self.file.seek(0)
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def model_numbers(cfg, n_layers):
    """Bytes and flops of the model at ``n_layers`` layers (bfloat16)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Nq, Nkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (Nq + 2 * Nkv) * D * H + Nq * D * H + 2 * I * H + I * H      # matrix elements
    gains = 2 * H + 2 * D
    weight_bytes = 2 * (n_layers * (per_layer + gains) + V * H + H)           # head read once (tied or not)
    kv_bytes_per_token = n_layers * 2 * Nkv * D * 2
    return {"matrix_per_layer": per_layer, "weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token}


def prefill_flops(cfg, n_layers, tokens):
    H, V = cfg["hidden_size"], cfg["vocab_size"]
    Nq, D = cfg["num_attention_heads"], cfg["head_dim"]
    numbers = model_numbers(cfg, n_layers)
    gemm = 2.0 * tokens * n_layers * numbers["matrix_per_layer"] + 2.0 * V * H      # head on one row
    attention = n_layers * 2.0 * 2.0 * Nq * D * tokens * (tokens + 1) / 2            # QK and PV, causal
    return gemm + attention


def run_ours(args):
    import torch
    from thing_htn_2026_b200 import Engine, ops
    from thing_htn_2026_b200.config import config_from_dict
    from thing_htn_2026_b200.engine.generation import Request
    from thing_htn_2026_b200.engine.step import StepEntry

    cfg = config_json(args.sizes)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_layers = cfg["num_hidden_layers"]
    config = config_from_dict(cfg)
    peak = peaks()
    torch.manual_seed(0)
    biggest = max(args.batch, 64 if not args.no_points else args.batch)
    per_seq = args.prompt_len + max(args.steps + args.warmup, 64) + 64
    max_tokens = max(biggest * -(-per_seq // 64) * 64, 4096)
    if not args.no_points:
        max_tokens = max(max_tokens, max(b * -(-(p + n) // 64) * 64 for b, p, n in WORKLOADS))
    engine = Engine.from_config(config, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_batch=biggest)
    backend, vocab = engine.backend, cfg["vocab_size"]
    g = torch.Generator().manual_seed(0)

    def prompts(batch, length):
        return torch.randint(0, vocab, (batch, length), generator=g).tolist()

    def decode_device(batch, steps, warmup, sample_clocks=False):
        """K graph replays timed with CUDA events; returns ms per step and context seen."""
        requests = [Request(p, warmup + steps + 1, 0.0, 0, i) for i, p in enumerate(prompts(batch, args.prompt_len))]
        slots = backend.open_batch(requests)
        try:
            backend.fetch(backend.launch_prefill(slots, [r.tokens for r in requests]))
            for _ in range(warmup):
                backend.fetch(backend.launch_decode(slots))
            torch.cuda.synchronize()
            before = ops.launch_count
            sampler = ClockSampler() if sample_clocks else None
            if sampler:
                sampler.start()
                time.sleep(0.3)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            if args.profiler_range == "decode" and sample_clocks:
                torch.cuda.profiler.start()
            start.record()
            handles = []
            for _ in range(steps):
                handles.append(backend.launch_decode(slots))
                if len(handles) > 3:
                    backend.fetch(handles.pop(0))
            end.record()
            torch.cuda.synchronize()
            for handle in handles:
                backend.fetch(handle)
            if args.profiler_range == "decode" and sample_clocks:
                torch.cuda.profiler.stop()
            clocks = sampler.stop() if sampler else None
            ms = start.elapsed_time(end) / steps
            ctx_mean = args.prompt_len + warmup + (steps - 1) / 2.0
            return ms, ctx_mean, clocks, ops.launch_count - before
        finally:
            backend.close_batch(slots)

    # graphs are captured (and their kernels counted) during warm-up
    ops.launch_count = 0
    ms, ctx_mean, clocks, host_calls = decode_device(args.batch, args.steps, max(args.warmup, 3), sample_clocks=True)
    value = args.batch * 1000.0 / ms
    numbers = model_numbers(cfg, n_layers)
    step_bytes = numbers["weight_bytes"] + args.batch * 2 * cfg["hidden_size"] \
        + args.batch * ctx_mean * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9

    # kernels of this library per decode step: count one eager run of the program
    eager_before = ops.launch_count
    probe = [Request(p, 3, 0.0, 0, i) for i, p in enumerate(prompts(args.batch, 8))]
    slots = backend.open_batch(probe)
    backend.fetch(backend.launch_prefill(slots, [r.tokens for r in probe]))
    backend._set_composition(slots)
    mark = ops.launch_count
    backend._decode_program(args.batch, ops.context_class(16)[1])
    backend.cache.commit(list(slots), [1] * args.batch)
    own_per_step = ops.launch_count - mark
    torch.cuda.synchronize()
    backend.close_batch(slots)

    # end to end through the public entry point
    e2e_prompts = prompts(args.batch, args.prompt_len)
    n_new = args.steps + 1
    list(engine.generate(e2e_prompts, 4))                   # warm: graphs for this batch exist already
    torch.cuda.synchronize()
    uploaded_before = backend.runner.uploaded_bytes
    t0 = time.perf_counter()
    t_first = None
    count = 0
    for step_tokens in engine.generate(e2e_prompts, n_new):
        if t_first is None:
            t_first = time.perf_counter()
        count += 1
    t1 = time.perf_counter()
    assert count == n_new
    e2e_uploaded = backend.runner.uploaded_bytes - uploaded_before
    e2e_decode = args.batch * (n_new - 1) / (t1 - t_first)
    e2e_total = args.batch * n_new / (t1 - t0)

    # prefill of one 2,048-token prompt, the same protocol in both arms.  How fast a GPU under its
    # power cap runs a step like this depends on how warm the minutes before have left it (the arm
    # that runs first on a fresh GPU measured 14.1 ms in its first steps, the other arm 15.3-15.6,
    # whichever engine it was), so the figure is taken where that history has faded: the step is
    # repeated for PREFILL_SETTLE_S seconds and the median of the last five counts.  The median of
    # PREFILL_TIMED steps after the first PREFILL_WARM is kept beside it as `ms_first`.
    runner = backend.runner
    times = []
    settle_started = time.perf_counter()
    rep = 0
    while rep < PREFILL_WARM + PREFILL_TIMED + PREFILL_MORE or time.perf_counter() - settle_started < PREFILL_SETTLE_S:
        (slot,) = backend.cache.open(1)
        toks = prompts(1, PREFILL_TOKENS)[0]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        profiled = args.profiler_range == "prefill" and rep == PREFILL_WARM + PREFILL_TIMED - 1
        if profiled:
            torch.cuda.profiler.start()
        start.record()
        logits = runner.step([StepEntry(slot, toks, (PREFILL_TOKENS - 1,))], check=False)
        end.record()
        torch.cuda.synchronize()
        if profiled:
            torch.cuda.profiler.stop()
        times.append(start.elapsed_time(end))
        backend.cache.close([slot])
        rep += 1
        if args.profiler_range == "prefill" and rep >= PREFILL_WARM + PREFILL_TIMED:
            break                                           # a profiled run needs no more than its one step
    first_ms = statistics.median(times[PREFILL_WARM:PREFILL_WARM + PREFILL_TIMED])
    prefill_ms = statistics.median(times[-5:])
    flops = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (prefill_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": flops / (prefill_ms * 1e-3) / (peak.get("bf16_tflops_sustained", peak["bf16_tflops"]) * 1e12),
               "peak_tflops": peak.get("bf16_tflops_sustained", peak["bf16_tflops"]),
               "frac_burst": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12),
               "ms_first": first_ms, "steps": len(times),
               "note": f"median of the last 5 of {len(times)} steps in a row ({PREFILL_SETTLE_S:.0f} s), so frac is against the "
                       f"peak of a seconds-long loop under the power cap (peak_tflops) and frac_burst against the burst "
                       f"peak; ms_first: median of {PREFILL_TIMED} steps after {PREFILL_WARM}"}

    points = {}
    if not args.no_points:
        for batch in (1, 64):
            pms, _, _, _ = decode_device(batch, min(args.steps, 64), 3)
            points[f"decode_b{batch}"] = batch * 1000.0 / pms

    # The reference's public workloads (batch x prompt x new tokens), by its own definition of
    # throughput: batch * new tokens / time of the whole call, prefill included.
    workloads = {}
    if not args.no_points:
        for batch, prompt_len, n_out in WORKLOADS:
            best = None
            for attempt in range(3):                             # the first call captures the graphs
                w_prompts = prompts(batch, prompt_len)
                torch.cuda.synchronize()
                w0 = time.perf_counter()
                produced = sum(1 for _ in engine.generate(w_prompts, n_out))
                w1 = time.perf_counter()
                assert produced == n_out
                if attempt:
                    best = min(best or w1 - w0, w1 - w0)
            workloads[f"gen_{batch}x{prompt_len}x{n_out}"] = batch * n_out / best

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.sizes.upper()} layer sizes, random bf16 weights, 1 B200)",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random-init weights, seeded uniform-random token ids",
        "impl": "ours",
        "config": {
            "model": f"Qwen3-{args.sizes.upper()} layer sizes", "layers": n_layers, "layers_full": full_layers,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "tied": bool(cfg["tie_word_embeddings"]),
            "global_batch": args.batch, "seq_len": max(CONTEXT, args.prompt_len + args.steps + max(args.warmup, 3) + 1), "prompt_len": args.prompt_len,
            "context_mean": ctx_mean, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (a step reads all weights)", "graphs": backend.use_graphs,
            "peaks": peak["source"],
        },
        "e2e": {"value": e2e_decode, "unit": "tok/s", "with_prefill": e2e_total,
                "h2d_bytes_per_step": e2e_uploaded / n_new,
                "d2h_bytes_per_step": args.batch * 4,
                "note": "whole generate() call: prompts from pinned host memory, one token per sequence "
                        "read back every step; value counts the decode steps, with_prefill the whole call"},
        "gpu_launches": own_per_step * args.steps,
        "own_kernels_per_step": own_per_step,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "points": points,
        "workloads": workloads,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


# ----------------------------------------------------------------------------- the larger workloads

LARGE_WORKLOADS = {
    # sizes, batch, (shortest, longest) prompt, decode steps, temperature of every second sequence
    "8b": ("8b", 16, (64, 2048), 128, 0.0),
    "14b": ("14b", 64, (1024, 1024), 256, 0.8),
}


def run_workload(args):
    """One of the two larger workloads, prefill and decode timed on the device."""
    import torch
    from thing_htn_2026_b200 import Engine
    from thing_htn_2026_b200.config import config_from_dict
    from thing_htn_2026_b200.engine.generation import Request

    sizes, batch, (shortest, longest), steps, temperature = LARGE_WORKLOADS[args.workload]
    steps = args.steps if args.steps_given else steps
    cfg = config_json(sizes)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_layers = cfg["num_hidden_layers"]
    peak = peaks()
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(shortest, longest + 1, (batch,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    warmup = max(args.warmup, 3)
    n_new = warmup + steps + 1
    max_tokens = sum(-(-(n + n_new) // 64) * 64 for n in lens)
    engine = Engine.from_config(config_from_dict(cfg), seed=0, dtype="bfloat16", max_tokens=max_tokens, max_batch=batch)
    backend = engine.backend
    requests = [Request(p, n_new, temperature if i % 2 else 0.0, 1234, i) for i, p in enumerate(prompts)]

    def one_run(timed):
        slots = backend.open_batch(requests)
        try:
            start, mid, end = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            torch.cuda.synchronize()
            start.record()
            first = backend.launch_prefill(slots, prompts)
            mid.record()
            backend.fetch(first)
            for _ in range(warmup):
                backend.fetch(backend.launch_decode(slots))
            torch.cuda.synchronize()
            sampler = ClockSampler() if timed else None
            if sampler:
                sampler.start()
                time.sleep(0.3)
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            handles = []
            for _ in range(steps):
                handles.append(backend.launch_decode(slots))
                if len(handles) > 3:
                    backend.fetch(handles.pop(0))
            t1.record()
            torch.cuda.synchronize()
            for h in handles:
                backend.fetch(h)
            clocks = sampler.stop() if sampler else None
            return start.elapsed_time(mid), t0.elapsed_time(t1) / steps, clocks
        finally:
            backend.close_batch(slots)

    one_run(False)                                   # captures the graphs, settles the allocator
    prefill_ms, ms, clocks = one_run(True)
    numbers = model_numbers(cfg, n_layers)
    context_mean = sum(lens) / batch + warmup + (steps - 1) / 2.0
    step_bytes = numbers["weight_bytes"] + batch * context_mean * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = sum(prefill_flops(cfg, n_layers, n) for n in lens)
    line = {
        "metric": f"decode tok/s at batch {batch} (Qwen3-{sizes.upper()} layer sizes, random bf16 weights, 1 B200)",
        "value": batch * 1000.0 / ms, "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random-init weights, seeded uniform-random token ids", "impl": "ours",
        "config": {"model": f"Qwen3-{sizes.upper()} layer sizes", "workload": args.workload, "layers": n_layers,
                   "layers_full": full_layers, "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "tied": bool(cfg["tie_word_embeddings"]), "global_batch": batch, "prompt_min": min(lens),
                   "prompt_max": max(lens), "prompt_tokens": sum(lens), "context_mean": context_mean,
                   "sampled_sequences": sum(1 for r in requests if r.temperature > 0), "temperature": temperature,
                   "parallelism": "single GPU", "peaks": peak["source"]},
        "prefill": {"value": sum(lens) / (prefill_ms * 1e-3), "tokens": sum(lens), "ms": prefill_ms,
                    "frac": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


# ----------------------------------------------------------------------------- another design beside the closest model

DESIGN_SIZES = ("lanilix-w2048", "lanilix-w4096")
FP32_CORE_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12        # FFMA peak of the CUDA cores at the maximum clock


def qwen3_like(lan):
    """A Qwen3 config.json of the same width, feed-forward, heads, head size, depth and
    vocabulary as a Lanilix configuration (its attention layer's head counts)."""
    attn = next(l for l in lan["layers"] if l["type"] == "attention")
    ff = next(l["mlp"]["ff"] for l in lan["layers"] if l["mlp"])
    m = attn["mixer"]
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "attention_bias": False,
            "rope_scaling": None, "vocab_size": lan["vocab"], "hidden_size": lan["width"], "intermediate_size": ff,
            "num_hidden_layers": len(lan["layers"]), "num_attention_heads": m["heads"],
            "num_key_value_heads": m["kv_heads"], "head_dim": m["dim"], "rms_norm_eps": lan["norm"]["eps"],
            "rope_theta": 1000000.0, "tie_word_embeddings": False, "max_position_embeddings": 8192}


def measure_model(torch, engine, vocab, batch, prompt_len, steps, warmup):
    """Prefill of one PREFILL_TOKENS prompt (median of 5 after 3) and graph decode steps at
    ``batch`` after ``prompt_len``-token prompts, both on the device with CUDA events."""
    from thing_htn_2026_b200.engine.generation import Request
    from thing_htn_2026_b200.engine.step import StepEntry
    backend = engine.backend
    g = torch.Generator().manual_seed(0)
    times = []
    for _ in range(8):
        (slot,) = backend.cache.open(1)
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        backend.runner.step([StepEntry(slot, toks, (PREFILL_TOKENS - 1,))], check=False)
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
        backend.cache.close([slot])
    prefill_ms = statistics.median(times[3:])
    requests = [Request(torch.randint(0, vocab, (prompt_len,), generator=g).tolist(), warmup + steps + 1, 0.0, 0, i)
                for i in range(batch)]
    slots = backend.open_batch(requests)
    try:
        backend.fetch(backend.launch_prefill(slots, [r.tokens for r in requests]))
        for _ in range(warmup):
            backend.fetch(backend.launch_decode(slots))
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        handles = []
        for _ in range(steps):
            handles.append(backend.launch_decode(slots))
            if len(handles) > 3:
                backend.fetch(handles.pop(0))
        end.record()
        torch.cuda.synchronize()
        for handle in handles:
            backend.fetch(handle)
        decode_ms = start.elapsed_time(end) / steps
    finally:
        backend.close_batch(slots)
    return {"prefill_ms": prefill_ms, "prefill_tok_s": PREFILL_TOKENS / (prefill_ms * 1e-3),
            "decode_ms_per_step": decode_ms, "decode_tok_s": batch * 1000.0 / decode_ms}


def kernel_table(torch, lan, peak, batch, context):
    """Every kernel of the new design alone, beside the like kernel of the Qwen3 path, cold
    caches (a buffer larger than L2 is written between timed launches): microseconds, and the
    fraction of the roofline that the kernel's algorithmic bytes or flops amount to."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache, StateSpec
    dev, bf = "cuda:0", torch.bfloat16
    attn = next(l for l in lan["layers"] if l["type"] == "attention")["mixer"]
    delta = next(l for l in lan["layers"] if l["type"] == "delta")["mixer"]
    W, I = lan["width"], next(l["mlp"]["ff"] for l in lan["layers"] if l["mlp"])
    H, G, D = attn["heads"], attn["kv_heads"], attn["dim"]
    window, keep = attn["mask"]["size"], attn["mask"]["keep_first"]
    T = PREFILL_TOKENS
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hbm, tensor = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12

    def timed(fn, reps=7):
        out = []
        for _ in range(reps):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            out.append(start.elapsed_time(end) * 1e3)
        return statistics.median(out[2:])

    rows = {}

    def row(name, fn, nbytes=0, flops=0, flop_peak=None, like=None):
        us = timed(fn)
        t_roof = max(nbytes / hbm, flops / (flop_peak or tensor)) * 1e6
        rows[name] = {"us": round(us, 2), "roofline_us": round(t_roof, 2), "frac": round(t_roof / us, 3), "like": like,
                      "bound": "hbm" if nbytes / hbm >= flops / (flop_peak or tensor) else "flops"}

    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev)
    err = ops.new_error_word(dev)
    for n, tag in ((T, "prefill"), (batch, "decode")):
        # ---- norms: float32 stream with a norm on both sides of the sublayer, against add + norm in bfloat16
        h32, d16 = rnd(n, W), rnd(n, W).to(bf)
        gain = ops.Gain(rnd(W) * 0.1, 1.0, 1e-6)
        h16, w16 = rnd(n, W).to(bf), (1 + rnd(W) * 0.1).to(bf)
        row(f"{tag}: residual_norm (float32 stream, two norms)", lambda: ops.residual_norm(h32, d16, gain, gain, bf),
            nbytes=n * W * (4 + 4 + 2 + 2), like=f"{tag}: add_rmsnorm")
        row(f"{tag}: add_rmsnorm", lambda: ops.add_rmsnorm(h16, d16, w16, 1e-6), nbytes=n * W * (2 + 2 + 2 + 2))
        # ---- gated units
        gu = rnd(n, 2 * I).to(bf)
        row(f"{tag}: clamped_glu", lambda: ops.clamped_glu(gu, 7.0, 1.702), nbytes=n * I * 6, like=f"{tag}: swiglu")
        row(f"{tag}: swiglu", lambda: ops.swiglu(gu), nbytes=n * I * 6)

    # ---- attention: one sequence of T tokens, then a decode step of `batch` sequences at `context` keys
    def attention_rows(spec, general, tag_new, likes):
        n_slots = batch + 1
        cache = SequenceCache([spec], max_tokens=(batch * (context + 64) + T + 64), dtype=bf, device=dev, max_slots=n_slots + 1)
        slots = cache.open(n_slots)
        width = (H + (1 if general else 2) * G) * D
        pos = ops.RotaryTables(torch.zeros(8192, D // 4 if general else D // 2, device=dev) + 1.0,
                               torch.zeros(8192, D // 4 if general else D // 2, device=dev), D // 2 if general else D,
                               "interleaved" if general else "half")
        qg, kg = (1 + rnd(H * D) * 0.1, 1 + rnd(G * D) * 0.1) if general else ((1 + rnd(D) * 0.1).to(bf), (1 + rnd(D) * 0.1).to(bf))

        def prepare(proj, rows_):
            kv = cache.kv_view(0)
            if general:
                return ops.qk_prepare(proj, qg, kg, "projection", 1e-6, pos, rows_, kv, H, True, True, err)
            return ops.qk_norm_rope_cache(proj, qg, kg, 1e-6, pos, rows_, kv, H, True, err)

        def step_of(slot_list, counts):
            cache.prepare(slot_list, counts)
            cu = [0]
            for c in counts:
                cu.append(cu[-1] + c)
            cu_dev = torch.tensor(cu, dtype=torch.int32, device=dev)
            slots_dev = torch.tensor(slot_list, dtype=torch.int32, device=dev)
            rows_ = ops.step_rows(cu_dev, slots_dev, cache.seq_lens, cu[-1], max(counts),
                                  max_context=max(cache.length(s) + c for s, c in zip(slot_list, counts)),
                                  lengths_differ=False)
            return rows_, cu_dev, slots_dev

        # the prompt
        rows_, cu_dev, slots_dev = step_of([slots[0]], [T])
        proj = rnd(T, width).to(bf)
        size = ops.prompt_attention_tile(bf, D, cache.page_size, H, G)
        r0, rn = ops.row_tiles_of([T], [0], size)
        tiles = ops.RowTiles(torch.tensor(r0, dtype=torch.int32, device=dev), torch.tensor(rn, dtype=torch.int32, device=dev),
                             len(r0), size)
        w, k = (spec.window, spec.keep_first)
        seen = sum(min(i + 1, (w or T) + (k if w else 0)) for i in range(T))
        row(f"prefill: {tag_new[0]}", lambda: prepare(proj, rows_), nbytes=T * width * 2 + T * (H + 2 * G) * D * 2,
            like=likes[0])
        q = prepare(proj, rows_)
        row(f"prefill: {tag_new[1]}", lambda: ops.attention(q, rows_, cache.kv_view(0), H, D ** -0.5, w, err, tiles, k),
            flops=4.0 * H * D * seen, nbytes=T * H * D * 4, like=likes[1])
        # the decode step: fill `batch` sequences with `context` keys first
        others = slots[1:]
        rows_, cu_dev, slots_dev = step_of(others, [context] * batch)
        prepare(rnd(batch * context, width).to(bf), rows_)
        ops.advance(cache.seq_lens, slots_dev, cu_dev)
        cache.commit(others, [context] * batch)
        rows_, cu_dev, slots_dev = step_of(others, [1] * batch)
        proj1 = rnd(batch, width).to(bf)
        row(f"decode: {tag_new[0]}", lambda: prepare(proj1, rows_), nbytes=batch * (width * 2 + (H + 2 * G) * D * 2),
            like=likes[2])
        q1 = prepare(proj1, rows_)
        keys = min(context + 1, (w or context + 1) + (k if w else 0))
        row(f"decode: {tag_new[1]}", lambda: ops.attention(q1, rows_, cache.kv_view(0), H, D ** -0.5, w, err, None, k),
            nbytes=batch * G * keys * D * 2 * 2, like=likes[3])

    attention_rows(KVSpec(G, D, None, 0), False, ("qk_norm_rope_cache", "attention (all keys)"), (None,) * 4)
    attention_rows(KVSpec(G, D, window, keep), True, ("qk_prepare", f"attention (window {window} + {keep} kept)"),
                   ("prefill: qk_norm_rope_cache", "prefill: attention (all keys)", "decode: qk_norm_rope_cache",
                    "decode: attention (all keys)"))

    # ---- the delta rule: a prompt of T tokens, then a step of `batch` sequences
    shape = ops.DeltaShape(delta["heads"], delta["kv_heads"], delta["dim"], delta["vdim"], delta["conv"])
    Hd, dk, dv = shape.n_heads, shape.key_dim, shape.value_dim
    cache = SequenceCache([(StateSpec((Hd, dv, dk), torch.float32), StateSpec((shape.taps, shape.conv_channels), bf))],
                          max_tokens=64 * (batch + 2), dtype=bf, device=dev, max_slots=batch + 2)
    slots = cache.open(batch + 1)
    conv_w, a_log, dt_bias = rnd(shape.conv_channels, shape.taps) * 0.5, rnd(Hd) - 3.0, rnd(Hd)
    state, ring = cache.state_view(0, 0), cache.state_view(0, 1)
    for n, who, tag in ((T, [slots[0]], "prefill"), (1, slots[1:], "decode"), (T, slots[1:], f"prefill of {batch} prompts")):
        cu = torch.arange(len(who) + 1, dtype=torch.int32, device=dev) * n
        slots_dev = torch.tensor(who, dtype=torch.int32, device=dev)
        rows_ = ops.step_rows(cu, slots_dev, cache.seq_lens, n * len(who), n)
        proj = rnd(n * len(who), shape.proj_width).to(bf)
        tokens = n * len(who)
        state_bytes = len(who) * Hd * dk * dv * 4 * 2
        row(f"{tag}: delta_rule (conv, norms, recurrence)",
            lambda: ops.delta_rule(proj, conv_w, a_log, dt_bias, state, ring, rows_, cache.seq_lens, shape, 1e-6),
            nbytes=state_bytes + tokens * (shape.proj_width * 2 + Hd * dv * 4), flops=6.0 * tokens * Hd * dk * dv,
            flop_peak=FP32_CORE_TFLOPS * 1e12, like=f"{tag}: attention (all keys)" if len(tag) < 8 else None)
        if len(tag) >= 8:
            continue
        o = rnd(tokens, Hd, dv)
        wn = 1 + rnd(dv) * 0.1
        row(f"{tag}: gated_head_norm", lambda: ops.gated_head_norm(o, proj, shape.gate_offset, wn, 1e-6, Hd, dv, bf),
            nbytes=tokens * Hd * dv * (4 + 2 + 2), like=f"{tag}: add_rmsnorm")
    ops.raise_on_device_error(err, "kernel table")
    for name, r in rows.items():
        if r["like"] in rows:
            r["times_farther_than_like"] = round(rows[r["like"]]["frac"] / r["frac"], 2)
    return rows


BUNUDRA_SIZES = ("bunudra-w2048", "bunudra-w4096")


def lanilix_like(bun):
    """A Lanilix config.json of the same width, depth, vocabulary, head counts and sizes as a
    Bunudra configuration: a gated-delta-rule layer for every matrix-memory layer, a windowed
    attention (window = the chunk or window size, four kept positions) for every attention layer,
    and a dense gated feed-forward with as many weights as all experts together."""
    attn = next(l for l in bun["layers"] if l["type"] == "attention")["mixer"]
    layers = []
    for layer in bun["layers"]:
        m, mlp = layer["mixer"], layer["mlp"]
        ff = (mlp["router"]["experts"] * mlp["expert"]["ff"] + mlp["shared"]["ff"]) * 2 // 3
        if layer["type"] == "mlstm":
            mixer = {"heads": m["heads"], "kv_heads": attn["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "conv": 4}
            kind = "delta"
        else:
            mixer = {"heads": m["heads"], "kv_heads": attn["kv_heads"], "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                     "rot": {"dims": 64, "base": 1000000.0}, "mask": {"size": m["mask"]["size"], "keep_first": 4}}
            kind = "attention"
        layers.append({"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff, "limit": 7.0}})
    return {"architecture": "Lanilix", "vocab": bun["vocab"], "width": bun["width"], "norm": bun["norm"], "layers": layers}


def bunudra_kernel_table(torch, bun, peak, batch, context):
    """Every kernel of the Bunudra design alone, beside the like kernel of the Lanilix path, cold
    caches (a buffer larger than L2 is written between timed launches): microseconds, and the
    fraction of the roofline that the kernel's algorithmic bytes or flops amount to."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache, StateSpec
    dev, bf = "cuda:0", torch.bfloat16
    attn = next(l for l in bun["layers"] if l["type"] == "attention")["mixer"]
    mem = next(l for l in bun["layers"] if l["type"] == "mlstm")["mixer"]
    lat = next(l for l in bun["layers"] if l["type"] == "latent_attention")["mixer"]
    mlp = bun["layers"][0]["mlp"]
    W, T = bun["width"], PREFILL_TOKENS
    E, ff, sff, top = mlp["router"]["experts"], mlp["expert"]["ff"], mlp["shared"]["ff"], mlp["router"]["top"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hbm, tensor = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12

    def timed(fn, reps=7):
        out = []
        for _ in range(reps):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            out.append(start.elapsed_time(end) * 1e3)
        return statistics.median(out[2:])

    rows = {}

    def row(name, fn, nbytes=0, flops=0, flop_peak=None, like=None):
        us = timed(fn)
        t_roof = max(nbytes / hbm, flops / (flop_peak or tensor)) * 1e6
        rows[name] = {"us": round(us, 2), "roofline_us": round(t_roof, 2), "frac": round(t_roof / us, 3), "like": like,
                      "bound": "hbm" if nbytes / hbm >= flops / (flop_peak or tensor) else "flops"}

    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev)
    err = ops.new_error_word(dev)
    for n, tag in ((T, "prefill"), (batch, "decode")):
        # ---- norms: layer norm of the branch, add, the sum rounded; against two RMS norms around the add
        h32, d16 = rnd(n, W), rnd(n, W).to(bf)
        layer = ops.Gain(1 + rnd(W) * 0.1, 0.0, 1e-6, rnd(W) * 0.1, "layer")
        rms = ops.Gain(rnd(W) * 0.1, 1.0, 1e-6)
        row(f"{tag}: residual_norm (layer norm of the branch, add, the sum as it is)",
            lambda: ops.residual_norm(h32, d16, layer, ops.STREAM_AS_IS, bf), nbytes=n * W * (4 + 4 + 2 + 2),
            like=f"{tag}: residual_norm (two RMS norms)")
        row(f"{tag}: residual_norm (two RMS norms)", lambda: ops.residual_norm(h32, d16, rms, rms, bf),
            nbytes=n * W * (4 + 4 + 2 + 2))
        # ---- the experts' activation with the routing weights, against the clamped gated unit
        z = rnd(n, E + 1)
        routing = ops.moe_route(z, E, mlp["router"]["groups"]["count"], mlp["router"]["groups"]["keep"], top, 2.0)
        u = rnd(n, E * ff + sff).to(bf)
        gu = rnd(n, 2 * (E * ff + sff) * 2 // 3 // 2 * 2).to(bf)
        row(f"{tag}: moe_route", lambda: ops.moe_route(z, E, mlp["router"]["groups"]["count"],
                                                        mlp["router"]["groups"]["keep"], top, 2.0),
            nbytes=n * ((E + 1) * 4 + E * 4 + top * 8))
        row(f"{tag}: routed_gelu", lambda: ops.routed_gelu(u, routing, ff, sff, z, E),
            nbytes=n * ((top * ff + sff) * 2 + (E * ff + sff) * 2), like=f"{tag}: clamped_glu")
        row(f"{tag}: clamped_glu", lambda: ops.clamped_glu(gu, 7.0, 1.702), nbytes=n * gu.shape[1] * 3)
        # ---- the output gate of latent attention, against the same
        Hl, El = lat["heads"], lat["vdim"]
        a16, g16 = rnd(n, Hl * El).to(bf), rnd(n, Hl * El + 64).to(bf)
        row(f"{tag}: logistic_gate", lambda: ops.logistic_gate(a16, g16, 64), nbytes=n * Hl * El * 6, like=f"{tag}: clamped_glu")

    # ---- attention over a paged cache: one sequence of T tokens, then `batch` sequences at `context` keys
    def attention_rows(tag, spec, H, prepare_of, chunk, window, keep, likes, exact=False):
        n_slots = batch + 1
        cache = SequenceCache([spec], max_tokens=(batch * (context + 64) + T + 64), dtype=bf, device=dev, max_slots=n_slots + 1)
        slots = cache.open(n_slots)
        D, G = spec.head_dim, spec.n_kv

        def step_of(slot_list, counts):
            cache.prepare(slot_list, counts)
            cu = [0]
            for c in counts:
                cu.append(cu[-1] + c)
            cu_dev = torch.tensor(cu, dtype=torch.int32, device=dev)
            slots_dev = torch.tensor(slot_list, dtype=torch.int32, device=dev)
            rows_ = ops.step_rows(cu_dev, slots_dev, cache.seq_lens, cu[-1], max(counts),
                                  max_context=max(cache.length(s) + c for s, c in zip(slot_list, counts)),
                                  lengths_differ=False)
            return rows_, cu_dev, slots_dev

        rows_, cu_dev, slots_dev = step_of([slots[0]], [T])
        prepare, prep_bytes = prepare_of(cache, T)
        size = ops.prompt_attention_tile(bf, D, cache.page_size, H, G)
        r0, rn = ops.row_tiles_of([T], [0], size)
        tiles = ops.RowTiles(torch.tensor(r0, dtype=torch.int32, device=dev), torch.tensor(rn, dtype=torch.int32, device=dev),
                             len(r0), size)
        first = lambda i: i // chunk * chunk if chunk else max(0, i - (window or T) + 1)
        seen = sum(i - first(i) + 1 + (min(keep, first(i)) if window else 0) for i in range(T))
        row(f"prefill: {tag[0]}", lambda: prepare(rows_), nbytes=prep_bytes(T), like=likes[0])
        q = prepare(rows_)
        row(f"prefill: {tag[1]}", lambda: ops.attention(q, rows_, cache.kv_view(0), H, D ** -0.5, window, err, tiles, keep, chunk, exact),
            flops=4.0 * H * D * seen, nbytes=T * H * D * 4, like=likes[1])
        if exact:      # the same on the mma.sync kernel, which takes the weights as two bfloat16 parts
            def two_parts():
                ops.USE_TCGEN05_ATTENTION = False
                try:
                    return ops.attention(q, rows_, cache.kv_view(0), H, D ** -0.5, window, err, tiles, keep, chunk, True)
                finally:
                    ops.USE_TCGEN05_ATTENTION = True
            row(f"prefill: {tag[1]}, weights in two parts (mma.sync)", two_parts, flops=4.0 * H * D * seen,
                nbytes=T * H * D * 4, like=likes[1])
        others = slots[1:]
        rows_, cu_dev, slots_dev = step_of(others, [context] * batch)
        prepare_c, _ = prepare_of(cache, batch * context)
        prepare_c(rows_)
        ops.advance(cache.seq_lens, slots_dev, cu_dev)
        cache.commit(others, [context] * batch)
        rows_, cu_dev, slots_dev = step_of(others, [1] * batch)
        prepare_1, _ = prepare_of(cache, batch)
        row(f"decode: {tag[0]}", lambda: prepare_1(rows_), nbytes=prep_bytes(batch), like=likes[2])
        q1 = prepare_1(rows_)
        keys = context + 1 - first(context) + (min(keep, first(context)) if window else 0)
        row(f"decode: {tag[1]}", lambda: ops.attention(q1, rows_, cache.kv_view(0), H, D ** -0.5, window, err, None, keep, chunk, exact),
            nbytes=batch * G * keys * D * 2 * 2, like=likes[3])

    H, G, D = attn["heads"], attn["kv_heads"], attn["dim"]
    size = attn["mask"]["size"]
    half_tables = ops.RotaryTables(torch.ones(8192, attn["rot"]["dims"] // 2, device=dev),
                                   torch.zeros(8192, attn["rot"]["dims"] // 2, device=dev), attn["rot"]["dims"], "half")
    pair_tables = ops.RotaryTables(torch.ones(8192, D // 4, device=dev), torch.zeros(8192, D // 4, device=dev), D // 2, "interleaved")

    def head_norm_prepare(cache, n):          # Bunudra: norm per head, rotate-half on the first entries, values of their own
        proj = rnd(n, (H + 2 * G) * D).to(bf)
        qg, kg = 1 + rnd(D) * 0.1, 1 + rnd(D) * 0.1
        return (lambda rows_: ops.qk_prepare(proj, qg, kg, "head", 1e-6, half_tables, rows_, cache.kv_view(0), H, False, True, err),
                lambda m: m * ((H + 2 * G) * D * 2 + (H + 2 * G) * D * 2))

    def whole_norm_prepare(cache, n):         # Lanilix: norm over the projection, interleaved pairs, values are the keys
        proj = rnd(n, (H + G) * D).to(bf)
        qg, kg = 1 + rnd(H * D) * 0.1, 1 + rnd(G * D) * 0.1
        return (lambda rows_: ops.qk_prepare(proj, qg, kg, "projection", 1e-6, pair_tables, rows_, cache.kv_view(0), H, True, True, err),
                lambda m: m * ((H + G) * D * 2 + (H + 2 * G) * D * 2))

    lanilix_tags = ("qk_prepare (Lanilix attention)", f"attention (window {size} + 4 kept)")
    attention_rows(lanilix_tags, KVSpec(G, D, size, 4), H, whole_norm_prepare, None, size, 4, (None,) * 4)
    likes = tuple(f"{t}: {x}" for t in ("prefill", "decode") for x in lanilix_tags)
    likes = (likes[0], likes[1], likes[2], likes[3])
    attention_rows(("qk_prepare (head norm, rotate-half)", f"attention (chunks of {size})"), KVSpec(G, D, None, 0, size), H,
                   head_norm_prepare, size, None, 0, likes, exact=True)

    Hl, P, R, El, C = lat["heads"], lat["dim"], lat["rot_dim"], lat["vdim"], lat["kv_rank"]
    lat_tables = ops.RotaryTables(torch.ones(8192, R // 2, device=dev), torch.zeros(8192, R // 2, device=dev), R, "interleaved")

    def latent_prepare(cache, n):
        width = Hl * (P + R) + C + R + Hl * El
        proj = rnd(n, width).to(bf)
        up = rnd(n, Hl * (P + El)).to(bf)
        gain = 1 + rnd(C) * 0.1

        def run(rows_):
            ops.latent_norm(proj, Hl * (P + R), C, gain, 1e-6)
            return ops.latent_assemble(proj, 0, Hl * (P + R) + C, up, lat_tables, rows_, cache.kv_view(0), Hl, P, R, err)
        return run, lambda m: m * ((Hl * (P + R) + 2 * C + R + Hl * (P + El)) * 2 + (Hl * (P + R) + Hl * (P + R + El)) * 2)

    attention_rows(("latent_norm + latent_assemble", f"attention (latent heads, window {lat['mask']['size']})"),
                   KVSpec(Hl, P + R, lat["mask"]["size"], 0, None, El), Hl, latent_prepare, None, lat["mask"]["size"], 0, likes,
                   exact=True)

    # ---- the matrix memory against the delta rule: a prompt of T tokens, a step of `batch` sequences, `batch` prompts
    Hm, dk, dv = mem["heads"], mem["dim"], mem["vdim"]
    blocks = ops.mlstm_column_blocks(dv)
    cache = SequenceCache([(StateSpec((Hm, dv, dk), torch.float32), StateSpec((Hm, blocks, dk + 1), torch.float32))],
                          max_tokens=64 * (batch + 2), dtype=bf, device=dev, max_slots=batch + 2)
    slots = cache.open(batch + 1)
    bias_i, bias_f = rnd(Hm) - 2.0, rnd(Hm) + 3.0
    shape = ops.DeltaShape(Hm, attn["kv_heads"], dk, dv, 4)
    dcache = SequenceCache([(StateSpec((Hm, dv, dk), torch.float32), StateSpec((shape.taps, shape.conv_channels), bf))],
                           max_tokens=64 * (batch + 2), dtype=bf, device=dev, max_slots=batch + 2)
    dslots = dcache.open(batch + 1)
    conv_w, a_log, dt_bias = rnd(shape.conv_channels, shape.taps) * 0.5, rnd(Hm) - 3.0, rnd(Hm)
    for n, pick, tag in ((T, slice(0, 1), "prefill"), (1, slice(1, None), "decode"), (T, slice(1, None), f"prefill of {batch} prompts")):
        who, dwho = slots[pick], dslots[pick]
        cu = torch.arange(len(who) + 1, dtype=torch.int32, device=dev) * n
        tokens = n * len(who)
        rows_ = ops.step_rows(cu, torch.tensor(who, dtype=torch.int32, device=dev), cache.seq_lens, tokens, n)
        drows = ops.step_rows(cu, torch.tensor(dwho, dtype=torch.int32, device=dev), dcache.seq_lens, tokens, n)
        proj = (rnd(tokens, Hm * (2 * dk + 2 * dv)) * 0.5).to(bf)
        pre = rnd(tokens, 2 * Hm)
        dproj = rnd(tokens, shape.proj_width).to(bf)
        state_bytes = len(who) * Hm * dk * dv * 4 * 2
        row(f"{tag}: delta_rule (conv, norms, recurrence)",
            lambda: ops.delta_rule(dproj, conv_w, a_log, dt_bias, dcache.state_view(0, 0), dcache.state_view(0, 1), drows,
                                   dcache.seq_lens, shape, 1e-6),
            nbytes=state_bytes + tokens * (shape.proj_width * 2 + Hm * dv * 4), flops=6.0 * tokens * Hm * dk * dv,
            flop_peak=FP32_CORE_TFLOPS * 1e12)
        row(f"{tag}: mlstm (gates, recurrence)",
            lambda: ops.mlstm(proj, pre, bias_i, bias_f, 15.0, cache.state_view(0, 0), cache.state_view(0, 1), rows_, Hm, dk, dv,
                              dk ** -0.5),
            nbytes=state_bytes + tokens * (Hm * (2 * dk + dv) * 2 + Hm * dv * 4), flops=6.0 * tokens * Hm * dk * dv,
            flop_peak=FP32_CORE_TFLOPS * 1e12, like=f"{tag}: delta_rule (conv, norms, recurrence)")
        if len(tag) >= 8:
            continue
        o = rnd(tokens, Hm, dv)
        w_all, w_one = 1 + rnd(Hm * dv) * 0.1, 1 + rnd(dv) * 0.1
        row(f"{tag}: gated_head_norm (silu, one gain)",
            lambda: ops.gated_head_norm(o, dproj, shape.gate_offset, w_one, 1e-6, Hm, dv, bf), nbytes=tokens * Hm * dv * 8)
        row(f"{tag}: gated_head_norm (logistic, a gain over all heads)",
            lambda: ops.gated_head_norm(o, proj, Hm * (2 * dk + dv), w_all, 1e-6, Hm, dv, bf, gate_kind="logistic"),
            nbytes=tokens * Hm * dv * 8, like=f"{tag}: gated_head_norm (silu, one gain)")
    ops.raise_on_device_error(err, "kernel table")
    for name, r in rows.items():
        if r["like"] in rows:
            r["times_farther_than_like"] = round(rows[r["like"]]["frac"] / r["frac"], 2)
    return rows


DITILIX_SIZES = ("ditilix-w2048", "ditilix-w4096")


def qwen3_like_ditilix(dit):
    """A Qwen3 config.json of the same width, depth, vocabulary, heads and head size as a Ditilix
    configuration, with a gated feed-forward as wide as all experts of a routed layer together
    (the routed layers run every expert's columns as one product, so the products are equal)."""
    m = dit["layers"][0]["mixer"]
    mlp = next(l["mlp"] for l in dit["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe")
    ff = mlp["router"]["experts"] * mlp["expert"]["ff"] + (mlp.get("shared") or {}).get("ff", 0)
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "attention_bias": False,
            "rope_scaling": None, "vocab_size": dit["vocab"], "hidden_size": dit["width"], "intermediate_size": ff,
            "num_hidden_layers": len(dit["layers"]), "num_attention_heads": m["heads"],
            "num_key_value_heads": m["kv_heads"], "head_dim": m["dim"], "rms_norm_eps": dit["norm"]["eps"],
            "rope_theta": 1000000.0, "tie_word_embeddings": False, "max_position_embeddings": 8192}


def ditilix_kernel_table(torch, dit, peak, batch, context):
    """Every kernel of the Ditilix design alone, beside the like kernel of the Qwen3 path (of the
    Bunudra path for the router), cold caches (a buffer larger than L2 is written between timed
    launches): microseconds, and the fraction of the roofline that the kernel's algorithmic bytes
    or flops amount to."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache
    dev, bf = "cuda:0", torch.bfloat16
    attn = dit["layers"][0]["mixer"]
    dense = next(l["mlp"] for l in dit["layers"] if l["mlp"] and l["mlp"]["kind"] == "dense")
    mlp = next(l["mlp"] for l in dit["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe")
    W, T, V = dit["width"], PREFILL_TOKENS, dit["vocab"]
    groups, mult = dit["norm"]["groups"], dit["residual_mult"]
    E, ff, top = mlp["router"]["experts"], mlp["expert"]["ff"], mlp["router"]["top"]
    sff = (mlp.get("shared") or {}).get("ff", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hbm, tensor = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12

    def timed(fn, reps=7):
        out = []
        for _ in range(reps):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            out.append(start.elapsed_time(end) * 1e3)
        return statistics.median(out[2:])

    rows = {}

    def row(name, fn, nbytes=0, flops=0, like=None):
        us = timed(fn)
        t_roof = max(nbytes / hbm, flops / tensor) * 1e6
        rows[name] = {"us": round(us, 2), "roofline_us": round(t_roof, 3), "frac": round(t_roof / us, 5), "like": like,
                      "bound": "hbm" if nbytes / hbm >= flops / tensor else "flops"}

    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev)
    err = ops.new_error_word(dev)
    table = rnd(V, W).to(bf)
    pair = torch.arange((W + 1) // 2, dtype=torch.float64, device=dev)
    frequencies = 10000.0 ** (-2.0 * pair / W)
    for n, tag in ((T, "prefill"), (batch, "decode")):
        # ---- the rows that start the stream: float32 rows with sinusoidal positions, against bfloat16 rows as they are
        index = torch.randint(0, V, (n,), generator=g, device=dev).to(torch.int32)
        positions = torch.arange(n, dtype=torch.int32, device=dev) + context
        row(f"{tag}: gather_rows_scaled (float32 rows, sinusoidal positions)",
            lambda: ops.gather_rows_scaled(table, index, 1.0, err, positions, frequencies), nbytes=n * W * (2 + 4),
            like=f"{tag}: gather_rows")
        row(f"{tag}: gather_rows", lambda: ops.gather_rows(table, index, err), nbytes=n * W * 4)
        # ---- the one norm of a layer: both branches times a factor into the float32 stream, a norm in groups
        h32, a16, b16 = rnd(n, W), rnd(n, W).to(bf), rnd(n, W).to(bf)
        grouped = ops.Gain(1 + rnd(W) * 0.1, 0.0, 1e-6, groups=groups)
        h16, w16 = rnd(n, W).to(bf), (1 + rnd(W) * 0.1).to(bf)
        row(f"{tag}: residual_norm (two branches, a factor, {groups} groups)",
            lambda: ops.residual_norm(h32, a16, None, grouped, bf, d2=b16, mult=mult), nbytes=n * W * (4 + 4 + 2 + 2 + 2),
            like=f"{tag}: add_rmsnorm")
        row(f"{tag}: add_rmsnorm", lambda: ops.add_rmsnorm(h16, a16, w16, 1e-6), nbytes=n * W * (2 + 2 + 2 + 2))
        # ---- activations: the polynomial of norms and the routed clamped unit, against the gated unit
        z = rnd(n, dense["ff"]).to(bf)
        coefficients = torch.tensor([0.5, 0.3, 0.2, 0.1], device=dev)
        gu = rnd(n, 2 * (E * ff + sff)).to(bf)
        logits = rnd(n, E + 1)
        routing = ops.moe_route(logits, E, 1, 1, top, 1.0, scoring="logistic")
        row(f"{tag}: polynorm", lambda: ops.polynorm(z, coefficients, 1e-6), nbytes=n * dense["ff"] * 4, like=f"{tag}: swiglu")
        row(f"{tag}: routed_clamped_glu",
            lambda: ops.routed_clamped_glu(gu, routing, ff, sff, mlp["expert"]["limit"], mlp["expert"]["limit"], 1.702,
                                           logits, E),
            nbytes=n * (2 * (top * ff + sff) * 2 + (E * ff + sff) * 2), like=f"{tag}: swiglu")
        row(f"{tag}: swiglu", lambda: ops.swiglu(gu), nbytes=n * (E * ff + sff) * 6)
        row(f"{tag}: moe_route (logistic scores)", lambda: ops.moe_route(logits, E, 1, 1, top, 1.0, scoring="logistic"),
            nbytes=n * ((E + 1) * 4 + E * 4 + top * 8), like=f"{tag}: moe_route (softmax, groups)")
        row(f"{tag}: moe_route (softmax, groups)", lambda: ops.moe_route(logits, E, 4 if E % 4 == 0 else 1, 2 if E % 4 == 0 else 1, top, 2.0),
            nbytes=n * ((E + 1) * 4 + E * 4 + top * 8))

    # ---- attention over a paged cache: one sequence of T tokens, then `batch` sequences at `context` keys
    H, G, D = attn["heads"], attn["kv_heads"], attn["dim"]
    shaped = ops.ScoreShape(float(attn.get("softcap") or 0.0), float(attn["q_temp"]["coef"]), int(attn["q_temp"]["every"]))
    tables = ops.RotaryTables(torch.ones(8192, D // 2, device=dev), torch.zeros(8192, D // 2, device=dev), D, "half")
    qg, kg = (1 + rnd(D) * 0.1).to(bf), (1 + rnd(D) * 0.1).to(bf)
    width = (H + 2 * G) * D

    def attention_rows(tags, prepare_of, shape, likes):
        cache = SequenceCache([KVSpec(G, D, None, 0)], max_tokens=(batch * (context + 64) + T + 64), dtype=bf, device=dev,
                              max_slots=batch + 2)
        slots = cache.open(batch + 1)
        prepare = prepare_of(cache)

        def step_of(slot_list, counts):
            cache.prepare(slot_list, counts)
            cu = [0]
            for c in counts:
                cu.append(cu[-1] + c)
            cu_dev = torch.tensor(cu, dtype=torch.int32, device=dev)
            slots_dev = torch.tensor(slot_list, dtype=torch.int32, device=dev)
            rows_ = ops.step_rows(cu_dev, slots_dev, cache.seq_lens, cu[-1], max(counts),
                                  max_context=max(cache.length(s) + c for s, c in zip(slot_list, counts)),
                                  lengths_differ=False)
            return rows_, cu_dev, slots_dev

        rows_, cu_dev, slots_dev = step_of([slots[0]], [T])
        proj = rnd(T, width).to(bf)
        size = ops.prompt_attention_tile(bf, D, cache.page_size, H, G)
        r0, rn = ops.row_tiles_of([T], [0], size)
        tiles = ops.RowTiles(torch.tensor(r0, dtype=torch.int32, device=dev), torch.tensor(rn, dtype=torch.int32, device=dev),
                             len(r0), size)
        row(f"prefill: {tags[0]}", lambda: prepare(proj, rows_), nbytes=T * width * 4, like=likes[0])
        q = prepare(proj, rows_)
        row(f"prefill: {tags[1]}", lambda: ops.attention(q, rows_, cache.kv_view(0), H, D ** -0.5, None, err, tiles, shape=shape),
            flops=4.0 * H * D * T * (T + 1) / 2, nbytes=T * H * D * 4, like=likes[1])
        others = slots[1:]
        rows_, cu_dev, slots_dev = step_of(others, [context] * batch)
        prepare(rnd(batch * context, width).to(bf), rows_)
        ops.advance(cache.seq_lens, slots_dev, cu_dev)
        cache.commit(others, [context] * batch)
        rows_, cu_dev, slots_dev = step_of(others, [1] * batch)
        proj1 = rnd(batch, width).to(bf)
        row(f"decode: {tags[0]}", lambda: prepare(proj1, rows_), nbytes=batch * width * 4, like=likes[2])
        q1 = prepare(proj1, rows_)
        row(f"decode: {tags[1]}", lambda: ops.attention(q1, rows_, cache.kv_view(0), H, D ** -0.5, None, err, None, shape=shape),
            nbytes=batch * G * (context + 1) * D * 2 * 2, like=likes[3])

    qwen_tags = ("qk_norm_rope_cache", "attention (all keys)")
    attention_rows(qwen_tags, lambda cache: (lambda proj, rows_: ops.qk_norm_rope_cache(proj, qg, kg, 1e-6, tables, rows_,
                                                                                        cache.kv_view(0), H, True, err)),
                   ops.PLAIN_SCORES, (None,) * 4)
    attention_rows(("qk_prepare (no norm, no rotation)", "attention (all keys, score cap, query temperature)"),
                   lambda cache: (lambda proj, rows_: ops.qk_prepare(proj, None, None, None, 1.0, None, rows_, cache.kv_view(0),
                                                                     H, False, True, err)),
                   shaped, tuple(f"{t}: {x}" for t in ("prefill", "decode") for x in qwen_tags))
    ops.raise_on_device_error(err, "kernel table")
    for name, r in rows.items():
        if r["like"] in rows and r["frac"] > 0:
            r["times_farther_than_like"] = round(rows[r["like"]]["frac"] / r["frac"], 2)
    return rows


DUBAZEN_SIZES = ("dubazen-w2048", "dubazen-w4096")


def bunudra_like(dub):
    """A Bunudra config.json of the same width, depth, vocabulary, head counts and sizes as a Dubazen
    configuration: a matrix-memory layer for every layer with a recurrent state alone (gated linear
    attention, selective scan), an attention layer over all keys for every pair of softmax and linear
    attention, and the same experts (as many, as wide, as many per token, a shared one)."""
    par = next(l for l in dub["layers"] if l["type"] == "parallel")["mixer"]["left"]
    layers = []
    for layer in dub["layers"]:
        mlp = layer["mlp"]
        moe = {"kind": "moe", "expert": {"ff": mlp["expert"]["ff"]},
               "router": {"experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "scale": 1.0},
               "shared": {"ff": mlp["shared"]["ff"]}}
        if layer["type"] == "parallel":
            mixer = {"heads": par["heads"], "kv_heads": par["kv_heads"], "dim": par["dim"], "vdim": par["vdim"],
                     "scale": par["scale"], "rot": dict(par["rot"])}
            kind = "attention"
        else:
            mixer = {"heads": par["heads"], "dim": 128, "vdim": 128, "gate_cap": 15.0}
            kind = "mlstm"
        layers.append({"type": kind, "mixer": mixer, "mlp": moe})
    return {"architecture": "Bunudra", "vocab": dub["vocab"], "width": dub["width"], "embedding": dub["embedding"],
            "norm": dub["norm"], "layers": layers}


def dubazen_kernel_table(torch, dub, peak, batch, context):
    """Every kernel of the Dubazen design alone, beside the like kernel of the Bunudra path, cold
    caches (a buffer larger than L2 is written between timed launches): microseconds, and the
    fraction of the roofline that the kernel's algorithmic bytes or flops amount to."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache, StateSpec
    dev, bf = "cuda:0", torch.bfloat16
    pair = next(l for l in dub["layers"] if l["type"] == "parallel")["mixer"]
    left, right = pair["left"], pair["right"]
    gla = next(l for l in dub["layers"] if l["type"] == "gla")["mixer"]
    scan = next(l for l in dub["layers"] if l["type"] == "mamba1")["mixer"]
    mlp = dub["layers"][0]["mlp"]
    W, T, S = dub["width"], PREFILL_TOKENS, dub["streams"]
    E, ff, sff, top = mlp["router"]["experts"], mlp["expert"]["ff"], mlp["shared"]["ff"], mlp["router"]["top"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hbm, tensor = peak["hbm_gbs"] * 1e9, peak["bf16_tflops"] * 1e12
    cores = FP32_CORE_TFLOPS * 1e12

    def timed(fn, reps=7):
        out = []
        for _ in range(reps):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            out.append(start.elapsed_time(end) * 1e3)
        return statistics.median(out[2:])

    rows = {}

    def row(name, fn, nbytes=0, flops=0, flop_peak=None, like=None):
        us = timed(fn)
        t_roof = max(nbytes / hbm, flops / (flop_peak or tensor)) * 1e6
        rows[name] = {"us": round(us, 2), "roofline_us": round(t_roof, 3), "frac": round(t_roof / us, 5), "like": like,
                      "bound": "hbm" if nbytes / hbm >= flops / (flop_peak or tensor) else "flops"}

    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev)
    err = ops.new_error_word(dev)
    H, G, D, DV = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
    for n, tag in ((T, "prefill"), (batch, "decode")):
        # ---- between two sublayers: the streams' write, read and norm, against "layer norm of the branch, add, the sum"
        X, y16 = rnd(n, S * W), rnd(n, W).to(bf)
        numbers = ops.StreamNumbers(rnd(S), rnd(S, S), rnd(S))
        gain1 = torch.ones(1, device=dev)
        row(f"{tag}: hyper_norm ({S} streams: write, read, norm)",
            lambda: ops.hyper_norm(X, S, bf, y=y16, written=numbers, read=numbers.read, gain=gain1, eps=1e-6),
            nbytes=n * W * (8 * S + 2 + 2), like=f"{tag}: residual_norm (layer norm of the branch, add, the sum as it is)")
        h32 = rnd(n, W)
        layer = ops.Gain(1 + rnd(W) * 0.1, 0.0, 1e-6, rnd(W) * 0.1, "layer")
        row(f"{tag}: residual_norm (layer norm of the branch, add, the sum as it is)",
            lambda: ops.residual_norm(h32, y16, layer, ops.STREAM_AS_IS, bf), nbytes=n * W * (4 + 4 + 2 + 2))
        # ---- routing and the experts' activation
        z = rnd(n, E + 1)
        routing = ops.moe_route(z, E, 1, 1, top, 1.0, renormalise=1e-20)
        row(f"{tag}: moe_route (softmax, renormalised)", lambda: ops.moe_route(z, E, 1, 1, top, 1.0, renormalise=1e-20),
            nbytes=n * ((E + 1) * 4 + E * 4 + top * 8), like=f"{tag}: moe_route (softmax, groups)")
        row(f"{tag}: moe_route (softmax, groups)",
            lambda: ops.moe_route(z, E, 4 if E % 4 == 0 else 1, 2 if E % 4 == 0 else 1, top, 2.0),
            nbytes=n * ((E + 1) * 4 + E * 4 + top * 8))
        gu, u = rnd(n, 2 * (E * ff + sff)).to(bf), rnd(n, E * ff + sff).to(bf)
        row(f"{tag}: routed_clamped_glu (weight on the output)",
            lambda: ops.routed_clamped_glu(gu, routing, ff, sff, mlp["expert"]["limit"], mlp["shared"]["limit"], 1.702,
                                           weight_at="output"),
            nbytes=n * (2 * (top * ff + sff) * 2 + (E * ff + sff) * 2), like=f"{tag}: routed_gelu")
        row(f"{tag}: routed_gelu", lambda: ops.routed_gelu(u, routing, ff, sff, z, E),
            nbytes=n * ((top * ff + sff) * 2 + (E * ff + sff) * 2))
        # ---- the read-outs on their way to the shared output product
        a16, g16 = rnd(n, H * DV).to(bf), rnd(n, H * DV + 64).to(bf)
        positions = ops.StepRows(None, torch.arange(n, dtype=torch.int32, device=dev) + (0 if n == T else context), None, None,
                                 n, 1, 1)
        turn = ops.RotaryTables(torch.ones(8192, DV // 2, device=dev), torch.zeros(8192, DV // 2, device=dev), DV, "half")
        joint = torch.empty(n, H * DV + right["heads"] * right["vdim"], dtype=bf, device=dev)
        row(f"{tag}: rotate_gate (turned back, gated, scaled, into its columns)",
            lambda: ops.rotate_gate(a16, g16, 64, H, DV, turn, positions, err, 0.6, joint, 0), nbytes=n * H * DV * 6,
            like=f"{tag}: logistic_gate")
        row(f"{tag}: logistic_gate", lambda: ops.logistic_gate(a16, g16, 64), nbytes=n * H * DV * 6)
        Hr, Er = right["heads"], right["vdim"]
        o32, gate_r = rnd(n, Hr, Er), rnd(n, Hr * Er).to(bf)
        w_all = 1 + rnd(Hr * Er) * 0.1
        row(f"{tag}: gated_head_norm (one norm over all heads, logistic, scaled, into its columns)",
            lambda: ops.gated_head_norm(o32, gate_r, 0, w_all, 1e-6, 1, Hr * Er, bf, "logistic", 0.9, joint, H * DV),
            nbytes=n * Hr * Er * 8, like=f"{tag}: gated_head_norm (per head, logistic, a gain over all heads)")
        row(f"{tag}: gated_head_norm (per head, logistic, a gain over all heads)",
            lambda: ops.gated_head_norm(o32, gate_r, 0, w_all, 1e-6, Hr, Er, bf, gate_kind="logistic"), nbytes=n * Hr * Er * 8)

    # ---- attention over a paged cache: one sequence of T tokens, then `batch` sequences at `context` keys
    tables = ops.RotaryTables(torch.ones(8192, left["rot"]["dims"] // 2, device=dev),
                              torch.zeros(8192, left["rot"]["dims"] // 2, device=dev), left["rot"]["dims"], "half")
    turn = ops.RotaryTables(torch.ones(8192, DV // 2, device=dev), torch.zeros(8192, DV // 2, device=dev), DV, "half")
    ones, gains = torch.ones(D, device=dev), 1 + rnd(D) * 0.1
    sinks = rnd(H)
    width = (H + G) * D + G * DV

    def attention_rows(tags, prepare_of, sink, likes):
        cache = SequenceCache([KVSpec(G, D, None, 0, None, DV)], max_tokens=(batch * (context + 64) + T + 64), dtype=bf,
                              device=dev, max_slots=batch + 2)
        slots = cache.open(batch + 1)
        prepare = prepare_of(cache)

        def step_of(slot_list, counts):
            cache.prepare(slot_list, counts)
            cu = [0]
            for c in counts:
                cu.append(cu[-1] + c)
            cu_dev = torch.tensor(cu, dtype=torch.int32, device=dev)
            slots_dev = torch.tensor(slot_list, dtype=torch.int32, device=dev)
            rows_ = ops.step_rows(cu_dev, slots_dev, cache.seq_lens, cu[-1], max(counts),
                                  max_context=max(cache.length(s) + c for s, c in zip(slot_list, counts)),
                                  lengths_differ=False)
            return rows_, cu_dev, slots_dev

        rows_, cu_dev, slots_dev = step_of([slots[0]], [T])
        proj = rnd(T, width).to(bf)
        size = ops.prompt_attention_tile(bf, D, cache.page_size, H, G, DV)
        tiles = None
        if size:
            r0, rn = ops.row_tiles_of([T], [0], size)
            tiles = ops.RowTiles(torch.tensor(r0, dtype=torch.int32, device=dev), torch.tensor(rn, dtype=torch.int32, device=dev),
                                 len(r0), size)
        row(f"prefill: {tags[0]}", lambda: prepare(proj, rows_), nbytes=T * width * 4, like=likes[0])
        q = prepare(proj, rows_)
        row(f"prefill: {tags[1]}",
            lambda: ops.attention(q, rows_, cache.kv_view(0), H, left["scale"], None, err, tiles, exact_weights=True, sinks=sink),
            flops=2.0 * H * (D + DV) * T * (T + 1) / 2, nbytes=T * H * (D + DV) * 2, like=likes[1])
        others = slots[1:]
        rows_, cu_dev, slots_dev = step_of(others, [context] * batch)
        prepare(rnd(batch * context, width).to(bf), rows_)
        ops.advance(cache.seq_lens, slots_dev, cu_dev)
        cache.commit(others, [context] * batch)
        rows_, cu_dev, slots_dev = step_of(others, [1] * batch)
        proj1 = rnd(batch, width).to(bf)
        row(f"decode: {tags[0]}", lambda: prepare(proj1, rows_), nbytes=batch * width * 4, like=likes[2])
        q1 = prepare(proj1, rows_)
        row(f"decode: {tags[1]}",
            lambda: ops.attention(q1, rows_, cache.kv_view(0), H, left["scale"], None, err, None, exact_weights=True, sinks=sink),
            nbytes=batch * G * (context + 1) * (D + DV) * 2, like=likes[3])

    like_tags = ("qk_prepare (head norm, rotation)", "attention (all keys, float32 weights)")
    attention_rows(like_tags, lambda cache: (lambda proj, rows_: ops.qk_prepare(proj, gains, gains, "head", 1e-6, tables, rows_,
                                                                                cache.kv_view(0), H, False, True, err)),
                   None, (None,) * 4)
    attention_rows(("qk_prepare (head norm, rotation, values turned)", "attention (all keys, float32 weights, sinks)"),
                   lambda cache: (lambda proj, rows_: ops.qk_prepare(proj, ones, ones, "head", 1e-6, tables, rows_,
                                                                     cache.kv_view(0), H, False, True, err, value_rotary=turn)),
                   sinks, tuple(f"{t}: {x}" for t in ("prefill", "decode") for x in like_tags))

    # ---- the recurrences: one sequence of T tokens, `batch` sequences of one token
    Hg, dk, dv = gla["heads"], gla["dim"], gla["vdim"]
    inner, N, taps = scan["inner"], scan["state"], scan["conv"]
    blocks = ops.mlstm_column_blocks(dv)
    n_slots = batch + 1
    cache = SequenceCache([(StateSpec((Hg, dv, dk)), StateSpec((Hg, blocks, dk + 1))), StateSpec((Hg, dv, dk)),
                           (StateSpec((inner, N)), StateSpec((taps, inner), bf))],
                          max_tokens=n_slots * 64, dtype=bf, device=dev, max_slots=n_slots + 1)
    slots = cache.open(n_slots)
    bias_i, bias_f = rnd(Hg), rnd(Hg) + 3.0
    decay = torch.tensor([1.0 - 2.0 ** -(3 + 8 * h / max(1, Hg - 1)) for h in range(Hg)], device=dev)
    conv_w, conv_b = rnd(inner, taps) * 0.5, rnd(inner) * 0.1
    a_neg, d_skip, dt_bias = -torch.exp(rnd(inner, N) * 0.5), 1 + rnd(inner) * 0.1, rnd(inner) * 0.1
    gate_bias = rnd(Hg * dk) + 3.0
    for n, pick, tag in ((T, slice(0, 1), "prefill"), (1, slice(1, None), "decode")):
        who = slots[pick]
        cu = torch.arange(len(who) + 1, dtype=torch.int32, device=dev) * n
        tokens = n * len(who)
        rows_ = ops.step_rows(cu, torch.tensor(who, dtype=torch.int32, device=dev), cache.seq_lens, tokens, n)
        proj = (rnd(tokens, Hg * (2 * dk + 2 * dv)) * 0.5).to(bf)
        pre = rnd(tokens, 2 * Hg)
        zgate = rnd(tokens, Hg * dk)
        state_bytes = len(who) * Hg * dk * dv * 4 * 2
        io_bytes = tokens * (Hg * (2 * dk + dv) * 2 + Hg * dv * 4)
        like = f"{tag}: mlstm (gates, recurrence)"
        row(like, lambda: ops.mlstm(proj, pre, bias_i, bias_f, 15.0, cache.state_view(0, 0), cache.state_view(0, 1), rows_, Hg, dk,
                                    dv, dk ** -0.5),
            nbytes=state_bytes + io_bytes, flops=6.0 * tokens * Hg * dk * dv, flop_peak=cores)
        row(f"{tag}: linear_attention (a constant decay per head, silu'd inputs)",
            lambda: ops.linear_attention(proj, (0, Hg * dk, 2 * Hg * dk), cache.state_view(1), rows_, Hg, dk, dv, decay=decay,
                                         silu_inputs=True),
            nbytes=state_bytes + io_bytes, flops=6.0 * tokens * Hg * dk * dv, flop_peak=cores, like=like)
        row(f"{tag}: linear_attention (a gated decay per key channel)",
            lambda: ops.linear_attention(proj, (0, Hg * dk, 2 * Hg * dk), cache.state_view(1), rows_, Hg, dk, dv, gate=zgate,
                                         gate_bias=gate_bias, tau=16.0, q_scale=dk ** -0.5),
            nbytes=state_bytes + io_bytes + tokens * Hg * dk * 4, flops=6.0 * tokens * Hg * dk * dv, flop_peak=cores, like=like)
        xz = rnd(tokens, 2 * inner).to(bf)
        row(f"{tag}: causal_conv (taps, bias, silu) and its ring",
            lambda: (ops.causal_conv(xz, 0, inner, conv_w, conv_b, cache.state_view(2, 1), rows_, cache.seq_lens),
                     ops.conv_ring_update(cache.state_view(2, 1), xz, 0, rows_, cache.seq_lens)),
            nbytes=tokens * inner * 4 + len(who) * taps * inner * 4)
        xc, dt_pre, bc = rnd(tokens, inner).to(bf), rnd(tokens, inner), rnd(tokens, 2 * N).to(bf)
        row(f"{tag}: selective_scan",
            lambda: ops.selective_scan(xc, dt_pre, dt_bias, bc, a_neg, d_skip, xz, inner, cache.state_view(2, 0), rows_),
            nbytes=len(who) * inner * N * 8 + tokens * (inner * (2 + 4 + 2 + 2) + 4 * N), flops=6.0 * tokens * inner * N,
            flop_peak=cores, like=like)
    ops.raise_on_device_error(err, "kernel table")
    for name, r in rows.items():
        if r["like"] in rows and r["frac"] > 0:
            r["times_farther_than_like"] = round(rows[r["like"]]["frac"] / r["frac"], 2)
    return rows


def run_design(args):
    import torch
    from thing_htn_2026_b200 import Engine, ops
    from thing_htn_2026_b200.config import config_from_dict, named_config_json
    peak = peaks()
    warmup = max(args.warmup, 3)
    steps = args.steps if args.steps_given else 64
    sizes = {}
    sampler = ClockSampler()
    sampler.start()
    ops.launch_count = 0
    design = args.design
    design_sizes = {"lanilix": DESIGN_SIZES, "bunudra": BUNUDRA_SIZES, "ditilix": DITILIX_SIZES, "dubazen": DUBAZEN_SIZES}[design]
    for name in design_sizes:
        lan = named_config_json(name)
        if args.layers:
            lan["layers"] = lan["layers"][:args.layers]
        per_seq = -(-(args.prompt_len + warmup + steps + 2) // 64) * 64
        max_tokens = max(args.batch * per_seq, PREFILL_TOKENS + 64) + 64
        entry = {"layers": [l["type"] for l in lan["layers"]], "width": lan["width"]}
        beside = {"lanilix": lambda: ("qwen3_same_size", qwen3_like(lan)),
                  "bunudra": lambda: ("lanilix_same_size", lanilix_like(lan)),
                  "ditilix": lambda: ("qwen3_same_size", qwen3_like_ditilix(lan)),
                  "dubazen": lambda: ("bunudra_same_size", bunudra_like(lan))}[design]()
        for label, data in ((design, lan), beside):
            engine = Engine.from_config(config_from_dict(data), seed=0, dtype="bfloat16", max_tokens=max_tokens,
                                        max_batch=args.batch)
            entry[label] = measure_model(torch, engine, data.get("vocab", data.get("vocab_size")), args.batch,
                                         args.prompt_len, steps, warmup)
            del engine
            torch.cuda.empty_cache()
        table = {"lanilix": kernel_table, "bunudra": bunudra_kernel_table, "ditilix": ditilix_kernel_table,
                 "dubazen": dubazen_kernel_table}[design]
        entry["kernels"] = table(torch, lan, peak, args.batch, args.prompt_len)
        sizes[name] = entry
    clocks = sampler.stop()
    first = sizes[design_sizes[0]]
    print(json.dumps({
        "metric": f"decode tok/s at batch {args.batch} ({design.capitalize()}, {design_sizes[0]}, random bf16 weights, 1 B200)",
        "value": first[design]["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": first[design]["decode_ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random-init weights, seeded uniform-random token ids",
        "impl": "ours", "design": design,
        "config": {"model": design_sizes[0], "global_batch": args.batch, "seq_len": args.prompt_len + warmup + steps,
                   "prompt_len": args.prompt_len, "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
                   "l2": "kernel table: a 256 MB buffer is written between timed launches", "peaks": peak["source"],
                   "fp32_core_tflops": FP32_CORE_TFLOPS},
        "gpu_launches": ops.launch_count, "sizes": sizes, "clocks": clocks}))
    return 0


# ----------------------------------------------------------------------------- the reference arm

REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def run_reference(args):
    """The unmodified reference: its ``engine/`` folder as copied to ``baseline/_ref/engine``,
    built by its own ``Engine(model_path)`` on a random Qwen3-4B-size folder and driven through
    its own ``generate(input_ids, max_new_tokens)``.  Nothing of this repository's package is
    imported into this process: the folder is written by a child process."""
    engine_dir = os.path.join(REF_DIR, "engine")
    if not os.path.isfile(os.path.join(engine_dir, "engine.py")):
        return unavailable(f"no copy of the reference's engine/ folder under baseline/_ref (looked for "
                           f"{os.path.relpath(engine_dir, ROOT)}/engine.py)")
    cfg = config_json(args.sizes)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_layers = cfg["num_hidden_layers"]
    warmup = max(args.warmup, 3)
    folder = tempfile.mkdtemp(prefix="thn_reference_model_")
    try:
        made = subprocess.run(
            [sys.executable, "-m", "thing_htn_2026_b200", "random-model", "--random-config", SIZES[args.sizes],
             "--layers", str(args.layers), "--seed", "0", "--dtype", "bfloat16", "--device", "cuda:0", "--out", folder],
            cwd=ROOT, capture_output=True, text=True)
        if made.returncode != 0:
            return unavailable(f"could not write the random model folder: {made.stderr.strip()[-300:]}")
        try:
            sys.path.insert(0, engine_dir)
            import torch
            import engine as reference_engine              # baseline/_ref/engine/engine.py
            ref = reference_engine.Engine(folder)
        except Exception as error:  # noqa: BLE001 - whatever stops the reference from starting is the answer
            return unavailable(f"the reference engine did not start: {type(error).__name__}: {error}")
        return time_reference(args, ref, torch, cfg, n_layers, full_layers, warmup)
    finally:
        import shutil
        shutil.rmtree(folder, ignore_errors=True)


def time_reference(args, ref, torch, cfg, n_layers, full_layers, warmup):
    peak = peaks()
    vocab = cfg["vocab_size"]
    g = torch.Generator().manual_seed(0)

    def prompts(batch, length):
        return torch.randint(0, vocab, (batch, length), generator=g).tolist()

    def decode(batch, steps, sample_clocks=False):
        """Wall time between the yields of ``generate`` after ``warmup`` decode steps: host token
        lists in, host token lists out, as its caller sees them."""
        n_new = 1 + warmup + steps
        list(ref.generate(prompts(batch, args.prompt_len), n_new))          # its per-shape preparation and graph capture
        sampler = ClockSampler() if sample_clocks else None
        ids = prompts(batch, args.prompt_len)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        stamps = []
        for i, tokens in enumerate(ref.generate(ids, n_new)):
            stamps.append(time.perf_counter())
            if i == warmup and sampler:
                sampler.start()
        clocks = sampler.stop() if sampler else None
        assert len(stamps) == n_new and len(tokens) == batch
        seconds = stamps[-1] - stamps[warmup]
        return 1e3 * seconds / steps, 1e3 * (stamps[0] - t0), clocks, batch * n_new / (stamps[-1] - t0)

    started = time.perf_counter()
    ms, _, clocks, with_prefill = decode(args.batch, args.steps, sample_clocks=True)
    value = args.batch * 1000.0 / ms
    numbers = model_numbers(cfg, n_layers)
    ctx_mean = args.prompt_len + warmup + (args.steps - 1) / 2.0
    step_bytes = numbers["weight_bytes"] + args.batch * 2 * cfg["hidden_size"] \
        + args.batch * ctx_mean * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9

    # time to the first token of one 2,048-token prompt, by the other arm's protocol: the calls
    # are repeated for PREFILL_SETTLE_S seconds and the median of the last five counts; the median
    # of PREFILL_TIMED calls after the first PREFILL_WARM (the first of them also prepares the
    # reference's state for this shape) is kept as `ms_first`.
    times = []
    list(ref.generate(prompts(1, PREFILL_TOKENS), 2))
    settle_started = time.perf_counter()
    rep = 1
    while rep < PREFILL_WARM + PREFILL_TIMED + PREFILL_MORE or time.perf_counter() - settle_started < PREFILL_SETTLE_S:
        ids = prompts(1, PREFILL_TOKENS)
        torch.cuda.synchronize()
        profiled = args.profiler_range == "prefill" and rep == PREFILL_WARM + PREFILL_TIMED - 1
        if profiled:
            torch.cuda.profiler.start()
        t0 = time.perf_counter()
        for tokens in ref.generate(ids, 1):
            times.append(1e3 * (time.perf_counter() - t0))
        if profiled:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        rep += 1
        if args.profiler_range == "prefill" and rep >= PREFILL_WARM + PREFILL_TIMED:
            break
    first_ms = statistics.median(times[PREFILL_WARM - 1:PREFILL_WARM - 1 + PREFILL_TIMED])
    prefill_ms = statistics.median(times[-5:])
    flops = prefill_flops(cfg, n_layers, PREFILL_TOKENS)

    points = {}
    if not args.no_points:
        for batch in (1, 64):
            if time.perf_counter() - started > 420:          # each new shape costs the reference a warm-up
                break
            pms, _, _, _ = decode(batch, min(args.steps, 64))
            points[f"decode_b{batch}"] = batch * 1000.0 / pms

    # Its own public workloads (batch x prompt x new tokens), by its own definition of throughput:
    # batch * new tokens / time of the whole call, prefill included; the best of two calls after one.
    workloads = {}
    if not args.no_points:
        for batch, prompt_len, n_out in WORKLOADS:
            if time.perf_counter() - started > 600:
                break
            best = None
            for attempt in range(3):
                w_prompts = prompts(batch, prompt_len)
                torch.cuda.synchronize()
                w0 = time.perf_counter()
                produced = sum(1 for _ in ref.generate(w_prompts, n_out))
                w1 = time.perf_counter()
                assert produced == n_out
                if attempt:
                    best = min(best or w1 - w0, w1 - w0)
            workloads[f"gen_{batch}x{prompt_len}x{n_out}"] = batch * n_out / best

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.sizes.upper()} layer sizes, random bf16 weights, 1 B200)",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random-init weights, seeded uniform-random token ids",
        "impl": "reference",
        "config": {
            "model": f"Qwen3-{args.sizes.upper()} layer sizes", "layers": n_layers, "layers_full": full_layers,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "tied": bool(cfg["tie_word_embeddings"]),
            "global_batch": args.batch, "seq_len": max(CONTEXT, args.prompt_len + args.steps + warmup + 1),
            "prompt_len": args.prompt_len, "context_mean": ctx_mean, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (a step reads all weights)", "graphs": bool(getattr(ref, "use_graphs", False)),
            "peaks": peak["source"],
        },
        "e2e": {"value": value, "unit": "tok/s", "with_prefill": with_prefill,
                "h2d_bytes_per_step": args.batch * args.prompt_len * 8 / (1 + warmup + args.steps),
                "d2h_bytes_per_step": args.batch * 8,
                "note": "the reference has one public call, generate(): value and e2e are the same wall-clock "
                        "measurement between its yields (prompt ids uploaded once as int64, one int64 token per "
                        "sequence read back every step)"},
        "gpu_launches": None,
        "triton": bool(getattr(ref, "use_triton", False)),
        "ops": {name: getattr(fn, "__module__", "?").split(".")[-1] for name, fn in getattr(ref, "ops", {}).items()},
        "prefill": {"value": PREFILL_TOKENS / (prefill_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": prefill_ms,
                    "frac": flops / (prefill_ms * 1e-3) / (peak.get("bf16_tflops_sustained", peak["bf16_tflops"]) * 1e12),
                    "peak_tflops": peak.get("bf16_tflops_sustained", peak["bf16_tflops"]),
                    "frac_burst": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12),
                    "ms_first": first_ms, "steps": len(times),
                    "note": f"time to the first token of generate(), host to host; median of the last 5 of {len(times)} "
                            f"calls in a row ({PREFILL_SETTLE_S:.0f} s); ms_first: median of {PREFILL_TIMED} calls after "
                            f"{PREFILL_WARM}"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "points": points,
        "workloads": workloads,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None, help="timed decode steps (default 256)")
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--sizes", default="4b", choices=sorted(SIZES),
                        help="layer sizes of Qwen3-4B (the default run), -8B or -14B")
    parser.add_argument("--prompt-len", type=int, default=PROMPT, help="tokens of each prompt before the decode steps")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0 = all)")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    parser.add_argument("--profiler-range", choices=["decode", "prefill"], default=None,
                        help="bracket the timed decode steps, or the last prefill, with cudaProfilerStart/Stop "
                             "(for ncu --profile-from-start off)")
    parser.add_argument("--workload", choices=sorted(LARGE_WORKLOADS), default=None,
                        help="one of the two larger workloads instead of the default run")
    parser.add_argument("--design", choices=["lanilix", "bunudra", "ditilix", "dubazen"], default=None,
                        help="another design beside its closest relative at the same sizes (Lanilix beside Qwen3, "
                             "Bunudra beside Lanilix, Ditilix beside Qwen3), model by model and kernel by kernel, "
                             "instead of the default run")
    args = parser.parse_args()
    args.steps_given = args.steps is not None
    if args.steps is None:
        args.steps = 256
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.workload:
        return run_workload(args)
    if args.design:
        return run_design(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
