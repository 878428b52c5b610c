"""Decode and prefill throughput of the engine on one B200, Qwen2.5-7B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

Prints ONE JSON line.  Every decode figure is taken over the whole range the configuration names: ``batch``
requests are each prefilled with 2,048 random token ids and then decoded to a context of 4,096 (one new token per
request per step, output head and token choice included).  After W untimed steps the rest of the range is timed in
windows of exactly K steps, a CUDA event between every two windows (at least ten windows: K is capped at a tenth of
the range).  ``value`` is decoded tokens per second over all windows at the given batch (default 8), ``ms_per_step``
the same as time per step; ``windows`` gives the median, the 10th and the 90th percentile of the windows' time per
step and the rate of the windows at contexts of about 2,048, 3,072 and 4,096 (the reference's protocol: at least ten
windows, median [p10, p90], docs/performance-log.md:5).  ``points`` holds the same whole-range figure at batch 1 and
64.  ``e2e`` is the same range through ``Engine.generate`` (token ids in from the host, sampled ids back to the host
every step), timed on the host.  ``prefill`` is one whole 2,048-token prompt in one step (from its third occurrence on
the engine replays a step shape from a captured graph, as it does for decode steps; the timed repetitions are such
replays): timed first, on an idle GPU, as a burst against the burst peak, and once more at the end as the median of
20 repetitions under sustained load (``sustained_*``, against the sustained peak: the board's power cap lowers the
clocks within a few hundred milliseconds of such steps).  ``roofline`` relates the decode step to the bytes it has to read (every weight it uses once, plus the
cache of the live requests at the mean context of the timed steps).  Weights (15 GB) are larger than L2, so every
step streams them from HBM.
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT = 2048
CONTEXT = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# What the reference publishes for this model: decode by batch on one H100 at context 512 (docs/performance-log.md:239-242).
# It has no number on a B200, none at contexts of 2,048 to 4,096 by batch, and none at batch 64.
BASELINE_TOK_S = {1: 146.0, 8: 1087.0}
BASELINE_LABEL = {"gpu": "H100 80GB", "context": 512, "unit": "tokens/s", "source": "docs/performance-log.md:239-242 of the reference"}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.path = Path(tempfile.mkstemp(suffix=".csv")[1])
        self.process = None

    def start(self):
        try:
            self.process = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                                            stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.path.read_text().splitlines():
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 6:
                continue
            try:
                clocks.append(float(fields[0]))
                maxima.append(float(fields[1]))
            except ValueError:
                continue
            for name, value in zip(names, fields[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.path.unlink(missing_ok=True)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(maxima) if maxima else None,
                "reasons": sorted(reasons)}


def reference_arm() -> int:
    # The reference's runtime is Rust (helios) with CUDA kernels built for sm_80/sm_90; this image has
    # no cargo or rustc, and pip finds no Python project at the root of the reference's tree.
    print(json.dumps({"impl": "reference", "unavailable": "the reference runtime is Rust + sm_90 CUDA; no Rust toolchain in this image and pip finds no installable project at its root"}))
    return 0


def model_config(layers: int):
    from hyperion_b200.config import Qwen2Config

    return Qwen2Config(num_hidden_layers=layers, hidden_size=3584, intermediate_size=18944, num_attention_heads=28,
                       num_key_value_heads=4, head_dim=128, vocab_size=152064, max_position_embeddings=32768, rope_theta=1e6,
                       rms_norm_eps=1e-6, tie_word_embeddings=False)


def weight_bytes(c) -> int:
    q, kv = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
    per_layer = (q + 2 * kv) * c.hidden_size + (q + 2 * kv) + q * c.hidden_size + 3 * c.hidden_size * c.intermediate_size
    return 2 * (c.num_hidden_layers * per_layer + c.vocab_size * c.hidden_size) + 4 * (2 * c.num_hidden_layers + 1) * c.hidden_size


def prefill_flops(c, tokens: int) -> float:
    q, kv = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
    linear = 2.0 * tokens * ((q + 2 * kv) * c.hidden_size + q * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
    attention = 4.0 * c.num_attention_heads * c.head_dim * tokens * (tokens + 1) / 2
    return c.num_hidden_layers * (linear + attention) + 2.0 * c.hidden_size * c.vocab_size


def random_prompt(seed: int, count: int, vocab: int) -> list[int]:
    import torch

    return torch.randint(0, vocab, (count,), generator=torch.Generator().manual_seed(seed)).tolist()


def percentile(values: list[float], fraction: float) -> float:
    ordered = sorted(values)
    at = fraction * (len(ordered) - 1)
    low = int(at)
    high = min(low + 1, len(ordered) - 1)
    return ordered[low] + (ordered[high] - ordered[low]) * (at - low)


def time_decode(engine, batch: int, window: int, warmup: int, decode_tokens: int = CONTEXT - PROMPT) -> dict:
    """``batch`` requests prefilled to 2,048 tokens and decoded by ``decode_tokens`` more: W untimed steps, then windows
    of exactly ``window`` steps with a CUDA event between every two, to the end of the range."""
    import torch

    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.ops import native
    from hyperion_b200.sampling import GREEDY, pack_options

    vocab = engine.model.spec.vocab_size
    names = [f"bench{batch}_{i}" for i in range(batch)]
    for i, name in enumerate(names):
        engine.step([StepEntry(name, random_prompt(i, PROMPT, vocab), [])])
    window = max(1, min(window, (decode_tokens - warmup) // 10))
    n_windows = (decode_tokens - warmup) // window
    steps = n_windows * window
    feed = torch.randint(0, vocab, (warmup + steps, batch), generator=torch.Generator().manual_seed(1000 + batch)).tolist()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(n_windows + 1)]
    options = {"sampling_options": ([w for name in names for w in pack_options(GREEDY, 0, engine.cache.slot(name))], (batch, 8))}

    def one(s):
        logits = engine.runner.step([StepEntry(name, [feed[s][i]], [0]) for i, name in enumerate(names)], options)
        engine.sampler.sample(logits, engine.runner.last_context.extra["sampling_options"], all_greedy=True)

    for s in range(warmup):
        one(s)
    torch.cuda.synchronize()
    launches_before = native.LAUNCHES[0] + getattr(engine.runner, "graph_launches", 0)
    host_start = time.perf_counter()
    events[0].record()
    for w in range(n_windows):
        for s in range(warmup + w * window, warmup + (w + 1) * window):
            one(s)
        events[w + 1].record()
    torch.cuda.synchronize()
    host_ms = (time.perf_counter() - host_start) * 1e3
    per_window = [events[w].elapsed_time(events[w + 1]) / window for w in range(n_windows)]  # ms per step
    ms = events[0].elapsed_time(events[-1])
    launches = native.LAUNCHES[0] + getattr(engine.runner, "graph_launches", 0) - launches_before
    mean_context = PROMPT + warmup + (steps + 1) / 2
    h2d = engine.runner.packer._cursor * 4
    for name in names:
        engine.finish(name)
    engine.check()

    def rate_at(context: int) -> float:
        index = min(n_windows - 1, max(0, (context - PROMPT - warmup) // window))
        return round(batch / (per_window[index] / 1e3), 1)

    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "host_ms_per_step": host_ms / steps,
            "launches": launches, "mean_context": mean_context, "h2d_bytes": h2d, "steps": steps, "window": window,
            "windows": {"count": n_windows, "steps_each": window, "ms_per_step_median": round(statistics.median(per_window), 4),
                        "ms_per_step_p10": round(percentile(per_window, 0.1), 4), "ms_per_step_p90": round(percentile(per_window, 0.9), 4),
                        "tokens_per_s_at_context": {str(c): rate_at(c) for c in (PROMPT, (PROMPT + PROMPT + decode_tokens) // 2, PROMPT + decode_tokens)}}}


def time_prefill(engine, reps: int = 5, warmup: int = 3) -> dict:
    import torch

    from hyperion_b200.engine.batch import StepEntry

    vocab = engine.model.spec.vocab_size
    times = []
    for r in range(warmup + reps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        prompt = random_prompt(50 + r, PROMPT, vocab)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry("prefill", prompt, [PROMPT - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.finish("prefill")
        if r >= warmup:
            times.append(start.elapsed_time(stop))
    engine.check()
    return {"ms": statistics.median(times)}


def time_e2e(engine, batch: int, window: int, warmup: int, decode_tokens: int = CONTEXT - PROMPT) -> dict:
    """The same range through ``Engine.generate``: prompts go in from the host; every step copies its metadata from
    pinned memory and its sampled ids back to pinned memory, where the callback reads them (one step behind the device,
    which takes each token from the step before on the device).  Timed on the host, from the W-th token of the last
    request to its last token."""
    from hyperion_b200.sampling import SamplingParams

    vocab = engine.model.spec.vocab_size
    prompts = [random_prompt(i, PROMPT, vocab) for i in range(batch)]
    stamps: list[float] = []

    def on_token(index, token):
        if index == batch - 1:
            stamps.append(time.perf_counter())

    engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=decode_tokens, ignore_eos=True), max_batch=batch,
                    max_batch_tokens=batch * PROMPT, prefill_chunk_busy=PROMPT, on_token=on_token)
    steps = len(stamps) - 1 - warmup
    seconds = stamps[-1] - stamps[warmup]
    window = max(1, min(window, steps // 10))
    per_window = [(stamps[warmup + (w + 1) * window] - stamps[warmup + w * window]) / window * 1e3 for w in range(steps // window)]
    return {"tok_s": batch * steps / seconds, "ms_per_step": seconds / steps * 1e3, "h2d_bytes": engine.runner.packer._cursor * 4,
            "d2h_bytes": batch * 4, "steps": steps, "ms_per_step_median": round(statistics.median(per_window), 4),
            "ms_per_step_p10": round(percentile(per_window, 0.1), 4), "ms_per_step_p90": round(percentile(per_window, 0.9), 4)}


def other_workload(name: str) -> int:
    """The two larger workloads: continuous batching through ``Engine.generate`` with host tokens in and out."""
    import torch

    from hyperion_b200.api import Engine
    from hyperion_b200.config import Qwen2Config
    from hyperion_b200.sampling import SamplingParams

    if name == "mixed-1.5b":
        config = Qwen2Config(num_hidden_layers=28, hidden_size=1536, intermediate_size=8960, num_attention_heads=12, num_key_value_heads=2,
                             head_dim=128, vocab_size=151936, max_position_embeddings=32768, rope_theta=1e6, rms_norm_eps=1e-6,
                             tie_word_embeddings=True)
        lengths = torch.randint(16, 4097, (128,), generator=torch.Generator().manual_seed(0)).tolist()
        new_tokens, max_batch, budget = 256, 128, 8192
    else:
        config = Qwen2Config(num_hidden_layers=64, hidden_size=5120, intermediate_size=27648, num_attention_heads=40, num_key_value_heads=8,
                             head_dim=128, vocab_size=152064, max_position_embeddings=32768, rope_theta=1e6, rms_norm_eps=1e-6,
                             tie_word_embeddings=False)
        lengths = [4096] * 16
        new_tokens, max_batch, budget = 512, 16, 8192
    prompts = [random_prompt(i, n, config.vocab_size) for i, n in enumerate(lengths)]
    cache_tokens = sum(-(-(n + new_tokens) // 16) * 16 for n in lengths)
    engine = Engine.from_random("Qwen2ForCausalLM", config, seed=0, dtype="bfloat16", page_size=16, max_tokens=cache_tokens, max_requests=max_batch)
    params = SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True)
    engine.generate(prompts[:2], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))  # warm-up: compiles, library set-up
    torch.cuda.synchronize()
    started = time.perf_counter()
    outputs = engine.generate(prompts, params, max_batch=max_batch, max_batch_tokens=budget, prefill_chunk_busy=2048)
    seconds = time.perf_counter() - started
    generated, prompt_tokens = sum(len(o) for o in outputs), sum(lengths)
    print(json.dumps({"workload": name, "requests": len(prompts), "prompt_tokens": prompt_tokens, "generated_tokens": generated,
                      "seconds": round(seconds, 3), "generated_tokens_per_s": round(generated / seconds, 1),
                      "all_tokens_per_s": round((generated + prompt_tokens) / seconds, 1), "steps": engine.runner.steps_run,
                      "graphs": len(engine.runner.graphs), "dtype": "bf16", "data": "synthetic: random weights and token ids",
                      "layers": config.num_hidden_layers, "hidden": config.hidden_size}))
    return 0


def reference_tables() -> int:
    """The reference's own published tables at their shapes (docs/performance-log.md:369-384,197,243-244,407, measured on an
    H100): decode ms per step by batch at context 512 and prefill ms by prompt length, for the 0.5B and the 7B shape."""
    import torch

    from hyperion_b200.api import Engine
    from hyperion_b200.config import Qwen2Config
    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.sampling import GREEDY, pack_options

    shapes = {
        "0.5b": (Qwen2Config(num_hidden_layers=24, hidden_size=896, intermediate_size=4864, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
                             vocab_size=151936, max_position_embeddings=32768, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True),
                 {"decode_ms_h100": {1: 1.502, 2: 1.747, 4: 1.771, 8: 1.806, 16: 1.918, 32: 2.219}, "prefill_ms_h100": {1024: 6.2, 4096: 23.3, 8192: 59.4, 16384: 175.5}}),
        "7b": (model_config(28),
               {"decode_ms_h100": {1: 6.763, 2: 6.780, 4: 6.826, 8: 7.263, 16: 7.793, 32: 8.855}, "prefill_ms_h100": {1024: 32.85, 4096: 146.36, 8192: 343.29, 16384: 916.06}}),
    }
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, (config, published) in shapes.items():
        engine = Engine.from_random("Qwen2ForCausalLM", config, seed=0, dtype="bfloat16", page_size=16, max_tokens=32 * 640 + 17000, max_requests=32)
        vocab = config.vocab_size
        prefill = {}
        for tokens in published["prefill_ms_h100"]:
            ids = random_prompt(tokens, tokens, vocab)
            times = []
            for rep in range(5):  # the first two run directly, the third is captured, the last two are replays
                torch.cuda.synchronize()
                start.record()
                engine.step([StepEntry(f"p{tokens}_{rep}", ids, [tokens - 1])])
                stop.record()
                torch.cuda.synchronize()
                times.append(start.elapsed_time(stop))
                engine.finish(f"p{tokens}_{rep}")
            prefill[tokens] = round(min(times[3:]), 3)
        decode = {}
        for batch in published["decode_ms_h100"]:
            names = [f"d{batch}_{i}" for i in range(batch)]
            for i, request in enumerate(names):
                engine.step([StepEntry(request, random_prompt(i, 512, vocab), [])])
            options = {"sampling_options": ([w for request in names for w in pack_options(GREEDY, 0, engine.cache.slot(request))], (batch, 8))}

            def one():
                logits = engine.runner.step([StepEntry(request, [5], [0]) for request in names], options)
                engine.sampler.sample(logits, engine.runner.last_context.extra["sampling_options"], all_greedy=True)

            for _ in range(5):
                one()
            torch.cuda.synchronize()
            start.record()
            for _ in range(32):
                one()
            stop.record()
            torch.cuda.synchronize()
            decode[batch] = round(start.elapsed_time(stop) / 32, 3)
            for request in names:
                engine.finish(request)
        engine.check()
        print(json.dumps({"workload": "reference-tables", "shape": name, "dtype": "bf16", "data": "synthetic: random weights and token ids",
                          "decode_ms_per_step_at_context_512": decode, "prefill_ms": prefill, "published_h100": published}))
        del engine
        torch.cuda.empty_cache()
    return 0


NUNIVIK_SIZES = {
    # width, attention (heads, kv heads, head size, window), feed-forward, delta rule (heads, q/k heads, key size, value size),
    # state space (heads, value size, state, groups); eight layers in the order A A D S A A D S, 32,000 tokens
    "2k": {"width": 2048, "attention": (16, 4, 128, 1024), "ff": 8192, "delta": (16, 8, 128, 128), "mamba2": (64, 64, 128, 1)},
    "4k": {"width": 4096, "attention": (32, 8, 128, 1024), "ff": 14336, "delta": (32, 16, 128, 128), "mamba2": (128, 64, 128, 8)},
}


def nunivik_document(size: dict, vocab: int = 32000) -> dict:
    heads, kv_heads, dim, window = size["attention"]
    attention = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 50.0,
                                                "mask": {"size": window}, "rot": {"dims": dim, "base": 1e6, "scaling": {"factor": 1.0}}, "v_mix": True},
                 "mlp": {"kind": "dense", "ff": size["ff"]}}
    d = size["delta"]
    delta = {"type": "delta", "mixer": {"heads": d[0], "kv_heads": d[1], "dim": d[2], "vdim": d[3], "conv": 4}, "mlp": None}
    m = size["mamba2"]
    mamba = {"type": "mamba2", "mixer": {"heads": m[0], "vdim": m[1], "state": m[2], "groups": m[3], "norm_groups": m[3], "conv": 4}, "mlp": None}
    return {"architecture": "Nunivik", "vocab": vocab, "width": size["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": [attention, attention, delta, mamba, attention, attention, delta, mamba]}


def timed(fn, reps: int = 10, warmup: int = 3) -> float:
    """Median milliseconds of ``fn`` by CUDA events, L2 flushed (a 256 MB buffer written) before every timed call."""
    import torch

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    times = []
    for r in range(warmup + reps):
        flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        if r >= warmup:
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


def nunivik_kernels(size: dict, measured: dict) -> dict:
    """The design's own kernels alone at this size, a prompt of 2,048 tokens in one row and 8 rows of one decoded token: time, the bytes
    each must move and, for the scans, the float32 operations, against the measured copy bandwidth (no float32 peak is measured: the
    nominal 148 SMs x 128 lanes x 2 x 1.9 GHz = 72 TFLOP/s stands in)."""
    import torch

    from hyperion_b200 import ops
    from hyperion_b200.ops import attention as fast, recurrent

    dev = torch.device("cuda")
    hbm = measured["hbm_gbs"] * 1e9
    out: dict = {}
    width = size["width"]

    def rows_of(counts):
        starts = [0]
        for c in counts:
            starts.append(starts[-1] + c)
        token_row = torch.tensor([r for r, c in enumerate(counts) for _ in range(c)], dtype=torch.int32, device=dev)
        return torch.tensor(starts, dtype=torch.int32, device=dev), token_row, torch.arange(len(counts), dtype=torch.int32, device=dev)

    def report(name, ms, bytes_moved, flops=None):
        entry = {"us": round(ms * 1e3, 2), "bytes": int(bytes_moved), "of_measured_bandwidth": round(bytes_moved / (ms / 1e3) / hbm, 3)}
        if flops is not None:
            entry["fp32_tflops"] = round(flops / (ms / 1e3) / 1e12, 2)
        out[name] = entry

    for shape, counts in (("prefill_2048", [PROMPT]), ("decode_8", [1] * 8)):
        tokens = sum(counts)
        row_start, token_row, slots = rows_of(counts)
        h = torch.randn(tokens, width, device=dev)
        y = torch.randn(tokens, width, device=dev).to(torch.bfloat16)
        weight = torch.ones(width, device=dev)
        report(f"rmsnorm_add/{shape}", timed(lambda: ops.rmsnorm_add(h, y, weight, 1e-6, copy_dtype=torch.bfloat16)), tokens * width * (4 + 4 + 2 + 2))
        # the like kernel of the closest model: its residual add fused with the norm that reads the sum
        report(f"qwen2.add_rmsnorm/{shape}", timed(lambda: ops.add_rmsnorm(h, y, weight, 1e-6, torch.bfloat16)), tokens * width * (4 + 4 + 2 + 2))
        for kind, mode in (("delta", recurrent.MODE_DELTA), ("mamba2", recurrent.MODE_STATE_SPACE)):
            if kind == "delta":
                heads, groups, n, e = size["delta"]
                channels = 2 * groups * n + heads * e
                proj_width = channels + heads * e + 2 * heads
                k_off, q_off, v_off, col0, decay_off, step_off, gate_off = groups * n, 0, 2 * groups * n, 0, channels + heads * e + heads, channels + heads * e, channels
                group_width, gate_first = e, False
            else:
                heads, e, n, groups = size["mamba2"]
                inner = heads * e
                channels = inner + 2 * groups * n
                proj_width = inner + channels + heads
                k_off, q_off, v_off, col0, decay_off, step_off, gate_off = inner, inner + groups * n, 0, inner, inner + channels, inner + channels, 0
                group_width, gate_first = inner // groups, True
            taps = 4
            record = -(-(heads * e * n + (taps - 1) * channels) // 4) * 4
            state = torch.zeros(len(counts), record, device=dev)
            proj = torch.randn(tokens, proj_width, device=dev) * 0.5
            w_conv, a_log, dt_bias = torch.randn(channels, taps, device=dev) * 0.3, torch.zeros(heads, device=dev), torch.zeros(heads, device=dev)
            skip = torch.ones(heads, device=dev)
            conv = recurrent.causal_conv_silu(proj, col0, w_conv, None, state, heads * e * n, slots, token_row, row_start)
            report(f"{kind}.conv/{shape}", timed(lambda: recurrent.causal_conv_silu(proj, col0, w_conv, None, state, heads * e * n, slots, token_row, row_start)),
                   tokens * channels * 8)
            scan = lambda: recurrent.state_scan(mode, conv, k_off, q_off, v_off, proj, decay_off, step_off, a_log, dt_bias, skip, state, 0, slots, row_start,
                                                len(counts), heads, groups, n, n, e, q_scale=n ** -0.5)
            moved = 4 * (tokens * (2 * groups * n + 2 * heads * e + 2 * heads) + 2 * len(counts) * heads * e * n)
            report(f"{kind}.scan/{shape}", timed(scan), moved, flops=2.0 * (3 if kind == "delta" else 2) * tokens * heads * n * e)
            o = scan()
            norm_w = torch.ones(e if kind == "delta" else heads * e, device=dev)
            report(f"{kind}.gated_norm/{shape}", timed(lambda: recurrent.gated_group_norm(o, proj, gate_off, norm_w, group_width, gate_first, 1e-6, torch.bfloat16)),
                   tokens * heads * e * (4 + 4 + 2))
    return out


def nunivik_workload(args) -> int:
    """Prefill (one prompt of 2,048 tokens in one step) and decode (batch 8 from a context of 2,048) of the Nunivik design at two sizes that
    resemble real layers, beside the Qwen2 model of equal size (as many layers of the same width, heads and feed-forward), random weights."""
    import torch

    from hyperion_b200.api import Engine
    from hyperion_b200.config import NunivikConfig, Qwen2Config

    measured, kind = peaks()
    for name, size in NUNIVIK_SIZES.items():
        if args.size and name != args.size:
            continue
        heads, kv_heads, dim, _ = size["attention"]
        arms = {
            "nunivik": ("Nunivik", NunivikConfig.from_dict(nunivik_document(size))),
            "qwen2": ("Qwen2ForCausalLM", Qwen2Config(num_hidden_layers=8, hidden_size=size["width"], intermediate_size=size["ff"], num_attention_heads=heads,
                                                      num_key_value_heads=kv_heads, head_dim=dim, vocab_size=32000, max_position_embeddings=8192,
                                                      rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False)),
        }
        line = {"workload": "nunivik", "size": name, "dtype": "bf16", "data": "synthetic: random weights and token ids", "layers": "A A D S A A D S",
                "peaks": kind}
        for arm, (architecture, config) in arms.items():
            engine = Engine.from_random(architecture, config, seed=0, dtype="bfloat16", page_size=16, max_tokens=8 * (PROMPT + 256), max_requests=8)
            prefill = time_prefill(engine)
            decode = time_decode(engine, 8, 16, max(3, args.warmup), decode_tokens=max(3, args.warmup) + 160)
            line[arm] = {"prefill_ms": round(prefill["ms"], 3), "prefill_tokens_per_s": round(PROMPT / prefill["ms"] * 1e3),
                         "decode_ms_per_step": round(decode["ms_per_step"], 4), "decode_tokens_per_s": round(decode["tok_s"], 1),
                         "decode_launches_per_step": round(decode["launches"] / decode["steps"], 1)}
            del engine
            torch.cuda.empty_cache()
        line["kernels"] = nunivik_kernels(size, measured)
        print(json.dumps(line))
    return 0


MIROVIK_SIZES = {
    # width; attention beside retention (heads, kv heads, head size; retention heads, key size, value size); dense feed-forward; experts
    # (count, per token, inner width, shared inner width); selective scan (channels, state, step rank).  Four layers P+dense, P+experts,
    # S+dense, P+experts passed twice = eight layer runs, 32,000 tokens
    "2k": {"width": 2048, "left": (16, 4, 128), "right": (16, 128, 128), "ff": 8192, "experts": (16, 2, 2048, 2048), "selective": (4096, 16, 128)},
    "4k": {"width": 4096, "left": (32, 8, 128), "right": (32, 128, 128), "ff": 14336, "experts": (16, 2, 3584, 3584), "selective": (8192, 16, 256)},
}


def mirovik_document(size: dict, vocab: int = 32000) -> dict:
    heads, kv_heads, dim = size["left"]
    r_heads, r_dim, r_vdim = size["right"]
    mixer = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "bias_max": 256, "buckets": 32},
             "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": [1.0 - 2.0 ** (-5 - 5 * h / max(1, r_heads - 1)) for h in range(r_heads)],
                       "rot": {"dims": r_dim // 2, "base": 1e6}}, "left_scale": 1.0, "right_scale": 1.0}
    count, top, inner, shared = size["experts"]
    dense = {"kind": "dense", "ff": size["ff"]}
    routed = {"kind": "moe", "router": {"experts": count, "top": top}, "expert": {"ff": inner}, "shared": {"ff": shared}}
    channels, state, rank = size["selective"]
    selective = {"inner": channels, "state": state, "dt_rank": rank, "conv": 4}
    return {"architecture": "Mirovik", "vocab": vocab, "width": size["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": [{"type": "parallel", "mixer": mixer, "mlp": dense}, {"type": "parallel", "mixer": mixer, "mlp": routed},
                       {"type": "mamba1", "mixer": selective, "mlp": dense}, {"type": "parallel", "mixer": mixer, "mlp": routed}],
            "loop": {"start": 0, "stop": 4, "times": 2}}


def mirovik_kernels(size: dict, measured: dict) -> dict:
    """The design's own kernels alone at this size, a prompt of 2,048 tokens in one row and 8 rows of one decoded token: time and the bytes each
    must move against the measured copy bandwidth, for the scans also the float32 operations, for the products of the experts the
    bfloat16 operations against the measured product rate; beside each the like kernel of the closest model (Nunivik) where there is one."""
    import torch

    from hyperion_b200 import ops
    from hyperion_b200.ops import moe, recurrent

    dev = torch.device("cuda")
    hbm, peak = measured["hbm_gbs"] * 1e9, measured["bf16_tflops"] * 1e12
    out: dict = {}
    width = size["width"]

    def rows_of(counts):
        starts = [0]
        for c in counts:
            starts.append(starts[-1] + c)
        token_row = torch.tensor([r for r, c in enumerate(counts) for _ in range(c)], dtype=torch.int32, device=dev)
        return torch.tensor(starts, dtype=torch.int32, device=dev), token_row, torch.arange(len(counts), dtype=torch.int32, device=dev)

    def report(name, ms, bytes_moved, fp32_flops=None, bf16_flops=None):
        entry = {"us": round(ms * 1e3, 2), "bytes": int(bytes_moved), "of_measured_bandwidth": round(bytes_moved / (ms / 1e3) / hbm, 3)}
        if fp32_flops is not None:
            entry["fp32_tflops"] = round(fp32_flops / (ms / 1e3) / 1e12, 2)
        if bf16_flops is not None:
            entry["of_measured_bf16_rate"] = round(bf16_flops / (ms / 1e3) / peak, 3)
        out[name] = entry

    for shape, counts in (("prefill_2048", [PROMPT]), ("decode_8", [1] * 8)):
        tokens = sum(counts)
        row_start, token_row, slots = rows_of(counts)
        positions = torch.cat([torch.arange(c, dtype=torch.int32) + (0 if c > 1 else PROMPT) for c in counts]).to(dev)
        h = torch.randn(tokens, width, device=dev)
        y = torch.randn(tokens, width, device=dev).to(torch.bfloat16)
        weight = torch.ones(width, device=dev)
        report(f"norm_add_norm/{shape}", timed(lambda: ops.norm_add_norm(h, y, weight, 1e-6, None, weight, 1e-6, torch.bfloat16)), tokens * width * (4 + 4 + 2 + 2))
        report(f"nunivik.rmsnorm_add/{shape}", timed(lambda: ops.rmsnorm_add(h, y, weight, 1e-6, copy_dtype=torch.bfloat16)), tokens * width * (4 + 4 + 2 + 2))
        # retention: rotation of queries and keys in place, the scan, the gated unit norm
        heads, n, e = size["right"]
        proj = torch.randn(tokens, 2 * heads * n + 2 * heads * e, device=dev) * 0.5
        inv_freq = torch.rand(n // 4, device=dev)
        k_off, v_off, g_off = heads * n, 2 * heads * n, 2 * heads * n + heads * e
        report(f"retention.rotate/{shape}", timed(lambda: ops.heads_prepare_wide(proj, 0, k_off, v_off, heads, heads, n, e, positions, q_out=proj[:, :k_off],
                                                                              k_out=proj[:, k_off:v_off], inv_freq=inv_freq, rot_dims=n // 2, rot_half=True,
                                                                              k_scale=1.0)), tokens * 2 * heads * n * 8)
        decay = torch.full((heads,), 0.99, device=dev)
        state = torch.zeros(len(counts), heads * e * n, device=dev)
        scan = lambda: recurrent.state_scan(recurrent.MODE_RETENTION, proj, k_off, 0, v_off, proj, 0, 0, decay, decay, None, state, 0, slots, row_start,
                                            len(counts), heads, heads, n, n, e)
        report(f"retention.scan/{shape}", timed(scan), 4 * (tokens * (2 * heads * n + 2 * heads * e) + 2 * len(counts) * heads * e * n), fp32_flops=4.0 * tokens * heads * n * e)
        o = scan()
        cut = recurrent.plan_segments(counts)
        if cut is not None:  # the long row in segments side by side, as the bfloat16 engine walks it
            seg_start, seg_row = torch.tensor(cut[0], dtype=torch.int32, device=dev), torch.tensor(cut[1], dtype=torch.int32, device=dev)
            report(f"retention.scan_in_segments/{shape}", timed(lambda: recurrent.retention_in_segments(proj, k_off, 0, v_off, decay, state, slots, seg_start, seg_row,
                                                                                                         len(cut[1]), heads, n, n, e)),
                   4 * (tokens * (2 * heads * n + 2 * heads * e) + 2 * len(counts) * heads * e * n), fp32_flops=8.0 * tokens * heads * n * e)
        gated = torch.empty(tokens, heads * e, dtype=torch.bfloat16, device=dev)
        report(f"retention.gated_norm/{shape}", timed(lambda: recurrent.gated_group_norm(o, proj, g_off, None, e, False, 1e-6, torch.bfloat16, out=gated)),
               tokens * heads * e * (4 + 4 + 2))
        # the like kernel of the closest model: its state-space scan at the same state size
        ones, zeros = torch.ones(heads, device=dev), torch.zeros(heads, device=dev)
        like = lambda: recurrent.state_scan(recurrent.MODE_STATE_SPACE, proj, k_off, 0, v_off, proj, g_off, g_off, zeros, zeros, ones, state, 0, slots, row_start,
                                            len(counts), heads, heads, n, n, e)
        report(f"nunivik.state_space_scan/{shape}", timed(like), 4 * (tokens * (2 * heads * n + 2 * heads * e) + 2 * len(counts) * heads * e * n),
               fp32_flops=4.0 * tokens * heads * n * e)
        # selective scan
        channels, states, rank = size["selective"]
        x = torch.randn(tokens, channels, device=dev) * 0.5
        dt = torch.randn(tokens, channels, device=dev) - 2.0
        bc = torch.randn(tokens, rank + 2 * states, device=dev)
        gate = torch.randn(tokens, 2 * channels, device=dev)
        a = -torch.rand(channels, states, device=dev) - 0.5
        skip = torch.ones(channels, device=dev)
        s_state = torch.zeros(len(counts), channels * states, device=dev)
        report(f"selective.scan/{shape}", timed(lambda: recurrent.selective_scan(x, dt, bc, rank, rank + states, a, skip, gate, channels, s_state, 0, slots, row_start,
                                                                                 len(counts), states, states, torch.bfloat16)),
               4 * (tokens * (3 * channels + 2 * states) + 2 * len(counts) * channels * states) + 2 * tokens * channels, fp32_flops=6.0 * tokens * channels * states)
        if cut is not None:
            report(f"selective.scan_in_segments/{shape}", timed(lambda: recurrent.selective_in_segments(x, dt, bc, rank, rank + states, a, skip, gate, channels, s_state, slots,
                                                                                                         seg_start, seg_row, len(cut[1]), states, states, torch.bfloat16)),
                   4 * (tokens * (3 * channels + 2 * states) + 2 * len(counts) * channels * states) + 2 * tokens * channels, fp32_flops=12.0 * tokens * channels * states)
        w_conv, b_conv = torch.randn(channels, 4, device=dev) * 0.3, torch.zeros(channels, device=dev)
        c_state = torch.zeros(len(counts), 3 * channels, device=dev)
        report(f"selective.conv/{shape}", timed(lambda: recurrent.causal_conv_silu(gate, 0, w_conv, b_conv, c_state, 0, slots, token_row, row_start)), tokens * channels * 8)
        # routed experts: router, plan, gather, the two grouped products, the sum
        count, top, inner, _ = size["experts"]
        xb = (torch.randn(tokens, width, device=dev)).to(torch.bfloat16)
        router = torch.randn(count, width, device=dev) * 0.05
        w_gu = (torch.randn(count, 2 * inner, width, device=dev) * 0.02).to(torch.bfloat16)
        w_down = (torch.randn(count, width, inner, device=dev) * 0.02).to(torch.bfloat16)
        report(f"experts.route/{shape}", timed(lambda: moe.route(xb, router, top)), tokens * width * 2 + count * width * 4)
        chosen, weights = moe.route(xb, router, top)
        report(f"experts.plan/{shape}", timed(lambda: moe.plan(chosen, weights, count)), tokens * top * 16)
        where = moe.plan(chosen, weights, count)
        report(f"experts.gather/{shape}", timed(lambda: moe.gather(xb, where)), tokens * top * width * 4)
        rows = moe.gather(xb, where)
        used = min(count, tokens * top)  # experts whose matrices are read at all
        report(f"experts.gate_up_product/{shape}", timed(lambda: moe.grouped_linear(rows, w_gu, where)), used * 2 * inner * width * 2 + tokens * top * (width + 2 * inner) * 2,
               bf16_flops=2.0 * tokens * top * 2 * inner * width)
        act = ops.swiglu(moe.grouped_linear(rows, w_gu, where))
        report(f"experts.down_product/{shape}", timed(lambda: moe.grouped_linear(act, w_down, where)), used * inner * width * 2 + tokens * top * (width + inner) * 2,
               bf16_flops=2.0 * tokens * top * inner * width)
        z = moe.grouped_linear(act, w_down, where)
        report(f"experts.combine/{shape}", timed(lambda: moe.combine(z, where, xb, tokens)), tokens * (top + 2) * width * 2)
        # the like kernel of the closest model: one dense product of as many operations (a feed-forward's up projection over top * inner columns)
        dense_w = (torch.randn(top * 2 * inner, width, device=dev) * 0.02).to(torch.bfloat16)
        report(f"nunivik.dense_product/{shape}", timed(lambda: ops.linear(xb, dense_w, None, torch.bfloat16)), top * 2 * inner * width * 2 + tokens * (width + top * 2 * inner) * 2,
               bf16_flops=2.0 * tokens * top * 2 * inner * width)
    return out


def mirovik_workload(args) -> int:
    """Prefill (one prompt of 2,048 tokens in one step) and decode (batch 8 from a context of 2,048) of the Mirovik design at two sizes that
    resemble real layers, beside the closest model of the package, Nunivik, at equal width, heads, feed-forward and number of layer runs;
    random weights."""
    import torch

    from hyperion_b200.api import Engine
    from hyperion_b200.config import MirovikConfig, NunivikConfig

    measured, kind = peaks()
    for name, size in MIROVIK_SIZES.items():
        if args.size and name != args.size:
            continue
        arms = {"mirovik": ("Mirovik", MirovikConfig.from_dict(mirovik_document(size))),
                "nunivik": ("Nunivik", NunivikConfig.from_dict(nunivik_document(NUNIVIK_SIZES[name])))}
        line = {"workload": "mirovik", "size": name, "dtype": "bf16", "data": "synthetic: random weights and token ids",
                "layers": "(P+dense P+experts S+dense P+experts) x 2 beside A A D S A A D S", "peaks": kind}
        for arm, (architecture, config) in arms.items():
            engine = Engine.from_random(architecture, config, seed=0, dtype="bfloat16", page_size=16, max_tokens=8 * (PROMPT + 256), max_requests=8)
            prefill = time_prefill(engine)
            decode = time_decode(engine, 8, 16, max(3, args.warmup), decode_tokens=max(3, args.warmup) + 160)
            line[arm] = {"prefill_ms": round(prefill["ms"], 3), "prefill_tokens_per_s": round(PROMPT / prefill["ms"] * 1e3),
                         "decode_ms_per_step": round(decode["ms_per_step"], 4), "decode_tokens_per_s": round(decode["tok_s"], 1),
                         "decode_launches_per_step": round(decode["launches"] / decode["steps"], 1)}
            del engine
            torch.cuda.empty_cache()
        line["kernels"] = mirovik_kernels(size, measured)
        print(json.dumps(line))
    return 0


KUDAZEN_SIZES = {
    # width; chunked attention (heads, kv heads, head size, chunk); attention over latents (heads, plain size, rotated size, value size, latent,
    # query latent); time mixing (heads, head size); feed-forward.  Eight layers A L L W A L L W with tensors of their own, 32,000 tokens
    "2k": {"width": 2048, "attention": (16, 4, 128, 1024), "latent": (16, 128, 64, 128, 512, 1536), "wkv": (32, 64), "ff": 8192},
    "4k": {"width": 4096, "attention": (32, 8, 128, 2048), "latent": (32, 128, 64, 128, 512, 1536), "wkv": (64, 64), "ff": 14336},
}


def kudazen_document(size: dict, vocab: int = 32000) -> dict:
    heads, kv_heads, dim, chunk = size["attention"]
    mlp = {"kind": "dense", "ff": size["ff"], "limit": 7.0}
    attention = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": chunk}}, "mlp": mlp}
    l = size["latent"]
    latent = {"type": "latent_attention", "mixer": {"heads": l[0], "dim": l[1], "rot_dim": l[2], "vdim": l[3], "kv_rank": l[4], "q_rank": l[5],
                                                    "scale": (l[1] + l[2]) ** -0.5, "rot": {"dims": l[2], "base": 1e6}}, "mlp": mlp}
    w = size["wkv"]
    wkv = {"type": "wkv", "mixer": {"heads": w[0], "dim": w[1], "decay_rank": 64}, "mlp": mlp}
    return {"architecture": "Kudazen", "vocab": vocab, "width": size["width"], "norm": {"eps": 1e-6, "groups": 4},
            "layers": [attention, latent, latent, wkv, attention, latent, latent, wkv]}


def kudazen_kernels(size: dict, measured: dict) -> dict:
    """The design's own kernels alone at this size, a prompt of 2,048 tokens in one row and 8 rows of one decoded token behind 2,048: time, the
    bytes each must move against the measured copy bandwidth, for attention the bfloat16 operations against the measured product rate, for
    the scan the float32 operations; beside each the like kernel of the closest model (Qwen2; for the scan, the package's retention)."""
    import types

    import torch

    from hyperion_b200 import ops
    from hyperion_b200.ops import attention as fast, recurrent

    dev = torch.device("cuda")
    hbm, peak = measured["hbm_gbs"] * 1e9, measured["bf16_tflops"] * 1e12
    out: dict = {}
    width, page = size["width"], 16

    def report(name, ms, bytes_moved, fp32_flops=None, bf16_flops=None):
        entry = {"us": round(ms * 1e3, 2), "bytes": int(bytes_moved), "of_measured_bandwidth": round(bytes_moved / (ms / 1e3) / hbm, 3)}
        if fp32_flops is not None:
            entry["fp32_tflops"] = round(fp32_flops / (ms / 1e3) / 1e12, 2)
        if bf16_flops is not None:
            entry["of_measured_bf16_rate"] = round(bf16_flops / (ms / 1e3) / peak, 3)
        out[name] = entry

    for shape, counts, before in (("prefill_2048", [PROMPT], 0), ("decode_8", [1] * 8, PROMPT)):
        tokens, rows = sum(counts), len(counts)
        starts = [0]
        for c in counts:
            starts.append(starts[-1] + c)
        row_start = torch.tensor(starts, dtype=torch.int32, device=dev)
        token_row = torch.tensor([r for r, c in enumerate(counts) for _ in range(c)], dtype=torch.int32, device=dev)
        slots = torch.arange(rows, dtype=torch.int32, device=dev)
        positions = torch.cat([torch.arange(c, dtype=torch.int32) + before for c in counts]).to(dev)
        context = before + max(counts)
        per_row = -(-context // page)
        table = torch.arange(rows * per_row, dtype=torch.int32, device=dev).view(rows, per_row)
        # the stream's norm and the feed-forward's activation
        h = torch.randn(tokens, width, device=dev)
        a, b = (torch.randn(tokens, width, device=dev).to(torch.bfloat16) for _ in range(2))
        weight = torch.ones(width, device=dev)
        report(f"add_group_rmsnorm/{shape}", timed(lambda: ops.add_group_rmsnorm(h, a, b, weight, 4, 1e-6, torch.bfloat16)), tokens * width * (4 + 4 + 2 + 2 + 2))
        report(f"qwen2.add_rmsnorm/{shape}", timed(lambda: ops.add_rmsnorm(h, a, weight, 1e-6, torch.bfloat16)), tokens * width * (4 + 4 + 2 + 2))
        gu = torch.randn(tokens, 2 * size["ff"], device=dev).to(torch.bfloat16)
        report(f"clamped_glu/{shape}", timed(lambda: ops.clamped_glu(gu, 7.0, 1.702)), tokens * size["ff"] * 6)
        report(f"qwen2.swiglu/{shape}", timed(lambda: ops.swiglu(gu)), tokens * size["ff"] * 6)
        # chunked attention with slopes in the tensor-core kernels, beside the same kernels as Qwen2 calls them (no chunk, no table)
        heads, kv_heads, dim, chunk = size["attention"]
        proj = torch.randn(tokens, (heads + 2 * kv_heads) * dim, device=dev)
        cache = (torch.randn(rows * per_row, 2, kv_heads, page, dim, device=dev) * 0.5).to(torch.bfloat16)
        q = torch.empty(tokens, heads * dim, dtype=torch.bfloat16, device=dev)
        temp = torch.ones(heads, device=dev)
        report(f"attention.prepare/{shape}", timed(lambda: ops.heads_prepare_wide(proj, 0, heads * dim, (heads + kv_heads) * dim, heads, kv_heads, dim, dim, positions, q_out=q,
                                                                               cache=cache, block_table=table, token_row=token_row, page_size=page, v_unit_eps=1e-6,
                                                                               q_head_scale=temp)), tokens * (heads + 2 * kv_heads) * dim * 6)
        slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / heads) for i in range(heads)], device=dev)
        by_distance = (-(slopes[:, None] * torch.arange(chunk, device=dev)[None, :]) * 1.4426950408889634).contiguous()
        attn = torch.empty(tokens, heads * dim, dtype=torch.bfloat16, device=dev)
        fake_rows = [types.SimpleNamespace(count=c, position=before) for c in counts]
        tile = fast.tile_rows(dim, page)
        tiles, items = fast.plan(fake_rows, fast.tile_tokens(heads, kv_heads, tile))
        seen_chunked = sum(min(p % chunk + 1, p + 1) for p in positions.tolist())
        seen_all = sum(p + 1 for p in positions.tolist())
        per_position = (-slopes * 1.4426950408889634).contiguous()
        for label, window, bias, seen in (("attention.chunked_sloped", -chunk, by_distance, seen_chunked), ("qwen2.attention", 0, None, seen_all)):
            if len(tiles):
                t_dev = torch.tensor(tiles, dtype=torch.int32, device=dev)
                run = lambda: fast.attention_tiles(q, heads, cache, table, token_row, positions, t_dev, len(tiles) // 3, dim ** -0.5, window, attn, tile_size=tile, bias=bias,
                                                   bias_per_position=per_position if bias is not None else None)
            else:
                i_dev = torch.tensor(items, dtype=torch.int32, device=dev)
                splits = fast.choose_splits(len(items), heads, kv_heads, min(context, chunk + fast.KEY_TILE) if window else context)
                space = torch.empty(len(items) * heads * max(splits, 1) * (dim + 2), dtype=torch.float32, device=dev)
                run = lambda: fast.attention_tokens(q, heads, cache, table, token_row, positions, i_dev, len(items), splits, dim ** -0.5, window, attn, workspace=space, bias=bias)
            keys_read = rows * min(context, chunk if window else context) * 2 * kv_heads * dim * 2
            report(f"{label}/{shape}", timed(run), keys_read + tokens * heads * dim * 4, bf16_flops=4.0 * seen * heads * dim)
        # attention over latents: the records, the queries, attention itself (one key/value head of kv_rank + rot_dim entries for all heads)
        l_heads, l_dim, l_rot, l_vdim, rank, q_rank = size["latent"]
        record = rank + l_rot
        down = torch.randn(tokens, q_rank + record, device=dev)
        l_cache = (torch.randn(rows * per_row, 1, page, record, device=dev) * 0.3).to(torch.bfloat16)
        ones_q, ones_kv = torch.ones(q_rank, device=dev), torch.ones(rank, device=dev)
        inv_freq = torch.rand(l_rot // 2, device=dev)
        report(f"latent.prepare/{shape}", timed(lambda: ops.latent_prepare(down, 0, q_rank, q_rank, rank, l_rot, ones_q, ones_kv, 1e-6, inv_freq, l_rot, positions, torch.bfloat16,
                                                                          l_cache, table, token_row, page)), tokens * (q_rank + record) * 6)
        uq = torch.randn(tokens, l_heads * (l_dim + l_rot), device=dev).to(torch.bfloat16)
        q_lat = torch.randn(l_heads, tokens, rank, device=dev)
        report(f"latent.query/{shape}", timed(lambda: ops.latent_query(uq, q_lat, l_heads, l_dim, l_rot, inv_freq, l_rot, positions)),
               tokens * l_heads * (rank * 4 + l_rot * 2 + record * 2))
        query = ops.latent_query(uq, q_lat, l_heads, l_dim, l_rot, inv_freq, l_rot, positions)
        sinks = torch.zeros(l_heads, device=dev)
        latent_flops = 2.0 * seen_all * l_heads * (record + rank)
        latent_bytes = rows * context * record * 2 + tokens * l_heads * (record + rank) * 2
        l_shape = fast.choose_latent_shape(rows, max(counts), l_heads, context)
        l_out = torch.empty(tokens, l_heads * rank, dtype=torch.bfloat16, device=dev)
        l_space = torch.empty(tokens * l_heads * l_shape[1] * (rank + 2), dtype=torch.float32, device=dev)
        report(f"latent.attention/{shape}", timed(lambda: fast.attention_latent(query, l_heads, record, rank, l_cache, table, row_start, positions, rows, max(counts),
                                                                              context, record ** -0.5, sinks=sinks, out=l_out, workspace=l_space, shape=l_shape), reps=5),
               latent_bytes, bf16_flops=latent_flops)
        report(f"latent.attention_float_lanes/{shape}", timed(lambda: ops.attention_general(query, l_heads, 1, record, rank, l_cache, table, token_row, positions, page,
                                                                                          record ** -0.5, sinks=sinks, value_prefix=True), reps=3),
               latent_bytes, bf16_flops=latent_flops)
        # time mixing: the five mixes, the scan, the gated unit norm; beside the scan, the package's retention at the same sizes
        w_heads, n = size["wkv"]
        x = torch.randn(tokens, width, device=dev).to(torch.bfloat16)
        mu = torch.rand(5, width, device=dev)
        state = torch.zeros(rows, w_heads * n * n + width, device=dev)
        report(f"wkv.shift_mix/{shape}", timed(lambda: recurrent.token_shift_mix(x, mu, state, w_heads * n * n, slots, token_row, row_start)), tokens * width * 12)
        k, r, v, d = (torch.randn(tokens, w_heads * n, device=dev) * 0.5 for _ in range(4))
        w0, bonus = torch.full((w_heads * n,), -3.0, device=dev), torch.rand(w_heads * n, device=dev)
        scan = lambda: recurrent.wkv_scan(k, r, v, d, 0, w0, bonus, state, 0, slots, row_start, rows, w_heads, n, n, n)
        moved = 4 * (tokens * 5 * w_heads * n + 2 * rows * w_heads * n * n)
        report(f"wkv.scan/{shape}", timed(scan), moved, fp32_flops=5.0 * tokens * w_heads * n * n)
        o = scan()
        report(f"wkv.gated_norm/{shape}", timed(lambda: recurrent.gated_group_norm(o, d, 0, w0, n, False, 1e-6, torch.bfloat16)), tokens * w_heads * n * (4 + 4 + 2))
        kqv = torch.cat([k, r, v], dim=1).contiguous()
        decay = torch.full((w_heads,), 0.99, device=dev)
        like = lambda: recurrent.state_scan(recurrent.MODE_RETENTION, kqv, 0, w_heads * n, 2 * w_heads * n, kqv, 0, 0, decay, decay, None, state, 0, slots, row_start,
                                            rows, w_heads, w_heads, n, n, n)
        report(f"mirovik.retention_scan/{shape}", timed(like), 4 * (tokens * 4 * w_heads * n + 2 * rows * w_heads * n * n), fp32_flops=4.0 * tokens * w_heads * n * n)
    return out


def kudazen_workload(args) -> int:
    """Prefill (one prompt of 2,048 tokens in one step) and decode (batch 8 from a context of 2,048) of the Kudazen design at two sizes that
    resemble real layers, beside the closest model of the package, Qwen2, at equal width, heads, feed-forward and number of layers;
    random weights."""
    import torch

    from hyperion_b200.api import Engine
    from hyperion_b200.config import KudazenConfig, Qwen2Config

    measured, kind = peaks()
    for name, size in KUDAZEN_SIZES.items():
        if args.size and name != args.size:
            continue
        heads, kv_heads, dim, _ = size["attention"]
        arms = {
            "kudazen": ("Kudazen", KudazenConfig.from_dict(kudazen_document(size))),
            "qwen2": ("Qwen2ForCausalLM", Qwen2Config(num_hidden_layers=8, hidden_size=size["width"], intermediate_size=size["ff"], num_attention_heads=heads,
                                                      num_key_value_heads=kv_heads, head_dim=dim, vocab_size=32000, max_position_embeddings=8192,
                                                      rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False)),
        }
        line = {"workload": "kudazen", "size": name, "dtype": "bf16", "data": "synthetic: random weights and token ids", "layers": "A L L W A L L W",
                "peaks": kind}
        for arm, (architecture, config) in arms.items():
            engine = Engine.from_random(architecture, config, seed=0, dtype="bfloat16", page_size=16, max_tokens=8 * (PROMPT + 256), max_requests=8)
            prefill = time_prefill(engine)
            decode = time_decode(engine, 8, 16, max(3, args.warmup), decode_tokens=max(3, args.warmup) + 160)
            line[arm] = {"prefill_ms": round(prefill["ms"], 3), "prefill_tokens_per_s": round(PROMPT / prefill["ms"] * 1e3),
                         "decode_ms_per_step": round(decode["ms_per_step"], 4), "decode_tokens_per_s": round(decode["tok_s"], 1),
                         "decode_launches_per_step": round(decode["launches"] / decode["steps"], 1)}
            del engine
            torch.cuda.empty_cache()
        line["kernels"] = kudazen_kernels(size, measured)
        print(json.dumps(line))
    return 0


TOBADRA_SIZES = {
    # width; window attention (heads, kv heads, head size, window, rotated entries of queries and keys); lightning (heads, key size, value
    # size); delta rule with a decay per key channel (heads, key size, value size, inner size of decay and gate); dense feed-forward; experts
    # (count, identities, per token, inner width, shared inner width, groups, groups kept).  Eight layer runs A+dense A+experts L+experts
    # D+experts A+experts A+experts L+experts D+experts, the last with the tensors of the fourth; 32,000 tokens
    "2k": {"width": 2048, "attention": (16, 4, 128, 1024, 64), "lightning": (16, 128, 128), "delta": (16, 128, 128, 64), "ff": 8192,
           "experts": (16, 2, 2, 2048, 2048, 6, 4)},
    "4k": {"width": 4096, "attention": (32, 8, 128, 2048, 64), "lightning": (32, 128, 128), "delta": (32, 128, 128, 64), "ff": 14336,
           "experts": (16, 2, 2, 3584, 3584, 6, 4)},
}


def tobadra_document(size: dict, vocab: int = 32000) -> dict:
    heads, kv_heads, dim, window, rot = size["attention"]
    count, identity, top, inner, shared, groups, keep = size["experts"]
    experts = {"kind": "moe", "expert": {"ff": inner}, "router": {"experts": count, "top": top, "scale": 2.5, "identity": identity, "groups": {"count": groups, "keep": keep}},
               "shared": {"ff": shared}}
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": window}, "rot": {"dims": rot, "base": 1e6}}
    l_heads, l_dim, l_vdim = size["lightning"]
    lightning = {"heads": l_heads, "dim": l_dim, "vdim": l_vdim, "decay": [1.0 - 2.0 ** (-5 - 3 * i / l_heads) for i in range(l_heads)]}
    d_heads, d_dim, d_vdim, rank = size["delta"]
    delta = {"heads": d_heads, "kv_heads": d_heads, "dim": d_dim, "vdim": d_vdim, "conv": 4, "decay_rank": rank, "gate_rank": rank}
    layers = [{"type": "attention", "mixer": attention, "mlp": {"kind": "dense", "ff": size["ff"]}}, {"type": "attention", "mixer": attention, "mlp": experts},
              {"type": "lightning", "mixer": lightning, "mlp": experts}, {"type": "channel_delta", "mixer": delta, "mlp": experts},
              {"type": "attention", "mixer": attention, "mlp": experts}, {"type": "attention", "mixer": attention, "mlp": experts},
              {"type": "lightning", "mixer": lightning, "mlp": experts}, {"type": "channel_delta", "mixer": delta, "mlp": experts, "weights_of": 3}]
    return {"architecture": "Tobadra", "vocab": vocab, "width": size["width"], "norm": {"eps": 1e-6}, "canon": {"taps": 4}, "logit_scale": 1.0, "layers": layers}


def tobadra_kernels(size: dict, measured: dict) -> dict:
    """The design's own kernels alone at this size, a prompt of 2,048 tokens in one row and 8 rows of one decoded token behind 2,048: time, the
    bytes each must move against the measured copy bandwidth, for the scans the float32 operations; beside each the like kernel of the
    closest models (Mirovik's router, sum and retention; Nunivik's delta rule and convolution)."""
    import torch

    from hyperion_b200 import ops
    from hyperion_b200.ops import moe, recurrent

    dev = torch.device("cuda")
    hbm = measured["hbm_gbs"] * 1e9
    out: dict = {}
    width = size["width"]

    def report(name, ms, bytes_moved, fp32_flops=None):
        entry = {"us": round(ms * 1e3, 2), "bytes": int(bytes_moved), "of_measured_bandwidth": round(bytes_moved / (ms / 1e3) / hbm, 3)}
        if fp32_flops is not None:
            entry["fp32_tflops"] = round(fp32_flops / (ms / 1e3) / 1e12, 2)
        out[name] = entry

    for shape, counts, before in (("prefill_2048", [PROMPT], 0), ("decode_8", [1] * 8, PROMPT)):
        tokens, rows = sum(counts), len(counts)
        starts = [0]
        for c in counts:
            starts.append(starts[-1] + c)
        row_start = torch.tensor(starts, dtype=torch.int32, device=dev)
        token_row = torch.tensor([r for r, c in enumerate(counts) for _ in range(c)], dtype=torch.int32, device=dev)
        slots = torch.arange(rows, dtype=torch.int32, device=dev)
        positions = torch.cat([torch.arange(c, dtype=torch.int32) + before for c in counts]).to(dev)
        # the convolution every mixer reads through, its state, and the gate on a sublayer's result
        x = torch.randn(tokens, width, device=dev).to(torch.bfloat16)
        w_canon = torch.randn(width, 4, device=dev) * 0.3
        kept = torch.zeros(rows, 3 * width, device=dev)
        report(f"residual_conv/{shape}", timed(lambda: recurrent.residual_conv(x, w_canon, kept, 0, slots, token_row, row_start)), tokens * width * 4)
        report(f"conv_state_keep/{shape}", timed(lambda: recurrent.conv_state_keep(x, 4, kept, 0, slots, row_start, rows)), rows * 3 * width * 6)
        wide = torch.randn(tokens, width, device=dev)
        report(f"nunivik.conv_silu/{shape}", timed(lambda: recurrent.causal_conv_silu(wide, 0, w_canon, None, kept, 0, slots, token_row, row_start)), tokens * width * 8)
        gate = torch.randn(tokens, width, device=dev)
        y = torch.randn(tokens, width, device=dev).to(torch.bfloat16)
        report(f"sigmoid_gate/{shape}", timed(lambda: ops.sigmoid_gate_(y, gate, 0)), tokens * width * 8)
        # the values' rotation and the result's rotation back, beside the rotation of queries and keys with the cache write
        heads, kv_heads, dim, _, rot = size["attention"]
        proj = torch.randn(tokens, (heads + 2 * kv_heads) * dim, device=dev)
        freq_v, freq_qk = torch.rand(dim // 2, device=dev), torch.rand(rot // 2, device=dev)
        page, context = 16, before + max(counts)
        per_row = -(-context // page)
        table = torch.arange(rows * per_row, dtype=torch.int32, device=dev).view(rows, per_row)
        cache = torch.zeros(rows * per_row, 2, kv_heads, page, dim, dtype=torch.bfloat16, device=dev)
        q = torch.empty(tokens, heads * dim, dtype=torch.bfloat16, device=dev)
        prepare = lambda turned: ops.heads_prepare_wide(proj, 0, heads * dim, (heads + kv_heads) * dim, heads, kv_heads, dim, dim, positions, q_out=q, inv_freq=freq_qk, rot_dims=rot,
                                                        rot_half=True, cache=cache, block_table=table, token_row=token_row, page_size=page,
                                                        v_inv_freq=freq_v if turned else None, v_rot_dims=dim if turned else 0, v_rot_half=True)
        report(f"attention.prepare_with_turned_values/{shape}", timed(lambda: prepare(True)), tokens * (heads + 2 * kv_heads) * dim * 6)
        report(f"mirovik.attention_prepare/{shape}", timed(lambda: prepare(False)), tokens * (heads + 2 * kv_heads) * dim * 6)
        attn = torch.randn(tokens, heads * dim, device=dev).to(torch.bfloat16)
        report(f"rotate_result_back/{shape}", timed(lambda: ops.rotate_heads_(attn, 0, heads, dim, positions, freq_v, dim, True, -1.0)), tokens * heads * dim * 4)
        # the two recurrences and their gated norms; the like kernels: the delta rule with one decay per head, the same scan as retention
        d_heads, n, e, rank = size["delta"]
        conv = torch.randn(tokens, 2 * d_heads * n + d_heads * e, device=dev) * 0.5
        decay_in, step_in = torch.randn(tokens, d_heads * n, device=dev), torch.randn(tokens, 2 * d_heads, device=dev)
        a_log, dt_bias, dt_head = torch.zeros(d_heads, device=dev), torch.zeros(d_heads * n, device=dev), torch.zeros(d_heads, device=dev)
        state = torch.zeros(rows, d_heads * e * n, device=dev)
        scan_bytes = 4 * (tokens * (3 * d_heads * n + 2 * d_heads * e) + 2 * rows * d_heads * e * n)
        report(f"channel_delta.scan/{shape}", timed(lambda: recurrent.channel_delta_scan(conv, d_heads * n, 0, 2 * d_heads * n, decay_in, step_in, 0, a_log, dt_bias, state, 0, slots,
                                                                                      row_start, rows, d_heads, d_heads, n, n, e, q_scale=n ** -0.5)),
               scan_bytes, fp32_flops=7.0 * tokens * d_heads * n * e)
        report(f"nunivik.delta_scan/{shape}", timed(lambda: recurrent.state_scan(recurrent.MODE_DELTA, conv, d_heads * n, 0, 2 * d_heads * n, step_in, d_heads, 0, a_log, dt_head, None,
                                                                              state, 0, slots, row_start, rows, d_heads, d_heads, n, n, e, q_scale=n ** -0.5)),
               scan_bytes - 4 * tokens * d_heads * n, fp32_flops=6.0 * tokens * d_heads * n * e)
        o = torch.randn(tokens, d_heads * e, device=dev)
        g_in = torch.randn(tokens, d_heads * e, device=dev)
        norm_head, norm_all = torch.ones(e, device=dev), torch.ones(d_heads * e, device=dev)
        report(f"channel_delta.gated_norm/{shape}", timed(lambda: recurrent.gated_group_norm(o, g_in, 0, norm_head, e, False, 1e-6, torch.bfloat16, sigmoid_gate=True)),
               tokens * d_heads * e * 10)
        l_heads, ln, le = size["lightning"]
        qkv = torch.randn(tokens, 2 * l_heads * ln + 2 * l_heads * le, device=dev)
        report(f"lightning.silu/{shape}", timed(lambda: recurrent.silu_columns_(qkv, 0, 2 * l_heads * ln + l_heads * le)), tokens * (2 * l_heads * ln + l_heads * le) * 8)
        l_decay = torch.full((l_heads,), 0.99, device=dev)
        l_state = torch.zeros(rows, l_heads * le * ln, device=dev)
        l_bytes = 4 * (tokens * (2 * l_heads * ln + 2 * l_heads * le) + 2 * rows * l_heads * le * ln)
        report(f"lightning.scan/{shape}", timed(lambda: recurrent.state_scan(recurrent.MODE_RETENTION, qkv, l_heads * ln, 0, 2 * l_heads * ln, qkv, 0, 0, l_decay, l_decay, None, l_state, 0,
                                                                          slots, row_start, rows, l_heads, l_heads, ln, ln, le)), l_bytes, fp32_flops=4.0 * tokens * l_heads * ln * le)
        cut = recurrent.plan_segments(counts)
        if cut is not None:  # the long row in segments side by side, as the bfloat16 engine walks it
            seg_start, seg_row = torch.tensor(cut[0], dtype=torch.int32, device=dev), torch.tensor(cut[1], dtype=torch.int32, device=dev)
            report(f"lightning.scan_in_segments/{shape}", timed(lambda: recurrent.retention_in_segments(qkv, l_heads * ln, 0, 2 * l_heads * ln, l_decay, l_state, slots, seg_start, seg_row,
                                                                                                         len(cut[1]), l_heads, ln, ln, le)), l_bytes,
                   fp32_flops=8.0 * tokens * l_heads * ln * le)
        lo = torch.randn(tokens, l_heads * le, device=dev)
        report(f"lightning.gated_norm_over_all_heads/{shape}", timed(lambda: recurrent.gated_group_norm(lo, qkv, 2 * l_heads * ln + l_heads * le, norm_all[: l_heads * le], l_heads * le, False,
                                                                                                     1e-6, torch.bfloat16, sigmoid_gate=True)), tokens * l_heads * le * 10)
        report(f"mirovik.gated_norm_per_head/{shape}", timed(lambda: recurrent.gated_group_norm(lo, qkv, 2 * l_heads * ln + l_heads * le, None, le, False, 1e-6, torch.bfloat16)),
               tokens * l_heads * le * 10)
        # experts: the router with scores, correction and groups, the plan, the activation, the weighted sum; beside Mirovik's router and sum
        count, identity, top, inner, _, groups, keep = size["experts"]
        outputs = count + identity
        router, correction = torch.randn(outputs, width, device=dev) * 0.05, torch.randn(outputs, device=dev) * 0.05
        report(f"experts.route_scored/{shape}", timed(lambda: moe.route_scored(x, router, correction, top, groups, keep, 2.5)), tokens * width * 2 + outputs * width * 4)
        report(f"mirovik.route/{shape}", timed(lambda: moe.route(x, router[:count].contiguous(), top)), tokens * width * 2 + count * width * 4)
        chosen, weights = moe.route_scored(x, router, correction, top, groups, keep, 2.5)
        where = moe.plan(chosen, None, count)
        up = torch.randn(where.capacity, inner, device=dev).to(torch.bfloat16)
        report(f"experts.gelu_erf/{shape}", timed(lambda: ops.gelu_erf(up)), where.capacity * inner * 4)
        report(f"mirovik.gelu_tanh/{shape}", timed(lambda: ops.gelu_tanh(up)), where.capacity * inner * 4)
        z = torch.randn(where.capacity, width, device=dev).to(torch.bfloat16)
        base, base_gate = torch.randn(tokens, width, device=dev).to(torch.bfloat16), torch.randn(tokens, device=dev)
        report(f"experts.combine_weighted/{shape}", timed(lambda: moe.combine_weighted(z, where, weights, x, base, base_gate)), tokens * (top + 3) * width * 2)
        plain_where = moe.plan(chosen.clamp(max=count - 1), weights, count)
        report(f"mirovik.combine/{shape}", timed(lambda: moe.combine(z, plain_where, base, tokens)), tokens * (top + 2) * width * 2)
    return out


def tobadra_workload(args) -> int:
    """Prefill (one prompt of 2,048 tokens in one step) and decode (batch 8 from a context of 2,048) of the Tobadra design at two sizes that
    resemble real layers, beside the closest model of the package, Mirovik (sublayers normalised on both sides, experts, a constant-decay
    recurrence), at equal width and number of layer runs; random weights."""
    import torch

    from hyperion_b200.api import Engine
    from hyperion_b200.config import MirovikConfig, TobadraConfig

    measured, kind = peaks()
    for name, size in TOBADRA_SIZES.items():
        if args.size and name != args.size:
            continue
        arms = {"tobadra": ("Tobadra", TobadraConfig.from_dict(tobadra_document(size))),
                "mirovik": ("Mirovik", MirovikConfig.from_dict(mirovik_document(MIROVIK_SIZES[name])))}
        line = {"workload": "tobadra", "size": name, "dtype": "bf16", "data": "synthetic: random weights and token ids",
                "layers": "A+dense A+experts L+experts D+experts A+experts A+experts L+experts D+experts beside (P+dense P+experts S+dense P+experts) x 2", "peaks": kind}
        for arm, (architecture, config) in arms.items():
            engine = Engine.from_random(architecture, config, seed=0, dtype="bfloat16", page_size=16, max_tokens=8 * (PROMPT + 256), max_requests=8)
            prefill = time_prefill(engine)
            decode = time_decode(engine, 8, 16, max(3, args.warmup), decode_tokens=max(3, args.warmup) + 160)
            line[arm] = {"prefill_ms": round(prefill["ms"], 3), "prefill_tokens_per_s": round(PROMPT / prefill["ms"] * 1e3),
                         "decode_ms_per_step": round(decode["ms_per_step"], 4), "decode_tokens_per_s": round(decode["tok_s"], 1),
                         "decode_launches_per_step": round(decode["launches"] / decode["steps"], 1)}
            del engine
            torch.cuda.empty_cache()
        if not args.skip_points:
            line["kernels"] = tobadra_kernels(size, measured)
        print(json.dumps(line), flush=True)
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128, help="decode steps per timed window (at most a tenth of the range, so that there are ten windows)")
    parser.add_argument("--warmup", type=int, default=8, help="untimed decode steps before the first window (at least 3)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=28, help="fewer than the configuration's 28 only to save memory or time")
    parser.add_argument("--decode-tokens", type=int, default=CONTEXT - PROMPT,
                        help="tokens decoded after the 2,048-token prompts (the configuration's range is 2,048, to context 4,096); fewer only for profiling")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--skip-points", action="store_true", help="leave out the batch 1 / 64 points, prefill and e2e")
    parser.add_argument("--only", default=None, choices=["prefill"], help="time one part alone (for profiling)")
    parser.add_argument("--workload", default=None, choices=["mixed-1.5b", "batch-32b", "reference-tables", "nunivik", "mirovik", "kudazen", "tobadra"],
                        help="one of the other workloads instead: 128 requests with prompts of 16..4096 tokens and 256 decoded tokens "
                             "each through generate() at the 1.5B shape; batch 16 with prompts of 4,096 and 512 decoded tokens at the 32B shape; "
                             "or the reference's own published tables (decode by batch at context 512, prefill by length) at the 0.5B and 7B shapes; "
                             "or the Nunivik design at two layer sizes beside the Qwen2 model of equal size, with its own kernels timed alone; "
                             "or the Mirovik design at two layer sizes beside the Nunivik model of equal size, likewise")
    parser.add_argument("--size", default=None, choices=["2k", "4k"], help="with --workload nunivik, mirovik, kudazen or tobadra: one of its sizes only")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.workload == "reference-tables":
        return reference_tables()
    if args.workload == "nunivik":
        return nunivik_workload(args)
    if args.workload == "mirovik":
        return mirovik_workload(args)
    if args.workload == "kudazen":
        return kudazen_workload(args)
    if args.workload == "tobadra":
        return tobadra_workload(args)
    if args.workload:
        return other_workload(args.workload)
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print("bench.py: this engine runs on one GPU; --gpus > 1 is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    args.steps = max(1, args.steps)
    decode_tokens = max(args.warmup + 10, min(args.decode_tokens, CONTEXT - PROMPT))

    import torch

    from hyperion_b200.api import Engine

    measured, source = peaks()
    config = model_config(args.layers)
    largest = args.batch if args.skip_points else max(args.batch, 64)
    tokens_needed = largest * (PROMPT + decode_tokens + 16) + PROMPT + 16
    engine = Engine.from_random("Qwen2ForCausalLM", config, seed=0, dtype="bfloat16", page_size=16,
                                max_tokens=tokens_needed, max_requests=max(largest, 8))
    if args.only == "prefill":  # for profiling: the prefill step alone
        prefill = time_prefill(engine, reps=max(1, args.steps), warmup=args.warmup)
        print(json.dumps({"only": "prefill", "layers": args.layers, "tokens": PROMPT, "ms": round(prefill["ms"], 3),
                          "tokens_per_s": round(PROMPT / (prefill["ms"] / 1e3), 1)}))
        return 0
    # The prompt step first, on a GPU that has been idle: a burst of eight 22 ms steps, set against the burst peak. Under
    # sustained load the board's power cap lowers the clocks within a few hundred milliseconds; that figure is taken at
    # the end, after the decode runs, and set against the sustained peak.
    prefill = None if args.skip_points else time_prefill(engine)
    clocks = ClockSampler()
    clocks.start()
    main_run = time_decode(engine, args.batch, args.steps, args.warmup, decode_tokens)
    clock_record = clocks.stop()

    def roofline(run: dict, batch: int) -> dict:
        bytes_per_step = weight_bytes(config) + batch * run["mean_context"] * engine.cache.bytes_per_token()
        achieved = bytes_per_step / (run["ms_per_step"] / 1e3) / 1e9
        return {"bound": "hbm", "achieved": round(achieved, 1), "peak": measured["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / measured["hbm_gbs"], 4), "of": source, "mean_context": round(run["mean_context"], 1)}

    record = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen2.5-7B)",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": main_run["window"], "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        # the only published number there is: another GPU and a shorter context (see "baseline"), so a ratio across hardware
        "vs_baseline": round(main_run["tok_s"] / BASELINE_TOK_S[args.batch], 3) if args.batch in BASELINE_TOK_S else None,
        "baseline": {**BASELINE_LABEL, "value": BASELINE_TOK_S.get(args.batch)},
        "dtype": "bf16", "data": "synthetic: seeded random weights (N(0, 0.02)) and uniform random token ids",
        "impl": "ours",
        "config": {"model": "Qwen2.5-7B shape", "layers": args.layers, "layers_of_config": 28, "hidden": config.hidden_size,
                   "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                   "intermediate": config.intermediate_size, "vocab": config.vocab_size, "global_batch": args.batch,
                   "seq_len": PROMPT + decode_tokens, "prompt_len": PROMPT, "decoded_tokens_per_request": decode_tokens,
                   "timed_steps": main_run["steps"], "page_size": 16, "parallelism": "single GPU",
                   "l2": "weights (15 GB) exceed L2; every step streams them", "peaks": source},
        "windows": main_run["windows"],
        "clocks": clock_record,
        "gpu_launches": main_run["launches"],
        "host_ms_per_step": round(main_run["host_ms_per_step"], 4),
        "roofline": roofline(main_run, args.batch),
    }
    if not args.skip_points:
        flops = prefill_flops(config, PROMPT)
        record["prefill"] = {"value": round(PROMPT / (prefill["ms"] / 1e3), 1), "tokens": PROMPT, "ms": round(prefill["ms"], 3),
                             "frac": round(flops / (prefill["ms"] / 1e3) / (measured["bf16_tflops"] * 1e12), 4), "of": source,
                             "regime": "burst: median of 5 replays after 3 warm-ups on an idle GPU, against the burst peak"}
        record["points"], record["points_detail"] = {}, {}
        for batch in (1, 64):
            run = time_decode(engine, batch, args.steps, args.warmup, decode_tokens)
            record["points"][f"decode_b{batch}"] = round(run["tok_s"], 1)
            record["points_detail"][f"decode_b{batch}"] = {"ms_per_step": round(run["ms_per_step"], 4), "timed_steps": run["steps"], "windows": run["windows"],
                                                           "roofline_frac": roofline(run, batch)["frac"]}
        sustained = time_prefill(engine, reps=20, warmup=10)  # the GPU has been under load for a while by now
        sustained_peak = measured.get("bf16_tflops_sustained", measured["bf16_tflops"])
        record["prefill"].update({"sustained_ms": round(sustained["ms"], 3), "sustained_value": round(PROMPT / (sustained["ms"] / 1e3), 1),
                                  "sustained_frac": round(flops / (sustained["ms"] / 1e3) / (sustained_peak * 1e12), 4)})
        e2e = time_e2e(engine, args.batch, args.steps, args.warmup, decode_tokens)
        record["e2e"] = {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d_bytes"],
                         "d2h_bytes_per_step": e2e["d2h_bytes"], "ms_per_step": round(e2e["ms_per_step"], 4), "timed_steps": e2e["steps"],
                         "ms_per_step_median": e2e["ms_per_step_median"], "ms_per_step_p10": e2e["ms_per_step_p10"],
                         "ms_per_step_p90": e2e["ms_per_step_p90"], "clock": "host"}
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
