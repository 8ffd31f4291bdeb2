"""Decode and prefill throughput of the engine at Qwen3-1.7B size with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  ``value`` is decoded tokens per second at batch 8 and the context
length below, timed on the device over exactly K decode steps through the step function;
``e2e`` is the same through the engine loop a user drives (host token ids in, sampled token
ids out, every step).  ``prefill`` times one 2,048-token prompt, ``roofline`` relates the
decode step to the memory bandwidth, ``points`` adds batch 1 and 64.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

# Qwen3-1.7B layer sizes.
MODEL = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=2048, intermediate_size=6144,
             num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8, head_dim=128, vocab_size=151936,
             max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, attention_dropout=0.0,
             hidden_act="silu", attention_bias=False, tie_word_embeddings=True)
# Other sizes of the same architecture, for runs beside the default one (--shape).
SHAPES = {
    "1.7b": {},
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, tie_word_embeddings=False),
    "32b": dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                num_key_value_heads=8, tie_word_embeddings=False),
}
CONTEXT = 4096           # tokens each request holds at the end of the timed decode steps
PREFILL_TOKENS = 2048
PAGE_SIZE = 64           # tokens per cache page (one TMA box per page and key tile in the prompt attention)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = REPO / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            flat = {}

            def walk(node):
                if isinstance(node, dict):
                    for key, value in node.items():
                        if isinstance(value, (int, float)):
                            flat.setdefault(key, float(value))
                        else:
                            walk(value)
            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return flat, "measured"
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs (reads only)."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self.process = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.process = None
        return self

    def _read(self) -> None:
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *exc) -> None:
        if self.process is not None:
            self.process.terminate()

    def summary(self) -> dict:
        clocks = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        maxima = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({name for s in self.samples for name, flag in zip(names, s[2:]) if flag.lower().startswith("active")})
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": max(maxima) if maxima else None,
                "reasons": reasons, "samples": len(self.samples)}


def reference_arm(args) -> int:
    """MiniServe itself, unmodified, from ``baseline/_ref`` (see ``baseline/reference_arm.py``): the same
    metric (decoded tokens per second at the same batch, context and model sizes), timed over the same
    number of steps around its own ``EngineCore.step_multi``.  Its steps return token ids to the host,
    so its device-timed and end-to-end numbers are one and the same."""
    sys.path.insert(0, str(REPO / "baseline"))
    import reference_arm as arm

    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "MiniServe runs on one GPU only"}))
        return 0
    warmup = max(args.warmup, 3)
    if args.steps < 1 or args.steps + warmup + 16 > CONTEXT:
        print(f"bench.py: --steps {args.steps} does not fit the context of {CONTEXT} tokens (or is not positive)")
        return 2
    steps = min(args.steps, 64)
    result = arm.main(dict(MODEL), args.batch, CONTEXT, steps, warmup, PAGE_SIZE)
    if "unavailable" in result:
        print(json.dumps(result))
        return 0
    line = {
        "metric": f"Qwen3-{args.shape.upper()} bf16 decode tok/s @ batch {args.batch} (context {CONTEXT}); "
                  f"prefill tok/s @ {PREFILL_TOKENS:,} tokens",
        "impl": "reference", "value": result["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": result["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded uniform token ids, random weights)",
        "config": {"model": "Qwen3-1.7B shape", "layers": MODEL["num_hidden_layers"], "hidden": MODEL["hidden_size"],
                   "global_batch": args.batch, "seq_len": CONTEXT, "context_len": CONTEXT, "page_size": PAGE_SIZE,
                   "parallelism": "single GPU", "decode_execution": "cuda_graph (batched)",
                   "attention_backend": "cuda_paged", "rmsnorm_backend": "cuda"},
        "e2e": {"value": result["value"], "unit": "tokens/s", "ms_per_step": result["ms_per_step"]},
        "prefill_seconds_total": result["prefill_seconds_total"],
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    global CONTEXT, PREFILL_TOKENS
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"],
                        help="fewer layers than the model has (named in the output); for quick checks only")
    parser.add_argument("--skip-points", action="store_true")
    parser.add_argument("--timeline", metavar="FILE", default=None,
                        help="with --profile: replay the decode step as a graph (or run the prompt step) under the "
                             "framework profiler and write every kernel's start, duration and exposed time to FILE")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="1.7b",
                        help="layer sizes of another model of the family (the default is the benchmark's)")
    parser.add_argument("--context", type=int, default=CONTEXT, help="tokens a request holds at the end of the timed steps")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                        help="tokens of the timed prompt step (the benchmark's is 2,048; others for profiles)")
    parser.add_argument("--profile", choices=("decode", "prefill"), default=None,
                        help="run only a few eager steps of one phase and exit (a small case for ncu; times nothing)")
    args = parser.parse_args()
    CONTEXT = args.context
    PREFILL_TOKENS = args.prefill_tokens
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)

    import torch

    import miniserve_b200  # noqa: F401
    from miniserve_b200 import kernels
    from miniserve_b200.config import EngineConfig
    from miniserve_b200.engine.llm import build_engine
    from miniserve_b200.engine.runtime import build_runtime
    from miniserve_b200.engine.step import StepEntry
    from miniserve_b200.sampling import SamplingParams

    shape = dict(MODEL, **SHAPES[args.shape])
    if args.layers == MODEL["num_hidden_layers"]:
        args.layers = shape["num_hidden_layers"]
    config = dict(shape, num_hidden_layers=args.layers)
    max_batch = args.batch if args.skip_points else max(args.batch, 64)
    pages = max(max_batch * ((CONTEXT + PAGE_SIZE - 1) // PAGE_SIZE), PREFILL_TOKENS // PAGE_SIZE) + 64
    runtime = build_runtime(None, EngineConfig(
        dtype="bfloat16", max_model_len=max(CONTEXT, PREFILL_TOKENS), max_num_seqs=max_batch, kv_block_size=PAGE_SIZE, num_kv_blocks=pages,
        max_num_batched_tokens=max(8192, PREFILL_TOKENS), enable_prefix_cache=False,
        decode_execution="eager" if args.profile and not args.timeline else "cuda_graph"),
        config_dict=config, weights_seed=0)
    manager, step_function = runtime.manager, runtime.step_function
    vocab = config["vocab_size"]
    generator = torch.Generator().manual_seed(1)

    def prompt(n: int) -> list[int]:
        return torch.randint(0, vocab, (n,), generator=generator).tolist()

    def event_time(fn, repeats: int = 1) -> float:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(repeats):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / 1e3

    def fill(batch: int, length: int) -> list[str]:
        """Admits ``batch`` requests and prefills ``length`` tokens each through the step function."""
        ids = [f"b{batch}-{i}" for i in range(batch)]
        for rid in ids:
            manager.admit(rid)
            runtime.storage.reset_slot(manager.requests[rid].slot, 0.0, 1.0, 0, 0)
            done = 0
            while done < length:
                take = min(2048, length - done)
                entries = [StepEntry(rid, prompt(take), [])]
                reservation = manager.prepare([(rid, take)])
                step_function.run(entries, reservation)
                manager.commit(reservation)
                done += take
        torch.cuda.synchronize()
        return ids

    def decode_steps(ids: list[str], count: int) -> None:
        tokens = [1] * len(ids)
        for _ in range(count):
            entries = [StepEntry(rid, [tokens[i]], [0]) for i, rid in enumerate(ids)]
            reservation = manager.prepare([(rid, 1) for rid in ids])
            step_function.run(entries, reservation, [0] * len(ids))
            manager.commit(reservation)

    def measure_decode(batch: int, steps: int) -> tuple[float, float, int]:
        """(seconds per step, mean live context over the timed steps, kernel launches per step)."""
        ids = fill(batch, CONTEXT - steps - warmup)
        decode_steps(ids, warmup)
        before = manager.length(ids[0])
        seconds = event_time(lambda: decode_steps(ids, steps)) / steps
        mean_context = (before + manager.length(ids[0]) + 1) / 2
        launches = step_function.graphs[next(b for b in sorted(step_function.graphs) if b >= batch)].kernel_launches
        for rid in ids:
            manager.release(rid)
        return seconds, mean_context, launches

    if args.profile and args.timeline:
        # The step under the framework's profiler (CUPTI): kernels of a replayed graph keep their programmatic
        # overlap, so "exposed" (how far a kernel's end lies past the end of everything before it) is what
        # the kernel adds to the step.
        from torch.profiler import ProfilerActivity, profile
        ids = [f"p{i}" for i in range(args.batch)]

        def one_step() -> None:
            if args.profile == "decode":
                entries = [StepEntry(rid, [1], [0]) for rid in ids]
                reservation = manager.prepare([(rid, 1) for rid in ids])
                step_function.run(entries, reservation, [0] * len(ids))
                manager.abort(reservation)                       # the context stays as long as it was
            else:
                manager.admit("p")
                reservation = manager.prepare([("p", PREFILL_TOKENS)])
                step_function.run([StepEntry("p", prefill_tokens, [PREFILL_TOKENS - 1])], reservation)
                manager.commit(reservation)
                manager.release("p")

        prefill_tokens = prompt(PREFILL_TOKENS)
        if args.profile == "decode":
            for rid in ids:
                manager.admit(rid)
                manager.commit(manager.prepare([(rid, CONTEXT - 1)]))
        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as profiler:
            one_step()
            torch.cuda.synchronize()
        trace_file = args.timeline + ".trace.json"
        profiler.export_chrome_trace(trace_file)
        with open(trace_file) as handle:
            events = [e for e in json.load(handle)["traceEvents"] if e.get("cat") in ("kernel", "gpu_memcpy")]
        os.remove(trace_file)
        events.sort(key=lambda e: e["ts"])
        origin = next((e["ts"] for e in events if e.get("cat") == "kernel"), events[0]["ts"])   # the first kernel
        reached = origin
        totals: dict[str, list[float]] = {}
        lines = [f"{'start us':>10} {'duration':>9} {'exposed':>8}  grid          kernel"]
        for event in events:
            end = event["ts"] + event["dur"]
            exposed = max(0.0, end - max(reached, event["ts"]))
            name = event["name"].split("(")[0].replace("void ", "")[:70]
            lines.append(f"{event['ts'] - origin:10.2f} {event['dur']:9.2f} {exposed:8.2f}  "
                         f"{str(event['args'].get('grid', '')):13s} {name}")
            entry = totals.setdefault(name, [0, 0.0, 0.0])
            entry[0] += 1
            entry[1] += event["dur"]
            entry[2] += exposed
            reached = max(reached, end)
        summary = [f"{'launches':>8} {'duration us':>12} {'exposed us':>11}  kernel"]
        for name, (count, duration, exposed) in sorted(totals.items(), key=lambda kv: -kv[1][2]):
            summary.append(f"{count:8d} {duration:12.2f} {exposed:11.2f}  {name}")
        with open(args.timeline, "w") as handle:
            handle.write(f"step: {args.profile}, batch {args.batch}, layers {args.layers}, context {CONTEXT}, "
                         f"span {reached - origin:.2f} us\n\n" + "\n".join(summary) + "\n\n" + "\n".join(lines) + "\n")
        print(json.dumps({"profile": args.profile, "timeline": args.timeline, "span_us": round(reached - origin, 2)}))
        return 0

    if args.profile:
        # A small, self-ending case for a profiler: the cache is reserved but not computed (its content
        # does not change what the kernels do), then a few eager steps of the chosen phase run.
        if args.profile == "decode":
            ids = [f"p{i}" for i in range(args.batch)]
            for rid in ids:
                manager.admit(rid)
                manager.commit(manager.prepare([(rid, CONTEXT - args.steps - warmup - 1)]))
            decode_steps(ids, warmup + args.steps)
        else:
            for _ in range(warmup + args.steps):
                manager.admit("p")
                reservation = manager.prepare([("p", PREFILL_TOKENS)])
                step_function.run([StepEntry("p", prompt(PREFILL_TOKENS), [PREFILL_TOKENS - 1])], reservation)
                manager.commit(reservation)
                manager.release("p")
        torch.cuda.synchronize()
        print(json.dumps({"profile": args.profile, "layers": args.layers, "batch": args.batch, "steps": args.steps}))
        return 0

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    def prefill_once() -> None:
        manager.admit("p")
        entries = [StepEntry("p", prefill_prompt, [PREFILL_TOKENS - 1])]
        reservation = manager.prepare([("p", PREFILL_TOKENS)])
        step_function.run(entries, reservation)
        manager.commit(reservation)
        manager.release("p")

    prefill_prompt = prompt(PREFILL_TOKENS)
    for _ in range(warmup):
        prefill_once()
    prefill_seconds = min(event_time(prefill_once) for _ in range(3))
    h, i_, nq, nkv, d, layers = (config[k] for k in ("hidden_size", "intermediate_size", "num_attention_heads",
                                                      "num_key_value_heads", "head_dim", "num_hidden_layers"))
    matrix_params = layers * (h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * i_)
    prefill_flops = 2 * matrix_params * PREFILL_TOKENS + 2 * vocab * h \
        + layers * 4 * nq * d * PREFILL_TOKENS * (PREFILL_TOKENS + 1) / 2
    peak, peak_source = peaks()

    # ---------------------------------------------------------------- decode, device-timed
    with ClockSampler() as clocks:
        step_seconds, mean_context, launches = measure_decode(args.batch, args.steps)
    clock_summary = clocks.summary()
    # the output matrix is read whole, tied or not; of the embedding only the rows of the step's tokens
    weight_bytes = 2 * (matrix_params + vocab * h) + 2 * h * (2 * layers + 1) + 2 * 2 * d * layers
    kv_bytes_per_token = 2 * layers * nkv * d * 2
    step_bytes = weight_bytes + kv_bytes_per_token * mean_context * args.batch
    achieved_gbs = step_bytes / step_seconds / 1e9

    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            seconds, _, _ = measure_decode(batch, min(args.steps, 32))
            points[f"decode_b{batch}"] = round(batch / seconds, 1)

    # ---------------------------------------------------------------- end to end through the engine loop
    engine = build_engine(runtime)
    for index in range(args.batch):
        # prompts finish on different steps (two fit a step's token budget): the margin keeps all of them
        # decoding through the timed steps and inside the context limit
        engine.submit(f"e{index}", prompt(CONTEXT - args.steps - warmup - 8),
                      SamplingParams(temperature=0.0, max_new_tokens=args.steps + warmup + 8))
    while any(not s.is_decoding for s in engine.sequences.values()):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    step_times = []
    started = time.perf_counter()
    for _ in range(args.steps):
        before_step = time.perf_counter()
        engine.step()                      # returns after the step's token ids are on the host
        step_times.append(time.perf_counter() - before_step)
    torch.cuda.synchronize()
    e2e_seconds = (time.perf_counter() - started) / args.steps
    slow_steps = [index for index, t in enumerate(step_times) if t > 2 * sorted(step_times)[len(step_times) // 2]]
    step_times.sort()
    graph = step_function.graphs[next(b for b in sorted(step_function.graphs) if b >= args.batch)]
    h2d_bytes = graph.host.numel() * 4
    d2h_bytes = args.batch * 4

    value = args.batch / step_seconds
    line = {
        "metric": f"Qwen3-{args.shape.upper()} bf16 decode tok/s @ batch {args.batch} (context {CONTEXT}); "
                  f"prefill tok/s @ {PREFILL_TOKENS:,} tokens",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(step_seconds * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded uniform token ids, random weights)",
        "impl": "ours",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": layers,
                   "layers_of_model": shape["num_hidden_layers"],
                   "hidden": h, "q_heads": nq, "kv_heads": nkv, "head_dim": d, "intermediate": i_, "vocab": vocab,
                   "tied_embeddings": config["tie_word_embeddings"], "global_batch": args.batch, "seq_len": CONTEXT,
                   "context_len": CONTEXT, "page_size": PAGE_SIZE, "parallelism": "single GPU",
                   "decode_execution": "cuda_graph", "l2": "inputs larger than L2 (weights + cache read every step)"},
        "e2e": {"value": round(args.batch / e2e_seconds, 1), "unit": "tokens/s", "ms_per_step": round(e2e_seconds * 1e3, 4),
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "ms_median_step": round(step_times[len(step_times) // 2] * 1e3, 4),
                "ms_slowest_step": round(step_times[-1] * 1e3, 4), "slow_steps": slow_steps},
        "gpu_launches": launches * args.steps,
        "prefill": {"value": round(PREFILL_TOKENS / prefill_seconds, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_seconds * 1e3, 3),
                    "frac": round(prefill_flops / prefill_seconds / (peak["bf16_tflops"] * 1e12), 4),
                    "peak": f"{peak['bf16_tflops']} TFLOP/s bf16 of {peak_source}"},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peak["hbm_gbs"], 4), "peak_source": peak_source,
                     "bytes_per_step": int(step_bytes)},
        "points": points,
        "clocks": clock_summary,
        # which kernel the measurement at start-up chose for the few-row products of each weight shape
        "few_row_products": {**{f"{n}x{k}": choice for (_, n, k), choice in sorted(kernels.linear_choices().items())},
                             **{"gated " + "x".join(str(size) for size in key[1:]): choice
                                for key, choice in sorted(kernels.gated_choices().items())}},
        # and what it measured, in microseconds per candidate
        "few_row_us": {("gated " if len(key) > 3 else "") + f"{key[1]}x{key[2]}": times
                       for key, times in sorted(kernels.choice_times().items(), key=lambda item: item[0][:3])},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
