"""Decode and prefill throughput of the engine at Qwen3-1.7B size with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --shape 8b --workload mixed        # decode streams beside prompt chunks in one step
    python bench.py --shape 32b --workload sweep       # batch 1 / 8 / 64, short prompts, a fixed number of new tokens

Prints one JSON line.  ``value`` is decoded tokens per second at batch 8 and the context
length below, timed on the device over blocks of exactly K decode steps through the step
function: the block is repeated from the same context (the cache is cut back in between) and
the median block counts, with the spread beside it.  ``e2e`` is the same through the engine loop
a user drives (host token ids in, sampled token ids out, every step).  ``prefill`` times one
2,048-token prompt, ``roofline`` relates the decode step to the memory bandwidth, ``points`` adds
batch 1 and 64 at the same context, the workload of 2,048-token prompts plus 256 generated
tokens at batch 1, 8 and 64, and the headline step run eagerly instead of as a replayed graph;
``points_frac`` gives each point's share of the memory roofline.
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
WORKLOAD_PROMPT, WORKLOAD_NEW = 2048, 256      # the decode workload of 2,048-token prompts plus 256 generated tokens
MIN_BLOCKS, MAX_BLOCKS, TIMED_SECONDS = 9, 60, 0.6


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


def config_record(shape_name: str, shape: dict, layers: int, batch: int, decode_execution: str) -> dict:
    """The sizes a line was measured at: the same keys from both arms (flat, at most 20)."""
    return {"model": f"Qwen3-{shape_name.upper()} shape", "layers": layers, "layers_of_model": shape["num_hidden_layers"],
            "hidden": shape["hidden_size"], "q_heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
            "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
            "tied_embeddings": shape["tie_word_embeddings"], "global_batch": batch, "seq_len": CONTEXT,
            "context_len": CONTEXT, "page_size": PAGE_SIZE, "parallelism": "single GPU",
            "decode_execution": decode_execution, "l2": "inputs larger than L2 (weights + cache read every step)"}


def metric_name(shape_name: str, batch: int) -> str:
    return (f"Qwen3-{shape_name.upper()} bf16 decode tok/s @ batch {batch} (context {CONTEXT}); "
            f"prefill tok/s @ {PREFILL_TOKENS:,} tokens")


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
    shape = dict(MODEL, **SHAPES[args.shape])
    result = arm.main(dict(shape), args.batch, CONTEXT, steps, warmup, PAGE_SIZE)
    if "unavailable" in result:
        print(json.dumps(result))
        return 0
    line = {
        "metric": metric_name(args.shape, args.batch),
        "impl": "reference", "value": result["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": result["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded uniform token ids, random weights)",
        # its batched decode graph, CUDA paged decode attention and CUDA RMSNorm (its fastest legal settings)
        "config": config_record(args.shape, shape, shape["num_hidden_layers"], args.batch, "cuda_graph"),
        # Every step its sampler hands one token id per request to the host, and its batch builder makes five
        # device tensors from host lists (miniserve/engine/flat_batch.py:433-447: token ids, positions and slots
        # as int64, context lengths and block tables as int32); the bytes are counted from those shapes.
        "e2e": {"value": result["value"], "unit": "tokens/s", "ms_per_step": result["ms_per_step"],
                "h2d_bytes_per_step": args.batch * (8 + 8 + 8 + 4 + 4 * ((CONTEXT + PAGE_SIZE - 1) // PAGE_SIZE)),
                "d2h_bytes_per_step": 8 * args.batch, "bytes": "counted from the shapes of its step inputs and outputs"},
        "prefill_seconds_total": result["prefill_seconds_total"],
    }
    print(json.dumps(line))
    return 0


class Bench:
    """The runtime under measurement and the few moves every workload is made of."""

    def __init__(self, args, shape: dict, config: dict, max_batch: int, max_context: int, budget: int) -> None:
        import torch

        import miniserve_b200  # noqa: F401
        from miniserve_b200.config import EngineConfig
        from miniserve_b200.engine.runtime import build_runtime
        from miniserve_b200.engine.step import StepEntry

        self.torch, self.StepEntry = torch, StepEntry
        self.args, self.shape, self.config = args, shape, config
        self.warmup = max(args.warmup, 3)
        extra = 1 if args.workload == "mixed" else 0          # the request whose prompt advances beside the streams
        pages = (max_batch + extra) * ((max_context + PAGE_SIZE - 1) // PAGE_SIZE) + budget // PAGE_SIZE + 64
        self.runtime = build_runtime(None, EngineConfig(
            dtype="bfloat16", max_model_len=max(max_context, budget), max_num_seqs=max_batch + extra, kv_block_size=PAGE_SIZE,
            num_kv_blocks=pages, max_num_batched_tokens=max(8192, budget), enable_prefix_cache=False,
            decode_execution="eager" if args.profile and not args.timeline else "cuda_graph"),
            config_dict=config, weights_seed=0)
        self.manager, self.step_function = self.runtime.manager, self.runtime.step_function
        self.vocab = config["vocab_size"]
        self.generator = torch.Generator().manual_seed(1)
        h, i_, nq, nkv, d, layers = (config[k] for k in ("hidden_size", "intermediate_size", "num_attention_heads",
                                                          "num_key_value_heads", "head_dim", "num_hidden_layers"))
        self.matrix_params = layers * (h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * i_)
        # the output matrix is read whole, tied or not; of the embedding only the rows of the step's tokens
        self.weight_bytes = 2 * (self.matrix_params + self.vocab * h) + 2 * h * (2 * layers + 1) + 2 * 2 * d * layers
        self.kv_bytes_per_token = 2 * layers * nkv * d * 2
        self.peak, self.peak_source = peaks()

    # ------------------------------------------------------------------ moves
    def prompt(self, n: int) -> list[int]:
        return self.torch.randint(0, self.vocab, (n,), generator=self.generator).tolist()

    def event_time(self, fn) -> float:
        torch = self.torch
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / 1e3

    def fill(self, ids: list[str], length: int, compute: bool = True) -> None:
        """Admits the requests and gives each ``length`` tokens of context: computed through the step function,
        or (``compute=False``) only reserved, where the cache's content does not change what is timed."""
        manager = self.manager
        for rid in ids:
            manager.admit(rid)
            self.runtime.storage.reset_slot(manager.requests[rid].slot, 0.0, 1.0, 0, 0)
            done = 0
            while done < length:
                take = min(2048, length - done) if compute else length - done
                reservation = manager.prepare([(rid, take)])
                if compute:
                    self.step_function.run([self.StepEntry(rid, self.prompt(take), [])], reservation)
                manager.commit(reservation)
                done += take
        self.torch.cuda.synchronize()

    def decode_steps(self, ids: list[str], count: int) -> None:
        manager, run, entry = self.manager, self.step_function.run, self.StepEntry
        draws = [0] * len(ids)
        for _ in range(count):
            entries = [entry(rid, [1], [0]) for rid in ids]
            reservation = manager.prepare([(rid, 1) for rid in ids])
            run(entries, reservation, draws)
            manager.commit(reservation)

    def rewind(self, ids: list[str], length: int) -> None:
        for rid in ids:
            self.manager.truncate(rid, length)

    def release(self, ids: list[str]) -> None:
        for rid in ids:
            self.manager.release(rid)

    def roofline(self, batch: int, mean_context: float, seconds: float) -> tuple[float, float, int]:
        """(achieved GB/s, share of the copy bandwidth, bytes) of a decode step: every weight once plus the
        cache of the live requests."""
        step_bytes = self.weight_bytes + self.kv_bytes_per_token * mean_context * batch
        achieved = step_bytes / seconds / 1e9
        return achieved, achieved / self.peak["hbm_gbs"], int(step_bytes)

    # ------------------------------------------------------------------ measurements
    def measure_decode(self, batch: int, start: int, steps: int, blocks: int = 0, eager: bool = False,
                       compute_fill: bool = True) -> dict:
        """Blocks of ``steps`` decode steps, every block from ``start`` tokens of context per request; the median
        block's seconds per step, the spread over blocks and the mean context of a block's steps."""
        ids = [f"d{batch}-{i}" for i in range(batch)]
        self.fill(ids, start, compute_fill)
        sf = self.step_function
        graphs = sf.use_graphs
        sf.use_graphs = graphs and not eager
        try:
            self.decode_steps(ids, self.warmup)
            self.rewind(ids, start)
            first = self.event_time(lambda: self.decode_steps(ids, steps))
            self.rewind(ids, start)
            if blocks <= 0:
                blocks = min(MAX_BLOCKS, max(MIN_BLOCKS, int(TIMED_SECONDS / max(first, 1e-6)) + 1))
            times = []
            for _ in range(blocks):
                times.append(self.event_time(lambda: self.decode_steps(ids, steps)) / steps)
                self.rewind(ids, start)
        finally:
            sf.use_graphs = graphs
        launches = 0
        if not eager and sf.graphs:
            launches = sf.graphs[next(b for b in sorted(sf.graphs) if b >= batch)].kernel_launches
        self.release(ids)
        times.sort()
        seconds = times[len(times) // 2]
        mean_context = start + (steps + 1) / 2
        achieved, frac, step_bytes = self.roofline(batch, mean_context, seconds)
        return {"seconds": seconds, "fastest": times[0], "slowest": times[-1], "blocks": blocks, "mean_context": mean_context,
                "launches": launches, "achieved_gbs": achieved, "frac": frac, "bytes": step_bytes,
                "timed_seconds": sum(times) * steps}

    def measure_prefill(self, tokens: int) -> float:
        import numpy

        manager = self.manager
        prompt = numpy.asarray(self.prompt(tokens), dtype=numpy.int64)      # as the engine's sequences hold their prompts

        def once() -> None:
            manager.admit("p")
            reservation = manager.prepare([("p", tokens)])
            self.step_function.run([self.StepEntry("p", prompt, [tokens - 1])], reservation)
            manager.commit(reservation)
            manager.release("p")

        for _ in range(self.warmup):
            once()
        return sorted(self.event_time(once) for _ in range(11))[5]

    def prefill_flops(self, tokens: int) -> float:
        c = self.config
        return 2 * self.matrix_params * tokens + 2 * self.vocab * c["hidden_size"] \
            + c["num_hidden_layers"] * 4 * c["num_attention_heads"] * c["head_dim"] * tokens * (tokens + 1) / 2

    def timeline(self, one_step, path: str, title: str) -> float:
        """Runs ``one_step`` under the framework's profiler (CUPTI) and writes every kernel's start, duration and
        exposed time (how far its end lies past the end of everything before it: kernels of a replayed graph keep
        their programmatic overlap, so that is what a kernel adds to the step)."""
        from torch.profiler import ProfilerActivity, profile

        torch = self.torch
        for _ in range(self.warmup):
            one_step()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as profiler:
            one_step()
            torch.cuda.synchronize()
        trace_file = path + ".trace.json"
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
        with open(path, "w") as handle:
            handle.write(f"{title}, span {reached - origin:.2f} us\n\n" + "\n".join(summary) + "\n\n" + "\n".join(lines) + "\n")
        return reached - origin


def profile_mode(bench: Bench, args) -> int:
    """``--profile``: a small, self-ending case of one phase, for a profiler (times nothing); with ``--timeline``
    the step is run under the framework's own profiler and its kernels are listed."""
    manager, step_function, entry = bench.manager, bench.step_function, bench.StepEntry
    ids = [f"p{i}" for i in range(args.batch)]
    prompt_tokens = bench.prompt(PREFILL_TOKENS)

    def prompt_step() -> None:
        manager.admit("p")
        reservation = manager.prepare([("p", PREFILL_TOKENS)])
        step_function.run([entry("p", prompt_tokens, [PREFILL_TOKENS - 1])], reservation)
        manager.commit(reservation)
        manager.release("p")

    if args.timeline:
        def decode_step() -> None:
            reservation = manager.prepare([(rid, 1) for rid in ids])
            step_function.run([entry(rid, [1], [0]) for rid in ids], reservation, [0] * len(ids))
            manager.abort(reservation)                       # the context stays as long as it was

        if args.profile == "decode":
            bench.fill(ids, CONTEXT - 1, compute=False)
        span = bench.timeline(decode_step if args.profile == "decode" else prompt_step, args.timeline,
                              f"step: {args.profile}, batch {args.batch}, layers {args.layers}, context {CONTEXT}")
        print(json.dumps({"profile": args.profile, "timeline": args.timeline, "span_us": round(span, 2)}))
        return 0
    # the cache is reserved but not computed (its content does not change what the kernels do)
    if args.profile == "decode":
        bench.fill(ids, CONTEXT - args.steps - bench.warmup - 1, compute=False)
        bench.decode_steps(ids, bench.warmup + args.steps)
    else:
        for _ in range(bench.warmup + args.steps):
            prompt_step()
    bench.torch.cuda.synchronize()
    print(json.dumps({"profile": args.profile, "layers": args.layers, "batch": args.batch, "steps": args.steps}))
    return 0


def mixed_workload(bench: Bench, args) -> int:
    """Decode streams beside a prompt chunk in ONE step (the engine's mixed batch): ``--batch`` requests at
    ``--context`` tokens decode one token each while another request's prompt advances by a chunk of
    ``--prefill-tokens`` tokens, at every chunk position up to the context.  Beside it the two kinds alone."""
    manager, step_function, entry, torch = bench.manager, bench.step_function, bench.StepEntry, bench.torch
    streams = [f"s{i}" for i in range(args.batch)]
    chunk = PREFILL_TOKENS
    bench.fill(streams, CONTEXT - 1, compute=False)
    chunk_tokens = bench.prompt(chunk)
    manager.admit("c")
    bench.runtime.storage.reset_slot(manager.requests["c"].slot, 0.0, 1.0, 0, 0)

    def step(with_streams: bool, with_chunk: bool) -> None:
        items, entries = [], []
        if with_streams:
            items += [(rid, 1) for rid in streams]
            entries += [entry(rid, [1], [0]) for rid in streams]
        if with_chunk:
            items.append(("c", chunk))
            entries.append(entry("c", chunk_tokens, [chunk - 1]))
        reservation = manager.prepare(items)
        step_function.run(entries, reservation)
        manager.abort(reservation)                           # every repeat sees the same contexts

    def timed(with_streams: bool, with_chunk: bool) -> float:
        for _ in range(bench.warmup):
            step(with_streams, with_chunk)
        return sorted(bench.event_time(lambda: step(with_streams, with_chunk)) for _ in range(7))[3]

    graphs = step_function.use_graphs
    rows = []
    decode_alone_graph = timed(True, False)
    step_function.use_graphs = False
    decode_alone_eager = timed(True, False)
    for position in range(0, CONTEXT - chunk + 1, chunk):
        if manager.length("c") != position:
            manager.commit(manager.prepare([("c", position - manager.length("c"))]))
        alone, mixed = timed(False, True), timed(True, True)
        rows.append({"chunk_context_before": position, "ms_mixed_step": round(mixed * 1e3, 3),
                     "ms_chunk_alone": round(alone * 1e3, 3),
                     "decode_tok_s_in_mixed_step": round(args.batch / mixed, 1),
                     "prefill_tok_s_in_mixed_step": round(chunk / mixed, 1),
                     "ms_saved_against_two_steps": round((alone + decode_alone_graph - mixed) * 1e3, 3)})
    if args.timeline:
        bench.timeline(lambda: step(True, True), args.timeline,
                       f"mixed step: {args.batch} decode streams at context {CONTEXT} beside a chunk of {chunk} tokens "
                       f"at context {manager.length('c')}, layers {args.layers}")
    step_function.use_graphs = graphs
    decode_bytes = bench.weight_bytes + bench.kv_bytes_per_token * CONTEXT * args.batch
    from miniserve_b200 import kernels
    print(json.dumps({
        "workload": "mixed", "impl": "ours", "dtype": "bf16",
        "config": config_record(args.shape, bench.shape, args.layers, args.batch, "eager (mixed steps), cuda_graph (decode alone)"),
        "decode_streams": args.batch, "stream_context": CONTEXT, "chunk_tokens": chunk,
        "ms_decode_alone_graph": round(decode_alone_graph * 1e3, 3), "ms_decode_alone_eager": round(decode_alone_eager * 1e3, 3),
        "decode_alone_roofline_frac": round(decode_bytes / decode_alone_graph / 1e9 / bench.peak["hbm_gbs"], 4),
        "steps": rows, "peak_source": bench.peak_source,
        "many_row_products": {f"{kind} {tiles} row tiles {n}x{k}": [choice, times]
                              for (_, kind, tiles, n, k), (choice, times) in sorted(kernels.many_row_choices().items())}}))
    return 0


def sweep_workload(bench: Bench, args) -> int:
    """Batch 1, 8 and 64 with prompts of ``--sweep-prompt`` tokens and ``--sweep-new`` generated tokens each:
    all the new tokens' steps are timed as one region, three times from the same start."""
    points = {}
    for batch in (1, 8, 64):
        m = bench.measure_decode(batch, args.sweep_prompt, args.sweep_new, blocks=3)
        points[f"decode_b{batch}"] = {"tok_s": round(batch / m["seconds"], 1), "ms_per_step": round(m["seconds"] * 1e3, 4),
                                      "roofline_frac": round(m["frac"], 4), "achieved_gbs": round(m["achieved_gbs"], 1),
                                      "ms_fastest": round(m["fastest"] * 1e3, 4), "ms_slowest": round(m["slowest"] * 1e3, 4)}
    seconds = bench.measure_prefill(args.sweep_prompt)
    from miniserve_b200 import kernels
    print(json.dumps({
        "workload": f"sweep: prompts of {args.sweep_prompt} tokens, {args.sweep_new} new tokens", "impl": "ours", "dtype": "bf16",
        "config": config_record(args.shape, bench.shape, args.layers, 64, "cuda_graph"), "points": points,
        "prefill": {"tokens": args.sweep_prompt, "ms": round(seconds * 1e3, 3), "tok_s": round(args.sweep_prompt / seconds, 1),
                    "frac": round(bench.prefill_flops(args.sweep_prompt) / seconds / (bench.peak["bf16_tflops"] * 1e12), 4)},
        "peak": {"hbm_gbs": bench.peak["hbm_gbs"], "bf16_tflops": bench.peak["bf16_tflops"], "source": bench.peak_source},
        "few_row_products": {f"{n}x{k}": choice for (_, n, k), choice in sorted(kernels.linear_choices().items())}}))
    return 0


def main() -> int:
    global CONTEXT, PREFILL_TOKENS
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--batch", type=int, default=None, help="decode requests (default 8; 32 for --workload mixed)")
    parser.add_argument("--layers", type=int, default=None,
                        help="fewer layers than the model has (named in the output); for quick checks only")
    parser.add_argument("--skip-points", action="store_true")
    parser.add_argument("--workload", choices=("default", "mixed", "sweep"), default="default")
    parser.add_argument("--sweep-prompt", type=int, default=1024)
    parser.add_argument("--sweep-new", type=int, default=128)
    parser.add_argument("--timeline", metavar="FILE", default=None,
                        help="with --profile or --workload mixed: run the step under the framework profiler and write "
                             "every kernel's start, duration and exposed time to FILE")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="1.7b",
                        help="layer sizes of another model of the family (the default is the benchmark's)")
    parser.add_argument("--context", type=int, default=None,
                        help="tokens a request holds at the end of the timed steps (default 4,096; 8,192 for --workload mixed)")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                        help="tokens of the timed prompt step (the benchmark's is 2,048; others for profiles)")
    parser.add_argument("--profile", choices=("decode", "prefill"), default=None,
                        help="run only a few eager steps of one phase and exit (a small case for ncu; times nothing)")
    args = parser.parse_args()
    if args.batch is None:
        args.batch = 32 if args.workload == "mixed" else 8
    CONTEXT = args.context or (8192 if args.workload == "mixed" else CONTEXT)
    PREFILL_TOKENS = args.prefill_tokens
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2

    shape = dict(MODEL, **SHAPES[args.shape])
    if args.layers is None:
        args.layers = shape["num_hidden_layers"]
    config = dict(shape, num_hidden_layers=args.layers)
    plain_run = args.workload == "default" and not args.profile
    if args.workload == "sweep":
        max_batch, max_context = 64, args.sweep_prompt + args.sweep_new + 8
    elif plain_run and not args.skip_points:
        max_batch, max_context = 64, max(CONTEXT, WORKLOAD_PROMPT + WORKLOAD_NEW)
    else:
        max_batch, max_context = args.batch, CONTEXT
    bench = Bench(args, shape, config, max_batch, max_context + 8, max(PREFILL_TOKENS, args.sweep_prompt if args.workload == "sweep" else 0))
    if args.profile:
        return profile_mode(bench, args)
    if args.workload == "mixed":
        return mixed_workload(bench, args)
    if args.workload == "sweep":
        return sweep_workload(bench, args)

    import torch
    from miniserve_b200 import kernels
    from miniserve_b200.engine.llm import build_engine
    from miniserve_b200.sampling import SamplingParams

    warmup, steps, batch = bench.warmup, args.steps, args.batch
    if steps < 1 or steps + warmup + 16 > CONTEXT:
        print(f"bench.py: --steps {steps} does not fit the context of {CONTEXT} tokens (or is not positive)")
        return 2

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    prefill_seconds = bench.measure_prefill(PREFILL_TOKENS)

    # ---------------------------------------------------------------- decode, device-timed
    with ClockSampler() as clocks:
        headline = bench.measure_decode(batch, CONTEXT - steps, steps)
    clock_summary = clocks.summary()

    points, fracs = {}, {}
    if not args.skip_points:
        for b in (1, 64):
            m = bench.measure_decode(b, CONTEXT - steps, steps)
            points[f"decode_b{b}"], fracs[f"decode_b{b}"] = round(b / m["seconds"], 1), round(m["frac"], 4)
        for b in (1, 8, 64):            # 2,048-token prompts plus 256 generated tokens: all 256 steps as one region
            m = bench.measure_decode(b, WORKLOAD_PROMPT, WORKLOAD_NEW, blocks=3)
            key = f"decode_b{b}_prompt{WORKLOAD_PROMPT}_new{WORKLOAD_NEW}"
            points[key], fracs[key] = round(b / m["seconds"], 1), round(m["frac"], 4)
        m = bench.measure_decode(batch, CONTEXT - steps, steps, blocks=5, eager=True)
        points[f"decode_b{batch}_eager"], fracs[f"decode_b{batch}_eager"] = round(batch / m["seconds"], 1), round(m["frac"], 4)

    # ---------------------------------------------------------------- end to end through the engine loop
    engine = build_engine(bench.runtime)
    e2e_blocks = 5
    new_tokens = e2e_blocks * steps + warmup + 8
    for index in range(batch):
        # prompts finish on different steps (two fit a step's token budget): the margin keeps all of them
        # decoding through the timed steps and inside the context limit
        engine.submit(f"e{index}", bench.prompt(CONTEXT - new_tokens), SamplingParams(temperature=0.0, max_new_tokens=new_tokens))
    while any(not s.is_decoding for s in engine.sequences.values()):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    step_times, block_seconds = [], []
    for _ in range(e2e_blocks):
        started = time.perf_counter()
        for _ in range(steps):
            before_step = time.perf_counter()
            engine.step()                      # returns after the step's token ids are on the host
            step_times.append(time.perf_counter() - before_step)
        block_seconds.append((time.perf_counter() - started) / steps)
    torch.cuda.synchronize()
    block_seconds.sort()
    e2e_seconds = block_seconds[len(block_seconds) // 2]
    median_step = sorted(step_times)[len(step_times) // 2]
    slow_steps = [index for index, t in enumerate(step_times) if t > 2 * median_step]
    graph = bench.step_function.graphs[next(b for b in sorted(bench.step_function.graphs) if b >= batch)]
    h2d_bytes = graph.host.numel() * 4
    d2h_bytes = batch * 4

    seconds = headline["seconds"]
    line = {
        "metric": metric_name(args.shape, batch),
        "value": round(batch / seconds, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(seconds * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded uniform token ids, random weights)",
        "impl": "ours",
        "config": config_record(args.shape, shape, args.layers, batch, "cuda_graph"),
        # the block of `steps` steps was timed this often, each time from the same context; `value` is the median block
        "blocks": {"count": headline["blocks"], "ms_per_step_fastest": round(headline["fastest"] * 1e3, 4),
                   "ms_per_step_slowest": round(headline["slowest"] * 1e3, 4),
                   "timed_seconds": round(headline["timed_seconds"], 3), "mean_context": headline["mean_context"]},
        "e2e": {"value": round(batch / e2e_seconds, 1), "unit": "tokens/s", "ms_per_step": round(e2e_seconds * 1e3, 4),
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes, "blocks": e2e_blocks,
                "ms_per_step_fastest_block": round(block_seconds[0] * 1e3, 4),
                "ms_per_step_slowest_block": round(block_seconds[-1] * 1e3, 4),
                "ms_median_step": round(median_step * 1e3, 4), "ms_slowest_step": round(max(step_times) * 1e3, 4),
                "slow_steps": slow_steps, "context": f"{CONTEXT - new_tokens + warmup} to {CONTEXT}"},
        "gpu_launches": headline["launches"] * steps,
        "prefill": {"value": round(PREFILL_TOKENS / prefill_seconds, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_seconds * 1e3, 3),
                    "frac": round(bench.prefill_flops(PREFILL_TOKENS) / prefill_seconds / (bench.peak["bf16_tflops"] * 1e12), 4),
                    "peak": f"{bench.peak['bf16_tflops']} TFLOP/s bf16 of {bench.peak_source}"},
        "roofline": {"bound": "hbm", "achieved": round(headline["achieved_gbs"], 1), "peak": bench.peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(headline["frac"], 4), "peak_source": bench.peak_source,
                     "bytes_per_step": headline["bytes"]},
        "points": points,
        "points_frac": fracs,
        "clocks": clock_summary,
        # which kernel ran the few-row products of each weight shape, and what the measurement behind it saw (us)
        "few_row_products": {**{f"{n}x{k}": choice for (_, n, k), choice in sorted(kernels.linear_choices().items())},
                             **{"gated " + "x".join(str(size) for size in key[1:]): choice
                                for key, choice in sorted(kernels.gated_choices().items())}},
        "many_row_products": {f"{kind} {tiles} row tiles {n}x{k}": [choice, times]
                              for (_, kind, tiles, n, k), (choice, times) in sorted(kernels.many_row_choices().items())},
        "few_row_us": {("gated " if len(key) > 3 else "") + f"{key[1]}x{key[2]}": times
                       for key, times in sorted(kernels.choice_times().items(), key=lambda item: item[0][:3])},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
