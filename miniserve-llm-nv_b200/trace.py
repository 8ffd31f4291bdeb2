"""Trace replay: feeds given token ids through the model step by step and writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps arrive on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry continues its request with the given tokens (the first appearance of an id admits
the request); all entries of a line run as one batch through the engine's own step function,
cache manager and kernels.  The float32 logits at the wanted places are written to
``OUT/<step>.f32`` in the order of the entries and of ``want``.  Requests named in ``end``
give back what they hold after the step.  After each step ``done <step>`` is printed.
Nothing is sampled.  The page pool holds ``--max-tokens`` tokens, so pages are used again.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PAGE_SIZE = 16          # divides 64, the granularity in which --max-tokens counts a request
MAX_LIVE_REQUESTS = 8


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    args = parser.parse_args(argv)

    import numpy  # noqa: F401  (the logits are written through it)
    import torch

    from . import kernels
    from .config.engine_config import EngineConfig
    from .engine.runtime import build_runtime
    from .engine.step import StepEntry

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    num_pages = max(1, (args.max_tokens + PAGE_SIZE - 1) // PAGE_SIZE)
    print(f"[trace_run] loading {args.model} ({args.dtype}); compiling kernels on first use", file=sys.stderr, flush=True)
    runtime = build_runtime(args.model, EngineConfig(
        dtype=args.dtype, kv_block_size=PAGE_SIZE, num_kv_blocks=num_pages, max_num_seqs=MAX_LIVE_REQUESTS,
        enable_prefix_cache=False, decode_execution="eager"))
    manager, step_function = runtime.manager, runtime.step_function
    print(f"[trace_run] ready: {num_pages} pages of {PAGE_SIZE} tokens", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [StepEntry(str(e["id"]), list(e["tokens"]), list(e.get("want", ()))) for e in record.get("entries", ())]
        entries = [e for e in entries if e.tokens]
        if entries:
            for entry in entries:
                if entry.request_id not in manager.requests:
                    manager.admit(entry.request_id)
                    runtime.storage.reset_slot(manager.requests[entry.request_id].slot, 0.0, 1.0, 0, 0)
            reservation = manager.prepare([(e.request_id, len(e.tokens)) for e in entries])
            try:
                logits = step_function.run(entries, reservation)
                if logits.shape[0]:
                    logits.cpu().numpy().astype("<f4", copy=False).tofile(out_dir / f"{step}.f32")
                else:
                    torch.cuda.synchronize()
                kernels.check_device_errors(step_function.device)
            except BaseException:
                manager.abort(reservation)
                raise
            manager.commit(reservation)
        for request_id in record.get("end", ()):
            if str(request_id) in manager.requests:
                manager.release(str(request_id))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
