"""Trace replay: feeds given token ids through the model step by step and writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
              [--page-size P] [--decode-execution eager|cuda_graph] [--prefix-cache] [--max-requests R]

Steps arrive on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry continues its request with the given tokens (the first appearance of an id admits
the request); all entries of a line run as one batch through the engine's own step function,
cache manager and kernels.  The float32 logits at the wanted places are written to
``OUT/<step>.f32`` in the order of the entries and of ``want``.  Requests named in ``end``
give back what they hold after the step.  After each step ``done <step>`` is printed.
Nothing is sampled.  The page pool holds ``--max-tokens`` tokens, so pages are used again.

``--decode-execution cuda_graph`` runs steps that consist of single tokens whose logits are all
wanted as the captured graphs that generation replays (other steps run eagerly, as there).

With ``--prefix-cache`` two more keys are read.  A step's ``"cache": [ids]`` offers the full pages
that those requests hold so far to later requests (after the step has run, before ``end``).  An
entry's ``"prefix": [tokens]`` on the first appearance of its id says that the request begins with
these tokens and that pages holding them must be attached from the cache instead of computed; the
entry's ``tokens`` follow them.  If the cache does not hold exactly that prefix the step fails.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Optional

DEFAULT_PAGE_SIZE = 16   # divides 64, the granularity in which --max-tokens counts a request
MAX_LIVE_REQUESTS = 8


class TraceError(RuntimeError):
    """A step of the trace cannot be run as written."""


class TraceSession:
    """Runs trace records against a runtime: admission, reservation, the step function, commit, release.

    It owns no model, cache or forward pass; it calls the cache manager and the step function that
    generation uses, in the order the engine loop does (miniserve/engine/core.py:278-439 without
    scheduler and sampler).
    """

    def __init__(self, runtime) -> None:
        self.runtime = runtime
        self.manager, self.step_function, self.storage = runtime.manager, runtime.step_function, runtime.storage
        self.tokens: dict[str, list[int]] = {}      # what each live request has been given so far
        self.attached: dict[str, int] = {}          # tokens each live request took from the prefix cache

    def _admit(self, request_id: str, prefix: list[int], tokens: list[int]) -> None:
        manager = self.manager
        record = manager.admit(request_id)
        self.storage.reset_slot(record.slot, 0.0, 1.0, 0, 0)
        self.tokens[request_id] = []
        self.attached[request_id] = 0
        if prefix:
            matched = manager.attach_prefix(request_id, prefix + tokens) if manager.prefix is not None else 0
            if matched != len(prefix):
                manager.release(request_id)
                del self.tokens[request_id], self.attached[request_id]
                raise TraceError(f"request {request_id!r} names a prefix of {len(prefix)} tokens; the cache holds "
                                 f"{matched} of them" + ("" if manager.prefix is not None else " (prefix reuse is off)"))
            self.tokens[request_id] = list(prefix)
            self.attached[request_id] = matched

    def run(self, record: dict):
        """Runs one record; returns the float32 logits ``[wanted, vocab]`` on the device (None: no entries)."""
        from .engine.step import StepEntry

        manager = self.manager
        entries, logits = [], None
        for raw in record.get("entries", ()):
            request_id, tokens = str(raw["id"]), [int(t) for t in raw["tokens"]]
            if not tokens:
                continue
            prefix = [int(t) for t in raw.get("prefix", ())]
            if request_id not in manager.requests:
                self._admit(request_id, prefix, tokens)
            elif prefix:
                raise TraceError(f"request {request_id!r} is live already; a prefix can only come with its first tokens")
            entries.append(StepEntry(request_id, tokens, [int(i) for i in raw.get("want", ())]))
        if entries:
            reservation = manager.prepare([(e.request_id, len(e.tokens)) for e in entries])
            try:
                logits = self.step_function.run(entries, reservation)
            except BaseException:
                manager.abort(reservation)
                raise
            manager.commit(reservation)
            for entry in entries:
                self.tokens[entry.request_id].extend(entry.tokens)
        for request_id in record.get("cache", ()):
            request_id = str(request_id)
            if request_id in manager.requests:
                manager.cache_prefix(request_id, self.tokens[request_id])
        for request_id in record.get("end", ()):
            request_id = str(request_id)
            if request_id in manager.requests:
                manager.release(request_id)
                del self.tokens[request_id], self.attached[request_id]
        return logits


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    parser.add_argument("--page-size", type=int, default=DEFAULT_PAGE_SIZE,
                        help="tokens per cache page (a request's count is rounded up to a multiple of max(64, this))")
    parser.add_argument("--decode-execution", choices=("eager", "cuda_graph"), default="eager",
                        help="cuda_graph: steps of single tokens replay the captured graphs that generation uses")
    parser.add_argument("--prefix-cache", action="store_true",
                        help="reuse of whole pages between requests; reads the 'cache' and 'prefix' keys of the trace")
    parser.add_argument("--max-requests", type=int, default=MAX_LIVE_REQUESTS, help="most requests live at a time")
    args = parser.parse_args(argv)
    if args.page_size < 1 or args.max_requests < 1 or args.max_tokens < 1:
        parser.error("--page-size, --max-requests and --max-tokens must be positive")

    import numpy  # noqa: F401  (the logits are written through it)
    import torch

    from . import kernels
    from .config.engine_config import EngineConfig
    from .engine.runtime import build_runtime

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    num_pages = max(1, (args.max_tokens + args.page_size - 1) // args.page_size)
    print(f"[trace_run] loading {args.model} ({args.dtype}); compiling kernels on first use", file=sys.stderr, flush=True)
    runtime = build_runtime(args.model, EngineConfig(
        dtype=args.dtype, kv_block_size=args.page_size, num_kv_blocks=num_pages, max_num_seqs=args.max_requests,
        enable_prefix_cache=args.prefix_cache, decode_execution=args.decode_execution))
    session = TraceSession(runtime)
    print(f"[trace_run] ready: {num_pages} pages of {args.page_size} tokens, {args.decode_execution} decode steps"
          + (", prefix reuse on" if args.prefix_cache else ""), file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits: Optional[torch.Tensor] = session.run(record)
        if logits is not None:
            if logits.shape[0]:
                logits.cpu().numpy().astype("<f4", copy=False).tofile(out_dir / f"{step}.f32")
            else:
                torch.cuda.synchronize()
            kernels.check_device_errors(session.step_function.device)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
