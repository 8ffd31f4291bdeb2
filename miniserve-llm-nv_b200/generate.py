"""Command line: generate token ids from token ids.

    python -m miniserve_b200.generate --model DIR --prompt-ids 1,2,3 --prompt-ids 4,5 --max-new-tokens 16

The engine options have the names and meanings of MiniServe's server command
(miniserve/api/server.py:350-397): ``--model``, ``--max-model-len``, ``--num-kv-blocks``,
``--max-num-seqs``, ``--max-pending-requests``, ``--max-num-batched-tokens``, ``--kv-block-size``,
``--decode-execution cuda_graph|eager``, ``--no-prefix-cache``, ``--chunked-prefill`` /
``--no-chunked-prefill``, ``--prefill-chunk-size``.  Its backend switches have no counterpart:
there is one path.  The sampling options are those of its request schema
(miniserve/engine/request.py:9-59).  ``--model`` is a folder with ``config.json`` and
safetensors; ``--random-config FILE`` writes such a folder with seeded random weights first.
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile
from pathlib import Path


def build_cli_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="miniserve_b200.generate", description="Generate token ids with the engine.")
    source = parser.add_mutually_exclusive_group(required=True)
    source.add_argument("--model", help="folder with config.json and *.safetensors")
    source.add_argument("--random-config", help="a config.json; weights are drawn from --weights-seed")
    parser.add_argument("--weights-seed", type=int, default=0)
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; repeatable")
    parser.add_argument("--prompt-lens", default=None, help="comma-separated lengths of seeded random prompts")
    parser.add_argument("--prompt-seed", type=int, default=0)
    parser.add_argument("--max-new-tokens", type=int, default=4)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--seed", type=int, default=None, help="seed of the requests' random streams (request i uses seed + i)")
    parser.add_argument("--stop-token-ids", default="", help="comma-separated token ids that end a request")
    parser.add_argument("--max-model-len", type=int, default=None)
    parser.add_argument("--num-kv-blocks", type=int, default=None)
    parser.add_argument("--max-num-seqs", type=int, default=8)
    parser.add_argument("--max-pending-requests", type=int, default=64)
    parser.add_argument("--max-num-batched-tokens", type=int, default=None)
    parser.add_argument("--kv-block-size", type=int, default=16)
    parser.add_argument("--decode-execution", choices=("cuda_graph", "eager"), default="cuda_graph")
    parser.add_argument("--no-decode-look-ahead", action="store_true",
                        help="read every decode step's tokens before the next step starts")
    parser.add_argument("--no-prefix-cache", action="store_true")
    chunk = parser.add_mutually_exclusive_group()
    chunk.add_argument("--chunked-prefill", dest="enable_chunked_prefill", action="store_true")
    chunk.add_argument("--no-chunked-prefill", dest="enable_chunked_prefill", action="store_false")
    parser.set_defaults(enable_chunked_prefill=True)
    parser.add_argument("--prefill-chunk-size", type=int, default=None)
    parser.add_argument("--json", action="store_true", help="print one JSON object per request")
    return parser


def _ids(text: str) -> list[int]:
    return [int(part) for part in text.split(",") if part.strip()]


def main(argv=None) -> int:
    args = build_cli_parser().parse_args(argv)
    import random

    from .config.registry import read_config_json
    from .engine.llm import LLM
    from .sampling.params import SamplingParams
    from .weights.random_init import write_random_model

    holder = None
    model_dir = args.model
    if args.random_config:
        holder = tempfile.TemporaryDirectory(prefix="miniserve_b200_random_")
        config = json.loads(Path(args.random_config).read_text(encoding="utf-8"))
        model_dir = str(write_random_model(holder.name, config, args.weights_seed,
                                           "bfloat16" if args.dtype == "bfloat16" else "float32"))
    vocab = int(read_config_json(model_dir)["vocab_size"])
    prompts = [_ids(text) for text in args.prompt_ids]
    if args.prompt_lens:
        rng = random.Random(args.prompt_seed)
        prompts += [[rng.randrange(vocab) for _ in range(n)] for n in _ids(args.prompt_lens)]
    if not prompts:
        print("no prompts: give --prompt-ids or --prompt-lens", file=sys.stderr)
        return 2
    llm = LLM(model_dir, dtype=args.dtype, max_model_len=args.max_model_len, num_kv_blocks=args.num_kv_blocks,
              max_num_seqs=args.max_num_seqs, max_pending_requests=args.max_pending_requests,
              max_num_batched_tokens=args.max_num_batched_tokens, kv_block_size=args.kv_block_size,
              decode_execution=args.decode_execution, decode_look_ahead=not args.no_decode_look_ahead, enable_prefix_cache=not args.no_prefix_cache,
              enable_chunked_prefill=args.enable_chunked_prefill, prefill_chunk_size=args.prefill_chunk_size)
    params = [SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                             max_new_tokens=args.max_new_tokens, stop_token_ids=tuple(_ids(args.stop_token_ids)),
                             seed=None if args.seed is None else args.seed + index)
              for index in range(len(prompts))]
    for index, result in enumerate(llm.generate(prompts, params)):
        if args.json:
            print(json.dumps({"request": index, "token_ids": result.token_ids, "finish_reason": result.finish_reason}))
        else:
            print(",".join(str(t) for t in result.token_ids))
    if holder is not None:
        holder.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
