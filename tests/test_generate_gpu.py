"""Generation through the Python entry point and the command line, against the plain
implementation: greedy and sampled tokens, long decoding, scheduling under few pages."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import helpers
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent


def check_against_plain(folder, prompt, produced, params, dtype, seed=None):
    """Follows the produced tokens and checks each against the plain rule; a different token is
    accepted only where the plain scores of the two are within the path's rounding."""
    config, weights = plain.load_folder(folder, torch.float64)
    tokens = list(prompt)
    for draw, token in enumerate(produced):
        logits = plain.plain_logits(tokens, weights, config)[-1]
        expected = plain.plain_sample(logits.float(), params.temperature, params.top_k, params.top_p, seed or 0, draw)
        if token != expected:
            limit = (1e-4 if dtype == "float32" else 4e-2) * max(1.0, float(logits.abs().max()))
            if params.temperature == 0:
                assert float(logits[expected] - logits[token]) <= limit, (draw, token, expected)
            else:
                scaled = logits / params.temperature
                noisy = [float(scaled[t]) + plain.plain_gumbel(seed, draw, t) for t in (expected, token)]
                assert noisy[0] - noisy[1] <= limit / params.temperature, (draw, token, expected)
        tokens.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size,execution", [("a", 16, "eager"), ("b", 8, "cuda_graph"), ("c", 4, "cuda_graph")])
def test_greedy_generation(tmp_path, dtype, name, page_size, execution):
    from miniserve_b200.engine.llm import LLM
    from miniserve_b200.sampling import SamplingParams

    folder = helpers.make_folder(tmp_path, name, seed=5)
    vocab = helpers.TINY[name]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=400 + n) for n in (1, 7, 16, 33)]
    llm = LLM(str(folder), dtype=dtype, kv_block_size=page_size, num_kv_blocks=40, max_num_seqs=4,
              max_num_batched_tokens=24, prefill_chunk_size=12, decode_execution=execution)
    params = SamplingParams(temperature=0.0, max_new_tokens=8)
    results = llm.generate(prompts, params)
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == 8 and result.finish_reason == "length"
        check_against_plain(folder, prompt, result.token_ids, params, dtype)
    # the same prompts one at a time give the same tokens as in the batch
    alone = [llm.generate([p], params)[0].token_ids for p in prompts]
    if dtype == "float32":
        assert alone == [r.token_ids for r in results]
    llm.runtime.manager.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sampled_generation_with_prefix_and_chunks(tmp_path, dtype):
    """Config B of the brief: five prompts, two sharing 16 tokens, chunk 12, temperature 0.8, a seed each."""
    from miniserve_b200.engine.llm import LLM
    from miniserve_b200.sampling import SamplingParams

    folder = helpers.make_folder(tmp_path, "b", seed=6)
    vocab = helpers.TINY_B["vocab_size"]
    shared = helpers.random_tokens(vocab, 16, seed=1)
    prompts = [helpers.random_tokens(vocab, 3, 2), helpers.random_tokens(vocab, 9, 3),
               shared + helpers.random_tokens(vocab, 8, 4), shared + helpers.random_tokens(vocab, 24, 5),
               helpers.random_tokens(vocab, 65, 6)]
    params = [SamplingParams(temperature=0.8, max_new_tokens=10, seed=1000 + i, top_k=(0, 20, 0, 0, 50)[i],
                             top_p=(1.0, 1.0, 0.9, 1.0, 0.8)[i]) for i in range(5)]
    llm = LLM(str(folder), dtype=dtype, kv_block_size=8, num_kv_blocks=48, max_num_seqs=3, max_num_batched_tokens=32,
              prefill_chunk_size=12)
    first = llm.generate(prompts, params)
    for prompt, param, result in zip(prompts, params, first):
        check_against_plain(folder, prompt, result.token_ids, param, dtype, seed=param.seed)
    assert llm.engine.stats.prefix_hit_tokens >= 16
    again = llm.generate(prompts, params)               # same seeds, now with every prompt's pages cached
    assert [r.token_ids for r in again] == [r.token_ids for r in first]
    other = llm.generate(prompts[:1], SamplingParams(temperature=0.8, max_new_tokens=10, seed=7))
    assert other[0].token_ids != first[0].token_ids


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_under_few_pages(tmp_path, dtype):
    """200 decoded tokens per request with so few pages that requests are preempted and recomputed."""
    from miniserve_b200.engine.llm import LLM
    from miniserve_b200.sampling import SamplingParams

    folder = helpers.make_folder(tmp_path, "a", seed=7)
    prompts = [helpers.random_tokens(256, n, seed=500 + n) for n in (5, 12, 30)]
    params = SamplingParams(temperature=0.0, max_new_tokens=200)
    llm = LLM(str(folder), dtype=dtype, kv_block_size=16, num_kv_blocks=30, max_num_seqs=3)
    results = llm.generate(prompts, params)
    assert llm.engine.stats.preemptions >= 1
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == 200
        check_against_plain(folder, prompt, result.token_ids, params, dtype)     # bfloat16: under the near-tie rule
    assert llm.runtime.manager.capacity().free_slots == 3


def test_command_line(tmp_path):
    folder = helpers.make_folder(tmp_path, "a", seed=8)
    command = [sys.executable, "-m", "miniserve_b200.generate", "--model", str(folder), "--dtype", "float32",
               "--prompt-ids", "5,17,3", "--prompt-lens", "9", "--max-new-tokens", "5", "--num-kv-blocks", "16",
               "--max-num-seqs", "2", "--json"]
    done = subprocess.run(command, cwd=REPO, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr
    lines = [json.loads(line) for line in done.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(line["token_ids"]) == 5 for line in lines)
    from miniserve_b200.sampling import SamplingParams
    check_against_plain(folder, [5, 17, 3], lines[0]["token_ids"], SamplingParams(), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_one_step_ahead_on_the_device(tmp_path, dtype):
    """Replayed decode steps started before the last tokens are read (the device feeds them back itself)
    give the tokens of the step-by-step engine: greedy and seeded sampling, budgets that end at different
    steps, and stop tokens that are found one step late."""
    from miniserve_b200.engine.llm import LLM
    from miniserve_b200.sampling import SamplingParams

    folder = helpers.make_folder(tmp_path, "b", seed=9)
    vocab = helpers.TINY_B["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=700 + n) for n in (5, 11, 2, 19)]
    outcomes = {}
    for look_ahead in (False, True):
        llm = LLM(str(folder), dtype=dtype, kv_block_size=8, num_kv_blocks=40, max_num_seqs=4,
                  max_num_batched_tokens=64, decode_execution="cuda_graph", decode_look_ahead=look_ahead)
        assert llm.engine.look_ahead == look_ahead
        free = llm.generate(prompts, [SamplingParams(temperature=(0.0, 0.9)[i % 2], seed=50 + i,
                                                     max_new_tokens=(24, 7, 16, 30)[i]) for i in range(4)])
        # now stop each request on a token it is known to produce part-way
        stops = [(r.token_ids[len(r.token_ids) // 2],) for r in free]
        stopped = llm.generate(prompts, [SamplingParams(temperature=(0.0, 0.9)[i % 2], seed=50 + i, stop_token_ids=stops[i],
                                                        max_new_tokens=(24, 7, 16, 30)[i]) for i in range(4)])
        for r, stop in zip(stopped, stops):
            assert r.finish_reason == "stop" and r.token_ids[-1] == stop[0] and stop[0] not in r.token_ids[:-1]
        outcomes[look_ahead] = [(r.token_ids, r.finish_reason) for r in free + stopped]
        llm.runtime.manager.check_invariants()
        assert not llm.runtime.manager.requests
        if look_ahead:
            assert llm.runtime.step_function.graph_replays > 0
    assert outcomes[True] == outcomes[False]


def test_requests_arriving_while_others_decode(tmp_path):
    """Thirty requests of random lengths, budgets and sampling settings arrive a few at a time while the
    engine runs (replayed graphs, decoding ahead, a prefix cache, so few pages that requests are preempted
    and recomputed); every request's tokens follow the plain rule from its own prompt and seed."""
    import random

    from miniserve_b200.engine.llm import LLM
    from miniserve_b200.sampling import SamplingParams

    folder = helpers.make_folder(tmp_path, "c", seed=11)
    vocab = helpers.TINY["c"]["vocab_size"]
    rng = random.Random(5)
    llm = LLM(str(folder), dtype="float32", kv_block_size=4, num_kv_blocks=24, max_num_seqs=4, max_num_batched_tokens=32,
              max_pending_requests=64, decode_execution="cuda_graph")
    engine = llm.engine
    shared = helpers.random_tokens(vocab, 12, seed=77)
    submitted = {}
    for index in range(30):
        prompt = (shared if index % 3 == 0 else []) + helpers.random_tokens(vocab, rng.randint(1, 40), seed=1000 + index)
        params = SamplingParams(temperature=rng.choice([0.0, 0.0, 0.7]), top_k=rng.choice([0, 0, 5]), seed=index,
                                max_new_tokens=rng.randint(1, 20))
        submitted[f"s{index}"] = (prompt, params)
    waiting = list(submitted.items())
    steps = 0
    while waiting or engine.has_unfinished():
        for _ in range(rng.randint(0, 2)):
            if waiting:
                rid, (prompt, params) = waiting.pop(0)
                engine.submit(rid, prompt, params)
        engine.step()
        steps += 1
        assert steps < 3000
    engine.run_until_done()
    assert engine.stats.preemptions > 0 and engine.stats.prefix_hit_tokens > 0
    for rid, (prompt, params) in submitted.items():
        result = engine.finished[rid]
        assert result.finish_reason == "length" and len(result.token_ids) == params.max_new_tokens
        check_against_plain(folder, prompt, result.token_ids, params, "float32", seed=params.seed)
    llm.runtime.manager.check_invariants()
    assert not llm.runtime.manager.requests
