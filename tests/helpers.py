"""Tiny configurations, model folders and trace cuttings shared by the tests."""

from __future__ import annotations

import random
from pathlib import Path

import torch

import plain_qwen3 as plain

# Two configurations of the architecture that differ in every size and option.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64, intermediate_size=128,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256,
              max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=10000.0, attention_dropout=0.0,
              hidden_act="silu", attention_bias=False, tie_word_embeddings=True)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=96, intermediate_size=224,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=32, vocab_size=384,
              max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=1000000.0, attention_dropout=0.0,
              hidden_act="silu", attention_bias=False, tie_word_embeddings=False)
# A third one with awkward sizes: width and vocabulary that are no power of two, one kv head, head size 48.
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=72, intermediate_size=200,
              num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=1, head_dim=48, vocab_size=331,
              max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=50000.0, attention_dropout=0.0,
              hidden_act="silu", attention_bias=False, tie_word_embeddings=True)
# A fourth with the head size of real checkpoints' smaller siblings (64), four query heads per kv head.
TINY_D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=128, intermediate_size=192,
              num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64, vocab_size=500,
              max_position_embeddings=4096, rms_norm_eps=1e-6, rope_theta=1000000.0, attention_dropout=0.0,
              hidden_act="silu", attention_bias=False, tie_word_embeddings=False)
# Head sizes that the configuration allows (even) but no tensor-core kernel is built for: 24 with as many kv heads as
# query heads, 40 with an intermediate size that is no multiple of eight (gate and up rows are then not interleaved).
TINY_E = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=80, intermediate_size=144,
              num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5, head_dim=24, vocab_size=211,
              max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=10000.0, attention_dropout=0.0,
              hidden_act="silu", attention_bias=False, tie_word_embeddings=True)
TINY_F = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=56, intermediate_size=100,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=40, vocab_size=300,
              max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=500000.0, attention_dropout=0.0,
              hidden_act="silu", attention_bias=False, tie_word_embeddings=False)
TINY = {"a": TINY_A, "b": TINY_B, "c": TINY_C, "d": TINY_D, "e": TINY_E, "f": TINY_F}


def make_folder(tmp_path: Path, name: str, seed: int = 0, stored_dtype: str = "bfloat16", matrix_std: float = 0.05) -> Path:
    import miniserve_b200  # noqa: F401
    from miniserve_b200.weights import write_random_model

    folder = Path(tmp_path) / f"tiny_{name}_{seed}_{stored_dtype}"
    if not folder.exists():
        write_random_model(folder, TINY[name], seed, stored_dtype, matrix_std)
    return folder


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(length)]


def oracle_logits(folder: Path, tokens: list[int]) -> torch.Tensor:
    """float64 logits of the plain implementation for one whole sequence."""
    config, weights = plain.load_folder(folder, torch.float64)
    return plain.plain_logits(tokens, weights, config)


# --------------------------------------------------------------------------- cuttings of a set of requests


def cut_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, one step each, all logits wanted."""
    steps = []
    for step, (rid, tokens) in enumerate(requests.items()):
        steps.append({"step": step, "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}],
                      "end": [rid]})
    return steps


def cut_decode_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, then its last ``tail`` tokens one by one."""
    steps, step = [], 0
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": step, "entries": [{"id": rid, "tokens": tokens[:head], "want": list(range(head))}], "end": []})
        step += 1
        for index in range(head, len(tokens)):
            steps.append({"step": step, "entries": [{"id": rid, "tokens": [tokens[index]], "want": [0]}],
                          "end": [rid] if index == len(tokens) - 1 else []})
            step += 1
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def cut_portions(requests: dict[str, list[int]], seed: int = 0, sizes=(2, 3, 5, 7, 16, 17, 31, 64)) -> list[dict]:
    """Each request in portions of changing size, down to two tokens."""
    rng = random.Random(seed)
    steps, step = [], 0
    for rid, tokens in requests.items():
        cursor = 0
        while cursor < len(tokens):
            take = min(rng.choice(sizes), len(tokens) - cursor)
            steps.append({"step": step, "entries": [{"id": rid, "tokens": tokens[cursor:cursor + take],
                                                     "want": list(range(take))}],
                          "end": [rid] if cursor + take == len(tokens) else []})
            cursor += take
            step += 1
    return steps


def cut_mixed(requests: dict[str, list[int]], seed: int = 0, max_live: int = 4) -> list[dict]:
    """Up to ``max_live`` live requests; portions of some beside single tokens of others; requests
    end at different times so that their pages are handed to later ones."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, list] = {}     # id -> [tokens, cursor, prompt_part]
    steps, step = [], 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            rid, tokens = waiting.pop(0)
            live[rid] = [tokens, 0, max(1, int(len(tokens) * rng.uniform(0.3, 0.9)))]
        entries, ended = [], []
        for rid, state in list(live.items()):
            tokens, cursor, prompt_part = state
            if rng.random() < 0.15 and len(live) > 1:
                continue                      # left out of this step, goes on later
            if cursor < prompt_part:
                take = min(rng.choice((2, 3, 5, 8, 13, 16, 21)), prompt_part - cursor)
            else:
                take = 1
            take = min(take, len(tokens) - cursor)
            entries.append({"id": rid, "tokens": tokens[cursor:cursor + take], "want": list(range(take))})
            state[1] = cursor + take
            if state[1] == len(tokens):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": step, "entries": entries, "end": ended})
            step += 1
    return steps


def cut_many_live(requests: dict[str, list[int]], prompt_lens: dict[str, int], seed: int = 0, per_step: int = 5) -> list[dict]:
    """All requests live at once: prompts whole, a few per step (the last position wanted), then every request
    decoded token by token, teacher-forced, in steps of single tokens whose live set changes: all of them, the
    first five eighths, every other one in reverse order, a random subset, all again ... until every request
    has had all its tokens.  A step of single tokens is what a captured decode graph replays, so this walks
    the graphs through full buckets, padded buckets and rows that change owner between replays."""
    rng = random.Random(seed)
    ids = list(requests)
    steps, step = [], 0
    for start in range(0, len(ids), per_step):
        entries = [{"id": rid, "tokens": requests[rid][:prompt_lens[rid]], "want": [prompt_lens[rid] - 1]}
                   for rid in ids[start:start + per_step]]
        steps.append({"step": step, "entries": entries, "end": []})
        step += 1
    cursor = {rid: prompt_lens[rid] for rid in ids}
    round_index = 0
    while any(cursor[rid] < len(requests[rid]) for rid in ids):
        alive = [rid for rid in ids if cursor[rid] < len(requests[rid])]
        kind = round_index % 5
        if kind == 1:
            chosen = alive[:max(1, (5 * len(alive) + 7) // 8)]
        elif kind == 2:
            chosen = alive[::2][::-1]
        elif kind == 3:
            chosen = rng.sample(alive, max(1, rng.randrange(len(alive) // 2, len(alive) + 1)))
        else:
            chosen = alive
        entries, ended = [], []
        for rid in chosen:
            entries.append({"id": rid, "tokens": [requests[rid][cursor[rid]]], "want": [0]})
            cursor[rid] += 1
            if cursor[rid] == len(requests[rid]):
                ended.append(rid)
        steps.append({"step": step, "entries": entries, "end": ended})
        step += 1
        round_index += 1
    return steps


def max_live_tokens(steps: list[dict], granule: int = 64) -> int:
    """The --max-tokens a trace needs: most tokens live at once, each request rounded up to ``granule``."""
    held: dict[str, int] = {}
    peak = 0
    for record in steps:
        for entry in record["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum((n + granule - 1) // granule * granule for n in held.values()))
        for rid in record["end"]:
            held.pop(rid, None)
    return peak


WORST_RATIOS: dict[str, float] = {}     # test case -> worst error / bound seen; printed at the end of a run


def note_ratio(case: str, ratio: float) -> None:
    WORST_RATIOS[case] = max(WORST_RATIOS.get(case, 0.0), ratio)


def collect(steps: list[dict], outputs: dict[int, torch.Tensor]) -> dict[str, dict[int, torch.Tensor]]:
    """{request: {position: logits}} from per-step outputs ``[wanted, vocab]``."""
    result: dict[str, dict[int, torch.Tensor]] = {}
    cursor: dict[str, int] = {}
    for record in steps:
        row = 0
        out = outputs.get(record["step"])
        for entry in record["entries"]:
            start = cursor.get(entry["id"], 0)
            for index in entry["want"]:
                result.setdefault(entry["id"], {})[start + index] = out[row]
                row += 1
            cursor[entry["id"]] = start + len(entry["tokens"])
        for rid in record["end"]:
            cursor.pop(rid, None)
    return result


def run_shared_prefix_trace(runtime, vocab: int, page_size: int):
    """Three requests through the trace session of ``runtime`` (built with prefix reuse on): 'p' computes its
    prompt and offers its pages; 'q', arriving while 'p' is live, starts with the same 16 tokens and attaches
    them; 'r' starts with 32 tokens of 'p'.  Checks who holds which pages on the way.  Returns the token
    lists and {request: {position: logits}} of every position that was computed."""
    from miniserve_b200.trace import TraceSession

    shared = random_tokens(vocab, 16, seed=40)
    first = shared + random_tokens(vocab, 21, seed=41)
    second = shared + random_tokens(vocab, 30, seed=42)
    third = list(first[:32]) + random_tokens(vocab, 5, seed=43)
    session, manager = TraceSession(runtime), runtime.manager
    shared_pages = 16 // page_size
    steps = [
        {"step": 0, "entries": [{"id": "p", "tokens": first[:20], "want": list(range(20))}], "cache": ["p"], "end": []},
        # the second request arrives while the first is live: it names the prefix and runs the rest in two portions
        {"step": 1, "entries": [{"id": "p", "tokens": first[20:30], "want": list(range(10))},
                                {"id": "q", "prefix": shared, "tokens": second[16:29], "want": list(range(13))}], "end": []},
        {"step": 2, "entries": [{"id": "p", "tokens": first[30:], "want": list(range(len(first) - 30))},
                                {"id": "q", "tokens": second[29:], "want": list(range(len(second) - 29))}],
         "cache": ["p"], "end": []},
        # by now 32 tokens of the first request are cached: the third attaches all of them
        {"step": 3, "entries": [{"id": "r", "prefix": third[:32], "tokens": third[32:], "want": list(range(5))}],
         "end": ["p", "q", "r"]},
    ]
    outputs = {}
    for record in steps:
        outputs[record["step"]] = session.run(record).double().cpu()
        if record["step"] == 1:
            p, q = manager.requests["p"], manager.requests["q"]
            assert p.tables[0][:shared_pages] == q.tables[0][:shared_pages]
            assert all(manager.allocators[0].refcount(page) == 3 for page in q.tables[0][:shared_pages])   # p, q, the cache
            assert not set(p.tables[0][shared_pages:]) & set(q.tables[0][shared_pages:])
        manager.check_invariants()
    got: dict[str, dict[int, torch.Tensor]] = {"p": {}, "q": {}, "r": {}}
    got["p"].update({i: outputs[0][i] for i in range(20)})
    got["p"].update({20 + i: outputs[1][i] for i in range(10)})
    got["q"].update({16 + i: outputs[1][10 + i] for i in range(13)})
    got["p"].update({30 + i: outputs[2][i] for i in range(len(first) - 30)})
    got["q"].update({29 + i: outputs[2][len(first) - 30 + i] for i in range(len(second) - 29)})
    got["r"].update({32 + i: outputs[3][i] for i in range(5)})
    assert sorted(got["q"]) == list(range(16, len(second))) and sorted(got["p"]) == list(range(len(first)))
    return {"p": first, "q": second, "r": third}, got
