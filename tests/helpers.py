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
TINY = {"a": TINY_A, "b": TINY_B, "c": TINY_C, "d": TINY_D}


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
