"""The engine against the plain implementation on the GPU, in float32 and in bfloat16: the
same requests whole, with the last tokens decoded one by one, in portions of changing size,
and mixed with other requests in a pool so small that pages are used again; through the
engine in-process and through ``bin/trace_run`` as a user runs it."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent

CUTTINGS = {
    "whole": helpers.cut_whole,
    "tail": lambda r: helpers.cut_decode_tail(r, 32),
    "portions": helpers.cut_portions,
    "mixed": helpers.cut_mixed,
}
LENGTHS = (1, 7, 16, 33, 65, 150)


def build(folder, dtype, num_pages, page_size):
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import EngineConfig
    from miniserve_b200.engine.runtime import build_runtime

    return build_runtime(folder, EngineConfig(dtype=dtype, kv_block_size=page_size, num_kv_blocks=num_pages,
                                              max_num_seqs=4, enable_prefix_cache=False, decode_execution="eager"))


def replay(runtime, steps):
    from miniserve_b200.engine.step import StepEntry

    outputs, manager = {}, runtime.manager
    for record in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in record["entries"]]
        for entry in entries:
            if entry.request_id not in manager.requests:
                runtime.storage.reset_slot(manager.admit(entry.request_id).slot, 0.0, 1.0, 0, 0)
        reservation = manager.prepare([(e.request_id, len(e.tokens)) for e in entries])
        outputs[record["step"]] = runtime.step_function.run(entries, reservation).double().cpu()
        manager.commit(reservation)
        for rid in record["end"]:
            manager.release(rid)
    manager.check_invariants()
    return outputs


def error_bounds(dtype, expected):
    scale = float(expected.abs().max())
    if dtype == "float32":
        return 2e-5 * max(scale, 1.0)
    return 3e-2 * max(scale, 1.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("a", 16), ("b", 8), ("c", 4), ("d", 16)])
@pytest.mark.parametrize("cutting", list(CUTTINGS))
def test_cuttings_match_plain(tmp_path, dtype, name, page_size, cutting):
    vocab = helpers.TINY[name]["vocab_size"]
    requests = {f"r{i}": helpers.random_tokens(vocab, n, seed=100 + i) for i, n in enumerate(LENGTHS)}
    steps = CUTTINGS[cutting](requests)
    folder = helpers.make_folder(tmp_path, name, seed=2)
    pages = (helpers.max_live_tokens(steps, granule=2 * page_size) + page_size - 1) // page_size
    runtime = build(folder, dtype, pages, page_size)
    got = helpers.collect(steps, replay(runtime, steps))
    worst = 0.0
    for rid, tokens in requests.items():
        expected = helpers.oracle_logits(folder, tokens)
        bound = error_bounds(dtype, expected)
        assert sorted(got[rid]) == list(range(len(tokens)))
        for position, row in got[rid].items():
            error = float((row - expected[position]).abs().max())
            worst = max(worst, error / bound)
            assert error <= bound, (rid, position, error, bound)
    assert all(a.free_count == a.num_pages for a in runtime.manager.allocators)
    print(f"worst error / bound = {worst:.3f}")


REAL = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=2048, intermediate_size=6144,
            num_hidden_layers=2, num_attention_heads=16, num_key_value_heads=8, head_dim=128, vocab_size=151936,
            max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, attention_dropout=0.0,
            hidden_act="silu", attention_bias=False, tie_word_embeddings=True)
_real: dict = {}


@pytest.fixture(scope="module")
def real_model(tmp_path_factory):
    """Two layers of Qwen3-1.7B's sizes (full vocabulary, tied) with random weights, and the plain logits
    of three short requests; made once for the tests below."""
    if not _real:
        import miniserve_b200  # noqa: F401
        from miniserve_b200.weights import write_random_model

        folder = write_random_model(tmp_path_factory.mktemp("real") / "model", REAL, seed=3)
        requests = {f"q{i}": helpers.random_tokens(REAL["vocab_size"], n, seed=900 + i) for i, n in enumerate((5, 70, 41))}
        _real.update(folder=folder, requests=requests,
                     expected={rid: helpers.oracle_logits(folder, tokens) for rid, tokens in requests.items()})
    return _real


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["tail", "mixed"])
def test_layers_of_real_size(real_model, dtype, cutting):
    """Qwen3-1.7B's layer sizes (hidden 2,048, 16 / 8 heads of 128, intermediate 6,144, 151,936 tokens):
    the kernels that the benchmark times (tcgen05 attention of prompt portions, split-key decode attention,
    the few-row products in whichever form was measured fastest, the output matrix) against the plain
    implementation, with 64-token pages as there."""
    requests = real_model["requests"]
    steps = CUTTINGS[cutting](requests)
    pages = (helpers.max_live_tokens(steps, granule=128) + 63) // 64
    runtime = build(real_model["folder"], dtype, pages, 64)
    got = helpers.collect(steps, replay(runtime, steps))
    for rid, tokens in requests.items():
        expected = real_model["expected"][rid]
        bound = error_bounds(dtype, expected)
        assert sorted(got[rid]) == list(range(len(tokens)))
        for position, row in got[rid].items():
            assert float((row - expected[position]).abs().max()) <= bound, (rid, position)
    assert all(a.free_count == a.num_pages for a in runtime.manager.allocators)


def test_generation_at_real_size_graph_against_eager(real_model):
    """Greedy tokens at Qwen3-1.7B's layer sizes: replayed graphs with decoding one step ahead (the path the
    benchmark times) against eager steps, and the first tokens against the plain implementation."""
    import plain_qwen3 as plain
    from miniserve_b200.engine.llm import LLM
    from miniserve_b200.sampling import SamplingParams

    prompts = [tokens for tokens in real_model["requests"].values()]
    params = SamplingParams(temperature=0.0, max_new_tokens=12)
    outcomes = {}
    for execution, look_ahead in (("eager", False), ("cuda_graph", True)):
        llm = LLM(str(real_model["folder"]), dtype="bfloat16", kv_block_size=64, num_kv_blocks=16, max_num_seqs=4,
                  max_model_len=256, decode_execution=execution, decode_look_ahead=look_ahead)
        outcomes[execution] = [r.token_ids for r in llm.generate(prompts, params)]
        del llm
        torch.cuda.empty_cache()
    config, weights = plain.load_folder(real_model["folder"], torch.float64)
    for prompt, eager, graph in zip(prompts, outcomes["eager"], outcomes["cuda_graph"]):
        tokens = list(prompt)
        for index, (a, b) in enumerate(zip(eager, graph)):
            if a != b or index < 3:
                # a difference between the two paths, like one from the plain rule, must be a near tie
                logits = plain.plain_logits(tokens, weights, config)[-1]
                limit = 4e-2 * max(1.0, float(logits.abs().max()))
                best = int(logits.argmax())
                assert float(logits[best] - logits[a]) <= limit and float(logits[best] - logits[b]) <= limit, (index, a, b, best)
            if a != b:
                break                      # after a tie broken differently the sequences are different ones
            tokens.append(a)


@pytest.mark.parametrize("name,page_size", [("d", 16), ("b", 8)])
def test_whole_prompts_through_the_tcgen05_products(tmp_path, monkeypatch, name, page_size):
    """The library's own tcgen05 matrix product in place of cuBLAS for portions of 128 rows and more."""
    import miniserve_b200  # noqa: F401
    from miniserve_b200 import kernels

    monkeypatch.setattr(kernels, "USE_TCGEN05_GEMM", True)
    vocab = helpers.TINY[name]["vocab_size"]
    requests = {f"r{i}": helpers.random_tokens(vocab, n, seed=300 + i) for i, n in enumerate((128, 150, 333))}
    steps = helpers.cut_whole(requests)
    folder = helpers.make_folder(tmp_path, name, seed=2)
    runtime = build(folder, "bfloat16", (400 + page_size - 1) // page_size, page_size)
    before = kernels.launch_count
    got = helpers.collect(steps, replay(runtime, steps))
    kernels.check_device_errors(runtime.model.device)
    assert kernels.launch_count > before
    for rid, tokens in requests.items():
        expected = helpers.oracle_logits(folder, tokens)
        bound = error_bounds("bfloat16", expected)
        for position, row in got[rid].items():
            assert float((row - expected[position]).abs().max()) <= bound, (rid, position)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("b", 8), ("d", 16)])
def test_long_decoding_and_first_tokens(tmp_path, dtype, name, page_size):
    """A sequence decoded one token at a time from its very first token, across many page edges."""
    vocab = helpers.TINY[name]["vocab_size"]
    tokens = helpers.random_tokens(vocab, 300, seed=77)
    steps = [{"step": i, "entries": [{"id": "r", "tokens": [t], "want": [0]}], "end": ["r"] if i == 299 else []}
             for i, t in enumerate(tokens)]
    folder = helpers.make_folder(tmp_path, name, seed=2)
    runtime = build(folder, dtype, (300 + page_size - 1) // page_size, page_size)
    got = helpers.collect(steps, replay(runtime, steps))["r"]
    expected = helpers.oracle_logits(folder, tokens)
    bound = error_bounds(dtype, expected)
    errors = [float((got[p] - expected[p]).abs().max()) for p in range(300)]
    assert max(errors) <= bound, (errors.index(max(errors)), max(errors), bound)
    assert max(errors[:3]) <= bound                       # the first tokens of a sequence


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """bin/trace_run as a subprocess: protocol, files, page reuse."""
    name, vocab = "b", helpers.TINY["b"]["vocab_size"]
    requests = {f"q{i}": helpers.random_tokens(vocab, n, seed=200 + i) for i, n in enumerate((40, 3, 70, 25, 90, 64))}
    steps = helpers.cut_mixed(requests, seed=5)
    folder = helpers.make_folder(tmp_path, name, seed=3)
    out_dir = tmp_path / f"out_{dtype}"
    max_tokens = helpers.max_live_tokens(steps, granule=64)
    process = subprocess.Popen(
        [sys.executable, str(REPO / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
         "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for record in steps:
        process.stdin.write(json.dumps(record) + "\n")
        process.stdin.flush()
        assert process.stdout.readline().strip() == f"done {record['step']}"
    process.stdin.close()
    assert process.wait(timeout=120) == 0
    outputs = {}
    for record in steps:
        wanted = sum(len(e["want"]) for e in record["entries"])
        path = out_dir / f"{record['step']}.f32"
        if wanted:
            outputs[record["step"]] = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(wanted, vocab)).double()
        else:
            assert not path.exists()
    got = helpers.collect(steps, outputs)
    for rid, tokens in requests.items():
        expected = helpers.oracle_logits(folder, tokens)
        bound = error_bounds(dtype, expected)
        for position, row in got[rid].items():
            assert float((row - expected[position]).abs().max()) <= bound, (rid, position)
