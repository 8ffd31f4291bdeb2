"""Host-side logic of the step function and the cache manager, run on the CPU with plain
PyTorch functions standing in for the kernels: every cutting of a set of requests must give
the logits of the plain implementation."""

from __future__ import annotations

import pytest
import torch

import helpers
import plain_ops


@pytest.fixture
def cpu_runtime(monkeypatch, tmp_path):
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import EngineConfig
    from miniserve_b200.engine import runtime as runtime_module

    plain_ops.install(monkeypatch)
    monkeypatch.setattr(runtime_module, "require_device", lambda device: torch.device("cpu"))
    monkeypatch.setattr(runtime_module.kernels, "library", lambda: None)
    monkeypatch.setattr(torch.cuda, "set_device", lambda device: None)

    def build(name, num_pages, page_size=16, dtype="float32", max_seqs=4, prefix_cache=False):
        folder = helpers.make_folder(tmp_path, name, seed=1)
        runtime = runtime_module.build_runtime(folder, EngineConfig(
            dtype=dtype, kv_block_size=page_size, num_kv_blocks=num_pages, max_num_seqs=max_seqs,
            enable_prefix_cache=prefix_cache, device="cpu", decode_execution="eager"))
        return folder, runtime
    return build


def replay(runtime, steps):
    from miniserve_b200.trace import TraceSession

    session, outputs = TraceSession(runtime), {}
    for record in steps:
        outputs[record["step"]] = session.run(record).double()
        runtime.manager.check_invariants()
    return outputs


@pytest.mark.parametrize("name,page_size", [("a", 16), ("b", 8), ("c", 4), ("f", 8)])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_cuttings_match_plain_on_cpu(cpu_runtime, name, page_size, cutting):
    vocab = helpers.TINY[name]["vocab_size"]
    requests = {f"r{i}": helpers.random_tokens(vocab, n, seed=10 + i) for i, n in enumerate((1, 7, 16, 33, 50))}
    steps = {"whole": helpers.cut_whole, "tail": lambda r: helpers.cut_decode_tail(r, 12),
             "portions": helpers.cut_portions, "mixed": helpers.cut_mixed}[cutting](requests)
    pages = (helpers.max_live_tokens(steps, granule=page_size * 2) + page_size - 1) // page_size
    folder, runtime = cpu_runtime(name, pages, page_size)
    got = helpers.collect(steps, replay(runtime, steps))
    for rid, tokens in requests.items():
        expected = helpers.oracle_logits(folder, tokens)
        assert sorted(got[rid]) == list(range(len(tokens)))
        for position, row in got[rid].items():
            assert torch.allclose(row, expected[position], atol=1e-4, rtol=1e-4), (rid, position)
    assert not runtime.manager.requests
    assert all(a.free_count == a.num_pages for a in runtime.manager.allocators)


@pytest.mark.parametrize("name,page_size", [("a", 16), ("b", 8)])
def test_requests_sharing_a_prefix_on_cpu(cpu_runtime, name, page_size):
    """Pages attached from the prefix cache instead of computed: the bookkeeping of the trace session and the
    cache manager, with the logits of every later position against the plain implementation."""
    folder, runtime = cpu_runtime(name, 160 // page_size, page_size, prefix_cache=True)
    sequences, got = helpers.run_shared_prefix_trace(runtime, helpers.TINY[name]["vocab_size"], page_size)
    for rid, rows in got.items():
        expected = helpers.oracle_logits(folder, sequences[rid])
        for position, row in rows.items():
            assert torch.allclose(row, expected[position], atol=1e-4, rtol=1e-4), (rid, position)
    assert all(a.free_count + len(runtime.manager.prefix.entries) == a.num_pages for a in runtime.manager.allocators)


def test_many_requests_live_at_once_on_cpu(cpu_runtime):
    """The cutting that the GPU tests use for 8 to 64 rows, at 9 rows: host-side batch building for many rows."""
    import random

    rng = random.Random(3)
    vocab = helpers.TINY["b"]["vocab_size"]
    prompt_lens = {f"m{i}": rng.randrange(1, 20) for i in range(9)}
    requests = {rid: helpers.random_tokens(vocab, n + 4, seed=70 + i) for i, (rid, n) in enumerate(prompt_lens.items())}
    steps = helpers.cut_many_live(requests, prompt_lens, seed=3)
    pages = (helpers.max_live_tokens(steps, granule=8) + 7) // 8
    folder, runtime = cpu_runtime("b", pages, 8, max_seqs=9)
    got = helpers.collect(steps, replay(runtime, steps))
    for rid, tokens in requests.items():
        expected = helpers.oracle_logits(folder, tokens)
        assert sorted(got[rid]) == list(range(prompt_lens[rid] - 1, len(tokens)))
        for position, row in got[rid].items():
            assert torch.allclose(row, expected[position], atol=1e-4, rtol=1e-4), (rid, position)
    assert all(a.free_count == a.num_pages for a in runtime.manager.allocators)
