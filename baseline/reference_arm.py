"""The reference arm of ``bench.py``: MiniServe-LLM-NV itself, unmodified, from ``baseline/_ref``.

Install (once, offline; from a writable copy of the project, because its build writes into the source
tree, with a wheel directory for the build tools):

    python -m pip install --no-index --no-build-isolation --no-deps --find-links <wheel directory> \
        --target baseline/_ref <writable copy of MiniServe-LLM-NV>

The engine is wired exactly as MiniServe's own start-up wires it
(miniserve/api/bootstrap.py:85-163: ModelConfig, EngineConfig, Qwen3ForCausalLM, KVLayout,
PagedKVCacheBackend, KVCacheManager, CudaPagedDecodeAttention, ModelExecutor, EngineCore) with
its fastest combination that its capability check accepts (CUDA paged decode kernel, CUDA RMSNorm,
batched decode replayed from its batched CUDA graph, its reference sampler), minus the tokenizer and the model lock, which a model of
random weights does not have.  Requests go in through ``EngineCore.submit`` and steps through
``EngineCore.step_multi``, as in its own benchmark driver (miniserve/benchmark/compare_hf.py:384-424).
None of this repository's model, kernels or engine is involved.
"""

from __future__ import annotations

import json
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent


def run(model: dict, batch: int, context: int, steps: int, warmup: int, page_size: int) -> dict:
    sys.path.insert(0, str(HERE / "_ref"))
    import torch
    from miniserve.attention.cuda_paged import CudaPagedDecodeAttention
    from miniserve.config.engine_config import EngineConfig
    from miniserve.config.model_config import ModelConfig
    from miniserve.config.runtime_config import RuntimeConfig
    from miniserve.engine.core import EngineCore
    from miniserve.engine.executor import ModelExecutor
    from miniserve.engine.request import EngineRequest, SamplingParams
    from miniserve.kv.layout import KVLayout
    from miniserve.kv.manager import KVCacheManager
    from miniserve.kv.paged import PagedKVCacheBackend
    from miniserve.model.qwen3 import Qwen3ForCausalLM

    device = torch.device("cuda:0")
    torch.manual_seed(0)
    model_config = ModelConfig.from_hf_config(model, model_id_or_path="random-weights", dtype="bfloat16",
                                              max_model_len=context)
    blocks = batch * ((context + page_size - 1) // page_size) + 64
    engine_config = EngineConfig(
        max_num_seqs=batch, max_num_batched_tokens=context, kv_block_size=page_size, num_kv_blocks=blocks,
        enable_prefix_cache=False, enable_chunked_prefill=False, attention_backend="cuda_paged", kv_backend="paged",
        rmsnorm_backend="cuda", decode_execution="cuda_graph", decode_batching="batched", batched_graph=True,
        sampling_execution="reference", max_pending_requests=max(batch, 4))
    runtime_config = RuntimeConfig(model_config, engine_config)
    runtime_config.validate_capabilities()
    network = Qwen3ForCausalLM(model_config, device=device, dtype=torch.bfloat16)   # its own default random init
    network.eval()
    layout = KVLayout(model_config.num_hidden_layers, context, model_config.num_key_value_heads, model_config.head_dim,
                      torch.bfloat16, device, num_blocks=blocks, block_size=page_size)
    backend = PagedKVCacheBackend(layout, max_sequences=batch)
    manager = KVCacheManager(backend, prefix_cache=None)
    attention = CudaPagedDecodeAttention(backend)
    core = EngineCore(runtime_config, ModelExecutor(network, attention, retain_last_logits=False,
                                                    validate_logits_finite=False, sampling_execution="reference"),
                      kv_manager=manager)

    generator = torch.Generator().manual_seed(1)
    # MiniServe runs one whole prompt per step while the earlier requests already decode: the first request
    # has decoded `batch` tokens before the last prompt is in, so every request gets that many tokens more
    new_tokens = steps + warmup + batch + 2
    prompt_len = context - new_tokens
    with torch.no_grad():
        for index in range(batch):
            prompt = tuple(torch.randint(0, model["vocab_size"], (prompt_len,), generator=generator).tolist())
            core.submit(EngineRequest(f"ref-{index}", prompt, SamplingParams(max_new_tokens=new_tokens, stop_token_ids=()),
                                      time.monotonic_ns()))
        prefill_started = time.perf_counter()
        guard = 0
        while True:                                       # prompts first (one whole prompt per step)
            views = core.step_multi()
            guard += 1
            plan = core.last_plan
            if plan is not None and not plan.prefill_items and plan.decode_items and len(plan.decode_items) == batch:
                break
            if guard > 4 * batch + 16:
                raise RuntimeError("the reference engine did not reach steady decoding")
        torch.cuda.synchronize()
        prefill_seconds = time.perf_counter() - prefill_started
        for _ in range(max(warmup - 1, 0)):
            core.step_multi()
        torch.cuda.synchronize()
        started = time.perf_counter()
        for _ in range(steps):
            core.step_multi()
        torch.cuda.synchronize()
        seconds = (time.perf_counter() - started) / steps
    histogram = getattr(core, "decode_forward_row_histogram", None)     # rows per decode forward: {8: n} if batched
    if callable(histogram):
        histogram = histogram()
    return {"seconds_per_step": seconds, "prefill_seconds_total": prefill_seconds,
            "decode_rows": {str(k): v for k, v in dict(histogram).items()} if histogram else None}


def main(model: dict, batch: int, context: int, steps: int, warmup: int, page_size: int) -> dict:
    marker = HERE / "_ref" / "miniserve"
    if not marker.is_dir():
        return {"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref "
                "(pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <copy of the reference>)"}
    try:
        result = run(model, batch, context, steps, warmup, page_size)
    except Exception as error:  # the line must be printed whatever the reference does
        text = " ".join(str(error).split())[:300]
        return {"impl": "reference", "unavailable": f"the reference failed on this GPU: {type(error).__name__}: {text}"}
    seconds = result["seconds_per_step"]
    return {"impl": "reference", "value": round(batch / seconds, 1), "ms_per_step": round(seconds * 1e3, 4),
            "prefill_seconds_total": round(result["prefill_seconds_total"], 2), "decode_rows": result["decode_rows"]}
