"""The Python entry point: ``LLM(model_folder, **engine_options).generate(prompts, sampling_params)``.

Token ids in, token ids out (tokenizers are outside this engine).  The engine options carry
MiniServe's names (``max_model_len``, ``num_kv_blocks``, ``max_num_seqs``, ``kv_block_size``,
``max_num_batched_tokens``, ``max_pending_requests``, ``enable_prefix_cache``,
``enable_chunked_prefill``, ``prefill_chunk_size``, ``decode_execution``); ``decode_look_ahead`` is this
engine's own.
"""

from __future__ import annotations

from typing import Optional, Sequence as Seq, Union

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from .core import Engine, GenerationResult
from .executor import DeviceExecutor
from .runtime import Runtime, build_runtime
from .scheduler import Scheduler


def build_engine(runtime: Runtime) -> Engine:
    config = runtime.engine_config
    budget = config.max_num_batched_tokens or min(runtime.max_model_len, 8192)
    scheduler = Scheduler(max_num_seqs=config.max_num_seqs, max_num_batched_tokens=budget,
                          enable_chunked_prefill=config.enable_chunked_prefill,
                          prefill_chunk_size=config.prefill_chunk_size)
    executor = DeviceExecutor(runtime.step_function, runtime.storage)
    runtime.step_function.capture_decode_graphs(config.max_num_seqs)
    return Engine(runtime.manager, scheduler, executor, vocab_size=runtime.model.spec.vocab_size,
                  max_model_len=runtime.max_model_len, max_pending_requests=config.max_pending_requests,
                  look_ahead=config.decode_look_ahead and config.decode_execution == "cuda_graph")


class LLM:
    def __init__(self, model: str, dtype: str = "bfloat16", **engine_options) -> None:
        self.runtime = build_runtime(model, EngineConfig(dtype=dtype, **engine_options))
        self.engine = build_engine(self.runtime)
        self._counter = 0

    def generate(self, prompts: Seq[Seq[int]],
                 sampling_params: Union[SamplingParams, Seq[SamplingParams], None] = None) -> list[GenerationResult]:
        """Generates for every prompt (a list of token ids); results come back in the order of the prompts."""
        if sampling_params is None:
            sampling_params = SamplingParams()
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = []
        pending = list(zip(prompts, sampling_params))
        limit = self.engine.max_pending_requests
        results: dict[str, GenerationResult] = {}
        while pending or self.engine.has_unfinished():
            while pending and len(self.engine.sequences) < limit:
                prompt, params = pending.pop(0)
                request_id = f"req-{self._counter}"
                self._counter += 1
                self.engine.submit(request_id, prompt, params)
                ids.append(request_id)
            self.engine.run_until_done() if not pending else self.engine.step()
            for request_id in list(self.engine.finished):
                results[request_id] = self.engine.take_result(request_id)
        return [results[request_id] for request_id in ids]
