"""Engine options, named as MiniServe names them (miniserve/config/engine_config.py:16-31).

The switches that chose between backends there (attention, RMSNorm, KV backend, decode
batching) have no counterpart: there is one path.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"                      # "bfloat16" or "float32"
    max_model_len: Optional[int] = None          # default: the model's max_position_embeddings
    max_num_seqs: int = 8                        # live requests (= state slots)
    max_num_batched_tokens: Optional[int] = None  # token budget of a step; default min(max_model_len, 8192)
    kv_block_size: int = 16                      # tokens per page
    num_kv_blocks: Optional[int] = None          # pages per layer group; default: sized from free device memory
    max_pending_requests: int = 64               # admitted plus waiting
    enable_prefix_cache: bool = True
    prefix_cache_max_entries: int = 64
    enable_chunked_prefill: bool = True
    prefill_chunk_size: Optional[int] = None
    decode_execution: str = "cuda_graph"         # "cuda_graph" or "eager"
    decode_look_ahead: bool = True               # with graphs: start the next decode step before reading the last tokens
    gpu_memory_utilization: float = 0.85         # share of free memory given to pages when num_kv_blocks is None
    device: str = "cuda:0"

    def validate(self) -> None:
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be at least 1")
        if self.kv_block_size < 1:
            raise ValueError("kv_block_size must be at least 1")
        if self.num_kv_blocks is not None and self.num_kv_blocks < 1:
            raise ValueError("num_kv_blocks must be at least 1")
        if self.max_model_len is not None and self.max_model_len < 1:
            raise ValueError("max_model_len must be positive")
        if self.max_num_batched_tokens is not None and self.max_num_batched_tokens < 1:
            raise ValueError("max_num_batched_tokens must be positive")
        if self.max_pending_requests < 1:
            raise ValueError("max_pending_requests must be at least 1")
        if self.prefill_chunk_size is not None:
            if self.prefill_chunk_size < 1:
                raise ValueError("prefill_chunk_size must be positive")
            if not self.enable_chunked_prefill:
                raise ValueError("prefill_chunk_size needs enable_chunked_prefill")
            if self.max_num_batched_tokens is not None and self.prefill_chunk_size > self.max_num_batched_tokens:
                raise ValueError("prefill_chunk_size must not exceed max_num_batched_tokens")
        if self.decode_execution not in ("cuda_graph", "eager"):
            raise ValueError("decode_execution must be 'cuda_graph' or 'eager'")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
