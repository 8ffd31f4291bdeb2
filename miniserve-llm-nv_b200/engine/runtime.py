"""Builds the pieces of a running engine from a model folder: model, weights, cache, step function.

The recipe of miniserve/api/bootstrap.py:40-183 without the service around it: read the
configuration, pick the model through the registry, load the weights strictly, size and
allocate the page pools once, wire the cache manager and the step function.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Optional, Union

import torch

from .. import kernels
from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..config.engine_config import EngineConfig
from ..config.registry import load_model_config, resolve_architecture
from ..parts.model import DecoderModel
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensors_on_device
from .step import StepFunction

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}
log = logging.getLogger("miniserve_b200")


@dataclass
class Runtime:
    config: object
    engine_config: EngineConfig
    model: DecoderModel
    storage: CacheStorage
    manager: CacheManager
    step_function: StepFunction
    max_model_len: int
    load_report: object
    attention_kernels: list = field(default_factory=list)    # per paged cache group: what kernels.attention_kernels says


def require_device(device: str) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: this engine runs on an NVIDIA B200 only and has no CPU path")
    dev = torch.device(device)
    major, minor = torch.cuda.get_device_capability(dev)
    if major != 10:
        raise RuntimeError(f"device {dev} has compute capability {major}.{minor}; the kernels are built for sm_100a")
    return dev


def build_runtime(model_dir: Union[str, Path, None], engine_config: Optional[EngineConfig] = None, *,
                  config_dict: Optional[dict] = None, weights_seed: Optional[int] = None) -> Runtime:
    """Builds a runtime from a model folder, or (``model_dir=None``) from a ``config.json`` mapping with
    random weights drawn on the device from ``weights_seed`` (for benchmarks of real sizes, where writing
    and reading gigabytes of random numbers would only cost time)."""
    engine_config = engine_config or EngineConfig()
    engine_config.validate()
    device = require_device(engine_config.device)
    torch.cuda.set_device(device)
    kernels.library()          # build or load the CUDA library now; fail here if that is impossible
    dtype = _DTYPES[engine_config.dtype]

    if model_dir is not None:
        architecture, config = load_model_config(model_dir)
    else:
        architecture = resolve_architecture(config_dict)
        config = architecture.config_class.from_dict(config_dict)
    spec = architecture.build_spec(config)
    model = DecoderModel(spec, dtype, device)
    if model_dir is not None:
        tied = [(name, spec.embedding_name) for name in spec.optional_names] if spec.output_name is None else []
        tensors, report = load_tensors(model_dir, model.param_specs(), dtype, device, spec.optional_names, tied)
    else:
        tensors, report = random_tensors_on_device(model.param_specs(), weights_seed or 0, dtype, device), None
    model.load(tensors)
    del tensors

    max_model_len = engine_config.max_model_len or spec.max_positions
    if max_model_len > spec.max_positions:
        raise ValueError(f"max_model_len {max_model_len} exceeds the model's position limit {spec.max_positions}")
    page_size = engine_config.kv_block_size
    num_pages = engine_config.num_kv_blocks
    if num_pages is None:
        per_page = max(CacheStorage.bytes_per_page(model.cache_groups, page_size, dtype), 1)
        free, _total = torch.cuda.mem_get_info(device)
        by_memory = int(free * engine_config.gpu_memory_utilization) // per_page
        by_need = engine_config.max_num_seqs * ((max_model_len + page_size - 1) // page_size)
        num_pages = max(1, min(by_memory, by_need))
    storage = CacheStorage(model.cache_groups, page_size, num_pages, engine_config.max_num_seqs, dtype, device)
    origin = Path(model_dir).resolve() if model_dir is not None else f"random:{weights_seed}"
    namespace = f"{origin};{engine_config.dtype};page={page_size}"
    manager = CacheManager(model.cache_groups, page_size, num_pages, engine_config.max_num_seqs,
                           engine_config.enable_prefix_cache, engine_config.prefix_cache_max_entries, namespace)
    step_function = StepFunction(model, storage, manager, max_model_len,
                                 use_graphs=engine_config.decode_execution == "cuda_graph")
    resolved = replace(engine_config, max_model_len=max_model_len, num_kv_blocks=num_pages)
    chosen = _report_attention_kernels(model, dtype, page_size)
    return Runtime(config, resolved, model, storage, manager, step_function, max_model_len, report, chosen)


def _report_attention_kernels(model: DecoderModel, dtype: torch.dtype, page_size: int) -> list:
    """Says once per build which attention kernel each paged cache group gets, loudly where bfloat16 falls back
    to the general float32-arithmetic kernel (right, but many times slower than the tensor-core kernels)."""
    from ..parts.base import PagedKVNeed

    chosen = []
    for index, run in enumerate(model.spec.order):
        plan = model.run_caches[index]
        mixer = model.blocks[run.layer].mixer
        if plan is None or not plan.writable or plan.slot != 0 or not isinstance(model.cache_groups[plan.group].need, PagedKVNeed):
            continue
        need = model.cache_groups[plan.group].need
        n_q = getattr(mixer, "num_heads", need.num_kv_heads)
        modified = bool(getattr(mixer, "score_softcap", None)) or getattr(mixer, "score_bias_slopes", None) is not None
        names = kernels.attention_kernels(dtype, need.head_dim, n_q, need.num_kv_heads, page_size, modified)
        chosen.append(dict(group=plan.group, head_dim=need.head_dim, window=need.window, **names))
        slow = dtype == torch.bfloat16 and "general" in names.values()
        log.log(logging.WARNING if slow else logging.INFO,
                "cache group %d (head size %d, %d/%d heads, pages of %d%s): decode steps on the %s kernel, prompt "
                "portions on the %s kernel%s", plan.group, need.head_dim, n_q, need.num_kv_heads, page_size,
                f", window {need.window}" if need.window else "", names["decode"], names["prompt"],
                " (no tensor-core kernel is built for this head size or for modified scores)" if slow else "")
    return chosen
