"""Loads a model's tensors from safetensors files by tensor name.

Contract (after miniserve/model/loader.py:105-217): the files are those the single
``*.safetensors.index.json`` names, else every ``*.safetensors`` of the folder; a name may
appear in one file only; the set of names must be exactly what the model declares (names the
architecture marks optional may be present) and every shape must match.  Everything that is
wrong is collected and raised as **one** :class:`WeightLoadError` that lists the missing
names, the unexpected names and the wrong shapes.

Kept types: a ``matrix`` takes the compute type (bfloat16 stays bfloat16; float32 compute
widens exactly); a ``vector`` stored in 32 bits stays float32 even when computing in
bfloat16; a ``table`` of integers becomes int32.  When the output matrix is tied to the
embedding and the checkpoint still stores it, the stored copy must equal the embedding bit for
bit (loader.py:132-152).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Iterable, Sequence, Union

import torch

from ..parts.base import ParamSpec


class WeightLoadError(RuntimeError):
    """The checkpoint does not fit the model; lists everything that is wrong."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str], wrong_shapes: Sequence[str],
                 other: Sequence[str] = ()) -> None:
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shapes, self.other = list(wrong_shapes), list(other)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): {self.missing}")
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): {self.unexpected}")
        if self.wrong_shapes:
            lines.append(f"  wrong shapes ({len(self.wrong_shapes)}): {self.wrong_shapes}")
        for item in self.other:
            lines.append(f"  {item}")
        super().__init__("\n".join(lines))


@dataclass
class WeightLoadReport:
    folder: str
    loaded_tensors: int = 0
    source_bytes: int = 0
    source_dtype_counts: dict[str, int] = field(default_factory=dict)
    kept_float32: list[str] = field(default_factory=list)


def weight_files(folder: Path) -> list[Path]:
    index_files = sorted(folder.glob("*.safetensors.index.json"))
    if len(index_files) > 1:
        raise RuntimeError(f"{folder} holds more than one safetensors index")
    if index_files:
        weight_map = json.loads(index_files[0].read_text(encoding="utf-8")).get("weight_map")
        if not isinstance(weight_map, dict) or not weight_map:
            raise ValueError(f"{index_files[0]} has no non-empty weight_map")
        files = [folder / name for name in sorted(set(weight_map.values()))]
    else:
        files = sorted(folder.glob("*.safetensors"))
    missing = [str(path) for path in files if not path.is_file()]
    if not files or missing:
        raise FileNotFoundError(f"no safetensors files in {folder}" if not files else f"missing shards: {missing}")
    return files


def kept_dtype(spec: ParamSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.kind == "table":
        return torch.int32
    if spec.kind == "vector" and stored in (torch.float32, torch.float64):
        return torch.float32
    return compute


def load_tensors(folder: Union[str, Path], specs: Iterable[ParamSpec], compute_dtype: torch.dtype,
                 device: Union[str, torch.device], optional_names: Sequence[str] = (),
                 tied: Sequence[tuple[str, str]] = ()) -> tuple[dict[str, torch.Tensor], WeightLoadReport]:
    """``{name: tensor on device}`` for ``specs``, or one error that lists every mismatch.

    ``tied`` pairs ``(optional stored name, name it must equal)`` are compared bit for bit when
    the optional name is present.
    """
    from safetensors import safe_open

    folder = Path(folder)
    specs = list(specs)
    expected = {spec.name: spec for spec in specs}
    report = WeightLoadReport(folder=str(folder))
    locations: dict[str, Path] = {}
    shapes: dict[str, tuple[int, ...]] = {}
    other: list[str] = []
    for path in weight_files(folder):
        report.source_bytes += path.stat().st_size
        with safe_open(path, framework="pt", device="cpu") as handle:
            for key in handle.keys():
                if key in locations:
                    other.append(f"tensor {key!r} appears in {locations[key].name} and in {path.name}")
                    continue
                locations[key] = path
                shapes[key] = tuple(handle.get_slice(key).get_shape())

    missing = sorted(set(expected) - set(locations))
    unexpected = sorted(set(locations) - set(expected) - set(optional_names))
    wrong = [f"{name}: stored {shapes[name]}, model {tuple(spec.shape)}"
             for name, spec in expected.items() if name in shapes and shapes[name] != tuple(spec.shape)]
    if missing or unexpected or wrong or other:
        raise WeightLoadError(missing, unexpected, wrong, other)

    tensors: dict[str, torch.Tensor] = {}
    handles = {}
    try:
        for name, spec in expected.items():
            path = locations[name]
            if path not in handles:
                handles[path] = safe_open(path, framework="pt", device="cpu").__enter__()
            stored = handles[path].get_tensor(name)
            report.source_dtype_counts[str(stored.dtype)] = report.source_dtype_counts.get(str(stored.dtype), 0) + 1
            target = kept_dtype(spec, stored.dtype, compute_dtype)
            if target == torch.float32 and compute_dtype != torch.float32:
                report.kept_float32.append(name)
            tensors[name] = stored.to(device=device, dtype=target).contiguous()
            report.loaded_tensors += 1
        for stored_name, same_as in tied:
            if stored_name in locations and stored_name not in expected:
                path = locations[stored_name]
                if path not in handles:
                    handles[path] = safe_open(path, framework="pt", device="cpu").__enter__()
                a = handles[path].get_tensor(stored_name)
                b = handles[locations[same_as]].get_tensor(same_as)
                if a.shape != b.shape or a.dtype != b.dtype or not torch.equal(a, b):
                    raise WeightLoadError([], [], [], [
                        f"{stored_name} is stored although it is tied to {same_as}, and the two differ"])
    finally:
        for handle in handles.values():
            handle.__exit__(None, None, None)
    return tensors, report
