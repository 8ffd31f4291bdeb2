"""Seeded random weights: writes a model folder (``config.json`` + ``model.safetensors``).

Every tensor a model declares is drawn in float32 from one generator seeded with ``seed``, in
the order of declaration: matrices (embedding and output included) from ``N(0, std^2)`` with
``std`` 0.02, vectors (norm weights) as ``1 + N(0, 0.1^2)`` so that their position in the
formulas matters, then cast to the stored type.  The same seed gives the same folder.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Union

import torch

from ..config.registry import resolve_architecture
from ..parts.model import DecoderModel

_STORED = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(config_dict: Mapping[str, Any], seed: int, stored_dtype: str = "bfloat16",
                   matrix_std: float = 0.02, vector_std: float = 0.1) -> dict[str, torch.Tensor]:
    architecture = resolve_architecture(config_dict)
    config = architecture.config_class.from_dict(config_dict)
    model = DecoderModel(architecture.build_spec(config), torch.float32, "cpu")
    generator = torch.Generator().manual_seed(int(seed))
    dtype = _STORED[stored_dtype]
    tensors: dict[str, torch.Tensor] = {}
    for spec in model.param_specs():
        if spec.kind == "vector":
            value = 1.0 + torch.randn(spec.shape, generator=generator) * vector_std
        elif spec.kind == "table":
            value = torch.zeros(spec.shape, dtype=torch.int32)
        else:
            value = torch.randn(spec.shape, generator=generator) * matrix_std
        tensors[spec.name] = value if spec.kind == "table" else value.to(dtype)
    return tensors


def random_tensors_on_device(specs, seed: int, dtype: torch.dtype, device, matrix_std: float = 0.02,
                             vector_std: float = 0.1) -> dict[str, torch.Tensor]:
    """The same distributions drawn with the device's generator (another stream than the CPU's)."""
    generator = torch.Generator(device=device).manual_seed(int(seed))
    tensors: dict[str, torch.Tensor] = {}
    for spec in specs:
        if spec.kind == "table":
            tensors[spec.name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        value = torch.randn(spec.shape, generator=generator, device=device, dtype=torch.float32)
        value = 1.0 + value * vector_std if spec.kind == "vector" else value * matrix_std
        tensors[spec.name] = value.to(dtype)
    return tensors


def write_random_model(folder: Union[str, Path], config_dict: Mapping[str, Any], seed: int,
                       stored_dtype: str = "bfloat16", matrix_std: float = 0.02) -> Path:
    """Creates ``folder`` with ``config.json`` and ``model.safetensors`` for the configuration."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(config_dict, seed, stored_dtype, matrix_std)
    config_out = dict(config_dict)
    config_out["torch_dtype"] = stored_dtype
    (folder / "config.json").write_text(json.dumps(config_out, indent=2) + "\n", encoding="utf-8")
    save_file({name: tensor.contiguous() for name, tensor in tensors.items()}, str(folder / "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    return folder


def main(argv=None) -> None:
    import argparse

    parser = argparse.ArgumentParser(description="Write a model folder with seeded random weights.")
    parser.add_argument("--config", required=True, help="a config.json to take the sizes from")
    parser.add_argument("--out", required=True, help="folder to create")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--dtype", choices=sorted(_STORED), default="bfloat16", help="stored element type")
    args = parser.parse_args(argv)
    config = json.loads(Path(args.config).read_text(encoding="utf-8"))
    print(write_random_model(args.out, config, args.seed, args.dtype))


if __name__ == "__main__":
    main()
