"""The plain implementation against logits of MiniServe's own model code (CPU, float32)."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch
from safetensors.torch import load_file

import plain_qwen3 as plain
from golden.make_golden import GOLDEN_CONFIGS, golden_tokens, golden_weights

GOLDEN = Path(__file__).parent / "golden" / "reference_logits.safetensors"


@pytest.mark.parametrize("name", ["a", "b"])
def test_plain_logits_equal_reference_model(name):
    config = GOLDEN_CONFIGS[name]
    weights = golden_weights(config, seed=7 + ord(name))
    expected = load_file(str(GOLDEN))[f"logits_{name}"]
    got32 = plain.plain_logits(golden_tokens(name), weights, config)
    assert got32.dtype == torch.float32
    assert torch.allclose(got32, expected, atol=2e-6, rtol=1e-5), float((got32 - expected).abs().max())
    got64 = plain.plain_logits(golden_tokens(name), {k: v.double() for k, v in weights.items()}, config)
    assert float((got64 - expected.double()).abs().max()) < 2e-6


def test_plain_prefix_of_sequence_is_causal():
    config = GOLDEN_CONFIGS["b"]
    weights = {k: v.double() for k, v in golden_weights(config, seed=3).items()}
    tokens = golden_tokens("b")
    whole = plain.plain_logits(tokens, weights, config)
    part = plain.plain_logits(tokens[:19], weights, config)
    assert torch.allclose(whole[:19], part, atol=1e-12)
