"""Writes ``tests/golden/reference_logits.safetensors``: logits of MiniServe's own
``Qwen3ForCausalLM`` (miniserve/model/qwen3.py) on the CPU in float32, for two tiny
random models, so that the plain implementation in ``tests/plain_qwen3.py`` can be
compared with the project it restates without that project being present.

Run once, from the repository root, with a checkout of MiniServe-LLM-NV on disk:

    python tests/golden/make_golden.py /path/to/MiniServe-LLM-NV

MiniServe refuses untied output embeddings (miniserve/config/model_config.py:214-215),
so the untied model is built tied and then given a separate ``lm_head.weight``; it
also wants a half-precision dtype name in its config although the module itself is
built in float32 here.
"""

from __future__ import annotations

import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent

GOLDEN_CONFIGS = {
    "a": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64, intermediate_size=128,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256,
              max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=10000.0, attention_dropout=0.0,
              hidden_act="silu", attention_bias=False, tie_word_embeddings=True),
    "b": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=96, intermediate_size=224,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=32, vocab_size=384,
              max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=1000000.0, attention_dropout=0.0,
              hidden_act="silu", attention_bias=False, tie_word_embeddings=False),
}
GOLDEN_TOKENS = {"a": 37, "b": 45}


def golden_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Matrices N(0, 0.02^2), norm weights 1 + N(0, 0.1^2), drawn in a fixed name order."""
    gen = torch.Generator().manual_seed(seed)
    h, i, d = config["hidden_size"], config["intermediate_size"], config["head_dim"]
    nq, nkv, v = config["num_attention_heads"], config["num_key_value_heads"], config["vocab_size"]

    def matrix(*shape):
        return torch.randn(*shape, generator=gen) * 0.02

    def norm(n):
        return 1.0 + torch.randn(n, generator=gen) * 0.1

    w = {"model.embed_tokens.weight": matrix(v, h)}
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        w[p + "input_layernorm.weight"] = norm(h)
        w[p + "self_attn.q_proj.weight"] = matrix(nq * d, h)
        w[p + "self_attn.k_proj.weight"] = matrix(nkv * d, h)
        w[p + "self_attn.v_proj.weight"] = matrix(nkv * d, h)
        w[p + "self_attn.q_norm.weight"] = norm(d)
        w[p + "self_attn.k_norm.weight"] = norm(d)
        w[p + "self_attn.o_proj.weight"] = matrix(h, nq * d)
        w[p + "post_attention_layernorm.weight"] = norm(h)
        w[p + "mlp.gate_proj.weight"] = matrix(i, h)
        w[p + "mlp.up_proj.weight"] = matrix(i, h)
        w[p + "mlp.down_proj.weight"] = matrix(h, i)
    w["model.norm.weight"] = norm(h)
    if not config["tie_word_embeddings"]:
        w["lm_head.weight"] = matrix(v, h)
    return w


def golden_tokens(name: str) -> list[int]:
    gen = torch.Generator().manual_seed(1000 + ord(name))
    return torch.randint(0, GOLDEN_CONFIGS[name]["vocab_size"], (GOLDEN_TOKENS[name],), generator=gen).tolist()


def main() -> None:
    from safetensors.torch import save_file

    sys.path.insert(0, sys.argv[1])
    from miniserve.config.model_config import ModelConfig
    from miniserve.model.qwen3 import Qwen3ForCausalLM

    out = {}
    for name, config in GOLDEN_CONFIGS.items():
        weights = golden_weights(config, seed=7 + ord(name))
        tied_config = dict(config, tie_word_embeddings=True)
        model_config = ModelConfig.from_hf_config(tied_config, model_id_or_path="golden", dtype="bfloat16")
        model = Qwen3ForCausalLM(model_config, device="cpu", dtype=torch.float32)
        state = dict(weights)
        state["lm_head.weight"] = weights["model.embed_tokens.weight"]  # the module is tied while loading
        model.load_state_dict(state, strict=True)
        if not config["tie_word_embeddings"]:
            model.lm_head.weight = torch.nn.Parameter(weights["lm_head.weight"].clone())
        else:
            model.tie_weights()
        tokens = torch.tensor([golden_tokens(name)], dtype=torch.long)
        with torch.no_grad():
            logits, _ = model.forward_recompute(tokens)
        out[f"logits_{name}"] = logits[0].contiguous()
    save_file(out, str(HERE / "reference_logits.safetensors"))
    print({k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    main()
