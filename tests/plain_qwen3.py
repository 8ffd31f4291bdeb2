"""Plain, slow restatement of the Qwen3 dense decoder: whole sequences, no cache.

Every function is written from the formulas of MiniServe's own model code
(cited per function as ``path:line`` inside that project) and shares no code
with the engine.  Tensors keep the dtype of the weights they are given, so the
same functions serve as a float32 restatement (compared once with MiniServe's
``Qwen3ForCausalLM`` on the CPU, see ``tests/golden/``) and as a float64 oracle
for the engine's float32 and bfloat16 paths.

One deliberate difference: MiniServe rounds the normalised activations, the
rotation tables and the softmax to the model dtype between the steps (it runs in
half precision).  With float32/float64 weights those casts are the identity, so
they do not appear here.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# --------------------------------------------------------------------------- parts


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``w * (x * rsqrt(mean(x^2) + eps))`` over the last dim.

    miniserve/model/layers.py:30-34 (variance in float32, normalise, then scale).
    """
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def plain_rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin of ``position * theta^(-2j/d)``, duplicated over both halves.

    miniserve/model/rope.py:24-29.  The inverse frequencies are formed in
    float32 exactly as there (``1 / theta ** (arange(0, d, 2) / d)``) so that the
    angle table is the one MiniServe uses; they are widened afterwards.
    """
    frequencies = torch.arange(0, head_dim, 2, dtype=torch.float32)
    inverse_frequency = (1.0 / (theta ** (frequencies / head_dim))).to(dtype)
    angles = positions.to(dtype).unsqueeze(-1) * inverse_frequency
    embedding = torch.cat((angles, angles), dim=-1)
    return embedding.cos(), embedding.sin()


def plain_rotate_half(x: torch.Tensor) -> torch.Tensor:
    """``concat(-x[d/2:], x[:d/2])``; miniserve/model/rope.py:32-34."""
    first, second = x.chunk(2, dim=-1)
    return torch.cat((-second, first), dim=-1)


def plain_apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x*cos + rotate_half(x)*sin`` with x ``[T, heads, d]``, tables ``[T, d]``.

    miniserve/model/rope.py:47-52.
    """
    return x * cos[:, None, :] + plain_rotate_half(x) * sin[:, None, :]


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor,
                    window: int | None = None) -> torch.Tensor:
    """Causal grouped-query attention of a whole sequence.

    q ``[T, nq, d]``, k and v ``[T, nkv, d]``; query head h reads kv head
    ``h // (nq // nkv)`` (miniserve/model/qwen3.py:20-27), scores are scaled by
    ``d ** -0.5`` (qwen3.py:66,243), a key is visible iff its position is not
    after the query's (qwen3.py:37-53), softmax over the keys (qwen3.py:247),
    then the weighted sum of values (qwen3.py:248).  ``window`` (not a MiniServe
    option; used by the tests of the attention part alone) additionally hides
    keys that lie ``window`` or more positions behind the query.
    """
    n_tokens, n_q, head_dim = q.shape
    n_kv = k.shape[1]
    group = n_q // n_kv
    out = torch.empty_like(q)
    neg_inf = float("-inf")
    for head in range(n_q):
        kv_head = head // group
        scores = (q[:, head, :] @ k[:, kv_head, :].T) * (head_dim ** -0.5)
        visible = positions[None, :] <= positions[:, None]
        if window is not None:
            visible &= positions[None, :] > positions[:, None] - window
        scores = scores.masked_fill(~visible, neg_inf)
        out[:, head, :] = torch.softmax(scores, dim=-1) @ v[:, kv_head, :]
    return out


def plain_swiglu(x: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor) -> torch.Tensor:
    """``down(silu(gate(x)) * up(x))``; miniserve/model/layers.py:86-87."""
    gate = x @ gate_w.T
    return ((gate * torch.sigmoid(gate)) * (x @ up_w.T)) @ down_w.T


# --------------------------------------------------------------------------- model


def plain_attention_block(x, weights, prefix, config, positions):
    """Projections, per-head q/k norm, RoPE, attention, output projection.

    miniserve/model/qwen3.py:108-139 (norm over the last dim before RoPE:
    qwen3.py:124-126, 97-106).
    """
    n_tokens = x.shape[0]
    n_q, n_kv, d = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    eps = config["rms_norm_eps"]
    q = (x @ weights[prefix + "q_proj.weight"].T).view(n_tokens, n_q, d)
    k = (x @ weights[prefix + "k_proj.weight"].T).view(n_tokens, n_kv, d)
    v = (x @ weights[prefix + "v_proj.weight"].T).view(n_tokens, n_kv, d)
    q = plain_rmsnorm(q, weights[prefix + "q_norm.weight"], eps)
    k = plain_rmsnorm(k, weights[prefix + "k_norm.weight"], eps)
    cos, sin = plain_rope_tables(positions, d, config["rope_theta"], x.dtype)
    q = plain_apply_rope(q, cos, sin)
    k = plain_apply_rope(k, cos, sin)
    attended = plain_attention(q, k, v, positions)
    return attended.reshape(n_tokens, n_q * d) @ weights[prefix + "o_proj.weight"].T


def plain_decoder_layer(x, weights, layer, config, positions):
    """Pre-norm residual block; miniserve/model/qwen3.py:336-346."""
    prefix = f"model.layers.{layer}."
    eps = config["rms_norm_eps"]
    x = x + plain_attention_block(
        plain_rmsnorm(x, weights[prefix + "input_layernorm.weight"], eps),
        weights, prefix + "self_attn.", config, positions)
    x = x + plain_swiglu(
        plain_rmsnorm(x, weights[prefix + "post_attention_layernorm.weight"], eps),
        weights[prefix + "mlp.gate_proj.weight"],
        weights[prefix + "mlp.up_proj.weight"],
        weights[prefix + "mlp.down_proj.weight"])
    return x


def plain_logits(token_ids, weights: dict[str, torch.Tensor], config: dict, rows=None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence starting at position 0 (``rows``: of these positions only,
    where a large vocabulary would make all of them slow).

    Embedding without scaling (miniserve/model/qwen3.py:475), the layers in
    order (qwen3.py:482-485), final norm (qwen3.py:486), then the output matrix,
    which is the embedding when ``tie_word_embeddings`` (qwen3.py:537-540, 591).
    """
    tokens = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = weights["model.embed_tokens.weight"][tokens]
    for layer in range(config["num_hidden_layers"]):
        x = plain_decoder_layer(x, weights, layer, config, positions)
    x = plain_rmsnorm(x, weights["model.norm.weight"], config["rms_norm_eps"])
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    if config.get("tie_word_embeddings", False):
        head = weights["model.embed_tokens.weight"]
    else:
        head = weights["lm_head.weight"]
    return x @ head.T


# --------------------------------------------------------------------------- sampling


def plain_filter_top_k(logits: torch.Tensor, top_k: int) -> torch.Tensor:
    """Keep exactly the k largest (lowest index first among equals), others -inf.

    miniserve/model/sampling.py:34-43.
    """
    if top_k == 0:
        return logits
    order = sorted(range(logits.numel()), key=lambda i: (-float(logits[i]), i))
    kept = torch.full_like(logits, float("-inf"))
    for i in order[:top_k]:
        kept[i] = logits[i]
    return kept


def plain_filter_top_p(logits: torch.Tensor, top_p: float) -> torch.Tensor:
    """Nucleus filter: in descending order drop a token once the mass before it exceeds p.

    miniserve/model/sampling.py:46-58 (the token that crosses the threshold is kept).
    """
    if top_p == 1.0:
        return logits
    order = sorted(range(logits.numel()), key=lambda i: (-float(logits[i]), i))
    probs = torch.softmax(logits.double(), dim=-1)
    kept = torch.full_like(logits, float("-inf"))
    mass = 0.0
    for i in order:
        if mass > top_p:
            break
        kept[i] = logits[i]
        mass += float(probs[i])
    return kept


_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def plain_philox4x32(counter: tuple[int, int, int, int], key: tuple[int, int]) -> tuple[int, int, int, int]:
    """Ten rounds of Philox-4x32 (Salmon et al., 2011), the engine's random source."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(10):
        p0 = _PHILOX_M0 * c0
        p1 = _PHILOX_M1 * c2
        c0, c1, c2, c3 = (((p1 >> 32) ^ c1 ^ k0) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
                          ((p0 >> 32) ^ c3 ^ k1) & 0xFFFFFFFF, p0 & 0xFFFFFFFF)
        k0 = (k0 + _PHILOX_W0) & 0xFFFFFFFF
        k1 = (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def plain_gumbel(seed: int, step: int, index: int) -> float:
    """Standard Gumbel noise of vocabulary entry ``index`` at a request's ``step``-th draw.

    The uniform comes from the upper 24 bits of word ``index % 4`` of
    Philox(counter=(index // 4, step, 0, 0), key=seed) as ``(bits + 0.5) / 2^24``.
    """
    words = plain_philox4x32((index // 4, step & 0xFFFFFFFF, 0, 0), (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    u = ((words[index % 4] >> 8) + 0.5) / 16777216.0
    return -math.log(-math.log(u))


def plain_sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, step: int) -> int:
    """One token from one row of logits.

    Order as in miniserve/model/sampling.py:70-79: temperature 0 is argmax;
    otherwise divide by the temperature, top-k, top-p, then draw from the
    softmax.  The draw is taken as ``argmax(logit + Gumbel noise)``, which has
    that softmax as its distribution and needs no running sum over the row.
    """
    if temperature == 0:
        return int(torch.argmax(logits))
    scaled = logits.to(torch.float32) / temperature
    scaled = plain_filter_top_k(scaled, top_k)
    scaled = plain_filter_top_p(scaled, top_p)
    best, best_value = -1, float("-inf")
    for i in range(scaled.numel()):
        if scaled[i] == float("-inf"):
            continue
        value = float(scaled[i]) + plain_gumbel(seed, step, i)
        if value > best_value:
            best, best_value = i, value
    return best


# --------------------------------------------------------------------------- helpers


def load_folder(folder: str | Path, dtype=torch.float64) -> tuple[dict, dict[str, torch.Tensor]]:
    """Read ``config.json`` and every ``*.safetensors`` of a model folder."""
    from safetensors import safe_open

    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights: dict[str, torch.Tensor] = {}
    for path in sorted(folder.glob("*.safetensors")):
        with safe_open(path, framework="pt", device="cpu") as handle:
            for key in handle.keys():
                weights[key] = handle.get_tensor(key).to(dtype)
    return config, weights
