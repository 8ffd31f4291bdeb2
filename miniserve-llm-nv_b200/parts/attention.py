"""The attention mixer: grouped-query attention over a paged cache.

Computes what miniserve/model/qwen3.py:144-250 computes for one layer: q/k/v projections
without bias, optional RMSNorm of every q and k head over the head size before the rotation
(qwen3.py:177-178), the position encoding, the append of k and v to the cache, causal
attention by absolute position with softmax in float32 scaled by ``head_dim ** -0.5``
(qwen3.py:66, 243-248), and the output projection.  Differences in form: the three
projections run as one matrix product over a row-concatenated weight, and norm, rotation and
append are one kernel.

All sizes are arguments.  ``window`` limits a query to the last ``window`` keys; ``scale``
overrides the score scale; ``position`` is a :class:`~.spec.PartSpec` of the position family.
``score_softcap`` c turns a scaled score s into ``c * tanh(s / c)`` and ``score_bias_slopes`` (one
number per query head) adds ``slope * (key position - query position)`` to it: position
encodings that act on the scores instead of on queries and keys.  Either of them selects the
general attention kernel.
"""

from __future__ import annotations

from typing import Optional, Sequence, Union

import torch

from .. import kernels
from .base import POSITIONS, FoldedInput, NormFold, PagedKVNeed, ParamSpec, Part, ResidualAdd, register_mixer
from .context import PagedKVView, StepContext
from .spec import PartSpec


@register_mixer("attention")
class Attention(Part):
    def __init__(self, *, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qk_norm: bool, eps: float, position: PartSpec, window: Optional[int] = None,
                 scale: Optional[float] = None, score_softcap: Optional[float] = None,
                 score_bias_slopes: Optional[Sequence[float]] = None,
                 q_name: str = "q_proj.weight", k_name: str = "k_proj.weight",
                 v_name: str = "v_proj.weight", o_name: str = "o_proj.weight", q_norm_name: str = "q_norm.weight",
                 k_norm_name: str = "k_norm.weight") -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
        if head_dim % 2 or not 2 <= head_dim <= kernels.MAX_HEAD_DIM:
            # what the general attention kernel and the fused append take; the tensor-core kernels take fewer
            # sizes, and kernels.attention_kernels() says which of them a given size gets
            raise ValueError(f"head size {head_dim} is not an even number in 2..{kernels.MAX_HEAD_DIM}")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.qk_norm, self.eps = bool(qk_norm), float(eps)
        self.window = window
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.score_softcap = float(score_softcap) if score_softcap else None
        if score_bias_slopes is not None and len(score_bias_slopes) != num_heads:
            raise ValueError(f"{len(score_bias_slopes)} score bias slopes for {num_heads} query heads")
        self.score_bias_slopes = None if score_bias_slopes is None else tuple(float(s) for s in score_bias_slopes)
        self._slopes_on_device: Optional[torch.Tensor] = None
        self.position = POSITIONS.build(position, head_dim=head_dim) if "head_dim" not in position.args \
            else POSITIONS.build(position)
        self.names = dict(q=prefix + q_name, k=prefix + k_name, v=prefix + v_name, o=prefix + o_name,
                          q_norm=prefix + q_norm_name, k_norm=prefix + k_norm_name)
        self.qkv_weight: Optional[torch.Tensor] = None
        self.o_weight: Optional[torch.Tensor] = None
        self.q_norm_weight: Optional[torch.Tensor] = None
        self.k_norm_weight: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ declaration
    def param_specs(self) -> list[ParamSpec]:
        h, d = self.hidden_size, self.head_dim
        specs = [ParamSpec(self.names["q"], (self.num_heads * d, h)),
                 ParamSpec(self.names["k"], (self.num_kv_heads * d, h)),
                 ParamSpec(self.names["v"], (self.num_kv_heads * d, h)),
                 ParamSpec(self.names["o"], (h, self.num_heads * d))]
        if self.qk_norm:
            specs += [ParamSpec(self.names["q_norm"], (d,), "vector"), ParamSpec(self.names["k_norm"], (d,), "vector")]
        return specs

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window)

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.qkv_weight = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.o_weight = tensors[n["o"]]
        if self.qk_norm:
            self.q_norm_weight, self.k_norm_weight = tensors[n["q_norm"]], tensors[n["k_norm"]]
            if self.q_norm_weight.dtype != self.k_norm_weight.dtype:
                self.q_norm_weight = self.q_norm_weight.float()
                self.k_norm_weight = self.k_norm_weight.float()

    # ------------------------------------------------------------------ norms folded into the projections
    def fold_input_weight(self, ctx: StepContext) -> Optional[torch.Tensor]:
        return self.qkv_weight

    def fold_output_weight(self, ctx: StepContext) -> Optional[torch.Tensor]:
        return self.o_weight

    # ------------------------------------------------------------------ work
    def forward(self, x, ctx: StepContext, cache: PagedKVView, fold: Union[None, NormFold, ResidualAdd] = None):
        """``x``: the normed input, or a :class:`FoldedInput`.  With a :class:`NormFold` the output projection adds
        into the residual stream and a :class:`FoldedInput` for the part behind the following norm is returned;
        with a :class:`ResidualAdd` it adds into the stream and nothing is returned."""
        stats = None
        if isinstance(x, FoldedInput):
            x, stats = x.x, x.stats
        n, d = x.shape[0], self.head_dim
        n_q, n_kv = self.num_heads, self.num_kv_heads
        slots = cache.slots if cache.writable else torch.full_like(cache.slots, -1)
        fused = self.position.fused_args(ctx)
        attended = ctx.buffer("attention.attended", (n, n_q, d), x.dtype)
        in_product = fused is not None and kernels.qkv_in_product_supported(n, x.dtype, self.qkv_weight, d, n_q, n_kv, *fused)
        if not in_product:
            qkv = ctx.buffer("attention.qkv", (n, (n_q + 2 * n_kv) * d), x.dtype)
            kernels.linear(x, self.qkv_weight, qkv, row_stats=stats)
        if in_product:
            # many rows: norm, rotation and append happen as the projection's tiles are stored
            q = ctx.buffer("attention.q", (n, n_q, d), x.dtype)
            kernels.linear_pair_qkv(x, self.qkv_weight, slots, self.q_norm_weight, self.k_norm_weight, self.eps, fused[0],
                                    cache.key_pool, cache.value_pool, n_q, n_kv, q, row_stats=stats)
            self._attend(q, ctx, cache, attended)
        elif self._decode_in_the_attention_kernel(ctx, fused, x.dtype):
            # a step of single tokens: norm, rotation and append happen inside the split-key attention kernel
            kernels.decode_attention_fused(qkv, slots, self.q_norm_weight, self.k_norm_weight, self.eps, fused[0],
                                           cache.key_pool, cache.value_pool, cache.block_tables, ctx.query_start,
                                           ctx.context_lens, ctx.max_context_len, self.scale, self.window, n_q, n_kv, d,
                                           attended)
        else:
            q = ctx.buffer("attention.q", (n, n_q, d), x.dtype)
            if fused is not None:
                cos_sin, rotary_dim, interleaved = fused
                kernels.qk_norm_rope_append(qkv, slots, self.q_norm_weight, self.k_norm_weight, self.eps, cos_sin,
                                            rotary_dim, interleaved, cache.key_pool, cache.value_pool, n_q, n_kv, d, q)
            else:
                self._append_with_external_position(qkv, slots, ctx, cache, q)
            self._attend(q, ctx, cache, attended)
        if isinstance(fold, ResidualAdd):
            kernels.linear_add(attended.view(n, n_q * d), self.o_weight, fold.residual)
            return None
        out = ctx.buffer("attention.out", (n, self.hidden_size), x.dtype)
        if fold is not None:
            partials = ctx.buffer("attention.partials", kernels.residual_partials_shape(n, *self.o_weight.shape), torch.float32)
            stats = kernels.linear_residual(attended.view(n, n_q * d), self.o_weight, fold.residual, fold.weight,
                                                 fold.eps, out, partials)
            return FoldedInput(out, stats)
        kernels.linear(attended.view(n, n_q * d), self.o_weight, out)
        return out

    def _attend(self, q: torch.Tensor, ctx: StepContext, cache: PagedKVView, attended: torch.Tensor) -> None:
        if self.score_bias_slopes is not None and self._slopes_on_device is None:
            self._slopes_on_device = torch.tensor(self.score_bias_slopes, dtype=torch.float32, device=q.device)
        kernels.paged_attention(q, cache.key_pool, cache.value_pool, cache.block_tables, ctx.request_of_token,
                                ctx.positions, ctx.query_start, ctx.context_lens, ctx.max_query_len,
                                ctx.max_context_len, self.scale, self.window, attended,
                                ctx.host_query_start or None, self.score_softcap, self._slopes_on_device)

    def _decode_in_the_attention_kernel(self, ctx: StepContext, fused, dtype: torch.dtype) -> bool:
        """Whether this step's norm, rotation and append run inside the attention kernel
        (``kernels.decode_attention_fused``): one token per request, a position encoding in that kernel's form (none,
        or half-split rotation over the whole head), no score modifiers, sizes that the kernel takes."""
        if ctx.max_query_len != 1 or ctx.n_tokens != ctx.n_requests or fused is None:
            return False
        if not kernels.decode_attention_fused_preferred(ctx.n_requests):
            return False
        cos_sin, rotary_dim, interleaved = fused
        if cos_sin is not None and (interleaved or rotary_dim != self.head_dim):
            return False
        if self.score_softcap or self.score_bias_slopes is not None:
            return False
        return kernels.decode_attention_fused_supported(dtype, self.head_dim, self.num_heads, self.num_kv_heads)

    def _append_with_external_position(self, qkv, slots, ctx, cache, q_out) -> None:
        """Position parts without a fused form: norm, ``position.apply``, then a plain append."""
        n, d, n_q, n_kv = qkv.shape[0], self.head_dim, self.num_heads, self.num_kv_heads
        heads = qkv.view(n, n_q + 2 * n_kv, d)
        q = heads[:, :n_q].contiguous()
        k = heads[:, n_q:n_q + n_kv].contiguous()
        if self.qk_norm:
            kernels.rmsnorm(q, self.q_norm_weight, self.eps, q)
            kernels.rmsnorm(k, self.k_norm_weight, self.eps, k)
        q, k = self.position.apply(q, k, ctx)
        packed = torch.cat([q, k, heads[:, n_q + n_kv:]], dim=1).contiguous().view(n, -1)
        kernels.qk_norm_rope_append(packed, slots, None, None, self.eps, None, 0, False, cache.key_pool,
                                    cache.value_pool, n_q, n_kv, d, q_out)
