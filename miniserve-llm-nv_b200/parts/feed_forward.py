"""Feed-forward parts.  ``gated_mlp``: ``down(act(gate(x)) * up(x))`` without biases
(miniserve/model/layers.py:71-87) with ``silu`` as the activation; gate and up run as one
matrix product over one weight that holds both.  Where the intermediate size is a multiple of eight
the rows of the two alternate in blocks of eight (``kernels.interleave_gate_up``), which lets the
product of a decode step apply the activation as it stores; else the up rows follow the gate rows."""

from __future__ import annotations

from typing import Optional, Union

import torch

from .. import kernels
from .base import FoldedInput, NormFold, ParamSpec, Part, ResidualAdd, register_feed_forward
from .context import StepContext


@register_feed_forward("gated_mlp")
class GatedMLP(Part):
    def __init__(self, *, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 gate_name: str = "gate_proj.weight", up_name: str = "up_proj.weight",
                 down_name: str = "down_proj.weight") -> None:
        if activation != "silu":
            raise ValueError(f"gated_mlp implements the 'silu' activation, not {activation!r}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.names = dict(gate=prefix + gate_name, up=prefix + up_name, down=prefix + down_name)
        self.gate_up_weight: Optional[torch.Tensor] = None
        self.down_weight: Optional[torch.Tensor] = None
        self.paired = False

    def param_specs(self) -> list[ParamSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return [ParamSpec(self.names["gate"], (i, h)), ParamSpec(self.names["up"], (i, h)),
                ParamSpec(self.names["down"], (h, i))]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        gate, up = tensors[self.names["gate"]], tensors[self.names["up"]]
        self.paired = self.intermediate_size % kernels.GATE_UP_BLOCK == 0
        if self.paired:
            self.gate_up_weight = kernels.interleave_gate_up(gate, up).contiguous()
        else:
            self.gate_up_weight = torch.cat([gate, up], dim=0).contiguous()
        self.down_weight = tensors[self.names["down"]]

    # norms folded into the projections (the gate/up weight only in its interleaved form: the product that
    # completes the norm is the one that applies the activation)
    fold_input_gated = True

    def fold_input_weight(self, ctx: StepContext) -> Optional[torch.Tensor]:
        return self.gate_up_weight if self.paired else None

    def fold_output_weight(self, ctx: StepContext) -> Optional[torch.Tensor]:
        return self.down_weight if self.paired else None

    def forward(self, x, ctx: StepContext, fold: Union[None, NormFold, ResidualAdd] = None):
        """``x``: the normed input, or a :class:`FoldedInput`.  With a :class:`NormFold` the down projection adds into
        the residual stream and a :class:`FoldedInput` for the part behind the following norm is returned; with a
        :class:`ResidualAdd` it adds into the stream and nothing is returned."""
        stats = None
        if isinstance(x, FoldedInput):
            x, stats = x.x, x.stats
        n = x.shape[0]
        out = ctx.buffer("gated_mlp.out", (n, self.hidden_size), x.dtype)
        if self.paired:
            hidden = ctx.buffer("gated_mlp.hidden", (n, self.intermediate_size), x.dtype)
            kernels.gated_up(x, self.gate_up_weight, hidden, row_stats=stats)
            if isinstance(fold, ResidualAdd):
                kernels.linear_add(hidden, self.down_weight, fold.residual)
                return None
            if fold is not None:
                partials = ctx.buffer("gated_mlp.partials", kernels.residual_partials_shape(n, *self.down_weight.shape), torch.float32)
                stats = kernels.linear_residual(hidden, self.down_weight, fold.residual, fold.weight, fold.eps, out,
                                                     partials)
                return FoldedInput(out, stats)
            kernels.linear(hidden, self.down_weight, out)
        else:
            gate_up = ctx.buffer("gated_mlp.gate_up", (n, 2 * self.intermediate_size), x.dtype)
            kernels.linear(x, self.gate_up_weight, gate_up)
            kernels.gated_linear(gate_up, self.down_weight, out)
        return out
