"""A small input by token id that a block adds to the stream after its sublayers."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import ParamSpec, Part
from .registry import register_side


@register_side("token_side")
class TokenSide(Part):
    """e = table[token, column : column + dim]; g = act(W_gate x) * e; y = W_proj g;
    x <- x + y / sqrt(mean(y^2) + eps) * gain, with x the stream after the block's sublayers.  The table
    ``[vocab, table_width]`` is one tensor that all blocks of a model are bound to; each reads its own columns."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "act", "norm")
    graph_safe = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        if spec.column < 0 or spec.column + spec.dim > spec.table_width:
            raise ValueError(f"token_side: columns {spec.column}..{spec.column + spec.dim} lie outside a row of {spec.table_width}")
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} is not built; known: {', '.join(sorted(ops.ACTIVATIONS))}")
        self.act = ops.ACTIVATIONS[spec.activation]

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        return {"embed": ParamSpec((s.vocab_size, s.table_width)), "gate": ParamSpec((s.dim, s.width)),
                "proj": ParamSpec((s.width, s.dim)), "norm": ParamSpec((s.width,), init="ones")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.table, self.gain = tensors["embed"], tensors["norm"]
        gate, proj = tensors["gate"], tensors["proj"]
        pad = -s.dim % 8  # the products' inner and outer sizes stay multiples of 8; the added zeros add nothing
        if pad:
            gate = torch.cat([gate, torch.zeros((pad, s.width), dtype=gate.dtype, device=gate.device)]).contiguous()
            proj = torch.cat([proj, torch.zeros((s.width, pad), dtype=proj.dtype, device=proj.device)], dim=1).contiguous()
        self.w_gate, self.w_proj, self.dim_padded = gate, proj, s.dim + pad

    def delta(self, x_cast, ctx):
        """y for the rows ``x_cast`` (the stream in the compute type), float32 and not yet normed."""
        s = self.spec
        pre = ops.linear(x_cast, self.w_gate, out_dtype=self.build.dtype)
        g = ops.gated_lookup(pre, self.table, s.column, ctx.tokens, s.dim, self.act)
        if self.dim_padded != s.dim:
            g = torch.nn.functional.pad(g, (0, self.dim_padded - s.dim))
        return ops.linear(g, self.w_proj, out_dtype=torch.float32)
