"""Gated delta rule with a decay per key channel: a recurrent mixer whose per-sequence state is a matrix per head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Mixer, ParamSpec, StateRequest
from .registry import register_mixer


@register_mixer("delta_rule")
class DeltaRule(Mixer):
    """q, k (kv_heads x dim) and v (heads x vdim) = W h, each through a short causal convolution per channel and
    SiLU; q and k made unit vectors per head, q times dim^-1/2; beta = sigmoid(W_b h) per head; one decay per
    head and key channel, g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias)); per head, from the sequence's
    state S (zero at its start, float32, kept by the cache together with the convolutions' last inputs)

        S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q

    each head's o divided by its root mean square, times a gain shared by the heads, times
    sigmoid(W_g2 W_g1 h); output projection.  Query head h uses q/k head h // (heads / kv_heads)."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "delta_rule")
    graph_safe = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        if min(spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.v_head_dim, spec.decay_rank, spec.gate_rank) <= 0:
            raise ValueError("delta_rule: heads, head sizes and ranks must be positive")
        if spec.n_heads % spec.n_kv_heads or spec.head_dim > 256 or not 1 <= spec.conv_taps <= 16:
            raise ValueError("delta_rule: heads must be a multiple of kv_heads, dim at most 256, 1 to 16 taps")
        self.w_in: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        qk, vv = s.n_kv_heads * s.head_dim, s.n_heads * s.v_head_dim
        return {"q": ParamSpec((qk, s.width)), "q.conv": ParamSpec((qk, s.conv_taps)),
                "k": ParamSpec((qk, s.width)), "k.conv": ParamSpec((qk, s.conv_taps)),
                "v": ParamSpec((vv, s.width)), "v.conv": ParamSpec((vv, s.conv_taps)),
                "b": ParamSpec((s.n_heads, s.width)), "A_log": ParamSpec((s.n_heads,)),
                "a1": ParamSpec((s.decay_rank, s.width)), "a2": ParamSpec((s.n_heads * s.head_dim, s.decay_rank)),
                "dt_bias": ParamSpec((s.n_heads * s.head_dim,)),
                "g1": ParamSpec((s.gate_rank, s.width)), "g2": ParamSpec((vv, s.gate_rank)),
                "norm": ParamSpec((s.v_head_dim,), init="ones"), "o": ParamSpec((s.width, vv))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        qk, vv = s.n_kv_heads * s.head_dim, s.n_heads * s.v_head_dim

        def stack(names, width):
            parts = [tensors[n] for n in names]
            dt = parts[0].dtype if all(t.dtype == parts[0].dtype for t in parts) else torch.float32
            rows = sum(t.shape[0] for t in parts)
            pad = -rows % 8  # rows of the product's result stay 16-byte aligned
            if pad:
                parts.append(torch.zeros((pad, width), dtype=dt, device=parts[0].device))
            return torch.cat([t.to(dt) for t in parts], dim=0).contiguous()

        # q, k, v and beta's pre-activations are one product of the mixer's input; the two low-rank inputs another
        self.w_in = stack(("q", "k", "v", "b"), s.width)
        self.k_off, self.v_off, self.b_off = qk, 2 * qk, 2 * qk + vv
        self.w_low = stack(("a1", "g1"), s.width)
        # [a2 0; 0 g2]: the decays' and the output gate's pre-activations from the low-rank inputs, one float32 product
        low = self.w_low.shape[0]
        w2 = torch.zeros((s.n_heads * s.head_dim + vv, low), dtype=self.w_low.dtype, device=self.w_low.device)
        w2[: s.n_heads * s.head_dim, : s.decay_rank] = tensors["a2"]
        w2[s.n_heads * s.head_dim:, s.decay_rank: s.decay_rank + s.gate_rank] = tensors["g2"]
        self.w_up = w2.contiguous()
        small = [tensors[n] for n in ("q.conv", "k.conv", "v.conv", "dt_bias", "A_log")]
        cdt = small[0].dtype if all(t.dtype == small[0].dtype for t in small) else torch.float32
        self.conv = torch.cat([tensors[n].to(cdt) for n in ("q.conv", "k.conv", "v.conv")], dim=0).contiguous()
        self.dt_bias, self.a_log = tensors["dt_bias"].to(cdt).contiguous(), tensors["A_log"].to(cdt).contiguous()
        self.gain = tensors["norm"]
        self.w_o = tensors["o"]

    def state_request(self) -> StateRequest:
        s = self.spec
        return StateRequest((ops.delta_state_floats(s.n_heads, s.n_kv_heads, s.head_dim, s.v_head_dim, s.conv_taps),), torch.float32)

    def forward(self, h, ctx, kv, state):
        s = self.spec
        proj = ops.linear(h, self.w_in, out_dtype=self.build.dtype)
        low = ops.linear(h, self.w_low, out_dtype=self.build.dtype)
        up = ops.linear(low, self.w_up, out_dtype=torch.float32)  # [n, decays' | gate's pre-activations]
        o = ops.delta_rule(proj, 0, self.k_off, self.v_off, self.conv, s.conv_taps, self.b_off, up, self.dt_bias, self.a_log,
                           state, ctx.tok_seq, ctx.seq_start, ctx.slots, ctx.n_seqs, s.n_heads, s.n_kv_heads, s.head_dim,
                           s.v_head_dim)
        ctx.tap("delta_raw", o)
        y = ops.delta_output(o, self.gain, up[:, s.n_heads * s.head_dim:], s.n_heads, s.v_head_dim, s.norm_eps, self.build.dtype)
        return ops.linear(y, self.w_o, out_dtype=torch.float32)
