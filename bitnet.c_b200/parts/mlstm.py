"""mLSTM: a recurrent mixer whose per-sequence state is a matrix memory per head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Mixer, ParamSpec, StateRequest
from .registry import register_mixer


@register_mixer("mlstm")
class Mlstm(Mixer):
    """q, k, v and the output gate's pre-activation = W h in one product; per head the soft-capped log
    input gate i and log forget gate f = log sigmoid(.) in float32; the stabilised recurrence

        m_t = max(f_t + m_{t-1}, i_t),  S_t = e^{f_t + m_{t-1} - m_t} S_{t-1} + e^{i_t - m_t} k_t v_t^T,
        n_t likewise with k_t,  o_t = S_t^T q_t / (max(|n_t . q_t|, e^{-m_t}) + 1e-6),  q scaled by dim^-1/2

    from the sequence's state (zero at its start, float32, kept by the cache from step to step); each
    head's o divided by its root mean square, times a gain over all heads, times sigmoid(gate); output
    projection."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "mlstm")
    graph_safe = True
    CHUNKED_MIN_TOKENS = 16  # bfloat16 steps with a run of so many new tokens take the recurrence chunk by chunk

    def __init__(self, spec, build):
        super().__init__(spec, build)
        if min(spec.n_heads, spec.head_dim, spec.v_head_dim) <= 0 or not spec.gate_cap > 0:
            raise ValueError("mlstm: heads, head sizes and the gate cap must be positive")
        self.w_in: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        qk, vv = s.n_heads * s.head_dim, s.n_heads * s.v_head_dim
        return {"q": ParamSpec((qk, s.width)), "k": ParamSpec((qk, s.width)), "v": ParamSpec((vv, s.width)),
                "g": ParamSpec((vv, s.width)), "o": ParamSpec((s.width, vv)), "norm": ParamSpec((vv,), init="ones"),
                "i": ParamSpec((s.n_heads, s.width)), "i.b": ParamSpec((s.n_heads,)),
                "f": ParamSpec((s.n_heads, s.width)), "f.b": ParamSpec((s.n_heads,))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        qk, vv = s.n_heads * s.head_dim, s.n_heads * s.v_head_dim
        parts = [tensors[n] for n in ("q", "k", "v", "g")]
        dt = parts[0].dtype if all(t.dtype == parts[0].dtype for t in parts) else torch.float32
        self.k_off, self.v_off, self.g_off = qk, 2 * qk, 2 * qk + vv
        pad = -(2 * qk + 2 * vv) % 8
        if pad:
            parts.append(torch.zeros((pad, s.width), dtype=dt, device=parts[0].device))
        self.w_in = torch.cat([t.to(dt) for t in parts], dim=0).contiguous()
        self.row = 2 * qk + 2 * vv + pad
        gates = [tensors[n] for n in ("i", "f", "i.b", "f.b")]
        gdt = gates[0].dtype if all(t.dtype == gates[0].dtype for t in gates) else torch.float32
        self.w_gates = torch.cat([tensors["i"].to(gdt), tensors["f"].to(gdt)], dim=0).contiguous()
        self.b_gates = torch.cat([tensors["i.b"].to(gdt), tensors["f.b"].to(gdt)], dim=0).contiguous()
        self.gain = tensors["norm"]
        self.w_o = tensors["o"]

    def state_request(self) -> StateRequest:
        s = self.spec
        return StateRequest((s.n_heads, ops.mlstm_state_floats(s.head_dim, s.v_head_dim)), torch.float32)

    def forward(self, h, ctx, kv, state):
        s = self.spec
        proj = ops.linear(h, self.w_in, out_dtype=self.build.dtype)
        gates = ops.mlstm_gates(h, self.w_gates, self.b_gates, s.n_heads, s.gate_cap)
        o = ops.mlstm_recurrence(proj, self.k_off, self.v_off, gates, state, ctx.seq_start, ctx.slots, ctx.n_seqs,
                                 s.n_heads, s.head_dim, s.v_head_dim, s.head_dim ** -0.5,
                                 chunks=(self.build.dtype == torch.bfloat16 and not ctx.decode
                                         and ctx.max_new >= self.CHUNKED_MIN_TOKENS))
        ctx.tap("mlstm_raw", o)
        y = ops.mlstm_output(o, self.gain, proj[:, self.g_off: self.g_off + s.n_heads * s.v_head_dim], self.row,
                             s.n_heads, s.v_head_dim, s.norm_eps, self.build.dtype)
        return ops.linear(y, self.w_o, out_dtype=torch.float32)
