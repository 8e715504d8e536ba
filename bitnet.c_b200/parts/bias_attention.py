"""Softmax attention in its general form: a value width of its own, unit-norm queries and keys, a
learned bias by distance, a window that keeps the first tokens, a gate per head, shared keys and values."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import KvRequest, Mixer, ParamSpec
from .registry import build_part, register_mixer


def distance_buckets(n_buckets: int, max_distance: int) -> torch.Tensor:
    """The bucket of every distance 0 .. max_distance (int64): a distance below half the number of
    buckets is its own bucket; from there on buckets widen logarithmically and the last one begins
    at ``max_distance`` at the latest.  Single precision, as positions are everywhere."""
    half = n_buckets // 2
    if n_buckets < 2 or max_distance <= half:
        raise ValueError(f"{n_buckets} distance buckets up to a distance of {max_distance} cannot be laid out")
    n = torch.arange(0, max_distance + 1, dtype=torch.float32)
    far = torch.log(n.clamp(min=1.0) / half) / math.log(max_distance / half) * (n_buckets - half)
    far = (half + far.floor().to(torch.int64)).clamp(max=n_buckets - 1)
    return torch.where(n < half, n.to(torch.int64), far)


@register_mixer("bias_attention")
class BiasAttention(Mixer):
    """q, k, v (and one gate number per head) = W h in one product; q and k divided by their root mean
    square per head; k (normed) and v appended to the cache; for every head
    softmax(q k^T * scale + bias[bucket(distance)]) over the keys the window lets through; the head's
    output times the logistic function of its gate; output projection.  A run without projections of
    keys and values reads the cache of the run its schedule entry names.  Optional: a position encoding on q
    and k (``position``); chunks in place of the window (``chunk``); no value projection, the values being the
    keys as projected, before the encoding (``values_are_keys``)."""

    kernels = ("linear", "linear_mma", "linear_tc", "gemm_tc", "attention", "attention_prefill", "unit_norm", "rotary_pairs")
    TILED_MIN_TOKENS = 16  # runs of new tokens from this many on take the tensor-core kernel (bfloat16)
    graph_safe = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} heads are not a multiple of {spec.n_kv_heads} key/value heads")
        if not 0 < spec.head_dim <= 256 or not 0 < spec.v_head_dim <= 256:
            raise ValueError(f"head_dim={spec.head_dim} and v_head_dim={spec.v_head_dim} must be at most 256")
        if spec.values_are_keys and (spec.v_head_dim != spec.head_dim or not spec.own_kv or spec.unit_norm):
            raise ValueError("values that are the keys need equal widths, projections of their own and no unit norm")
        if spec.chunk and (spec.window or spec.keep_first):
            raise ValueError("chunks take the place of a window")
        self.position = build_part("position", spec.position, build) if spec.position is not None else None
        if self.position is not None and (spec.unit_norm or not hasattr(self.position, "apply")):
            raise ValueError("this mixer takes a position encoding that offers ``apply`` (rotary_pairs), and no unit norm with it")
        self.w_in: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.rel: Optional[torch.Tensor] = None

    def children(self):
        return {"position": self.position} if self.position is not None else {}

    @property
    def q_dim(self) -> int:
        return self.spec.n_heads * self.spec.head_dim

    @property
    def k_dim(self) -> int:
        return self.spec.n_kv_heads * self.spec.head_dim

    @property
    def v_dim(self) -> int:
        return self.spec.n_kv_heads * self.spec.v_head_dim

    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        p = {"q": ParamSpec((self.q_dim, s.width)), "o": ParamSpec((s.width, s.n_heads * s.v_head_dim))}
        if s.own_kv:
            p["k"] = ParamSpec((self.k_dim, s.width))
            if not s.values_are_keys:
                p["v"] = ParamSpec((self.v_dim, s.width))
        if s.bias_buckets:
            p["rel"] = ParamSpec((s.bias_buckets, s.n_heads))
        if s.head_gate:
            p["g"] = ParamSpec((s.n_heads, s.width))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        parts = [tensors["q"]]
        self.k_off = self.v_off = self.g_off = 0
        at = self.q_dim
        if s.own_kv and s.values_are_keys:
            parts.append(tensors["k"])
            self.k_off = self.v_off = at
            at += self.k_dim
        elif s.own_kv:
            parts += [tensors["k"], tensors["v"]]
            self.k_off, self.v_off = at, at + self.k_dim
            at += self.k_dim + self.v_dim
        if s.head_gate:
            parts.append(tensors["g"])
            self.g_off = at
            at += s.n_heads
        dt = parts[0].dtype if all(t.dtype == parts[0].dtype for t in parts) else torch.float32
        pad = -at % 8  # rows of the product's result stay 16-byte aligned
        if pad:
            parts.append(torch.zeros((pad, s.width), dtype=dt, device=parts[0].device))
        # one stacked matrix: all projections of the mixer's input are one product
        self.w_in = torch.cat([t.to(dt) for t in parts], dim=0).contiguous()
        self.row = at + pad
        self.w_o = tensors["o"]
        if s.bias_buckets:
            # the table by distance instead of by bucket: row n serves distance n, the last row every longer one
            buckets = distance_buckets(s.bias_buckets, s.bias_max_distance).to(tensors["rel"].device)
            self.rel = tensors["rel"].float()[buckets].contiguous()

    def cache_request(self) -> KvRequest:
        s = self.spec
        return KvRequest(n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window, v_head_dim=s.v_head_dim,
                         keep_first=s.keep_first if s.window > 0 else 0, chunk=s.chunk)

    def forward(self, h, ctx, kv, state):
        s = self.spec
        n = h.shape[0]
        if kv.owner != s.own_kv:
            raise ValueError("a mixer with key/value projections owns its cache plane, one without reads another's")
        proj = ops.linear(h, self.w_in, out_dtype=self.build.dtype)
        if self.position is not None:
            # values (the keys before the encoding, or projections of their own) to the cache, q and k encoded in
            # place, keys to the cache: one launch
            places = dict(q_off=0, n_q_heads=s.n_heads, q_head_stride=s.head_dim)
            if kv.owner:
                places.update(k_off=self.k_off, n_k_heads=s.n_kv_heads, k_head_stride=s.head_dim, k_row=s.head_dim,
                              v_off=self.v_off, v_head_stride=s.v_head_dim, v_row=s.v_head_dim, tok_seq=ctx.tok_seq,
                              slots=ctx.slots, page_table=kv.page_table, k_cache=kv.k, v_cache=kv.v)
            self.position.apply(proj, ctx, **places)
        elif not s.unit_norm:
            if kv.owner:  # queries and keys as the projections gave them
                kv.append(proj, self.k_off, self.v_off, ctx)
        elif kv.owner:
            ops.unit_norm_append(proj, s.n_heads, s.head_dim, s.norm_eps, ctx.tok_pos, k_off=self.k_off, v_off=self.v_off,
                                 n_kv_heads=s.n_kv_heads, tok_seq=ctx.tok_seq, slots=ctx.slots, page_table=kv.page_table,
                                 k_cache=kv.k, v_cache=kv.v)
        else:
            ops.unit_norm_append(proj, s.n_heads, s.head_dim, s.norm_eps, ctx.tok_pos)
        if ctx.diag is not None:
            ctx.tap("attn_q", lambda: proj[:, : self.q_dim])
        out = torch.empty((n, s.n_heads * s.v_head_dim), dtype=self.build.dtype, device=h.device)
        gate = proj[:, self.g_off:] if s.head_gate else None
        keep = s.keep_first if s.window > 0 else 0
        if (self.build.dtype == torch.bfloat16 and not ctx.decode and ctx.tile_seq is not None and ctx.max_new >= self.TILED_MIN_TOKENS
                and s.v_head_dim % 16 == 0 and s.head_dim % 16 == 0):
            # runs of new tokens: 64 tokens of a sequence and a head per block on the tensor cores, the
            # softmax weights with 16 bits of mantissa
            ops.attention_prefill(proj, self.row, out, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window, ctx.tile_seq,
                                  ctx.tile_row0, ctx.seq_start, ctx.seq_pos0, ctx.slots, kv.page_table, kv.k, kv.v,
                                  keep_first=keep, rel=self.rel, gate=gate, gate_stride=self.row, precise=True, chunk=s.chunk)
        else:
            ops.attention_general(proj, self.row, out, n, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window, ctx.tok_seq,
                                  ctx.tok_pos, ctx.slots, kv.page_table, kv.k, kv.v, keep_first=keep,
                                  rel=self.rel, gate=gate, gate_stride=self.row, chunk=s.chunk,
                                  max_keys=min(ctx.max_len, s.chunk or (s.window + keep)) if (s.window > 0 or s.chunk > 0) else ctx.max_len)
        ctx.tap("attn_out", out)
        return ops.linear(out, self.w_o, out_dtype=torch.float32)
