"""Lotilix: a decoder of parallel blocks whose layers are listed one by one in ``config.json``.

Every layer is a parallel block: one norm, whose output the mixer and the feed-forward both read, and their
sum added to the stream; then a small gated input looked up by token id.  The mixer is softmax attention
through low-rank latents with a sliding window (``latent_attention``), grouped-query attention whose values
are its unrotated keys and whose mask is cut into chunks (``attention``), or a gated delta rule with a decay
per key channel (``channel_delta``).  The feed-forward is dense with the tanh form of GELU, or absent.
The keys of ``config.json``:

    architecture            "Lotilix"
    vocab, width            sizes of the embedding and the residual stream
    norm.eps                eps of every norm
    token_side.dim          (optional) numbers per layer of the per-token input
    layers[i].type          "latent_attention" | "attention" | "channel_delta"
    layers[i].mixer         latent_attention: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot.base, rot.dims,
                            mask.size; attention: heads, kv_heads, dim, vdim, scale, rot.base, rot.dims,
                            rot.scaling (optional: factor, low, high, original), mask.size;
                            channel_delta: heads, kv_heads, dim, vdim, conv
    layers[i].mlp           null, or kind "dense" with ff
    max_positions           (optional) the longest sequence; the design itself has no limit

Sizes that only the file's tensors fix (the inner sizes of the delta rule's decay and gate projections) are
read from them when the model is loaded from a folder; a configuration without a folder may name them as
``decay_rank`` and ``gate_rank`` in the mixer.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, Optional

from .spec import (BiasAttentionSpec, ConfigError, DeltaRuleSpec, GatedMlpSpec, LatentAttentionSpec, ModelSpec,
                   ParallelBlockSpec, RmsNormSpec, RotaryPairsSpec, ScheduleEntry, TokenSideSpec)

ARCHITECTURE = "Lotilix"
DEFAULT_MAX_POSITIONS = 1 << 20
DEFAULT_LOW_RANK = 16  # decay_rank / gate_rank of a configuration that names none and has no folder


def _need(d: Dict[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} has no '{key}'")
    return d[key]


def _int(d, key, where, minimum=1) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer of at least {minimum}, got {v!r}")
    return v


def _num(d, key, where) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


def _mask_size(m: Dict[str, Any], where: str) -> int:
    mask = m.get("mask")
    if mask is None:
        return 0
    return _int(mask, "size", where + ".mask")


def _rotary(m: Dict[str, Any], where: str, most: int) -> RotaryPairsSpec:
    rot = _need(m, "rot", where)
    dims = _int(rot, "dims", where + ".rot", minimum=2)
    if dims % 2 or dims > most:
        raise ConfigError(f"config.json: {where}.rot.dims={dims} must be even and at most {most}")
    scaling = rot.get("scaling")
    if scaling is not None:
        sw = where + ".rot.scaling"
        scaling = (_num(scaling, "factor", sw), _num(scaling, "low", sw), _num(scaling, "high", sw), _num(scaling, "original", sw))
        if scaling[2] == scaling[1] or min(scaling) <= 0:
            raise ConfigError(f"config.json: {sw}: factor, low, high and original must be positive and low != high")
    return RotaryPairsSpec(dims=dims, base=_num(rot, "base", where + ".rot"), scaling=scaling)


@dataclass(frozen=True)
class LotilixConfig:
    """The file as it was read (``text``: canonical JSON, so that the record is hashable and can be written back
    unchanged) plus the checked top-level numbers."""

    text: str
    vocab: int
    width: int
    n_layers: int
    max_positions: int

    @property
    def data(self) -> Dict[str, Any]:
        return json.loads(self.text)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LotilixConfig":
        layers = _need(d, "layers", "the file")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        if not _num(_need(d, "norm", "the file"), "eps", "norm") > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if d.get("token_side") is not None:
            _int(d["token_side"], "dim", "token_side")
        mp = d.get("max_positions") or DEFAULT_MAX_POSITIONS
        cfg = cls(text=json.dumps(d, sort_keys=True), vocab=_int(d, "vocab", "the file"), width=_int(d, "width", "the file"),
                  n_layers=len(layers), max_positions=int(mp))
        cfg.to_spec()  # every layer is checked by building its spec
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return self.data

    def with_max_positions(self, max_seq: int) -> "LotilixConfig":
        if max_seq and 0 < max_seq < self.max_positions:
            d = self.data
            d["max_positions"] = int(max_seq)
            return LotilixConfig.from_dict(d)
        return self

    # ---- translation into parts ------------------------------------------------------------
    def _mixer(self, i: int, layer: Dict[str, Any], eps: float) -> Any:
        where = f"layers[{i}].mixer"
        m = _need(layer, "mixer", f"layers[{i}]")
        kind = _need(layer, "type", f"layers[{i}]")
        if kind == "latent_attention":
            rot_dim = _int(m, "rot_dim", where, minimum=2)
            position = _rotary(m, where, rot_dim)
            if position.dims != rot_dim:
                raise ConfigError(f"config.json: {where}: rot.dims={position.dims} must equal rot_dim={rot_dim}")
            return LatentAttentionSpec(
                width=self.width, n_heads=_int(m, "heads", where), head_dim=_int(m, "dim", where), rot_dim=rot_dim,
                v_head_dim=_int(m, "vdim", where), q_rank=_int(m, "q_rank", where), kv_rank=_int(m, "kv_rank", where),
                scale=_num(m, "scale", where), position=position, norm_eps=eps, window=_mask_size(m, where))
        if kind == "attention":
            heads, kv_heads, dim = _int(m, "heads", where), _int(m, "kv_heads", where), _int(m, "dim", where)
            if heads % kv_heads:
                raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
            if m.get("vdim") is not None and _int(m, "vdim", where) != dim:
                raise ConfigError(f"config.json: {where}: the values are the keys, so vdim={m['vdim']} must equal dim={dim}")
            return BiasAttentionSpec(
                width=self.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=dim, v_head_dim=dim, scale=_num(m, "scale", where),
                chunk=_mask_size(m, where), position=_rotary(m, where, dim), values_are_keys=True, norm_eps=eps)
        if kind == "channel_delta":
            heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
            if heads % kv_heads:
                raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
            dim = _int(m, "dim", where)
            if dim > 256:
                raise ConfigError(f"config.json: {where}: dim={dim} must be at most 256")
            taps = _int(m, "conv", where)
            if taps > 16:
                raise ConfigError(f"config.json: {where}: conv={taps} must be at most 16")
            return DeltaRuleSpec(
                width=self.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=dim, v_head_dim=_int(m, "vdim", where),
                conv_taps=taps, decay_rank=int(m.get("decay_rank") or DEFAULT_LOW_RANK),
                gate_rank=int(m.get("gate_rank") or DEFAULT_LOW_RANK), norm_eps=eps)
        raise ConfigError(f"config.json: layers[{i}].type is 'latent_attention', 'attention' or 'channel_delta', not {kind!r}")

    def _ffn(self, i: int, layer: Dict[str, Any]) -> Optional[GatedMlpSpec]:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        where = f"layers[{i}].mlp"
        if mlp.get("kind", "dense") != "dense":
            raise ConfigError(f"config.json: {where}.kind is 'dense', not {mlp.get('kind')!r}")
        return GatedMlpSpec(width=self.width, intermediate=_int(mlp, "ff", where), activation="gelu_tanh", wide_output=True)

    def to_spec(self) -> ModelSpec:
        d = self.data
        eps = float(d["norm"]["eps"])
        norm = RmsNormSpec(width=self.width, eps=eps)
        side_dim = int(d["token_side"]["dim"]) if d.get("token_side") else 0
        blocks, schedule = [], []
        for i, layer in enumerate(d["layers"]):
            side = None
            if side_dim:
                side = TokenSideSpec(width=self.width, vocab_size=self.vocab, dim=side_dim, column=i * side_dim,
                                     table_width=self.n_layers * side_dim, eps=eps)
            blocks.append(ParallelBlockSpec(mixer=self._mixer(i, layer, eps), ffn=self._ffn(i, layer), norm=norm, side=side))
            schedule.append(ScheduleEntry(block=i))
        spec = ModelSpec(vocab_size=self.vocab, width=self.width, blocks=tuple(blocks), schedule=tuple(schedule),
                         final_norm=norm, max_positions=self.max_positions)
        spec.validate()
        return spec


def with_sizes_of(config: Dict[str, Any], shapes: Dict[str, Any]) -> Dict[str, Any]:
    """``config`` with the sizes that only the file's tensors fix filled in: the inner sizes of each delta-rule
    layer's decay and gate projections."""
    out = json.loads(json.dumps(config))
    for i, layer in enumerate(out.get("layers") or []):
        if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
            continue
        for key, tensor in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
            shape = shapes.get(tensor)
            if shape is not None:
                layer["mixer"][key] = int(shape[0])
    return out


def tensor_name(path: str) -> str:
    """Checkpoint name of the parameter at ``path``: ``blocks.3.mixer.q`` is ``l3.mix.q``; the table of the
    per-token inputs is one tensor, ``side.embed``, whichever block asks for it."""
    fixed = {"embedding.table": "embed", "final_norm.weight": "final.norm", "head.weight": "head"}
    if path in fixed:
        return fixed[path]
    parts = path.split(".")
    if parts[0] == "blocks" and len(parts) >= 4:
        i, role, rest = parts[1], parts[2], ".".join(parts[3:])
        if role == "norm" and rest == "weight":
            return f"l{i}.norm1"
        if role == "mixer":
            return f"l{i}.mix.{rest}"
        if role == "ffn":
            return f"l{i}.mlp.{rest}"
        if role == "side":
            return "side.embed" if rest == "embed" else f"l{i}.side.{rest}"
    raise KeyError(f"the Lotilix architecture has no tensor for parameter '{path}'")
